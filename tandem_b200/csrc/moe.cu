// Routed experts: a token's router scores pick `top` of E small gated feed-forwards.
//
//   z = W_router x (float32, computed by the caller);  s = sigmoid(z)  (or softmax(z))
//   chosen = the `top` largest s, found as the `top` largest z (the lower index wins a tie);  w_k = s_k / (sum of the chosen s + 1e-20) * scale
//   y = sum_k w_k * W_down[e_k] (SiLU(W_gate[e_k] x) * (W_up[e_k] x))
//
// `route` takes the logits to (expert, weight) pairs, one warp per token.  A (token, k) pair is a *slot*.
// `expert_gate_up` computes the activated hidden row of every slot, `expert_down` the weighted sum of a
// token's slots in slot order: no atomics, and a token's result does not depend on the batch.  Both read
// the expert weights as stacked tensors [E, 2 F, K] (gate rows, then up rows) and [E, N, F], one warp per
// output element with 16-byte loads along the reduction, sums in float32.  These are the kernels for steps
// of few tokens (the experts' rows stream once per slot that uses them) and for the 32-bit path.
//
// Steps of many tokens in bfloat16 sort the slots by expert on the device (`sort_slots`: counts, offsets
// padded to whole tiles, the slot list; one block, no host round trip) and run `expert_tiles_*`: 64 slots x
// 64 outputs per block on mma.sync m16n8k16 with float32 accumulators, the expert of a tile found from the
// padded offsets, operands staged through shared memory.
#include "common.cuh"

namespace tb {

constexpr int ROUTE_WARPS = 4;

// logits float32 [T, E] -> ids int32 [T, top], weights float32 [T, top].  score: 0 sigmoid, 1 softmax.
__global__ void __launch_bounds__(ROUTE_WARPS * 32)
route_kernel(const float* __restrict__ logits, int* __restrict__ ids, float* __restrict__ weights, int T_tokens, int E, int top,
             int score, int normalize, float scale) {
  extern __shared__ float smem[];  // ROUTE_WARPS * E scores
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int t = blockIdx.x * ROUTE_WARPS + warp;
  if (t >= T_tokens) return;
  float* s = smem + warp * E;
  const float* z = logits + (size_t)t * E;
  // Both scores grow with the logit, so the choice is made on the logits: scores that round to the same number
  // (a sigmoid near one) are still told apart.
  float m = -INFINITY, sum = 1.f;
  for (int e = lane; e < E; e += 32) { s[e] = z[e]; m = fmaxf(m, z[e]); }
  if (score == 1) {
    m = warp_max(m);
    sum = 0.f;
    for (int e = lane; e < E; e += 32) sum += expf(z[e] - m);
    sum = warp_sum(sum);
  }
  __syncwarp();
  float total = 0.f;
  for (int k = 0; k < top; ++k) {
    float best = -INFINITY;
    int at = 0x7fffffff;
    for (int e = lane; e < E; e += 32)
      if (s[e] > best) { best = s[e]; at = e; }  // ascending e: the lowest index among equals of this lane
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oa = __shfl_xor_sync(0xffffffffu, at, o);
      if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
    }
    const float sc = score == 1 ? expf(best - m) / sum : 1.f / (1.f + expf(-best));
    if (lane == 0) {
      ids[(size_t)t * top + k] = at;
      weights[(size_t)t * top + k] = sc;
      s[at] = -INFINITY;
    }
    total += sc;
    __syncwarp();
  }
  if (lane < top) {
    const float w = weights[(size_t)t * top + lane];
    weights[(size_t)t * top + lane] = (normalize ? w / (total + 1e-20f) : w) * scale;
  }
}

template <typename W>
__device__ __forceinline__ float dot_row(const float* xs, const W* row, int K, int lane);

template <>
__device__ __forceinline__ float dot_row<float>(const float* xs, const float* row, int K, int lane) {
  float acc = 0.f;
  if ((K & 3) == 0 && (reinterpret_cast<uintptr_t>(row) & 15) == 0) {
    for (int k = lane * 4; k < K; k += 128) {
      const float4 w = *reinterpret_cast<const float4*>(row + k);
      acc = fmaf(xs[k], w.x, acc); acc = fmaf(xs[k + 1], w.y, acc); acc = fmaf(xs[k + 2], w.z, acc); acc = fmaf(xs[k + 3], w.w, acc);
    }
  } else {
    for (int k = lane; k < K; k += 32) acc = fmaf(xs[k], row[k], acc);
  }
  return warp_sum(acc);
}

template <>
__device__ __forceinline__ float dot_row<__nv_bfloat16>(const float* xs, const __nv_bfloat16* row, int K, int lane) {
  float acc = 0.f;
  if ((K & 7) == 0 && (reinterpret_cast<uintptr_t>(row) & 15) == 0) {
    for (int k = lane * 8; k < K; k += 256) {
      const uint4 raw = *reinterpret_cast<const uint4*>(row + k);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(h[i]);
        acc = fmaf(xs[k + 2 * i], f.x, acc);
        acc = fmaf(xs[k + 2 * i + 1], f.y, acc);
      }
    }
  } else {
    for (int k = lane; k < K; k += 32) acc = fmaf(xs[k], __bfloat162float(row[k]), acc);
  }
  return warp_sum(acc);
}

// grid (ceil(F / (8 warps)), slots): act[slot, j] = SiLU(x_t . gate[e][j]) * (x_t . up[e][j]).
template <typename X, typename W>
__global__ void __launch_bounds__(256)
expert_gate_up_kernel(const X* __restrict__ x, const W* __restrict__ w, const int* __restrict__ ids, X* __restrict__ act, int top,
                      int F, int K) {
  extern __shared__ float xs[];  // K floats
  pdl_launch_dependents();
  pdl_wait();
  const int slot = blockIdx.y, t = slot / top;
  const int e = ids[slot];
  const X* xr = x + (size_t)t * K;
  for (int k = threadIdx.x; k < K; k += blockDim.x) xs[k] = to_float(xr[k]);
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int j = blockIdx.x * 8 + warp;
  if (j >= F) return;
  const W* we = w + (size_t)e * 2 * F * K;
  const float g = dot_row<W>(xs, we + (size_t)j * K, K, lane);
  const float u = dot_row<W>(xs, we + (size_t)(F + j) * K, K, lane);
  if (lane == 0) act[(size_t)slot * F + j] = from_float<X>(g / (1.f + expf(-g)) * u);
}

// grid (ceil(N / 8), tokens): y[t, n] = sum_k weight[t, k] * (act[t top + k] . down[e_k][n]).
template <typename X, typename W>
__global__ void __launch_bounds__(256)
expert_down_kernel(const X* __restrict__ act, const W* __restrict__ w, const int* __restrict__ ids,
                   const float* __restrict__ weights, float* __restrict__ y, int top, int N, int F) {
  extern __shared__ float as[];  // top * F floats
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.y;
  for (int i = threadIdx.x; i < top * F; i += blockDim.x) as[i] = to_float(act[(size_t)t * top * F + i]);
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int n = blockIdx.x * 8 + warp;
  if (n >= N) return;
  float acc = 0.f;
  for (int k = 0; k < top; ++k) {
    const int e = ids[(size_t)t * top + k];
    const float d = dot_row<W>(as + k * F, w + ((size_t)e * N + n) * F, F, lane);
    acc = fmaf(weights[(size_t)t * top + k], d, acc);
  }
  if (lane == 0) y[(size_t)t * N + n] = acc;
}

// ---------------------------------------------------------------------------------------------
// Many tokens: slots sorted by expert, tiles on the tensor cores.
constexpr int ET_M = 64, ET_N = 64, ET_K = 32, ET_PAD = 8;

// One block.  counts the slots of each expert, gives expert e the rows [offsets[e], offsets[e + 1]) of the sorted
// list with offsets rounded up to whole tiles of ET_M (rows that pad a tile hold -1), and lists the slots of an
// expert in ascending slot order.  offsets int32 [E + 1]; sorted int32 [capacity], capacity >= slots + E * (ET_M - 1).
__global__ void sort_slots_kernel(const int* __restrict__ ids, int* __restrict__ offsets, int* __restrict__ sorted, int slots,
                                  int E, int capacity) {
  extern __shared__ int sm[];  // E counts, then E + 1 offsets
  pdl_launch_dependents();
  pdl_wait();
  int* count = sm;
  int* off = sm + E;
  for (int e = threadIdx.x; e < E; e += blockDim.x) count[e] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < slots; i += blockDim.x) atomicAdd(&count[ids[i]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int at = 0;
    for (int e = 0; e < E; ++e) {
      off[e] = at;
      at += (count[e] + ET_M - 1) / ET_M * ET_M;
    }
    off[E] = at;
  }
  __syncthreads();
  for (int e = threadIdx.x; e <= E; e += blockDim.x) offsets[e] = off[e];
  for (int i = threadIdx.x; i < capacity; i += blockDim.x) sorted[i] = -1;
  __syncthreads();
  // expert by expert, a warp lists its expert's slots in ascending order (ballot + prefix over runs of 32 slots)
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  for (int e = warp; e < E; e += nw) {
    int at = off[e];
    for (int base = 0; base < slots; base += 32) {
      const int i = base + lane;
      const bool mine = i < slots && ids[i] == e;
      const unsigned m = __ballot_sync(0xffffffffu, mine);
      if (mine) sorted[at + __popc(m & ((1u << lane) - 1u))] = i;
      at += __popc(m);
    }
  }
}

__device__ __forceinline__ void mma_bf16(float* c, const uint32_t* a, const uint32_t* b) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

// A tile of ET_M sorted rows x ET_N outputs of one expert.  GATED: outputs are SiLU(gate) * up for ET_N hidden
// columns (both weight tiles are multiplied), rows are gathered from x by token = slot / top, and the result goes to
// act[sorted position]; else: rows are act[sorted position], the result (float32) goes to part[slot].
// 128 threads = 4 warps, warp w owns rows 16 w .. 16 w + 15 of the tile and all ET_N columns.
template <bool GATED>
__global__ void __launch_bounds__(128)
expert_tiles_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ w, const int* __restrict__ offsets,
                    const int* __restrict__ sorted, void* __restrict__ out, int top, int E, int N, int K) {
  __shared__ __align__(16) __nv_bfloat16 As[ET_M][ET_K + ET_PAD];
  __shared__ __align__(16) __nv_bfloat16 Bs[GATED ? 2 : 1][ET_N][ET_K + ET_PAD];
  __shared__ int row_src[ET_M];
  pdl_launch_dependents();
  pdl_wait();
  const int row0 = blockIdx.y * ET_M;
  if (row0 >= offsets[E]) return;
  int e = 0;
  while (e + 1 < E && offsets[e + 1] <= row0) ++e;
  const int n0 = blockIdx.x * ET_N;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid < ET_M) {
    const int slot = sorted[row0 + tid];
    row_src[tid] = slot < 0 ? -1 : (GATED ? slot / top : row0 + tid);
  }
  __syncthreads();
  const __nv_bfloat16* we = w + (size_t)e * (GATED ? 2 : 1) * N * K;
  float acc[GATED ? 2 : 1][ET_N / 8][4];
#pragma unroll
  for (int g = 0; g < (GATED ? 2 : 1); ++g)
#pragma unroll
    for (int j = 0; j < ET_N / 8; ++j)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[g][j][i] = 0.f;

  for (int k0 = 0; k0 < K; k0 += ET_K) {
    // 64 rows x 32 columns of 2 bytes = 4 chunks of 16 bytes a row: 256 chunks per operand, two per thread
    for (int c = tid; c < ET_M * 4; c += 128) {
      const int r = c >> 2, kk = (c & 3) * 8;
      uint4 v = make_uint4(0, 0, 0, 0);
      const int src = row_src[r];
      if (src >= 0 && k0 + kk < K) v = *reinterpret_cast<const uint4*>(a + (size_t)src * K + k0 + kk);
      *reinterpret_cast<uint4*>(&As[r][kk]) = v;
    }
#pragma unroll
    for (int g = 0; g < (GATED ? 2 : 1); ++g)
      for (int c = tid; c < ET_N * 4; c += 128) {
        const int r = c >> 2, kk = (c & 3) * 8;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (n0 + r < N && k0 + kk < K) v = *reinterpret_cast<const uint4*>(we + ((size_t)g * N + n0 + r) * K + k0 + kk);
        *reinterpret_cast<uint4*>(&Bs[g][r][kk]) = v;
      }
    __syncthreads();
#pragma unroll
    for (int ks = 0; ks < ET_K; ks += 16) {
      uint32_t af[4];
      const int ar = warp * 16 + (lane >> 2), ac = ks + (lane & 3) * 2;
      af[0] = *reinterpret_cast<const uint32_t*>(&As[ar][ac]);
      af[1] = *reinterpret_cast<const uint32_t*>(&As[ar + 8][ac]);
      af[2] = *reinterpret_cast<const uint32_t*>(&As[ar][ac + 8]);
      af[3] = *reinterpret_cast<const uint32_t*>(&As[ar + 8][ac + 8]);
#pragma unroll
      for (int g = 0; g < (GATED ? 2 : 1); ++g)
#pragma unroll
        for (int j = 0; j < ET_N / 8; ++j) {
          uint32_t bf[2];
          const int br = j * 8 + (lane >> 2);
          bf[0] = *reinterpret_cast<const uint32_t*>(&Bs[g][br][ac]);
          bf[1] = *reinterpret_cast<const uint32_t*>(&Bs[g][br][ac + 8]);
          mma_bf16(acc[g][j], af, bf);
        }
    }
    __syncthreads();
  }
#pragma unroll
  for (int j = 0; j < ET_N / 8; ++j)
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int r = warp * 16 + (lane >> 2) + half * 8;
      const int n = n0 + j * 8 + (lane & 3) * 2;
      const int slot = sorted[row0 + r];
      if (slot < 0 || n >= N) continue;
      if (GATED) {
        const float g0 = acc[0][j][2 * half], g1 = acc[0][j][2 * half + 1];
        const float v0 = g0 / (1.f + expf(-g0)) * acc[GATED ? 1 : 0][j][2 * half];
        const float v1 = g1 / (1.f + expf(-g1)) * acc[GATED ? 1 : 0][j][2 * half + 1];
        __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(out) + (size_t)(row0 + r) * N + n;
        o[0] = __float2bfloat16_rn(v0);
        if (n + 1 < N) o[1] = __float2bfloat16_rn(v1);
      } else {
        float* o = reinterpret_cast<float*>(out) + (size_t)slot * N + n;
        o[0] = acc[0][j][2 * half];
        if (n + 1 < N) o[1] = acc[0][j][2 * half + 1];
      }
    }
}

// y[t, n] = sum_k weight[t, k] * part[t top + k, n], in slot order.
__global__ void combine_slots_kernel(const float* __restrict__ part, const float* __restrict__ weights, float* __restrict__ y,
                                     long long total, int N, int top) {
  pdl_launch_dependents();
  pdl_wait();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / N;
    const int n = (int)(i % N);
    float acc = 0.f;
    for (int k = 0; k < top; ++k) acc = fmaf(weights[t * top + k], part[((size_t)t * top + k) * N + n], acc);
    y[i] = acc;
  }
}

}  // namespace tb

extern "C" {

int tb_moe_route(void* stream, const float* logits, int* ids, float* weights, int T_tokens, int E, int top, int score,
                 int normalize, float scale) {
  if (T_tokens <= 0) return 0;
  if (E <= 0 || top <= 0 || top > E || top > 32 || score < 0 || score > 1) return TB_ERR_BAD_SIZE;
  const size_t smem = (size_t)tb::ROUTE_WARPS * E * sizeof(float);
  if (smem > 48 * 1024) return TB_ERR_BAD_SIZE;
  return tb::launch(tb::route_kernel, dim3((T_tokens + tb::ROUTE_WARPS - 1) / tb::ROUTE_WARPS), dim3(tb::ROUTE_WARPS * 32), smem,
                    stream, logits, ids, weights, T_tokens, E, top, score, normalize, scale);
}

// x [T, K], w [E, 2 F, K], act [T top, F] of the activations' type `dtype`; the weights of type `dtype` too.
int tb_moe_gate_up(void* stream, const void* x, const void* w, const int* ids, void* act, int T_tokens, int top, int F, int K,
                   int dtype) {
  if (T_tokens <= 0) return 0;
  if (top <= 0 || F <= 0 || K <= 0 || (long long)T_tokens * top > 65535 || K * sizeof(float) > 48 * 1024) return TB_ERR_BAD_SIZE;
  const dim3 grid((F + 7) / 8, T_tokens * top);
  TB_DISPATCH_DTYPE(dtype, tb::launch(tb::expert_gate_up_kernel<T, T>, grid, dim3(256), (size_t)K * sizeof(float), stream, (const T*)x,
                                      (const T*)w, ids, (T*)act, top, F, K));
}

// act [T top, F], w [E, N, F] of type `dtype`; weights float32 [T, top]; y float32 [T, N].
int tb_moe_down(void* stream, const void* act, const void* w, const int* ids, const float* weights, float* y, int T_tokens,
                int top, int N, int F, int dtype) {
  if (T_tokens <= 0) return 0;
  if (top <= 0 || F <= 0 || N <= 0 || T_tokens > 65535 || (size_t)top * F * sizeof(float) > 48 * 1024) return TB_ERR_BAD_SIZE;
  const dim3 grid((N + 7) / 8, T_tokens);
  TB_DISPATCH_DTYPE(dtype, tb::launch(tb::expert_down_kernel<T, T>, grid, dim3(256), (size_t)top * F * sizeof(float), stream,
                                      (const T*)act, (const T*)w, ids, weights, y, top, N, F));
}

int tb_moe_tile_rows() { return tb::ET_M; }

// The tensor-core path (bfloat16).  offsets int32 [E + 1], sorted int32 [capacity] and act bfloat16 [capacity, F]
// and part float32 [T top, N] are scratch of the caller; capacity = T top + E (tile rows - 1) rounded up to whole tiles.
int tb_moe_tiles(void* stream, const void* x, const void* w_gate_up, const void* w_down, const int* ids, const float* weights,
                 int* offsets, int* sorted, void* act, float* part, float* y, int T_tokens, int top, int E, int N, int F, int K,
                 int capacity) {
  if (T_tokens <= 0) return 0;
  const int slots = T_tokens * top;
  if (top <= 0 || E <= 0 || E > 4096 || (F & 7) || (K & 7) || N != K || capacity % tb::ET_M || capacity < slots + E * (tb::ET_M - 1))
    return TB_ERR_BAD_SIZE;
  int rc = tb::launch(tb::sort_slots_kernel, dim3(1), dim3(1024), (size_t)(2 * E + 1) * sizeof(int), stream, ids, offsets, sorted,
                      slots, E, capacity);
  if (rc != 0) return rc;
  const int row_tiles = capacity / tb::ET_M;
  rc = tb::launch(tb::expert_tiles_kernel<true>, dim3((F + tb::ET_N - 1) / tb::ET_N, row_tiles), dim3(128), 0, stream,
                  (const __nv_bfloat16*)x, (const __nv_bfloat16*)w_gate_up, offsets, sorted, act, top, E, F, K);
  if (rc != 0) return rc;
  rc = tb::launch(tb::expert_tiles_kernel<false>, dim3((N + tb::ET_N - 1) / tb::ET_N, row_tiles), dim3(128), 0, stream,
                  (const __nv_bfloat16*)act, (const __nv_bfloat16*)w_down, offsets, sorted, part, top, E, N, F);
  if (rc != 0) return rc;
  const long long total = (long long)T_tokens * N;
  long long blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  return tb::launch(tb::combine_slots_kernel, dim3((int)blocks), dim3(256), 0, stream, part, weights, y, total, N, top);
}

}  // extern "C"
