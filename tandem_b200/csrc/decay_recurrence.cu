// Linear attention with a fixed decay per head (no softmax, no denominator), carried as a state:
//
//   S_t = decay[h] * S_(t-1) + k_t v_t^T          S: [dk, dv] per head, float32, one per live request
//   o_t = S_t^T q_t
//
// Three kernels, all float32 on the CUDA cores.  `decay_recurrence_prep` works in place on the raw
// projection [q | k | v | ...] of each token: an activation on q, k and v (none or SiLU), the rotary
// encoding of the first `rd` dims of every q and k head (dim i paired with i + rd/2; angle =
// position * freq[i], in float32), and a constant factor on k after the rotation.
// `decay_recurrence_scan` walks each request's tokens in order from the state its slot holds and
// leaves the new state there.  The columns of S are independent, so a block owns 32 of them for one
// (request, head); warp w of the block holds a few rows (16, or 32 for large keys) of those columns in registers.
// Tokens are staged sixteen at a time in shared memory (two stages, the next one copied in while
// this one is worked through); per token a thread updates its rows of the state and multiplies them
// into its part of o, and the parts of the warps are summed in warp order after the sixteen.  The order of operations for a token never depends on how the request was cut
// into steps or on the batch, so the state and the output are the same bits under any schedule.
// `decay_recurrence_post` divides o by a root mean square (per head without weight, or over all
// heads with a weight), multiplies by a gate (SiLU or sigmoid of its own projection) and rounds to
// the storage type of the output projection's input.
#include "common.cuh"

namespace tb {

constexpr int DR_CHUNK = 16;  // tokens staged at once

__device__ __forceinline__ float act_apply(float x, int act) {
  if (act == 1) return x / (1.f + expf(-x));  // SiLU
  if (act == 2) return 1.f / (1.f + expf(-x));  // sigmoid
  return x;
}

// One thread per (token, column) of the first 2 H dk + H dv columns.
__global__ void decay_recurrence_prep_kernel(float* __restrict__ proj, int stride, const int* __restrict__ positions,
                                             const float* __restrict__ freq, long long total, int cols, int H, int dk, int dv,
                                             int rd, int act, float key_scale) {
  pdl_launch_dependents();
  pdl_wait();
  const int half = rd >> 1;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
    const int t = (int)(idx / cols), c = (int)(idx % cols);
    float* row = proj + (size_t)t * stride;
    if (c >= 2 * H * dk) {  // v
      if (act) row[c] = act_apply(row[c], act);
      continue;
    }
    const bool is_k = c >= H * dk;
    const float factor = is_k ? key_scale : 1.f;
    const int d = c % dk;
    if (d >= rd) {
      row[c] = act_apply(row[c], act) * factor;
    } else if (d < half) {  // this thread turns the pair (d, d + rd/2)
      const float u = act_apply(row[c], act), v = act_apply(row[c + half], act);
      const float a = (float)positions[t] * freq[d];
      const float cs = cosf(a), sn = sinf(a);
      row[c] = (u * cs - v * sn) * factor;
      row[c + half] = (v * cs + u * sn) * factor;
    }
  }
}

__device__ __forceinline__ void dr_cp_async16(void* dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}

// Tokens [c0, c0 + n) of one head into a stage: q and k rows of dk floats (row pitch dkp), 32 value columns.
// `vec`: every row piece starts on 16 bytes, so the copies are asynchronous 16-byte ones.
__device__ __forceinline__ void dr_load_stage(const float* proj, int stride, int c0, int n, int q_col, int k_col, int v_col,
                                              int v_cols, int dk, int dkp, float* q_s, float* k_s, float* v_s, bool vec) {
  if (vec) {
    const int per_row = dk >> 2;
    for (int e = threadIdx.x; e < n * per_row; e += blockDim.x) {
      const int c = e / per_row, d = (e % per_row) << 2;
      const float* row = proj + (size_t)(c0 + c) * stride;
      dr_cp_async16(q_s + c * dkp + d, row + q_col + d);
      dr_cp_async16(k_s + c * dkp + d, row + k_col + d);
    }
    for (int e = threadIdx.x; e < n * 8; e += blockDim.x) {
      const int c = e >> 3, l = (e & 7) << 2;
      if (l < v_cols) dr_cp_async16(v_s + c * 32 + l, proj + (size_t)(c0 + c) * stride + v_col + l);
    }
  } else {
    for (int e = threadIdx.x; e < n * dk; e += blockDim.x) {
      const int c = e / dk, d = e % dk;
      const float* row = proj + (size_t)(c0 + c) * stride;
      q_s[c * dkp + d] = row[q_col + d];
      k_s[c * dkp + d] = row[k_col + d];
    }
    for (int e = threadIdx.x; e < n * 32; e += blockDim.x) {
      const int c = e >> 5, l = e & 31;
      if (l < v_cols) v_s[e] = proj[(size_t)(c0 + c) * stride + v_col + l];
    }
  }
  asm volatile("cp.async.commit_group;" ::: "memory");
}

// grid (ceil(dv / 32), H, requests); block = ceil(dk / R) warps, each holding R rows of the block's 32 columns
// (R = 16 gives a scheduler two warps to choose from at a key size of 128 and costs 0.6 of the instructions of
// R = 8, which was bound by instruction issue: 60 a token and warp; R = 32 serves key sizes beyond 512).
// Two stages of sixteen tokens: the next one is on its way while this one is worked through.
template <int R>
__device__ __forceinline__ void decay_recurrence_scan_body(const float* __restrict__ proj, int stride, const int* __restrict__ cu_seqlens,
                                                           const int* __restrict__ state_slots, float* __restrict__ state,
                                                           const float* __restrict__ decay, float* __restrict__ out, int H, int dk, int dv) {
  extern __shared__ __align__(16) float smem[];
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const int dkp = nw * R;  // dk rounded up to whole warps
  const int stage_floats = 2 * DR_CHUNK * dkp + DR_CHUNK * 32;  // q, k, v of a stage
  float* part_s = smem + 2 * stage_floats;                      // [DR_CHUNK][nw][32]
  const int h = blockIdx.y, b = blockIdx.z;
  const int j = blockIdx.x * 32 + lane;       // this thread's column of S
  const bool col_ok = j < dv;
  const int t0 = cu_seqlens[b], t1 = cu_seqlens[b + 1];
  if (t1 <= t0) return;
  const float g = decay[h];
  float* S = state + (((size_t)state_slots[b] * H + h) * dk) * dv;
  float s[R];
#pragma unroll
  for (int i = 0; i < R; ++i) {
    const int d = w * R + i;
    s[i] = (col_ok && d < dk) ? S[(size_t)d * dv + j] : 0.f;
  }
  for (int e = threadIdx.x; e < 2 * stage_floats; e += blockDim.x) smem[e] = 0.f;  // rows beyond dk and columns beyond dv stay zero
  __syncthreads();
  const int q_col = h * dk, k_col = H * dk + h * dk, v_col = 2 * H * dk + h * dv + blockIdx.x * 32;
  const int v_cols = min(32, dv - blockIdx.x * 32);
  const bool vec = ((dk | dv | stride) & 3) == 0 && (reinterpret_cast<uintptr_t>(proj) & 15) == 0;
  dr_load_stage(proj, stride, t0, min(DR_CHUNK, t1 - t0), q_col, k_col, v_col, v_cols, dk, dkp, smem, smem + DR_CHUNK * dkp,
                smem + 2 * DR_CHUNK * dkp, vec);
  int slot = 0;
  for (int c0 = t0; c0 < t1; c0 += DR_CHUNK, slot ^= 1) {
    const int n = min(DR_CHUNK, t1 - c0);
    if (c0 + DR_CHUNK < t1) {
      float* nxt = smem + (slot ^ 1) * stage_floats;
      dr_load_stage(proj, stride, c0 + DR_CHUNK, min(DR_CHUNK, t1 - c0 - DR_CHUNK), q_col, k_col, v_col, v_cols, dk, dkp, nxt,
                    nxt + DR_CHUNK * dkp, nxt + 2 * DR_CHUNK * dkp, vec);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    const float* q_s = smem + slot * stage_floats;
    const float* k_s = q_s + DR_CHUNK * dkp;
    const float* v_s = k_s + DR_CHUNK * dkp;
    for (int c = 0; c < n; ++c) {
      const float vj = v_s[c * 32 + lane];
      const float4* kc = reinterpret_cast<const float4*>(k_s + c * dkp + w * R);
      const float4* qc = reinterpret_cast<const float4*>(q_s + c * dkp + w * R);
      float part[4] = {0.f, 0.f, 0.f, 0.f};  // four chains: i mod 4; summed in a fixed order
#pragma unroll
      for (int i = 0; i < R / 4; ++i) {
        const float4 k4 = kc[i], q4 = qc[i];
        s[4 * i] = fmaf(k4.x, vj, g * s[4 * i]);
        s[4 * i + 1] = fmaf(k4.y, vj, g * s[4 * i + 1]);
        s[4 * i + 2] = fmaf(k4.z, vj, g * s[4 * i + 2]);
        s[4 * i + 3] = fmaf(k4.w, vj, g * s[4 * i + 3]);
        part[0] = fmaf(s[4 * i], q4.x, part[0]);
        part[1] = fmaf(s[4 * i + 1], q4.y, part[1]);
        part[2] = fmaf(s[4 * i + 2], q4.z, part[2]);
        part[3] = fmaf(s[4 * i + 3], q4.w, part[3]);
      }
      part_s[(c * nw + w) * 32 + lane] = (part[0] + part[1]) + (part[2] + part[3]);
    }
    __syncthreads();
    for (int c = w; c < n; c += nw) {  // the warps' parts in warp order
      float o = 0.f;
      for (int ww = 0; ww < nw; ++ww) o += part_s[(c * nw + ww) * 32 + lane];
      if (col_ok) out[(size_t)(c0 + c) * H * dv + h * dv + j] = o;
    }
    // the next turn's loads go into the stage that was read two turns ago, and its parts are written behind its own barrier
  }
#pragma unroll
  for (int i = 0; i < R; ++i) {
    const int d = w * R + i;
    if (col_ok && d < dk) S[(size_t)d * dv + j] = s[i];
  }
}

// Key sizes up to 256 run blocks of up to 512 threads with the registers the compiler wants; larger ones run blocks
// of up to 1,024 threads, which leaves 64 registers a thread.
__global__ void decay_recurrence_scan_kernel(const float* __restrict__ proj, int stride, const int* __restrict__ cu_seqlens,
                                             const int* __restrict__ state_slots, float* __restrict__ state,
                                             const float* __restrict__ decay, float* __restrict__ out, int H, int dk, int dv) {
  decay_recurrence_scan_body<16>(proj, stride, cu_seqlens, state_slots, state, decay, out, H, dk, dv);
}
template <int R>
__global__ void __launch_bounds__(1024)
decay_recurrence_scan_wide_kernel(const float* __restrict__ proj, int stride, const int* __restrict__ cu_seqlens,
                                  const int* __restrict__ state_slots, float* __restrict__ state, const float* __restrict__ decay,
                                  float* __restrict__ out, int H, int dk, int dv) {
  decay_recurrence_scan_body<R>(proj, stride, cu_seqlens, state_slots, state, decay, out, H, dk, dv);
}

// One block per token.  mode 0: each head divided by its own root mean square; mode 1: all heads
// together, times `weight` [H dv].  Then times gate_act(gate), rounded to T.
template <typename T>
__global__ void decay_recurrence_post_kernel(const float* __restrict__ o, const float* __restrict__ gate, int gate_stride,
                                             const float* __restrict__ weight, T* __restrict__ y, int H, int dv, int mode,
                                             int gate_act, float eps) {
  __shared__ float scratch[33];
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x, lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const float* orow = o + (size_t)t * H * dv;
  const float* grow = gate ? gate + (size_t)t * gate_stride : nullptr;
  T* yrow = y + (size_t)t * H * dv;
  if (mode == 0) {
    for (int h = w; h < H; h += nw) {
      float ss = 0.f;
      for (int d = lane; d < dv; d += 32) { const float x = orow[h * dv + d]; ss += x * x; }
      ss = warp_sum(ss);
      const float inv = rsqrtf(ss / (float)dv + eps);
      for (int d = lane; d < dv; d += 32) {
        const int c = h * dv + d;
        yrow[c] = from_float<T>(orow[c] * inv * (grow ? act_apply(grow[c], gate_act) : 1.f));
      }
    }
    return;
  }
  const int n = H * dv;
  float ss = 0.f;
  for (int c = threadIdx.x; c < n; c += blockDim.x) { const float x = orow[c]; ss += x * x; }
  ss = block_sum(ss, scratch);
  const float inv = rsqrtf(ss / (float)n + eps);
  for (int c = threadIdx.x; c < n; c += blockDim.x)
    yrow[c] = from_float<T>(orow[c] * inv * (weight ? weight[c] : 1.f) * (grow ? act_apply(grow[c], gate_act) : 1.f));
}

}  // namespace tb

extern "C" {

// proj float32 [T, stride]: columns [q: H dk | k: H dk | v: H dv | anything else].  freq [rd / 2] (rd 0: no rotation).
int tb_decay_recurrence_prep(void* stream, float* proj, int stride, const int* positions, const float* freq, int T_tokens, int H,
                             int dk, int dv, int rd, int act, float key_scale) {
  if (T_tokens <= 0) return 0;
  if (H <= 0 || dk <= 0 || dv <= 0 || rd < 0 || rd > dk || (rd & 1) || (rd && !freq) || act < 0 || act > 1) return TB_ERR_BAD_SIZE;
  const int cols = 2 * H * dk + H * dv;
  const long long total = (long long)T_tokens * cols;
  long long blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  return tb::launch(tb::decay_recurrence_prep_kernel, dim3((int)blocks), dim3(256), 0, stream, proj, stride, positions, freq, total,
                    cols, H, dk, dv, rd, act, key_scale);
}

// state float32 [slots, H, dk, dv]; out float32 [T, H dv]; cu_seqlens [requests + 1]; state_slots [requests].
int tb_decay_recurrence_scan(void* stream, const float* proj, int stride, const int* cu_seqlens, const int* state_slots,
                             float* state, const float* decay, float* out, int requests, int H, int dk, int dv) {
  if (requests <= 0) return 0;
  if (H <= 0 || dk <= 0 || dk > 1024 || dv <= 0 || H > 65535 || requests > 65535) return TB_ERR_BAD_SIZE;
  const int R = dk <= 512 ? 16 : 32;
  const int nw = (dk + R - 1) / R, dkp = nw * R;
  const size_t smem = (size_t)(2 * (2 * tb::DR_CHUNK * dkp + tb::DR_CHUNK * 32) + tb::DR_CHUNK * nw * 32) * sizeof(float);
  auto kernel = dk <= 256 ? tb::decay_recurrence_scan_kernel
                          : (R == 16 ? tb::decay_recurrence_scan_wide_kernel<16> : tb::decay_recurrence_scan_wide_kernel<32>);
  if (smem > 48 * 1024) {
    const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  return tb::launch(kernel, dim3((dv + 31) / 32, H, requests), dim3(nw * 32), smem, stream, proj, stride, cu_seqlens, state_slots,
                    state, decay, out, H, dk, dv);
}

// o float32 [T, H dv]; gate float32 rows of H dv values (stride gate_stride) or null; weight [H dv] or null (mode 1).
int tb_decay_recurrence_post(void* stream, const float* o, const float* gate, int gate_stride, const float* weight, void* y,
                             int T_tokens, int H, int dv, int mode, int gate_act, float eps, int dtype) {
  if (T_tokens <= 0) return 0;
  if (H <= 0 || dv <= 0 || mode < 0 || mode > 1 || gate_act < 0 || gate_act > 2) return TB_ERR_BAD_SIZE;
  TB_DISPATCH_DTYPE(dtype, tb::launch(tb::decay_recurrence_post_kernel<T>, dim3(T_tokens), dim3(256), 0, stream, o, gate, gate_stride,
                                      weight, (T*)y, H, dv, mode, gate_act, eps));
}

}  // extern "C"
