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
//
// The scan also serves recurrences whose decay is made from the token (`decay_tok` [T, H]: the decay of
// head h at token t replaces the fixed one) and whose q and k are shared by groups of heads (`qk_heads`
// sets of q and k for H heads of v: head h reads set h / (H / qk_heads)); where q, k and v start in a row
// and how far apart the states of two slots lie are arguments.  For such a "selective" state-space layer
// S <- exp(-exp(A_log_h) dt) S + dt B x^T, y = S^T C + D_h x  is the scan with q = C, k = B, v = dt x and
// decay exp(-exp(A_log_h) dt): `selective_prep` makes those rows from the layer's projection (a causal
// convolution per channel over the request's earlier inputs, the last of which it finds in the request's
// state, SiLU, softplus of the step size), `conv_state_update` leaves the newest inputs in the state, and
// `selective_post` adds D x, multiplies by SiLU(z), then divides by the root mean square in equal parts
// of the row and multiplies by a weight.
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
                                              int v_cols, int dk, int dkp, float* q_s, float* k_s, float* v_s, bool vec,
                                              const float* decay_tok, int H, int h, float* g_s) {
  if (decay_tok && (int)threadIdx.x < n) g_s[threadIdx.x] = decay_tok[(size_t)(c0 + threadIdx.x) * H + h];  // read two turns later
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
                                                           const float* __restrict__ decay, float* __restrict__ out, int H, int dk, int dv,
                                                           const float* __restrict__ decay_tok, int qk_heads, int q_off, int k_off,
                                                           int v_off, long long state_stride) {
  extern __shared__ __align__(16) float smem[];
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const int dkp = nw * R;  // dk rounded up to whole warps
  const int stage_floats = 2 * DR_CHUNK * dkp + DR_CHUNK * 32 + DR_CHUNK;  // q, k, v and the decays of a stage
  float* part_s = smem + 2 * stage_floats;                      // [DR_CHUNK][nw][32]
  const int h = blockIdx.y, b = blockIdx.z;
  const int j = blockIdx.x * 32 + lane;       // this thread's column of S
  const bool col_ok = j < dv;
  const int t0 = cu_seqlens[b], t1 = cu_seqlens[b + 1];
  if (t1 <= t0) return;
  const float g_fixed = decay ? decay[h] : 1.f;
  float* S = state + (size_t)state_slots[b] * state_stride + ((size_t)h * dk) * dv;
  float s[R];
#pragma unroll
  for (int i = 0; i < R; ++i) {
    const int d = w * R + i;
    s[i] = (col_ok && d < dk) ? S[(size_t)d * dv + j] : 0.f;
  }
  for (int e = threadIdx.x; e < 2 * stage_floats; e += blockDim.x) smem[e] = 0.f;  // rows beyond dk and columns beyond dv stay zero
  __syncthreads();
  const int set = h / (H / qk_heads);  // which q and k the head reads
  const int q_col = q_off + set * dk, k_col = k_off + set * dk, v_col = v_off + h * dv + blockIdx.x * 32;
  const int v_cols = min(32, dv - blockIdx.x * 32);
  const bool vec = ((dk | dv | stride | q_off | k_off | v_off) & 3) == 0 && (reinterpret_cast<uintptr_t>(proj) & 15) == 0;
  dr_load_stage(proj, stride, t0, min(DR_CHUNK, t1 - t0), q_col, k_col, v_col, v_cols, dk, dkp, smem, smem + DR_CHUNK * dkp,
                smem + 2 * DR_CHUNK * dkp, vec, decay_tok, H, h, smem + 2 * DR_CHUNK * dkp + DR_CHUNK * 32);
  int slot = 0;
  for (int c0 = t0; c0 < t1; c0 += DR_CHUNK, slot ^= 1) {
    const int n = min(DR_CHUNK, t1 - c0);
    if (c0 + DR_CHUNK < t1) {
      float* nxt = smem + (slot ^ 1) * stage_floats;
      dr_load_stage(proj, stride, c0 + DR_CHUNK, min(DR_CHUNK, t1 - c0 - DR_CHUNK), q_col, k_col, v_col, v_cols, dk, dkp, nxt,
                    nxt + DR_CHUNK * dkp, nxt + 2 * DR_CHUNK * dkp, vec, decay_tok, H, h, nxt + 2 * DR_CHUNK * dkp + DR_CHUNK * 32);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    const float* q_s = smem + slot * stage_floats;
    const float* k_s = q_s + DR_CHUNK * dkp;
    const float* v_s = k_s + DR_CHUNK * dkp;
    const float* g_s = v_s + DR_CHUNK * 32;
    for (int c = 0; c < n; ++c) {
      const float g = decay_tok ? g_s[c] : g_fixed;
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
                                             const float* __restrict__ decay, float* __restrict__ out, int H, int dk, int dv,
                                             const float* __restrict__ decay_tok, int qk_heads, int q_off, int k_off, int v_off,
                                             long long state_stride) {
  decay_recurrence_scan_body<16>(proj, stride, cu_seqlens, state_slots, state, decay, out, H, dk, dv, decay_tok, qk_heads, q_off,
                                 k_off, v_off, state_stride);
}
template <int R>
__global__ void __launch_bounds__(1024)
decay_recurrence_scan_wide_kernel(const float* __restrict__ proj, int stride, const int* __restrict__ cu_seqlens,
                                  const int* __restrict__ state_slots, float* __restrict__ state, const float* __restrict__ decay,
                                  float* __restrict__ out, int H, int dk, int dv, const float* __restrict__ decay_tok, int qk_heads,
                                  int q_off, int k_off, int v_off, long long state_stride) {
  decay_recurrence_scan_body<R>(proj, stride, cu_seqlens, state_slots, state, decay, out, H, dk, dv, decay_tok, qk_heads, q_off,
                                k_off, v_off, state_stride);
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

// ---------------------------------------------------------------------------------------------
// The selective layer's prologue.  proj float32 [T, stride] = [z: inner | u: C channels | dt: H | ...] with the
// channels u = [x: inner | B: G N | C: G N] and inner = H P.  One thread per (token, channel):
//   c_t = SiLU(bias + sum_j taps[K-1-j] u_(t-j)),  u before this step's first token from the request's state
//   (the inputs at positions start-(K-1) .. start-1, zeros in front of the sequence), float32 [slots][K-1][C].
// Written to rows [x | B | C | dt x] (stride 2 inner + 2 G N) for the scan and the epilogue.  dt = softplus(dt + dt_bias)
// and the heads' decays exp(-exp(A_log) dt) are made once per (token, head) by a small kernel in front.
__device__ __forceinline__ float softplus_f(float x) { return fmaxf(x, 0.f) + log1pf(expf(-fabsf(x))); }

// One thread per (token, head): dt = softplus(dt + dt_bias) and the head's decay exp(-exp(A_log) dt).
__global__ void selective_step_kernel(const float* __restrict__ proj, int stride, int dt_col, const float* __restrict__ dt_bias,
                                      const float* __restrict__ a_log, float* __restrict__ dt_out, float* __restrict__ decay, int total,
                                      int H) {
  pdl_launch_dependents();
  pdl_wait();
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const int t = idx / H, h = idx % H;
  const float dt = softplus_f(proj[(size_t)t * stride + dt_col + h] + dt_bias[h]);
  dt_out[idx] = dt;
  decay[idx] = expf(-expf(a_log[h]) * dt);
}

__global__ void selective_prep_kernel(const float* __restrict__ proj, int stride, const float* __restrict__ taps,
                                      const float* __restrict__ conv_bias, const float* __restrict__ dt,
                                      const float* __restrict__ conv_state, long long state_stride,
                                      const int* __restrict__ seq_of_token, const int* __restrict__ positions,
                                      const int* __restrict__ seq_starts, const int* __restrict__ state_slots,
                                      float* __restrict__ rows, long long total, int H, int P, int GN2, int K) {
  pdl_launch_dependents();
  pdl_wait();
  const int inner = H * P, C = inner + GN2, out_stride = 2 * inner + GN2;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
    const int t = (int)(idx / C), c = (int)(idx % C);
    const int b = seq_of_token[t];
    const int local = positions[t] - seq_starts[b];  // tokens of the request in this step in front of this one
    const float* old = conv_state + (size_t)state_slots[b] * state_stride;
    float acc = conv_bias[c];
    for (int j = K - 1; j >= 0; --j) {  // oldest input first
      const float u = j <= local ? proj[(size_t)(t - j) * stride + inner + c] : old[(size_t)(local - j + K - 1) * C + c];
      acc = fmaf(taps[(size_t)c * K + (K - 1 - j)], u, acc);
    }
    const float v = acc / (1.f + expf(-acc));
    float* row = rows + (size_t)t * out_stride;
    row[c] = v;
    if (c < inner) row[inner + GN2 + c] = dt[(size_t)t * H + c / P] * v;
  }
}

// One thread per (request, channel): the last K-1 inputs of the convolution after this step, oldest first.
__global__ void conv_state_update_kernel(const float* __restrict__ proj, int stride, int col0, float* __restrict__ conv_state,
                                         long long state_stride, const int* __restrict__ cu_seqlens,
                                         const int* __restrict__ state_slots, int requests, int C, int K) {
  pdl_launch_dependents();
  pdl_wait();
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)requests * C) return;
  const int b = (int)(idx / C), c = (int)(idx % C);
  const int t0 = cu_seqlens[b], n = cu_seqlens[b + 1] - t0;
  if (n <= 0) return;
  float* st = conv_state + (size_t)state_slots[b] * state_stride;
  for (int k = 0; k < K - 1; ++k) {  // entry k moves down by n places: st[k + n] is read before any turn writes it
    const int i = n - (K - 1) + k;   // the token of this step that the entry holds, if not negative
    st[(size_t)k * C + c] = i >= 0 ? proj[(size_t)(t0 + i) * stride + col0 + c] : st[(size_t)(k + n) * C + c];
  }
}

// y = (o + D_h x) * SiLU(z), divided by its root mean square in `parts` equal parts of the row, times weight.
// grid (tokens, parts).  o float32 [T, H P]; x at rows[t][0 .. H P); z at proj[t][0 .. H P).
constexpr int SP_KEEP = 8;  // values a thread keeps between the two passes

template <typename T>
__global__ void selective_post_kernel(const float* __restrict__ o, const float* __restrict__ rows, int rows_stride,
                                      const float* __restrict__ z, int z_stride, const float* __restrict__ D,
                                      const float* __restrict__ weight, T* __restrict__ y, int H, int P, int parts, float eps) {
  __shared__ float scratch[33];
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x, part = blockIdx.y, n = H * P / parts, c0 = part * n;
  const float* orow = o + (size_t)t * H * P;
  const float* xrow = rows + (size_t)t * rows_stride;
  const float* zrow = z + (size_t)t * z_stride;
  const bool keep = n <= SP_KEEP * (int)blockDim.x;  // else the second pass computes the values again
  float held[SP_KEEP];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < SP_KEEP; ++i) {
    const int c = c0 + threadIdx.x + i * blockDim.x;
    held[i] = 0.f;
    if (keep && c < c0 + n) {
      const float zz = zrow[c];
      held[i] = fmaf(D[c / P], xrow[c], orow[c]) * (zz / (1.f + expf(-zz)));
      ss = fmaf(held[i], held[i], ss);
    }
  }
  if (!keep)
    for (int c = c0 + threadIdx.x; c < c0 + n; c += blockDim.x) {
      const float zz = zrow[c];
      const float v = fmaf(D[c / P], xrow[c], orow[c]) * (zz / (1.f + expf(-zz)));
      ss = fmaf(v, v, ss);
    }
  ss = block_sum(ss, scratch);
  const float inv = rsqrtf(ss / (float)n + eps);
  if (keep) {
#pragma unroll
    for (int i = 0; i < SP_KEEP; ++i) {
      const int c = c0 + threadIdx.x + i * blockDim.x;
      if (c < c0 + n) y[(size_t)t * H * P + c] = from_float<T>(held[i] * inv * weight[c]);
    }
    return;
  }
  for (int c = c0 + threadIdx.x; c < c0 + n; c += blockDim.x) {
    const float zz = zrow[c];
    const float v = fmaf(D[c / P], xrow[c], orow[c]) * (zz / (1.f + expf(-zz)));
    y[(size_t)t * H * P + c] = from_float<T>(v * inv * weight[c]);
  }
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

// The scan with everything as an argument.  state float32: slot s begins at state + s * state_stride and holds
// [H, dk, dv]; out float32 [T, H dv]; cu_seqlens [requests + 1]; state_slots [requests]; decay [H] or null (1);
// decay_tok [T, H] or null; q of set i at column q_off + i dk, k at k_off + i dk, v of head h at v_off + h dv.
int tb_recurrence_scan(void* stream, const float* proj, int stride, const int* cu_seqlens, const int* state_slots,
                       float* state, long long state_stride, const float* decay, const float* decay_tok, float* out, int requests,
                       int H, int qk_heads, int dk, int dv, int q_off, int k_off, int v_off) {
  if (requests <= 0) return 0;
  if (H <= 0 || dk <= 0 || dk > 1024 || dv <= 0 || H > 65535 || requests > 65535 || qk_heads <= 0 || H % qk_heads ||
      state_stride < (long long)H * dk * dv || q_off < 0 || k_off < 0 || v_off < 0)
    return TB_ERR_BAD_SIZE;
  const int R = dk <= 512 ? 16 : 32;
  const int nw = (dk + R - 1) / R, dkp = nw * R;
  const size_t smem = (size_t)(2 * (2 * tb::DR_CHUNK * dkp + tb::DR_CHUNK * 32 + tb::DR_CHUNK) + tb::DR_CHUNK * nw * 32) * sizeof(float);
  auto kernel = dk <= 256 ? tb::decay_recurrence_scan_kernel
                          : (R == 16 ? tb::decay_recurrence_scan_wide_kernel<16> : tb::decay_recurrence_scan_wide_kernel<32>);
  if (smem > 48 * 1024) {
    const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  return tb::launch(kernel, dim3((dv + 31) / 32, H, requests), dim3(nw * 32), smem, stream, proj, stride, cu_seqlens, state_slots,
                    state, decay, out, H, dk, dv, decay_tok, qk_heads, q_off, k_off, v_off, state_stride);
}

// The fixed-decay layout: columns [q: H dk | k: H dk | v: H dv], state float32 [slots, H, dk, dv].
int tb_decay_recurrence_scan(void* stream, const float* proj, int stride, const int* cu_seqlens, const int* state_slots,
                             float* state, const float* decay, float* out, int requests, int H, int dk, int dv) {
  return tb_recurrence_scan(stream, proj, stride, cu_seqlens, state_slots, state, (long long)H * dk * dv, decay, nullptr, out,
                            requests, H, H, dk, dv, 0, H * dk, 2 * H * dk);
}

// proj float32 [T, stride >= 2 H P + GN2 + H]; taps [H P + GN2, K]; conv_state: slot s at conv_state + s * state_stride,
// [K - 1][H P + GN2]; rows float32 [T, 2 H P + GN2] = [x | B | C | dt x]; decay and dt float32 [T, H].
int tb_selective_prep(void* stream, const float* proj, int stride, const float* taps, const float* conv_bias, const float* dt_bias,
                      const float* a_log, const float* conv_state, long long state_stride, const int* seq_of_token,
                      const int* positions, const int* seq_starts, const int* state_slots, float* rows, float* decay, float* dt,
                      int T_tokens, int H, int P, int GN2, int K) {
  if (T_tokens <= 0) return 0;
  if (H <= 0 || P <= 0 || GN2 < 0 || K <= 0 || stride < 2 * H * P + GN2 + H) return TB_ERR_BAD_SIZE;
  if ((long long)T_tokens * H > 0x7fffffffLL) return TB_ERR_BAD_SIZE;
  const int steps = T_tokens * H;
  int rc = tb::launch(tb::selective_step_kernel, dim3((steps + 255) / 256), dim3(256), 0, stream, proj, stride, 2 * H * P + GN2, dt_bias,
                      a_log, dt, decay, steps, H);
  if (rc != 0) return rc;
  const long long total = (long long)T_tokens * (H * P + GN2);
  long long blocks = (total + 255) / 256;
  if (blocks > 148 * 64) blocks = 148 * 64;
  return tb::launch(tb::selective_prep_kernel, dim3((int)blocks), dim3(256), 0, stream, proj, stride, taps, conv_bias, (const float*)dt,
                    conv_state, state_stride, seq_of_token, positions, seq_starts, state_slots, rows, total, H, P, GN2, K);
}

int tb_conv_state_update(void* stream, const float* proj, int stride, int col0, float* conv_state, long long state_stride,
                         const int* cu_seqlens, const int* state_slots, int requests, int C, int K) {
  if (requests <= 0 || K <= 1) return 0;
  if (C <= 0 || col0 < 0) return TB_ERR_BAD_SIZE;
  const long long total = (long long)requests * C;
  return tb::launch(tb::conv_state_update_kernel, dim3((int)((total + 255) / 256)), dim3(256), 0, stream, proj, stride, col0,
                    conv_state, state_stride, cu_seqlens, state_slots, requests, C, K);
}

int tb_selective_post(void* stream, const float* o, const float* rows, int rows_stride, const float* z, int z_stride, const float* D,
                      const float* weight, void* y, int T_tokens, int H, int P, int parts, float eps, int dtype) {
  if (T_tokens <= 0) return 0;
  if (H <= 0 || P <= 0 || parts <= 0 || (H * P) % parts || parts > 65535) return TB_ERR_BAD_SIZE;
  const int n = H * P / parts;
  const int threads = n >= 8192 ? 1024 : n >= 2048 ? 512 : 256;
  TB_DISPATCH_DTYPE(dtype, tb::launch(tb::selective_post_kernel<T>, dim3(T_tokens, parts), dim3(threads), 0, stream, o, rows, rows_stride,
                                      z, z_stride, D, weight, (T*)y, H, P, parts, eps));
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
