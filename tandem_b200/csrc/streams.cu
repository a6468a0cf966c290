// A residual of several parallel streams ("hyper-connections"), and the norm that reads it.
//
// X [T, S, H] float32 are S streams per token.  A sublayer reads u = sum_s read[s] X_s and, with its
// output y [T, H], every stream is rewritten from the old ones:
//
//   X_t <- sum_s mix[s, t] X_s + (mult * out[t]) * y            (mix indexed [from, to])
//
// One kernel does the write that the sublayer in front left pending (if any), then the read of the
// next sublayer and its RMSNorm: y_out = u * rsqrt(mean(u^2) + eps) * weight.  read == null sums the
// streams (the end of the model).  With S = 1, mix = out = read = 1 this is the plain "add into the
// residual, then normalise" with a factor on the added term.  All arithmetic is float32; the result is
// rounded once, to the storage type of the next product's input.  One block per output row; with
// `rows` only those rows are updated and returned.
#include "common.cuh"

namespace tb {

constexpr int MAX_STREAMS = 8;

template <typename T, typename Y>
__global__ void stream_norm_kernel(float* __restrict__ X, const Y* __restrict__ y, const float* __restrict__ mix,
                                   const float* __restrict__ outc, float mult, const float* __restrict__ read,
                                   const float* __restrict__ weight, T* __restrict__ u_out, const int* __restrict__ rows, int S,
                                   int H, float eps) {
  __shared__ float scratch[33];
  __shared__ float cm[MAX_STREAMS * MAX_STREAMS], co[MAX_STREAMS], cr[MAX_STREAMS];
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x;
  const int src = rows ? rows[r] : r;
  if (threadIdx.x < S * S) cm[threadIdx.x] = y ? mix[threadIdx.x] : 0.f;
  if (threadIdx.x < S) {
    co[threadIdx.x] = y ? mult * outc[threadIdx.x] : 0.f;
    cr[threadIdx.x] = read ? read[threadIdx.x] : 1.f;
  }
  __syncthreads();
  float* xs = X + (size_t)src * S * H;
  const Y* yr = y ? y + (size_t)src * H : nullptr;
  float ss = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float old[MAX_STREAMS];
#pragma unroll
    for (int s = 0; s < MAX_STREAMS; ++s) old[s] = s < S ? xs[(size_t)s * H + i] : 0.f;
    float u = 0.f;
    if (yr) {
      const float yv = to_float(yr[i]);
#pragma unroll
      for (int t = 0; t < MAX_STREAMS; ++t) {
        if (t < S) {
          float acc = 0.f;
#pragma unroll
          for (int s = 0; s < MAX_STREAMS; ++s)
            if (s < S) acc = fmaf(cm[s * S + t], old[s], acc);
          acc = fmaf(co[t], yv, acc);
          xs[(size_t)t * H + i] = acc;
          u = fmaf(cr[t], acc, u);
        }
      }
    } else {
#pragma unroll
      for (int t = 0; t < MAX_STREAMS; ++t)
        if (t < S) u = fmaf(cr[t], old[t], u);
    }
    ss = fmaf(u, u, ss);
  }
  if (!u_out) return;
  ss = block_sum(ss, scratch);
  const float inv = rsqrtf(ss / (float)H + eps);
  T* o = u_out + (size_t)r * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {  // the thread reads back what it wrote itself
    float u = 0.f;
#pragma unroll
    for (int t = 0; t < MAX_STREAMS; ++t)
      if (t < S) u = fmaf(cr[t], xs[(size_t)t * H + i], u);
    o[i] = from_float<T>(u * inv * weight[i]);
  }
}

}  // namespace tb

extern "C" {

// X float32 [T, S, H]; y [T, H] of type y_dtype (or null: nothing to write); mix [S, S], outc [S] (needed with y);
// read [S] or null (sum); weight [H]; u_out [rows, H] of type dtype (null: only the write); rows int32 or null.
int tb_stream_norm(void* stream, float* X, const void* y, int y_dtype, const float* mix, const float* outc, float mult,
                   const float* read, const float* weight, void* u_out, const int* rows, int num_rows, int S, int H, float eps,
                   int dtype) {
  if (num_rows <= 0) return 0;
  if (S <= 0 || S > tb::MAX_STREAMS || H <= 0 || (y && (!mix || !outc)) || (u_out && !weight)) return TB_ERR_BAD_SIZE;
  const int threads = H >= 4096 ? 512 : 256;
#define TB_STREAM(TT, YY)                                                                                                      \
  return tb::launch(tb::stream_norm_kernel<TT, YY>, dim3(num_rows), dim3(threads), 0, stream, X, (const YY*)y, mix, outc, mult, \
                    read, weight, (TT*)u_out, rows, S, H, eps)
  if (dtype == TB_F32 && (y_dtype == TB_F32 || !y)) TB_STREAM(float, float);
  if (dtype == TB_BF16 && (y_dtype == TB_F32 || !y)) TB_STREAM(__nv_bfloat16, float);
  if (dtype == TB_BF16 && y_dtype == TB_BF16) TB_STREAM(__nv_bfloat16, __nv_bfloat16);
#undef TB_STREAM
  return TB_ERR_BAD_DTYPE;
}

}  // extern "C"
