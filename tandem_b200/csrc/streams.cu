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

template <typename T, typename Y, bool VEC>
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
  T* o = u_out ? u_out + (size_t)r * H : nullptr;
  float ss = 0.f;
  if (VEC) {  // four neighbouring elements per thread and turn: 16-byte loads and stores (H a multiple of 4)
    for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
      float4 old[MAX_STREAMS];
#pragma unroll
      for (int s = 0; s < MAX_STREAMS; ++s)
        if (s < S) old[s] = *reinterpret_cast<const float4*>(xs + (size_t)s * H + i);
      float4 u = make_float4(0.f, 0.f, 0.f, 0.f);
      if (yr) {
        float4 yv;
        if (sizeof(Y) == 4) {
          yv = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(yr) + i);
        } else {
          const uint2 raw = *reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(yr) + i);
          const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
          const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
          yv = make_float4(lo.x, lo.y, hi.x, hi.y);
        }
#pragma unroll
        for (int t = 0; t < MAX_STREAMS; ++t) {
          if (t < S) {
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int s = 0; s < MAX_STREAMS; ++s)
              if (s < S) {
                const float m = cm[s * S + t];
                acc.x = fmaf(m, old[s].x, acc.x); acc.y = fmaf(m, old[s].y, acc.y);
                acc.z = fmaf(m, old[s].z, acc.z); acc.w = fmaf(m, old[s].w, acc.w);
              }
            acc.x = fmaf(co[t], yv.x, acc.x); acc.y = fmaf(co[t], yv.y, acc.y);
            acc.z = fmaf(co[t], yv.z, acc.z); acc.w = fmaf(co[t], yv.w, acc.w);
            *reinterpret_cast<float4*>(xs + (size_t)t * H + i) = acc;
            u.x = fmaf(cr[t], acc.x, u.x); u.y = fmaf(cr[t], acc.y, u.y);
            u.z = fmaf(cr[t], acc.z, u.z); u.w = fmaf(cr[t], acc.w, u.w);
          }
        }
      } else {
#pragma unroll
        for (int t = 0; t < MAX_STREAMS; ++t)
          if (t < S) {
            u.x = fmaf(cr[t], old[t].x, u.x); u.y = fmaf(cr[t], old[t].y, u.y);
            u.z = fmaf(cr[t], old[t].z, u.z); u.w = fmaf(cr[t], old[t].w, u.w);
          }
      }
      ss = fmaf(u.x, u.x, ss); ss = fmaf(u.y, u.y, ss); ss = fmaf(u.z, u.z, ss); ss = fmaf(u.w, u.w, ss);
    }
  } else {
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
  }
  if (!o) return;
  ss = block_sum(ss, scratch);
  const float inv = rsqrtf(ss / (float)H + eps);
  if (VEC) {  // the thread reads back what it wrote itself
    for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
      float4 u = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int t = 0; t < MAX_STREAMS; ++t)
        if (t < S) {
          const float4 v = *reinterpret_cast<const float4*>(xs + (size_t)t * H + i);
          u.x = fmaf(cr[t], v.x, u.x); u.y = fmaf(cr[t], v.y, u.y); u.z = fmaf(cr[t], v.z, u.z); u.w = fmaf(cr[t], v.w, u.w);
        }
      const float4 w = *reinterpret_cast<const float4*>(weight + i);
      if (sizeof(T) == 2)
        *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(o) + i) = make_uint2(pack2(u.x * inv * w.x, u.y * inv * w.y), pack2(u.z * inv * w.z, u.w * inv * w.w));
      else
        *reinterpret_cast<float4*>(reinterpret_cast<float*>(o) + i) = make_float4(u.x * inv * w.x, u.y * inv * w.y, u.z * inv * w.z, u.w * inv * w.w);
    }
    return;
  }
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
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
  const bool vec = (H & 3) == 0 && (((uintptr_t)X | (uintptr_t)y | (uintptr_t)weight | (uintptr_t)u_out) & 15) == 0;
#define TB_STREAM(TT, YY)                                                                                                              \
  return vec ? tb::launch(tb::stream_norm_kernel<TT, YY, true>, dim3(num_rows), dim3(threads), 0, stream, X, (const YY*)y, mix, outc,  \
                          mult, read, weight, (TT*)u_out, rows, S, H, eps)                                                              \
             : tb::launch(tb::stream_norm_kernel<TT, YY, false>, dim3(num_rows), dim3(threads), 0, stream, X, (const YY*)y, mix, outc, \
                          mult, read, weight, (TT*)u_out, rows, S, H, eps)
  if (dtype == TB_F32 && (y_dtype == TB_F32 || !y)) TB_STREAM(float, float);
  if (dtype == TB_BF16 && (y_dtype == TB_F32 || !y)) TB_STREAM(__nv_bfloat16, float);
  if (dtype == TB_BF16 && y_dtype == TB_BF16) TB_STREAM(__nv_bfloat16, __nv_bfloat16);
#undef TB_STREAM
  return TB_ERR_BAD_DTYPE;
}

}  // extern "C"
