// Several residual streams per token, kept in float: the update after a sublayer and the combination before the next,
// fused with the norm that the next sublayer begins with.
//
// A token has S streams x_1..x_S of D floats, stored [token][stream][D].  One launch does, for every token,
//   (1) either the start:   x_s = e  for all s (e: the embedded token), or, with y the output of the sublayer before,
//       the update:         x'_t = sum_s M[s][t] x_s + b[t] * y      (the sum runs over the streams as they were; M is [from][to])
//   (2) and, if asked:      u = sum_s a[s] x'_s ;  out = u / sqrt(mean(u^2) + eps) * g      (g: one number)
// so that a sublayer costs one pass over the streams: S*D floats read and written, where the fused add+norm of a
// single bfloat16 stream moves a quarter of that.  With one stream and M = a = b = 1 this is the plain residual sum in
// float.  With a list of rows the combination is computed for those source rows only and nothing is stored (the model's
// last norm, on the rows whose logits are wanted; a row may be named twice).
//
// Everything is float; y, e and out are of the model's type T.  The sum of squares is taken by a block of fixed size,
// so its order of additions depends on D only.
#include "common.cuh"

namespace vob {

constexpr int STREAM_NT = 256;

template <typename T, int MAXS>
__global__ void __launch_bounds__(STREAM_NT)
stream_step_kernel(float* streams, const T* y, const T* init, const float* __restrict__ mix, const float* __restrict__ out_w,
                   const float* __restrict__ in_w, const float* __restrict__ gain, T* normed, const int* __restrict__ rows,
                   int num_src_rows, int S, int D, float eps, int* err) {
  extern __shared__ float urow[];  // D floats: the combined row (only with `normed`)
  __shared__ float scratch[32];
  __shared__ float cm[MAXS * MAXS], co[MAXS], ci[MAXS];
  pdl_launch_dependents();
  for (int i = threadIdx.x; i < S * S; i += STREAM_NT) cm[i] = mix ? mix[i] : ((i / S == i % S) ? 1.f : 0.f);
  for (int i = threadIdx.x; i < S; i += STREAM_NT) {
    co[i] = out_w ? out_w[i] : 1.f;
    ci[i] = in_w ? in_w[i] : 1.f;
  }
  const float g = gain ? gain[0] : 1.f;
  pdl_wait();
  const int r = blockIdx.x;
  int src = r;
  if (rows) {
    src = rows[r];
    if (src < 0 || src >= num_src_rows) {
      if (threadIdx.x == 0) atomicOr(err, VOB_ERR_ROW);
      return;
    }
  }
  __syncthreads();
  float* xs = streams + (size_t)src * S * D;
  const bool store = rows == nullptr;
  float ss = 0.f;
  for (int d = threadIdx.x; d < D; d += STREAM_NT) {
    float x[MAXS];
    if (init) {
      const float e = to_f<T>(init[(size_t)src * D + d]);
#pragma unroll
      for (int s = 0; s < MAXS; ++s)
        if (s < S) {
          x[s] = e;
          if (store) xs[(size_t)s * D + d] = e;
        }
    } else {
#pragma unroll
      for (int s = 0; s < MAXS; ++s) x[s] = s < S ? xs[(size_t)s * D + d] : 0.f;
      if (y) {
        const float yv = to_f<T>(y[(size_t)src * D + d]);
        float nx[MAXS];
#pragma unroll
        for (int t = 0; t < MAXS; ++t) {
          float a = 0.f;
          if (t < S) {
#pragma unroll
            for (int s = 0; s < MAXS; ++s)
              if (s < S) a = fmaf(cm[s * S + t], x[s], a);
            a = fmaf(co[t], yv, a);
            if (store) xs[(size_t)t * D + d] = a;
          }
          nx[t] = a;
        }
#pragma unroll
        for (int s = 0; s < MAXS; ++s) x[s] = nx[s];
      }
    }
    if (normed) {
      float u = 0.f;
#pragma unroll
      for (int s = 0; s < MAXS; ++s)
        if (s < S) u = fmaf(ci[s], x[s], u);
      urow[d] = u;
      ss += u * u;
    }
  }
  if (!normed) return;
  const float total = block_sum<STREAM_NT>(ss, scratch);
  const float denom = sqrtf(total / (float)D + eps);
  for (int d = threadIdx.x; d < D; d += STREAM_NT) normed[(size_t)r * D + d] = from_f<T>(urow[d] / denom * g);
}

// The same with 16-byte accesses: a thread takes four neighbouring elements of every stream (D a multiple of 4, rows that
// start on 16-byte boundaries).  Which of the two kernels runs depends on D and S alone.
template <typename T> __device__ __forceinline__ void load4(const T* p, float (&v)[4]);
template <> __device__ __forceinline__ void load4<float>(const float* p, float (&v)[4]) {
  const float4 r = *reinterpret_cast<const float4*>(p);
  v[0] = r.x; v[1] = r.y; v[2] = r.z; v[3] = r.w;
}
template <> __device__ __forceinline__ void load4<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[4]) {
  const uint2 r = *reinterpret_cast<const uint2*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&r);
  const float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]);
  v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
}
template <typename T> __device__ __forceinline__ void store4(T* p, const float (&v)[4]);
template <> __device__ __forceinline__ void store4<float>(float* p, const float (&v)[4]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
template <> __device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16* p, const float (&v)[4]) {
  uint2 r;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&r);
  h[0] = __floats2bfloat162_rn(v[0], v[1]);
  h[1] = __floats2bfloat162_rn(v[2], v[3]);
  *reinterpret_cast<uint2*>(p) = r;
}

template <typename T, int MAXS>
__global__ void __launch_bounds__(STREAM_NT)
stream_step_vec_kernel(float* streams, const T* y, const T* init, const float* __restrict__ mix, const float* __restrict__ out_w,
                       const float* __restrict__ in_w, const float* __restrict__ gain, T* normed, const int* __restrict__ rows,
                       int num_src_rows, int S, int D, float eps, int* err) {
  extern __shared__ float4 urow4[];  // D floats: the combined row (only with `normed`)
  float* urow = reinterpret_cast<float*>(urow4);
  __shared__ float scratch[32];
  __shared__ float cm[MAXS * MAXS], co[MAXS], ci[MAXS];
  pdl_launch_dependents();
  for (int i = threadIdx.x; i < S * S; i += STREAM_NT) cm[i] = mix ? mix[i] : ((i / S == i % S) ? 1.f : 0.f);
  for (int i = threadIdx.x; i < S; i += STREAM_NT) {
    co[i] = out_w ? out_w[i] : 1.f;
    ci[i] = in_w ? in_w[i] : 1.f;
  }
  const float g = gain ? gain[0] : 1.f;
  pdl_wait();
  const int r = blockIdx.x;
  int src = r;
  if (rows) {
    src = rows[r];
    if (src < 0 || src >= num_src_rows) {
      if (threadIdx.x == 0) atomicOr(err, VOB_ERR_ROW);
      return;
    }
  }
  __syncthreads();
  float* xs = streams + (size_t)src * S * D;
  const bool store = rows == nullptr;
  float ss = 0.f;
  for (int d = threadIdx.x * 4; d < D; d += STREAM_NT * 4) {
    float x[MAXS][4];
    if (init) {
      float e[4];
      load4<T>(init + (size_t)src * D + d, e);
#pragma unroll
      for (int s = 0; s < MAXS; ++s)
        if (s < S) {
#pragma unroll
          for (int k = 0; k < 4; ++k) x[s][k] = e[k];
          if (store) store4<float>(xs + (size_t)s * D + d, e);
        }
    } else {
#pragma unroll
      for (int s = 0; s < MAXS; ++s) {
        if (s < S) load4<float>(xs + (size_t)s * D + d, x[s]);
        else x[s][0] = x[s][1] = x[s][2] = x[s][3] = 0.f;
      }
      if (y) {
        float yv[4], nx[MAXS][4];
        load4<T>(y + (size_t)src * D + d, yv);
#pragma unroll
        for (int t = 0; t < MAXS; ++t) {
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            float a = 0.f;
            if (t < S) {
#pragma unroll
              for (int s = 0; s < MAXS; ++s)
                if (s < S) a = fmaf(cm[s * S + t], x[s][k], a);
              a = fmaf(co[t], yv[k], a);
            }
            nx[t][k] = a;
          }
          if (t < S && store) store4<float>(xs + (size_t)t * D + d, nx[t]);
        }
#pragma unroll
        for (int s = 0; s < MAXS; ++s)
#pragma unroll
          for (int k = 0; k < 4; ++k) x[s][k] = nx[s][k];
      }
    }
    if (normed) {
      float u[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        float a = 0.f;
#pragma unroll
        for (int s = 0; s < MAXS; ++s)
          if (s < S) a = fmaf(ci[s], x[s][k], a);
        u[k] = a;
        ss += a * a;
      }
      store4<float>(urow + d, u);
    }
  }
  if (!normed) return;
  const float total = block_sum<STREAM_NT>(ss, scratch);
  const float denom = sqrtf(total / (float)D + eps);
  for (int d = threadIdx.x * 4; d < D; d += STREAM_NT * 4) {
    float u[4];
    load4<float>(urow + d, u);
#pragma unroll
    for (int k = 0; k < 4; ++k) u[k] = u[k] / denom * g;
    store4<T>(normed + (size_t)r * D + d, u);
  }
}

// sums[t] = sum_s x_s (float [T, D]): what a single-stream model would call its residual stream.
template <int MAXS>
__global__ void stream_sum_kernel(const float* streams, float* sums, int S, int D) {
  const int t = blockIdx.x;
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float u = 0.f;
    for (int s = 0; s < S; ++s) u += streams[((size_t)t * S + s) * D + d];
    sums[(size_t)t * D + d] = u;
  }
}

template <typename T, int MAXS>
int launch_stream_step(float* streams, const void* y, const void* init, const float* mix, const float* out_w, const float* in_w,
                       const float* gain, void* normed, const int* rows, int n_out, int n_src, int S, int D, float eps, int* err,
                       cudaStream_t stream) {
  const size_t smem = normed ? (size_t)D * sizeof(float) : 0;
  auto aligned = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  const bool vec = MAXS <= 8 && D % 4 == 0 && aligned(streams) && aligned(y) && aligned(init) && aligned(normed);
  auto k = vec ? stream_step_vec_kernel<T, (MAXS <= 8 ? MAXS : 1)> : stream_step_kernel<T, MAXS>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  return launch_kernel(k, dim3(n_out), dim3(STREAM_NT), smem, stream, streams, (const T*)y, (const T*)init, mix, out_w, in_w, gain,
                       (T*)normed, rows, n_src, S, D, eps, err);
}

}  // namespace vob

using namespace vob;

// streams float [n_src, S, D]; y, init [n_src, D] or null; mix [S,S], out_w [S], in_w [S] float or null (identity / ones);
// gain one float or null (1); normed [n_out, D] or null; rows [n_out] or null (then n_out must equal n_src).
VOB_API int vob_stream_step(float* streams, const void* y, const void* init, const float* mix, const float* out_w,
                            const float* in_w, const float* gain, void* normed, const int* rows, int n_out, int n_src, int S,
                            int D, float eps, int dtype, int* err, cudaStream_t stream) {
  if (n_out <= 0) return 0;
  if (S <= 0 || S > 16 || D <= 0 || (D > 56 * 1024) || (!rows && n_out != n_src)) return VOB_UNSUPPORTED;
#define VOB_STREAM_CASE(TT, MS) \
  return launch_stream_step<TT, MS>(streams, y, init, mix, out_w, in_w, gain, normed, rows, n_out, n_src, S, D, eps, err, stream)
  if (dtype == VOB_F32) {
    if (S <= 1) VOB_STREAM_CASE(float, 1);
    if (S <= 4) VOB_STREAM_CASE(float, 4);
    if (S <= 8) VOB_STREAM_CASE(float, 8);
    VOB_STREAM_CASE(float, 16);
  }
  if (dtype == VOB_BF16) {
    if (S <= 1) VOB_STREAM_CASE(__nv_bfloat16, 1);
    if (S <= 4) VOB_STREAM_CASE(__nv_bfloat16, 4);
    if (S <= 8) VOB_STREAM_CASE(__nv_bfloat16, 8);
    VOB_STREAM_CASE(__nv_bfloat16, 16);
  }
#undef VOB_STREAM_CASE
  return VOB_BAD_ARGUMENT;
}

VOB_API int vob_stream_sum(const float* streams, float* sums, int T, int S, int D, cudaStream_t stream) {
  if (T <= 0) return 0;
  stream_sum_kernel<16><<<T, 256, 0, stream>>>(streams, sums, S, D);
  return launch_status();
}
