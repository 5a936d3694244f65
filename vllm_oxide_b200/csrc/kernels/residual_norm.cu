// One float residual stream with a norm on both sides of every sublayer ("sandwich" norms):
//
//     x <- x + RMSNorm(y) * w_post          y: the output of the sublayer before (mixer or feed-forward)
//     h  = RMSNorm(x) * w_pre               what the next sublayer reads
//
// One launch does, for every token, any part of that chain in a single pass over the row:
//   (1) x = 0 (`init`: the row begins here, e.g. with the embedded token as y) or x = stream[token];
//   (2) with y:       x += y / sqrt(mean(y^2) + eps) * w_post      (w_post null: x += y)
//   (3) with inject:  x += inject[token]                           (a float row added as it is)
//   (4) x is stored to the stream if (1)-(3) changed it, and to `keep` if given (a second copy that later steps add back);
//   (5) with w_pre:   out = x / sqrt(mean(x^2) + eps) * w_pre.
// With a list of rows, (5) is computed for those source rows only and nothing is stored (the model's last norm on the
// rows whose logits are wanted).
//
// The stream, the norms and the sums are float on both paths; y and out are of the model's type T.  A block of fixed
// size takes a row, so the order of additions in a sum of squares depends on the row's width only.
#include "common.cuh"

namespace vob {

constexpr int RN_NT = 256;

template <typename T, int V> struct RowAccess;   // V elements at a time
template <typename T> struct RowAccess<T, 1> {
  static __device__ __forceinline__ void load(const T* p, float (&v)[1]) { v[0] = to_f<T>(p[0]); }
  static __device__ __forceinline__ void store(T* p, const float (&v)[1]) { p[0] = from_f<T>(v[0]); }
};
template <> struct RowAccess<float, 4> {
  static __device__ __forceinline__ void load(const float* p, float (&v)[4]) {
    const float4 r = *reinterpret_cast<const float4*>(p);
    v[0] = r.x; v[1] = r.y; v[2] = r.z; v[3] = r.w;
  }
  static __device__ __forceinline__ void store(float* p, const float (&v)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  }
};
template <> struct RowAccess<__nv_bfloat16, 4> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&v)[4]) {
    const uint2 r = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&r);
    const float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]);
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&v)[4]) {
    uint2 r;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&r);
    h[0] = __floats2bfloat162_rn(v[0], v[1]);
    h[1] = __floats2bfloat162_rn(v[2], v[3]);
    *reinterpret_cast<uint2*>(p) = r;
  }
};

template <typename T, int V>
__global__ void __launch_bounds__(RN_NT)
residual_norm_step_kernel(float* stream, const T* y, const float* __restrict__ w_post, const float* inject, float* keep,
                          const float* __restrict__ w_pre, T* out, const int* __restrict__ rows, int num_src_rows, int D,
                          float eps, int init, int* err) {
  extern __shared__ float4 rn_smem4[];
  float* xrow = reinterpret_cast<float*>(rn_smem4);   // [D] the new row
  float* yrow = xrow + D;                              // [D] the sublayer's output (only with y)
  __shared__ float scratch[32];
  pdl_launch_dependents();
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
  const size_t base = (size_t)src * D;
  float inv_y = 1.f;
  if (y) {
    float ss = 0.f;
    for (int d = threadIdx.x * V; d < D; d += RN_NT * V) {
      float v[V];
      RowAccess<T, V>::load(y + base + d, v);
#pragma unroll
      for (int j = 0; j < V; ++j) {
        yrow[d + j] = v[j];
        ss = fmaf(v[j], v[j], ss);
      }
    }
    const float total = block_sum<RN_NT>(ss, scratch);
    if (w_post) inv_y = 1.f / sqrtf(total / (float)D + eps);
  }
  const bool changed = init || y || inject;
  const bool store = rows == nullptr;
  float ss = 0.f;
  for (int d = threadIdx.x * V; d < D; d += RN_NT * V) {
    float x[V];
    if (init) {
#pragma unroll
      for (int j = 0; j < V; ++j) x[j] = 0.f;
    } else {
      RowAccess<float, V>::load(stream + base + d, x);
    }
    if (y) {
#pragma unroll
      for (int j = 0; j < V; ++j) x[j] += w_post ? yrow[d + j] * inv_y * w_post[d + j] : yrow[d + j];
    }
    if (inject) {
      float e[V];
      RowAccess<float, V>::load(inject + base + d, e);
#pragma unroll
      for (int j = 0; j < V; ++j) x[j] += e[j];
    }
    if (store && changed) RowAccess<float, V>::store(stream + base + d, x);
    if (store && keep) RowAccess<float, V>::store(keep + base + d, x);
#pragma unroll
    for (int j = 0; j < V; ++j) {
      xrow[d + j] = x[j];
      ss = fmaf(x[j], x[j], ss);
    }
  }
  if (!out) return;
  const float total = block_sum<RN_NT>(ss, scratch);
  const float inv_x = 1.f / sqrtf(total / (float)D + eps);
  for (int d = threadIdx.x * V; d < D; d += RN_NT * V) {
    float o[V];
#pragma unroll
    for (int j = 0; j < V; ++j) o[j] = xrow[d + j] * inv_x * (w_pre ? w_pre[d + j] : 1.f);
    RowAccess<T, V>::store(out + (size_t)r * D + d, o);
  }
}

}  // namespace vob

using namespace vob;

// stream [num_src_rows, D] float; y [num_src_rows, D] and out [n_out, D] of `dtype`; w_post, w_pre [D] float; inject and
// keep [num_src_rows, D] float; rows [n_out] source rows or null (then n_out == num_src_rows).  Any of y, w_post, inject,
// keep, w_pre / out may be null.
VOB_API int vob_residual_norm_step(float* stream, const void* y, const float* w_post, const float* inject, float* keep,
                                   const float* w_pre, void* out, const int* rows, int n_out, int num_src_rows, int D,
                                   float eps, int init, int dtype, int* err, cudaStream_t stream_) {
  if (n_out <= 0) return 0;
  if (D <= 0 || (rows && (keep || !out))) return VOB_BAD_ARGUMENT;
  const size_t smem = (size_t)2 * D * sizeof(float);
  if (smem > 200 * 1024) return VOB_UNSUPPORTED;
  const bool vec = D % 4 == 0 && (((uintptr_t)stream | (uintptr_t)y | (uintptr_t)inject | (uintptr_t)keep | (uintptr_t)out |
                                    (uintptr_t)w_post | (uintptr_t)w_pre) % 16) == 0;
#define VOB_RN_LAUNCH(TYPE, V)                                                                                            \
  do {                                                                                                                    \
    if (smem > 48 * 1024)                                                                                                 \
      cudaFuncSetAttribute(residual_norm_step_kernel<TYPE, V>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);   \
    return launch_kernel(residual_norm_step_kernel<TYPE, V>, dim3(n_out), RN_NT, smem, stream_, stream, (const TYPE*)y,   \
                         w_post, inject, keep, w_pre, (TYPE*)out, rows, num_src_rows, D, eps, init, err);                 \
  } while (0)
  if (dtype == VOB_F32) {
    if (vec) VOB_RN_LAUNCH(float, 4);
    VOB_RN_LAUNCH(float, 1);
  }
  if (dtype == VOB_BF16) {
    if (vec) VOB_RN_LAUNCH(__nv_bfloat16, 4);
    VOB_RN_LAUNCH(__nv_bfloat16, 1);
  }
#undef VOB_RN_LAUNCH
  return VOB_BAD_ARGUMENT;
}
