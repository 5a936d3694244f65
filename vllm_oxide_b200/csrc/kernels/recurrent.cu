// Recurrent token mixers: the state of a request is carried in float from token to token, in a state slot.
//
// Both kernels walk the tokens of one request in order, whatever the step holds of it (a whole prompt, a portion, one
// decoded token), starting from the slot's state and leaving the new state there.  The chain of float operations of a
// channel therefore depends on the request's tokens only: not on how they were cut into steps nor on the batch.
// Projections come in the model's type T (bfloat16 when serving); gates, decays, the state and the norm are float.
#include "common.cuh"

namespace vob {

__device__ __forceinline__ float sigmoid_f(float x) { return 1.f / (1.f + expf(-x)); }

// ---------------------------------------------------------------- minGRU
// zxg [tokens, 3W]: pre-activations of the gate z, of the candidate u and of the output gate g (no bias yet).
//   z = sigmoid(z + bz);  c = u + bx;  c = c >= 0 ? c + 1/2 : sigmoid(c);  s = (1 - z) s + z c;  out = s * silu(g)
// One thread per (request, channel); neighbouring threads read neighbouring channels.
template <typename T>
__global__ void mingru_scan_kernel(const T* zxg, const T* __restrict__ bz, const T* __restrict__ bx, float* state,
                                   const int* __restrict__ cu_q, const int* __restrict__ state_slots, T* out, int W,
                                   int num_slots, int* err) {
  pdl_launch_dependents();
  const int b = blockIdx.y, c = blockIdx.x * blockDim.x + threadIdx.x;
  const int t0 = cu_q[b], t1 = cu_q[b + 1];
  const int slot = state_slots[b];
  const float biasz = c < W ? to_f<T>(bz[c]) : 0.f, biasx = c < W ? to_f<T>(bx[c]) : 0.f;
  pdl_wait();
  if (c >= W || t1 <= t0) return;
  if (slot < 0 || slot >= num_slots) {
    atomicOr(err, VOB_ERR_SLOT);
    return;
  }
  float s = state[(size_t)slot * W + c];
#pragma unroll 4
  for (int t = t0; t < t1; ++t) {
    const T* row = zxg + (size_t)t * 3 * W;
    const float z = sigmoid_f(to_f<T>(row[c]) + biasz);
    const float u = to_f<T>(row[W + c]) + biasx;
    const float g = to_f<T>(row[2 * W + c]);
    const float cand = u >= 0.f ? u + 0.5f : sigmoid_f(u);
    s = fmaf(z, cand, (1.f - z) * s);
    out[(size_t)t * W + c] = from_f<T>(s * (g * sigmoid_f(g)));
  }
  state[(size_t)slot * W + c] = s;
}

// ---------------------------------------------------------------- HGRN2
// qfv [tokens, heads*dk | heads*dk | heads*dv]: pre-activations of q and of the forget gate, and the values.
//   q = silu(q);  f = l + (1 - l) sigmoid(f + bf);  M = diag(f) M + (1 - f) v^T;  o = M^T q;  out = o / rms(o) * w
// A block owns (request, head) or a range of its value columns; thread j keeps column j of M (dk floats) in registers, so
// a token costs dk multiply-adds a thread and no exchange between threads.  The gates of HG_TT tokens are made by the
// whole block at once and parked in shared memory.  FUSE: the block holds all dv columns of the head and also takes
// the norm over them; otherwise o leaves in float and head_gain_norm_kernel follows.
constexpr int HG_TT = 8;

template <typename T, int R, bool FUSE>
__global__ void __launch_bounds__(128)
hgrn2_scan_kernel(const T* qfv, const T* __restrict__ bf, const float* __restrict__ lower, const float* __restrict__ nw,
                  float* state, const int* __restrict__ cu_q, const int* __restrict__ state_slots, T* out, float* raw,
                  int heads, int dk, int dv, int col_blocks, float eps, int num_slots, int* err) {
  extern __shared__ float sm[];
  float* qs = sm;                   // [HG_TT][dk]
  float* fs = qs + HG_TT * dk;      // [HG_TT][dk]
  float* os = fs + HG_TT * dk;      // [HG_TT][blockDim.x]
  pdl_launch_dependents();
  const int h = blockIdx.x / col_blocks, j = (blockIdx.x % col_blocks) * blockDim.x + threadIdx.x;
  const int b = blockIdx.y;
  const int t0 = cu_q[b], t1 = cu_q[b + 1];
  const int slot = state_slots[b];
  pdl_wait();
  if (t1 <= t0) return;
  if (slot < 0 || slot >= num_slots) {
    if (threadIdx.x == 0) atomicOr(err, VOB_ERR_SLOT);
    return;
  }
  const size_t width = (size_t)heads * (2 * dk + dv);
  float* mine = state + (((size_t)slot * heads + h) * dk) * dv + j;
  float M[R];
#pragma unroll
  for (int i = 0; i < R; ++i) M[i] = (i < dk && j < dv) ? mine[(size_t)i * dv] : 0.f;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  for (int ts = t0; ts < t1; ts += HG_TT) {
    const int n = min(HG_TT, t1 - ts);
    for (int idx = threadIdx.x; idx < n * dk; idx += blockDim.x) {
      const int tt = idx / dk, i = idx % dk;
      const T* row = qfv + (size_t)(ts + tt) * width;
      const float qv = to_f<T>(row[h * dk + i]);
      qs[tt * dk + i] = qv * sigmoid_f(qv);
      const float l = lower[h * dk + i];
      fs[tt * dk + i] = l + (1.f - l) * sigmoid_f(to_f<T>(row[(heads + h) * dk + i]) + to_f<T>(bf[h * dk + i]));
    }
    __syncthreads();
    for (int tt = 0; tt < n; ++tt) {
      float o = 0.f;
      if (j < dv) {
        const float v = to_f<T>(qfv[(size_t)(ts + tt) * width + (size_t)2 * heads * dk + h * dv + j]);
#pragma unroll
        for (int i = 0; i < R; ++i)
          if (i < dk) {
            const float f = fs[tt * dk + i];
            M[i] = fmaf(f, M[i], (1.f - f) * v);
            o = fmaf(M[i], qs[tt * dk + i], o);
          }
        if (!FUSE) raw[(size_t)(ts + tt) * heads * dv + h * dv + j] = o;
      }
      if (FUSE) os[tt * blockDim.x + threadIdx.x] = o;
    }
    __syncthreads();
    if (FUSE) {
      for (int tt = warp; tt < n; tt += nwarps) {
        float ss = 0.f;
        for (int c = lane; c < dv; c += 32) ss += os[tt * blockDim.x + c] * os[tt * blockDim.x + c];
        const float denom = sqrtf(warp_sum(ss) / (float)dv + eps);
        for (int c = lane; c < dv; c += 32)
          out[(size_t)(ts + tt) * heads * dv + h * dv + c] = from_f<T>(os[tt * blockDim.x + c] / denom * nw[c]);
      }
      __syncthreads();
    }
  }
  if (j < dv) {
#pragma unroll
    for (int i = 0; i < R; ++i)
      if (i < dk) mine[(size_t)i * dv] = M[i];
  }
}

// out[t, h, :] = raw[t, h, :] / sqrt(mean(raw[t, h, :]^2) + eps) * w; one warp per (token, head).
template <typename T>
__global__ void head_gain_norm_kernel(const float* raw, const float* __restrict__ w, T* out, int rows, int dv, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= rows) return;
  const float* x = raw + (size_t)row * dv;
  float ss = 0.f;
  for (int c = lane; c < dv; c += 32) ss += x[c] * x[c];
  const float denom = sqrtf(warp_sum(ss) / (float)dv + eps);
  for (int c = lane; c < dv; c += 32) out[(size_t)row * dv + c] = from_f<T>(x[c] / denom * w[c]);
}

template <typename T, int R>
int launch_hgrn2(const void* qfv, const void* bf, const float* lower, const float* nw, float* state, const int* cu_q,
                 const int* state_slots, void* out, float* raw, int B, int heads, int dk, int dv, float eps, int num_slots,
                 int* err, cudaStream_t stream) {
  const bool fuse = dv <= 128;
  const int threads = fuse ? (dv + 31) / 32 * 32 : 128;
  const int col_blocks = fuse ? 1 : (dv + 127) / 128;
  const size_t smem = ((size_t)2 * HG_TT * dk + (size_t)HG_TT * threads) * sizeof(float);
  dim3 grid(heads * col_blocks, B);
  if (fuse)
    return launch_kernel(hgrn2_scan_kernel<T, R, true>, grid, dim3(threads), smem, stream, (const T*)qfv, (const T*)bf, lower, nw,
                         state, cu_q, state_slots, (T*)out, raw, heads, dk, dv, col_blocks, eps, num_slots, err);
  return launch_kernel(hgrn2_scan_kernel<T, R, false>, grid, dim3(threads), smem, stream, (const T*)qfv, (const T*)bf, lower, nw,
                       state, cu_q, state_slots, (T*)out, raw, heads, dk, dv, col_blocks, eps, num_slots, err);
}

template <typename T>
int dispatch_hgrn2(const void* qfv, const void* bf, const float* lower, const float* nw, float* state, const int* cu_q,
                   const int* state_slots, void* out, float* raw, int Tn, int B, int heads, int dk, int dv, float eps,
                   int num_slots, int* err, cudaStream_t stream) {
  int code;
#define VOB_HG(RR) code = launch_hgrn2<T, RR>(qfv, bf, lower, nw, state, cu_q, state_slots, out, raw, B, heads, dk, dv, eps, num_slots, err, stream)
  if (dk <= 16) VOB_HG(16);
  else if (dk <= 32) VOB_HG(32);
  else if (dk <= 64) VOB_HG(64);
  else if (dk <= 128) VOB_HG(128);
  else VOB_HG(256);
#undef VOB_HG
  if (code != 0 || dv <= 128) return code;
  const int rows = Tn * heads;
  return launch_kernel(head_gain_norm_kernel<T>, dim3((rows + 3) / 4), dim3(128), 0, stream, (const float*)raw, nw, (T*)out, rows, dv,
                       eps);
}

}  // namespace vob

using namespace vob;

// zxg [T, 3W], bz and bx [W] of the model's type; state float [num_slots, W]; cu_q [B+1]; state_slots [B]; out [T, W].
VOB_API int vob_mingru_scan(const void* zxg, const void* bz, const void* bx, float* state, const int* cu_q,
                            const int* state_slots, void* out, int B, int W, int num_slots, int dtype, int* err,
                            cudaStream_t stream) {
  if (B <= 0 || W <= 0) return 0;
  if (B > 65535) return VOB_UNSUPPORTED;
  dim3 grid((W + 63) / 64, B);
  if (dtype == VOB_F32)
    return launch_kernel(mingru_scan_kernel<float>, grid, dim3(64), 0, stream, (const float*)zxg, (const float*)bz, (const float*)bx,
                         state, cu_q, state_slots, (float*)out, W, num_slots, err);
  if (dtype == VOB_BF16)
    return launch_kernel(mingru_scan_kernel<__nv_bfloat16>, grid, dim3(64), 0, stream, (const __nv_bfloat16*)zxg,
                         (const __nv_bfloat16*)bz, (const __nv_bfloat16*)bx, state, cu_q, state_slots, (__nv_bfloat16*)out, W,
                         num_slots, err);
  return VOB_BAD_ARGUMENT;
}

// qfv [T, heads*(2 dk + dv)], bf [heads*dk] of the model's type; lower [heads*dk], nw [dv] float; state float
// [num_slots, heads, dk, dv]; out [T, heads*dv]; raw: float [T, heads*dv], needed when dv > 128.
VOB_API int vob_hgrn2_scan(const void* qfv, const void* bf, const float* lower, const float* nw, float* state, const int* cu_q,
                           const int* state_slots, void* out, float* raw, int T, int B, int heads, int dk, int dv, float eps,
                           int num_slots, int dtype, int* err, cudaStream_t stream) {
  if (B <= 0 || T <= 0) return 0;
  if (heads <= 0 || dk <= 0 || dv <= 0 || dk > 256 || B > 65535 || (dv > 128 && !raw)) return VOB_UNSUPPORTED;
  if (dtype == VOB_F32)
    return dispatch_hgrn2<float>(qfv, bf, lower, nw, state, cu_q, state_slots, out, raw, T, B, heads, dk, dv, eps, num_slots, err,
                                 stream);
  if (dtype == VOB_BF16)
    return dispatch_hgrn2<__nv_bfloat16>(qfv, bf, lower, nw, state, cu_q, state_slots, out, raw, T, B, heads, dk, dv, eps,
                                         num_slots, err, stream);
  return VOB_BAD_ARGUMENT;
}
