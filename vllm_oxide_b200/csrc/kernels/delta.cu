// The gated delta rule: a matrix state per head that forgets by a decay and is corrected toward each new value.
//
// Per head, with S [dim, vdim] float, carried from token to token in the request's state slot:
//     S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q          (the read-out sees the token's own write)
// q and k are unit vectors (x / sqrt(sum x^2 + 1e-6)), q also times dim^(-1/2); beta = sigmoid(b);
// g = exp(-exp(A_log) * softplus(a + dt_bias)).  q, k and v come out of short causal convolutions over time (one filter a
// channel, `taps` taps, the last one the current token's) followed by SiLU; the last taps - 1 inputs of every channel are
// part of the request's state, behind S in the same slot.  Query/key head h / (heads / kv_heads) serves value head h.
//
// Four kernels:
//   short_conv_silu    out[t, c] = SiLU(sum_j w[c, j] x[t - (taps-1) + j, c]), inputs before the portion's start from the slot
//   short_conv_state   the slot's taps - 1 inputs after this portion (run after the first: it overwrites what that one reads)
//   delta_scan         the recurrence.  A column of S lives in the registers of LANES threads (ROWS rows each, rows
//                      interleaved so that a warp's loads of the state fill whole sectors); a block takes the columns
//                      c0.. of one (request, head) and walks the request's tokens in order, CH at a time through shared
//                      memory (unit vectors, decay and beta are made there, in float).
//   delta_out_norm     o / sqrt(mean(o^2) + eps) * w * SiLU(gate), per head over vdim
// Everything but the inputs' type T is float on both paths.  The chain of operations of an output depends only on the
// request's tokens and the state it starts from, not on the cut, the batch or the slot.
#include "common.cuh"

namespace vob {

constexpr int DELTA_MAX_TAPS = 9;

__device__ __forceinline__ float silu_f(float x) { return x / (1.f + expf(-x)); }

template <typename T>
__global__ void __launch_bounds__(128)
short_conv_silu_kernel(const T* x, long x_stride, const float* __restrict__ w, const float* state, long state_stride,
                       long conv_off, const int* __restrict__ token_req, const int* __restrict__ cu_q,
                       const int* __restrict__ state_slots, float* out, int C, int taps, long num_slots, int* err) {
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const int c = blockIdx.y * 128 + threadIdx.x;
  const int req = token_req[t];
  if (req < 0) return;
  const int j = t - cu_q[req];
  const int slot = state_slots[req];
  pdl_wait();
  if (slot < 0 || slot >= num_slots) {
    if (threadIdx.x == 0) atomicOr(err, VOB_ERR_SLOT);
    return;
  }
  if (c >= C) return;
  const float* st = state + (size_t)slot * state_stride + conv_off;
  float acc = 0.f;
  for (int k = taps - 1; k >= 0; --k) {      // oldest input first
    const int rel = j - k;
    const float xv = rel >= 0 ? to_f<T>(x[(size_t)(t - k) * x_stride + c]) : st[(size_t)(taps - 1 + rel) * C + c];
    acc = fmaf(w[(size_t)c * taps + (taps - 1 - k)], xv, acc);
  }
  out[(size_t)t * C + c] = silu_f(acc);
}

template <typename T>
__global__ void __launch_bounds__(128)
short_conv_state_kernel(const T* x, long x_stride, float* state, long state_stride, long conv_off,
                        const int* __restrict__ cu_q, const int* __restrict__ state_slots, int C, int taps, long num_slots) {
  pdl_launch_dependents();
  const int b = blockIdx.y;
  const int c = blockIdx.x * 128 + threadIdx.x;
  const int t0 = cu_q[b], n = cu_q[b + 1] - t0;
  const int slot = state_slots[b];
  pdl_wait();
  if (n <= 0 || slot < 0 || slot >= num_slots || c >= C) return;
  float* st = state + (size_t)slot * state_stride + conv_off;
  float nv[DELTA_MAX_TAPS - 1];
#pragma unroll
  for (int s = 0; s < DELTA_MAX_TAPS - 1; ++s) {
    if (s < taps - 1) {
      const int rel = n - (taps - 1) + s;     // place within the portion of the input that entry s holds afterwards
      nv[s] = rel >= 0 ? to_f<T>(x[(size_t)(t0 + rel) * x_stride + c]) : st[(size_t)(s + n) * C + c];
    }
  }
#pragma unroll
  for (int s = 0; s < DELTA_MAX_TAPS - 1; ++s)
    if (s < taps - 1) st[(size_t)s * C + c] = nv[s];
}

// ---------------------------------------------------------------- the recurrence
constexpr int DS_CH = 16;      // tokens a round through shared memory
constexpr int DS_ROWS = 32;    // rows of a column a thread keeps

// qkv: float [tokens, 2 * kvh * dim + heads * vdim] (q heads, k heads, v heads: the convolutions' output);
// ab: rows of ab_stride elements of T, beta's pre-activation of head h at b_off + h, the decay's at a_off + h.
template <typename T, int LANES>
__global__ void __launch_bounds__(128)
delta_scan_kernel(const float* qkv, const T* ab, long ab_stride, int b_off, int a_off, const float* __restrict__ A_log,
                  const float* __restrict__ dt_bias, float* state, long state_stride, const int* __restrict__ cu_q,
                  const int* __restrict__ state_slots, float* raw, int heads, int kvh, int dim, int vdim, long num_slots,
                  int* err) {
  constexpr int COLS = 128 / LANES;
  constexpr int KW = LANES * DS_ROWS;          // padded length of a key in shared memory
  __shared__ __align__(16) float ks[DS_CH][KW], qs[DS_CH][KW];
  __shared__ float vs[DS_CH][COLS], os[DS_CH][COLS];
  __shared__ float gs[DS_CH], bs[DS_CH];
  pdl_launch_dependents();
  const int b = blockIdx.z, h = blockIdx.y, c0 = blockIdx.x * COLS;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int col = c0 + tid / LANES, seg = tid % LANES;
  const bool live = col < vdim;
  const int t0 = cu_q[b], t1 = cu_q[b + 1];
  const int slot = state_slots[b];
  const float neg_rate = -expf(A_log[h]), bias = dt_bias[h];
  pdl_wait();
  if (t1 <= t0) return;
  if (slot < 0 || slot >= num_slots) {
    if (tid == 0) atomicOr(err, VOB_ERR_SLOT);
    return;
  }
  const int kh = h / (heads / kvh);
  const int C = 2 * kvh * dim + heads * vdim;
  const float qscale = 1.f / sqrtf((float)dim);
  // this thread's rows of its column: seg, seg + LANES, ... (row r of the thread is row seg + LANES * r of the head)
  float S[DS_ROWS];
  float* mine = state + (size_t)slot * state_stride + (size_t)h * dim * vdim + col;
#pragma unroll
  for (int r = 0; r < DS_ROWS; ++r) {
    const int row = seg + LANES * r;
    S[r] = (live && row < dim) ? mine[(size_t)row * vdim] : 0.f;
  }
  for (int base = t0; base < t1; base += DS_CH) {
    const int n = min(DS_CH, t1 - base);
    __syncthreads();
    // unit vectors: a warp takes tokens warp, warp + 4, ...; element d goes to [d % LANES][d / LANES], where its thread looks
    for (int i = warp; i < n; i += 4) {
      const float* qrow = qkv + (size_t)(base + i) * C + (size_t)kh * dim;
      const float* krow = qrow + (size_t)kvh * dim;
      float sq = 0.f, sk = 0.f;
      for (int d = lane; d < dim; d += 32) {
        const float a = qrow[d], c = krow[d];
        sq = fmaf(a, a, sq);
        sk = fmaf(c, c, sk);
      }
      sq = warp_sum(sq);
      sk = warp_sum(sk);
      const float iq = qscale / sqrtf(sq + 1e-6f), ik = 1.f / sqrtf(sk + 1e-6f);
      for (int d = lane; d < KW; d += 32) {
        const int row = (d / DS_ROWS) + LANES * (d % DS_ROWS);     // shared index d = seg * ROWS + r holds head row seg + LANES r
        qs[i][d] = row < dim ? qrow[row] * iq : 0.f;
        ks[i][d] = row < dim ? krow[row] * ik : 0.f;
      }
      if (lane == 0) {
        const T* abrow = ab + (size_t)(base + i) * ab_stride;
        const float bv = to_f<T>(abrow[b_off + h]), av = to_f<T>(abrow[a_off + h]) + bias;
        const float sp = av > 20.f ? av : log1pf(expf(av));
        bs[i] = 1.f / (1.f + expf(-bv));
        gs[i] = expf(neg_rate * sp);
      }
    }
    for (int i = tid; i < n * COLS; i += 128) {
      const int tk = i / COLS, cc = i % COLS;
      vs[tk][cc] = c0 + cc < vdim ? qkv[(size_t)(base + tk) * C + (size_t)2 * kvh * dim + (size_t)h * vdim + c0 + cc] : 0.f;
    }
    __syncthreads();
    for (int i = 0; i < n; ++i) {
      const float g = gs[i], beta = bs[i];
      const float4* k4 = reinterpret_cast<const float4*>(&ks[i][seg * DS_ROWS]);
      const float4* q4 = reinterpret_cast<const float4*>(&qs[i][seg * DS_ROWS]);
      float a = 0.f;
#pragma unroll
      for (int r = 0; r < DS_ROWS / 4; ++r) {
        const float4 kv = k4[r];
        S[4 * r] *= g; S[4 * r + 1] *= g; S[4 * r + 2] *= g; S[4 * r + 3] *= g;
        a = fmaf(S[4 * r], kv.x, a); a = fmaf(S[4 * r + 1], kv.y, a);
        a = fmaf(S[4 * r + 2], kv.z, a); a = fmaf(S[4 * r + 3], kv.w, a);
      }
#pragma unroll
      for (int o = 1; o < LANES; o <<= 1) a += __shfl_xor_sync(0xffffffffu, a, o);
      const float u = beta * (vs[i][tid / LANES] - a);
      float o_ = 0.f;
#pragma unroll
      for (int r = 0; r < DS_ROWS / 4; ++r) {
        const float4 kv = k4[r], qv = q4[r];
        S[4 * r] = fmaf(kv.x, u, S[4 * r]); S[4 * r + 1] = fmaf(kv.y, u, S[4 * r + 1]);
        S[4 * r + 2] = fmaf(kv.z, u, S[4 * r + 2]); S[4 * r + 3] = fmaf(kv.w, u, S[4 * r + 3]);
        o_ = fmaf(S[4 * r], qv.x, o_); o_ = fmaf(S[4 * r + 1], qv.y, o_);
        o_ = fmaf(S[4 * r + 2], qv.z, o_); o_ = fmaf(S[4 * r + 3], qv.w, o_);
      }
#pragma unroll
      for (int o = 1; o < LANES; o <<= 1) o_ += __shfl_xor_sync(0xffffffffu, o_, o);
      if (seg == 0) os[i][tid / LANES] = o_;
    }
    __syncthreads();
    for (int i = tid; i < n * COLS; i += 128) {
      const int tk = i / COLS, cc = i % COLS;
      if (c0 + cc < vdim) raw[(size_t)(base + tk) * heads * vdim + (size_t)h * vdim + c0 + cc] = os[tk][cc];
    }
  }
#pragma unroll
  for (int r = 0; r < DS_ROWS; ++r) {
    const int row = seg + LANES * r;
    if (live && row < dim) mine[(size_t)row * vdim] = S[r];
  }
}

// out[t, h, :] = raw[t, h, :] / sqrt(mean(raw[t, h, :]^2) + eps) * w * SiLU(gate[t, h, :]); one warp a (token, head).
template <typename T>
__global__ void __launch_bounds__(128)
delta_out_norm_kernel(const float* raw, const T* gate, long gate_stride, const float* __restrict__ w, T* out, int heads,
                      int vdim, float eps, int total) {
  pdl_launch_dependents();
  pdl_wait();
  const int idx = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (idx >= total) return;
  const int t = idx / heads, h = idx % heads;
  const float* o = raw + ((size_t)t * heads + h) * vdim;
  float ss = 0.f;
  for (int d = lane; d < vdim; d += 32) ss = fmaf(o[d], o[d], ss);
  ss = warp_sum(ss);
  const float inv = 1.f / sqrtf(ss / (float)vdim + eps);
  const T* grow = gate + (size_t)t * gate_stride + (size_t)h * vdim;
  T* orow = out + ((size_t)t * heads + h) * vdim;
  for (int d = lane; d < vdim; d += 32) orow[d] = from_f<T>(o[d] * inv * w[d] * silu_f(to_f<T>(grow[d])));
}

}  // namespace vob

using namespace vob;

// x: rows of x_stride elements of `dtype`, the C channels first; w float [C, taps]; state float [num_slots, state_stride]
// with the convolutions' part ((taps - 1) x C) at conv_off; out float [T, C].
VOB_API int vob_short_conv_silu(const void* x, long x_stride, const float* w, const float* state, long state_stride,
                                long conv_off, const int* token_req, const int* cu_q, const int* state_slots, float* out,
                                int T, int C, int taps, long num_slots, int dtype, int* err, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (C <= 0 || taps < 1 || taps > DELTA_MAX_TAPS) return VOB_UNSUPPORTED;
  dim3 grid(T, (C + 127) / 128);
  if (grid.y > 65535) return VOB_UNSUPPORTED;
  if (dtype == VOB_F32)
    return launch_kernel(short_conv_silu_kernel<float>, grid, 128, 0, stream, (const float*)x, x_stride, w, state, state_stride,
                         conv_off, token_req, cu_q, state_slots, out, C, taps, num_slots, err);
  if (dtype == VOB_BF16)
    return launch_kernel(short_conv_silu_kernel<__nv_bfloat16>, grid, 128, 0, stream, (const __nv_bfloat16*)x, x_stride, w,
                         state, state_stride, conv_off, token_req, cu_q, state_slots, out, C, taps, num_slots, err);
  return VOB_BAD_ARGUMENT;
}

VOB_API int vob_short_conv_state(const void* x, long x_stride, float* state, long state_stride, long conv_off,
                                 const int* cu_q, const int* state_slots, int B, int C, int taps, long num_slots, int dtype,
                                 cudaStream_t stream) {
  if (B <= 0 || taps <= 1) return 0;
  if (C <= 0 || taps > DELTA_MAX_TAPS) return VOB_UNSUPPORTED;
  dim3 grid((C + 127) / 128, B);
  if (dtype == VOB_F32)
    return launch_kernel(short_conv_state_kernel<float>, grid, 128, 0, stream, (const float*)x, x_stride, state, state_stride,
                         conv_off, cu_q, state_slots, C, taps, num_slots);
  if (dtype == VOB_BF16)
    return launch_kernel(short_conv_state_kernel<__nv_bfloat16>, grid, 128, 0, stream, (const __nv_bfloat16*)x, x_stride,
                         state, state_stride, conv_off, cu_q, state_slots, C, taps, num_slots);
  return VOB_BAD_ARGUMENT;
}

template <typename T>
static int launch_delta_scan(const float* qkv, const void* ab, long ab_stride, int b_off, int a_off, const float* A_log,
                             const float* dt_bias, float* state, long state_stride, const int* cu_q, const int* state_slots,
                             float* raw, int B, int heads, int kvh, int dim, int vdim, long num_slots, int* err,
                             cudaStream_t stream) {
  const int lanes = dim <= 32 ? 1 : (dim <= 64 ? 2 : (dim <= 128 ? 4 : 8));
#define VOB_DS(L)                                                                                                          \
  if (lanes == L) {                                                                                                        \
    dim3 grid((vdim + 128 / L - 1) / (128 / L), heads, B);                                                                 \
    return launch_kernel(delta_scan_kernel<T, L>, grid, 128, 0, stream, qkv, (const T*)ab, ab_stride, b_off, a_off, A_log,  \
                         dt_bias, state, state_stride, cu_q, state_slots, raw, heads, kvh, dim, vdim, num_slots, err);     \
  }
  VOB_DS(1) VOB_DS(2) VOB_DS(4) VOB_DS(8)
#undef VOB_DS
  return VOB_UNSUPPORTED;
}

VOB_API int vob_delta_scan(const float* qkv, const void* ab, long ab_stride, int b_off, int a_off, const float* A_log,
                           const float* dt_bias, float* state, long state_stride, const int* cu_q, const int* state_slots,
                           float* raw, int B, int heads, int kvh, int dim, int vdim, long num_slots, int dtype, int* err,
                           cudaStream_t stream) {
  if (B <= 0) return 0;
  if (heads <= 0 || kvh <= 0 || heads % kvh || dim <= 0 || dim > 256 || vdim <= 0 || B > 65535) return VOB_UNSUPPORTED;
  if (dtype == VOB_F32)
    return launch_delta_scan<float>(qkv, ab, ab_stride, b_off, a_off, A_log, dt_bias, state, state_stride, cu_q, state_slots, raw,
                                    B, heads, kvh, dim, vdim, num_slots, err, stream);
  if (dtype == VOB_BF16)
    return launch_delta_scan<__nv_bfloat16>(qkv, ab, ab_stride, b_off, a_off, A_log, dt_bias, state, state_stride, cu_q,
                                            state_slots, raw, B, heads, kvh, dim, vdim, num_slots, err, stream);
  return VOB_BAD_ARGUMENT;
}

VOB_API int vob_delta_out_norm(const float* raw, const void* gate, long gate_stride, const float* w, void* out, int T, int heads,
                               int vdim, float eps, int dtype, cudaStream_t stream) {
  if (T <= 0) return 0;
  const int total = T * heads;
  dim3 grid((total + 3) / 4);
  if (dtype == VOB_F32)
    return launch_kernel(delta_out_norm_kernel<float>, grid, 128, 0, stream, raw, (const float*)gate, gate_stride, w,
                         (float*)out, heads, vdim, eps, total);
  if (dtype == VOB_BF16)
    return launch_kernel(delta_out_norm_kernel<__nv_bfloat16>, grid, 128, 0, stream, raw, (const __nv_bfloat16*)gate,
                         gate_stride, w, (__nv_bfloat16*)out, heads, vdim, eps, total);
  return VOB_BAD_ARGUMENT;
}
