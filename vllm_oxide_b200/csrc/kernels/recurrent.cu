// Recurrent token mixers: the state of a request is carried in float from token to token, in a state slot.
//
// Both kernels walk the tokens of one request in order, whatever the step holds of it (a whole prompt, a portion, one
// decoded token), starting from the slot's state and leaving the new state there.  The chain of float operations of a
// channel therefore depends on the request's tokens only: not on how they were cut into steps nor on the batch.
// Projections come in the model's type T (bfloat16 when serving); gates, decays, the state and the norm are float.
#include "common.cuh"

namespace vob {

__device__ __forceinline__ float sigmoid_f(float x) { return 1.f / (1.f + expf(-x)); }
// f = l + (1 - l) sigmoid(pre + bias): one spelling for every kernel that needs the gate
__device__ __forceinline__ float forget_gate(float l, float pre, float bias) { return fmaf(1.f - l, sigmoid_f(pre + bias), l); }

// ---------------------------------------------------------------- minGRU
// zxg [tokens, 3W]: pre-activations of the gate z, of the candidate u and of the output gate g (no bias yet).
//   z = sigmoid(z + bz);  c = u + bx;  c = c >= 0 ? c + 1/2 : sigmoid(c);  s = (1 - z) s + z c;  out = s * silu(g)
// A block owns 32 channels of one request; neighbouring threads read neighbouring channels.  With NCH > 1 the request's
// tokens of this step are cut into NCH ranges, one per thread row: every row first folds its range into (A, B) with
// s_end = A s_start + B, the rows' starts follow from the state and the (A, B) before them, and a second walk writes
// the outputs.  A recurrence is a chain: without the cut a prompt of thousands of tokens runs on a thread per channel.
// The cut changes where a channel's additions are rounded, never what is computed.
struct GruStep { float z, c, g; };

template <typename T>
__device__ __forceinline__ GruStep gru_step(const T* row, int c, int W, float biasz, float biasx) {
  GruStep r;
  r.z = sigmoid_f(to_f<T>(row[c]) + biasz);
  const float u = to_f<T>(row[W + c]) + biasx;
  r.c = u >= 0.f ? u + 0.5f : sigmoid_f(u);
  r.g = to_f<T>(row[2 * W + c]);
  return r;
}

template <typename T, int NCH>
__global__ void __launch_bounds__(32 * NCH)
mingru_scan_kernel(const T* zxg, const T* __restrict__ bz, const T* __restrict__ bx, float* state,
                   const int* __restrict__ cu_q, const int* __restrict__ state_slots, T* out, int W,
                   int num_slots, int* err) {
  __shared__ float As[NCH][32], Bs[NCH][32];
  pdl_launch_dependents();
  const int b = blockIdx.y, lane = threadIdx.x, ch = threadIdx.y;
  const int c = min(blockIdx.x * 32 + lane, W - 1);
  const bool live = blockIdx.x * 32 + lane < W;
  const int t0 = cu_q[b], t1 = cu_q[b + 1];
  const int slot = state_slots[b];
  const float biasz = to_f<T>(bz[c]), biasx = to_f<T>(bx[c]);
  pdl_wait();
  if (t1 <= t0) return;
  if (slot < 0 || slot >= num_slots) {
    if (threadIdx.x == 0 && ch == 0) atomicOr(err, VOB_ERR_SLOT);
    return;
  }
  const int per = (t1 - t0 + NCH - 1) / NCH;
  const int lo = min(t1, t0 + ch * per), hi = min(t1, lo + per);
  float s = state[(size_t)slot * W + c];
  if (NCH > 1) {
    float A = 1.f, B = 0.f;
#pragma unroll 4
    for (int t = lo; t < hi; ++t) {
      const GruStep g = gru_step<T>(zxg + (size_t)t * 3 * W, c, W, biasz, biasx);
      A *= 1.f - g.z;
      B = fmaf(g.z, g.c, (1.f - g.z) * B);
    }
    As[ch][lane] = A;
    Bs[ch][lane] = B;
    __syncthreads();
    for (int k = 0; k < ch; ++k) s = fmaf(As[k][lane], s, Bs[k][lane]);
  }
  // four tokens at a time: their loads are issued before the first store (the compiler cannot know that `out` is
  // another buffer, and would otherwise wait for every store before the next token's loads)
  int t = lo;
  for (; t + 4 <= hi; t += 4) {
    GruStep g[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) g[k] = gru_step<T>(zxg + (size_t)(t + k) * 3 * W, c, W, biasz, biasx);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      s = fmaf(g[k].z, g[k].c, (1.f - g[k].z) * s);
      if (live) out[(size_t)(t + k) * W + c] = from_f<T>(s * (g[k].g * sigmoid_f(g[k].g)));
    }
  }
  for (; t < hi; ++t) {
    const GruStep g = gru_step<T>(zxg + (size_t)t * 3 * W, c, W, biasz, biasx);
    s = fmaf(g.z, g.c, (1.f - g.z) * s);
    if (live) out[(size_t)t * W + c] = from_f<T>(s * (g.g * sigmoid_f(g.g)));
  }
  if (ch == NCH - 1 && live) state[(size_t)slot * W + c] = s;
}

// ---------------------------------------------------------------- HGRN2
// qfv [tokens, heads*dk | heads*dk | heads*dv]: pre-activations of q and of the forget gate, and the values.
//   q = silu(q);  f = l + (1 - l) sigmoid(f + bf);  M = diag(f) M + (1 - f) v^T;  o = M^T q;  out = o / rms(o) * w
// Column j of a head's state M (dk floats) is shared by PARTS neighbouring lanes, R rows each, in registers: a token costs
// a thread R multiply-adds twice, and the lanes of a column add their parts of o by shuffles.  The gates of HG_TT tokens are
// made by the whole block at once and parked in shared memory (rows padded so that the PARTS lanes of a column read
// different banks).  FUSE: the block holds all dv columns of the head and also takes the norm over them (decoding: one
// launch); otherwise a block holds as many columns as 128 threads cover, so that a long portion of one request spreads
// over more blocks, o leaves in float and head_gain_norm_kernel follows.  Both give the same numbers: an element's
// chain of operations depends on (R, PARTS) alone, and those follow from dk.
//
// A long portion is also cut along the tokens (`chunks` > 1, four launches): MODE 1 walks every range from a zero state
// and leaves its end state L; hgrn2_range_gates_kernel takes the product F of every range's gates; hgrn2_join_kernel goes
// through the ranges in order,
// M_start(c+1) = diag(F_c) M_start(c) + L_c, leaves every range's start where its L was and the last state in the
// slot; MODE 2 walks the ranges again from their starts and writes the outputs.  Twice the arithmetic, on as many more
// blocks as there are ranges.  MODE 0 is the walk from the slot's state to the slot's state in one launch.
constexpr int HG_TT = 16;

// index of gate i in a row of shared memory: four floats of padding after every 32, so that the lanes that share a column
// (32 or 64 rows apart) read different banks with 16-byte loads
__device__ __forceinline__ int hg_pad(int i) { return i + 4 * (i >> 5); }

// FULL: dk = R * PARTS, every row a thread holds exists (no test per element: the tests were two of seven instructions).
template <typename T, int R, int PARTS, bool FUSE, int MODE, bool FULL>
__global__ void __launch_bounds__(FUSE ? (R > 32 ? 256 : 512) : 128)
hgrn2_scan_kernel(const T* qfv, const T* __restrict__ bf, const float* __restrict__ lower, const float* __restrict__ nw,
                  float* state, const int* __restrict__ cu_q, const int* __restrict__ state_slots, T* out, float* raw,
                  float* ends, float* gates, int heads, int dk, int dv, int col_blocks, float eps, int num_slots, int* err) {
  extern __shared__ float4 sm4[];
  float* sm = reinterpret_cast<float*>(sm4);
  const int gate_row = hg_pad(R * PARTS);
  const int cols = blockDim.x / PARTS;
  float* qs = sm;                        // [HG_TT][gate_row]
  float* fs = qs + HG_TT * gate_row;     // [HG_TT][gate_row]  f
  float* gs = fs + HG_TT * gate_row;     // [HG_TT][gate_row]  1 - f
  float* vs = gs + HG_TT * gate_row;     // [HG_TT][cols]
  float* os = vs + HG_TT * cols;         // [HG_TT][cols]  (FUSE)
  pdl_launch_dependents();
  const int part = threadIdx.x % PARTS, jj = threadIdx.x / PARTS;
  const int h = blockIdx.x / col_blocks, cb = blockIdx.x % col_blocks, j = cb * cols + jj;
  const int b = blockIdx.y, chunk = blockIdx.z, chunks = gridDim.z;
  const int q0 = cu_q[b], q1 = cu_q[b + 1];
  const int slot = state_slots[b];
  pdl_wait();
  if (q1 <= q0) return;
  if (slot < 0 || slot >= num_slots) {
    if (threadIdx.x == 0) atomicOr(err, VOB_ERR_SLOT);
    return;
  }
  const int per = (q1 - q0 + chunks - 1) / chunks;
  const int t0 = min(q1, q0 + chunk * per), t1 = min(q1, t0 + per);
  const size_t width = (size_t)heads * (2 * dk + dv);
  const int i0 = part * R;
  float* mine = MODE == 0 ? state + (((size_t)slot * heads + h) * dk + i0) * dv + j
                          : ends + ((((size_t)b * chunks + chunk) * heads + h) * dk + i0) * dv + j;
  float M[R];
#pragma unroll
  for (int i = 0; i < R; ++i) M[i] = (MODE != 1 && i0 + i < dk && j < dv) ? mine[(size_t)i * dv] : 0.f;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  // the gates of a tile: thread rows over tokens, thread columns over gates (one division, here)
  const int gate_lanes = min(dk, (int)blockDim.x), gate_step = blockDim.x / gate_lanes;
  const int gate_i = threadIdx.x % gate_lanes, gate_t = threadIdx.x / gate_lanes < gate_step ? threadIdx.x / gate_lanes : HG_TT;
  for (int ts = t0; ts < t1; ts += HG_TT) {
    const int n = min(HG_TT, t1 - ts);
    for (int i = gate_i; i < dk; i += gate_lanes) {
      const float l = lower[h * dk + i], bias = to_f<T>(bf[h * dk + i]);
      // eight tokens' loads are issued before the first of them is used
      for (int tb = gate_t; tb < n; tb += 8 * gate_step) {
        float qa[8], fa[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const int tt = min(tb + k * gate_step, n - 1);
          const T* row = qfv + (size_t)(ts + tt) * width;
          qa[k] = to_f<T>(row[h * dk + i]);
          fa[k] = to_f<T>(row[(heads + h) * dk + i]);
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const int tt = tb + k * gate_step;
          if (tt < n) {
            const float f = forget_gate(l, fa[k], bias);
            if (MODE != 1) qs[tt * gate_row + hg_pad(i)] = qa[k] * sigmoid_f(qa[k]);
            fs[tt * gate_row + hg_pad(i)] = f;
            gs[tt * gate_row + hg_pad(i)] = 1.f - f;
          }
        }
      }
    }
    for (int idx = threadIdx.x; idx < n * cols; idx += blockDim.x) {
      const int tt = idx / cols, c = idx % cols;
      vs[idx] = cb * cols + c < dv ? to_f<T>(qfv[(size_t)(ts + tt) * width + (size_t)2 * heads * dk + h * dv + cb * cols + c]) : 0.f;
    }
    __syncthreads();
#pragma unroll 2
    for (int tt = 0; tt < n; ++tt) {
      float o = 0.f;
      const float v = vs[tt * cols + jj];
      const float* fr = fs + tt * gate_row + hg_pad(i0);
      const float* gr = gs + tt * gate_row + hg_pad(i0);
      const float* qr = qs + tt * gate_row + hg_pad(i0);
#pragma unroll
      for (int i = 0; i < R; i += 4) {
        const float4 f4 = *reinterpret_cast<const float4*>(fr + hg_pad(i));      // hg_pad(i0 + i) = hg_pad(i0) + hg_pad(i)
        const float4 g4 = *reinterpret_cast<const float4*>(gr + hg_pad(i));
        const float4 q4 = MODE == 1 ? f4 : *reinterpret_cast<const float4*>(qr + hg_pad(i));
        const float fv[4] = {f4.x, f4.y, f4.z, f4.w}, gv[4] = {g4.x, g4.y, g4.z, g4.w}, qv[4] = {q4.x, q4.y, q4.z, q4.w};
#pragma unroll
        for (int k = 0; k < 4; ++k)
          if (FULL || i0 + i + k < dk) {
            M[i + k] = fmaf(fv[k], M[i + k], gv[k] * v);
            if (MODE != 1) o = fmaf(M[i + k], qv[k], o);
          }
      }
      if (MODE != 1) {
#pragma unroll
        for (int d = 1; d < PARTS; d <<= 1) o += __shfl_xor_sync(0xffffffffu, o, d);
        if (FUSE) {
          if (part == 0) os[tt * cols + jj] = o;
        } else if (part == 0 && j < dv) {
          raw[(size_t)(ts + tt) * heads * dv + h * dv + j] = o;
        }
      }
    }
    __syncthreads();
    if (FUSE && MODE != 1) {
      for (int tt = warp; tt < n; tt += nwarps) {
        float ss = 0.f;
        for (int c = lane; c < dv; c += 32) ss += os[tt * cols + c] * os[tt * cols + c];
        const float denom = sqrtf(warp_sum(ss) / (float)dv + eps);
        for (int c = lane; c < dv; c += 32)
          out[(size_t)(ts + tt) * heads * dv + h * dv + c] = from_f<T>(os[tt * cols + c] / denom * nw[c]);
      }
      __syncthreads();
    }
  }
  if (MODE == 2) return;
  if (j < dv) {
#pragma unroll
    for (int i = 0; i < R; ++i)
      if (i0 + i < dk) mine[(size_t)i * dv] = M[i];
  }
}

// gates[b][c][h][i] = the product of the forget gates of range c of request b: what an end state of that range owes to its start.
// A block takes 32 gates of one range; its eight warps take every eighth token, and their partial products are multiplied
// in the order of the warps.
template <typename T>
__global__ void __launch_bounds__(256)
hgrn2_range_gates_kernel(const T* qfv, const T* __restrict__ bf, const float* __restrict__ lower, float* gates,
                         const int* __restrict__ cu_q, int heads, int dk, int dv) {
  __shared__ float part[8][32];
  pdl_launch_dependents();
  pdl_wait();
  const int b = blockIdx.y, chunk = blockIdx.z, chunks = gridDim.z;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int e = min(blockIdx.x * 32 + lane, heads * dk - 1);      // (head, i)
  const int q0 = cu_q[b], q1 = cu_q[b + 1];
  if (q1 <= q0) return;
  const int per = (q1 - q0 + chunks - 1) / chunks;
  const int t0 = min(q1, q0 + chunk * per), t1 = min(q1, t0 + per);
  const size_t width = (size_t)heads * (2 * dk + dv);
  const float l = lower[e], bias = to_f<T>(bf[e]);
  float F = 1.f;
#pragma unroll 4
  for (int t = t0 + warp; t < t1; t += 8) F *= forget_gate(l, to_f<T>(qfv[(size_t)t * width + (size_t)heads * dk + e]), bias);
  part[warp][lane] = F;
  __syncthreads();
  if (warp == 0 && blockIdx.x * 32 + lane < heads * dk) {
    F = part[0][lane];
#pragma unroll
    for (int k = 1; k < 8; ++k) F *= part[k][lane];
    gates[((size_t)b * chunks + chunk) * heads * dk + e] = F;
  }
}

// One thread per element of a request's state: through the ranges in order, start(c) takes the place of L_c.  All of a
// thread's loads are issued before its first store (at most HG_MAX_CHUNKS ranges), or every store would wait for a load.
constexpr int HG_MAX_CHUNKS = 16;

__global__ void hgrn2_join_kernel(float* state, float* ends, const float* __restrict__ gates, const int* __restrict__ cu_q,
                                  const int* __restrict__ state_slots, int chunks, int heads, int dk, int dv, int num_slots) {
  pdl_launch_dependents();
  pdl_wait();
  const int b = blockIdx.y;
  const long e = (long)blockIdx.x * blockDim.x + threadIdx.x, per = (long)heads * dk * dv;
  const int slot = state_slots[b];
  if (e >= per || cu_q[b + 1] <= cu_q[b] || slot < 0 || slot >= num_slots) return;
  const long row = e / dv;      // (head, i)
  float L[HG_MAX_CHUNKS], F[HG_MAX_CHUNKS];
#pragma unroll
  for (int c = 0; c < HG_MAX_CHUNKS; ++c)
    if (c < chunks) {
      L[c] = ends[((size_t)b * chunks + c) * per + e];
      F[c] = gates[((size_t)b * chunks + c) * heads * dk + row];
    }
  float M = state[(size_t)slot * per + e];
#pragma unroll
  for (int c = 0; c < HG_MAX_CHUNKS; ++c)
    if (c < chunks) {
      ends[((size_t)b * chunks + c) * per + e] = M;
      M = fmaf(F[c], M, L[c]);
    }
  state[(size_t)slot * per + e] = M;
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

template <typename T, int R, int PARTS, int MODE>
int launch_hgrn2(const void* qfv, const void* bf, const float* lower, const float* nw, float* state, const int* cu_q,
                 const int* state_slots, void* out, float* raw, float* ends, float* gates, int B, int chunks, int heads, int dk,
                 int dv, float eps, int num_slots, int fuse, int* err, cudaStream_t stream) {
  const int gate_row = R * PARTS + 4 * ((R * PARTS) / 32);
  const int threads = fuse ? (dv * PARTS + 31) / 32 * 32 : 128;
  const int cols = threads / PARTS;
  const int col_blocks = fuse ? 1 : (dv + cols - 1) / cols;
  const size_t smem = ((size_t)3 * HG_TT * gate_row + (fuse ? 2 : 1) * (size_t)HG_TT * cols) * sizeof(float);
  dim3 grid(heads * col_blocks, B, chunks);
  auto launch = [&](auto kernel) -> int {
    if (smem > 48 * 1024) {      // a head of 256 gates: three rows of gates for 16 tokens pass the default limit
      cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return (int)e;
    }
    return launch_kernel(kernel, grid, dim3(threads), smem, stream, (const T*)qfv, (const T*)bf, lower, nw, state, cu_q, state_slots,
                         (T*)out, raw, ends, gates, heads, dk, dv, col_blocks, eps, num_slots, err);
  };
  if (fuse) return launch(hgrn2_scan_kernel<T, R, PARTS, true, 0, false>);
  if (dk == R * PARTS) return launch(hgrn2_scan_kernel<T, R, PARTS, false, MODE, true>);
  return launch(hgrn2_scan_kernel<T, R, PARTS, false, MODE, false>);
}

// rows of the state a thread keeps, and lanes that share a column: from dk alone
inline int hgrn2_parts(int dk) { return dk <= 32 ? 1 : dk <= 64 ? 2 : 4; }

template <typename T, int MODE>
int dispatch_hgrn2_mode(const void* qfv, const void* bf, const float* lower, const float* nw, float* state, const int* cu_q,
                        const int* state_slots, void* out, float* raw, float* ends, float* gates, int B, int chunks, int heads,
                        int dk, int dv, float eps, int num_slots, int fuse, int* err, cudaStream_t stream) {
#define VOB_HG(RR, PP) return launch_hgrn2<T, RR, PP, MODE>(qfv, bf, lower, nw, state, cu_q, state_slots, out, raw, ends, gates, B, chunks, heads, dk, dv, eps, num_slots, fuse, err, stream)
  if (dk <= 16) VOB_HG(16, 1);
  if (dk <= 32) VOB_HG(32, 1);
  if (dk <= 64) VOB_HG(32, 2);
  if (dk <= 128) VOB_HG(32, 4);
  VOB_HG(64, 4);
#undef VOB_HG
}

template <typename T>
int dispatch_hgrn2(const void* qfv, const void* bf, const float* lower, const float* nw, float* state, const int* cu_q,
                   const int* state_slots, void* out, float* raw, float* scratch, int Tn, int B, int chunks, int heads, int dk,
                   int dv, float eps, int num_slots, int fuse, int* err, cudaStream_t stream) {
  int code;
  if (chunks <= 1) {
    code = dispatch_hgrn2_mode<T, 0>(qfv, bf, lower, nw, state, cu_q, state_slots, out, raw, nullptr, nullptr, B, 1, heads, dk, dv,
                                     eps, num_slots, fuse, err, stream);
  } else {
    float* ends = scratch;
    float* gates = scratch + (size_t)B * chunks * heads * dk * dv;
    code = dispatch_hgrn2_mode<T, 1>(qfv, bf, lower, nw, state, cu_q, state_slots, out, raw, ends, gates, B, chunks, heads, dk, dv,
                                     eps, num_slots, 0, err, stream);
    if (code != 0) return code;
    code = launch_kernel(hgrn2_range_gates_kernel<T>, dim3((heads * dk + 31) / 32, B, chunks), dim3(256), 0, stream, (const T*)qfv,
                         (const T*)bf, lower, gates, cu_q, heads, dk, dv);
    if (code != 0) return code;
    const long per = (long)heads * dk * dv;
    code = launch_kernel(hgrn2_join_kernel, dim3((unsigned)((per + 255) / 256), B), dim3(256), 0, stream, state, ends,
                         (const float*)gates, cu_q, state_slots, chunks, heads, dk, dv, num_slots);
    if (code != 0) return code;
    code = dispatch_hgrn2_mode<T, 2>(qfv, bf, lower, nw, state, cu_q, state_slots, out, raw, ends, gates, B, chunks, heads, dk, dv,
                                     eps, num_slots, 0, err, stream);
  }
  if (code != 0 || fuse) return code;
  const int rows = Tn * heads;
  return launch_kernel(head_gain_norm_kernel<T>, dim3((rows + 3) / 4), dim3(128), 0, stream, (const float*)raw, nw, (T*)out, rows, dv,
                       eps);
}

}  // namespace vob

using namespace vob;

// zxg [T, 3W], bz and bx [W] of the model's type; state float [num_slots, W]; cu_q [B+1]; state_slots [B]; out [T, W].
// `chunks`: 1, 8 or 32 ranges that a request's tokens are cut into (more for longer portions).
VOB_API int vob_mingru_scan(const void* zxg, const void* bz, const void* bx, float* state, const int* cu_q,
                            const int* state_slots, void* out, int B, int W, int num_slots, int chunks, int dtype, int* err,
                            cudaStream_t stream) {
  if (B <= 0 || W <= 0) return 0;
  if (B > 65535 || (chunks != 1 && chunks != 8 && chunks != 32)) return VOB_UNSUPPORTED;
  dim3 grid((W + 31) / 32, B), block(32, chunks);
#define VOB_GRU(TT, NN) \
  return launch_kernel(mingru_scan_kernel<TT, NN>, grid, block, 0, stream, (const TT*)zxg, (const TT*)bz, (const TT*)bx, state, cu_q, \
                       state_slots, (TT*)out, W, num_slots, err)
  if (dtype == VOB_F32) {
    if (chunks == 1) VOB_GRU(float, 1);
    if (chunks == 8) VOB_GRU(float, 8);
    VOB_GRU(float, 32);
  }
  if (dtype == VOB_BF16) {
    if (chunks == 1) VOB_GRU(__nv_bfloat16, 1);
    if (chunks == 8) VOB_GRU(__nv_bfloat16, 8);
    VOB_GRU(__nv_bfloat16, 32);
  }
#undef VOB_GRU
  return VOB_BAD_ARGUMENT;
}

// qfv [T, heads*(2 dk + dv)], bf [heads*dk] of the model's type; lower [heads*dk], nw [dv] float; state float
// [num_slots, heads, dk, dv]; out [T, heads*dv].  `fuse`: one block a (request, head) that also takes the norm (it must
// be able to hold the head: vob_hgrn2_can_fuse); else blocks of 128 threads and raw, float [T, heads*dv], in between.
// `chunks` > 1 (not with fuse): ranges that a request's tokens are cut into, with scratch of
// B * chunks * heads * dk * (dv + 1) floats.
VOB_API int vob_hgrn2_can_fuse(int dk, int dv) { return dv * hgrn2_parts(dk) <= (dk > 128 ? 256 : 512) ? 1 : 0; }

VOB_API int vob_hgrn2_scan(const void* qfv, const void* bf, const float* lower, const float* nw, float* state, const int* cu_q,
                           const int* state_slots, void* out, float* raw, float* scratch, int T, int B, int chunks, int heads,
                           int dk, int dv, float eps, int num_slots, int fuse, int dtype, int* err, cudaStream_t stream) {
  if (B <= 0 || T <= 0) return 0;
  if (heads <= 0 || dk <= 0 || dv <= 0 || dk > 256 || B > 65535 || (!fuse && !raw) || (fuse && !vob_hgrn2_can_fuse(dk, dv)) ||
      chunks < 1 || chunks > HG_MAX_CHUNKS || (chunks > 1 && (fuse || !scratch)))
    return VOB_UNSUPPORTED;
  if (dtype == VOB_F32)
    return dispatch_hgrn2<float>(qfv, bf, lower, nw, state, cu_q, state_slots, out, raw, scratch, T, B, chunks, heads, dk, dv, eps,
                                 num_slots, fuse, err, stream);
  if (dtype == VOB_BF16)
    return dispatch_hgrn2<__nv_bfloat16>(qfv, bf, lower, nw, state, cu_q, state_slots, out, raw, scratch, T, B, chunks, heads, dk,
                                         dv, eps, num_slots, fuse, err, stream);
  return VOB_BAD_ARGUMENT;
}
