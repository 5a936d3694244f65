// Attention whose values are its keys: rotation and cache write of a merged q|k row.
//
// A token's row holds nh query heads and kvh key heads of hd elements (whatever follows them in the row is not
// touched).  A query head is rotated in place.  A key head is written twice: as projected into the value plane, and
// rotated into the key plane, both at the token's slot (planes [pages, kvh, block_size, hd]; a slot of -1 writes
// nothing).  The rotation turns the first rot_dim elements of a head, element i with element i + rot_dim/2, by the angle
// float(position) * freq[i] (freq float [rot_dim/2]); angle, cosine and sine are float on both paths, and there is no
// table and so no largest position.  rot_dim 0 rotates nothing.
//
// One warp a head.  The products are spelled out with rounding intrinsics, so that a head gets the same bits whatever
// the launch shape.
#include "common.cuh"

namespace vob {

template <typename T>
__global__ void __launch_bounds__(128)
rope_shared_kv_write_kernel(T* qk, long row_stride, const int* __restrict__ positions, const int* __restrict__ slots,
                            const float* __restrict__ freq, T* kcache, T* vcache, int nh, int kvh, int hd, int rot_dim,
                            long num_slots, int block_size, int write_kv, int* err) {
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int head = blockIdx.y * (blockDim.x >> 5) + warp;
  const int pos = positions[t];
  const int slot = slots ? slots[t] : -1;
  pdl_wait();
  if (head >= nh + kvh) return;
  const bool is_q = head < nh;
  if (!is_q && (!write_kv || slot < 0)) return;
  if (!is_q && slot >= num_slots) {
    if (lane == 0) atomicOr(err, VOB_ERR_SLOT);
    return;
  }
  if (pos < 0) {
    if (lane == 0) atomicOr(err, VOB_ERR_POSITION);
    return;
  }
  T* row = qk + (size_t)t * row_stride + (size_t)head * hd;
  T* kdst = row;
  T* vdst = nullptr;
  if (!is_q) {
    const size_t off = (((size_t)(slot / block_size) * kvh + (head - nh)) * block_size + slot % block_size) * hd;
    kdst = kcache + off;
    vdst = vcache + off;
  }
  const int half = rot_dim >> 1;
  // pairs (i, i + half) for i < half; the elements from rot_dim on pass
  for (int i = lane; i < half; i += 32) {
    const float u = to_f<T>(row[i]), v = to_f<T>(row[i + half]);
    float sn, cs;
    sincosf(__fmul_rn((float)pos, freq[i]), &sn, &cs);
    if (vdst) { vdst[i] = from_f<T>(u); vdst[i + half] = from_f<T>(v); }
    kdst[i] = from_f<T>(__fsub_rn(__fmul_rn(u, cs), __fmul_rn(v, sn)));
    kdst[i + half] = from_f<T>(__fadd_rn(__fmul_rn(v, cs), __fmul_rn(u, sn)));
  }
  if (!is_q)
    for (int d = rot_dim + lane; d < hd; d += 32) {
      const T x = row[d];
      kdst[d] = x;
      vdst[d] = x;
    }
}

}  // namespace vob

using namespace vob;

VOB_API int vob_rope_shared_kv_write(void* qk, long row_stride, const int* positions, const int* slots, const float* freq,
                                     void* kcache, void* vcache, int T, int nh, int kvh, int hd, int rot_dim, long num_slots,
                                     int block_size, int write_kv, int dtype, int* err, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (hd <= 0 || block_size <= 0 || rot_dim < 0 || rot_dim > hd || rot_dim % 2 || (rot_dim > 0 && !freq)) return VOB_BAD_ARGUMENT;
  const int warps = 4;
  dim3 grid(T, (nh + kvh + warps - 1) / warps);
  if (dtype == VOB_F32)
    return launch_kernel(rope_shared_kv_write_kernel<float>, grid, warps * 32, 0, stream, (float*)qk, row_stride, positions,
                         slots, freq, (float*)kcache, (float*)vcache, nh, kvh, hd, rot_dim, num_slots, block_size, write_kv, err);
  if (dtype == VOB_BF16)
    return launch_kernel(rope_shared_kv_write_kernel<__nv_bfloat16>, grid, warps * 32, 0, stream, (__nv_bfloat16*)qk,
                         row_stride, positions, slots, freq, (__nv_bfloat16*)kcache, (__nv_bfloat16*)vcache, nh, kvh, hd,
                         rot_dim, num_slots, block_size, write_kv, err);
  return VOB_BAD_ARGUMENT;
}
