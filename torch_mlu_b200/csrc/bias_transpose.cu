// Transposed copy of an attention bias for the backward pass: [.., Lq, Lk] -> [.., Lk, ld >= Lq].
//
// The dK/dV kernel's threads own keys and walk over queries, so it reads a bias stored query-major two bytes
// at a time; with this copy (sdpa_b200_params.bias_t) it reads 16 bytes at a time. HBM-bound: every element is
// read once and written once through a 64 x 64 shared-memory tile, 16 bytes per thread on both sides.
#include "kernels.h"

namespace sdpa_b200 {
namespace {

struct TransposeParams {
  const uint16_t* src;
  uint16_t* dst;
  int64_t batch_stride, head_stride, row_stride;  // of src, in elements
  int heads, seqlen_q, seqlen_k, ld;
};

__global__ void __launch_bounds__(256) bias_transpose_kernel(const TransposeParams p) {
  // [key][query]; 33 words per row: the transposing 2-byte writes of a warp (rows 8 apart) fall on 4 banks instead of
  // one, the 4-byte reads of the second phase on 32 different banks
  __shared__ uint16_t tile[64][66];
  const int t = threadIdx.x;
  const int q0 = blockIdx.y * 64, k0 = blockIdx.x * 64;
  const int z = blockIdx.z, b = z / p.heads, h = z - b * p.heads;
  const uint16_t* src = p.src + b * p.batch_stride + h * p.head_stride;
#pragma unroll
  for (int pass = 0; pass < 2; ++pass) {
    const int r = pass * 32 + (t >> 3), c = (t & 7) * 8;
    const int q = q0 + r, k = k0 + c;
    uint4 w = make_uint4(0u, 0u, 0u, 0u);
    // a chunk that straddles the last key reads row padding, which the bias rules guarantee
    if (q < p.seqlen_q && k < p.seqlen_k) w = *reinterpret_cast<const uint4*>(src + static_cast<int64_t>(q) * p.row_stride + k);
    const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const uint16_t e = static_cast<uint16_t>(ww[i >> 1] >> ((i & 1) * 16));
      tile[c + i][r] = (k + i < p.seqlen_k) ? e : static_cast<uint16_t>(0);
    }
  }
  __syncthreads();
#pragma unroll
  for (int pass = 0; pass < 2; ++pass) {
    const int kr = pass * 32 + (t >> 3), c = (t & 7) * 8;
    const int k = k0 + kr, q = q0 + c;
    if (k < p.seqlen_k && q < p.ld) {
      uint32_t o[4];
#pragma unroll
      for (int i = 0; i < 4; ++i)
        o[i] = static_cast<uint32_t>(tile[kr][c + 2 * i]) | (static_cast<uint32_t>(tile[kr][c + 2 * i + 1]) << 16);
      *reinterpret_cast<uint4*>(p.dst + (static_cast<int64_t>(z) * p.seqlen_k + k) * p.ld + q) = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
}

}  // namespace
}  // namespace sdpa_b200

using namespace sdpa_b200;

extern "C" SDPA_B200_API int sdpa_b200_transpose_bias(const void* bias, int64_t batch_stride, int64_t head_stride,
                                                      int64_t row_stride, int32_t batch, int32_t heads, int32_t seqlen_q,
                                                      int32_t seqlen_k, void* out, int64_t out_row_stride, void* stream) {
  auto bad = [](int64_t s) { return s < 0 || (s % 8) != 0; };
  if (bias == nullptr || out == nullptr || (reinterpret_cast<uintptr_t>(bias) & 15u) || (reinterpret_cast<uintptr_t>(out) & 15u) ||
      bad(batch_stride) || bad(head_stride) || bad(row_stride) || row_stride == 0) {
    set_error("transpose_bias: 16-byte aligned pointers, strides that are multiples of 8 elements and a non-zero row stride");
    return SDPA_B200_INVALID_ARG;
  }
  if (batch <= 0 || heads <= 0 || seqlen_q <= 0 || seqlen_k <= 0 || static_cast<int64_t>(batch) * heads > 65535 ||
      out_row_stride < (static_cast<int64_t>(seqlen_q) + 7) / 8 * 8 || (out_row_stride % 8) != 0) {
    set_error("transpose_bias: sizes must be positive, batch*heads at most 65535, out_row_stride a multiple of 8 that "
              "holds seqlen_q");
    return SDPA_B200_INVALID_ARG;
  }
  TransposeParams t;
  t.src = static_cast<const uint16_t*>(bias);
  t.dst = static_cast<uint16_t*>(out);
  t.batch_stride = batch_stride;
  t.head_stride = head_stride;
  t.row_stride = row_stride;
  t.heads = heads;
  t.seqlen_q = seqlen_q;
  t.seqlen_k = seqlen_k;
  t.ld = static_cast<int>(out_row_stride);
  dim3 grid((seqlen_k + 63) / 64, (static_cast<int>(out_row_stride) + 63) / 64, batch * heads);
  if (grid.y > 65535) {
    set_error("transpose_bias: seqlen_q too long (%d)", seqlen_q);
    return SDPA_B200_INVALID_ARG;
  }
  bias_transpose_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(t);
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) {
    set_error("transpose_bias: launch failed: %s", cudaGetErrorString(err));
    return SDPA_B200_LAUNCH_FAILED;
  }
  count_launch();
  return SDPA_B200_OK;
}
