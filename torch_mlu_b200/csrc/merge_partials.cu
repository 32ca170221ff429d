// Log-sum-exp merge of partial attention results: the combine step of ring / context-parallel
// prefill, where a rank's queries meet the key/value blocks of every rank one block at a time.
// The reference has no counterpart (its attention runs on one device only); semantics follow
// the logsumexp mha_varlen_fwd returns (FlashAttention_internal.cpp:129): for each query row
//   lse' = log(exp(lse_acc) + exp(lse_part))
//   o_acc' = o_acc * exp(lse_acc - lse') + o_part * exp(lse_part - lse')
// with o_acc in fp32 (so that many blocks can be folded without 16-bit re-rounding), o_part the
// bf16 / f16 output of sdpa_b200_fwd. A row whose partial saw no key (lse_part = +inf, the library's
// convention) contributes nothing; an accumulator that has seen no key yet holds lse_acc = -inf.
// HBM-bound elementwise kernel: one warp per row, 128-bit accesses.
#include "kernels.h"
#include "ptx_sm100.cuh"

namespace sdpa_b200 {
namespace {

struct MergeParams {
  float* o_acc;               // [batch, heads, rows, head_dim] fp32, contiguous
  float* lse_acc;             // [batch, heads, rows] fp32, contiguous
  const uint16_t* o_part;     // bf16 or f16 bits
  const float* lse_part;      // [batch, heads, rows] fp32, contiguous
  int64_t p_batch_stride, p_head_stride, p_row_stride;  // o_part element strides
  int batch, heads, rows, head_dim;
};

template <bool kF16>
__global__ void __launch_bounds__(256) merge_partial_kernel(const MergeParams p) {
  const int lane = threadIdx.x & 31;
  const int64_t row_id = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  const int64_t total = static_cast<int64_t>(p.batch) * p.heads * p.rows;
  if (row_id >= total) return;
  const int r = static_cast<int>(row_id % p.rows);
  const int h = static_cast<int>((row_id / p.rows) % p.heads);
  const int b = static_cast<int>(row_id / (static_cast<int64_t>(p.rows) * p.heads));
  const float la = p.lse_acc[row_id];
  float lp = p.lse_part[row_id];
  if (lp == INFINITY) lp = -INFINITY;  // the partial saw no key for this row
  const float mx = fmaxf(la, lp);
  float wa = 0.f, wp = 0.f, ln = -INFINITY;
  if (mx != -INFINITY) {
    const float ea = __expf(la - mx), ep = __expf(lp - mx);
    const float sum = ea + ep;
    ln = mx + __logf(sum);
    wa = ea / sum;
    wp = ep / sum;
  }
  if (lane == 0) p.lse_acc[row_id] = ln;
  if (lane * 4 >= p.head_dim) return;
  float4* acc = reinterpret_cast<float4*>(p.o_acc + row_id * p.head_dim) + lane;
  const uint2 pv = *reinterpret_cast<const uint2*>(p.o_part + b * p.p_batch_stride + h * p.p_head_stride +
                                                   static_cast<int64_t>(r) * p.p_row_stride + lane * 4);
  const float2 p01 = unpack_16x2<kF16>(pv.x), p23 = unpack_16x2<kF16>(pv.y);
  float4 a = *acc;
  // wa == 0 also covers the uninitialised first fold (lse_acc = -inf): the old contents are ignored
  a.x = (wa == 0.f ? 0.f : a.x * wa) + p01.x * wp;
  a.y = (wa == 0.f ? 0.f : a.y * wa) + p01.y * wp;
  a.z = (wa == 0.f ? 0.f : a.z * wa) + p23.x * wp;
  a.w = (wa == 0.f ? 0.f : a.w * wa) + p23.y * wp;
  *acc = a;
}

}  // namespace
}  // namespace sdpa_b200

extern "C" SDPA_B200_API int sdpa_b200_merge_partial(float* o_acc, float* lse_acc, const void* o_part,
                                                     const float* lse_part, int32_t batch, int32_t heads,
                                                     int32_t rows, int32_t head_dim, int32_t dtype,
                                                     int64_t part_batch_stride,
                                                     int64_t part_head_stride, int64_t part_row_stride, void* stream) {
  using namespace sdpa_b200;
  if (o_acc == nullptr || lse_acc == nullptr || o_part == nullptr || lse_part == nullptr) {
    set_error("merge_partial: NULL pointer");
    return SDPA_B200_INVALID_ARG;
  }
  if (dtype != SDPA_B200_BF16 && dtype != SDPA_B200_F16) {
    set_error("merge_partial: o_part must be bf16 or f16 (dtype code %d)", dtype);
    return SDPA_B200_UNSUPPORTED;
  }
  if (head_dim <= 0 || head_dim > 128 || head_dim % 8 != 0) {
    set_error("merge_partial: head_dim must be a multiple of 8 up to 128 (got %d)", head_dim);
    return SDPA_B200_UNSUPPORTED;
  }
  if (batch <= 0 || heads <= 0 || rows <= 0 || part_row_stride % 4 != 0 || part_head_stride % 4 != 0 ||
      part_batch_stride % 4 != 0 || (reinterpret_cast<uintptr_t>(o_acc) & 15u) || (reinterpret_cast<uintptr_t>(o_part) & 7u)) {
    set_error("merge_partial: sizes must be positive, o_acc 16-byte aligned, o_part strides multiples of 4 elements");
    return SDPA_B200_INVALID_ARG;
  }
  MergeParams m;
  m.o_acc = o_acc;
  m.lse_acc = lse_acc;
  m.o_part = static_cast<const uint16_t*>(o_part);
  m.lse_part = lse_part;
  m.p_batch_stride = part_batch_stride;
  m.p_head_stride = part_head_stride;
  m.p_row_stride = part_row_stride;
  m.batch = batch;
  m.heads = heads;
  m.rows = rows;
  m.head_dim = head_dim;
  const int64_t total = static_cast<int64_t>(batch) * heads * rows;
  const unsigned grid = static_cast<unsigned>((total + 7) / 8);
  if (dtype == SDPA_B200_F16) merge_partial_kernel<true><<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(m);
  else merge_partial_kernel<false><<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(m);
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) {
    set_error("merge_partial: launch failed: %s", cudaGetErrorString(err));
    return SDPA_B200_LAUNCH_FAILED;
  }
  count_launch();
  return SDPA_B200_OK;
}
