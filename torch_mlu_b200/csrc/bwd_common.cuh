// Pieces shared by the backward kernels (bwd_sm100.cu: dK/dV and dQ kernels with a fixed summation order;
// bwd_fused_sm100.cu: the fused kernel): tile constants, the kernel parameter block and the MMA issue helpers.
#pragma once

#include <cuda_bf16.h>

#include "kernels.h"
#include "ptx_sm100.cuh"

namespace sdpa_b200 {

#ifndef SDPA_BWD_POLY_DKDV
#define SDPA_BWD_POLY_DKDV 2  // of every 4 column pairs, how many use the polynomial 2^x (dK/dV kernel)
#endif
#ifndef SDPA_BWD_POLY_DQ
#define SDPA_BWD_POLY_DQ 1    // the same for the dQ kernel
#endif

constexpr int kTile = 128;  // rows per tile (queries or keys)
constexpr uint32_t kTileBytes = kTile * 128 * 2;  // one shared-memory slot (head_dim 64 uses half of it)
constexpr uint32_t kHalfBytes = kTileBytes / 2;

struct BwdKernelParams {
  const float* lse2;   // padded [batch, heads_q, lq_pad]
  const float* delta;  // padded [batch, heads_q, lq_pad]
  uint16_t* dq;  // bf16 or f16 bits
  uint16_t* dk;
  uint16_t* dv;
  const int32_t* cu_q;
  const int32_t* cu_k;
  uint32_t* status;
  int64_t dq_batch_stride, dq_head_stride, dq_row_stride;
  int64_t dk_batch_stride, dk_head_stride, dk_row_stride;
  int64_t dv_batch_stride, dv_head_stride, dv_row_stride;
  int seqlen_q, seqlen_k, heads_q, heads_kv, kv_group, lq_pad;
  int num_row_blocks;  // blocks of 128 stationary rows (keys for dK/dV, queries for dQ)
  int num_bh, heads_x, heads_per_wave;  // CTA order, see the top of bwd_tile_kernel
  float scale, scale_log2;
  int is_causal;
  int head_dim;  // <= kD (the kernels are built for 64 and 128 columns; TMA pads loads and clips stores)
  // dropout (kernels built with kDrop): one keep bit per (query, key) pair in both orientations, see
  // dropout_mask.cu. P is recomputed without dropout; dV takes P o M / (1 - p), dS = P o (M o dP / (1 - p) - delta).
  const uint32_t* keep_rows;  // [batch*heads_q][keep_lq_pad][keep_lk_pad / 32]: dQ kernel
  const uint32_t* keep_cols;  // [batch*heads_q][keep_lk_pad][keep_lq_pad / 32]: dK/dV kernel
  int keep_lq_pad, keep_lk_pad;  // longest sequences rounded up to 128: the bits per row
  int keep_q_rows, keep_k_rows;  // rows per leading index: the same for dense tensors, total tokens + 128 when packed
  float keep_scale;  // 1 / (1 - dropout_p)
  // additive bias (kernels built with kBias): the scores are scale * Q K^T + bias; the gradient of the bias is
  // dS itself, written by the dQ kernel (whose thread owns a query row and 64 consecutive keys of it)
  const uint16_t* bias;
  int64_t bias_batch_stride, bias_head_stride, bias_row_stride;
  const uint16_t* bias_t;  // or null: the bias with keys and queries exchanged (unit query stride), for dK/dV
  int64_t bias_t_batch_stride, bias_t_head_stride, bias_t_row_stride;
  uint16_t* dbias;  // or null
  int64_t dbias_batch_stride, dbias_head_stride, dbias_row_stride;
  float inv_scale;  // 1 / softmax_scale
  // fused kernel: fp32 dQ accumulator, 128-row tiles of [head_dim / 4][128 rows][4] floats (a warp's 32 rows of one
  // 4-column group are 512 contiguous bytes). Row index: dense (batch * heads_q + head) * lq_pad + query, packed
  // head * dq_acc_rows + token.
  float* dq_acc;
  int dq_acc_rows;  // packed: rows per head (total_q rounded up to 128, plus 128)
#ifdef SDPA_BWD_STAMPS
  float* stamps;  // [mode 2][role 4][item 24][event 8] SM cycles since CTA start, one CTA per mode
#endif
};

// bwd_fused_sm100.cu: the fused kernel and the dQ conversion behind it. `grid` and the CTA-order fields of `kp` are
// those of the dK/dV kernel (one CTA per key block); dq_acc holds bwd_fused_workspace_bytes() bytes.
size_t bwd_fused_workspace_bytes(const sdpa_b200_params& p, int lq_pad);
int launch_bwd_fused(const sdpa_b200_params& p, BwdKernelParams kp, float* dq_acc, int grid, cudaStream_t stream,
                     const CUtensorMap& tm_q, const CUtensorMap& tm_k, const CUtensorMap& tm_v, const CUtensorMap& tm_do,
                     const CUtensorMap& tm_dv, const CUtensorMap& tm_dk);

template <bool kF16>
constexpr uint32_t kIdescSS = umma_idesc_16(kTile, kTile, false, false, kF16);
template <int kD, bool kF16>
constexpr uint32_t kIdescTS = umma_idesc_16(kTile, kD, false, true, kF16);

// T = X Y^T, contraction over head_dim, both operands K-major in shared memory
template <int kD, bool kF16>
__device__ __forceinline__ void issue_xyT(uint32_t t, uint32_t x_smem, uint32_t y_smem) {
  const uint32_t a_lo = umma_desc_lo_kmajor(x_smem);
  const uint32_t b_lo = umma_desc_lo_kmajor(y_smem);
  umma_ss_lo<kIdescSS<kF16>, false>(t, a_lo, b_lo);
#pragma unroll
  for (int ks = 1; ks < kD / 16; ++ks) {
    const uint32_t off = ((ks >> 2) * kHalfBytes + (ks & 3) * 32) >> 4;
    umma_ss_lo<kIdescSS<kF16>, true>(t, a_lo + off, b_lo + off);
  }
}

// ACC (+)= W Y over rows [64*half, 64*half + 64) of the Y tile. W (bf16, lane = stationary row)
// for those rows starts at TMEM column `w` (32 columns).
template <int kD, bool kF16>
__device__ __forceinline__ void issue_wy_half(uint32_t acc, uint32_t w, uint32_t y_smem, int half, bool accumulate) {
  const uint32_t b_lo = umma_desc_lo_mnmajor(y_smem, kHalfBytes);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int ks = half * 4 + i;
    umma_ts_lo<kIdescTS<kD, kF16>>(acc, w + i * 8, b_lo + ks * (2048 >> 4), (accumulate || ks > 0) ? 1u : 0u);
  }
}

__device__ __forceinline__ void bulk_load_1d(uint32_t dst_smem, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst_smem),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}

// A grid launched with programmatic stream serialization may start before the grid in front of it has finished. This
// wait returns once that grid has completed and its stores are visible; a CTA that executes it before it exits keeps its
// own grid from completing first, so whatever follows in the stream is ordered behind BOTH grids, as it would be without
// the overlap. (A no-op for a grid launched the ordinary way.)
__device__ __forceinline__ void wait_for_previous_grid() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// both halves of a packed 16-bit pair survive or die by two keep bits (bit 0 -> low half)
__device__ __forceinline__ uint32_t keep_pair_mask(uint32_t two_bits) {
  return ((two_bits & 1u) ? 0x0000ffffu : 0u) | ((two_bits & 2u) ? 0xffff0000u : 0u);
}

}  // namespace sdpa_b200
