// Dropout keep-masks for the attention kernels, one bit per (query, key) pair.
//
// The reference draws its dropout pattern inside the vendor kernel from a Philox seed / offset pair
// (torch_mlu/csrc/aten/operators/cnnl/internal/FlashAttention_internal.cpp:190-214) and hands the pair to
// the backward pass, which has to reproduce the pattern. Here the pattern is a separate, HBM-cheap
// product: one bit per pair (Lq*Lk/8 bytes per head against 2*(Lq+Lk)*D of Q/K/V/O), written in both
// orientations so that every attention kernel finds the bits of its thread's row in one aligned load:
//   keep_rows [batch*heads][Lq_pad][Lk_pad/32]  bit (k & 31) of word (q, k >> 5): forward and dQ kernels
//   keep_cols [batch*heads][Lk_pad][Lq_pad/32]  bit (q & 31) of word (k, q >> 5): dK/dV kernel
// with Lq_pad, Lk_pad the lengths rounded up to 128 (a tile), so rows are 16-byte multiples and tiles
// never read outside the array.
//
// Random stream: Philox4x32-10 (Salmon et al., SC'11). One call yields 16 bytes = the keep decisions of
// 16 consecutive queries for one key: counter = (key, query / 16, batch*heads + head, low half of the
// offset), key = (low half of the seed, high half of the seed xor high half of the offset). Element (q, k) is
// kept when byte (q & 15) of the output >= round(p * 256).
#include "kernels.h"

namespace sdpa_b200 {
namespace {

__device__ __forceinline__ uint4 philox4x32_10(uint4 c, uint2 k) {
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint32_t hi0 = __umulhi(0xD2511F53u, c.x), lo0 = 0xD2511F53u * c.x;
    const uint32_t hi1 = __umulhi(0xCD9E8D57u, c.z), lo1 = 0xCD9E8D57u * c.z;
    c = make_uint4(hi1 ^ c.y ^ k.x, lo1, hi0 ^ c.w ^ k.y, lo0);
    k.x += 0x9E3779B9u;
    k.y += 0xBB67AE85u;
  }
  return c;
}

// 16 keep bits from 16 bytes: bit j set when byte j >= drop. `drop4` holds the threshold in all four bytes. The
// per-byte unsigned compare is done on the whole word: with H = 0x80 in every byte, (w | H) - (t & ~H) cannot borrow
// across bytes and its top bit per byte says whether the low seven bits of w reach those of t; the bytes' own top bits
// decide the rest: w >= t  <=>  (wh & ~th) | (~(wh ^ th) & zh), one three-input logic instruction. One multiply then
// gathers the four top bits into adjacent bits (2^21 + 2^14 + 2^7 + 2^0 moves bits 7, 15, 23, 31 to 28, 29, 30, 31).
__device__ __forceinline__ uint32_t keep_bits16(uint4 r, uint32_t drop4) {
  const uint32_t w[4] = {r.x, r.y, r.z, r.w};
  const uint32_t t_low = drop4 & 0x7f7f7f7fu;
  uint32_t bits = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint32_t z = (w[i] | 0x80808080u) - t_low;
    const uint32_t ge = ((w[i] & ~drop4) | (~(w[i] ^ drop4) & z)) & 0x80808080u;
    bits |= ((ge * 0x00204081u) >> 28) << (4 * i);
  }
  return bits;
}

// Transposes a 32 x 32 bit block held one word per lane: afterwards bit c of lane r is what bit r of lane c was.
// Five butterfly stages (block sizes 16 ... 1): each lane keeps the half of its word that stays and takes the other
// half from the lane `j` away.
__device__ __forceinline__ uint32_t transpose_bits_32x32(uint32_t x, int lane) {
  constexpr uint32_t kMask[5] = {0x0000ffffu, 0x00ff00ffu, 0x0f0f0f0fu, 0x33333333u, 0x55555555u};
#pragma unroll
  for (int s = 0; s < 5; ++s) {
    const int j = 16 >> s;
    const uint32_t m = kMask[s];
    const uint32_t y = __shfl_xor_sync(0xffffffffu, x, j);
    x = (lane & j) ? (((y >> j) & m) | (x & ~m)) : ((x & m) | ((y << j) & ~m));
  }
  return x;
}

struct MaskParams {
  uint32_t* keep_rows;
  uint32_t* keep_cols;
  int lq_pad, lk_pad;
  uint32_t seed_lo, seed_hi, offset, drop4;
  int causal_shift;  // tiles whose first key lies past (last query of the tile + causal_shift) are zero-filled
  // packed (varlen) form: rows are packed token indices, bits are positions inside the token's sequence
  const int32_t* cu_q;
  const int32_t* cu_k;
  int heads, total_q_pad, total_k_pad, is_causal;
};

// One CTA (4 warps) per 128 x 128 tile of one head; warp w owns keys [32w, 32w + 32), lane = key.
__global__ void __launch_bounds__(128) dropout_mask_kernel(const MaskParams p) {
  __shared__ uint32_t rows[128][4];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t bh = blockIdx.z;
  const int q0 = blockIdx.y * 128, k0 = blockIdx.x * 128;
  const uint32_t k = k0 + warp * 32 + lane;
  uint32_t col[4] = {0u, 0u, 0u, 0u};
  // a tile the causal mask hides completely is never read for its bits: write zeros and skip the generator
  const bool hidden = k0 > q0 + 127 + p.causal_shift;
  if (!hidden) {
#pragma unroll
    for (int qb = 0; qb < 4; ++qb) {
      const uint32_t g = (q0 + qb * 32) >> 4;  // first group of 16 queries
      const uint32_t lo = keep_bits16(philox4x32_10(make_uint4(k, g, bh, p.offset), make_uint2(p.seed_lo, p.seed_hi)), p.drop4);
      const uint32_t hi = keep_bits16(philox4x32_10(make_uint4(k, g + 1, bh, p.offset), make_uint2(p.seed_lo, p.seed_hi)), p.drop4);
      col[qb] = lo | (hi << 16);
    }
  }
  // key-major words: four consecutive words (128 queries) per key
  *reinterpret_cast<uint4*>(p.keep_cols + (static_cast<size_t>(bh) * p.lk_pad + k) * (p.lq_pad >> 5) + (q0 >> 5)) =
      make_uint4(col[0], col[1], col[2], col[3]);
  // query-major words: transpose the 32 x 32 bit blocks across the warp, gather the four key blocks of the
  // tile in shared memory, then one 16-byte store per query row
#pragma unroll
  for (int qb = 0; qb < 4; ++qb) {
    rows[qb * 32 + lane][warp] = hidden ? 0u : transpose_bits_32x32(col[qb], lane);  // `hidden` is uniform for the CTA
  }
  __syncthreads();
  const int q = q0 + threadIdx.x;
  *reinterpret_cast<uint4*>(p.keep_rows + (static_cast<size_t>(bh) * p.lq_pad + q) * (p.lk_pad >> 5) + (k0 >> 5)) =
      make_uint4(rows[threadIdx.x][0], rows[threadIdx.x][1], rows[threadIdx.x][2], rows[threadIdx.x][3]);
}

// Packed form: one CTA per 128 x 128 tile of one (sequence, head) in the sequence's own coordinates, so that the
// pattern of a sequence is the dense pattern of the same batch index. keep_rows [heads][total_q_pad][lk_pad/32],
// keep_cols [heads][total_k_pad][lq_pad/32] with lq_pad / lk_pad from the longest sequences. Only words that an
// attention kernel can read are written (the arrays arrive zero-filled): rows of real tokens, tiles the causal
// mask does not hide completely.
__global__ void __launch_bounds__(128) dropout_mask_varlen_kernel(const MaskParams p) {
  __shared__ uint32_t rows[128][4];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int z = blockIdx.z, b = z / p.heads, h = z - b * p.heads;
  const int q_off = p.cu_q[b], len_q = p.cu_q[b + 1] - q_off;
  const int k_off = p.cu_k[b], len_k = p.cu_k[b + 1] - k_off;
  const int q0 = blockIdx.y * 128, k0 = blockIdx.x * 128;
  if (q0 >= len_q || k0 >= len_k) return;
  if (p.is_causal && k0 > q0 + 127 + (len_k - len_q)) return;
  const uint32_t k = k0 + warp * 32 + lane;
  uint32_t col[4];
#pragma unroll
  for (int qb = 0; qb < 4; ++qb) {
    const uint32_t g = (q0 + qb * 32) >> 4;
    const uint32_t lo = keep_bits16(philox4x32_10(make_uint4(k, g, z, p.offset), make_uint2(p.seed_lo, p.seed_hi)), p.drop4);
    const uint32_t hi = keep_bits16(philox4x32_10(make_uint4(k, g + 1, z, p.offset), make_uint2(p.seed_lo, p.seed_hi)), p.drop4);
    col[qb] = lo | (hi << 16);
  }
  if (static_cast<int>(k) < len_k)
    *reinterpret_cast<uint4*>(p.keep_cols + (static_cast<size_t>(h) * p.total_k_pad + k_off + k) * (p.lq_pad >> 5) + (q0 >> 5)) =
        make_uint4(col[0], col[1], col[2], col[3]);
#pragma unroll
  for (int qb = 0; qb < 4; ++qb) {
    rows[qb * 32 + lane][warp] = transpose_bits_32x32(col[qb], lane);
  }
  __syncthreads();
  const int q = q0 + threadIdx.x;
  if (q < len_q)
    *reinterpret_cast<uint4*>(p.keep_rows + (static_cast<size_t>(h) * p.total_q_pad + q_off + q) * (p.lk_pad >> 5) + (k0 >> 5)) =
        make_uint4(rows[threadIdx.x][0], rows[threadIdx.x][1], rows[threadIdx.x][2], rows[threadIdx.x][3]);
}

}  // namespace

uint32_t dropout_drop_byte(float dropout_p) {
  int d = static_cast<int>(dropout_p * 256.0f + 0.5f);
  return static_cast<uint32_t>(d < 0 ? 0 : (d > 255 ? 255 : d));
}

}  // namespace sdpa_b200

using namespace sdpa_b200;

extern "C" SDPA_B200_API int sdpa_b200_dropout_keep_mask(uint64_t seed, uint64_t offset, float dropout_p, int32_t batch,
                                                         int32_t heads, int32_t seqlen_q, int32_t seqlen_k,
                                                         int32_t is_causal, uint32_t* keep_rows, uint32_t* keep_cols,
                                                         void* stream) {
  if (keep_rows == nullptr || keep_cols == nullptr || (reinterpret_cast<uintptr_t>(keep_rows) & 15u) ||
      (reinterpret_cast<uintptr_t>(keep_cols) & 15u)) {
    set_error("dropout_keep_mask: keep_rows and keep_cols must be 16-byte aligned device pointers");
    return SDPA_B200_INVALID_ARG;
  }
  if (batch <= 0 || heads <= 0 || seqlen_q <= 0 || seqlen_k <= 0 || static_cast<int64_t>(batch) * heads > 65535) {
    set_error("dropout_keep_mask: sizes must be positive and batch*heads at most 65535 (got %d, %d, %d, %d)", batch, heads,
              seqlen_q, seqlen_k);
    return SDPA_B200_INVALID_ARG;
  }
  if (!(dropout_p > 0.f) || !(dropout_p < 1.f)) {
    set_error("dropout_keep_mask: dropout_p must be inside (0, 1) (got %g)", static_cast<double>(dropout_p));
    return SDPA_B200_INVALID_ARG;
  }
  MaskParams m = {};
  m.keep_rows = keep_rows;
  m.keep_cols = keep_cols;
  m.lq_pad = (seqlen_q + 127) / 128 * 128;
  m.lk_pad = (seqlen_k + 127) / 128 * 128;
  m.seed_lo = static_cast<uint32_t>(seed);
  m.seed_hi = static_cast<uint32_t>(seed >> 32) ^ static_cast<uint32_t>(offset >> 32);  // all 64 offset bits count
  m.offset = static_cast<uint32_t>(offset);
  m.drop4 = dropout_drop_byte(dropout_p) * 0x01010101u;
  // bottom-right aligned causal mask: key k is visible to query q when k <= q + seqlen_k - seqlen_q
  m.causal_shift = is_causal ? seqlen_k - seqlen_q : (1 << 30);
  dim3 grid(m.lk_pad / 128, m.lq_pad / 128, batch * heads);
  if (grid.y > 65535) {
    set_error("dropout_keep_mask: seqlen_q too long (%d)", seqlen_q);
    return SDPA_B200_INVALID_ARG;
  }
  dropout_mask_kernel<<<grid, 128, 0, static_cast<cudaStream_t>(stream)>>>(m);
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) {
    set_error("dropout_keep_mask: launch failed: %s", cudaGetErrorString(err));
    return SDPA_B200_LAUNCH_FAILED;
  }
  count_launch();
  return SDPA_B200_OK;
}

extern "C" SDPA_B200_API int sdpa_b200_dropout_keep_mask_varlen(uint64_t seed, uint64_t offset, float dropout_p, int32_t batch,
                                                                int32_t heads, const int32_t* cu_seqlens_q,
                                                                const int32_t* cu_seqlens_k, int32_t total_q, int32_t total_k,
                                                                int32_t max_seqlen_q, int32_t max_seqlen_k, int32_t is_causal,
                                                                uint32_t* keep_rows, uint32_t* keep_cols, void* stream) {
  if (keep_rows == nullptr || keep_cols == nullptr || cu_seqlens_q == nullptr || cu_seqlens_k == nullptr ||
      (reinterpret_cast<uintptr_t>(keep_rows) & 15u) || (reinterpret_cast<uintptr_t>(keep_cols) & 15u)) {
    set_error("dropout_keep_mask_varlen: NULL pointer, or keep_rows / keep_cols not 16-byte aligned");
    return SDPA_B200_INVALID_ARG;
  }
  if (batch <= 0 || heads <= 0 || total_q <= 0 || total_k <= 0 || max_seqlen_q <= 0 || max_seqlen_k <= 0 ||
      static_cast<int64_t>(batch) * heads > 65535) {
    set_error("dropout_keep_mask_varlen: sizes must be positive and batch*heads at most 65535");
    return SDPA_B200_INVALID_ARG;
  }
  if (!(dropout_p > 0.f) || !(dropout_p < 1.f)) {
    set_error("dropout_keep_mask_varlen: dropout_p must be inside (0, 1) (got %g)", static_cast<double>(dropout_p));
    return SDPA_B200_INVALID_ARG;
  }
  MaskParams m = {};
  m.keep_rows = keep_rows;
  m.keep_cols = keep_cols;
  m.lq_pad = (max_seqlen_q + 127) / 128 * 128;
  m.lk_pad = (max_seqlen_k + 127) / 128 * 128;
  m.seed_lo = static_cast<uint32_t>(seed);
  m.seed_hi = static_cast<uint32_t>(seed >> 32) ^ static_cast<uint32_t>(offset >> 32);
  m.offset = static_cast<uint32_t>(offset);
  m.drop4 = dropout_drop_byte(dropout_p) * 0x01010101u;
  m.causal_shift = 0;
  m.cu_q = cu_seqlens_q;
  m.cu_k = cu_seqlens_k;
  m.heads = heads;
  m.total_q_pad = total_q + 128;
  m.total_k_pad = total_k + 128;
  m.is_causal = is_causal;
  dim3 grid(m.lk_pad / 128, m.lq_pad / 128, batch * heads);
  if (grid.y > 65535) {
    set_error("dropout_keep_mask_varlen: max_seqlen_q too long (%d)", max_seqlen_q);
    return SDPA_B200_INVALID_ARG;
  }
  dropout_mask_varlen_kernel<<<grid, 128, 0, static_cast<cudaStream_t>(stream)>>>(m);
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) {
    set_error("dropout_keep_mask_varlen: launch failed: %s", cudaGetErrorString(err));
    return SDPA_B200_LAUNCH_FAILED;
  }
  count_launch();
  return SDPA_B200_OK;
}
