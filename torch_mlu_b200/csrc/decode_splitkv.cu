// Split-KV decode attention (seqlen_q == 1) for sm_100a: the HBM-bandwidth-bound member of
// the forward path. The reference has no counterpart - its dispatcher turns Lq = 1 away from
// the fused kernel (torch_mlu/csrc/aten/operators/cnnl/transformers/sdp_utils.h:510-521) -
// so semantics follow mha_varlen_fwd (FlashAttention_internal.cpp:57-267) with one query row.
//
// Work unit: (batch, kv head, split of the key range). A CTA of 4 warps streams its keys
// once; each thread reads K and V rows with 128-bit loads straight into mma.sync fragments
// (the contraction index of Q K^T is permuted so a 16-byte load IS a B fragment pair; V
// pairs of keys are interleaved with two byte-permutes per word). All query heads of the
// GQA group ride in the M dimension of m16n8k16, so K/V bytes are read once per group.
// Per-split partial (O, lse) go to the workspace; a second kernel merges the splits with
// warp shuffles.
#include <cuda_bf16.h>

#include <mutex>

#include "kernels.h"
#include "ptx_sm100.cuh"

namespace sdpa_b200 {
namespace {

constexpr int kDecWarps = 4;
constexpr int kDecThreads = kDecWarps * 32;
constexpr int kKeysPerStep = 16;  // keys one warp handles per loop iteration
constexpr int kMaxD = 128;  // head_dim 64 and 128 are built
constexpr int kMaxSplits = 128;

struct DecodeParams {
  const uint16_t* q;  // bf16 or f16 bits (f16 != 0)
  const uint16_t* k;
  const uint16_t* v;
  uint16_t* out;
  float* lse;
  float* part_o;    // [batch, heads_q, splits, head_dim] fp32, normalised per split
  float* part_lse;  // [batch, heads_q, splits] fp32, log2 domain
  int64_t q_batch_stride, q_head_stride;
  int64_t k_batch_stride, k_head_stride, k_row_stride;
  int64_t v_batch_stride, v_head_stride, v_row_stride;
  int64_t o_batch_stride, o_head_stride;
  int heads_q, heads_kv, group, chunks, len_k, num_splits, keys_per_split, head_dim;
  float scale_log2;
  int f16;
};

__device__ __forceinline__ uint4 ld_stream_16(const void* p) {
  uint4 r;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(p));
  return r;
}

template <bool kF16>
__device__ __forceinline__ void mma_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                          uint32_t a3, uint32_t b0, uint32_t b1) {
  if constexpr (kF16)
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, "
        "{%8, %9}, {%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  else
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, "
        "{%8, %9}, {%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Same MMA when only fragment rows 0-7 carry query heads: rows 8-15 of A are zero, so their
// accumulators are constants and need no live registers.
template <bool kF16>
__device__ __forceinline__ void mma_16816_lo(float& c0, float& c1, uint32_t a0, uint32_t a2,
                                             uint32_t b0, uint32_t b1) {
  float d2, d3;
  if constexpr (kF16)
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %5}, "
        "{%7, %8}, {%0, %1, %9, %9};"
        : "+f"(c0), "+f"(c1), "=f"(d2), "=f"(d3)
        : "r"(a0), "r"(0u), "r"(a2), "r"(b0), "r"(b1), "f"(0.f));
  else
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %5}, "
        "{%7, %8}, {%0, %1, %9, %9};"
        : "+f"(c0), "+f"(c1), "=f"(d2), "=f"(d3)
        : "r"(a0), "r"(0u), "r"(a2), "r"(b0), "r"(b1), "f"(0.f));
}

template <bool kHi, bool kF16>
__device__ __forceinline__ void mma_rows(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  if constexpr (kHi) mma_16816<kF16>(c, a[0], a[1], a[2], a[3], b0, b1);
  else mma_16816_lo<kF16>(c[0], c[1], a[0], a[2], b0, b1);
}

__device__ __forceinline__ float quad_max(float x) {
  x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, 1));
  x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, 2));
  return x;
}

__device__ __forceinline__ float quad_sum(float x) {
  x += __shfl_xor_sync(0xffffffffu, x, 1);
  x += __shfl_xor_sync(0xffffffffu, x, 2);
  return x;
}

// Shared scratch for the 4-warp merge: per warp 16 rows x (128 O + m + l).
template <int kD>
struct DecodeSmem {
  float o[kDecWarps][16][kD];
  float m[kDecWarps][16];
  float l[kDecWarps][16];
};

// kHi: the GQA group has more than 8 query heads, so fragment rows 8-15 are in use too.
template <bool kHi, int kD, bool kF16>
__global__ void __launch_bounds__(kDecThreads, 3) decode_splitkv_kernel(const DecodeParams p) {
  __shared__ DecodeSmem<kD> sm;
  constexpr int kKSteps = kD / 16;   // MMAs over head_dim for Q K^T
  constexpr int kLoads = kD / 32;    // 16-byte K loads per thread and key
  constexpr int kHalves = kD / 64;   // 64-column halves of V / O
  constexpr int kNBlocks = kD / 8;   // 8-column output blocks of P V
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int g = lane >> 2;  // fragment row (query head within the chunk) / key within a block
  const int t = lane & 3;
  const int split = blockIdx.x;
  const int hkv = blockIdx.y / p.chunks;
  const int chunk = blockIdx.y % p.chunks;
  const int b = blockIdx.z;
  const int head0 = hkv * p.group + chunk * 16;        // first query head of this CTA
  const int nheads = min(16, p.group - chunk * 16);    // query heads this CTA serves

  const int k_begin = split * p.keys_per_split;
  const int k_end = min(p.len_k, k_begin + p.keys_per_split);

  // ---- Q fragments. MMA i (0..7) contracts over d = (i/2)*32 + 8t + 4(i&1) + {0,1 | 2,3}.
  uint32_t qa[kKSteps][4];
  {
    const uint16_t* qb = p.q + b * p.q_batch_stride;
#pragma unroll
    for (int i = 0; i < kKSteps; ++i) {
      const int d0 = (i >> 1) * 32 + 8 * t + 4 * (i & 1);
      uint2 lo = make_uint2(0u, 0u), hi = make_uint2(0u, 0u);
      if (g < nheads) lo = *reinterpret_cast<const uint2*>(qb + (head0 + g) * p.q_head_stride + d0);
      if (kHi && g + 8 < nheads) hi = *reinterpret_cast<const uint2*>(qb + (head0 + g + 8) * p.q_head_stride + d0);
      qa[i][0] = lo.x;  // row g,   k 2t..2t+1
      qa[i][1] = hi.x;  // row g+8, k 2t..2t+1
      qa[i][2] = lo.y;  // row g,   k 2t+8..2t+9
      qa[i][3] = hi.y;  // row g+8, k 2t+8..2t+9
    }
  }

  const uint16_t* kbase = p.k + b * p.k_batch_stride + hkv * p.k_head_stride;
  const uint16_t* vbase = p.v + b * p.v_batch_stride + hkv * p.v_head_stride;
  const int last_key = p.len_k - 1;

  float o[kNBlocks][4];
#pragma unroll
  for (int nb = 0; nb < kNBlocks; ++nb) o[nb][0] = o[nb][1] = o[nb][2] = o[nb][3] = 0.f;
  float m_lo = -INFINITY, m_hi = kHi ? -INFINITY : 0.f;  // running max (log2 domain) of rows g and g+8
  float l_lo = 0.f, l_hi = 0.f;              // this thread's share of the running sums
  const float c = p.scale_log2;

  uint4 kbuf[2][kLoads];
  auto load_k = [&](int key0) {
#pragma unroll
    for (int blk = 0; blk < 2; ++blk) {
      const int key = min(key0 + blk * 8 + g, last_key);
      const uint16_t* row = kbase + static_cast<int64_t>(key) * p.k_row_stride + 8 * t;
#pragma unroll
      for (int l4 = 0; l4 < kLoads; ++l4) kbuf[blk][l4] = ld_stream_16(row + l4 * 32);
    }
  };

  int key0 = k_begin + warp * kKeysPerStep;
  if (key0 < k_end) load_k(key0);
  for (; key0 < k_end; key0 += kDecWarps * kKeysPerStep) {
    // ---- V rows of this step: keys 2t, 2t+1, 2t+8, 2t+9 at d = half*64 + 8g .. +7
    uint4 vbuf[kHalves][4];
    {
      const int r0 = key0 + 2 * t;
#pragma unroll
      for (int half = 0; half < kHalves; ++half) {
        const uint16_t* col = vbase + half * 64 + 8 * g;
        vbuf[half][0] = ld_stream_16(col + static_cast<int64_t>(min(r0, last_key)) * p.v_row_stride);
        vbuf[half][1] = ld_stream_16(col + static_cast<int64_t>(min(r0 + 1, last_key)) * p.v_row_stride);
        vbuf[half][2] = ld_stream_16(col + static_cast<int64_t>(min(r0 + 8, last_key)) * p.v_row_stride);
        vbuf[half][3] = ld_stream_16(col + static_cast<int64_t>(min(r0 + 9, last_key)) * p.v_row_stride);
      }
    }
    // ---- S = Q K^T for two blocks of 8 keys
    float s[2][4];
#pragma unroll
    for (int blk = 0; blk < 2; ++blk) {
      s[blk][0] = s[blk][1] = s[blk][2] = s[blk][3] = 0.f;
#pragma unroll
      for (int l4 = 0; l4 < kLoads; ++l4) {
        const uint4 w = kbuf[blk][l4];
        mma_rows<kHi, kF16>(s[blk], qa[2 * l4], w.x, w.y);
        mma_rows<kHi, kF16>(s[blk], qa[2 * l4 + 1], w.z, w.w);
      }
    }
    const int next = key0 + kDecWarps * kKeysPerStep;
    if (next < k_end) load_k(next);

    // ---- mask the tail, online softmax (thread holds keys key0 + blk*8 + 2t + {0,1})
#pragma unroll
    for (int blk = 0; blk < 2; ++blk) {
      const int kk = key0 + blk * 8 + 2 * t;
      if (kk >= k_end) { s[blk][0] = -INFINITY; s[blk][2] = -INFINITY; }
      if (kk + 1 >= k_end) { s[blk][1] = -INFINITY; s[blk][3] = -INFINITY; }
    }
    const float mx_lo = quad_max(fmaxf(fmaxf(s[0][0], s[0][1]), fmaxf(s[1][0], s[1][1]))) * c;
    const float mx_hi = kHi ? quad_max(fmaxf(fmaxf(s[0][2], s[0][3]), fmaxf(s[1][2], s[1][3]))) * c : 0.f;
    const float mn_lo = fmaxf(m_lo, mx_lo);
    const float mn_hi = fmaxf(m_hi, mx_hi);
    if (__any_sync(0xffffffffu, (mn_lo > m_lo) || (mn_hi > m_hi))) {
      // every key0 < k_end step has at least one visible key, so mn_* is finite here
      const float a_lo = ex2_approx(m_lo - mn_lo);
      const float a_hi = ex2_approx(m_hi - mn_hi);
      l_lo *= a_lo;
      l_hi *= a_hi;
#pragma unroll
      for (int nb = 0; nb < kNBlocks; ++nb) {
        o[nb][0] *= a_lo;
        o[nb][1] *= a_lo;
        if (kHi) {
          o[nb][2] *= a_hi;
          o[nb][3] *= a_hi;
        }
      }
      m_lo = mn_lo;
      m_hi = mn_hi;
    }
    float pr[2][4];
#pragma unroll
    for (int blk = 0; blk < 2; ++blk) {
      pr[blk][0] = ex2_approx(fmaf(s[blk][0], c, -m_lo));
      pr[blk][1] = ex2_approx(fmaf(s[blk][1], c, -m_lo));
      pr[blk][2] = kHi ? ex2_approx(fmaf(s[blk][2], c, -m_hi)) : 0.f;
      pr[blk][3] = kHi ? ex2_approx(fmaf(s[blk][3], c, -m_hi)) : 0.f;
      l_lo += pr[blk][0] + pr[blk][1];
      l_hi += pr[blk][2] + pr[blk][3];
    }
    const uint32_t pa0 = pack_16x2<kF16>(pr[0][0], pr[0][1]);  // row g,   keys 2t, 2t+1
    const uint32_t pa1 = pack_16x2<kF16>(pr[0][2], pr[0][3]);  // row g+8
    const uint32_t pa2 = pack_16x2<kF16>(pr[1][0], pr[1][1]);  // row g,   keys 8+2t, 9+2t
    const uint32_t pa3 = pack_16x2<kF16>(pr[1][2], pr[1][3]);  // row g+8

    // ---- O += P V. n-block (half, q) covers d = half*64 + 8*n + q for fragment column n.
#pragma unroll
    for (int half = 0; half < kHalves; ++half) {
      const uint32_t x0[4] = {vbuf[half][0].x, vbuf[half][0].y, vbuf[half][0].z, vbuf[half][0].w};
      const uint32_t x1[4] = {vbuf[half][1].x, vbuf[half][1].y, vbuf[half][1].z, vbuf[half][1].w};
      const uint32_t x2[4] = {vbuf[half][2].x, vbuf[half][2].y, vbuf[half][2].z, vbuf[half][2].w};
      const uint32_t x3[4] = {vbuf[half][3].x, vbuf[half][3].y, vbuf[half][3].z, vbuf[half][3].w};
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        const uint32_t sel = (q & 1) ? 0x7632u : 0x5410u;
        const uint32_t b0 = __byte_perm(x0[q >> 1], x1[q >> 1], sel);
        const uint32_t b1 = __byte_perm(x2[q >> 1], x3[q >> 1], sel);
        const uint32_t pa[4] = {pa0, pa1, pa2, pa3};
        mma_rows<kHi, kF16>(o[half * 8 + q], pa, b0, b1);
      }
    }
  }

  // ---- merge the 4 warps. Fragment column n = 2t + e of n-block (half, q) is
  //      d = half*64 + 8*(2t+e) + q.
  l_lo = quad_sum(l_lo);
  l_hi = quad_sum(l_hi);
  if (t == 0) {
    sm.m[warp][g] = m_lo;
    sm.m[warp][g + 8] = m_hi;
    sm.l[warp][g] = l_lo;
    sm.l[warp][g + 8] = l_hi;
  }
#pragma unroll
  for (int half = 0; half < kHalves; ++half) {
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      const int nb = half * 8 + q;
      const int d = half * 64 + 16 * t + q;
      sm.o[warp][g][d] = o[nb][0];
      sm.o[warp][g][d + 8] = o[nb][1];
      if (kHi) {
        sm.o[warp][g + 8][d] = o[nb][2];
        sm.o[warp][g + 8][d + 8] = o[nb][3];
      }
    }
  }
  __syncthreads();

  const int d = threadIdx.x;  // thread <-> output column (threads beyond head_dim idle)
  for (int r = 0; d < kD && r < nheads; ++r) {
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < kDecWarps; ++w) mm = fmaxf(mm, sm.m[w][r]);
    float ll = 0.f, acc = 0.f;
#pragma unroll
    for (int w = 0; w < kDecWarps; ++w) {
      const float mw = sm.m[w][r];
      const float sc = (mw == -INFINITY) ? 0.f : ex2_approx(mw - mm);
      ll += sm.l[w][r] * sc;
      acc += sm.o[w][r][d] * sc;
    }
    const int hq = head0 + r;
    const float inv = (ll > 0.f) ? 1.f / ll : 0.f;
    const float lse2 = (ll > 0.f) ? mm + log2f(ll) : -INFINITY;
    if (p.num_splits == 1) {
      p.out[b * p.o_batch_stride + hq * p.o_head_stride + d] = to_16<kF16>(acc * inv);
      if (d == 0)
        p.lse[static_cast<int64_t>(b) * p.heads_q + hq] = (ll > 0.f) ? lse2 * 0.6931471805599453f : INFINITY;
    } else {
      const int64_t slot = (static_cast<int64_t>(b) * p.heads_q + hq) * p.num_splits + split;
      p.part_o[slot * kD + d] = acc * inv;
      if (d == 0) p.part_lse[slot] = lse2;
    }
  }
}

// One warp per (batch, query head): merge the per-split partials.
__global__ void __launch_bounds__(128) decode_combine_kernel(const DecodeParams p, int rows) {
  const int kD = p.head_dim;
  const int warp_global = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp_global >= rows) return;
  const int b = warp_global / p.heads_q;
  const int hq = warp_global % p.heads_q;
  const float* pl = p.part_lse + static_cast<int64_t>(warp_global) * p.num_splits;
  const float* po = p.part_o + static_cast<int64_t>(warp_global) * p.num_splits * kD;

  // lane-strided pass over the split lse values, then a shuffle tree
  float mx = -INFINITY;
  for (int s = lane; s < p.num_splits; s += 32) mx = fmaxf(mx, pl[s]);
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
  float sum = 0.f;
  for (int s = lane; s < p.num_splits; s += 32) {
    const float v = pl[s];
    sum += (v == -INFINITY) ? 0.f : exp2f(v - mx);
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);

  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  const float inv = (sum > 0.f) ? 1.f / sum : 0.f;
  const bool active = lane * 4 < kD;
  for (int s = 0; active && s < p.num_splits; ++s) {
    const float v = pl[s];
    const float w = (v == -INFINITY) ? 0.f : exp2f(v - mx) * inv;
    const float4 x = *reinterpret_cast<const float4*>(po + static_cast<int64_t>(s) * kD + lane * 4);
    acc.x += w * x.x;
    acc.y += w * x.y;
    acc.z += w * x.z;
    acc.w += w * x.w;
  }
  if (active) {
    uint16_t* dst = p.out + b * p.o_batch_stride + hq * p.o_head_stride + lane * 4;
    const uint2 packed = p.f16 ? make_uint2(pack_f16x2(acc.x, acc.y), pack_f16x2(acc.z, acc.w))
                               : make_uint2(pack_bf16x2(acc.x, acc.y), pack_bf16x2(acc.z, acc.w));
    *reinterpret_cast<uint2*>(dst) = packed;
  }
  if (lane == 0)
    p.lse[warp_global] = (sum > 0.f) ? (mx + log2f(sum)) * 0.6931471805599453f : INFINITY;
}

template <int kD, bool kF16>
void launch_decode_kernel_t(const DecodeParams& d, dim3 grid, cudaStream_t stream) {
  if (d.group > 8) decode_splitkv_kernel<true, kD, kF16><<<grid, kDecThreads, 0, stream>>>(d);
  else decode_splitkv_kernel<false, kD, kF16><<<grid, kDecThreads, 0, stream>>>(d);
}

void launch_decode_kernel(const DecodeParams& d, dim3 grid, cudaStream_t stream) {
  if (d.head_dim == 64) {
    if (d.f16) launch_decode_kernel_t<64, true>(d, grid, stream);
    else launch_decode_kernel_t<64, false>(d, grid, stream);
  } else {
    if (d.f16) launch_decode_kernel_t<128, true>(d, grid, stream);
    else launch_decode_kernel_t<128, false>(d, grid, stream);
  }
}

int choose_splits(const sdpa_b200_params& p) {
  if (p.num_splits > 0) return p.num_splits > kMaxSplits ? kMaxSplits : p.num_splits;
  const int group = p.heads_q / p.heads_kv;
  const int chunks = (group + 15) / 16;
  const long units = static_cast<long>(p.batch) * p.heads_kv * chunks;
  // about 2048 keys per split, but enough CTAs for several waves of 148 SMs x 3 CTAs
  int splits = (p.max_seqlen_k + 2047) / 2048;
  const long want = 4L * 148 * 3;
  while (units * splits < want && p.max_seqlen_k / (splits * 2) >= 256) splits *= 2;
  if (splits < 1) splits = 1;
  if (splits > kMaxSplits) splits = kMaxSplits;
  return splits;
}

}  // namespace

size_t decode_workspace_bytes(const sdpa_b200_params& p, int* num_splits_out) {
  const int splits = choose_splits(p);
  if (num_splits_out) *num_splits_out = splits;
  if (splits == 1) return 0;
  const size_t rows = static_cast<size_t>(p.batch) * p.heads_q * splits;
  return rows * sizeof(float) * (p.head_dim + 1) + 256;
}

namespace {

// Kernel arguments for one decode call; the split partials go to part_o / part_lse
// (rows = batch * heads_q * splits slots of head_dim and of one float).
DecodeParams fill_decode_params(const sdpa_b200_params& p, int splits, float* part_o, float* part_lse) {
  DecodeParams d;
  d.q = static_cast<const uint16_t*>(p.q);
  d.k = static_cast<const uint16_t*>(p.k);
  d.v = static_cast<const uint16_t*>(p.v);
  d.out = static_cast<uint16_t*>(p.out);
  d.lse = p.lse;
  d.part_o = part_o;
  d.part_lse = part_lse;
  d.q_batch_stride = p.q_batch_stride;
  d.q_head_stride = p.q_head_stride;
  d.k_batch_stride = p.k_batch_stride;
  d.k_head_stride = p.k_head_stride;
  d.k_row_stride = p.k_row_stride;
  d.v_batch_stride = p.v_batch_stride;
  d.v_head_stride = p.v_head_stride;
  d.v_row_stride = p.v_row_stride;
  d.o_batch_stride = p.o_batch_stride;
  d.o_head_stride = p.o_head_stride;
  d.heads_q = p.heads_q;
  d.heads_kv = p.heads_kv;
  d.group = p.heads_q / p.heads_kv;
  d.chunks = (d.group + 15) / 16;
  d.len_k = p.max_seqlen_k;
  d.num_splits = splits;
  d.head_dim = p.head_dim;
  const int kps = (p.max_seqlen_k + splits - 1) / splits;
  d.keys_per_split = ((kps + 63) / 64) * 64;  // whole 4-warp steps
  d.scale_log2 = p.softmax_scale * 1.4426950408889634f;
  d.f16 = p.dtype == SDPA_B200_F16;
  return d;
}

// The split kernel and, with more than one split, the merge kernel.
int launch_decode_pair(const DecodeParams& d, int batch, const char* who, cudaStream_t stream) {
  dim3 grid(d.num_splits, d.heads_kv * d.chunks, batch);
  launch_decode_kernel(d, grid, stream);
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) {
    set_error("%s: launch failed: %s", who, cudaGetErrorString(err));
    return SDPA_B200_LAUNCH_FAILED;
  }
  count_launch();
  if (d.num_splits > 1) {
    const int nrows = batch * d.heads_q;
    decode_combine_kernel<<<(nrows + 3) / 4, 128, 0, stream>>>(d, nrows);
    err = cudaGetLastError();
    if (err != cudaSuccess) {
      set_error("%s merge: launch failed: %s", who, cudaGetErrorString(err));
      return SDPA_B200_LAUNCH_FAILED;
    }
    count_launch();
  }
  return SDPA_B200_OK;
}

}  // namespace

// What the streaming kernels cannot do; shared by every entry point that launches them.
int check_decode_request(const sdpa_b200_params& p) {
  if (p.cu_seqlens_q != nullptr || p.cu_seqlens_k != nullptr) {
    set_error("the decode kernel takes dense tensors only");
    return SDPA_B200_UNSUPPORTED;
  }
  if (p.max_seqlen_q != 1) {
    set_error("decode kernel needs seqlen_q == 1 (got %d)", p.max_seqlen_q);
    return SDPA_B200_UNSUPPORTED;
  }
  if (p.head_dim != 64 && p.head_dim != 128) {
    set_error("the decode kernel is built for head_dim 64 and 128 only (got %d)", p.head_dim);
    return SDPA_B200_UNSUPPORTED;
  }
  if (p.dropout_p != 0.f || p.keep_rows != nullptr || p.keep_cols != nullptr) {
    set_error("the decode kernel has no dropout");
    return SDPA_B200_UNSUPPORTED;
  }
  if (p.bias != nullptr) {
    set_error("the decode kernel takes no additive bias");
    return SDPA_B200_UNSUPPORTED;
  }
  return SDPA_B200_OK;
}

int launch_fwd_decode(const sdpa_b200_params& p, void* workspace, size_t workspace_bytes,
                      cudaStream_t stream) {
  int st = check_decode_request(p);
  if (st != SDPA_B200_OK) return st;
  int splits = 1;
  const size_t need = decode_workspace_bytes(p, &splits);
  if (workspace_bytes < kWorkspaceHeaderBytes + need) {
    set_error("decode workspace too small: %zu < %zu", workspace_bytes, kWorkspaceHeaderBytes + need);
    return SDPA_B200_INVALID_ARG;
  }
  const size_t rows = static_cast<size_t>(p.batch) * p.heads_q * splits;
  float* ws = reinterpret_cast<float*>(static_cast<char*>(workspace) + kWorkspaceHeaderBytes);
  const DecodeParams d = fill_decode_params(p, splits, ws, ws + rows * p.head_dim);
  return launch_decode_pair(d, p.batch, "decode", stream);
}

}  // namespace sdpa_b200

// ---------------------------------------------------------------------------------------
// Decode without any caller- or library-allocated scratch memory.
//
// Some callers may not allocate device memory at the point where they need attention: code
// running inside a memory-pool callback or an allocator hook, a serving loop whose memory plan
// was frozen at start-up, or a process that has handed the whole device to another allocator.
// For them the split-KV partials live in a fixed array that is part of this library's image;
// every GPU that loads the library carries those SDPA_B200_STATIC_SCRATCH_BYTES until exit.
//
// The array name below is only a host-side handle: in host code it is not a device address and
// must never be handed to a kernel. The real address is asked from the runtime with
// cudaGetSymbolAddress, once per device, with that device current, on the first call made on
// that device (so make that first call outside any stream capture). Nothing is allocated or
// freed here, and no library routine that allocates is called.
//
// All calls on a device share the one array and it keeps whatever the previous call left in
// it. That is harmless for this kernel pair - every (row, split) slot the merge kernel reads is
// written by the split kernel of the same call first, so nothing has to start at zero - but two
// calls whose kernels overlap on the GPU (different streams, no ordering) race on it.
// ---------------------------------------------------------------------------------------
namespace sdpa_b200 {
namespace {

static __device__ __align__(256) unsigned char g_decode_static_scratch[SDPA_B200_STATIC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
void* g_static_scratch_ptr[kMaxDevices] = {};
std::mutex g_static_scratch_mutex;

// Device address of the static array on the current device (looked up once per device).
int static_scratch_address(void** out) {
  int dev = -1;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    (void)cudaGetLastError();
    set_error("decode_static: cannot identify the current device");
    return SDPA_B200_NO_DEVICE;
  }
  std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
  if (g_static_scratch_ptr[dev] == nullptr) {
    void* ptr = nullptr;
    err = cudaGetSymbolAddress(&ptr, g_decode_static_scratch);
    if (err != cudaSuccess || ptr == nullptr) {
      (void)cudaGetLastError();
      set_error("decode_static: cudaGetSymbolAddress failed on device %d: %s", dev, cudaGetErrorString(err));
      return SDPA_B200_LAUNCH_FAILED;
    }
    g_static_scratch_ptr[dev] = ptr;
  }
  *out = g_static_scratch_ptr[dev];
  return SDPA_B200_OK;
}

}  // namespace
}  // namespace sdpa_b200

extern "C" SDPA_B200_API int sdpa_b200_decode_static(const sdpa_b200_params* p, void* stream) {
  using namespace sdpa_b200;
  // argument checks first, the device last: a refused request never needs a GPU
  int st = validate_forward_args(p);
  if (st != SDPA_B200_OK) return st;
  if (p->kernel == SDPA_B200_KERNEL_PREFILL) {
    set_error("decode_static runs the split-KV decode kernel only (kernel must be AUTO or DECODE)");
    return SDPA_B200_UNSUPPORTED;
  }
  st = check_decode_request(*p);
  if (st != SDPA_B200_OK) return st;
  const int splits = choose_splits(*p);
  const size_t rows = static_cast<size_t>(p->batch) * p->heads_q * splits;
  const size_t need = rows * sizeof(float) * (p->head_dim + 1);
  if (need > SDPA_B200_STATIC_SCRATCH_BYTES) {
    set_error("decode_static: batch %d x heads_q %d x %d splits needs %zu bytes of split partials, more than the "
              "%u bytes built into the library; lower num_splits or use sdpa_b200_fwd with a workspace",
              p->batch, p->heads_q, splits, need, static_cast<unsigned>(SDPA_B200_STATIC_SCRATCH_BYTES));
    return SDPA_B200_INVALID_ARG;
  }
  st = check_device();
  if (st != SDPA_B200_OK) return st;
  void* scratch = nullptr;
  st = static_scratch_address(&scratch);
  if (st != SDPA_B200_OK) return st;
  float* part_o = static_cast<float*>(scratch);
  const DecodeParams d = fill_decode_params(*p, splits, part_o, part_o + rows * p->head_dim);
  return launch_decode_pair(d, p->batch, "decode_static", static_cast<cudaStream_t>(stream));
}
