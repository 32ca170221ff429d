// Attention kernels for head dims above 128 (up to 256) on sm_100a.
//
// The reference admits 64 <= head_dim <= 256 (sdp_utils.h:231-255, FlashAttention_internal.cpp:119-121) and its value
// tests run 256 (test/torch_ops/test_scaled_dot_product_attention.py:728-1285). The 128-column tile kernels do not
// stretch to that: two 128 x 256 operands of one score GEMM alone fill half the shared memory, and a 128 x 256 fp32
// accumulator half the tensor memory. The kernels here turn the layout around:
//   * the stationary operand of a CTA - 128 rows of Q (forward), or of K / V / dO / Q (backward) - lives in TENSOR
//     memory as the A operand of every GEMM (its threads load their own rows once from global memory: a 256-element
//     16-bit row is 128 TMEM columns), so shared memory holds nothing but the stream;
//   * the other side streams through a ring of seven 32 KB slots in blocks of 64 rows x 256 columns (four TMA boxes of
//     64 columns, 128-byte swizzle), read K-major (contraction over head_dim) or MN-major (contraction over the 64
//     rows) without a transpose;
//   * scores are 128 x 64 blocks (N = 64 MMAs with the A operand in TMEM cost 32 cycles: tensor-bound, not bound by
//     shared-memory reads), double-buffered where tensor memory allows.
// Head dims between 128 and 256 run here with zero padding (TMA fills the missing columns, stores are clipped).
//
// Forward (fwd_d256_kernel): one CTA per (batch, head, 128 query rows). TMEM: Q [0,128) S0 [128,192) S1 [192,256)
// O [256,512). Per 64-key block j: S[j&1] = Q K_j^T (16 MMAs), online softmax by four warps (thread = query row) in
// the log2 domain, P (16-bit) over the front of S[j&1], O += P V_j (4 MMAs of N = 256). The issuer runs QK(j+2)
// behind PV(j), so the next block's scores are formed while this block is exponentiated.
#include <cuda_bf16.h>

#include "kernels.h"
#include "ptx_sm100.cuh"

namespace sdpa_b200 {
namespace {

constexpr int kRowsA = 128;                 // stationary rows per CTA
constexpr int kRowsB = 64;                  // streamed rows per block
constexpr int kWide = 256;                  // columns every tile is padded to
constexpr uint32_t kSlotBytes = 32768;      // one streamed block: 64 rows x 256 columns x 2 bytes
constexpr uint32_t kBoxBytes = 8192;        // one TMA box: 64 rows x 64 columns
constexpr int kSlots = 7;
constexpr uint32_t kSmemRing = 0;
constexpr uint32_t kSmemBars = kSlots * kSlotBytes;
constexpr uint32_t kSmemBytesD256 = kSmemBars + 512 + 1024;  // barriers, then slack for the 1024-byte alignment
constexpr float kRescaleLog2 = 8.0f;        // O is rescaled only when a row maximum grows by more than 2^8

// barrier offsets (bytes from kSmemBars)
constexpr uint32_t kBFull = 0;                    // kSlots
constexpr uint32_t kBEmpty = kBFull + 8 * kSlots; // kSlots
constexpr uint32_t kBAReady = kBEmpty + 8 * kSlots;  // 4: the stationary rows are in TMEM
constexpr uint32_t kBSFull = kBAReady + 8;        // 2
constexpr uint32_t kBPFull = kBSFull + 16;        // 2 x 4 warps
constexpr uint32_t kBODone = kBPFull + 16;        // PV(j) has finished
constexpr uint32_t kBStage = kBODone + 8;         // 4: the output rows are staged
constexpr uint32_t kTmemPtr = kBStage + 8;
constexpr uint32_t kAbortWord = kTmemPtr + 4;

struct D256Params {
  const uint16_t* q;
  uint16_t* out;
  float* lse;
  const int32_t* cu_q;
  const int32_t* cu_k;
  uint32_t* status;
  int64_t q_batch_stride, q_head_stride, q_row_stride;
  int64_t o_batch_stride, o_head_stride, o_row_stride;
  int seqlen_q, seqlen_k, total_q, heads_q, kv_group, head_dim;
  int num_m_blocks, num_bh, heads_per_wave;
  float scale_log2;
  int is_causal;
  // dropout (kernels built with kDrop): one keep bit per (query, key) pair, see dropout_mask.cu
  const uint32_t* keep_rows;  // dense [batch*heads_q][keep_rows_per][lk_words]; packed [heads_q][total_q + 128][lk_words]
  int keep_rows_per, lk_words;
  float keep_scale;           // 1 / (1 - dropout_p)
};

// both halves of a packed 16-bit pair survive or die by two keep bits (bit 0 -> low half)
__device__ __forceinline__ uint32_t keep_pair(uint32_t two_bits) {
  return ((two_bits & 1u) ? 0x0000ffffu : 0u) | ((two_bits & 2u) ? 0xffff0000u : 0u);
}

template <bool kF16>
constexpr uint32_t kIdescS64 = umma_idesc_16(kRowsA, kRowsB, false, false, kF16);   // scores: N = 64, B K-major
template <bool kF16>
constexpr uint32_t kIdescAcc256 = umma_idesc_16(kRowsA, kWide, false, true, kF16);  // accumulation: N = 256, B MN-major

// S (128 x 64) = A (TMEM, 128 rows x 256) * B^T, B = one streamed block read K-major: 16 steps of 16 columns
template <bool kF16>
__device__ __forceinline__ void issue_scores(uint32_t t_s, uint32_t a_tmem, uint32_t slot) {
#pragma unroll
  for (int ks = 0; ks < kWide / 16; ++ks) {
    const uint32_t b_lo = umma_desc_lo_kmajor(slot + (ks >> 2) * kBoxBytes + (ks & 3) * 32);
    umma_ts_lo<kIdescS64<kF16>>(t_s, a_tmem + ks * 8, b_lo, ks > 0 ? 1u : 0u);
  }
}

// ACC (128 x 256) (+)= W (TMEM, 128 x 64, 16-bit) * B, B = one streamed block read MN-major: 4 steps of 16 rows
template <bool kF16>
__device__ __forceinline__ void issue_accumulate256(uint32_t acc, uint32_t w_tmem, uint32_t slot, bool accumulate) {
#pragma unroll
  for (int ks = 0; ks < kRowsB / 16; ++ks) {
    const uint32_t b_lo = umma_desc_lo_mnmajor(slot + ks * 2048, kBoxBytes);
    umma_ts_lo<kIdescAcc256<kF16>>(acc, w_tmem + ks * 8, b_lo, (accumulate || ks > 0) ? 1u : 0u);
  }
}

// One thread's row of a [rows, head_dim] 16-bit matrix into its TMEM lane as 128 columns (two elements per column),
// zero beyond head_dim or when the row does not exist. Four stores of 32 columns; the caller waits for them.
__device__ __forceinline__ void row_to_tmem(uint32_t taddr, const uint16_t* row, int head_dim) {
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    uint32_t w[32];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      uint4 x = make_uint4(0u, 0u, 0u, 0u);
      const int col = c * 64 + i * 8;
      if (row != nullptr && col < head_dim) x = *reinterpret_cast<const uint4*>(row + col);
      w[4 * i] = x.x;
      w[4 * i + 1] = x.y;
      w[4 * i + 2] = x.z;
      w[4 * i + 3] = x.w;
    }
    tmem_st_x32(taddr + c * 32, w);
  }
}

template <bool kF16, bool kDrop>
__global__ void __launch_bounds__(192, 1)
fwd_d256_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                const __grid_constant__ CUtensorMap tm_o, const D256Params p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw_addr);
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // CTA order: (batch, head) pairs in groups of `heads_per_wave` whose K/V fit L2 together; inside a group the 128-row
  // blocks go heaviest first (with a causal mask the last block sees the most keys) across all its heads.
  int b, h, mb;
  {
    const int per_group = p.heads_per_wave * p.num_m_blocks;
    const int grp = blockIdx.x / per_group;
    const int w = blockIdx.x - grp * per_group;
    const int size = min(p.heads_per_wave, p.num_bh - grp * p.heads_per_wave);
    const int rank = w / size;
    const int bh = grp * p.heads_per_wave + (w - rank * size);
    if (rank >= p.num_m_blocks) return;  // padding slots of a short last group
    mb = p.num_m_blocks - 1 - rank;
    b = bh / p.heads_q;
    h = bh - b * p.heads_q;
  }
  int q_off = 0, k_off = 0, len_q = p.seqlen_q, len_k = p.seqlen_k, bcoord = b;
  if (p.cu_q != nullptr) {
    q_off = p.cu_q[b];
    len_q = p.cu_q[b + 1] - q_off;
    k_off = p.cu_k[b];
    len_k = p.cu_k[b + 1] - k_off;
    bcoord = 0;
  }
  const int m0 = mb * kRowsA;
  if (m0 >= len_q) return;
  const int hk = h / p.kv_group;
  const int causal_off = len_k - len_q;
  // keys visible to the tile's last row bound the block count
  int vis_end = len_k;
  if (p.is_causal) vis_end = min(len_k, m0 + kRowsA + causal_off);
  const int n_blocks = vis_end > 0 ? (vis_end + kRowsB - 1) / kRowsB : 0;

  const uint32_t bar = base + kSmemBars;
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(smem + kSmemBars + kAbortWord);
  volatile uint32_t* tmem_ptr_smem = reinterpret_cast<volatile uint32_t*>(smem + kSmemBars + kTmemPtr);

  if (warp == 4 && lane == 0) {
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_v);
    for (int s = 0; s < kSlots; ++s) {
      mbar_init(bar + kBFull + 8 * s, 1);
      mbar_init(bar + kBEmpty + 8 * s, 1);
    }
    mbar_init(bar + kBAReady, 4);
    mbar_init(bar + kBSFull, 1);
    mbar_init(bar + kBSFull + 8, 1);
    mbar_init(bar + kBPFull, 4);
    mbar_init(bar + kBPFull + 8, 4);
    mbar_init(bar + kBODone, 1);
    mbar_init(bar + kBStage, 4);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 0) {
    __syncwarp();
    tmem_alloc(base + kSmemBars + kTmemPtr, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_ptr_smem;
  const uint32_t t_q = tmem_base, t_s0 = tmem_base + 128, t_o = tmem_base + 256;

  if (warp == 4) {
    // ------------------------------------------------------------------ TMA producer: K(0) V(0) K(1) V(1) ...
    if (lane == 0) {
      for (int t = 0; t < 2 * n_blocks; ++t) {
        const int s = t % kSlots;
        const uint32_t lap = static_cast<uint32_t>(t / kSlots);
        if (!mbar_wait(bar + kBEmpty + 8 * s, (lap & 1u) ^ 1u, abort_flag)) break;
        const CUtensorMap* tm = (t & 1) ? &tm_v : &tm_k;
        const uint32_t full = bar + kBFull + 8 * s;
        const uint32_t dst = base + kSmemRing + s * kSlotBytes;
        const int row = k_off + (t >> 1) * kRowsB;
        mbar_arrive_expect_tx(full, kSlotBytes);
#pragma unroll
        for (int c = 0; c < 4; ++c) tma_load_4d(dst + c * kBoxBytes, tm, full, c * 64, row, hk, bcoord);
      }
      drain_after_abort(abort_flag);
    }
  } else if (warp == 5) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0 && n_blocks > 0) {
      auto slot_of = [&](int t) { return base + kSmemRing + (t % kSlots) * kSlotBytes; };
      auto wait_full = [&](int t) { return mbar_wait(bar + kBFull + 8 * (t % kSlots), (t / kSlots) & 1, abort_flag); };
      auto issue_qk = [&](int j) {
        tc_fence_after_sync();
        issue_scores<kF16>(t_s0 + (j & 1) * 64, t_q, slot_of(2 * j));
        umma_commit(bar + kBSFull + 8 * (j & 1));
        umma_commit(bar + kBEmpty + 8 * ((2 * j) % kSlots));  // the K block may be overwritten
      };
      bool ok = mbar_wait(bar + kBAReady, 0, abort_flag) && wait_full(0);
      if (ok) issue_qk(0);
      if (ok && n_blocks > 1) {
        ok = wait_full(2);
        if (ok) issue_qk(1);
      }
      for (int j = 0; ok && j < n_blocks; ++j) {
        ok = mbar_wait(bar + kBPFull + 8 * (j & 1), (j >> 1) & 1, abort_flag) && wait_full(2 * j + 1);
        if (!ok) break;
        tc_fence_after_sync();
        issue_accumulate256<kF16>(t_o, t_s0 + (j & 1) * 64, slot_of(2 * j + 1), j > 0);
        umma_commit(bar + kBODone);
        umma_commit(bar + kBEmpty + 8 * ((2 * j + 1) % kSlots));  // the V block may be overwritten
        if (j + 2 < n_blocks) {
          // S[j&1] is free: P(j) has been read by the MMAs just issued, and the pipe keeps this thread's order
          ok = wait_full(2 * j + 4);
          if (!ok) break;
          issue_qk(j + 2);
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax warps (thread = query row)
    const int r = warp * 32 + lane;
    const int row = m0 + r;
    const bool valid = row < len_q;
    const uint32_t lane_base = static_cast<uint32_t>(warp * 32) << 16;
    {
      const uint16_t* qrow = nullptr;
      if (valid)
        qrow = p.q + ((p.cu_q != nullptr) ? static_cast<int64_t>(q_off + row) * p.q_row_stride
                                          : b * p.q_batch_stride + static_cast<int64_t>(row) * p.q_row_stride) +
               h * p.q_head_stride;
      row_to_tmem(t_q + lane_base, qrow, p.head_dim);
      tmem_wait_st();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar + kBAReady);
    }
    const float c = p.scale_log2;
    const float neg_inf = -INFINITY;
    // keys at index >= col_limit are invisible to this row; blocks reaching past mask_from need the element mask
    const int col_limit = p.is_causal ? min(len_k, row + causal_off + 1) : len_k;
    const int mask_from = p.is_causal ? min(len_k, m0 + causal_off + 1) : len_k;
    float m_run = neg_inf, l_run = 0.f;
    bool ok = true;
    const uint32_t* keep_row = nullptr;  // this row's keep bits, 2 words per key block
    if constexpr (kDrop)
      keep_row = p.keep_rows + (p.cu_q != nullptr ? static_cast<size_t>(h) * p.keep_rows_per + q_off + row
                                                  : static_cast<size_t>(b * p.heads_q + h) * p.keep_rows_per + row) * p.lk_words;
    for (int j = 0; j < n_blocks; ++j) {
      const uint32_t t_s = t_s0 + (j & 1) * 64 + lane_base;
      uint2 keep = make_uint2(0u, 0u);
      if constexpr (kDrop) keep = *reinterpret_cast<const uint2*>(keep_row + 2 * j);  // in flight under the wait
      ok = __all_sync(0xffffffffu, mbar_wait(bar + kBSFull + 8 * (j & 1), (j >> 1) & 1, abort_flag));
      if (!ok) break;
      tc_fence_after_sync();
      float s[kRowsB];
      {
        uint32_t raw[kRowsB];
        tmem_ld_x64(t_s, raw);
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < kRowsB; ++i) s[i] = __uint_as_float(raw[i]);
      }
      const int n0 = j * kRowsB;
      if (n0 + kRowsB > mask_from) {
        const int lim = col_limit - n0;
#pragma unroll
        for (int i = 0; i < kRowsB; ++i) s[i] = (i < lim) ? s[i] : neg_inf;
      }
      float mx0 = neg_inf, mx1 = neg_inf;
#pragma unroll
      for (int i = 0; i < kRowsB; i += 4) {
        mx0 = max3(mx0, s[i], s[i + 1]);
        mx1 = max3(mx1, s[i + 2], s[i + 3]);
      }
      const float m_new = fmaxf(m_run, fmaxf(mx0, mx1) * c);
      bool pv_seen = (j == 0);  // has this thread observed the end of PV(j-1) yet?
      if (j == 0) {
        m_run = m_new;
      } else {
        const bool grow = (m_new - m_run) > kRescaleLog2;  // false for NaN (-inf - -inf)
        if (__any_sync(0xffffffffu, grow)) {
          const float alpha = (m_new == neg_inf) ? 1.f : ex2_approx(m_run - m_new);
          m_run = m_new;
          l_run *= alpha;
          // O still receives PV(j-1): wait for it before touching the accumulator
          ok = __all_sync(0xffffffffu, mbar_wait(bar + kBODone, (j - 1) & 1, abort_flag));
          if (!ok) break;
          pv_seen = true;
          tc_fence_after_sync();
#pragma unroll
          for (int cc = 0; cc < kWide / 32; ++cc) {
            uint32_t o[32];
            tmem_ld_x32(t_o + lane_base + cc * 32, o);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st_x32(t_o + lane_base + cc * 32, o);
          }
        }
      }
      const float neg_m = (m_run == neg_inf) ? 0.f : -m_run;
      const float2 c2 = make_float2(c, c), nm2 = make_float2(neg_m, neg_m);
      float2 la = make_float2(0.f, 0.f), lb = make_float2(0.f, 0.f);
      uint32_t pk[kRowsB / 2];
#pragma unroll
      for (int i = 0; i < kRowsB / 2; ++i) {
        const float2 x = fma2(make_float2(s[2 * i], s[2 * i + 1]), c2, nm2);
        const float2 pr = make_float2(ex2_approx(x.x), ex2_approx(x.y));
        if (i & 1) lb = add2(lb, pr); else la = add2(la, pr);
        pk[i] = pack_16x2<kF16>(pr.x, pr.y);
        // the row sum keeps every pair (softmax is normalised before dropout); only P V loses the dropped ones
        if constexpr (kDrop) pk[i] &= keep_pair((i < 16 ? keep.x : keep.y) >> ((2 * i) & 31));
      }
      l_run += (la.x + la.y) + (lb.x + lb.y);
      // Every phase of the PV barrier is observed, in order, and before this block's P is handed over (PV(j) cannot end
      // before that): a parity wait only tells "this phase is over" from "it is not" while the barrier is at most one
      // phase further on, and the epilogue's wait for the last PV relies on it. PV(j-1) ended long ago as a rule.
      if (!pv_seen) {
        ok = __all_sync(0xffffffffu, mbar_wait(bar + kBODone, (j - 1) & 1, abort_flag));
        if (!ok) break;
      }
      tmem_st_x32(t_s, pk);  // P over the front of S: 32 columns = 64 keys
      tmem_wait_st();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar + kBPFull + 8 * (j & 1));
    }

    // ---- epilogue: O / l -> 16 bit, logsumexp
    if (ok && n_blocks > 0) ok = __all_sync(0xffffffffu, mbar_wait(bar + kBODone, (n_blocks - 1) & 1, abort_flag));
    if (ok) {
      tc_fence_after_sync();
      float inv_l = (l_run > 0.f) ? 1.f / l_run : 0.f;
      if constexpr (kDrop) inv_l *= p.keep_scale;
      if (valid) {
        const size_t li = (p.cu_q != nullptr) ? static_cast<size_t>(h) * p.total_q + q_off + row
                                              : (static_cast<size_t>(b) * p.heads_q + h) * p.seqlen_q + row;
        p.lse[li] = (l_run > 0.f) ? (m_run + lg2_approx(l_run)) * 0.6931471805599453f : INFINITY;
      }
      // A whole tile leaves through shared memory (the ring is idle by now: 4 boxes of 128 rows x 64 columns) and TMA
      // stores; dense tensors are clipped by the tensor map. A packed tile that ends inside its sequence's last rows
      // would spill into the next sequence and is written row by row instead.
      const bool use_tma = (p.cu_q == nullptr) || (m0 + kRowsA <= len_q);
      uint16_t* orow = p.out + ((p.cu_q != nullptr) ? static_cast<int64_t>(q_off + row) * p.o_row_stride
                                                    : b * p.o_batch_stride + static_cast<int64_t>(row) * p.o_row_stride) +
                       h * p.o_head_stride;
#pragma unroll
      for (int cc = 0; cc < kWide / 32; ++cc) {
        uint32_t o[32];
        if (n_blocks > 0) {
          tmem_ld_x32(t_o + lane_base + cc * 32, o);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = 0u;
        }
        uint4 w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          w[i].x = pack_16x2<kF16>(__uint_as_float(o[8 * i]) * inv_l, __uint_as_float(o[8 * i + 1]) * inv_l);
          w[i].y = pack_16x2<kF16>(__uint_as_float(o[8 * i + 2]) * inv_l, __uint_as_float(o[8 * i + 3]) * inv_l);
          w[i].z = pack_16x2<kF16>(__uint_as_float(o[8 * i + 4]) * inv_l, __uint_as_float(o[8 * i + 5]) * inv_l);
          w[i].w = pack_16x2<kF16>(__uint_as_float(o[8 * i + 6]) * inv_l, __uint_as_float(o[8 * i + 7]) * inv_l);
        }
        const int col = cc * 32;
        if (use_tma) {
          // box (col / 64) of the staged tile: 128 rows of 128 bytes, 16-byte chunks XOR-swizzled by (row % 8)
          uint8_t* srow = smem + kSmemRing + (col >> 6) * (kRowsA * 128) + r * 128;
          const int chunk0 = (col & 63) >> 3;
#pragma unroll
          for (int i = 0; i < 4; ++i) *reinterpret_cast<uint4*>(srow + (((chunk0 + i) ^ (r & 7)) << 4)) = w[i];
        } else if (valid) {
#pragma unroll
          for (int i = 0; i < 4; ++i)
            if (col + 8 * i < p.head_dim) *reinterpret_cast<uint4*>(orow + col + 8 * i) = w[i];
        }
      }
      if (use_tma) {
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar + kBStage);
        if (threadIdx.x == 0) {
          if (mbar_wait(bar + kBStage, 0, abort_flag)) {
#pragma unroll
            for (int c4 = 0; c4 < 4; ++c4)
              tma_store_4d(&tm_o, base + kSmemRing + c4 * (kRowsA * 128), c4 * 64, q_off + m0, h, bcoord);
            tma_store_commit();
            tma_store_wait_read();
          }
        }
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
  if (threadIdx.x == 0 && *abort_flag != 0) atomicExch(p.status, static_cast<uint32_t>(SDPA_B200_DEVICE_TIMEOUT));
}

// ---------------------------------------------------------------------------------------------------------------
// Backward. Three kernels from one template, all with 128 stationary rows in tensor memory and 64-row streamed blocks:
//   kDV: CTA = 128 keys. X1 = K (TMEM). Streams (Q, dO) blocks of 64 queries of every query head of the KV head.
//        S^T = K Q^T; P^T = exp2(S^T c - lse2[q]); dV += P^T dO.                                TMEM: K | S0 S1 | dV
//   kDK: CTA = 128 keys. X1 = K (TMEM), X2 = V (shared memory, 64 KB). Streams (Q, dO).
//        S^T = K Q^T, dP^T = V dO^T; dS^T = P^T o (dP^T - delta[q]); dK += dS^T Q.               TMEM: K | TA TB | dK
//   kDQ: CTA = 128 queries. X1 = Q (TMEM), X2 = dO (shared memory). Streams (K, V) blocks of 64 keys.
//        S = Q K^T, dP = dO V^T; dS = P o (dP - delta[row]); dQ += dS K.                          TMEM: Q | TA TB | dQ
// A 128 x 256 fp32 accumulator is half the tensor memory, so every kernel owns exactly one; dK and dV therefore come from
// two kernels that both form S (9 GEMM-equivalents per tile pair against the 5 of the algorithm). The score GEMM with X2
// reads both operands from shared memory (N = 64: 48 cycles per MMA instead of 32).
// Score buffers rotate as in the 128-column kernels: S(i) in T[i&1], dP(i) in the other one; the 16-bit dS goes over the
// front of S(i); S(i+1) takes dP(i)'s buffer once the compute warps have read it, dP(i+1) follows the accumulation of
// item i in the issuer's own order.
// ---------------------------------------------------------------------------------------------------------------
constexpr int kDV = 0, kDK = 1, kDQ = 2;
// warps 0-3 / 4-7: two compute warpgroups, one per 32-row half of every streamed block (thread = stationary row);
// warp 8 TMA producer, warps 9 and 10 MMA issuers
constexpr int kBwdThreads = 352;

__host__ __device__ constexpr int ring_slots_for(int mode) { return mode == kDV ? 6 : (mode == kDK ? 4 : 5); }
__host__ __device__ constexpr uint32_t ring_base_for(int mode) { return mode == kDV ? 0u : 2u * kSlotBytes; }  // behind X2
// per ring slot: lse2[64], delta[64] of the streamed queries (kDV, kDK). Those two kernels use six of the seven 32 KB
// slots (kDV: ring of 6; kDK: V + ring of 4), so the vectors live at the start of the seventh.
constexpr uint32_t kSmemVecs = 6 * kSlotBytes;
constexpr uint32_t kSmemBytesBwd256 = kSmemBytesD256;
static_assert(ring_base_for(kDQ) + ring_slots_for(kDQ) * kSlotBytes <= kSmemBars && 6 * 512 <= kSlotBytes,
              "shared memory map does not fit");

// barrier offsets of the backward kernels (bytes from kSmemBars); kBFull / kBEmpty / kBAReady / kBStage as above
constexpr uint32_t kBX2Full = kBAReady + 8;
constexpr uint32_t kBTFull = kBX2Full + 8;     // 2: the score GEMM into T[b] has finished
constexpr uint32_t kBDFree = kBTFull + 16;     // 4 warps: dP has been read out of TMEM
constexpr uint32_t kBWFull = kBDFree + 8;      // 4 warps: the 16-bit P / dS is in TMEM
constexpr uint32_t kBWRead = kBWFull + 8;      // the accumulation GEMM of an item has read its P / dS
constexpr uint32_t kBAccFull = kBWRead + 8;
constexpr uint32_t kBStageB = kBAccFull + 8;   // 4 warps
constexpr uint32_t kTmemPtrB = kBStageB + 8;
constexpr uint32_t kAbortWordB = kTmemPtrB + 4;
static_assert(kAbortWordB + 4 <= 512, "barrier block too small");

struct Bwd256Params {
  const uint16_t* x1;        // rows kept in tensor memory: K (kDV, kDK) or Q (kDQ)
  uint16_t* out;             // dV, dK or dQ
  const float* lse2;         // padded [batch, heads_q, lq_pad]
  const float* delta;
  const int32_t* cu_q;
  const int32_t* cu_k;
  uint32_t* status;
  int64_t x1_batch_stride, x1_head_stride, x1_row_stride;
  int64_t o_batch_stride, o_head_stride, o_row_stride;
  int seqlen_q, seqlen_k, heads_q, heads_kv, kv_group, head_dim, lq_pad;
  int num_row_blocks, num_bh, heads_x, heads_per_wave;
  float scale, scale_log2;
  int is_causal;
  // dropout (kernels built with kDrop): P is recomputed without it; dV takes P o M / (1 - p), dS = P o (M o dP / (1 - p) - delta)
  const uint32_t* keep_rows;  // [batch*heads_q][keep_q_rows][keep_lk_pad / 32]: kDQ
  const uint32_t* keep_cols;  // [batch*heads_q][keep_k_rows][keep_lq_pad / 32]: kDV, kDK
  int keep_lq_pad, keep_lk_pad, keep_q_rows, keep_k_rows;
  float keep_scale;
};

template <bool kF16>
constexpr uint32_t kIdescS64SS = umma_idesc_16(kRowsA, kRowsB, false, false, kF16);

// ACC (128 x 256) (+)= W * B with W written by two warpgroups, each over the front of its own 32 score columns: the 16-bit
// rows 0-31 of the block sit in columns [0,16) of the buffer, rows 32-63 in columns [32,48)
template <bool kF16>
__device__ __forceinline__ void issue_accumulate256_split(uint32_t acc, uint32_t w_tmem, uint32_t slot, bool accumulate) {
#pragma unroll
  for (int ks = 0; ks < kRowsB / 16; ++ks) {
    const uint32_t b_lo = umma_desc_lo_mnmajor(slot + ks * 2048, kBoxBytes);
    umma_ts_lo<kIdescAcc256<kF16>>(acc, w_tmem + (ks >> 1) * 32 + (ks & 1) * 8, b_lo, (accumulate || ks > 0) ? 1u : 0u);
  }
}

// half of a row (128 of its 256 elements = 64 TMEM columns), for a loader split over two warpgroups
__device__ __forceinline__ void row_half_to_tmem(uint32_t taddr, const uint16_t* row, int head_dim, int half) {
#pragma unroll
  for (int c2 = 0; c2 < 2; ++c2) {
    const int c = half * 2 + c2;
    uint32_t w[32];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      uint4 x = make_uint4(0u, 0u, 0u, 0u);
      const int col = c * 64 + i * 8;
      if (row != nullptr && col < head_dim) x = *reinterpret_cast<const uint4*>(row + col);
      w[4 * i] = x.x;
      w[4 * i + 1] = x.y;
      w[4 * i + 2] = x.z;
      w[4 * i + 3] = x.w;
    }
    tmem_st_x32(taddr + c * 32, w);
  }
}

// T (128 x 64) = X2 (shared memory, 128 rows x 256 as four boxes of 64 columns) * Y^T, Y = one streamed block, both K-major
template <bool kF16>
__device__ __forceinline__ void issue_scores_ss(uint32_t t, uint32_t x2_smem, uint32_t slot) {
#pragma unroll
  for (int ks = 0; ks < kWide / 16; ++ks) {
    const uint32_t a_lo = umma_desc_lo_kmajor(x2_smem + (ks >> 2) * (kRowsA * 128) + (ks & 3) * 32);
    const uint32_t b_lo = umma_desc_lo_kmajor(slot + (ks >> 2) * kBoxBytes + (ks & 3) * 32);
    umma_ss_lo_acc<kIdescS64SS<kF16>>(t, a_lo, b_lo, ks > 0 ? 1u : 0u);
  }
}

template <int kMode, bool kF16, bool kDrop>
__global__ void __launch_bounds__(kBwdThreads, 1)
bwd_d256_kernel(const __grid_constant__ CUtensorMap tm_x2, const __grid_constant__ CUtensorMap tm_y1,
                const __grid_constant__ CUtensorMap tm_y2, const __grid_constant__ CUtensorMap tm_out,
                const Bwd256Params p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw_addr);
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  constexpr int kRing = ring_slots_for(kMode);
  constexpr uint32_t kRingBase = ring_base_for(kMode);
  constexpr bool kKeys = kMode != kDQ;  // the stationary rows are keys

  // CTA order as in the forward: groups of heads whose streamed tensors fit L2, heaviest row blocks first
  // (key block 0 sees every query; the last query block sees every key)
  int b, hx, xb;
  {
    const int per_group = p.heads_per_wave * p.num_row_blocks;
    const int grp = blockIdx.x / per_group;
    const int w = blockIdx.x - grp * per_group;
    const int size = min(p.heads_per_wave, p.num_bh - grp * p.heads_per_wave);
    const int rank = w / size;
    const int bh = grp * p.heads_per_wave + (w - rank * size);
    if (rank >= p.num_row_blocks) return;
    xb = kKeys ? rank : p.num_row_blocks - 1 - rank;
    b = bh / p.heads_x;
    hx = bh - b * p.heads_x;
  }
  int q_off = 0, k_off = 0, len_q = p.seqlen_q, len_k = p.seqlen_k, bcoord = b;
  if (p.cu_q != nullptr) {
    q_off = p.cu_q[b];
    len_q = p.cu_q[b + 1] - q_off;
    k_off = p.cu_k[b];
    len_k = p.cu_k[b + 1] - k_off;
    bcoord = 0;
  }
  const int causal_off = len_k - len_q;
  const int len_x = kKeys ? len_k : len_q;
  const int x0 = xb * kRowsA;
  if (x0 >= len_x) return;
  const int x_off = kKeys ? k_off : q_off;
  const int y_off = kKeys ? q_off : k_off;

  // streamed 64-row blocks [y_lo, y_hi) per head, and heads per CTA
  int y_lo = 0, y_hi;
  if (kKeys) {
    y_hi = (len_q + kRowsB - 1) / kRowsB;
    if (p.is_causal) {
      y_lo = max(0, (x0 - causal_off) / kRowsB);  // first query block with a row >= x0 - off
      if (x0 - causal_off > len_q - 1) y_lo = y_hi;
    }
  } else {
    int vis_end = len_k;
    if (p.is_causal) vis_end = min(len_k, x0 + kRowsA + causal_off);
    y_hi = vis_end > 0 ? (vis_end + kRowsB - 1) / kRowsB : 0;
  }
  const int blocks_per_head = max(0, y_hi - y_lo);
  const int heads_here = kKeys ? p.kv_group : 1;
  const int n_items = blocks_per_head * heads_here;
  const int hkv = kKeys ? hx : hx / p.kv_group;

  const uint32_t bar = base + kSmemBars;
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(smem + kSmemBars + kAbortWordB);
  volatile uint32_t* tmem_ptr_smem = reinterpret_cast<volatile uint32_t*>(smem + kSmemBars + kTmemPtrB);

  if (warp == 8 && lane == 0) {
    tma_prefetch_desc(&tm_y1);
    tma_prefetch_desc(&tm_y2);
    for (int s = 0; s < kRing; ++s) {
      mbar_init(bar + kBFull + 8 * s, 1);
      mbar_init(bar + kBEmpty + 8 * s, 1);
    }
    mbar_init(bar + kBAReady, 8);
    mbar_init(bar + kBX2Full, 1);
    mbar_init(bar + kBTFull, 1);
    mbar_init(bar + kBTFull + 8, 1);
    mbar_init(bar + kBDFree, 8);
    mbar_init(bar + kBWFull, 8);
    mbar_init(bar + kBWRead, 1);
    mbar_init(bar + kBAccFull, 1);
    mbar_init(bar + kBStageB, 8);
    *abort_flag = 0;
    fence_mbar_init();
    if (kMode != kDV && n_items > 0) {
      // X2: 128 rows x 256 columns as four boxes of 128 rows x 64 columns at the start of shared memory
      mbar_arrive_expect_tx(bar + kBX2Full, 4 * kRowsA * 128);
#pragma unroll
      for (int c = 0; c < 4; ++c)
        tma_load_4d(base + c * (kRowsA * 128), &tm_x2, bar + kBX2Full, c * 64, x_off + x0, kKeys ? hkv : hx, bcoord);
    }
  }
  if (warp == 0) {
    __syncwarp();
    tmem_alloc(base + kSmemBars + kTmemPtrB, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_ptr_smem;
  const uint32_t t_x1 = tmem_base, t_a = tmem_base + 128, t_b = tmem_base + 192, t_acc = tmem_base + 256;
  // ring tile t: Y1(t/2) if even, Y2(t/2) if odd; item i = (head index i / blocks_per_head, block y_lo + i % blocks_per_head)
  auto slot_index = [&](int t) { return t % kRing; };
  auto slot_addr = [&](int t) { return base + kRingBase + (t % kRing) * kSlotBytes; };

  if (warp == 8) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      for (int t = 0; t < 2 * n_items; ++t) {
        const int i = t >> 1;
        const int s = slot_index(t);
        if (!mbar_wait(bar + kBEmpty + 8 * s, ((static_cast<uint32_t>(t / kRing)) & 1u) ^ 1u, abort_flag)) break;
        const int hi = i / blocks_per_head;
        const int yb = y_lo + (i - hi * blocks_per_head);
        const int hy = kKeys ? hx * p.kv_group + hi : hkv;  // streamed head: a query head of the group, or the KV head
        const uint32_t full = bar + kBFull + 8 * s;
        const uint32_t dst = slot_addr(t);
        const int row = y_off + yb * kRowsB;
        const bool first = (t & 1) == 0;
        if (kKeys && first) {
          mbar_arrive_expect_tx(full, kSlotBytes + 512);
          const size_t vec = (static_cast<size_t>(b) * p.heads_q + hy) * p.lq_pad + static_cast<size_t>(yb) * kRowsB;
          const uint32_t vdst = base + kSmemVecs + s * 512;
          asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(vdst),
                       "l"(p.lse2 + vec), "r"(256), "r"(full) : "memory");
          asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(vdst + 256),
                       "l"(p.delta + vec), "r"(256), "r"(full) : "memory");
        } else {
          mbar_arrive_expect_tx(full, kSlotBytes);
        }
        const CUtensorMap* tm = first ? &tm_y1 : &tm_y2;
#pragma unroll
        for (int c = 0; c < 4; ++c) tma_load_4d(dst + c * kBoxBytes, tm, full, c * 64, row, hy, bcoord);
      }
      drain_after_abort(abort_flag);
    }
  } else if (warp == 9 || warp == 10) {
    // ------------------------------------------------------------------ MMA issuers
    // One thread needs ~50 cycles to issue an MMA, and the N = 64 score MMAs run for 32 (48 with both operands in shared
    // memory): a single issuer would hold the pipe back. So warp 9 issues the score GEMMs and warp 10 the accumulations;
    // what the pipe's own order would guarantee between the two is the `W read` barrier (warp 10 commits it behind an item's
    // accumulation, warp 9 waits for it before a score GEMM overwrites that item's P / dS).
    if (lane == 0 && n_items > 0) {
      auto wait_full = [&](int t) { return mbar_wait(bar + kBFull + 8 * slot_index(t), (t / kRing) & 1, abort_flag); };
      auto release = [&](int t) { umma_commit(bar + kBEmpty + 8 * slot_index(t)); };
      auto t_buf = [&](int k) { return (k & 1) ? t_b : t_a; };
      bool ok = mbar_wait(bar + kBAReady, 0, abort_flag);
      if (kMode != kDV) ok = ok && mbar_wait(bar + kBX2Full, 0, abort_flag);
      if (warp == 10) {
        // ---------------- accumulations: ACC += W(i) Y, W = P^T (kDV, Y = dO block) or dS (Y = the Y1 block)
        for (int i = 0; ok && i < n_items; ++i) {
          const int ty = (kMode == kDV) ? 2 * i + 1 : 2 * i;
          ok = mbar_wait(bar + kBWFull, i & 1, abort_flag) && wait_full(ty);
          if (!ok) break;
          tc_fence_after_sync();
          issue_accumulate256_split<kF16>(t_acc, t_buf(i), slot_addr(ty), i > 0);
          umma_commit(bar + kBWRead);
          // kDV: the Q block goes too - its slot carries the per-query vectors the compute warps have just used
          release(2 * i);
          if (kMode == kDV) release(2 * i + 1);
          if (i == n_items - 1) umma_commit(bar + kBAccFull);
        }
      } else if (kMode == kDV) {
        // ---------------- scores: S(i) in T[i&1]; S(i+2) follows the accumulation of item i
        for (int i = 0; ok && i < n_items; ++i) {
          if (i >= 2) ok = mbar_wait(bar + kBWRead, (i - 2) & 1, abort_flag);
          ok = ok && wait_full(2 * i);
          if (!ok) break;
          tc_fence_after_sync();
          issue_scores<kF16>(t_buf(i), t_x1, slot_addr(2 * i));
          umma_commit(bar + kBTFull + 8 * (i & 1));
        }
      } else {
        // ---------------- scores: S(i) in T[i&1], dP(i) in T[(i&1)^1]
        ok = ok && wait_full(0);
        if (ok) {
          tc_fence_after_sync();
          issue_scores<kF16>(t_buf(0), t_x1, slot_addr(0));
          umma_commit(bar + kBTFull);
        }
        ok = ok && wait_full(1);
        if (ok) {
          tc_fence_after_sync();
          issue_scores_ss<kF16>(t_buf(1), base, slot_addr(1));
          umma_commit(bar + kBTFull + 8);
          release(1);  // a Y2 block is read by this GEMM only
        }
        for (int i = 0; ok && i + 1 < n_items; ++i) {
          // dP(i) has left TMEM once the compute warps have read it: its buffer takes S(i+1)
          ok = mbar_wait(bar + kBDFree, i & 1, abort_flag) && wait_full(2 * i + 2);
          if (!ok) break;
          tc_fence_after_sync();
          issue_scores<kF16>(t_buf(i + 1), t_x1, slot_addr(2 * i + 2));
          umma_commit(bar + kBTFull + 8 * ((i + 1) & 1));
          // dS(i) has left TMEM once the accumulation of item i has read it: its buffer takes dP(i+1)
          ok = mbar_wait(bar + kBWRead, i & 1, abort_flag) && wait_full(2 * i + 3);
          if (!ok) break;
          tc_fence_after_sync();
          issue_scores_ss<kF16>(t_buf(i), base, slot_addr(2 * i + 3));
          umma_commit(bar + kBTFull + 8 * (i & 1));
          release(2 * i + 3);
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ compute warps (thread = stationary row)
    const int half = warp >> 2;              // which 32 of a block's 64 streamed rows this thread works on
    const int r = (warp & 3) * 32 + lane;    // stationary row = TMEM lane
    const int xr = x0 + r;
    const bool valid = xr < len_x;
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    {
      const uint16_t* xrow = nullptr;
      if (valid)
        xrow = p.x1 + ((p.cu_q != nullptr) ? static_cast<int64_t>(x_off + xr) * p.x1_row_stride
                                           : b * p.x1_batch_stride + static_cast<int64_t>(xr) * p.x1_row_stride) +
               (kKeys ? hkv : hx) * p.x1_head_stride;
      row_half_to_tmem(t_x1 + lane_base, xrow, p.head_dim, half);  // each warpgroup brings half of the row's columns
      tmem_wait_st();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar + kBAReady);
    }
    const float c = p.scale_log2;
    float my_lse2 = INFINITY, my_delta = 0.f;  // kDQ: this row's own values
    if (kMode == kDQ && valid) {
      const size_t vec = (static_cast<size_t>(b) * p.heads_q + hx) * p.lq_pad + xr;
      my_lse2 = p.lse2[vec];
      my_delta = p.delta[vec];
    }
    bool ok = true;
    // phase counters of the two score barriers (a buffer receives S and dP alternately)
    uint32_t seen[2] = {0u, 0u};
    for (int i = 0; i < n_items; ++i) {
      const int hi = i / blocks_per_head;
      const int y0 = (y_lo + (i - hi * blocks_per_head)) * kRowsB;
      const int sb = i & 1;                              // buffer of S(i)
      const int db = (kMode == kDV) ? sb : (sb ^ 1);     // buffer of dP(i)
      const uint32_t t_s = ((sb) ? t_b : t_a) + lane_base + half * 32;  // this thread's 32 fp32 columns
      const uint32_t t_d = ((db) ? t_b : t_a) + lane_base + half * 32;
      // keep bits of this thread's 64 (row, column) pairs, in flight under the waits below
      uint32_t keep = 0u;
      if constexpr (kDrop) {
        const int hq = kKeys ? hx * p.kv_group + hi : hx;  // the query head the pattern belongs to
        const uint32_t* words =
            kKeys ? p.keep_cols + (p.cu_q != nullptr ? static_cast<size_t>(hq) * p.keep_k_rows + k_off + xr
                                                     : static_cast<size_t>(b * p.heads_q + hq) * p.keep_k_rows + xr) *
                                      (p.keep_lq_pad >> 5)
                  : p.keep_rows + (p.cu_q != nullptr ? static_cast<size_t>(hq) * p.keep_q_rows + q_off + xr
                                                     : static_cast<size_t>(b * p.heads_q + hq) * p.keep_q_rows + xr) *
                                      (p.keep_lk_pad >> 5);
        keep = words[(y0 >> 5) + half];
      }
      ok = mbar_wait(bar + kBTFull + 8 * sb, seen[sb] & 1u, abort_flag);
      ++seen[sb];
      if (kKeys) ok = ok && mbar_wait(bar + kBFull + 8 * slot_index(2 * i), ((2 * i) / kRing) & 1, abort_flag);  // the vectors
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after_sync();
      const float* vec_lse = reinterpret_cast<const float*>(smem + kSmemVecs + slot_index(2 * i) * 512) + half * 32;
      const float* vec_delta = vec_lse + 64;
      // visibility of element (row xr, column y0 + j)
      //   keys as rows : key xr, query y0+j : visible iff j >= xr - off - y0 (and the key exists)
      //   queries      : query xr, key y0+j : visible iff y0 + j <= xr + off and y0 + j < len_k
      constexpr int kCols = kRowsB / 2;  // columns per thread
      int j_lo = 0, j_hi = kRowsB;
      if (kKeys) {
        if (p.is_causal) j_lo = xr - causal_off - y0;
        if (!valid) j_lo = kRowsB;  // a row past the last key holds zeros (or, packed, the next sequence's key)
      } else {
        j_hi = len_k - y0;
        if (p.is_causal) j_hi = min(j_hi, xr + causal_off + 1 - y0);
      }
      j_lo -= half * kCols;  // relative to this thread's columns
      j_hi -= half * kCols;
      float pr[kCols];
      {
        uint32_t a[kCols];
        tmem_ld_x32(t_s, a);
        tmem_wait_ld();
#pragma unroll
        for (int j = 0; j < kCols; ++j) {
          const float l2 = kKeys ? vec_lse[j] : my_lse2;
          pr[j] = ex2_approx(fmaf(__uint_as_float(a[j]), c, -l2));
        }
        if (__any_sync(0xffffffffu, j_lo > 0 || j_hi < kCols)) {
#pragma unroll
          for (int j = 0; j < kCols; ++j) pr[j] = (j >= j_lo && j < j_hi) ? pr[j] : 0.f;
        }
      }
      uint32_t w[kCols / 2];
      if (kMode == kDV) {
#pragma unroll
        for (int j2 = 0; j2 < kCols / 2; ++j2) {
          w[j2] = pack_16x2<kF16>(pr[2 * j2], pr[2 * j2 + 1]);
          if constexpr (kDrop) w[j2] &= keep_pair(keep >> (2 * j2));
        }
      } else {
        ok = __all_sync(0xffffffffu, mbar_wait(bar + kBTFull + 8 * db, seen[db] & 1u, abort_flag));
        ++seen[db];
        if (!ok) break;
        tc_fence_after_sync();
        uint32_t d[kCols];
        tmem_ld_x32(t_d, d);
        tmem_wait_ld();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar + kBDFree);  // the dP buffer may be overwritten
#pragma unroll
        for (int j2 = 0; j2 < kCols / 2; ++j2) {
          const float dl0 = kKeys ? vec_delta[2 * j2] : my_delta;
          const float dl1 = kKeys ? vec_delta[2 * j2 + 1] : my_delta;
          float dp0 = __uint_as_float(d[2 * j2]), dp1 = __uint_as_float(d[2 * j2 + 1]);
          if constexpr (kDrop) {
            const uint32_t two = keep >> (2 * j2);
            dp0 = (two & 1u) ? dp0 * p.keep_scale : 0.f;
            dp1 = (two & 2u) ? dp1 * p.keep_scale : 0.f;
          }
          w[j2] = pack_16x2<kF16>(pr[2 * j2] * (dp0 - dl0), pr[2 * j2 + 1] * (dp1 - dl1));
        }
      }
      // the 16-bit result over the front of this thread's OWN score columns (16 columns = 32 streamed rows): the other
      // warpgroup may still be reading its half of the scores
      tmem_st_x16(t_s, w);
      tmem_wait_st();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar + kBWFull);
    }

    // ---- epilogue: accumulator -> scale -> 16 bit -> global
    if (ok && n_items > 0) ok = __all_sync(0xffffffffu, mbar_wait(bar + kBAccFull, 0, abort_flag));
    if (ok) {
      tc_fence_after_sync();
      const float mul = (kMode == kDV) ? (kDrop ? p.keep_scale : 1.f) : p.scale;
      const bool use_tma = (p.cu_q == nullptr) || (x0 + kRowsA <= len_x);
      uint16_t* orow = p.out + ((p.cu_q != nullptr) ? static_cast<int64_t>(x_off + xr) * p.o_row_stride
                                                    : b * p.o_batch_stride + static_cast<int64_t>(xr) * p.o_row_stride) +
                       hx * p.o_head_stride;
#pragma unroll
      for (int c2 = 0; c2 < kWide / 64; ++c2) {
        const int cc = half * (kWide / 64) + c2;  // this warpgroup's half of the 256 columns
        uint32_t o[32];
        if (n_items > 0) {
          tmem_ld_x32(t_acc + lane_base + cc * 32, o);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) o[j] = 0u;
        }
        uint4 wv[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          wv[j].x = pack_16x2<kF16>(__uint_as_float(o[8 * j]) * mul, __uint_as_float(o[8 * j + 1]) * mul);
          wv[j].y = pack_16x2<kF16>(__uint_as_float(o[8 * j + 2]) * mul, __uint_as_float(o[8 * j + 3]) * mul);
          wv[j].z = pack_16x2<kF16>(__uint_as_float(o[8 * j + 4]) * mul, __uint_as_float(o[8 * j + 5]) * mul);
          wv[j].w = pack_16x2<kF16>(__uint_as_float(o[8 * j + 6]) * mul, __uint_as_float(o[8 * j + 7]) * mul);
        }
        const int col = cc * 32;
        if (use_tma) {
          // staged behind X2 (the ring is idle by now): four boxes of 128 rows x 64 columns
          uint8_t* srow = smem + kRingBase + (col >> 6) * (kRowsA * 128) + r * 128;
          const int chunk0 = (col & 63) >> 3;
#pragma unroll
          for (int j = 0; j < 4; ++j) *reinterpret_cast<uint4*>(srow + (((chunk0 + j) ^ (r & 7)) << 4)) = wv[j];
        } else if (valid) {
#pragma unroll
          for (int j = 0; j < 4; ++j)
            if (col + 8 * j < p.head_dim) *reinterpret_cast<uint4*>(orow + col + 8 * j) = wv[j];
        }
      }
      if (use_tma) {
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar + kBStageB);
        if (threadIdx.x == 0) {
          if (mbar_wait(bar + kBStageB, 0, abort_flag)) {
#pragma unroll
            for (int c4 = 0; c4 < 4; ++c4)
              tma_store_4d(&tm_out, base + kRingBase + c4 * (kRowsA * 128), c4 * 64, x_off + x0, hx, bcoord);
            tma_store_commit();
            tma_store_wait_read();
          }
        }
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
  if (threadIdx.x == 0 && *abort_flag != 0) atomicExch(p.status, static_cast<uint32_t>(SDPA_B200_DEVICE_TIMEOUT));
}

// delta[row] = sum_d dO[row, d] O[row, d] and lse2 = lse * log2(e) into the padded [batch, heads_q, lq_pad] vectors (padding
// rows: lse2 = +inf, delta = 0). One warp per row: 32 lanes x 8 elements cover 256 columns.
struct Pre256Params {
  const uint16_t* out;
  const uint16_t* dout;
  const float* lse;
  float* lse2;
  float* delta;
  const int32_t* cu_q;
  int64_t o_batch_stride, o_head_stride, o_row_stride;
  int64_t do_batch_stride, do_head_stride, do_row_stride;
  int seqlen_q, total_q, heads_q, lq_pad, head_dim;
};

template <bool kF16>
__global__ void __launch_bounds__(256) bwd_d256_preprocess_kernel(const Pre256Params p) {
  const int h = blockIdx.x, b = blockIdx.z;
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.y * 8 + (threadIdx.x >> 5);
  if (row >= p.lq_pad) return;
  int q_off = 0, len_q = p.seqlen_q;
  if (p.cu_q != nullptr) {
    q_off = p.cu_q[b];
    len_q = p.cu_q[b + 1] - q_off;
  }
  float acc = 0.f;
  if (row < len_q && lane * 8 < p.head_dim) {
    const uint16_t* o;
    const uint16_t* dout;
    if (p.cu_q != nullptr) {
      o = p.out + static_cast<int64_t>(q_off + row) * p.o_row_stride + h * p.o_head_stride;
      dout = p.dout + static_cast<int64_t>(q_off + row) * p.do_row_stride + h * p.do_head_stride;
    } else {
      o = p.out + b * p.o_batch_stride + h * p.o_head_stride + static_cast<int64_t>(row) * p.o_row_stride;
      dout = p.dout + b * p.do_batch_stride + h * p.do_head_stride + static_cast<int64_t>(row) * p.do_row_stride;
    }
    const uint4 ov = *reinterpret_cast<const uint4*>(o + lane * 8);
    const uint4 dv = *reinterpret_cast<const uint4*>(dout + lane * 8);
    const uint32_t ow[4] = {ov.x, ov.y, ov.z, ov.w}, dw[4] = {dv.x, dv.y, dv.z, dv.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 a = unpack_16x2<kF16>(ow[i]), d = unpack_16x2<kF16>(dw[i]);
      acc += a.x * d.x + a.y * d.y;
    }
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  if (lane == 0) {
    const size_t dst = (static_cast<size_t>(b) * p.heads_q + h) * p.lq_pad + row;
    if (row < len_q) {
      const float lse = (p.cu_q != nullptr) ? p.lse[static_cast<size_t>(h) * p.total_q + q_off + row]
                                            : p.lse[(static_cast<size_t>(b) * p.heads_q + h) * p.seqlen_q + row];
      p.lse2[dst] = lse * 1.4426950408889634f;  // +inf stays +inf
      p.delta[dst] = acc;
    } else {
      p.lse2[dst] = INFINITY;
      p.delta[dst] = 0.f;
    }
  }
}

// heads per group so that the streamed K + V of a group stay within ~48 MB of L2
int heads_per_wave_for(double bytes_per_head, int num_bh) {
  int hpw = static_cast<int>((48.0 * 1024 * 1024) / bytes_per_head);
  hpw = hpw < 1 ? 1 : (hpw > 32 ? 32 : hpw);
  return hpw > num_bh ? num_bh : hpw;
}

}  // namespace

namespace {
using Bwd256Kernel = void (*)(const CUtensorMap, const CUtensorMap, const CUtensorMap, const CUtensorMap, const Bwd256Params);
template <int kMode>
Bwd256Kernel pick_bwd256(bool f16, bool drop) {
  if (drop) return f16 ? bwd_d256_kernel<kMode, true, true> : bwd_d256_kernel<kMode, false, true>;
  return f16 ? bwd_d256_kernel<kMode, true, false> : bwd_d256_kernel<kMode, false, false>;
}
}  // namespace

size_t bwd_d256_workspace_bytes(const sdpa_b200_params& p) {
  const size_t lq_pad = (static_cast<size_t>(p.max_seqlen_q) + kRowsA - 1) / kRowsA * kRowsA;
  return 2 * static_cast<size_t>(p.batch) * p.heads_q * lq_pad * sizeof(float);
}

int launch_bwd_d256(const sdpa_b200_params& p, void* workspace, cudaStream_t stream) {
  const bool f16 = p.dtype == SDPA_B200_F16;
  const bool varlen = p.cu_seqlens_q != nullptr;
  const int lq_pad = (p.max_seqlen_q + kRowsA - 1) / kRowsA * kRowsA;
  const size_t vec_elems = static_cast<size_t>(p.batch) * p.heads_q * lq_pad;
  float* lse2 = reinterpret_cast<float*>(static_cast<char*>(workspace) + kWorkspaceHeaderBytes);
  float* delta = lse2 + vec_elems;

  Pre256Params pre;
  pre.out = static_cast<const uint16_t*>(p.out);
  pre.dout = static_cast<const uint16_t*>(p.dout);
  pre.lse = p.lse;
  pre.lse2 = lse2;
  pre.delta = delta;
  pre.cu_q = p.cu_seqlens_q;
  pre.o_batch_stride = p.o_batch_stride;
  pre.o_head_stride = p.o_head_stride;
  pre.o_row_stride = p.o_row_stride;
  pre.do_batch_stride = p.do_batch_stride;
  pre.do_head_stride = p.do_head_stride;
  pre.do_row_stride = p.do_row_stride;
  pre.seqlen_q = p.max_seqlen_q;
  pre.total_q = p.total_q;
  pre.heads_q = p.heads_q;
  pre.lq_pad = lq_pad;
  pre.head_dim = p.head_dim;
  const dim3 pre_grid(p.heads_q, lq_pad / 8, p.batch);
  if (f16) bwd_d256_preprocess_kernel<true><<<pre_grid, 256, 0, stream>>>(pre);
  else bwd_d256_preprocess_kernel<false><<<pre_grid, 256, 0, stream>>>(pre);
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) {
    set_error("head_dim 256 backward pre-pass: launch failed: %s", cudaGetErrorString(err));
    return SDPA_B200_LAUNCH_FAILED;
  }
  count_launch();

  const int64_t rows_q = varlen ? p.total_q : p.max_seqlen_q;
  const int64_t rows_k = varlen ? p.total_k : p.max_seqlen_k;
  const int64_t nb = varlen ? 1 : p.batch;
  // streamed blocks (64 rows), shared-memory resident tiles and outputs (128 rows)
  CUtensorMap q64, k64, v64, do64, v128, do128, dq128, dk128, dv128;
  int st;
  auto map = [&](CUtensorMap* m, const void* ptr, int64_t rows, int heads, int64_t rs, int64_t hs, int64_t bs, int box) {
    return make_tensor_map_16(f16, m, ptr, p.head_dim, rows, heads, nb, rs, hs, bs, box);
  };
  if ((st = map(&q64, p.q, rows_q, p.heads_q, p.q_row_stride, p.q_head_stride, p.q_batch_stride, kRowsB)) != SDPA_B200_OK) return st;
  if ((st = map(&k64, p.k, rows_k, p.heads_kv, p.k_row_stride, p.k_head_stride, p.k_batch_stride, kRowsB)) != SDPA_B200_OK) return st;
  if ((st = map(&v64, p.v, rows_k, p.heads_kv, p.v_row_stride, p.v_head_stride, p.v_batch_stride, kRowsB)) != SDPA_B200_OK) return st;
  if ((st = map(&do64, p.dout, rows_q, p.heads_q, p.do_row_stride, p.do_head_stride, p.do_batch_stride, kRowsB)) != SDPA_B200_OK) return st;
  if ((st = map(&v128, p.v, rows_k, p.heads_kv, p.v_row_stride, p.v_head_stride, p.v_batch_stride, kRowsA)) != SDPA_B200_OK) return st;
  if ((st = map(&do128, p.dout, rows_q, p.heads_q, p.do_row_stride, p.do_head_stride, p.do_batch_stride, kRowsA)) != SDPA_B200_OK) return st;
  if ((st = map(&dq128, p.dq, rows_q, p.heads_q, p.dq_row_stride, p.dq_head_stride, p.dq_batch_stride, kRowsA)) != SDPA_B200_OK) return st;
  if ((st = map(&dk128, p.dk, rows_k, p.heads_kv, p.dk_row_stride, p.dk_head_stride, p.dk_batch_stride, kRowsA)) != SDPA_B200_OK) return st;
  if ((st = map(&dv128, p.dv, rows_k, p.heads_kv, p.dv_row_stride, p.dv_head_stride, p.dv_batch_stride, kRowsA)) != SDPA_B200_OK) return st;

  Bwd256Params kp;
  kp.lse2 = lse2;
  kp.delta = delta;
  kp.cu_q = p.cu_seqlens_q;
  kp.cu_k = p.cu_seqlens_k;
  kp.status = p.device_status != nullptr ? p.device_status : static_cast<uint32_t*>(workspace);
  kp.seqlen_q = p.max_seqlen_q;
  kp.seqlen_k = p.max_seqlen_k;
  kp.heads_q = p.heads_q;
  kp.heads_kv = p.heads_kv;
  kp.kv_group = p.heads_q / p.heads_kv;
  kp.head_dim = p.head_dim;
  kp.lq_pad = lq_pad;
  kp.scale = p.softmax_scale;
  kp.scale_log2 = p.softmax_scale * 1.4426950408889634f;
  kp.is_causal = p.is_causal;
  const bool drop = p.dropout_p > 0.f;
  kp.keep_rows = drop ? p.keep_rows : nullptr;
  kp.keep_cols = drop ? p.keep_cols : nullptr;
  kp.keep_lq_pad = (p.max_seqlen_q + 127) / 128 * 128;
  kp.keep_lk_pad = (p.max_seqlen_k + 127) / 128 * 128;
  kp.keep_q_rows = varlen ? p.total_q + 128 : kp.keep_lq_pad;
  kp.keep_k_rows = varlen ? p.total_k + 128 : kp.keep_lk_pad;
  kp.keep_scale = drop ? 1.f / (1.f - p.dropout_p) : 1.f;

  auto launch = [&](int mode, const CUtensorMap& x2, const CUtensorMap& y1, const CUtensorMap& y2, const CUtensorMap& out) {
    void (*kernel)(const CUtensorMap, const CUtensorMap, const CUtensorMap, const CUtensorMap, const Bwd256Params);
    if (mode == kDV) kernel = pick_bwd256<kDV>(f16, drop);
    else if (mode == kDK) kernel = pick_bwd256<kDK>(f16, drop);
    else kernel = pick_bwd256<kDQ>(f16, drop);
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytesBwd256);
    if (e != cudaSuccess) {
      set_error("head_dim 256 backward: cudaFuncSetAttribute(%u bytes smem): %s", kSmemBytesBwd256, cudaGetErrorString(e));
      return static_cast<int>(SDPA_B200_LAUNCH_FAILED);
    }
    const bool keys = mode != kDQ;
    kp.heads_x = keys ? p.heads_kv : p.heads_q;
    kp.num_bh = p.batch * kp.heads_x;
    kp.num_row_blocks = ((keys ? p.max_seqlen_k : p.max_seqlen_q) + kRowsA - 1) / kRowsA;
    // bytes one stationary head streams: Q + dO of its group (keys), or K + V (queries)
    const double streamed = 2.0 * (keys ? p.max_seqlen_q : p.max_seqlen_k) * p.head_dim * 2 * (keys ? kp.kv_group : 1);
    kp.heads_per_wave = heads_per_wave_for(streamed, kp.num_bh);
    const int groups = (kp.num_bh + kp.heads_per_wave - 1) / kp.heads_per_wave;
    const int grid = groups * kp.heads_per_wave * kp.num_row_blocks;
    kernel<<<grid, kBwdThreads, kSmemBytesBwd256, stream>>>(x2, y1, y2, out, kp);
    e = cudaGetLastError();
    if (e != cudaSuccess) {
      set_error("head_dim 256 backward (kernel %d): launch failed: %s", mode, cudaGetErrorString(e));
      return static_cast<int>(SDPA_B200_LAUNCH_FAILED);
    }
    count_launch();
    return static_cast<int>(SDPA_B200_OK);
  };
  auto set_io = [&](const void* x1, int64_t bs, int64_t hs, int64_t rs, void* out, int64_t obs, int64_t ohs, int64_t ors) {
    kp.x1 = static_cast<const uint16_t*>(x1);
    kp.x1_batch_stride = bs;
    kp.x1_head_stride = hs;
    kp.x1_row_stride = rs;
    kp.out = static_cast<uint16_t*>(out);
    kp.o_batch_stride = obs;
    kp.o_head_stride = ohs;
    kp.o_row_stride = ors;
  };
  set_io(p.k, p.k_batch_stride, p.k_head_stride, p.k_row_stride, p.dv, p.dv_batch_stride, p.dv_head_stride, p.dv_row_stride);
  if ((st = launch(kDV, v128 /*unused*/, q64, do64, dv128)) != SDPA_B200_OK) return st;
  set_io(p.k, p.k_batch_stride, p.k_head_stride, p.k_row_stride, p.dk, p.dk_batch_stride, p.dk_head_stride, p.dk_row_stride);
  if ((st = launch(kDK, v128, q64, do64, dk128)) != SDPA_B200_OK) return st;
  set_io(p.q, p.q_batch_stride, p.q_head_stride, p.q_row_stride, p.dq, p.dq_batch_stride, p.dq_head_stride, p.dq_row_stride);
  return launch(kDQ, do128, k64, v64, dq128);
}

int launch_fwd_d256(const sdpa_b200_params& p, void* workspace, cudaStream_t stream) {
  const bool f16 = p.dtype == SDPA_B200_F16;
  const bool varlen = p.cu_seqlens_q != nullptr;
  const int64_t rows_q = varlen ? p.total_q : p.max_seqlen_q;
  const int64_t rows_k = varlen ? p.total_k : p.max_seqlen_k;
  const int64_t nb = varlen ? 1 : p.batch;
  CUtensorMap tm_k, tm_v, tm_o;
  int st;
  if ((st = make_tensor_map_16(f16, &tm_k, p.k, p.head_dim, rows_k, p.heads_kv, nb, p.k_row_stride, p.k_head_stride,
                               p.k_batch_stride, kRowsB)) != SDPA_B200_OK)
    return st;
  if ((st = make_tensor_map_16(f16, &tm_v, p.v, p.head_dim, rows_k, p.heads_kv, nb, p.v_row_stride, p.v_head_stride,
                               p.v_batch_stride, kRowsB)) != SDPA_B200_OK)
    return st;
  if ((st = make_tensor_map_16(f16, &tm_o, p.out, p.head_dim, rows_q, p.heads_q, nb, p.o_row_stride, p.o_head_stride,
                               p.o_batch_stride, kRowsA)) != SDPA_B200_OK)
    return st;
  D256Params kp;
  kp.q = static_cast<const uint16_t*>(p.q);
  kp.out = static_cast<uint16_t*>(p.out);
  kp.lse = p.lse;
  kp.cu_q = p.cu_seqlens_q;
  kp.cu_k = p.cu_seqlens_k;
  kp.status = p.device_status != nullptr ? p.device_status : static_cast<uint32_t*>(workspace);
  kp.q_batch_stride = p.q_batch_stride;
  kp.q_head_stride = p.q_head_stride;
  kp.q_row_stride = p.q_row_stride;
  kp.o_batch_stride = p.o_batch_stride;
  kp.o_head_stride = p.o_head_stride;
  kp.o_row_stride = p.o_row_stride;
  kp.seqlen_q = p.max_seqlen_q;
  kp.seqlen_k = p.max_seqlen_k;
  kp.total_q = p.total_q;
  kp.heads_q = p.heads_q;
  kp.kv_group = p.heads_q / p.heads_kv;
  kp.head_dim = p.head_dim;
  kp.num_m_blocks = (p.max_seqlen_q + kRowsA - 1) / kRowsA;
  kp.num_bh = p.batch * p.heads_q;
  kp.heads_per_wave = heads_per_wave_for(2.0 * p.max_seqlen_k * p.head_dim * 2 / kp.kv_group, kp.num_bh);
  kp.scale_log2 = p.softmax_scale * 1.4426950408889634f;
  kp.is_causal = p.is_causal;
  const bool drop = p.dropout_p > 0.f;
  kp.keep_rows = drop ? p.keep_rows : nullptr;
  kp.keep_rows_per = varlen ? p.total_q + 128 : (p.max_seqlen_q + 127) / 128 * 128;
  kp.lk_words = (p.max_seqlen_k + 127) / 128 * 4;
  kp.keep_scale = drop ? 1.f / (1.f - p.dropout_p) : 1.f;
  auto kernel = drop ? (f16 ? fwd_d256_kernel<true, true> : fwd_d256_kernel<false, true>)
                     : (f16 ? fwd_d256_kernel<true, false> : fwd_d256_kernel<false, false>);
  cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytesD256);
  if (err != cudaSuccess) {
    set_error("head_dim 256 forward: cudaFuncSetAttribute(%u bytes smem): %s", kSmemBytesD256, cudaGetErrorString(err));
    return SDPA_B200_LAUNCH_FAILED;
  }
  const int groups = (kp.num_bh + kp.heads_per_wave - 1) / kp.heads_per_wave;
  const int grid = groups * kp.heads_per_wave * kp.num_m_blocks;
  kernel<<<grid, 192, kSmemBytesD256, stream>>>(tm_k, tm_v, tm_o, kp);
  err = cudaGetLastError();
  if (err != cudaSuccess) {
    set_error("head_dim 256 forward: launch failed: %s", cudaGetErrorString(err));
    return SDPA_B200_LAUNCH_FAILED;
  }
  count_launch();
  return SDPA_B200_OK;
}

}  // namespace sdpa_b200
