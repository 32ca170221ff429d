// Prefill / forward attention kernel for sm_100a.
//
// Replaces the device work behind mha_varlen_fwd -> cnnlFlashAttentionForward_v2
// (torch_mlu/csrc/aten/operators/cnnl/internal/FlashAttention_internal.cpp:231-258):
//   O = softmax(scale * Q K^T + causal mask) V,  LSE = logsumexp(scale * Q K^T)
// for bf16 or f16 Q/K/V with head_dim 64 or 128, dense or packed-varlen, GQA by head broadcast.
//
// One CTA owns 256 query rows of one (batch, head): two 128-row Q tiles. Roles:
//   warps 0-3  softmax warpgroup for Q tile 0  (thread = one query row = one TMEM lane)
//   warps 4-7  softmax warpgroup for Q tile 1
//   warp  8    TMA producer: Q once, then K(j), V(j) tiles into a 4-stage 32 KB ring
//   warp  9    MMA issuer: S_t = Q_t K^T and O_t += P_t V on tcgen05, accumulators in TMEM
//   warps 10-11 idle; they complete the third warpgroup so it can hand its registers to the
//              softmax warpgroups (setmaxnreg), which hold a whole 128-column S row per thread
// TMEM (512 columns): S0 [0,128) S1 [128,256) O0 [256,384) O1 [384,512); P_t (16-bit, 64
// columns) overwrites the front of S_t once the softmax thread holds the whole S row in
// registers. The two Q tiles ping-pong: while one warpgroup exponentiates, the tensor core
// runs the other tile's GEMMs. Online softmax works in the log2 domain; O is rescaled lazily
// (only when a row maximum grows by more than 2^8), by the softmax thread that owns the row.
#include <cuda_bf16.h>

#include "kernels.h"
#include "ptx_sm100.cuh"

namespace sdpa_b200 {
namespace {

constexpr int kBlockM = 128;
constexpr int kBlockN = 128;
constexpr int kMaxHeadDim = 128;  // shared-memory slots are sized for it; head_dim 64 uses half of each
constexpr int kStages = 4;
constexpr uint32_t kTileBytes = kBlockN * kMaxHeadDim * 2;  // 32768: one shared-memory slot
constexpr uint32_t kHalfBytes = kTileBytes / 2;          // one 64-column TMA box
constexpr int kNumThreads = 384;  // 3 warpgroups; warps 10-11 idle
constexpr int kProducerWarp = 8;
constexpr int kMmaWarp = 9;
constexpr float kRescaleThreshold = 8.0f;  // log2 units

// shared memory map (offsets from a 1024-byte aligned base)
constexpr uint32_t kSmemQ = 0;                                // 2 x 32 KB
constexpr uint32_t kSmemKV = 2 * kTileBytes;                  // kStages x 32 KB
constexpr uint32_t kSmemBar = kSmemKV + kStages * kTileBytes; // barriers
constexpr uint32_t kBarQFull = 0;
constexpr uint32_t kBarKVFull = 8;                    // kStages
constexpr uint32_t kBarKVEmpty = kBarKVFull + 8 * kStages;
constexpr uint32_t kBarSFull = kBarKVEmpty + 8 * kStages;  // 2
constexpr uint32_t kBarPFull = kBarSFull + 16;             // 2 tiles x 2 halves (keys 0-63, 64-127)
constexpr uint32_t kBarOFull = kBarPFull + 32;             // 2
constexpr uint32_t kSmemTmemPtr = kBarOFull + 16;
constexpr uint32_t kSmemAbort = kSmemTmemPtr + 4;
constexpr uint32_t kSmemUsed = kSmemBar + 256;
constexpr uint32_t kSmemBytes = kSmemUsed + 1024;  // slack for manual 1024-byte alignment

struct FwdKernelParams {
  uint16_t* out;  // bf16 or f16 bits
  float* lse;
  float* debug;
  const int32_t* cu_q;
  const int32_t* cu_k;
  uint32_t* status;
  int64_t o_batch_stride, o_head_stride, o_row_stride;
  int seqlen_q, seqlen_k, total_q, heads_q, kv_group;
  int num_m_blocks, num_bh, heads_per_wave;  // tile scheduler, see tile_coords()
  float scale_log2;
  int is_causal;
};

// Debug builds of the kernel time-stamp pipeline events of one CTA (the heaviest tile of
// batch 0, head 0) into the debug buffer: [role 0..2][iteration 0..23][event 0..7] floats of
// SM cycles since the CTA's set-up barrier, after the 2*128*260 per-row dump.
constexpr int kStampBase = 2 * 128 * 260;
#define SDPA_STAMP(role, iter, ev)                                                              \
  do {                                                                                          \
    if (kDebug && stamp_on && (iter) < 24)                                                      \
      p.debug[kStampBase + ((role) * 24 + (iter)) * 8 + (ev)] = static_cast<float>(clock64() - t_start); \
  } while (0)

template <bool kF16>
constexpr uint32_t kIdescQK = umma_idesc_16(kBlockM, kBlockN, false, false, kF16);
template <int kD, bool kF16>
constexpr uint32_t kIdescPV = umma_idesc_16(kBlockM, kD, false, true, kF16);

template <int kD, bool kF16>
__device__ __forceinline__ void issue_qk(uint32_t t_s, uint32_t q_smem, uint32_t k_smem) {
  const uint32_t a_lo = umma_desc_lo_kmajor(q_smem);
  const uint32_t b_lo = umma_desc_lo_kmajor(k_smem);
  umma_ss_lo<kIdescQK<kF16>, false>(t_s, a_lo, b_lo);
#pragma unroll
  for (int ks = 1; ks < kD / 16; ++ks) {
    const uint32_t off = ((ks >> 2) * kHalfBytes + (ks & 3) * 32) >> 4;
    umma_ss_lo<kIdescQK<kF16>, true>(t_s, a_lo + off, b_lo + off);
  }
}

// O_t (+)= P_t V for keys [64*half, 64*half + 64) of the block: four K = 16 steps
template <int kD, bool kF16>
__device__ __forceinline__ void issue_pv_half(uint32_t t_o, uint32_t t_p, uint32_t v_smem, int half,
                                              bool accumulate) {
  const uint32_t b_lo = umma_desc_lo_mnmajor(v_smem, kHalfBytes);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int ks = half * 4 + i;
    umma_ts_lo<kIdescPV<kD, kF16>>(t_o, t_p + ks * 8, b_lo + ks * (2048 >> 4), (accumulate || ks > 0) ? 1u : 0u);
  }
}

template <bool kDebug, int kD, bool kF16>
__global__ void __launch_bounds__(kNumThreads, 1)
fwd_prefill_kernel(const __grid_constant__ CUtensorMap tm_q,
                   const __grid_constant__ CUtensorMap tm_k,
                   const __grid_constant__ CUtensorMap tm_v, const FwdKernelParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw_addr);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // Tile order. (batch, head) pairs are taken in groups of `heads_per_wave` whose K/V fit
  // L2 together; inside a group the 256-row tiles go heaviest first (largest m_block, i.e.
  // most causal key blocks) across all its heads, so each group - and the whole grid - ends
  // on its lightest tiles instead of on one long straggler.
  int b, h, m_block;
  {
    const int per_group = p.heads_per_wave * p.num_m_blocks;
    const int grp = blockIdx.x / per_group;
    const int w = blockIdx.x - grp * per_group;
    const int size = min(p.heads_per_wave, p.num_bh - grp * p.heads_per_wave);
    const int rank = w / size;
    const int bh = grp * p.heads_per_wave + (w - rank * size);
    if (rank >= p.num_m_blocks) return;  // padding slots of a short last group
    m_block = p.num_m_blocks - 1 - rank;
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
  const int m0 = m_block * (2 * kBlockM);
  if (m0 >= len_q) return;

  const int causal_off = len_k - len_q;  // bottom-right alignment
  int nblk[2];
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    const int row_lo = m0 + t * kBlockM;
    int vis_end = len_k;
    if (p.is_causal) vis_end = min(len_k, row_lo + kBlockM + causal_off);
    nblk[t] = (row_lo < len_q && vis_end > 0) ? (vis_end + kBlockN - 1) / kBlockN : 0;
  }
  const int n_iter = max(nblk[0], nblk[1]);

  const uint32_t bar = base + kSmemBar;
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(smem + kSmemBar + kSmemAbort);
  volatile uint32_t* tmem_ptr_smem = reinterpret_cast<volatile uint32_t*>(smem + kSmemBar + kSmemTmemPtr);

  if (threadIdx.x == 0) {
    mbar_init(bar + kBarQFull, 1);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(bar + kBarKVFull + 8 * s, 1);
      mbar_init(bar + kBarKVEmpty + 8 * s, 1);
    }
    for (int t = 0; t < 2; ++t) {
      mbar_init(bar + kBarSFull + 8 * t, 1);
      mbar_init(bar + kBarPFull + 16 * t, 4);  // one arrival per softmax warp
      mbar_init(bar + kBarPFull + 16 * t + 8, 4);
      mbar_init(bar + kBarOFull + 8 * t, 1);
    }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 0) {
    __syncwarp();
    tmem_alloc(base + kSmemBar + kSmemTmemPtr, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_ptr_smem;
  const long long t_start = kDebug ? clock64() : 0;
  const bool stamp_cta = kDebug && p.debug != nullptr && m_block == p.num_m_blocks - 1 && h == 0 && b == 0;

  if (warp >= 8) {
    reg_decrease<40>();
  if (warp == kProducerWarp) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0 && n_iter > 0) {
      tma_prefetch_desc(&tm_q);
      tma_prefetch_desc(&tm_k);
      tma_prefetch_desc(&tm_v);
      const int hk = h / p.kv_group;
      constexpr uint32_t kLoadBytes = kBlockN * kD * 2;  // bytes one Q/K/V tile brings in
      mbar_arrive_expect_tx(bar + kBarQFull, 2 * kLoadBytes);
#pragma unroll
      for (int t = 0; t < 2; ++t) {
        const uint32_t dst = base + kSmemQ + t * kTileBytes;
        tma_load_4d(dst, &tm_q, bar + kBarQFull, 0, q_off + m0 + t * kBlockM, h, bcoord);
        if (kD > 64)
          tma_load_4d(dst + kHalfBytes, &tm_q, bar + kBarQFull, 64, q_off + m0 + t * kBlockM, h, bcoord);
      }
      for (int i = 0; i < 2 * n_iter; ++i) {  // ring item i: K(i/2) if even, V(i/2) if odd
        const int s = i % kStages;
        const uint32_t use = static_cast<uint32_t>(i / kStages);
        if (!mbar_wait(bar + kBarKVEmpty + 8 * s, (use & 1u) ^ 1u, abort_flag)) break;
        const uint32_t full = bar + kBarKVFull + 8 * s;
        const uint32_t dst = base + kSmemKV + s * kTileBytes;
        const CUtensorMap* tm = (i & 1) ? &tm_v : &tm_k;
        const int row = k_off + (i >> 1) * kBlockN;
        mbar_arrive_expect_tx(full, kLoadBytes);
        tma_load_4d(dst, tm, full, 0, row, hk, bcoord);
        if (kD > 64) tma_load_4d(dst + kHalfBytes, tm, full, 64, row, hk, bcoord);
      }
    }
  } else if (warp == kMmaWarp) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0 && n_iter > 0) {
      const uint32_t q_smem[2] = {base + kSmemQ, base + kSmemQ + kTileBytes};
      const uint32_t t_s[2] = {tmem_base, tmem_base + 128};
      const uint32_t t_o[2] = {tmem_base + 256, tmem_base + 384};
      bool ok = mbar_wait(bar + kBarQFull, 0, abort_flag);
      // ring item 0 = K(0)
      ok = ok && mbar_wait(bar + kBarKVFull, 0, abort_flag);
      if (ok) {
        tc_fence_after_sync();
#pragma unroll
        for (int t = 0; t < 2; ++t) {
          if (nblk[t] > 0) {
            issue_qk<kD, kF16>(t_s[t], q_smem[t], base + kSmemKV);
            umma_commit(bar + kBarSFull + 8 * t);
          }
        }
        umma_commit(bar + kBarKVEmpty);
      }
      for (int j = 0; ok && j < n_iter; ++j) {
        const int iv = 2 * j + 1;  // ring item of V(j)
        const int ik = 2 * j + 2;  // ring item of K(j+1)
        const int sv = iv % kStages, sk = ik % kStages;
        const uint32_t v_smem = base + kSmemKV + sv * kTileBytes;
        const uint32_t k_smem = base + kSmemKV + sk * kTileBytes;
        const bool more = (j + 1 < n_iter);
        ok = mbar_wait(bar + kBarKVFull + 8 * sv, (iv / kStages) & 1, abort_flag);
        if (!ok) break;
        const bool stamp_on = stamp_cta;
        SDPA_STAMP(2, j, 0);
        bool k_ready = false;
#pragma unroll
        for (int t = 0; t < 2; ++t) {
          if (j < nblk[t]) {
            // P arrives in two halves so the first four MMAs overlap the second half's exponentials
            ok = mbar_wait(bar + kBarPFull + 16 * t, j & 1, abort_flag);
            if (!ok) break;
            SDPA_STAMP(2, j, 1 + 3 * t);
            tc_fence_after_sync();
            issue_pv_half<kD, kF16>(t_o[t], t_s[t], v_smem, 0, j > 0);
            ok = mbar_wait(bar + kBarPFull + 16 * t + 8, j & 1, abort_flag);
            if (!ok) break;
            if (t == 0) SDPA_STAMP(2, j, 7);
            tc_fence_after_sync();
            issue_pv_half<kD, kF16>(t_o[t], t_s[t], v_smem, 1, true);
            umma_commit(bar + kBarOFull + 8 * t);
          }
          if (t == 1) umma_commit(bar + kBarKVEmpty + 8 * sv);
          if (more && !k_ready) {
            ok = mbar_wait(bar + kBarKVFull + 8 * sk, (ik / kStages) & 1, abort_flag);
            if (!ok) break;
            tc_fence_after_sync();
            k_ready = true;
          }
          SDPA_STAMP(2, j, 2 + 3 * t);
          if (j + 1 < nblk[t]) {
            issue_qk<kD, kF16>(t_s[t], q_smem[t], k_smem);
            umma_commit(bar + kBarSFull + 8 * t);
          }
          SDPA_STAMP(2, j, 3 + 3 * t);
          if (t == 1 && more) umma_commit(bar + kBarKVEmpty + 8 * sk);
        }
      }
    }
  }
  } else {
    // ------------------------------------------------------------------ softmax + epilogue
    reg_increase<232>();
    const int t = warp >> 2;
    const int row_in_tile = (warp & 3) * 32 + lane;
    const int row_lo = m0 + t * kBlockM;
    const int row = row_lo + row_in_tile;
    const uint32_t lane_base = tmem_base + (static_cast<uint32_t>((warp & 3) * 32) << 16);
    const uint32_t t_s = lane_base + t * 128;
    const uint32_t t_o = lane_base + 256 + t * 128;
    const uint32_t bar_s = bar + kBarSFull + 8 * t;
    const uint32_t bar_p = bar + kBarPFull + 16 * t;
    const uint32_t bar_o = bar + kBarOFull + 8 * t;
    const float c = p.scale_log2;
    const float neg_inf = -INFINITY;
    const int my_blocks = nblk[t];
    // keys at index >= col_limit are invisible to this row
    const int col_limit = p.is_causal ? min(len_k, row + causal_off + 1) : len_k;

    float m_run = neg_inf;
    float l_run = 0.f;
    bool ok = true;

    for (int j = 0; j < my_blocks; ++j) {
      const int n0 = j * kBlockN;
      // warp-uniform, because the arrivals below are made by one lane on behalf of its warp
      ok = __all_sync(0xffffffffu, mbar_wait(bar_s, j & 1, abort_flag));
      if (!ok) break;
      const bool stamp_on = stamp_cta && row_in_tile == 0;
      SDPA_STAMP(t, j, 0);
      tc_fence_after_sync();

      float s[kBlockN];
      {
        uint32_t r[kBlockN];
        tmem_ld_x32_at<0>(t_s, r);
        tmem_ld_x32_at<32>(t_s + 32, r);
        tmem_ld_x32_at<64>(t_s + 64, r);
        tmem_ld_x32_at<96>(t_s + 96, r);
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < kBlockN; ++i) s[i] = __uint_as_float(r[i]);
      }
      SDPA_STAMP(t, j, 1);
      if (kDebug) {
        if (p.debug != nullptr && j == 0 && m_block == 0 && h == 0 && b == 0) {
          float* d = p.debug + (t * kBlockM + row_in_tile) * 260;
          for (int i = 0; i < kBlockN; ++i) d[i] = s[i];
        }
      }
      const bool need_mask =
          (n0 + kBlockN > len_k) || (p.is_causal && n0 + kBlockN > row_lo + causal_off + 1);
      if (need_mask) {
        const int lim = col_limit - n0;
#pragma unroll
        for (int i = 0; i < kBlockN; ++i) s[i] = (i < lim) ? s[i] : neg_inf;
      }
      float mx0 = neg_inf, mx1 = neg_inf, mx2 = neg_inf, mx3 = neg_inf;
#pragma unroll
      for (int i = 0; i < kBlockN; i += 8) {
        mx0 = max3(mx0, s[i], s[i + 1]);
        mx1 = max3(mx1, s[i + 2], s[i + 3]);
        mx2 = max3(mx2, s[i + 4], s[i + 5]);
        mx3 = max3(mx3, s[i + 6], s[i + 7]);
      }
      const float m_blk = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * c;
      const float m_new = fmaxf(m_run, m_blk);
      SDPA_STAMP(t, j, 2);
      if (j == 0) {
        m_run = m_new;
      } else {
        const bool grow = (m_new - m_run) > kRescaleThreshold;  // false for NaN (-inf - -inf)
        if (__any_sync(0xffffffffu, grow)) {
          const float alpha = (m_new == neg_inf) ? 1.f : ex2_approx(m_run - m_new);
          m_run = m_new;
          l_run *= alpha;
          // O_t still receives PV(j-1); wait for it before touching the accumulator
          ok = __all_sync(0xffffffffu, mbar_wait(bar_o, (j - 1) & 1, abort_flag));
          if (!ok) break;
          tc_fence_after_sync();
#pragma unroll
          for (int cc = 0; cc < kD / 32; ++cc) {
            uint32_t r[32];
            tmem_ld_x32(t_o + cc * 32, r);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
            tmem_st_x32(t_o + cc * 32, r);
          }
        }
      }
      const float m_use = (m_run == neg_inf) ? 0.f : m_run;
      const float neg_m = -m_use;
      const float2 c2 = make_float2(c, c);
      const float2 nm2 = make_float2(neg_m, neg_m);
      float2 la = make_float2(0.f, 0.f), lb = make_float2(0.f, 0.f);
#pragma unroll
      for (int cc = 0; cc < 8; ++cc) {
        uint32_t pk[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float2 x = fma2(make_float2(s[cc * 16 + 2 * i], s[cc * 16 + 2 * i + 1]), c2, nm2);
          const float2 pr = make_float2(ex2_approx(x.x), ex2_approx(x.y));
          if (i & 1) lb = add2(lb, pr); else la = add2(la, pr);
          pk[i] = pack_16x2<kF16>(pr.x, pr.y);
        }
        if (cc == 4) {
          // keys 0-63 of P were stored one chunk of arithmetic ago, so this wait is short:
          // let the MMA warp start on them while the rest of the row is exponentiated
          tmem_wait_st();
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_p);
        }
        // P_t overwrites the front of S_t: 8 columns = 16 keys per store
        asm volatile(
            "tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
            ::"r"(t_s + cc * 8), "r"(pk[0]), "r"(pk[1]), "r"(pk[2]), "r"(pk[3]), "r"(pk[4]),
            "r"(pk[5]), "r"(pk[6]), "r"(pk[7])
            : "memory");
      }
      l_run += (la.x + la.y) + (lb.x + lb.y);
      SDPA_STAMP(t, j, 3);
      tmem_wait_st();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_p + 8);
      SDPA_STAMP(t, j, 4);
    }

    // ---- epilogue: O / l -> 16-bit, LSE
    if (ok && my_blocks > 0) ok = mbar_wait(bar_o, (my_blocks - 1) & 1, abort_flag);
    if (ok && row_lo < len_q) {
      tc_fence_after_sync();
      const bool valid = row < len_q;
      const float inv_l = (l_run > 0.f) ? 1.f / l_run : 0.f;
      uint16_t* orow;
      float* lse_ptr;
      if (p.cu_q != nullptr) {
        orow = p.out + static_cast<int64_t>(q_off + row) * p.o_row_stride + h * p.o_head_stride;
        lse_ptr = p.lse + static_cast<int64_t>(h) * p.total_q + q_off + row;
      } else {
        orow = p.out + b * p.o_batch_stride + h * p.o_head_stride +
               static_cast<int64_t>(row) * p.o_row_stride;
        lse_ptr = p.lse + (static_cast<int64_t>(b) * p.heads_q + h) * p.seqlen_q + row;
      }
#pragma unroll
      for (int cc = 0; cc < kD / 32; ++cc) {
        uint32_t r[32];
        if (my_blocks > 0) {
          tmem_ld_x32(t_o + cc * 32, r);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] = 0u;
        }
        if (kDebug) {
          if (p.debug != nullptr && m_block == 0 && h == 0 && b == 0) {
            float* d = p.debug + (t * kBlockM + row_in_tile) * 260 + 128 + cc * 32;
            for (int i = 0; i < 32; ++i) d[i] = __uint_as_float(r[i]);
          }
        }
        uint32_t w[16];
#pragma unroll
        for (int i = 0; i < 16; ++i)
          w[i] = pack_16x2<kF16>(__uint_as_float(r[2 * i]) * inv_l, __uint_as_float(r[2 * i + 1]) * inv_l);
        if (valid) {
          uint4* dst = reinterpret_cast<uint4*>(orow + cc * 32);
#pragma unroll
          for (int i = 0; i < 4; ++i) dst[i] = make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]);
        }
      }
      if (kDebug) {
        if (p.debug != nullptr && m_block == 0 && h == 0 && b == 0) {
          float* d = p.debug + (t * kBlockM + row_in_tile) * 260 + 256;
          d[0] = m_run;
          d[1] = l_run;
        }
      }
      if (valid) {
        const float kLn2 = 0.6931471805599453f;
        *lse_ptr = (l_run > 0.f) ? (m_run + log2f(l_run)) * kLn2 : INFINITY;
      }
    }
  }

  // ------------------------------------------------------------------ tear-down
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
  if (threadIdx.x == 0 && *abort_flag != 0) atomicExch(p.status, SDPA_B200_DEVICE_TIMEOUT);
}

}  // namespace

int launch_fwd_prefill(const sdpa_b200_params& p, void* workspace, cudaStream_t stream,
                       float* debug) {
  const bool varlen = p.cu_seqlens_q != nullptr;
  CUtensorMap tm_q, tm_k, tm_v;
  int st;
  const int64_t rows_q = varlen ? p.total_q : p.max_seqlen_q;
  const int64_t rows_k = varlen ? p.total_k : p.max_seqlen_k;
  const int64_t nb = varlen ? 1 : p.batch;
  st = make_tensor_map_16(p.dtype == SDPA_B200_F16, &tm_q, p.q, p.head_dim, rows_q, p.heads_q, nb, p.q_row_stride,
                            p.q_head_stride, p.q_batch_stride, kBlockM);
  if (st != SDPA_B200_OK) return st;
  st = make_tensor_map_16(p.dtype == SDPA_B200_F16, &tm_k, p.k, p.head_dim, rows_k, p.heads_kv, nb, p.k_row_stride,
                            p.k_head_stride, p.k_batch_stride, kBlockN);
  if (st != SDPA_B200_OK) return st;
  st = make_tensor_map_16(p.dtype == SDPA_B200_F16, &tm_v, p.v, p.head_dim, rows_k, p.heads_kv, nb, p.v_row_stride,
                            p.v_head_stride, p.v_batch_stride, kBlockN);
  if (st != SDPA_B200_OK) return st;

  FwdKernelParams kp;
  kp.out = static_cast<uint16_t*>(p.out);
  kp.lse = p.lse;
  kp.debug = debug;
  kp.cu_q = p.cu_seqlens_q;
  kp.cu_k = p.cu_seqlens_k;
  kp.status = static_cast<uint32_t*>(workspace);
  kp.o_batch_stride = p.o_batch_stride;
  kp.o_head_stride = p.o_head_stride;
  kp.o_row_stride = p.o_row_stride;
  kp.seqlen_q = p.max_seqlen_q;
  kp.seqlen_k = p.max_seqlen_k;
  kp.total_q = p.total_q;
  kp.heads_q = p.heads_q;
  kp.kv_group = p.heads_q / p.heads_kv;
  kp.scale_log2 = p.softmax_scale * 1.4426950408889634f;
  kp.is_causal = p.is_causal;

  const bool f16 = p.dtype == SDPA_B200_F16;
  auto kernel = p.head_dim == 64
                    ? (f16 ? fwd_prefill_kernel<false, 64, true> : fwd_prefill_kernel<false, 64, false>)
                    : (f16 ? fwd_prefill_kernel<false, 128, true>
                           : (debug ? fwd_prefill_kernel<true, 128, false> : fwd_prefill_kernel<false, 128, false>));
  cudaError_t err =
      cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
  if (err != cudaSuccess) {
    set_error("prefill: cudaFuncSetAttribute(%u bytes smem): %s", kSmemBytes, cudaGetErrorString(err));
    return SDPA_B200_LAUNCH_FAILED;
  }
  kp.num_m_blocks = (p.max_seqlen_q + 2 * kBlockM - 1) / (2 * kBlockM);
  kp.num_bh = p.batch * p.heads_q;
  {
    // K+V bytes one query head streams, shared by the heads of its GQA group
    const double kv_bytes = 2.0 * p.max_seqlen_k * p.head_dim * 2 / kp.kv_group;
    int hpw = static_cast<int>((48.0 * 1024 * 1024) / kv_bytes);
    hpw = hpw < 1 ? 1 : (hpw > 32 ? 32 : hpw);
    if (hpw > kp.num_bh) hpw = kp.num_bh;
    kp.heads_per_wave = hpw;
  }
  const int groups = (kp.num_bh + kp.heads_per_wave - 1) / kp.heads_per_wave;
  dim3 grid(groups * kp.heads_per_wave * kp.num_m_blocks, 1, 1);
  kernel<<<grid, kNumThreads, kSmemBytes, stream>>>(tm_q, tm_k, tm_v, kp);
  err = cudaGetLastError();
  if (err != cudaSuccess) {
    set_error("prefill: launch failed: %s", cudaGetErrorString(err));
    return SDPA_B200_LAUNCH_FAILED;
  }
  count_launch();
  return SDPA_B200_OK;
}

}  // namespace sdpa_b200
