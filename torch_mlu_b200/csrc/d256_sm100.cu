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
};

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

template <bool kF16>
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
    for (int j = 0; j < n_blocks; ++j) {
      const uint32_t t_s = t_s0 + (j & 1) * 64 + lane_base;
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
      const float inv_l = (l_run > 0.f) ? 1.f / l_run : 0.f;
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

// heads per group so that the streamed K + V of a group stay within ~48 MB of L2
int heads_per_wave_for(double bytes_per_head, int num_bh) {
  int hpw = static_cast<int>((48.0 * 1024 * 1024) / bytes_per_head);
  hpw = hpw < 1 ? 1 : (hpw > 32 ? 32 : hpw);
  return hpw > num_bh ? num_bh : hpw;
}

}  // namespace

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
  auto kernel = f16 ? fwd_d256_kernel<true> : fwd_d256_kernel<false>;
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
