// Prefill / forward attention kernel for sm_100a.
//
// Replaces the device work behind mha_varlen_fwd -> cnnlFlashAttentionForward_v2
// (torch_mlu/csrc/aten/operators/cnnl/internal/FlashAttention_internal.cpp:231-258):
//   O = softmax(scale * Q K^T + causal mask) V,  LSE = logsumexp(scale * Q K^T)
// for bf16 or f16 Q/K/V with head_dim <= 128 (a multiple of 8), dense or packed-varlen, GQA by head
// broadcast. The kernel is built for 64 and 128 columns; other head dims run in the next larger one:
// TMA loads fill the missing columns with zeros and TMA stores clip them. Two optional extras are separate
// template instances, so that the plain kernel pays nothing for them: dropout (kDrop: keep bits per (query,
// key) pair from dropout_mask.cu) and the additive bias of the memory-efficient operators (kBias:
// softmax(scale * Q K^T + bias), mem_eff_fwd, FlashAttention_internal.cpp:485-690).
//
// A work unit is 256 query rows of one (batch, head): two 128-row Q tiles. One persistent CTA per SM
// walks the unit list; its barriers, TMEM and K/V ring live across units, so the next unit's loads
// and first QK^T overlap this unit's epilogue. Roles:
//   warps 0-3  softmax warpgroup for Q tile 0  (thread = one query row = one TMEM lane)
//   warps 4-7  softmax warpgroup for Q tile 1
//   warp  8    TMA producer: Q once, then K(j), V(j) tiles into a 4-stage 32 KB ring
//   warp  9    MMA issuer: S_t = Q_t K^T and O_t += P_t V on tcgen05, accumulators in TMEM
//   warp  10   unit scheduler (see below); warp 11 idle. They complete the third warpgroup so it can hand its registers to the
//              softmax warpgroups (setmaxnreg), which hold a whole 128-column S row per thread
// TMEM (512 columns): S0 [0,128) S1 [128,256) O0 [256,384) O1 [384,512); P_t (16-bit, 64
// columns) overwrites the front of S_t once the softmax thread holds the whole S row in
// registers. The two Q tiles ping-pong: while one warpgroup exponentiates, the tensor core
// runs the other tile's GEMMs. Online softmax works in the log2 domain; O is rescaled lazily
// (only when a row maximum grows by more than 2^8), by the softmax thread that owns the row.
#include <cuda_bf16.h>

#include <cstdlib>
#include <type_traits>

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
constexpr int kNumThreads = 384;  // 3 warpgroups; warp 11 idle
constexpr int kProducerWarp = 8;
constexpr int kMmaWarp = 9;
constexpr int kSchedulerWarp = 10;
constexpr float kRescaleThreshold = 8.0f;  // log2 units
// Register hand-over (setmaxnreg). The kernel is compiled for 65536 / 384 -> 168 registers per thread;
// the 4 non-softmax warps shrink to kRegsOther and the 8 softmax warps grow to kRegsSoftmax. The
// increase waits - without a time limit - until the pool holds enough registers, so what the
// shrinking warps release must cover what the growing warps take.
constexpr int kRegsLaunch = 168;
constexpr int kRegsOther = 56;
constexpr int kRegsSoftmax = 224;
static_assert((kRegsSoftmax - kRegsLaunch) * 8 <= (kRegsLaunch - kRegsOther) * 4,
              "setmaxnreg.inc would wait forever: the softmax warps ask for more than the others release");

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
constexpr uint32_t kBarOFree = kBarOFull + 16;             // 2: the epilogue has read O_t (persistent loop)
constexpr uint32_t kBarQFree = kBarOFree + 16;             // the unit's last QK^T has read the Q tiles
constexpr uint32_t kBarUnitFull = kBarQFree + 8;           // kUnitRing: the scheduler has written the entry
constexpr uint32_t kBarUnitEmpty = kBarUnitFull + 16;      // kUnitRing: every reader has copied the entry
constexpr uint32_t kBarStageFree = kBarUnitEmpty + 16;     // 2: the warpgroup's staging buffer may be rewritten
constexpr uint32_t kBarStageFull = kBarStageFree + 16;     // 2: all four warps have written their rows
constexpr uint32_t kSmemTmemPtr = kBarStageFull + 16;
constexpr uint32_t kSmemAbort = kSmemTmemPtr + 4;
constexpr uint32_t kSmemUnits = 256;  // offset of the Unit ring from kSmemBar (2 x 64 bytes)
constexpr uint32_t kSmemStash = 512;   // per softmax warp: the unit's coordinates for the epilogue (8 x 32 bytes)
constexpr uint32_t kSmemStage = kSmemBar + 1024;  // 2 x 16 KB: one 64-column half of an O tile per softmax warpgroup
constexpr uint32_t kStageBytes = kBlockM * 128;
constexpr uint32_t kSmemUsed = kSmemStage + 2 * kStageBytes;
constexpr uint32_t kSmemBytes = kSmemUsed + 1024;  // slack for manual 1024-byte alignment

struct FwdKernelParams {
  uint16_t* out;  // bf16 or f16 bits
  float* lse;
  const int32_t* cu_q;
  const int32_t* cu_k;
  uint32_t* status;
  uint32_t* unit_counter;  // zeroed by the caller before the launch
  int64_t o_batch_stride, o_head_stride, o_row_stride;
  int seqlen_q, seqlen_k, total_q, heads_q, kv_group;
  int head_dim;  // <= kD: the real row length, for the paths that write rows without TMA
  // dropout (kernels built with kDrop): one keep bit per (query, key) pair, see dropout_mask.cu
  const uint32_t* keep_rows;  // dense [batch*heads_q][lq_pad][lk_words]; packed [heads_q][total_q + 128][lk_words]
  int lq_pad, lk_words;       // lq_pad: rows per leading index (dense: padded seqlen_q; packed: total_q + 128)
  float keep_scale;  // 1 / (1 - dropout_p), applied with the final 1 / l
  // additive bias (kernels built with kBias): softmax(scale * Q K^T + bias), bias in the tensors' 16-bit type,
  // element strides for (batch, head, query row), 0 for a broadcast dimension; the key stride is 1
  const uint16_t* bias;
  int64_t bias_batch_stride, bias_head_stride, bias_row_stride;
  float inv_scale;  // 1 / softmax_scale: the bias joins the raw scores as bias / scale
  int num_m_blocks, num_bh, heads_per_wave, num_slots;  // work-unit order, see decode_unit()
  float scale_log2;
  int is_causal;
#ifdef SDPA_FWD_STAMPS
  float* stamps;  // [role 4][unit 16][event 8] SM cycles since CTA start, CTA 0 only
#endif
};

// Profiling builds (-DSDPA_FWD_STAMPS) time-stamp events of CTA 0's first units; role 0/1 = lane 0 of
// the first warp of each softmax warpgroup, 2 = MMA issuer, 3 = TMA producer.
#ifdef SDPA_FWD_STAMPS
#define FWD_STAMP(role, unit, ev)                                                                  \
  do {                                                                                             \
    if (p.stamps != nullptr && blockIdx.x == 0 && (unit) < 16)                                     \
      p.stamps[((role) * 16 + (unit)) * 8 + (ev)] = static_cast<float>(clock64() - t_start);        \
  } while (0)
#else
#define FWD_STAMP(role, unit, ev) do {} while (0)
#endif

template <bool kF16>
constexpr uint32_t kIdescQK = umma_idesc_16(kBlockM, kBlockN, false, false, kF16);
template <int kD, bool kF16>
constexpr uint32_t kIdescPV = umma_idesc_16(kBlockM, kD, false, true, kF16);

// byte offset >> 4 of K step ks inside a K-major 128-byte-swizzled tile (two 64-column halves)
__host__ __device__ constexpr uint32_t kmajor_step(int ks) { return ((ks >> 2) * kHalfBytes + (ks & 3) * 32) >> 4; }

template <int kD, bool kF16, int kS = 0>
__device__ __forceinline__ void issue_qk(uint32_t t_s, uint32_t a_lo, uint32_t b_lo) {
  // a_lo / b_lo: low descriptor words of the Q tile and the K tile (umma_desc_lo_kmajor)
  umma_ss_off<kIdescQK<kF16>, kmajor_step(kS), kmajor_step(kS), (kS > 0)>(t_s, a_lo, b_lo);
  if constexpr (kS + 1 < kD / 16) issue_qk<kD, kF16, kS + 1>(t_s, a_lo, b_lo);
}

// O_t (+)= P_t V for keys [64*half, 64*half + 64) of the block: four K = 16 steps. b_lo is the low
// descriptor word of the V tile read MN-major (umma_desc_lo_mnmajor).
template <int kD, bool kF16, int kHalf, int kI = 0>
__device__ __forceinline__ void issue_pv_half(uint32_t t_o, uint32_t t_p, uint32_t b_lo, bool accumulate) {
  constexpr int ks = kHalf * 4 + kI;
  umma_ts_off<kIdescPV<kD, kF16>, ks * 8, ks * (2048 >> 4)>(t_o, t_p, b_lo, (accumulate || ks > 0) ? 1u : 0u);
  if constexpr (kI + 1 < 4) issue_pv_half<kD, kF16, kHalf, kI + 1>(t_o, t_p, b_lo, accumulate);
}

// One work unit: 256 query rows (two 128-row tiles) of one (batch, head).
struct Unit {
  int b, h, hk, m0, q_off, k_off, len_q, len_k, bcoord, causal_off;
  int nblk[2];  // key blocks each Q tile visits
  int n_iter;
  int done;     // no unit left: the roles leave their loops
  int pad[2];   // 64 bytes: one shared-memory ring entry
};
static_assert(sizeof(Unit) == 64, "Unit is copied through shared memory as four 16-byte words");

// Unit order. (batch, head) pairs are taken in groups of `heads_per_wave` whose K/V fit L2
// together; inside a group the 256-row units go heaviest first (largest m_block, i.e. most causal
// key blocks) across all its heads. Returns false for padding slots and units without rows.
__device__ __forceinline__ bool decode_unit(const FwdKernelParams& p, int slot, Unit& u) {
  const int per_group = p.heads_per_wave * p.num_m_blocks;
  const int grp = slot / per_group;
  const int w = slot - grp * per_group;
  const int size = min(p.heads_per_wave, p.num_bh - grp * p.heads_per_wave);
  const int rank = w / size;
  const int bh = grp * p.heads_per_wave + (w - rank * size);
  if (rank >= p.num_m_blocks) return false;  // padding slots of a short last group
  const int m_block = p.num_m_blocks - 1 - rank;
  u.b = bh / p.heads_q;
  u.h = bh - u.b * p.heads_q;
  u.hk = u.h / p.kv_group;
  u.q_off = 0;
  u.k_off = 0;
  u.len_q = p.seqlen_q;
  u.len_k = p.seqlen_k;
  u.bcoord = u.b;
  if (p.cu_q != nullptr) {
    u.q_off = p.cu_q[u.b];
    u.len_q = p.cu_q[u.b + 1] - u.q_off;
    u.k_off = p.cu_k[u.b];
    u.len_k = p.cu_k[u.b + 1] - u.k_off;
    u.bcoord = 0;
  }
  u.m0 = m_block * (2 * kBlockM);
  if (u.m0 >= u.len_q) return false;
  u.causal_off = u.len_k - u.len_q;  // bottom-right alignment
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    const int row_lo = u.m0 + t * kBlockM;
    int vis_end = u.len_k;
    if (p.is_causal) vis_end = min(u.len_k, row_lo + kBlockM + u.causal_off);
    u.nblk[t] = (row_lo < u.len_q && vis_end > 0) ? (vis_end + kBlockN - 1) / kBlockN : 0;
  }
  u.n_iter = max(u.nblk[0], u.nblk[1]);
  u.done = 0;
  return true;
}

// Persistent kernel: gridDim.x CTAs (one per SM) take units off a global counter in list order, which
// balances the uneven causal units the way the hardware block scheduler would. Warp 10 is the unit
// scheduler: it claims the next slot, decodes it (integer divisions, cu_seqlens loads) off everyone's
// critical path and publishes the Unit through a two-entry shared-memory ring; the producer, the MMA
// issuer and the eight softmax warps each copy the entry and release it at once, so the scheduler
// runs one unit ahead. Barriers, TMEM and the K/V ring live across units; every role keeps running use
// counts, so the loads, the first QK^T and the softmax of the next unit start while this unit's
// epilogue runs.
constexpr int kUnitRing = 2;
constexpr uint32_t kUnitReaders = 10;  // producer + issuer + 8 softmax warps

// Copies ring entry (n mod kUnitRing) into `u` and releases it. All lanes of the calling warp (or its
// single active lane) take part; returns false on time-out. `n` counts the entries this role has read.
__device__ __forceinline__ bool read_unit(uint8_t* smem, uint32_t bar, uint32_t n, bool whole_warp,
                                          volatile uint32_t* abort_flag, Unit& u) {
  const uint32_t e = n % kUnitRing;
  bool ok = mbar_wait(bar + kBarUnitFull + 8 * e, (n / kUnitRing) & 1, abort_flag);
  if (whole_warp) ok = __all_sync(0xffffffffu, ok);
  if (!ok) return false;
  const uint4* src = reinterpret_cast<const uint4*>(smem + kSmemBar + kSmemUnits + e * sizeof(Unit));
  const uint4 w0 = src[0], w1 = src[1], w2 = src[2], w3 = src[3];
  u.b = w0.x; u.h = w0.y; u.hk = w0.z; u.m0 = w0.w;
  u.q_off = w1.x; u.k_off = w1.y; u.len_q = w1.z; u.len_k = w1.w;
  u.bcoord = w2.x; u.causal_off = w2.y; u.nblk[0] = w2.z; u.nblk[1] = w2.w;
  u.n_iter = w3.x; u.done = w3.y;
  if (whole_warp) {
    __syncwarp();
    if ((threadIdx.x & 31) == 0) mbar_arrive(bar + kBarUnitEmpty + 8 * e);
  } else {
    mbar_arrive(bar + kBarUnitEmpty + 8 * e);
  }
  return true;
}

// The producer needs the tile coordinates only.
__device__ __forceinline__ bool read_unit_coords(uint8_t* smem, uint32_t bar, uint32_t n, volatile uint32_t* abort_flag,
                                                 int& q_row, int& k_row, int& h, int& hk, int& bcoord, int& n_iter,
                                                 int& done) {
  const uint32_t e = n % kUnitRing;
  if (!mbar_wait(bar + kBarUnitFull + 8 * e, (n / kUnitRing) & 1, abort_flag)) return false;
  const int* w = reinterpret_cast<const int*>(smem + kSmemBar + kSmemUnits + e * sizeof(Unit));
  h = w[1];
  hk = w[2];
  q_row = w[3] + w[4];  // m0 + q_off
  k_row = w[5];
  bcoord = w[8];
  n_iter = w[12];
  done = w[13];
  mbar_arrive(bar + kBarUnitEmpty + 8 * e);
  return true;
}

// The MMA issuer only needs the block counts; it runs on few registers, so it reads nothing else.
__device__ __forceinline__ bool read_unit_counts(uint8_t* smem, uint32_t bar, uint32_t n, volatile uint32_t* abort_flag,
                                                 int& nblk0, int& nblk1, int& n_iter, int& done) {
  const uint32_t e = n % kUnitRing;
  if (!mbar_wait(bar + kBarUnitFull + 8 * e, (n / kUnitRing) & 1, abort_flag)) return false;
  const int* w = reinterpret_cast<const int*>(smem + kSmemBar + kSmemUnits + e * sizeof(Unit));
  nblk0 = w[10];
  nblk1 = w[11];
  n_iter = w[12];
  done = w[13];
  mbar_arrive(bar + kBarUnitEmpty + 8 * e);
  return true;
}

__device__ __forceinline__ void write_unit(uint8_t* smem, uint32_t e, const Unit& u) {
  uint4* dst = reinterpret_cast<uint4*>(smem + kSmemBar + kSmemUnits + e * sizeof(Unit));
  dst[0] = make_uint4(u.b, u.h, u.hk, u.m0);
  dst[1] = make_uint4(u.q_off, u.k_off, u.len_q, u.len_k);
  dst[2] = make_uint4(u.bcoord, u.causal_off, u.nblk[0], u.nblk[1]);
  dst[3] = make_uint4(u.n_iter, u.done, 0, 0);
}

// both halves of a packed 16-bit pair survive or die by two keep bits (bit 0 -> low half)
__device__ __forceinline__ uint32_t keep_pair_mask(uint32_t two_bits) {
  return ((two_bits & 1u) ? 0x0000ffffu : 0u) | ((two_bits & 2u) ? 0xffff0000u : 0u);
}

template <int kD, bool kF16, bool kDrop, bool kBias>
__global__ void __launch_bounds__(kNumThreads, 1)
fwd_prefill_kernel(const __grid_constant__ CUtensorMap tm_q,
                   const __grid_constant__ CUtensorMap tm_k,
                   const __grid_constant__ CUtensorMap tm_v,
                   const __grid_constant__ CUtensorMap tm_o, const FwdKernelParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw_addr);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t bar = base + kSmemBar;
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(smem + kSmemBar + kSmemAbort);
  volatile uint32_t* tmem_ptr_smem = reinterpret_cast<volatile uint32_t*>(smem + kSmemBar + kSmemTmemPtr);

  if (threadIdx.x == 0) {
    mbar_init(bar + kBarQFull, 1);
    mbar_init(bar + kBarQFree, 1);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(bar + kBarKVFull + 8 * s, 1);
      mbar_init(bar + kBarKVEmpty + 8 * s, 1);
    }
    for (int t = 0; t < 2; ++t) {
      mbar_init(bar + kBarSFull + 8 * t, 1);
      mbar_init(bar + kBarPFull + 16 * t, 4);  // one arrival per softmax warp
      mbar_init(bar + kBarPFull + 16 * t + 8, 4);
      mbar_init(bar + kBarOFull + 8 * t, 1);
      mbar_init(bar + kBarOFree + 8 * t, 4);
      mbar_init(bar + kBarStageFree + 8 * t, 1);
      mbar_init(bar + kBarStageFull + 8 * t, 4);
    }
    for (int e = 0; e < kUnitRing; ++e) {
      mbar_init(bar + kBarUnitFull + 8 * e, 1);
      mbar_init(bar + kBarUnitEmpty + 8 * e, kUnitReaders);
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
#ifdef SDPA_FWD_STAMPS
  const long long t_start = clock64();
#endif

  if (warp >= 8) {
    reg_decrease<kRegsOther>();
    if (warp == kProducerWarp) {
      // ------------------------------------------------------------------ TMA producer
      if (lane == 0) {
        tma_prefetch_desc(&tm_q);
        tma_prefetch_desc(&tm_k);
        tma_prefetch_desc(&tm_v);
        constexpr uint32_t kLoadBytes = kBlockN * kD * 2;  // bytes one Q/K/V tile brings in
        uint32_t kv_cnt = 0;  // K/V tiles loaded so far (ring position)
        uint32_t ucnt = 0;    // units started so far
        bool ok = true;
        for (uint32_t n = 0; ok; ++n) {
          int q_row, k_row, h, hk, bcoord, n_iter, done;
          ok = read_unit_coords(smem, bar, n, abort_flag, q_row, k_row, h, hk, bcoord, n_iter, done);
          if (!ok || done) break;
          if (n_iter == 0) continue;
          FWD_STAMP(3, ucnt, 0);
          // the Q tiles are free once the last QK^T of the previous unit has read them
          if (ucnt > 0) ok = mbar_wait(bar + kBarQFree, (ucnt - 1) & 1, abort_flag);
          if (!ok) break;
          FWD_STAMP(3, ucnt, 1);
          mbar_arrive_expect_tx(bar + kBarQFull, 2 * kLoadBytes);
#pragma unroll
          for (int t = 0; t < 2; ++t) {
            const uint32_t dst = base + kSmemQ + t * kTileBytes;
            tma_load_4d(dst, &tm_q, bar + kBarQFull, 0, q_row + t * kBlockM, h, bcoord);
            if (kD > 64) tma_load_4d(dst + kHalfBytes, &tm_q, bar + kBarQFull, 64, q_row + t * kBlockM, h, bcoord);
          }
          for (int i = 0; i < 2 * n_iter; ++i, ++kv_cnt) {  // K(i/2) if even, V(i/2) if odd
            const uint32_t s = kv_cnt % kStages;
            const uint32_t use = kv_cnt / kStages;
            ok = mbar_wait(bar + kBarKVEmpty + 8 * s, (use & 1u) ^ 1u, abort_flag);
            if (!ok) break;
            const uint32_t full = bar + kBarKVFull + 8 * s;
            const uint32_t dst = base + kSmemKV + s * kTileBytes;
            const CUtensorMap* tm = (i & 1) ? &tm_v : &tm_k;
            const int row = k_row + (i >> 1) * kBlockN;
            mbar_arrive_expect_tx(full, kLoadBytes);
            tma_load_4d(dst, tm, full, 0, row, hk, bcoord);
            if (kD > 64) tma_load_4d(dst + kHalfBytes, tm, full, 64, row, hk, bcoord);
            if (i == 0) FWD_STAMP(3, ucnt, 2);
          }
          FWD_STAMP(3, ucnt, 3);
          ++ucnt;
        }
        drain_after_abort(abort_flag);
      }
    } else if (warp == kMmaWarp) {
      // ------------------------------------------------------------------ MMA issuer
      if (lane == 0) {
        uint32_t kv_base = 0;          // ring position of this unit's K(0)
        uint32_t ucnt = 0;             // units started so far
        uint32_t cnt0 = 0, cnt1 = 0;   // key blocks issued so far per Q tile (phase of the S/P/O barriers)
        bool ok = true;
        auto kv_full = [&](uint32_t idx) {
          return mbar_wait(bar + kBarKVFull + 8 * (idx % kStages), (idx / kStages) & 1, abort_flag);
        };
        auto kv_smem = [&](uint32_t idx) { return base + kSmemKV + (idx % kStages) * kTileBytes; };
        auto kv_release = [&](uint32_t idx) { umma_commit(bar + kBarKVEmpty + 8 * (idx % kStages)); };
        for (uint32_t n = 0; ok; ++n) {
          int nblk0, nblk1, n_iter, done;
          ok = read_unit_counts(smem, bar, n, abort_flag, nblk0, nblk1, n_iter, done);
          if (!ok || done) break;
          if (n_iter == 0) continue;
          FWD_STAMP(2, ucnt, 0);
          ok = mbar_wait(bar + kBarQFull, ucnt & 1, abort_flag);
          FWD_STAMP(2, ucnt, 1);
          ok = ok && kv_full(kv_base);
          if (!ok) break;
          tc_fence_after_sync();
          if (nblk0 > 0) {
            issue_qk<kD, kF16>(tmem_base, umma_desc_lo_kmajor(base + kSmemQ), umma_desc_lo_kmajor(kv_smem(kv_base)));
            umma_commit(bar + kBarSFull);
          }
          if (nblk1 > 0) {
            issue_qk<kD, kF16>(tmem_base + 128, umma_desc_lo_kmajor(base + kSmemQ + kTileBytes), umma_desc_lo_kmajor(kv_smem(kv_base)));
            umma_commit(bar + kBarSFull + 8);
          }
          kv_release(kv_base);
          if (n_iter == 1) umma_commit(bar + kBarQFree);
          FWD_STAMP(2, ucnt, 2);
          for (int j = 0; ok && j < n_iter; ++j) {
            const uint32_t iv = kv_base + 2 * j + 1;  // ring position of V(j)
            const uint32_t ik = kv_base + 2 * j + 2;  // ring position of K(j+1)
            const uint32_t v_smem = kv_smem(iv);
            const uint32_t k_smem = kv_smem(ik);
            const bool more = (j + 1 < n_iter);
            ok = kv_full(iv);
            if (!ok) break;
            // One Q tile's share of block j: PV(j) in two halves, then QK^T(j+1). kT is a compile-time
            // tile index, so every address below is a register, not an indexed local array.
            auto tile_step = [&](auto kT, int nblk, uint32_t cnt, bool k_known_ready) -> bool {
              constexpr int t = decltype(kT)::value;
              const uint32_t ts = tmem_base + t * 128, to = tmem_base + 256 + t * 128;
              if (j < nblk) {
                const uint32_t par = (cnt + j) & 1;
                // the first PV of a unit overwrites O_t: the previous unit's epilogue must have read it
                if (j == 0 && ucnt > 0 && !mbar_wait(bar + kBarOFree + 8 * t, (ucnt - 1) & 1, abort_flag)) return false;
                if (j == 0 && t == 0) FWD_STAMP(2, ucnt, 3);
                // P arrives in two halves so the first four MMAs overlap the second half's exponentials
                if (!mbar_wait(bar + kBarPFull + 16 * t, par, abort_flag)) return false;
                tc_fence_after_sync();
                issue_pv_half<kD, kF16, 0>(to, ts, umma_desc_lo_mnmajor(v_smem, kHalfBytes), j > 0);
                if (!mbar_wait(bar + kBarPFull + 16 * t + 8, par, abort_flag)) return false;
                tc_fence_after_sync();
                issue_pv_half<kD, kF16, 1>(to, ts, umma_desc_lo_mnmajor(v_smem, kHalfBytes), true);
                umma_commit(bar + kBarOFull + 8 * t);
              }
              if (t == 1) kv_release(iv);
              if (more && !k_known_ready) {
                if (!kv_full(ik)) return false;
                tc_fence_after_sync();
              }
              if (j + 1 < nblk) {
                issue_qk<kD, kF16>(ts, umma_desc_lo_kmajor(base + kSmemQ + t * kTileBytes), umma_desc_lo_kmajor(k_smem));
                umma_commit(bar + kBarSFull + 8 * t);
              }
              return true;
            };
            ok = tile_step(std::integral_constant<int, 0>{}, nblk0, cnt0, false) &&
                 tile_step(std::integral_constant<int, 1>{}, nblk1, cnt1, true);
            if (!ok) break;
            if (more) {
              kv_release(ik);
              if (j + 2 == n_iter) umma_commit(bar + kBarQFree);  // that was the unit's last QK^T
            }
          }
          FWD_STAMP(2, ucnt, 4);
          cnt0 += nblk0;
          cnt1 += nblk1;
          kv_base += 2 * n_iter;
          ++ucnt;
        }
      }
    } else if (warp == kSchedulerWarp) {
      // ------------------------------------------------------------------ unit scheduler
      if (lane == 0) {
        bool ok = true;
        // Claiming ahead hides the claim (atomic + decode) and lets the producer prefetch the next Q
        // tiles, but near the end of the list a unit claimed early by a busy CTA is a unit an idle CTA
        // cannot take. For the last two rounds of the grid the scheduler therefore claims late: only
        // once the last QK^T of the unit it published before has been issued (the Q-free barrier).
        bool lazy = false;
        bool last_runs = false;  // the unit published last has key blocks (and so a Q-free phase)
        uint32_t ucnt = 0;       // such units published so far
        for (uint32_t n = 0; ok; ++n) {
          const uint32_t e = n % kUnitRing;
          ok = mbar_wait(bar + kBarUnitEmpty + 8 * e, ((n / kUnitRing) & 1u) ^ 1u, abort_flag);
          if (ok && lazy && last_runs) ok = mbar_wait(bar + kBarQFree, (ucnt - 1) & 1, abort_flag);
          if (!ok) break;
          Unit u;
          u.done = 1;
          for (;;) {
            const int slot = static_cast<int>(atomicAdd(p.unit_counter, 1u));
            if (slot >= p.num_slots) break;
            if (slot >= p.num_slots - 2 * static_cast<int>(gridDim.x)) lazy = true;
            if (decode_unit(p, slot, u)) break;  // padding slots and row-less units are skipped
            u.done = 1;
          }
          last_runs = !u.done && u.n_iter > 0;
          if (last_runs) ++ucnt;
          write_unit(smem, e, u);
          mbar_arrive(bar + kBarUnitFull + 8 * e);  // release: the entry is visible to whoever sees the phase
          if (u.done) break;
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax + epilogue
    reg_increase<kRegsSoftmax>();
    const int t = warp >> 2;
    const int row_in_tile = (warp & 3) * 32 + lane;
    const uint32_t lane_base = tmem_base + (static_cast<uint32_t>((warp & 3) * 32) << 16);
    const uint32_t t_s = lane_base + t * 128;
    const uint32_t t_o = lane_base + 256 + t * 128;
    const uint32_t bar_s = bar + kBarSFull + 8 * t;
    const uint32_t bar_p = bar + kBarPFull + 16 * t;
    const uint32_t bar_o = bar + kBarOFull + 8 * t;
    const float c = p.scale_log2;
    const float neg_inf = -INFINITY;
    uint32_t cnt = 0;     // key blocks this tile has processed so far (phase of the S/P/O barriers)
    uint32_t st_cnt = 0;  // 64-column output stores this warpgroup has staged so far
    uint32_t ucnt = 0;
    bool ok = true;

    for (uint32_t n = 0; ok; ++n) {
      Unit u;
      ok = read_unit(smem, bar, n, true, abort_flag, u);
      if (!ok || u.done) break;
      // everything the block loop needs from the unit, so that `u` dies here; what only the epilogue
      // needs waits in shared memory (one slot per warp), not in registers
      const int row_lo = u.m0 + t * kBlockM;
      const int row = row_lo + row_in_tile;
      const int my_blocks = u.nblk[t];
      int* info = reinterpret_cast<int*>(smem + kSmemBar + kSmemStash) + 8 * warp;
      if (lane == 0) {
        info[0] = u.q_off;
        info[1] = u.h;
        info[2] = u.b;
        info[3] = u.len_q;
      }
      __syncwarp();
      if (u.n_iter == 0) {
        // no key is visible to any row of the unit (causal with more queries than keys): the other
        // roles skip it, the rows get out = 0 and lse = +inf
        if (row < u.len_q) {
          uint16_t* orow;
          float* lse_ptr;
          if (p.cu_q != nullptr) {
            orow = p.out + static_cast<int64_t>(u.q_off + row) * p.o_row_stride + u.h * p.o_head_stride;
            lse_ptr = p.lse + static_cast<int64_t>(u.h) * p.total_q + u.q_off + row;
          } else {
            orow = p.out + u.b * p.o_batch_stride + u.h * p.o_head_stride + static_cast<int64_t>(row) * p.o_row_stride;
            lse_ptr = p.lse + (static_cast<int64_t>(u.b) * p.heads_q + u.h) * p.seqlen_q + row;
          }
          uint4* dst = reinterpret_cast<uint4*>(orow);
#pragma unroll
          for (int i = 0; i < kD / 8; ++i)
            if (8 * i < p.head_dim) dst[i] = make_uint4(0u, 0u, 0u, 0u);
          *lse_ptr = INFINITY;
        }
        continue;
      }
      const int len_k = u.len_k;
      // keys at index >= col_limit are invisible to this row; blocks reaching past mask_from need the mask
      const int col_limit = p.is_causal ? min(len_k, row + u.causal_off + 1) : len_k;
      const int mask_from = p.is_causal ? min(len_k, row_lo + u.causal_off + 1) : len_k;

      float m_run = neg_inf;
      float l_run = 0.f;
      if (row_in_tile == 0) FWD_STAMP(t, ucnt, 0);
      const uint16_t* bias_row = nullptr;  // this row's bias values, or null for a row past the sequence
      if constexpr (kBias) {
        if (row < u.len_q)
          bias_row = p.bias + u.b * p.bias_batch_stride + u.h * p.bias_head_stride + static_cast<int64_t>(row) * p.bias_row_stride;
      }
      const uint32_t* keep_row = nullptr;  // this row's keep bits, 4 words per key block
      if constexpr (kDrop)
        keep_row = p.keep_rows + (p.cu_q != nullptr ? static_cast<size_t>(u.h) * p.lq_pad + u.q_off + row
                                                    : static_cast<size_t>(u.b * p.heads_q + u.h) * p.lq_pad + row) * p.lk_words;

      for (int j = 0; j < my_blocks; ++j) {
        const int n0 = j * kBlockN;
        const uint32_t par = (cnt + j) & 1;
        uint4 keep = make_uint4(0u, 0u, 0u, 0u);
        if constexpr (kDrop) keep = *reinterpret_cast<const uint4*>(keep_row + (n0 >> 5));  // in flight under the wait
        if constexpr (kBias) {
          // the next block's 256 bytes of this row: into L2 now, so that the loads below find them there
          if (bias_row != nullptr && j + 1 < my_blocks) {
            const int last = len_k - 1;  // only addresses inside the row
            prefetch_l2(bias_row + min(n0 + kBlockN, last));
            prefetch_l2(bias_row + min(n0 + kBlockN + 64, last));
            prefetch_l2(bias_row + min(n0 + 2 * kBlockN - 1, last));
          }
        }
        // This block's bias values, packed as they come (64 registers): loaded before the wait for the scores,
        // whose 128 registers are not live yet, so the load latency passes under the tile's MMAs. A chunk that
        // starts past the last key is skipped; one that straddles it reads up to 7 elements of row padding,
        // which the caller guarantees. (Shared memory has no room for a 32 KB bias tile.)
        uint4 bw[kBias ? kBlockN / 8 : 1];
        if constexpr (kBias) {
#pragma unroll
          for (int ch = 0; ch < kBlockN / 8; ++ch) {
            bw[ch] = make_uint4(0u, 0u, 0u, 0u);
            if (bias_row != nullptr && n0 + ch * 8 < len_k) bw[ch] = *reinterpret_cast<const uint4*>(bias_row + n0 + ch * 8);
          }
        }
        // warp-uniform, because the arrivals below are made by one lane on behalf of its warp
        ok = __all_sync(0xffffffffu, mbar_wait(bar_s, par, abort_flag));
        if (!ok) break;
        if (row_in_tile == 0 && j == 0) FWD_STAMP(t, ucnt, 1);
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
        if constexpr (kBias) {
          // s <- s + bias / scale, so that everything below (maximum, s * c - m) stays as it is (a skipped chunk
          // holds zeros; its keys are masked further down)
#pragma unroll
          for (int ch = 0; ch < kBlockN / 8; ++ch) {
            const uint32_t ww[4] = {bw[ch].x, bw[ch].y, bw[ch].z, bw[ch].w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const float2 b2 = unpack_16x2<kF16>(ww[i]);
              s[ch * 8 + 2 * i] = fmaf(b2.x, p.inv_scale, s[ch * 8 + 2 * i]);
              s[ch * 8 + 2 * i + 1] = fmaf(b2.y, p.inv_scale, s[ch * 8 + 2 * i + 1]);
            }
          }
        }
        const bool need_mask = n0 + kBlockN > mask_from;
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
        if (j == 0) {
          m_run = m_new;
        } else {
          const bool grow = (m_new - m_run) > kRescaleThreshold;  // false for NaN (-inf - -inf)
          if (__any_sync(0xffffffffu, grow)) {
            const float alpha = (m_new == neg_inf) ? 1.f : ex2_approx(m_run - m_new);
            m_run = m_new;
            l_run *= alpha;
            // O_t still receives PV(j-1); wait for it before touching the accumulator
            ok = __all_sync(0xffffffffu, mbar_wait(bar_o, par ^ 1u, abort_flag));
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
            if constexpr (kDrop) {
              // the row sum above keeps every pair (softmax is normalised before dropout); only P.V loses them
              const uint32_t word = (cc >> 1) == 0 ? keep.x : (cc >> 1) == 1 ? keep.y : (cc >> 1) == 2 ? keep.z : keep.w;
              pk[i] &= keep_pair_mask(word >> ((cc & 1) * 16 + 2 * i));
            }
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
        tmem_wait_st();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_p + 8);
      }
      if (!ok) break;
      if (row_in_tile == 0) FWD_STAMP(t, ucnt, 2);

      // ---- epilogue: O / l -> 16-bit, LSE
      if (my_blocks > 0) {
        ok = __all_sync(0xffffffffu, mbar_wait(bar_o, (cnt + my_blocks - 1) & 1, abort_flag));
        if (!ok) break;
      }
      if (row_in_tile == 0) FWD_STAMP(t, ucnt, 3);
      const int u_q_off = info[0], u_h = info[1], u_b = info[2], u_len_q = info[3];
      if (row_lo < u_len_q) {
        tc_fence_after_sync();
        float inv_l = (l_run > 0.f) ? 1.f / l_run : 0.f;
        if constexpr (kDrop) inv_l *= p.keep_scale;
        uint32_t w[kD / 2];
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
#pragma unroll
          for (int i = 0; i < 16; ++i)
            w[cc * 16 + i] =
                pack_16x2<kF16>(__uint_as_float(r[2 * i]) * inv_l, __uint_as_float(r[2 * i + 1]) * inv_l);
        }
        // O_t is in registers: the next unit's first PV may overwrite the accumulator
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar + kBarOFree + 8 * t);
        if (row_in_tile == 0) FWD_STAMP(t, ucnt, 4);
        const bool valid = row < u_len_q;
        // A whole 128-row tile goes out as TMA stores (64 columns at a time through a 16 KB staging
        // buffer per warpgroup): asynchronous and fully coalesced. Dense tensors are clipped by the
        // tensor map; a packed (varlen) tile that ends inside its sequence's last rows would spill
        // into the next sequence, so it is written row by row from registers instead.
        if (p.cu_q == nullptr || row_lo + kBlockM <= u_len_q) {
          // (mbarriers with bounded waits rather than bar.sync: a warp that has given up must not
          // leave the other three waiting for it forever)
          uint8_t* stage = smem + kSmemStage + t * kStageBytes + row_in_tile * 128;
#pragma unroll
          for (int half = 0; half < kD / 64; ++half, ++st_cnt) {
            if (row_in_tile == 0) {
              tma_store_wait_read();  // the previous store has left the buffer
              mbar_arrive(bar + kBarStageFree + 8 * t);
            }
            ok = __all_sync(0xffffffffu, mbar_wait(bar + kBarStageFree + 8 * t, st_cnt & 1, abort_flag));
            if (!ok) break;
#pragma unroll
            for (int ch = 0; ch < 8; ++ch)
              *reinterpret_cast<uint4*>(stage + ((ch ^ (row_in_tile & 7)) << 4)) =
                  make_uint4(w[half * 32 + 4 * ch], w[half * 32 + 4 * ch + 1], w[half * 32 + 4 * ch + 2],
                             w[half * 32 + 4 * ch + 3]);
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar + kBarStageFull + 8 * t);
            if (row_in_tile == 0) {
              if (mbar_wait(bar + kBarStageFull + 8 * t, st_cnt & 1, abort_flag)) {
                tma_store_4d(&tm_o, base + kSmemStage + t * kStageBytes, half * 64, u_q_off + row_lo, u_h,
                             p.cu_q != nullptr ? 0 : u_b);
                tma_store_commit();
              }
            }
          }
          if (!ok) break;
        } else if (valid) {
          uint4* dst = reinterpret_cast<uint4*>(p.out + static_cast<int64_t>(u_q_off + row) * p.o_row_stride +
                                                u_h * p.o_head_stride);
#pragma unroll
          for (int i = 0; i < kD / 8; ++i)
            if (8 * i < p.head_dim) dst[i] = make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]);
        }
        if (valid) {
          float* lse_ptr = (p.cu_q != nullptr)
                               ? p.lse + static_cast<int64_t>(u_h) * p.total_q + u_q_off + row
                               : p.lse + (static_cast<int64_t>(u_b) * p.heads_q + u_h) * p.seqlen_q + row;
          const float kLn2 = 0.6931471805599453f;
          *lse_ptr = (l_run > 0.f) ? (m_run + log2f(l_run)) * kLn2 : INFINITY;
        }
      } else {
        __syncwarp();
        if (lane == 0) mbar_arrive(bar + kBarOFree + 8 * t);
      }
      if (row_in_tile == 0) FWD_STAMP(t, ucnt, 5);
      cnt += my_blocks;
      ++ucnt;
    }
    if (row_in_tile == 0) tma_store_wait_read();  // the CTA's shared memory must outlive its stores' reads of it
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

int launch_fwd_prefill(const sdpa_b200_params& p, void* workspace, cudaStream_t stream) {
  const bool varlen = p.cu_seqlens_q != nullptr;
  const bool f16 = p.dtype == SDPA_B200_F16;
  CUtensorMap tm_q, tm_k, tm_v, tm_o;
  int st;
  const int64_t rows_q = varlen ? p.total_q : p.max_seqlen_q;
  const int64_t rows_k = varlen ? p.total_k : p.max_seqlen_k;
  const int64_t nb = varlen ? 1 : p.batch;
  st = make_tensor_map_16(f16, &tm_q, p.q, p.head_dim, rows_q, p.heads_q, nb, p.q_row_stride,
                          p.q_head_stride, p.q_batch_stride, kBlockM);
  if (st != SDPA_B200_OK) return st;
  st = make_tensor_map_16(f16, &tm_k, p.k, p.head_dim, rows_k, p.heads_kv, nb, p.k_row_stride,
                          p.k_head_stride, p.k_batch_stride, kBlockN);
  if (st != SDPA_B200_OK) return st;
  st = make_tensor_map_16(f16, &tm_v, p.v, p.head_dim, rows_k, p.heads_kv, nb, p.v_row_stride,
                          p.v_head_stride, p.v_batch_stride, kBlockN);
  if (st != SDPA_B200_OK) return st;
  st = make_tensor_map_16(f16, &tm_o, p.out, p.head_dim, rows_q, p.heads_q, nb, p.o_row_stride,
                          p.o_head_stride, p.o_batch_stride, kBlockM);
  if (st != SDPA_B200_OK) return st;

  FwdKernelParams kp;
  kp.out = static_cast<uint16_t*>(p.out);
  kp.lse = p.lse;
  kp.cu_q = p.cu_seqlens_q;
  kp.cu_k = p.cu_seqlens_k;
  kp.status = p.device_status != nullptr ? p.device_status : static_cast<uint32_t*>(workspace);
  kp.unit_counter = static_cast<uint32_t*>(workspace) + 1;  // workspace header word 1, cleared with the header
  kp.o_batch_stride = p.o_batch_stride;
  kp.o_head_stride = p.o_head_stride;
  kp.o_row_stride = p.o_row_stride;
  kp.seqlen_q = p.max_seqlen_q;
  kp.seqlen_k = p.max_seqlen_k;
  kp.total_q = p.total_q;
  kp.heads_q = p.heads_q;
  kp.kv_group = p.heads_q / p.heads_kv;
  kp.head_dim = p.head_dim;
  const bool drop = p.dropout_p > 0.f;
  kp.keep_rows = p.keep_rows;
  kp.lq_pad = varlen ? p.total_q + 128 : (p.max_seqlen_q + 127) / 128 * 128;
  kp.lk_words = (p.max_seqlen_k + 127) / 128 * 4;
  kp.keep_scale = drop ? 1.f / (1.f - p.dropout_p) : 1.f;
  kp.bias = static_cast<const uint16_t*>(p.bias);
  kp.bias_batch_stride = p.bias_batch_stride;
  kp.bias_head_stride = p.bias_head_stride;
  kp.bias_row_stride = p.bias_row_stride;
  kp.inv_scale = 1.f / p.softmax_scale;
  kp.scale_log2 = p.softmax_scale * 1.4426950408889634f;
  kp.is_causal = p.is_causal;
#ifdef SDPA_FWD_STAMPS
  {
    const char* env = getenv("SDPA_FWD_STAMPS_PTR");
    kp.stamps = env ? reinterpret_cast<float*>(strtoull(env, nullptr, 10)) : nullptr;
  }
#endif

  auto pick = [&](auto drop_tag, auto bias_tag) {
    constexpr bool kDrop = decltype(drop_tag)::value;
    constexpr bool kBias = decltype(bias_tag)::value;
    return p.head_dim <= 64 ? (f16 ? fwd_prefill_kernel<64, true, kDrop, kBias> : fwd_prefill_kernel<64, false, kDrop, kBias>)
                            : (f16 ? fwd_prefill_kernel<128, true, kDrop, kBias> : fwd_prefill_kernel<128, false, kDrop, kBias>);
  };
  const bool with_bias = p.bias != nullptr;
  auto kernel = drop ? (with_bias ? pick(std::true_type{}, std::true_type{}) : pick(std::true_type{}, std::false_type{}))
                     : (with_bias ? pick(std::false_type{}, std::true_type{}) : pick(std::false_type{}, std::false_type{}));
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
  kp.num_slots = groups * kp.heads_per_wave * kp.num_m_blocks;
  const int sms = sm_count();
  if (sms <= 0) {
    set_error("prefill: cannot read the SM count of the current device");
    return SDPA_B200_NO_DEVICE;
  }
  // one persistent CTA per SM (shared memory and TMEM allow no second one), less the SMs the caller wants left free
  const int usable = sms - p.sm_margin > 1 ? sms - p.sm_margin : 1;
  dim3 grid(kp.num_slots < usable ? kp.num_slots : usable, 1, 1);
  kernel<<<grid, kNumThreads, kSmemBytes, stream>>>(tm_q, tm_k, tm_v, tm_o, kp);
  err = cudaGetLastError();
  if (err != cudaSuccess) {
    set_error("prefill: launch failed: %s", cudaGetErrorString(err));
    return SDPA_B200_LAUNCH_FAILED;
  }
  count_launch();
  return SDPA_B200_OK;
}

}  // namespace sdpa_b200
