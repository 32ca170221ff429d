// Fused backward attention kernel for sm_100a: dK, dV and the dQ contributions of one 128-key block from ONE
// recomputation of the scores.
//
// Stands, like bwd_sm100.cu, behind mha_varlen_bwd -> cnnlFlashAttentionBackward
// (torch_mlu/csrc/aten/operators/cnnl/internal/FlashAttention_internal.cpp:449-480: one fused backward call). The
// two-kernel path of bwd_sm100.cu forms S and dP twice (once per kernel): 7 GEMMs per 128 x 128 tile pair where the
// algorithm has 5. Here one CTA per (batch, kv head, 128-key block) streams the query tiles once and issues
//   S^T = K Q^T,  dP^T = V dO^T            (scores, into TMEM)
//   dV += P^T dO,  dK += dS^T Q            (accumulated in TMEM over the CTA's life)
//   dQ_tile = dS K                         (one GEMM per item, read out at once)
// with P^T = exp2(S^T c - lse2) and dS^T = P^T o (dP^T - delta) formed by two compute warpgroups (thread = key row =
// TMEM lane, one warpgroup per 64-query half). P^T goes back to TMEM as the A operand of the dV GEMM; dS^T goes to a
// 32 KB shared-memory tile in the 128-byte-swizzled layout, where it is the K-major A operand of the dK GEMM and the
// MN-major A operand of the dQ GEMM at the same time. A fourth warpgroup (thread = query row) reads each item's dQ tile
// out of TMEM and adds it into an fp32 accumulator in global memory with 16-byte reductions (red.global.add.v4.f32);
// a small kernel scales and converts the accumulator afterwards. Those reductions arrive in an order that varies from
// launch to launch, so dQ is reproducible only to fp32 rounding; dK and dV are summed in a fixed order.
//
// What bounds it (time stamps of the profiling build, B8 H16 L2048 causal): the reductions. One item adds 64 KB into
// the accumulator; with every SM sending them, the L2 takes about 20 bytes per clock and SM (a stand-alone test reaches
// 5.5 TB/s = 706 floats per clock over the chip with red.v4 and with cp.reduce.async.bulk alike, 3.6 TB/s once the
// accumulator exceeds L2), i.e. ~3400 cycles per item against 2560 cycles of tensor work, and a reduce warp needs
// ~90 cycles per red.v4. Item period ~5600 cycles: level with the two-kernel path on B8 H16 L2048 causal (0.540 ms
// against 0.536 ms for the whole backward), 5-9 % ahead at L = 8192 causal and at large unmasked shapes.
//
// TMEM (512 columns): T1 [0,128) T2 [128,256) dV [256,384) dK [384,512). Item i has S in T[i&1] and dP in the other
// buffer. Life of one buffer: S(i) -> P(i) (16-bit, front of each half) -> dQ(i) -> dP(i+1) -> S(i+2) ...:
//   dQ(i) is issued behind dV(i) by the same thread (the pipe keeps their order), so P(i) has been read;
//   dP(i+1) waits until the reduce warps have read dQ(i) (`Q free`);
//   S(i+2) waits until the compute warps have read dP(i+1) (`dP free`).
// So the next item's S is ready while this item's dS is formed, and dP(i+1) follows as soon as dQ(i) has left.
#include "bwd_common.cuh"

namespace sdpa_b200 {
namespace {

#ifndef SDPA_BWD_POLY_FUSED
#define SDPA_BWD_POLY_FUSED 2  // of every 4 column pairs, how many take 2^x from the FMA pipe (see exp2_poly3_x2)
#endif

constexpr int kFThreads = 512;  // warps 0-3 / 4-7 compute, 8 TMA, 9 score GEMMs, 10 accumulation GEMMs, 11 idle, 12-15 dQ reduce
// Register hand-over (setmaxnreg): compiled for 65536 / 512 = 128 registers per thread; the compute and reduce warpgroups
// grow, the fourth (producer, issuers) shrinks. The increase waits - without a time limit - until the pool holds enough registers, so what
// the shrinking warpgroups release must cover what the growing ones take.
constexpr int kRegsLaunch = 128;
constexpr int kRegsCompute = 152;
constexpr int kRegsReduce = 144;  // a thread holds a whole row of the dQ tile (up to 128 floats)
constexpr int kRegsUtil = 64;
static_assert(kRegsCompute >= kRegsLaunch && kRegsReduce >= kRegsLaunch && kRegsUtil <= kRegsLaunch &&
                  (kRegsCompute - kRegsLaunch) * 2 + (kRegsReduce - kRegsLaunch) <= (kRegsLaunch - kRegsUtil),
              "setmaxnreg.inc would wait forever: the compute and reduce warps ask for more than the others release");

// shared memory map (offsets from a 1024-byte aligned base)
constexpr uint32_t kFSmemX = 0;                            // K, V tiles: 2 x 32 KB
constexpr uint32_t kFSmemY = 2 * kTileBytes;               // ring: Q(i), dO(i), Q(i+1), dO(i+1)
constexpr uint32_t kFSmemDS = kFSmemY + 4 * kTileBytes;    // dS^T of the current item, 32 KB
constexpr uint32_t kFSmemVec = kFSmemDS + kTileBytes;      // per ring pair: lse2[128], delta[128]
constexpr uint32_t kFSmemBar = kFSmemVec + 2 * 1024;
constexpr uint32_t kFSmemUsed = kFSmemBar + 256;
constexpr uint32_t kFSmemRequest = 232448;  // everything a CTA may have: what is left over absorbs the base alignment
static_assert(kFSmemUsed + 512 <= kFSmemRequest, "shared memory map does not fit");

constexpr uint32_t kFBarXFull = 0;
constexpr uint32_t kFBarYFull = 8;     // 4 slots
constexpr uint32_t kFBarYEmpty = 40;   // 2 pairs: behind dK(i), the last reader of Q(i), dO(i) and of the dS tile
constexpr uint32_t kFBarSFull = 56;
constexpr uint32_t kFBarDFull = 64;
constexpr uint32_t kFBarDFree = 72;    // 8: all compute warps have read dP out of TMEM
constexpr uint32_t kFBarP1Full = 80;   // 8: all compute warps have stored P
constexpr uint32_t kFBarDSFull = 88;   // 8: all compute warps have stored dS in shared memory
constexpr uint32_t kFBarQFull = 96;    // dQ(i) is in TMEM
constexpr uint32_t kFBarQFree = 104;   // 4: all reduce warps have read dQ(i)
constexpr uint32_t kFBarAccFull = 112;
constexpr uint32_t kFBarEpiFull = 120; // 8
constexpr uint32_t kFSmemTmemPtr = 128;
constexpr uint32_t kFSmemAbort = 132;

// Profiling builds (-DSDPA_BWD_STAMPS) time-stamp pipeline events of one CTA: roles 0/1 = lane 0 of the first warp of each
// compute warpgroup, 2 / 3 = the two MMA issuers, 4 = lane 0 of the first reduce warp; [role 5][item 24][event 8] floats.
#ifdef SDPA_BWD_STAMPS
#define FSTAMP(role, item, ev)                                                                    \
  do {                                                                                            \
    if (stamp_on && (item) < 24)                                                                  \
      p.stamps[((role) * 24 + (item)) * 8 + (ev)] = static_cast<float>(clock64() - t_start);      \
  } while (0)
#else
#define FSTAMP(role, item, ev) do {} while (0)
#endif

template <int kD, bool kF16>
constexpr uint32_t kIdescDQ = umma_idesc_16(kTile, kD, true, true, kF16);  // A = dS (MN-major), B = K (MN-major)

// dQ_tile[q][d] = sum_key dS[q][key] K[key][d]. The dS tile is stored [key][query]: the query index is the contiguous
// one, i.e. the tile is an MN-major A operand (64-query chunks kHalfBytes apart); 16 keys are 2048 bytes in both tiles.
template <int kD, bool kF16>
__device__ __forceinline__ void issue_dq(uint32_t t, uint32_t ds_smem, uint32_t k_smem) {
  const uint32_t a_lo = umma_desc_lo_mnmajor(ds_smem, kHalfBytes);
  const uint32_t b_lo = umma_desc_lo_mnmajor(k_smem, kHalfBytes);
  umma_ss_lo<kIdescDQ<kD, kF16>, false>(t, a_lo, b_lo);
#pragma unroll
  for (int ks = 1; ks < kTile / 16; ++ks)
    umma_ss_lo<kIdescDQ<kD, kF16>, true>(t, a_lo + ks * (2048 >> 4), b_lo + ks * (2048 >> 4));
}

// dK[key][d] += sum_q dS^T[key][q] Q[q][d]: the same dS tile as a K-major A operand (the contraction index, the query,
// is contiguous: 16 queries are 32 bytes inside a 64-query half), Q as MN-major B.
template <int kD, bool kF16>
__device__ __forceinline__ void issue_dk(uint32_t acc, uint32_t ds_smem, uint32_t q_smem, bool accumulate) {
  const uint32_t a_lo = umma_desc_lo_kmajor(ds_smem);
  const uint32_t b_lo = umma_desc_lo_mnmajor(q_smem, kHalfBytes);
#pragma unroll
  for (int ks = 0; ks < kTile / 16; ++ks) {
    const uint32_t off_a = ((ks >> 2) * kHalfBytes + (ks & 3) * 32) >> 4;
    umma_ss_lo_acc<kIdescTS<kD, kF16>>(acc, a_lo + off_a, b_lo + ks * (2048 >> 4), (accumulate || ks > 0) ? 1u : 0u);
  }
}

// Index of the first float of `row` in the tiled fp32 dQ accumulator (see BwdKernelParams::dq_acc); the row's 4-column
// group g is 512 * g floats further on.
template <int kD>
__device__ __forceinline__ size_t dq_acc_index(size_t row) {
  return (row >> 7) * (static_cast<size_t>(kD / 4) * 512) + (row & 127) * 4;
}

template <int kD, bool kF16, bool kDrop>
__global__ void __launch_bounds__(kFThreads, 1)
bwd_fused_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                 const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_do,
                 const __grid_constant__ CUtensorMap tm_dv, const __grid_constant__ CUtensorMap tm_dk,
                 const BwdKernelParams p) {
  extern __shared__ uint8_t smem_raw[];
#ifdef SDPA_BWD_STAMPS
  const long long t_entry = clock64();
#endif
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw_addr);
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  if (base - raw_addr + kFSmemUsed > kFSmemRequest) {
    // the shared-memory window starts where the map does not fit behind the alignment: report, touch nothing
    if (threadIdx.x == 0) atomicExch(p.status, static_cast<uint32_t>(SDPA_B200_LAUNCH_FAILED));
    return;
  }

  // CTA order (1-D grid): (batch, kv head) pairs in groups of `heads_per_wave` whose streamed tensors fit L2 together;
  // inside a group the key blocks go heaviest first across all its heads (key block 0 sees every query).
  int b, hx, xb;
  {
    const int per_group = p.heads_per_wave * p.num_row_blocks;
    const int grp = blockIdx.x / per_group;
    const int w = blockIdx.x - grp * per_group;
    const int size = min(p.heads_per_wave, p.num_bh - grp * p.heads_per_wave);
    const int rank = w / size;
    const int bh = grp * p.heads_per_wave + (w - rank * size);
    if (rank >= p.num_row_blocks) return;  // padding slots of a short last group
    xb = rank;
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
  const int x0 = xb * kTile;
  if (x0 >= len_k) return;

  // query tiles [y_lo, y_hi) that see this key block, per query head of the group
  int y_hi = (len_q + kTile - 1) / kTile;
  int y_lo = 0;
  if (p.is_causal) {
    y_lo = max(0, (x0 - causal_off) / kTile);
    if (x0 - causal_off > len_q - 1) y_lo = y_hi;
  }
  const int tiles_per_head = max(0, y_hi - y_lo);
  const int n_items = tiles_per_head * p.kv_group;

  const uint32_t bar = base + kFSmemBar;
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(smem + kFSmemBar + kFSmemAbort);
  volatile uint32_t* tmem_ptr_smem = reinterpret_cast<volatile uint32_t*>(smem + kFSmemBar + kFSmemTmemPtr);

  constexpr uint32_t kLoadBytes = kTile * kD * 2;  // bytes one tile brings in
  constexpr int kPreloaded = 4;
  // ring tile idx: Q(idx/2) if even, dO(idx/2) if odd; slot idx % 4; false when a wait gave up
  auto load_tile = [&](int idx) -> bool {
    const int i = idx >> 1;
    const int s = idx & 3;
    // the slot pair of item i - 2 is released by one commit behind its dK GEMM
    if (!mbar_wait(bar + kFBarYEmpty + 8 * (s >> 1), ((static_cast<uint32_t>(idx) >> 2) & 1u) ^ 1u, abort_flag)) return false;
    const int hi = i / tiles_per_head;
    const int yt = y_lo + (i - hi * tiles_per_head);
    const int hy = hx * p.kv_group + hi;
    const uint32_t full = bar + kFBarYFull + 8 * s;
    const uint32_t dst = base + kFSmemY + s * kTileBytes;
    const int row = q_off + yt * kTile;
    const bool first = (idx & 1) == 0;
    if (first) {
      mbar_arrive_expect_tx(full, kLoadBytes + 1024);
      const size_t vec = (static_cast<size_t>(b) * p.heads_q + hy) * p.lq_pad + static_cast<size_t>(yt) * kTile;
      bulk_load_1d(base + kFSmemVec + (s >> 1) * 1024, p.lse2 + vec, 512, full);
      bulk_load_1d(base + kFSmemVec + (s >> 1) * 1024 + 512, p.delta + vec, 512, full);
    } else {
      mbar_arrive_expect_tx(full, kLoadBytes);
    }
    const CUtensorMap* tm = first ? &tm_q : &tm_do;
    tma_load_4d(dst, tm, full, 0, row, hy, bcoord);
    if (kD > 64) tma_load_4d(dst + kHalfBytes, tm, full, 64, row, hy, bcoord);
    return true;
  };

  if (warp == 8 && lane == 0) {
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&tm_v);
    tma_prefetch_desc(&tm_do);
    mbar_init(bar + kFBarXFull, 1);
    for (int s = 0; s < 4; ++s) mbar_init(bar + kFBarYFull + 8 * s, 1);
    mbar_init(bar + kFBarYEmpty, 1);
    mbar_init(bar + kFBarYEmpty + 8, 1);
    mbar_init(bar + kFBarSFull, 1);
    mbar_init(bar + kFBarDFull, 1);
    mbar_init(bar + kFBarDFree, 8);  // one arrival per compute warp
    mbar_init(bar + kFBarP1Full, 8);
    mbar_init(bar + kFBarDSFull, 8);
    mbar_init(bar + kFBarQFull, 1);
    mbar_init(bar + kFBarQFree, 4);  // one arrival per reduce warp
    mbar_init(bar + kFBarAccFull, 1);
    mbar_init(bar + kFBarEpiFull, 8);
    *abort_flag = 0;
    fence_mbar_init();
    if (n_items > 0) {
      const int x_row = k_off + x0;
      mbar_arrive_expect_tx(bar + kFBarXFull, 2 * kLoadBytes);
      tma_load_4d(base + kFSmemX, &tm_k, bar + kFBarXFull, 0, x_row, hx, bcoord);
      if (kD > 64) tma_load_4d(base + kFSmemX + kHalfBytes, &tm_k, bar + kFBarXFull, 64, x_row, hx, bcoord);
      tma_load_4d(base + kFSmemX + kTileBytes, &tm_v, bar + kFBarXFull, 0, x_row, hx, bcoord);
      if (kD > 64) tma_load_4d(base + kFSmemX + kTileBytes + kHalfBytes, &tm_v, bar + kFBarXFull, 64, x_row, hx, bcoord);
      for (int idx = 0; idx < kPreloaded && idx < 2 * n_items; ++idx) load_tile(idx);
    }
  }
  if (warp == 0) {
    __syncwarp();
    tmem_alloc(base + kFSmemBar + kFSmemTmemPtr, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_ptr_smem;
  const uint32_t t1 = tmem_base, t2 = tmem_base + 128, acc_dv = tmem_base + 256, acc_dk = tmem_base + 384;
  const uint32_t k_smem = base + kFSmemX, v_smem = base + kFSmemX + kTileBytes, ds_smem = base + kFSmemDS;
#ifdef SDPA_BWD_STAMPS
  const long long t_start = clock64();
  const bool stamp_on = p.stamps != nullptr && b == 0 && hx == 0 && xb == 0 && lane == 0 &&
                        (warp == 0 || warp == 4 || warp == 9 || warp == 10 || warp == 12);
#endif

  if (warp >= 12) {
    // ------------------------------------------------------------------ dQ reduce warps (thread = query row)
    reg_increase<kRegsReduce>();
    const int r = (warp & 3) * 32 + lane;
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    bool ok = true;
    for (int i = 0; i < n_items; ++i) {
      const int hi = i / tiles_per_head;
      const int yt = y_lo + (i - hi * tiles_per_head);
      const int hy = hx * p.kv_group + hi;
      const int qrow = yt * kTile + r;
      const size_t row = (p.cu_q != nullptr) ? static_cast<size_t>(hy) * p.dq_acc_rows + q_off + qrow
                                             : (static_cast<size_t>(b) * p.heads_q + hy) * p.lq_pad + qrow;
      float* dst = p.dq_acc + dq_acc_index<kD>(row);
      const bool valid = qrow < len_q;
      FSTAMP(4, i, 0);
      ok = __all_sync(0xffffffffu, mbar_wait(bar + kFBarQFull, i & 1, abort_flag));
      if (!ok) break;
      tc_fence_after_sync();
      FSTAMP(4, i, 1);
      const uint32_t src = ((i & 1) ? t2 : t1) + lane_base;
      // the whole tile goes into registers first, so that the buffer is handed on before the first reduction is issued:
      // the reductions run at the pace of the L2 (a few dozen cycles each once every SM is sending them)
      uint32_t v[kD];
#pragma unroll
      for (int c = 0; c < kD / 32; ++c) tmem_ld_x32_at<32 * 0, 32>(src + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&v[c * 32]));
      tmem_wait_ld();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar + kFBarQFree);
      FSTAMP(4, i, 2);
      if (valid) {
#pragma unroll
        for (int j = 0; j < kD / 4; ++j)
          red_add_f32x4(dst + static_cast<size_t>(j) * 512, __uint_as_float(v[4 * j]), __uint_as_float(v[4 * j + 1]),
                        __uint_as_float(v[4 * j + 2]), __uint_as_float(v[4 * j + 3]));
      }
      FSTAMP(4, i, 3);
    }
  } else if (warp >= 8) {
    reg_decrease<kRegsUtil>();
    if (warp == 8) {
      // ------------------------------------------------------------------ TMA producer (rest of the ring)
      if (lane == 0 && n_items > 0) {
        for (int idx = kPreloaded; idx < 2 * n_items; ++idx)
          if (!load_tile(idx)) break;
        drain_after_abort(abort_flag);
      }
    } else if (warp == 9) {
      // ------------------------------------------------------------------ score GEMMs: S = K Q^T, dP = V dO^T
      if (lane == 0 && n_items > 0) {
        auto y_full = [&](int idx) { return mbar_wait(bar + kFBarYFull + 8 * (idx & 3), (idx >> 2) & 1, abort_flag); };
        auto y_slot = [&](int idx) { return base + kFSmemY + (idx & 3) * kTileBytes; };
#ifdef SDPA_BWD_STAMPS
        if (stamp_on) p.stamps[(2 * 24 + 23) * 8 + 0] = static_cast<float>(t_start - t_entry);
#endif
        bool ok = mbar_wait(bar + kFBarXFull, 0, abort_flag) && y_full(0);
        FSTAMP(2, 23, 1);
        if (ok) {
          tc_fence_after_sync();
          issue_xyT<kD, kF16>(t1, k_smem, y_slot(0));
          umma_commit(bar + kFBarSFull);
        }
        FSTAMP(2, 23, 2);
        ok = ok && y_full(1);
        if (ok) {
          tc_fence_after_sync();
          issue_xyT<kD, kF16>(t2, v_smem, y_slot(1));
          umma_commit(bar + kFBarDFull);
        }
        for (int i = 0; ok && i + 1 < n_items; ++i) {
          const uint32_t sb = (i & 1) ? t2 : t1, db = (i & 1) ? t1 : t2;
          // dP(i) has left TMEM once all compute warps have read it: its buffer takes S(i+1)
          FSTAMP(2, i, 0);
          ok = mbar_wait(bar + kFBarDFree, i & 1, abort_flag) && y_full(2 * i + 2);
          if (!ok) break;
          FSTAMP(2, i, 1);
          tc_fence_after_sync();
          issue_xyT<kD, kF16>(db, k_smem, y_slot(2 * i + 2));
          umma_commit(bar + kFBarSFull);
          FSTAMP(2, i, 2);
          // dQ(i) has left TMEM once all reduce warps have read it: its buffer takes dP(i+1)
          ok = mbar_wait(bar + kFBarQFree, i & 1, abort_flag) && y_full(2 * i + 3);
          if (!ok) break;
          FSTAMP(2, i, 3);
          tc_fence_after_sync();
          issue_xyT<kD, kF16>(sb, v_smem, y_slot(2 * i + 3));
          umma_commit(bar + kFBarDFull);
          FSTAMP(2, i, 4);
        }
      }
    } else if (warp == 10) {
      // ------------------------------------------------------------------ dV += P^T dO, dQ = dS K, dK += dS^T Q
      if (lane == 0 && n_items > 0) {
        bool ok = mbar_wait(bar + kFBarXFull, 0, abort_flag);
        for (int i = 0; ok && i < n_items; ++i) {
          const int s0 = (2 * i) & 3;
          const uint32_t y_q = base + kFSmemY + s0 * kTileBytes, y_do = y_q + kTileBytes;
          const uint32_t sb = (i & 1) ? t2 : t1;
          const uint32_t par = ((2 * i) >> 2) & 1;
          // the tiles landed long ago (the other issuer has used them); these waits make the copies visible here too
          FSTAMP(3, i, 0);
          ok = mbar_wait(bar + kFBarYFull + 8 * s0, par, abort_flag) && mbar_wait(bar + kFBarYFull + 8 * (s0 + 1), par, abort_flag) &&
               mbar_wait(bar + kFBarP1Full, i & 1, abort_flag);
          if (!ok) break;
          FSTAMP(3, i, 1);
          tc_fence_after_sync();
          issue_wy_half<kD, kF16>(acc_dv, sb, y_do, 0, i > 0);
          issue_wy_half<kD, kF16>(acc_dv, sb + 64, y_do, 1, true);
          FSTAMP(3, i, 2);
          ok = mbar_wait(bar + kFBarDSFull, i & 1, abort_flag);
          if (!ok) break;
          FSTAMP(3, i, 3);
          tc_fence_after_sync();
          // dQ first: its read-out by the reduce warps then runs under the dK GEMM
          issue_dq<kD, kF16>(sb, ds_smem, k_smem);
          umma_commit(bar + kFBarQFull);
          FSTAMP(3, i, 4);
          issue_dk<kD, kF16>(acc_dk, ds_smem, y_q, i > 0);
          umma_commit(bar + kFBarYEmpty + 8 * (s0 >> 1));  // Q(i), dO(i) and the dS tile may be overwritten
          if (i == n_items - 1) umma_commit(bar + kFBarAccFull);
          FSTAMP(3, i, 5);
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ compute warpgroups (thread = key row)
    reg_increase<kRegsCompute>();
    // warps 0-3 own query columns [0,64) of every key row, warps 4-7 columns [64,128)
    const int half = warp >> 2;
    const int r = (warp & 3) * 32 + lane;  // key row in the tile = TMEM lane
    const int xr = x0 + r;                 // key index within the sequence
    const uint32_t lane_base = (static_cast<uint32_t>((warp & 3) * 32) << 16) + half * 64;
    const float c = p.scale_log2;
    uint8_t* ds_row = smem + kFSmemDS + half * kHalfBytes + r * 128;
    bool ok = true;
    for (int i = 0; i < n_items; ++i) {
      const int hi = i / tiles_per_head;
      const int y0 = (y_lo + (i - hi * tiles_per_head)) * kTile;
      const uint32_t sbuf = ((i & 1) ? t2 : t1) + lane_base;
      const uint32_t dbuf = ((i & 1) ? t1 : t2) + lane_base;
      // keep bits of this thread's 64 (key, query) pairs, in flight under the waits below
      uint2 keep = make_uint2(0u, 0u);
      if constexpr (kDrop) {
        const uint32_t* words =
            p.keep_cols + (p.cu_q != nullptr ? static_cast<size_t>(hx * p.kv_group + hi) * p.keep_k_rows + k_off + xr
                                             : static_cast<size_t>(b * p.heads_q + hx * p.kv_group + hi) * p.keep_k_rows + xr) *
                              (p.keep_lq_pad >> 5);
        keep = *reinterpret_cast<const uint2*>(words + ((y0 + half * 64) >> 5));
      }
      // `ok` is made warp-uniform after every wait: the warp-level arrivals below need all 32 lanes
      FSTAMP(half, i, 0);
      ok = mbar_wait(bar + kFBarSFull, i & 1, abort_flag) &&
           mbar_wait(bar + kFBarYFull + 8 * ((2 * i) & 3), ((2 * i) >> 2) & 1, abort_flag);  // the per-query vectors
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after_sync();
      FSTAMP(half, i, 1);
      const float* vec_lse = reinterpret_cast<const float*>(smem + kFSmemVec + (i & 1) * 1024) + half * 64;
      const float* vec_delta = vec_lse + 128;
      // key xr sees query y0 + j iff xr <= y0 + j + off  <=>  j >= xr - off - y0. A row past the last key sees nothing:
      // in a packed tensor it holds the next sequence's key, whose dS must not reach this sequence's dQ.
      int j_lo = p.is_causal ? xr - causal_off - y0 - half * 64 : 0;
      if (xr >= len_k) j_lo = 64;

      // phase 1 (needs S only): P = exp2(S c - lse2), masked; its 16-bit copy goes back to TMEM at once
      float pr[64];
      {
        uint32_t a[64];
        tmem_ld_x64(sbuf, a);
        tmem_wait_ld();
        FSTAMP(half, i, 2);
#pragma unroll
        for (int j = 0; j < 64; j += 2) {
          const float x0v = fmaf(__uint_as_float(a[j]), c, -vec_lse[j]);
          const float x1v = fmaf(__uint_as_float(a[j + 1]), c, -vec_lse[j + 1]);
          if (((j >> 1) & 3) < SDPA_BWD_POLY_FUSED) {
            const float2 e = exp2_poly3_x2(make_float2(x0v, x1v));
            pr[j] = e.x;
            pr[j + 1] = e.y;
          } else {
            pr[j] = ex2_approx(x0v);
            pr[j + 1] = ex2_approx(x1v);
          }
        }
        // only tiles on the causal diagonal or past the end of the keys need the element mask (queries past the end
        // have lse2 = +inf, i.e. P = 0)
        if (__any_sync(0xffffffffu, j_lo > 0)) {
#pragma unroll
          for (int j = 0; j < 64; ++j) pr[j] = (j >= j_lo) ? pr[j] : 0.f;
        }
        uint32_t pw[32];
#pragma unroll
        for (int j2 = 0; j2 < 32; ++j2) {
          pw[j2] = pack_16x2<kF16>(pr[2 * j2], pr[2 * j2 + 1]);
          if constexpr (kDrop) pw[j2] &= keep_pair_mask((j2 < 16 ? keep.x : keep.y) >> ((2 * j2) & 31));
        }
        tmem_st_x16(sbuf, pw);
        tmem_st_x16(sbuf + 16, pw + 16);
        tmem_wait_st();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar + kFBarP1Full);
      }
      FSTAMP(half, i, 3);
      // phase 2 (needs dP): dS = P o (dP - delta) into this thread's row of the shared-memory tile
      ok = __all_sync(0xffffffffu, mbar_wait(bar + kFBarDFull, i & 1, abort_flag));
      if (!ok) break;
      tc_fence_after_sync();
      FSTAMP(half, i, 4);
      {
        uint32_t d[64];
        tmem_ld_x64(dbuf, d);
        tmem_wait_ld();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar + kFBarDFree);  // the dP buffer may be overwritten
        FSTAMP(half, i, 5);
        uint32_t dw[32];
#pragma unroll
        for (int j2 = 0; j2 < 32; ++j2) {
          float dp0 = __uint_as_float(d[2 * j2]), dp1 = __uint_as_float(d[2 * j2 + 1]);
          if constexpr (kDrop) {
            const uint32_t two = (j2 < 16 ? keep.x : keep.y) >> ((2 * j2) & 31);
            dp0 = (two & 1u) ? dp0 * p.keep_scale : 0.f;
            dp1 = (two & 2u) ? dp1 * p.keep_scale : 0.f;
          }
          dw[j2] = pack_16x2<kF16>(pr[2 * j2] * (dp0 - vec_delta[2 * j2]), pr[2 * j2 + 1] * (dp1 - vec_delta[2 * j2 + 1]));
        }
        // the dS tile is free once dK(i-1), its last reader, is done (the commit that also releases that item's ring slots)
        if (i > 0) {
          ok = __all_sync(0xffffffffu, mbar_wait(bar + kFBarYEmpty + 8 * ((i - 1) & 1), ((i - 1) >> 1) & 1, abort_flag));
          if (!ok) break;
        }
        // 64 queries = one 128-byte row of this half, 16-byte chunks XOR-swizzled by (row % 8): the layout a TMA box of
        // {64, 128} with 128-byte swizzle would have written, which is what the MMA descriptors expect
#pragma unroll
        for (int ch = 0; ch < 8; ++ch)
          *reinterpret_cast<uint4*>(ds_row + ((ch ^ (r & 7)) << 4)) = make_uint4(dw[4 * ch], dw[4 * ch + 1], dw[4 * ch + 2], dw[4 * ch + 3]);
      }
      FSTAMP(half, i, 6);
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar + kFBarDSFull);
      FSTAMP(half, i, 7);
    }

    // ---- epilogue: dV, dK accumulators -> scale -> 16-bit -> global
    if (ok && n_items > 0) ok = mbar_wait(bar + kFBarAccFull, 0, abort_flag);
    FSTAMP(half, 23, 0);
    if (ok) {
      tc_fence_after_sync();
      const bool valid = xr < len_k;
      // A whole 128-row tile leaves through shared memory (ring slots 0 and 1, idle by now) and TMA stores. Dense
      // tensors are clipped by the tensor map; a packed tile that ends inside its sequence's last rows would spill
      // into the next sequence and is written row by row instead.
      const bool use_tma = (p.cu_q == nullptr) || (x0 + kTile <= len_k);
#pragma unroll
      for (int which = 0; which < 2; ++which) {
        uint16_t* dst;
        float mul;
        uint32_t acc;
        if (which == 0) {
          dst = p.dv + ((p.cu_q != nullptr) ? static_cast<int64_t>(k_off + xr) * p.dv_row_stride
                                            : b * p.dv_batch_stride + static_cast<int64_t>(xr) * p.dv_row_stride) +
                hx * p.dv_head_stride;
          mul = kDrop ? p.keep_scale : 1.f;
          acc = acc_dv;
        } else {
          dst = p.dk + ((p.cu_q != nullptr) ? static_cast<int64_t>(k_off + xr) * p.dk_row_stride
                                            : b * p.dk_batch_stride + static_cast<int64_t>(xr) * p.dk_row_stride) +
                hx * p.dk_head_stride;
          mul = p.scale;
          acc = acc_dk;
        }
        // this warpgroup converts head_dim columns [half * kD/2, (half + 1) * kD/2)
#pragma unroll
        for (int cc = 0; cc < kD / 64; ++cc) {
          uint32_t v[32];
          if (n_items > 0) {
            tmem_ld_x32(acc + (lane_base - half * 64) + half * (kD / 2) + cc * 32, v);
            tmem_wait_ld();
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = 0u;
          }
          uint4 w[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            w[j].x = pack_16x2<kF16>(__uint_as_float(v[8 * j + 0]) * mul, __uint_as_float(v[8 * j + 1]) * mul);
            w[j].y = pack_16x2<kF16>(__uint_as_float(v[8 * j + 2]) * mul, __uint_as_float(v[8 * j + 3]) * mul);
            w[j].z = pack_16x2<kF16>(__uint_as_float(v[8 * j + 4]) * mul, __uint_as_float(v[8 * j + 5]) * mul);
            w[j].w = pack_16x2<kF16>(__uint_as_float(v[8 * j + 6]) * mul, __uint_as_float(v[8 * j + 7]) * mul);
          }
          const int col = half * (kD / 2) + cc * 32;  // first of this thread's 32 columns
          if (use_tma) {
            uint8_t* row = smem + kFSmemY + which * kTileBytes + (col >> 6) * kHalfBytes + r * 128;
            const int chunk0 = (col & 63) >> 3;
#pragma unroll
            for (int j = 0; j < 4; ++j) *reinterpret_cast<uint4*>(row + (((chunk0 + j) ^ (r & 7)) << 4)) = w[j];
          } else if (valid) {
            uint4* o4 = reinterpret_cast<uint4*>(dst + col);
#pragma unroll
            for (int j = 0; j < 4; ++j)
              if (col + 8 * j < p.head_dim) o4[j] = w[j];
          }
        }
      }
      if (use_tma) {
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar + kFBarEpiFull);
        if (threadIdx.x == 0) {
          if (mbar_wait(bar + kFBarEpiFull, 0, abort_flag)) {
            const int row0 = k_off + x0;
#pragma unroll
            for (int which = 0; which < 2; ++which) {
              const CUtensorMap* tm = (which == 0) ? &tm_dv : &tm_dk;
#pragma unroll
              for (int ht = 0; ht < kD / 64; ++ht)
                tma_store_4d(tm, base + kFSmemY + which * kTileBytes + ht * kHalfBytes, ht * 64, row0, hx, bcoord);
            }
            tma_store_commit();
            tma_store_wait_read();  // the shared memory must outlive the stores' reads of it
          }
        }
      }
    }
  }

  if (warp < 8) FSTAMP(warp >> 2, 23, 1);
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
  if (warp == 0) FSTAMP(0, 23, 2);
  if (threadIdx.x == 0 && *abort_flag != 0) atomicExch(p.status, static_cast<uint32_t>(SDPA_B200_DEVICE_TIMEOUT));
}

// dq = scale * accumulator, one block per 128-row tile of the accumulator: thread (row, column half) reads its
// 4-column groups (consecutive rows = consecutive 16 bytes) and writes 16 bytes of 16-bit results at a time.
struct DqConvertParams {
  const float* acc;
  uint16_t* dq;
  const int32_t* cu_q;  // null for dense
  int64_t dq_batch_stride, dq_head_stride, dq_row_stride;
  int heads_q, seqlen_q, lq_pad, total_q, acc_rows, head_dim;
  float scale;
};

template <int kD, bool kF16>
__global__ void __launch_bounds__(256) bwd_dq_convert_kernel(const DqConvertParams p) {
  const int r = threadIdx.x & 127;
  const int part = threadIdx.x >> 7;  // 0 / 1: first or second half of the 4-column groups
  const size_t tile = blockIdx.x;
  uint16_t* dst;
  if (p.cu_q != nullptr) {
    const int tiles_per_head = p.acc_rows >> 7;
    const int h = static_cast<int>(tile / tiles_per_head);
    const int tok = static_cast<int>(tile - static_cast<size_t>(h) * tiles_per_head) * 128 + r;
    if (tok >= p.total_q) return;
    dst = p.dq + static_cast<int64_t>(tok) * p.dq_row_stride + h * p.dq_head_stride;
  } else {
    const int tiles_per_head = p.lq_pad >> 7;
    const int bh = static_cast<int>(tile / tiles_per_head);
    const int q = static_cast<int>(tile - static_cast<size_t>(bh) * tiles_per_head) * 128 + r;
    if (q >= p.seqlen_q) return;
    const int b = bh / p.heads_q, h = bh - b * p.heads_q;
    dst = p.dq + b * p.dq_batch_stride + h * p.dq_head_stride + static_cast<int64_t>(q) * p.dq_row_stride;
  }
  const float4* src = reinterpret_cast<const float4*>(p.acc + tile * (static_cast<size_t>(kD / 4) * 512)) + r;
  constexpr int kGroups = kD / 8;  // 4-column groups per thread
  float4 v[kGroups];
#pragma unroll
  for (int g = 0; g < kGroups; ++g) v[g] = src[static_cast<size_t>(part * kGroups + g) * 128];
#pragma unroll
  for (int g = 0; g < kGroups; g += 2) {
    const int col = (part * kGroups + g) * 4;
    if (col < p.head_dim) {
      uint4 w;
      w.x = pack_16x2<kF16>(v[g].x * p.scale, v[g].y * p.scale);
      w.y = pack_16x2<kF16>(v[g].z * p.scale, v[g].w * p.scale);
      w.z = pack_16x2<kF16>(v[g + 1].x * p.scale, v[g + 1].y * p.scale);
      w.w = pack_16x2<kF16>(v[g + 1].z * p.scale, v[g + 1].w * p.scale);
      *reinterpret_cast<uint4*>(dst + col) = w;
    }
  }
}

using FusedKernel = void (*)(const CUtensorMap, const CUtensorMap, const CUtensorMap, const CUtensorMap, const CUtensorMap,
                             const CUtensorMap, const BwdKernelParams);

template <bool kDrop>
FusedKernel pick_fused(int head_dim, bool f16) {
  if (head_dim <= 64) return f16 ? bwd_fused_kernel<64, true, kDrop> : bwd_fused_kernel<64, false, kDrop>;
  return f16 ? bwd_fused_kernel<128, true, kDrop> : bwd_fused_kernel<128, false, kDrop>;
}

}  // namespace

size_t bwd_fused_acc_rows(const sdpa_b200_params& p, int lq_pad) {
  if (p.cu_seqlens_q != nullptr)
    return static_cast<size_t>(p.heads_q) * ((static_cast<size_t>(p.total_q) + kTile - 1) / kTile * kTile + kTile);
  return static_cast<size_t>(p.batch) * p.heads_q * lq_pad;
}

size_t bwd_fused_workspace_bytes(const sdpa_b200_params& p, int lq_pad) {
  const int kd = p.head_dim <= 64 ? 64 : 128;
  return bwd_fused_acc_rows(p, lq_pad) * kd * sizeof(float);
}

int launch_bwd_fused(const sdpa_b200_params& p, BwdKernelParams kp, float* dq_acc, int grid, cudaStream_t stream,
                     const CUtensorMap& tm_q, const CUtensorMap& tm_k, const CUtensorMap& tm_v, const CUtensorMap& tm_do,
                     const CUtensorMap& tm_dv, const CUtensorMap& tm_dk) {
  const bool f16 = p.dtype == SDPA_B200_F16;
  const int kd = p.head_dim <= 64 ? 64 : 128;
  const size_t acc_rows = bwd_fused_acc_rows(p, kp.lq_pad);
  cudaError_t err = cudaMemsetAsync(dq_acc, 0, acc_rows * kd * sizeof(float), stream);
  if (err != cudaSuccess) {
    set_error("backward: clearing the dQ accumulator failed: %s", cudaGetErrorString(err));
    return SDPA_B200_LAUNCH_FAILED;
  }
  kp.dq_acc = dq_acc;
  kp.dq_acc_rows = p.cu_seqlens_q != nullptr ? static_cast<int>(acc_rows / p.heads_q) : 0;
  FusedKernel kernel = kp.keep_cols != nullptr ? pick_fused<true>(p.head_dim, f16) : pick_fused<false>(p.head_dim, f16);
  err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kFSmemRequest);
  if (err != cudaSuccess) {
    set_error("backward: cudaFuncSetAttribute(%u bytes smem): %s", kFSmemRequest, cudaGetErrorString(err));
    return SDPA_B200_LAUNCH_FAILED;
  }
  kernel<<<grid, kFThreads, kFSmemRequest, stream>>>(tm_q, tm_k, tm_v, tm_do, tm_dv, tm_dk, kp);
  err = cudaGetLastError();
  if (err != cudaSuccess) {
    set_error("backward (fused): launch failed: %s", cudaGetErrorString(err));
    return SDPA_B200_LAUNCH_FAILED;
  }
  count_launch();

  DqConvertParams cp;
  cp.acc = dq_acc;
  cp.dq = static_cast<uint16_t*>(p.dq);
  cp.cu_q = p.cu_seqlens_q;
  cp.dq_batch_stride = p.dq_batch_stride;
  cp.dq_head_stride = p.dq_head_stride;
  cp.dq_row_stride = p.dq_row_stride;
  cp.heads_q = p.heads_q;
  cp.seqlen_q = p.max_seqlen_q;
  cp.lq_pad = kp.lq_pad;
  cp.total_q = p.total_q;
  cp.acc_rows = kp.dq_acc_rows;
  cp.head_dim = p.head_dim;
  cp.scale = p.softmax_scale;
  const unsigned tiles = static_cast<unsigned>(acc_rows / kTile);
  if (kd == 64) {
    if (f16) bwd_dq_convert_kernel<64, true><<<tiles, 256, 0, stream>>>(cp);
    else bwd_dq_convert_kernel<64, false><<<tiles, 256, 0, stream>>>(cp);
  } else {
    if (f16) bwd_dq_convert_kernel<128, true><<<tiles, 256, 0, stream>>>(cp);
    else bwd_dq_convert_kernel<128, false><<<tiles, 256, 0, stream>>>(cp);
  }
  err = cudaGetLastError();
  if (err != cudaSuccess) {
    set_error("backward dQ conversion: launch failed: %s", cudaGetErrorString(err));
    return SDPA_B200_LAUNCH_FAILED;
  }
  count_launch();
  return SDPA_B200_OK;
}

}  // namespace sdpa_b200
