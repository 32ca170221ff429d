// Backward attention kernels for sm_100a.
//
// Replaces the device work behind mha_varlen_bwd -> cnnlFlashAttentionBackward
// (torch_mlu/csrc/aten/operators/cnnl/internal/FlashAttention_internal.cpp:449-480):
// given dO, Q, K, V, O and the saved logsumexp, recompute P = exp(scale*QK^T - lse) and
//   dV = P^T dO,  dP = dO V^T,  dS = P o (dP - delta),  dQ = scale dS K,  dK = scale dS^T Q
// with delta = rowsum(dO o O). GQA: dK/dV of one KV head sum over its query heads inside one
// CTA, so nothing is accumulated with atomics and results are bit-reproducible. With dropout (kDrop
// instances) dV takes P o M / (1 - p) and dS = P o (M o dP / (1 - p) - delta); with an additive bias (kBias
// instances) the scores are scale*QK^T + bias and the dQ kernel also writes dS as the bias gradient.
//
// Three launches:
//   1. bwd_preprocess_kernel: delta and the log2-domain logsumexp into a padded
//      [batch, heads_q, ceil128(max_seqlen_q)] workspace (rows past a sequence get lse = +inf,
//      which later turns their P into exact zeros).
//   2. bwd_tile_kernel<kModeDKDV>: one CTA per (batch, kv head, 128-key block). K and V tiles
//      stay in shared memory; (Q, dO) tiles stream through a 2-stage TMA ring. Per Q tile:
//      S^T = K Q^T and dP^T = V dO^T on tcgen05 into TMEM, two compute warpgroups (thread = key
//      row = TMEM lane, one warpgroup per 64-query half of the tile) form P^T and dS^T, write
//      them back to TMEM as bf16, and MMAs with the TMEM operand accumulate dV += P^T dO and
//      dK += dS^T Q half by half (the streamed tiles are re-read in place as MN-major operands).
//   3. bwd_tile_kernel<kModeDQ>: one CTA per (batch, query head, 128-query block); Q and dO
//      stay, (K, V) stream; S = Q K^T, dP = dO V^T, dS -> TMEM, dQ += dS K.
// TMEM: T1 [0,128) T2 [128,256) ACC1 [256,384) ACC2 [384,512). The bf16 P and dS of an item both
// live in the item's score buffer, so the buffer that held dP is free as soon as it has been read;
// the MMA issuer uses that (and, for dQ, the unused ACC2) to run the next item's score GEMMs and
// exponentials under the current item's accumulation MMAs (buffer schedule at the issuer).
#include <cstdlib>

#include "bwd_common.cuh"

namespace sdpa_b200 {
namespace {

// Ring of 32 KB streamed tiles Y1(0), Y2(0), Y1(1), Y2(1), ...: 4 slots for dK/dV (which also stages
// the per-query vectors), 5 for dQ so that K(i+2) can land while item i is still accumulating.
constexpr int kMaxStages = 5;
__host__ __device__ constexpr int stages_for(int mode) { return mode == 1 ? 5 : 4; }
constexpr int kThreads = 352;  // warps 0-3 / 4-7 compute (column halves), warp 8 TMA, warps 9 and 10 MMA issuers
constexpr int kModeDKDV = 0;
constexpr int kModeDQ = 1;

constexpr uint32_t kSmemX = 0;                                   // stationary pair, 64 KB
constexpr uint32_t kSmemY = 2 * kTileBytes;                      // stages x 32 KB
__host__ __device__ constexpr uint32_t smem_vec_off(int mode) { return kSmemY + stages_for(mode) * kTileBytes; }
// per-slot (lse2[128], delta[128]), dK/dV only
__host__ __device__ constexpr uint32_t smem_bar_off(int mode) { return smem_vec_off(mode) + (mode == 1 ? 0 : stages_for(mode) * 1024); }
__host__ __device__ constexpr uint32_t smem_bytes_for(int mode) { return smem_bar_off(mode) + 256 + 1024; }
constexpr uint32_t kBarXFull = 0;
constexpr uint32_t kBarYFull = 8;
constexpr uint32_t kBarYEmpty = kBarYFull + 8 * kMaxStages;
constexpr uint32_t kBarSFull = kBarYEmpty + 8 * kMaxStages;   // 2: first score GEMM (X1 Y1^T) of an item done
constexpr uint32_t kBarDFull = kBarSFull + 16;             // second score GEMM (X2 Y2^T) done
constexpr uint32_t kBarDFree = kBarDFull + 8;              // all compute warps have read dP out of TMEM
constexpr uint32_t kBarPFull = kBarDFree + 16;             // all compute warps have stored P / dS
constexpr uint32_t kBarAccFull = kBarPFull + 16;
constexpr uint32_t kBarP1Full = kBarAccFull + 8;           // dK/dV: all compute warps have stored P (dS still to come)
constexpr uint32_t kBarWFree = kBarP1Full + 8;             // 2 (item parity): the accumulation GEMMs have read P / dS
constexpr uint32_t kBarSIssued = kBarWFree + 16;           // dK/dV: the next item's score GEMM is in the pipe
constexpr uint32_t kBarEpiFull = kBarSIssued + 8;           // all compute warps have staged their output rows
constexpr uint32_t kSmemTmemPtr = kBarEpiFull + 8;
constexpr uint32_t kSmemAbort = kSmemTmemPtr + 4;

// Profiling builds (-DSDPA_BWD_STAMPS) time-stamp pipeline events of one CTA per kernel; role 0/1 =
// lane 0 of the first warp of each compute warpgroup, roles 2 and 3 = the MMA issuer.
#ifdef SDPA_BWD_STAMPS
#define BWD_STAMP(role, item, ev)                                                                       \
  do {                                                                                                  \
    if (stamp_on && (item) < 24)                                                                        \
      p.stamps[((kMode * 4 + (role)) * 24 + (item)) * 8 + (ev)] = static_cast<float>(clock64() - t_start); \
  } while (0)
#else
#define BWD_STAMP(role, item, ev) do {} while (0)
#endif

template <int kMode, int kD, bool kF16, bool kDrop, bool kBias>
__global__ void __launch_bounds__(kThreads, 1)
bwd_tile_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_do,
                const __grid_constant__ CUtensorMap tm_o1, const __grid_constant__ CUtensorMap tm_o2,
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
  // The dQ kernel follows in the stream and depends on nothing written here: once every dK/dV CTA has begun (this
  // signal), its CTAs may take over SMs as they free up, instead of waiting for the last dK/dV CTA to finish.
  if (kMode == kModeDKDV && threadIdx.x == 0) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  constexpr int kStages = stages_for(kMode);
  constexpr uint32_t kSmemVec = smem_vec_off(kMode);
  constexpr uint32_t kSmemBar = smem_bar_off(kMode);

  // CTA order (1-D grid): (batch, head) pairs in groups of `heads_per_wave` whose streamed tensors
  // fit L2 together; inside a group the 128-row blocks go heaviest first across all its heads
  // (dK/dV: key block 0 sees every query; dQ: the last query block sees every key), so the launch
  // ends on its lightest blocks.
  int b, hx, xb;
  {
    const int per_group = p.heads_per_wave * p.num_row_blocks;
    const int grp = blockIdx.x / per_group;
    const int w = blockIdx.x - grp * per_group;
    const int size = min(p.heads_per_wave, p.num_bh - grp * p.heads_per_wave);
    const int rank = w / size;
    const int bh = grp * p.heads_per_wave + (w - rank * size);
    if (rank >= p.num_row_blocks) {  // padding slots of a short last group
      if (kMode == kModeDQ) wait_for_previous_grid();
      return;
    }
    xb = (kMode == kModeDKDV) ? rank : p.num_row_blocks - 1 - rank;
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
  const int len_x = (kMode == kModeDKDV) ? len_k : len_q;
  const int x0 = xb * kTile;
  if (x0 >= len_x) {
    if (kMode == kModeDQ) wait_for_previous_grid();
    return;
  }

  // streamed tile range [y_lo, y_hi) (in tiles of 128) per head, and heads per CTA
  int y_lo = 0, y_hi = 0;
  if (kMode == kModeDKDV) {
    y_hi = (len_q + kTile - 1) / kTile;
    if (p.is_causal) y_lo = max(0, (x0 - causal_off) / kTile);  // first query tile with a row >= x0 - off
    if (p.is_causal && x0 - causal_off > len_q - 1) y_lo = y_hi;
  } else {
    int vis_end = len_k;
    if (p.is_causal) vis_end = min(len_k, x0 + kTile + causal_off);
    y_hi = vis_end > 0 ? (vis_end + kTile - 1) / kTile : 0;
  }
  const int tiles_per_head = max(0, y_hi - y_lo);
  const int heads_here = (kMode == kModeDKDV) ? p.kv_group : 1;
  const int n_items = tiles_per_head * heads_here;

  const uint32_t bar = base + kSmemBar;
  volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(smem + kSmemBar + kSmemAbort);
  volatile uint32_t* tmem_ptr_smem = reinterpret_cast<volatile uint32_t*>(smem + kSmemBar + kSmemTmemPtr);

  // TMA producer state. The producer thread also initialises the barriers and issues the first loads
  // (the stationary pair and the first kPreloaded ring tiles, whose slots are free by construction)
  // BEFORE the set-up barrier, so that their latency runs under the TMEM allocation.
  const CUtensorMap* tmx1 = (kMode == kModeDKDV) ? &tm_k : &tm_q;
  const CUtensorMap* tmx2 = (kMode == kModeDKDV) ? &tm_v : &tm_do;
  const CUtensorMap* tmy1 = (kMode == kModeDKDV) ? &tm_q : &tm_k;
  const CUtensorMap* tmy2 = (kMode == kModeDKDV) ? &tm_do : &tm_v;
  const int x_row = ((kMode == kModeDKDV) ? k_off : q_off) + x0;
  const int y_off = (kMode == kModeDKDV) ? q_off : k_off;
  constexpr uint32_t kLoadBytes = kTile * kD * 2;  // bytes one tile brings in
  constexpr int kPreloaded = 4;
  // ring tile idx: Y1(idx/2) if even, Y2(idx/2) if odd; false when a wait gave up
  auto load_tile = [&](int idx) -> bool {
        const int i = idx >> 1;
        int s = idx % kStages;
        uint32_t use = static_cast<uint32_t>(idx / kStages);
        if (kMode == kModeDQ) {  // K ring: slots 0-2, V ring: slots 3-4
          s = (idx & 1) ? 3 + (i & 1) : i % 3;
          use = static_cast<uint32_t>((idx & 1) ? (i >> 1) : i / 3);
        }
        // Slot reuse. dK/dV: the pair of slots of item i - 2 is released by one commit behind its
        // accumulation GEMMs. dQ has no release commits (they cost the issuer time) and watches a
        // barrier the GEMMs signal anyway: the score-full barrier of S(i-1), waited for before K(i).
        //   K(i) reuses the slot of K(i-3), last read by dQ(i-3); V(i) reuses the slot of V(i-2), read
        //   by dP(i-2) only. S(i-1) overwrites the buffer of dS(i-3), so its issuer has waited for
        //   dQ(i-3) (`W free`), and it issues dP(i-2) before S(i-1) itself (prologue: S0 dP0 S1; item j:
        //   dP(j+1), S(j+2)); the tensor pipe keeps the order of one thread's MMAs. So "S(i-1) done"
        //   covers both slots; V(i) is loaded right behind K(i) and needs no wait of its own.
        //   A parity wait can only tell "this phase is over" from "it is not" while the barrier is at
        //   most one phase further on. That holds here: the next phase of this barrier is S(i+1), and
        //   S(i+1) needs K(i+1), which this loop loads later. (The dP-full barrier would NOT do for
        //   V(i): dP(i-1) can finish as well before the producer looks, and two phases on the parity
        //   reads "not yet" again.)
        if (kMode == kModeDKDV) {
          if (!mbar_wait(bar + kBarYEmpty + 8 * (s & ~1), (use & 1u) ^ 1u, abort_flag)) return false;
        } else if ((idx & 1) == 0 && i >= 2) {
          if (!mbar_wait(bar + kBarSFull + 8 * ((i - 1) & 1), ((i - 1) >> 1) & 1, abort_flag)) return false;
        }
        const int hi = i / tiles_per_head;
        const int yt = y_lo + (i - hi * tiles_per_head);
        // dK/dV streams the query heads of this KV head; dQ streams the KV head of this query head
        const int hy = (kMode == kModeDKDV) ? hx * p.kv_group + hi : hx / p.kv_group;
        const uint32_t full = bar + kBarYFull + 8 * s;
        const uint32_t dst = base + kSmemY + s * kTileBytes;
        const int row = y_off + yt * kTile;
        const bool first = (idx & 1) == 0;
        if (kMode == kModeDKDV && first) {
          mbar_arrive_expect_tx(full, kLoadBytes + 1024);
          const size_t vec = (static_cast<size_t>(b) * p.heads_q + hy) * p.lq_pad + static_cast<size_t>(yt) * kTile;
          bulk_load_1d(base + kSmemVec + s * 1024, p.lse2 + vec, 512, full);
          bulk_load_1d(base + kSmemVec + s * 1024 + 512, p.delta + vec, 512, full);
        } else {
          mbar_arrive_expect_tx(full, kLoadBytes);
        }
        const CUtensorMap* tm = first ? tmy1 : tmy2;
        tma_load_4d(dst, tm, full, 0, row, hy, bcoord);
        if (kD > 64) tma_load_4d(dst + kHalfBytes, tm, full, 64, row, hy, bcoord);
    return true;
  };

  if (warp == 8 && lane == 0) {
    // descriptor fetches run under the barrier initialisation
    tma_prefetch_desc(tmx1);
    tma_prefetch_desc(tmy1);
    tma_prefetch_desc(tmx2);
    tma_prefetch_desc(tmy2);
    mbar_init(bar + kBarXFull, 1);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(bar + kBarYFull + 8 * s, 1);
      mbar_init(bar + kBarYEmpty + 8 * s, 1);
    }
    mbar_init(bar + kBarSFull, 1);
    mbar_init(bar + kBarSFull + 8, 1);
    mbar_init(bar + kBarDFull, 1);
    mbar_init(bar + kBarDFree, 8);  // one arrival per compute warp
    mbar_init(bar + kBarPFull, 8);
    mbar_init(bar + kBarP1Full, 8);
    mbar_init(bar + kBarWFree, 1);
    mbar_init(bar + kBarWFree + 8, 1);
    mbar_init(bar + kBarSIssued, 1);
    mbar_init(bar + kBarEpiFull, 8);
    mbar_init(bar + kBarAccFull, 1);
    *abort_flag = 0;
    fence_mbar_init();
    if (n_items > 0) {
      mbar_arrive_expect_tx(bar + kBarXFull, 2 * kLoadBytes);
      tma_load_4d(base + kSmemX, tmx1, bar + kBarXFull, 0, x_row, hx, bcoord);
      if (kD > 64) tma_load_4d(base + kSmemX + kHalfBytes, tmx1, bar + kBarXFull, 64, x_row, hx, bcoord);
      tma_load_4d(base + kSmemX + kTileBytes, tmx2, bar + kBarXFull, 0, x_row, hx, bcoord);
      if (kD > 64) tma_load_4d(base + kSmemX + kTileBytes + kHalfBytes, tmx2, bar + kBarXFull, 64, x_row, hx, bcoord);
      for (int idx = 0; idx < kPreloaded && idx < 2 * n_items; ++idx) load_tile(idx);
    }
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
  const uint32_t t1 = tmem_base, t2 = tmem_base + 128, acc1 = tmem_base + 256, acc2 = tmem_base + 384;
#ifdef SDPA_BWD_STAMPS
  const long long t_start = clock64();
  // a long-running block of batch 0, head 0 (non-causal: any; causal: the heaviest)
  const bool stamp_on = p.stamps != nullptr && b == 0 && hx == 0 &&
                        xb == ((kMode == kModeDKDV) ? 0 : p.num_row_blocks - 1) && (lane == 0) &&
                        (warp == 0 || warp == 4 || warp == 9 || warp == 10);
#endif

  if (warp == 8) {
    // ------------------------------------------------------------------ TMA producer (rest of the ring)
    if (lane == 0 && n_items > 0) {
      for (int idx = kPreloaded; idx < 2 * n_items; ++idx)
        if (!load_tile(idx)) break;
      drain_after_abort(abort_flag);
    }
  } else if (warp == 9 || warp == 10) {
    // ------------------------------------------------------------------ MMA issuers
    // One thread needs ~50-65 cycles to issue an MMA and ~70 for every barrier wait or commit, about
    // as long as the tensor pipe needs to execute it, and an item has 24 (dQ) or 32 (dK/dV) MMAs
    // plus half a dozen waits: a single issuer is the bottleneck. So two threads issue:
    //   warp 9  the score GEMMs   S = X1 Y1^T, dP = X2 Y2^T            (operands in shared memory)
    //   warp 10 the accumulations dV += P^T dO, dK += dS^T Q / dQ += dS K (A operand in TMEM)
    // What the in-order pipe would guarantee between the two groups is a barrier here: `W free`
    // (warp 10 commits it behind an item's accumulation MMAs; warp 9 waits for it before a score GEMM
    // overwrites that item's P / dS buffer). There is one per item parity, so that the barrier a wait
    // looks at cannot be a whole phase further on: its next phase belongs to item i+2, whose scores
    // only exist after this wait.
    if (lane == 0 && n_items > 0) {
      // Where the score GEMMs of item i land:
      //   dK/dV: S(i) in T[i&1], dP(i) in T[(i&1)^1]. The compute warpgroups put BOTH 16-bit results
      //          (P and dS) into the S buffer, so the dP buffer is free once it has been read and
      //          takes S(i+1) right away; dP(i+1) goes into the S buffer behind the accumulations.
      //   dQ:    ACC2 is unused, so S alternates between T1 and ACC2 and dP always uses T2: S(i+2)
      //          follows the accumulation of item i, dP(i+1) goes out as soon as dP(i) is read.
      // Either way the next item's scores and exponentials run under this item's accumulation.
      const uint32_t x1 = base + kSmemX, x2 = base + kSmemX + kTileBytes;
      auto s_buf = [&](int i) { return kMode == kModeDKDV ? ((i & 1) ? t2 : t1) : ((i & 1) ? acc2 : t1); };
      auto d_buf = [&](int i) { return kMode == kModeDKDV ? ((i & 1) ? t1 : t2) : t2; };
      auto s_bar = [&](int i) { return bar + kBarSFull + (kMode == kModeDQ ? 8 * (i & 1) : 0); };
      // ring position of tile 2i, kept incrementally (no division in the issue loop): slot = (2i) mod
      // kStages, lap = (2i) / kStages. Tiles 2i + k, k < kStages, follow from it with one wrap.
      // dQ splits its five slots into a K ring (slots 0-2) and a V ring (slots 3-4): a K tile lives
      // from its score GEMM to its accumulation GEMM two items later, a V tile only for one GEMM, so a
      // shared round-robin would free the slot V(i+1) needs too late to hide the load latency.
      int ring_slot = 0, ring_lap = 0;  // dK/dV: position of tile 2i; dQ: i mod 3 and i / 3
      int item = 0;
      auto pos = [&](int k, int& slot, int& lap) {
        if (kMode == kModeDKDV) {
          slot = ring_slot + k;
          lap = ring_lap;
          if (slot >= kStages) { slot -= kStages; ++lap; }
        } else if ((k & 1) == 0) {  // K(item + k/2)
          slot = ring_slot + (k >> 1);
          lap = ring_lap;
          if (slot >= 3) { slot -= 3; ++lap; }
        } else {  // V(item + k/2)
          const int j = item + (k >> 1);
          slot = 3 + (j & 1);
          lap = j >> 1;
        }
      };
      auto advance = [&]() {
        ++item;
        if (kMode == kModeDKDV) {
          ring_slot += 2;
          if (ring_slot >= kStages) { ring_slot -= kStages; ++ring_lap; }
        } else if (++ring_slot == 3) {
          ring_slot = 0;
          ++ring_lap;
        }
      };
      auto y_slot_k = [&](int k) { int sl, lp; pos(k, sl, lp); return base + kSmemY + sl * kTileBytes; };
      auto y_wait_k = [&](int k) { int sl, lp; pos(k, sl, lp); return mbar_wait(bar + kBarYFull + 8 * sl, lp & 1, abort_flag); };
      auto y_free_k = [&](int k) { int sl, lp; pos(k, sl, lp); umma_commit(bar + kBarYEmpty + 8 * sl); };
      bool ok = true;
      if (warp == 9) {
        // ---------------- score GEMMs
#ifdef SDPA_BWD_STAMPS
        if (stamp_on) p.stamps[((kMode * 4 + 2) * 24 + 23) * 8 + 0] = static_cast<float>(t_start - t_entry);
#endif
        ok = mbar_wait(bar + kBarXFull, 0, abort_flag) && y_wait_k(0);
        BWD_STAMP(2, 23, 1);
        if (ok) {
          tc_fence_after_sync();
          issue_xyT<kD, kF16>(s_buf(0), x1, y_slot_k(0));
          umma_commit(s_bar(0));
        }
        BWD_STAMP(2, 23, 2);
        ok = ok && y_wait_k(1);
        if (ok) {
          tc_fence_after_sync();
          issue_xyT<kD, kF16>(d_buf(0), x2, y_slot_k(1));
          umma_commit(bar + kBarDFull);
        }
        if (kMode == kModeDQ && ok && n_items > 1) {
          ok = y_wait_k(2);
          if (ok) {
            tc_fence_after_sync();
            issue_xyT<kD, kF16>(s_buf(1), x1, y_slot_k(2));
            umma_commit(s_bar(1));
          }
        }
        for (int i = 0; ok && i < n_items; ++i, advance()) {
          const uint32_t sbuf = s_buf(i);
          const bool more = i + 1 < n_items;
          BWD_STAMP(2, i, 0);
          // dP(i) has left TMEM once all compute warps have read it
          ok = mbar_wait(bar + kBarDFree, i & 1, abort_flag);
          if (!ok) break;
          BWD_STAMP(2, i, 1);
          if (kMode == kModeDKDV) {
            if (!more) {
              mbar_arrive(bar + kBarSIssued);
              continue;
            }
            ok = y_wait_k(2);
            if (!ok) break;
            tc_fence_after_sync();
            issue_xyT<kD, kF16>(d_buf(i), x1, y_slot_k(2));  // S(i+1) into the buffer dP(i) has just left
            umma_commit(s_bar(i + 1));
            // S(i+1) is what the compute warps wait for; dK(i) is not urgent. The other issuer holds
            // dK(i) back until this arrival, so the two GEMMs do not share the pipe MMA by MMA.
            mbar_arrive(bar + kBarSIssued);
            BWD_STAMP(2, i, 2);
            ok = mbar_wait(bar + kBarWFree + 8 * (i & 1), (i >> 1) & 1, abort_flag) && y_wait_k(3);
            if (!ok) break;
            BWD_STAMP(2, i, 3);
            tc_fence_after_sync();
            issue_xyT<kD, kF16>(sbuf, x2, y_slot_k(3));  // dP(i+1) into the buffer P(i), dS(i) have left
            umma_commit(bar + kBarDFull);
            BWD_STAMP(2, i, 4);
          } else {
            if (more) {
              ok = y_wait_k(3);
              if (!ok) break;
              tc_fence_after_sync();
              issue_xyT<kD, kF16>(t2, x2, y_slot_k(3));  // dP(i+1)
              umma_commit(bar + kBarDFull);
            }
            BWD_STAMP(2, i, 2);
            if (i + 2 < n_items) {
              ok = mbar_wait(bar + kBarWFree + 8 * (i & 1), (i >> 1) & 1, abort_flag) && y_wait_k(4);
              if (!ok) break;
              BWD_STAMP(2, i, 3);
              tc_fence_after_sync();
              issue_xyT<kD, kF16>(sbuf, x1, y_slot_k(4));  // S(i+2) into the buffer dS(i) has left
              umma_commit(s_bar(i + 2));
              BWD_STAMP(2, i, 4);
            }
          }
        }
      } else {
        // ---------------- accumulation GEMMs
        ok = mbar_wait(bar + kBarXFull, 0, abort_flag);
        for (int i = 0; ok && i < n_items; ++i, advance()) {
          const uint32_t y1 = y_slot_k(0), y2 = y_slot_k(1);
          const uint32_t sbuf = s_buf(i);
          // the tiles have landed long ago (the other issuer has used them); this wait makes the
          // copies visible to this thread's MMAs as well
          ok = y_wait_k(0) && (kMode == kModeDQ || y_wait_k(1));
          if (!ok) break;
          if (kMode == kModeDKDV) {
            // dV needs P only, which is stored a whole dS pass before the item is complete
            ok = mbar_wait(bar + kBarP1Full, i & 1, abort_flag);
            if (!ok) break;
            tc_fence_after_sync();
            issue_wy_half<kD, kF16>(acc1, sbuf, y2, 0, i > 0);       // dV += P^T dO
            issue_wy_half<kD, kF16>(acc1, sbuf + 64, y2, 1, true);
          }
          BWD_STAMP(3, i, 0);
          ok = mbar_wait(bar + kBarPFull, i & 1, abort_flag);
          if (!ok) break;
          BWD_STAMP(3, i, 1);
          tc_fence_after_sync();
          if (kMode == kModeDKDV) {
            ok = mbar_wait(bar + kBarSIssued, i & 1, abort_flag);
            if (!ok) break;
            issue_wy_half<kD, kF16>(acc2, sbuf + 32, y1, 0, i > 0);  // dK += dS^T Q
            issue_wy_half<kD, kF16>(acc2, sbuf + 96, y1, 1, true);
            y_free_k(0);  // releases the slot pair Q(i), dO(i)
          } else {
            issue_wy_half<kD, kF16>(acc1, sbuf + 32, y1, 0, i > 0);  // dQ += dS K
            issue_wy_half<kD, kF16>(acc1, sbuf + 96, y1, 1, true);
          }
          umma_commit(bar + kBarWFree + 8 * (i & 1));
          if (i == n_items - 1) umma_commit(bar + kBarAccFull);
          BWD_STAMP(3, i, 2);
          if (i == 0) BWD_STAMP(3, 23, 0);
          if (i == n_items - 1) BWD_STAMP(3, 23, 1);
        }
      }
    }
  } else if (warp < 8) {
    // ------------------------------------------------------------------ compute warpgroups
    // warps 0-3 own streamed columns [0,64) of every stationary row, warps 4-7 columns [64,128)
    const int half = warp >> 2;
    const int r = (warp & 3) * 32 + lane;  // stationary row in the tile = TMEM lane
    const int xr = x0 + r;                 // key index (dK/dV) or query index (dQ) within the sequence
    const uint32_t lane_base = (static_cast<uint32_t>((warp & 3) * 32) << 16) + half * 64;
    const float c = p.scale_log2;
    bool ok = true;
    float my_lse2 = 0.f, my_delta = 0.f;
    if (kMode == kModeDQ) {
      const size_t vec = (static_cast<size_t>(b) * p.heads_q + hx) * p.lq_pad + xr;
      my_lse2 = p.lse2[vec];
      my_delta = p.delta[vec];
    }
    for (int i = 0; i < n_items; ++i) {
      const int s = (2 * i) % kStages;  // ring slot of Y1(i), which carries the per-query vectors
      const int hi = i / tiles_per_head;
      const int y0 = (y_lo + (i - hi * tiles_per_head)) * kTile;
      const uint32_t sbuf = (kMode == kModeDKDV ? ((i & 1) ? t2 : t1) : ((i & 1) ? acc2 : t1)) + lane_base;
      const uint32_t dbuf = (kMode == kModeDKDV ? ((i & 1) ? t1 : t2) : t2) + lane_base;
      BWD_STAMP(half, i, 0);
      // keep bits of this thread's 64 (row, column) pairs, in flight under the waits below
      uint2 keep = make_uint2(0u, 0u);
      if constexpr (kDrop) {
        const uint32_t* words =
            (kMode == kModeDQ)
                ? p.keep_rows + (p.cu_q != nullptr ? static_cast<size_t>(hx) * p.keep_q_rows + q_off + xr
                                                   : static_cast<size_t>(b * p.heads_q + hx) * p.keep_q_rows + xr) *
                                    (p.keep_lk_pad >> 5)
                : p.keep_cols + (p.cu_q != nullptr
                                     ? static_cast<size_t>(hx * p.kv_group + hi) * p.keep_k_rows + k_off + xr
                                     : static_cast<size_t>(b * p.heads_q + hx * p.kv_group + hi) * p.keep_k_rows + xr) *
                                    (p.keep_lq_pad >> 5);
        keep = *reinterpret_cast<const uint2*>(words + ((y0 + half * 64) >> 5));
      }
      if constexpr (kBias) {
        // the next item's bias values of this thread's row: into L2 now (dQ: 128 contiguous bytes of the query
        // row; dK/dV: 64 query rows, two per lane, 64 bytes each around this warp's keys)
        if (i + 1 < n_items && xr < len_x) {
          const int hn = (i + 1) / tiles_per_head;
          const int cn = (y_lo + (i + 1 - hn * tiles_per_head)) * kTile + half * 64;
          if (kMode == kModeDQ) {
            const uint16_t* nx = p.bias + b * p.bias_batch_stride + hx * p.bias_head_stride +
                                 static_cast<int64_t>(xr) * p.bias_row_stride + cn;
            if (cn < len_k) {  // only addresses inside the row
              prefetch_l2(nx);
              prefetch_l2(nx + min(63, len_k - 1 - cn));
            }
          } else {
            if (p.bias_row_stride == 0) {
              // one value per key: nothing worth fetching ahead
            } else if (p.bias_t != nullptr) {
              const uint16_t* nx = p.bias_t + b * p.bias_t_batch_stride + (hx * p.kv_group + hn) * p.bias_t_head_stride +
                                   static_cast<int64_t>(xr) * p.bias_t_row_stride + cn;
              if (cn < len_q) {
                prefetch_l2(nx);
                prefetch_l2(nx + min(63, len_q - 1 - cn));
              }
            } else {
              const uint16_t* nx = p.bias + b * p.bias_batch_stride + (hx * p.kv_group + hn) * p.bias_head_stride + xr;
              const int q = cn + 2 * lane;
              if (q < len_q) prefetch_l2(nx + static_cast<int64_t>(q) * p.bias_row_stride);
              if (q + 1 < len_q) prefetch_l2(nx + static_cast<int64_t>(q + 1) * p.bias_row_stride);
            }
          }
        }
      }
      // This item's bias values where they are contiguous for this thread (dQ: its query row; dK/dV: its key's row
      // of the transposed copy): eight 16-byte loads issued before the waits, so their latency passes under the
      // score GEMM. A chunk that starts past the end is skipped (zeros); one that straddles it reads row padding.
      uint4 bw[kBias ? 8 : 1];
      bool bias_in_regs = false;
      if constexpr (kBias) {
        const int col0 = y0 + half * 64;
        const uint16_t* vrow = nullptr;
        int vlen = 0;
        if (kMode == kModeDQ) {
          vrow = p.bias + b * p.bias_batch_stride + hx * p.bias_head_stride + static_cast<int64_t>(xr) * p.bias_row_stride;
          vlen = len_k;
        } else if (p.bias_row_stride != 0 && p.bias_t != nullptr) {
          vrow = p.bias_t + b * p.bias_t_batch_stride + (hx * p.kv_group + hi) * p.bias_t_head_stride +
                 static_cast<int64_t>(xr) * p.bias_t_row_stride;
          vlen = len_q;
        }
        bias_in_regs = vrow != nullptr;
        if (bias_in_regs) {
#pragma unroll
          for (int ch = 0; ch < 8; ++ch) {
            bw[ch] = make_uint4(0u, 0u, 0u, 0u);
            if (xr < len_x && col0 + ch * 8 < vlen) bw[ch] = *reinterpret_cast<const uint4*>(vrow + col0 + ch * 8);
          }
        }
      }
      // `ok` is made warp-uniform after every wait: the warp-level arrivals below need all 32 lanes
      ok = mbar_wait(bar + kBarSFull + (kMode == kModeDQ ? 8 * (i & 1) : 0), (kMode == kModeDQ ? (i >> 1) : i) & 1,
                     abort_flag);
      if (kMode == kModeDKDV) {
        // the per-query vectors arrive with the stage's bulk copies; observe that barrier directly
        ok = ok && mbar_wait(bar + kBarYFull + 8 * s, ((2 * i) / kStages) & 1, abort_flag);
      }
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after_sync();
      BWD_STAMP(half, i, 1);
      const float* vec_lse = reinterpret_cast<const float*>(smem + kSmemVec + s * 1024) + half * 64;
      const float* vec_delta = vec_lse + 128;
      // visibility of element (row xr, column y0 + j)
      //   dK/dV: key xr, query y0+j : visible iff xr <= y0 + j + off  <=>  j >= xr - off - y0
      //   dQ   : query xr, key y0+j : visible iff y0 + j <= xr + off and y0 + j < len_k
      int j_lo = 0, j_hi = kTile;
      if (kMode == kModeDKDV) {
        if (p.is_causal) j_lo = xr - causal_off - y0;
      } else {
        j_hi = len_k - y0;
        if (p.is_causal) j_hi = min(j_hi, xr + causal_off + 1 - y0);
      }
      j_lo -= half * 64;  // relative to this thread's 64 columns
      j_hi -= half * 64;

      // phase 1 (needs S only): P = exp2(S c - lse2), masked; its bf16 copy goes back at once
      float pr[64];
      {
        uint32_t a[64];
        tmem_ld_x32_at<0>(sbuf, a);
        tmem_ld_x32_at<32>(sbuf + 32, a);
        tmem_wait_ld();
        BWD_STAMP(half, i, 2);
        if constexpr (kBias) {
          // S <- S + bias / scale (then x = S c - lse2 as without bias)
          const int col0 = y0 + half * 64;
          if (bias_in_regs) {
#pragma unroll
            for (int ch = 0; ch < 8; ++ch) {
              const uint32_t ww[4] = {bw[ch].x, bw[ch].y, bw[ch].z, bw[ch].w};
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const float2 b2 = unpack_16x2<kF16>(ww[e]);
                a[ch * 8 + 2 * e] = __float_as_uint(fmaf(b2.x, p.inv_scale, __uint_as_float(a[ch * 8 + 2 * e])));
                a[ch * 8 + 2 * e + 1] = __float_as_uint(fmaf(b2.y, p.inv_scale, __uint_as_float(a[ch * 8 + 2 * e + 1])));
              }
            }
          } else if (kMode == kModeDKDV && xr < len_x) {
            const uint16_t* bcol = p.bias + b * p.bias_batch_stride + (hx * p.kv_group + hi) * p.bias_head_stride + xr;
            if (p.bias_row_stride == 0) {
              // the bias does not depend on the query (ALiBi-like): one value for this thread's key
              const float bs = unpack_16x2<kF16>(static_cast<uint32_t>(bcol[0])).x * p.inv_scale;
#pragma unroll
              for (int j = 0; j < 64; ++j) a[j] = __float_as_uint(__uint_as_float(a[j]) + bs);
            } else {
              // no transposed copy: this key in 64 consecutive query rows, 64 two-byte loads (consecutive lanes on
              // consecutive keys)
#pragma unroll
              for (int j = 0; j < 64; ++j) {
                if (col0 + j < len_q) {
                  const uint32_t raw = bcol[static_cast<int64_t>(col0 + j) * p.bias_row_stride];
                  const float bv = unpack_16x2<kF16>(raw).x;
                  a[j] = __float_as_uint(fmaf(bv, p.inv_scale, __uint_as_float(a[j])));
                }
              }
            }
          }
        }
        // x = S c - lse2. In the dK/dV kernel this pass sits on the critical chain (score GEMM ->
        // exponentials -> dP read -> next score GEMM) and the exponential unit alone would bound it, so
        // kPolyOf4 of every four column pairs take their 2^x from the FMA pipe (exp2_poly3_x2). The dQ
        // kernel's compute warps are bound by issue slots as much as by the exponential unit; there one
        // pair in four is the measured optimum (two of four already cost time), here two of four.
        constexpr int kPolyOf4 = (kMode == kModeDKDV) ? SDPA_BWD_POLY_DKDV : SDPA_BWD_POLY_DQ;
#pragma unroll
        for (int j = 0; j < 64; j += 2) {
          const float l0 = (kMode == kModeDKDV) ? vec_lse[j] : my_lse2;
          const float l1 = (kMode == kModeDKDV) ? vec_lse[j + 1] : my_lse2;
          const float x0 = fmaf(__uint_as_float(a[j]), c, -l0);
          const float x1 = fmaf(__uint_as_float(a[j + 1]), c, -l1);
          if (((j >> 1) & 3) < kPolyOf4) {
            const float2 e = exp2_poly3_x2(make_float2(x0, x1));
            pr[j] = e.x;
            pr[j + 1] = e.y;
          } else {
            pr[j] = ex2_approx(x0);
            pr[j + 1] = ex2_approx(x1);
          }
        }
        // only tiles on the causal diagonal or past the end of the keys need the element mask
        if (__any_sync(0xffffffffu, j_lo > 0 || j_hi < 64)) {
#pragma unroll
          for (int j = 0; j < 64; ++j) pr[j] = (j >= j_lo && j < j_hi) ? pr[j] : 0.f;
        }
        if (kMode == kModeDKDV) {
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
          if (lane == 0) mbar_arrive(bar + kBarP1Full);
        }
      }
      // phase 2 (needs dP): dS = P o (dP - delta) into the second half of this thread's columns
      BWD_STAMP(half, i, 3);
      ok = __all_sync(0xffffffffu, mbar_wait(bar + kBarDFull, i & 1, abort_flag));
      if (!ok) break;
      tc_fence_after_sync();
      BWD_STAMP(half, i, 4);
      {
        uint32_t d[64];
        tmem_ld_x32_at<0>(dbuf, d);
        tmem_ld_x32_at<32>(dbuf + 32, d);
        tmem_wait_ld();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar + kBarDFree);  // the dP buffer may be overwritten
        BWD_STAMP(half, i, 5);
        uint32_t dw[32];
#pragma unroll
        for (int j2 = 0; j2 < 32; ++j2) {
          const float dl0 = (kMode == kModeDKDV) ? vec_delta[2 * j2] : my_delta;
          const float dl1 = (kMode == kModeDKDV) ? vec_delta[2 * j2 + 1] : my_delta;
          float dp0 = __uint_as_float(d[2 * j2]), dp1 = __uint_as_float(d[2 * j2 + 1]);
          if constexpr (kDrop) {
            const uint32_t two = (j2 < 16 ? keep.x : keep.y) >> ((2 * j2) & 31);
            dp0 = (two & 1u) ? dp0 * p.keep_scale : 0.f;
            dp1 = (two & 2u) ? dp1 * p.keep_scale : 0.f;
          }
          dw[j2] = pack_16x2<kF16>(pr[2 * j2] * (dp0 - dl0), pr[2 * j2 + 1] * (dp1 - dl1));
        }
        tmem_st_x16(sbuf + 32, dw);
        tmem_st_x16(sbuf + 48, dw + 16);
        if constexpr (kBias && kMode == kModeDQ) {
          // dbias = dS: this thread's 64 keys of its query row, already packed for the dQ GEMM
          const int col0 = y0 + half * 64;
          if (p.dbias != nullptr && xr < len_x) {
            uint16_t* drow = p.dbias + b * p.dbias_batch_stride + hx * p.dbias_head_stride +
                             static_cast<int64_t>(xr) * p.dbias_row_stride + col0;
#pragma unroll
            for (int ch = 0; ch < 8; ++ch)
              if (col0 + ch * 8 < len_k)
                *reinterpret_cast<uint4*>(drow + ch * 8) = make_uint4(dw[4 * ch], dw[4 * ch + 1], dw[4 * ch + 2], dw[4 * ch + 3]);
          }
        }
      }
      BWD_STAMP(half, i, 6);
      tmem_wait_st();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar + kBarPFull);
      BWD_STAMP(half, i, 7);
    }

    // ---- epilogue: accumulators -> scale -> 16-bit -> global
    if (ok && n_items > 0) ok = mbar_wait(bar + kBarAccFull, 0, abort_flag);
    BWD_STAMP(half, 23, 0);
    if (ok) {
      tc_fence_after_sync();
      const bool valid = xr < len_x;
      // A whole 128-row tile leaves through shared memory and TMA stores (the ring slots are idle by
      // now): coalesced and asynchronous, where row-wise stores from registers - 128 bytes per thread,
      // every lane on another row - kept the load/store unit busy for ~4000 cycles per CTA. Dense
      // tensors are clipped by the tensor map; a packed (varlen) tile that ends inside its sequence's
      // last rows would spill into the next sequence and is written row by row instead.
      const bool use_tma = (p.cu_q == nullptr) || (x0 + kTile <= len_x);
      const int n_out = (kMode == kModeDKDV) ? 2 : 1;
#pragma unroll
      for (int which = 0; which < n_out; ++which) {
        uint16_t* dst;
        float mul;
        uint32_t acc;
        if (kMode == kModeDQ) {
          dst = p.dq + ((p.cu_q != nullptr) ? static_cast<int64_t>(q_off + xr) * p.dq_row_stride
                                            : b * p.dq_batch_stride + static_cast<int64_t>(xr) * p.dq_row_stride) +
                hx * p.dq_head_stride;
          mul = p.scale;
          acc = acc1;
        } else if (which == 0) {
          dst = p.dv + ((p.cu_q != nullptr) ? static_cast<int64_t>(k_off + xr) * p.dv_row_stride
                                            : b * p.dv_batch_stride + static_cast<int64_t>(xr) * p.dv_row_stride) +
                hx * p.dv_head_stride;
          mul = kDrop ? p.keep_scale : 1.f;
          acc = acc1;
        } else {
          dst = p.dk + ((p.cu_q != nullptr) ? static_cast<int64_t>(k_off + xr) * p.dk_row_stride
                                            : b * p.dk_batch_stride + static_cast<int64_t>(xr) * p.dk_row_stride) +
                hx * p.dk_head_stride;
          mul = p.scale;
          acc = acc2;
        }
#pragma unroll
        // this warpgroup converts head_dim columns [half * kD/2, (half + 1) * kD/2)
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
            // output tile `which` is staged in ring slot `which`: two 64-column halves of 128-byte rows
            // in the 128-byte-swizzled layout the tensor map expects
            uint8_t* row = smem + kSmemY + which * kTileBytes + (col >> 6) * kHalfBytes + r * 128;
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
        if (lane == 0) mbar_arrive(bar + kBarEpiFull);
        if (threadIdx.x == 0) {
          if (mbar_wait(bar + kBarEpiFull, 0, abort_flag)) {
            const int row0 = ((kMode == kModeDKDV) ? k_off : q_off) + x0;
#pragma unroll
            for (int which = 0; which < n_out; ++which) {
              const CUtensorMap* tm = (which == 0) ? &tm_o1 : &tm_o2;
#pragma unroll
              for (int ht = 0; ht < kD / 64; ++ht)
                tma_store_4d(tm, base + kSmemY + which * kTileBytes + ht * kHalfBytes, ht * 64, row0, hx, bcoord);
            }
            tma_store_commit();
            tma_store_wait_read();  // the shared memory must outlive the stores' reads of it
          }
        }
      }
    }
  }

  if (warp < 8) BWD_STAMP(warp >> 2, 23, 1);
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
  if (warp == 0) BWD_STAMP(0, 23, 2);
  if (threadIdx.x == 0 && *abort_flag != 0) atomicExch(p.status, SDPA_B200_DEVICE_TIMEOUT);
  // the dQ grid overlaps the tail of the dK/dV grid: it must not be the first of the two to complete
  if (kMode == kModeDQ && threadIdx.x == 0) wait_for_previous_grid();
}

// delta[row] = sum_d dO[row,d] * O[row,d]; lse2[row] = lse[row] * log2(e);
// rows padded to lq_pad per (batch, head): padding rows get lse2 = +inf, delta = 0.
struct PreParams {
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

// 16 bytes (8 elements) per thread and head_dim / 8 threads per row; a 256-thread block covers 64 rows of
// the padded sequence in up to four passes whose loads are all issued before the first use.
constexpr int kPreRows = 64;
template <bool kF16>
__global__ void __launch_bounds__(256) bwd_preprocess_kernel(const PreParams p) {
  // heads vary fastest across the grid: with the usual [batch, row, head, dim] memory order the blocks
  // that run together then read neighbouring 256-byte pieces of the same rows
  const int h = blockIdx.x, b = blockIdx.z;
  const int tpr = p.head_dim <= 64 ? 8 : 16;  // threads per row (head dims in between leave lanes without data)
  const int rows_per_pass = 256 / tpr;      // 16 or 32
  const int passes = kPreRows / rows_per_pass;  // 4 or 2
  const int sub = threadIdx.x % tpr;
  const int r_in_pass = threadIdx.x / tpr;
  int q_off = 0, len_q = p.seqlen_q;
  if (p.cu_q != nullptr) {
    q_off = p.cu_q[b];
    len_q = p.cu_q[b + 1] - q_off;
  }
  uint4 ov[4], dv[4];
#pragma unroll
  for (int ps = 0; ps < 4; ++ps) {
    ov[ps] = make_uint4(0u, 0u, 0u, 0u);
    dv[ps] = make_uint4(0u, 0u, 0u, 0u);
    const int row = blockIdx.y * kPreRows + ps * rows_per_pass + r_in_pass;
    if (ps < passes && row < len_q) {
      const uint16_t* o;
      const uint16_t* dout;
      if (p.cu_q != nullptr) {
        o = p.out + static_cast<int64_t>(q_off + row) * p.o_row_stride + h * p.o_head_stride;
        dout = p.dout + static_cast<int64_t>(q_off + row) * p.do_row_stride + h * p.do_head_stride;
      } else {
        o = p.out + b * p.o_batch_stride + h * p.o_head_stride + static_cast<int64_t>(row) * p.o_row_stride;
        dout = p.dout + b * p.do_batch_stride + h * p.do_head_stride + static_cast<int64_t>(row) * p.do_row_stride;
      }
      if (sub * 8 < p.head_dim) {
        ov[ps] = *reinterpret_cast<const uint4*>(o + sub * 8);
        dv[ps] = *reinterpret_cast<const uint4*>(dout + sub * 8);
      }
    }
  }
#pragma unroll
  for (int ps = 0; ps < 4; ++ps) {
    if (ps >= passes) break;
    const int row = blockIdx.y * kPreRows + ps * rows_per_pass + r_in_pass;
    const float2 o0 = unpack_16x2<kF16>(ov[ps].x), o1 = unpack_16x2<kF16>(ov[ps].y);
    const float2 o2 = unpack_16x2<kF16>(ov[ps].z), o3 = unpack_16x2<kF16>(ov[ps].w);
    const float2 d0 = unpack_16x2<kF16>(dv[ps].x), d1 = unpack_16x2<kF16>(dv[ps].y);
    const float2 d2 = unpack_16x2<kF16>(dv[ps].z), d3 = unpack_16x2<kF16>(dv[ps].w);
    float acc = (o0.x * d0.x + o0.y * d0.y) + (o1.x * d1.x + o1.y * d1.y) + (o2.x * d2.x + o2.y * d2.y) +
                (o3.x * d3.x + o3.y * d3.y);
    // the tpr threads of a row are consecutive lanes of one warp
    for (int off = tpr >> 1; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
    if (sub == 0 && row < p.lq_pad) {
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
}


using TileKernel = void (*)(const CUtensorMap, const CUtensorMap, const CUtensorMap, const CUtensorMap,
                            const CUtensorMap, const CUtensorMap, const BwdKernelParams);

template <int kMode, bool kDrop, bool kBias>
TileKernel pick_tile_kernel(int head_dim, bool f16) {
  if (head_dim <= 64)
    return f16 ? bwd_tile_kernel<kMode, 64, true, kDrop, kBias> : bwd_tile_kernel<kMode, 64, false, kDrop, kBias>;
  return f16 ? bwd_tile_kernel<kMode, 128, true, kDrop, kBias> : bwd_tile_kernel<kMode, 128, false, kDrop, kBias>;
}

template <int kMode>
TileKernel pick_tile_kernel(bool drop, bool bias, int head_dim, bool f16) {
  if (drop) return bias ? pick_tile_kernel<kMode, true, true>(head_dim, f16) : pick_tile_kernel<kMode, true, false>(head_dim, f16);
  return bias ? pick_tile_kernel<kMode, false, true>(head_dim, f16) : pick_tile_kernel<kMode, false, false>(head_dim, f16);
}

// `overlap_previous`: launch with programmatic stream serialization, so that this grid's CTAs may start as soon as
// every CTA of the kernel before it in the stream has begun (see the launch_dependents signal at the top of the
// dK/dV kernel) and an SM has room. Used for the dQ kernel, which needs nothing the dK/dV kernel writes: its CTAs
// fill the SMs the last, partly empty wave of dK/dV CTAs leaves idle.
int launch_tile_kernel(int mode, int head_dim, bool f16, int grid, cudaStream_t stream, const CUtensorMap& tm_q,
                       const CUtensorMap& tm_k, const CUtensorMap& tm_v, const CUtensorMap& tm_do,
                       const CUtensorMap& tm_o1, const CUtensorMap& tm_o2, const BwdKernelParams& kp,
                       bool overlap_previous = false) {
  const bool drop = kp.keep_rows != nullptr;
  const bool bias = kp.bias != nullptr;
  TileKernel kernel = mode == kModeDKDV ? pick_tile_kernel<kModeDKDV>(drop, bias, head_dim, f16)
                                        : pick_tile_kernel<kModeDQ>(drop, bias, head_dim, f16);
  const uint32_t smem = smem_bytes_for(mode);
  cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (err != cudaSuccess) {
    set_error("backward: cudaFuncSetAttribute(%u bytes smem): %s", smem, cudaGetErrorString(err));
    return SDPA_B200_LAUNCH_FAILED;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = overlap_previous ? 1 : 0;
  err = cudaLaunchKernelEx(&cfg, kernel, tm_q, tm_k, tm_v, tm_do, tm_o1, tm_o2, kp);
  if (err == cudaSuccess) err = cudaGetLastError();
  if (err != cudaSuccess) {
    set_error("backward %s: launch failed: %s", mode == kModeDKDV ? "dK/dV" : "dQ", cudaGetErrorString(err));
    return SDPA_B200_LAUNCH_FAILED;
  }
  count_launch();
  return SDPA_B200_OK;
}

int lq_padded(const sdpa_b200_params& p) { return ((p.max_seqlen_q + kTile - 1) / kTile) * kTile; }

}  // namespace

// The fused kernel serves every call that does not ask for a fixed summation order and has no bias (the bias gradient
// is written by the dQ kernel, whose threads own query rows).
bool use_fused_backward(const sdpa_b200_params& p) { return p.deterministic == 0 && p.bias == nullptr; }

size_t bwd_vector_bytes(const sdpa_b200_params& p) {
  const size_t bytes = 2 * static_cast<size_t>(p.batch) * p.heads_q * lq_padded(p) * sizeof(float);
  return (bytes + 255) / 256 * 256;
}

size_t bwd_workspace_bytes(const sdpa_b200_params& p) {
  // lse2 and delta, then (fused kernel) the fp32 dQ accumulator
  return bwd_vector_bytes(p) + (use_fused_backward(p) ? bwd_fused_workspace_bytes(p, lq_padded(p)) : 0);
}

int launch_bwd(const sdpa_b200_params& p, void* workspace, size_t workspace_bytes, cudaStream_t stream) {
  (void)workspace_bytes;
  const bool f16 = p.dtype == SDPA_B200_F16;
  const bool varlen = p.cu_seqlens_q != nullptr;
  const int lq_pad = lq_padded(p);
  const size_t vec_elems = static_cast<size_t>(p.batch) * p.heads_q * lq_pad;
  float* lse2 = reinterpret_cast<float*>(static_cast<char*>(workspace) + kWorkspaceHeaderBytes);
  float* delta = lse2 + vec_elems;

  PreParams pre;
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
  if (f16)
    bwd_preprocess_kernel<true><<<dim3(p.heads_q, lq_pad / kPreRows, p.batch), 256, 0, stream>>>(pre);
  else
    bwd_preprocess_kernel<false><<<dim3(p.heads_q, lq_pad / kPreRows, p.batch), 256, 0, stream>>>(pre);
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) {
    set_error("backward preprocess: launch failed: %s", cudaGetErrorString(err));
    return SDPA_B200_LAUNCH_FAILED;
  }
  count_launch();

  CUtensorMap tm_q, tm_k, tm_v, tm_do;
  const int64_t rows_q = varlen ? p.total_q : p.max_seqlen_q;
  const int64_t rows_k = varlen ? p.total_k : p.max_seqlen_k;
  const int64_t nb = varlen ? 1 : p.batch;
  int st;
  if ((st = make_tensor_map_16(f16, &tm_q, p.q, p.head_dim, rows_q, p.heads_q, nb, p.q_row_stride, p.q_head_stride,
                                 p.q_batch_stride, kTile)) != SDPA_B200_OK)
    return st;
  if ((st = make_tensor_map_16(f16, &tm_k, p.k, p.head_dim, rows_k, p.heads_kv, nb, p.k_row_stride, p.k_head_stride,
                                 p.k_batch_stride, kTile)) != SDPA_B200_OK)
    return st;
  if ((st = make_tensor_map_16(f16, &tm_v, p.v, p.head_dim, rows_k, p.heads_kv, nb, p.v_row_stride, p.v_head_stride,
                                 p.v_batch_stride, kTile)) != SDPA_B200_OK)
    return st;
  if ((st = make_tensor_map_16(f16, &tm_do, p.dout, p.head_dim, rows_q, p.heads_q, nb, p.do_row_stride,
                                 p.do_head_stride, p.do_batch_stride, kTile)) != SDPA_B200_OK)
    return st;
  CUtensorMap tm_dq, tm_dk, tm_dv;  // outputs, stored tile by tile from the epilogue's staging buffers
  if ((st = make_tensor_map_16(f16, &tm_dq, p.dq, p.head_dim, rows_q, p.heads_q, nb, p.dq_row_stride, p.dq_head_stride,
                                 p.dq_batch_stride, kTile)) != SDPA_B200_OK)
    return st;
  if ((st = make_tensor_map_16(f16, &tm_dk, p.dk, p.head_dim, rows_k, p.heads_kv, nb, p.dk_row_stride, p.dk_head_stride,
                                 p.dk_batch_stride, kTile)) != SDPA_B200_OK)
    return st;
  if ((st = make_tensor_map_16(f16, &tm_dv, p.dv, p.head_dim, rows_k, p.heads_kv, nb, p.dv_row_stride, p.dv_head_stride,
                                 p.dv_batch_stride, kTile)) != SDPA_B200_OK)
    return st;

  BwdKernelParams kp;
  kp.lse2 = lse2;
  kp.delta = delta;
  kp.dq = static_cast<uint16_t*>(p.dq);
  kp.dk = static_cast<uint16_t*>(p.dk);
  kp.dv = static_cast<uint16_t*>(p.dv);
  kp.cu_q = p.cu_seqlens_q;
  kp.cu_k = p.cu_seqlens_k;
  kp.status = p.device_status != nullptr ? p.device_status : static_cast<uint32_t*>(workspace);
  kp.dq_batch_stride = p.dq_batch_stride;
  kp.dq_head_stride = p.dq_head_stride;
  kp.dq_row_stride = p.dq_row_stride;
  kp.dk_batch_stride = p.dk_batch_stride;
  kp.dk_head_stride = p.dk_head_stride;
  kp.dk_row_stride = p.dk_row_stride;
  kp.dv_batch_stride = p.dv_batch_stride;
  kp.dv_head_stride = p.dv_head_stride;
  kp.dv_row_stride = p.dv_row_stride;
  kp.seqlen_q = p.max_seqlen_q;
  kp.seqlen_k = p.max_seqlen_k;
  kp.heads_q = p.heads_q;
  kp.heads_kv = p.heads_kv;
  kp.kv_group = p.heads_q / p.heads_kv;
  kp.lq_pad = lq_pad;
  kp.scale = p.softmax_scale;
  kp.head_dim = p.head_dim;
  const bool drop = p.dropout_p > 0.f;
  kp.keep_rows = drop ? p.keep_rows : nullptr;
  kp.keep_cols = drop ? p.keep_cols : nullptr;
  kp.keep_lq_pad = (p.max_seqlen_q + 127) / 128 * 128;
  kp.keep_lk_pad = (p.max_seqlen_k + 127) / 128 * 128;
  kp.keep_q_rows = p.cu_seqlens_q != nullptr ? p.total_q + 128 : kp.keep_lq_pad;
  kp.keep_k_rows = p.cu_seqlens_q != nullptr ? p.total_k + 128 : kp.keep_lk_pad;
  kp.keep_scale = drop ? 1.f / (1.f - p.dropout_p) : 1.f;
  kp.bias = static_cast<const uint16_t*>(p.bias);
  kp.bias_batch_stride = p.bias_batch_stride;
  kp.bias_head_stride = p.bias_head_stride;
  kp.bias_row_stride = p.bias_row_stride;
  kp.bias_t = static_cast<const uint16_t*>(p.bias_t);
  kp.bias_t_batch_stride = p.bias_t_batch_stride;
  kp.bias_t_head_stride = p.bias_t_head_stride;
  kp.bias_t_row_stride = p.bias_t_row_stride;
  kp.dbias = static_cast<uint16_t*>(p.dbias);
  kp.dbias_batch_stride = p.dbias_batch_stride;
  kp.dbias_head_stride = p.dbias_head_stride;
  kp.dbias_row_stride = p.dbias_row_stride;
  kp.inv_scale = 1.f / p.softmax_scale;
  kp.scale_log2 = p.softmax_scale * 1.4426950408889634f;
  kp.is_causal = p.is_causal;
#ifdef SDPA_BWD_STAMPS
  {
    const char* env = getenv("SDPA_BWD_STAMPS_PTR");
    kp.stamps = env ? reinterpret_cast<float*>(strtoull(env, nullptr, 10)) : nullptr;
  }
#endif

  // heads per group: streamed bytes per head (q + dO of the group, or k + v) within ~48 MB of L2
  auto set_order = [&](int heads_x, int rows_streamed, int streams_per_head) {
    kp.heads_x = heads_x;
    kp.num_bh = p.batch * heads_x;
    const double bytes = 2.0 * rows_streamed * p.head_dim * 2 * streams_per_head;
    int hpw = static_cast<int>((48.0 * 1024 * 1024) / bytes);
    hpw = hpw < 1 ? 1 : (hpw > 32 ? 32 : hpw);
    if (hpw > kp.num_bh) hpw = kp.num_bh;
    kp.heads_per_wave = hpw;
    const int groups = (kp.num_bh + hpw - 1) / hpw;
    return groups * hpw * kp.num_row_blocks;
  };
  kp.num_row_blocks = (p.max_seqlen_k + kTile - 1) / kTile;
  const int grid_dkdv = set_order(p.heads_kv, p.max_seqlen_q, kp.kv_group);
  if (use_fused_backward(p)) {
    float* dq_acc = reinterpret_cast<float*>(static_cast<char*>(workspace) + kWorkspaceHeaderBytes + bwd_vector_bytes(p));
    return launch_bwd_fused(p, kp, dq_acc, grid_dkdv, stream, tm_q, tm_k, tm_v, tm_do, tm_dv, tm_dk);
  }
  if ((st = launch_tile_kernel(kModeDKDV, p.head_dim, f16, grid_dkdv, stream, tm_q, tm_k, tm_v, tm_do, tm_dv, tm_dk, kp)) !=
      SDPA_B200_OK)
    return st;
  kp.num_row_blocks = (p.max_seqlen_q + kTile - 1) / kTile;
  const int grid_dq = set_order(p.heads_q, p.max_seqlen_k, 1);
  return launch_tile_kernel(kModeDQ, p.head_dim, f16, grid_dq, stream, tm_q, tm_k, tm_v, tm_do, tm_dq, tm_dq, kp,
                            /*overlap_previous=*/true);
}

}  // namespace sdpa_b200
