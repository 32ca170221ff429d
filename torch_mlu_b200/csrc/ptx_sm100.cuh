// Inline-PTX wrappers for the Blackwell (sm_100a) primitives the attention kernels use:
// mbarrier, TMA (cp.async.bulk.tensor, never with cluster multicast), tcgen05 MMA / TMEM
// load-store / alloc, and the UMMA shared-memory and instruction descriptors.
//
// Every wait in this file is bounded: a wait that runs out returns false and the caller
// records a status word and leaves through its normal tear-down path (TMEM freed), so a
// broken pipeline turns into an error code instead of a hung device.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace sdpa_b200 {

// ---------------------------------------------------------------------------------------
// small helpers
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "elect.sync _|p, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}\n"
      : "=r"(pred));
  return pred != 0;
}

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ float lg2_approx(float x) {
  float y;
  asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// three-input max (one FMNMX3 instead of two FMNMX)
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

// packed fp32x2 arithmetic: one issue slot for two lanes of work
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) {
  float2 d;
  asm("{\n\t"
      ".reg .b64 ra, rb, rc, rd;\n\t"
      "mov.b64 ra, {%2, %3};\n\t"
      "mov.b64 rb, {%4, %5};\n\t"
      "mov.b64 rc, {%6, %7};\n\t"
      "fma.rn.f32x2 rd, ra, rb, rc;\n\t"
      "mov.b64 {%0, %1}, rd;\n\t"
      "}\n"
      : "=f"(d.x), "=f"(d.y)
      : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y), "f"(c.x), "f"(c.y));
  return d;
}

__device__ __forceinline__ float2 add2(float2 a, float2 b) {
  float2 d;
  asm("{\n\t"
      ".reg .b64 ra, rb, rd;\n\t"
      "mov.b64 ra, {%2, %3};\n\t"
      "mov.b64 rb, {%4, %5};\n\t"
      "add.rn.f32x2 rd, ra, rb;\n\t"
      "mov.b64 {%0, %1}, rd;\n\t"
      "}\n"
      : "=f"(d.x), "=f"(d.y)
      : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
  return d;
}

// 2^x for two values on the FMA pipe instead of the exponential unit (4 results/clk/SMSP, the scarce
// resource of the backward's recomputation). x is clamped to >= -125, split as n + f with n = round(x),
// |f| <= 0.5 (adding 1.5*2^23 leaves n in the low mantissa bits), 2^f is a cubic with relative error
// 7.5e-5 - below the half-ulp of a 16-bit result, which is all its callers keep - and n goes straight
// into the exponent field. Results below 2^-125 come out as ~2^-125 instead of 0.
__device__ __forceinline__ float2 exp2_poly3_x2(float2 x) {
  const float2 magic = make_float2(12582912.f, 12582912.f);
  x.x = fmaxf(x.x, -125.f);
  x.y = fmaxf(x.y, -125.f);
  const float2 t = add2(x, magic);
  const float2 r = add2(t, make_float2(-12582912.f, -12582912.f));
  const float2 f = fma2(r, make_float2(-1.f, -1.f), x);
  float2 p = fma2(f, make_float2(0.055171654f, 0.055171654f), make_float2(0.24261113f, 0.24261113f));
  p = fma2(p, f, make_float2(0.69326097f, 0.69326097f));
  p = fma2(p, f, make_float2(0.99992806f, 0.99992806f));
  return make_float2(__uint_as_float(__float_as_uint(p.x) + (__float_as_uint(t.x) << 23)),
                     __uint_as_float(__float_as_uint(p.y) + (__float_as_uint(t.y) << 23)));
}

// Ask L2 for the line holding `p` (no register, no wait): for global loads a later step will need
__device__ __forceinline__ void prefetch_l2(const void* p) {
  asm volatile("prefetch.global.L2 [%0];" ::"l"(p));
}

// Warpgroup-wide register re-allocation (all four warps of the warpgroup execute it).
template <int kRegs>
__device__ __forceinline__ void reg_increase() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegs));
}
template <int kRegs>
__device__ __forceinline__ void reg_decrease() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegs));
}

// two fp32 -> packed bf16x2 (lo in the low half), round to nearest even
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
__device__ __forceinline__ uint32_t pack_f16x2(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
// The kernels are templated on the 16-bit storage type: kF16 = true is IEEE half, false is bf16.
template <bool kF16>
__device__ __forceinline__ uint32_t pack_16x2(float lo, float hi) {
  return kF16 ? pack_f16x2(lo, hi) : pack_bf16x2(lo, hi);
}
// packed pair -> two fp32 (x = low half)
template <bool kF16>
__device__ __forceinline__ float2 unpack_16x2(uint32_t w) {
  if (kF16) {
    float2 r;
    asm("{\n\t.reg .b16 lo, hi;\n\tmov.b32 {lo, hi}, %2;\n\tcvt.f32.f16 %0, lo;\n\tcvt.f32.f16 %1, hi;\n\t}\n"
        : "=f"(r.x), "=f"(r.y)
        : "r"(w));
    return r;
  }
  return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
}
template <bool kF16>
__device__ __forceinline__ uint16_t to_16(float x) {
  return static_cast<uint16_t>(pack_16x2<kF16>(x, 0.f) & 0xffffu);
}

// ---------------------------------------------------------------------------------------
// mbarrier
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

// make generic-proxy smem writes visible to the async proxy (TMA / tcgen05 readers)
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}

__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}\n"
      : "=r"(done)
      : "r"(bar), "r"(parity)
      : "memory");
  return done != 0;
}

// Bounded wait. `abort_flag` is a CTA-shared word any role sets when it gives up, so the
// rest of the CTA stops waiting too. Returns false on abort or after `budget_ns`.
constexpr uint64_t kWaitBudgetNs = 2000000000ull;  // 2 s; a healthy kernel waits microseconds

__device__ __forceinline__ bool mbar_wait_budget(uint32_t bar, uint32_t parity, volatile uint32_t* abort_flag,
                                                 uint64_t budget_ns) {
  if (mbar_test(bar, parity)) return true;
  uint64_t t0 = 0;
  for (uint32_t spin = 1;; ++spin) {
    if (mbar_test(bar, parity)) return true;
    if ((spin & 0xff) == 0) {
      if (*abort_flag != 0) return false;
      uint64_t now = global_timer_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > budget_ns) {
        *abort_flag = 1;
        return false;
      }
    }
  }
}

__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity,
                                          volatile uint32_t* abort_flag) {
  return mbar_wait_budget(bar, parity, abort_flag, kWaitBudgetNs);
}

// After a time-out the CTA must not return while copies it started or MMAs it issued are still in
// flight (they would land in shared memory / TMEM that already belongs to another CTA). One thread
// calls this before the tear-down barrier; the rest of the CTA waits for it there. 200 us covers any
// copy or MMA that is still going to finish at all.
__device__ __forceinline__ void drain_after_abort(volatile uint32_t* abort_flag) {
  if (*abort_flag == 0) return;
  const uint64_t t0 = global_timer_ns();
  while (global_timer_ns() - t0 < 200000ull) {
  }
}

// ---------------------------------------------------------------------------------------
// TMA (tiled bulk tensor copies; CTA-local destination, no multicast)
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}

// The innermost coordinate c0 times the element size must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_4d(uint32_t dst_smem, const CUtensorMap* m, uint32_t bar,
                                            int c0, int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(dst_smem), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(c0), "r"(c1), "r"(c2),
      "r"(c3)
      : "memory");
}

__device__ __forceinline__ void tma_store_4d(const CUtensorMap* m, uint32_t src_smem, int c0,
                                             int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
      ::"l"(reinterpret_cast<uint64_t>(m)), "r"(src_smem), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}

__device__ __forceinline__ void tma_store_commit() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}

__device__ __forceinline__ void tma_store_wait_all() {
  asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
}

// the stores of this thread's committed groups have finished READING shared memory
__device__ __forceinline__ void tma_store_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}

// barrier `id` (1..15; 0 is __syncthreads) over `count` threads (a multiple of 32)
__device__ __forceinline__ void named_barrier_sync(uint32_t id, uint32_t count) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}

// ---------------------------------------------------------------------------------------
// tcgen05: TMEM allocation
// ---------------------------------------------------------------------------------------
// One full warp executes alloc/dealloc. `ncols` is a power of two in [32, 512].
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem),
               "r"(ncols)
               : "memory");
}

__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}

__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tmem_wait_ld() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_wait_st() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// ---------------------------------------------------------------------------------------
// tcgen05: TMEM <-> registers. Shape 32x32b: thread i of the warp owns TMEM lane
// (32 * (warp_id % 4) + i); xN moves N consecutive 32-bit columns of that lane.
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_ld_x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
        "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
        "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}

// 32 columns into r[kOff .. kOff+31] of a larger register array (lets a caller issue several
// loads back to back and wait once)
template <int kOff, int kN>
__device__ __forceinline__ void tmem_ld_x32_at(uint32_t taddr, uint32_t (&r)[kN]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[kOff + 0]), "=r"(r[kOff + 1]), "=r"(r[kOff + 2]), "=r"(r[kOff + 3]), "=r"(r[kOff + 4]),
        "=r"(r[kOff + 5]), "=r"(r[kOff + 6]), "=r"(r[kOff + 7]), "=r"(r[kOff + 8]), "=r"(r[kOff + 9]),
        "=r"(r[kOff + 10]), "=r"(r[kOff + 11]), "=r"(r[kOff + 12]), "=r"(r[kOff + 13]), "=r"(r[kOff + 14]),
        "=r"(r[kOff + 15]), "=r"(r[kOff + 16]), "=r"(r[kOff + 17]), "=r"(r[kOff + 18]), "=r"(r[kOff + 19]),
        "=r"(r[kOff + 20]), "=r"(r[kOff + 21]), "=r"(r[kOff + 22]), "=r"(r[kOff + 23]), "=r"(r[kOff + 24]),
        "=r"(r[kOff + 25]), "=r"(r[kOff + 26]), "=r"(r[kOff + 27]), "=r"(r[kOff + 28]), "=r"(r[kOff + 29]),
        "=r"(r[kOff + 30]), "=r"(r[kOff + 31])
      : "r"(taddr)
      : "memory");
}

__device__ __forceinline__ void tmem_st_x32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
      "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]),
      "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]),
      "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]),
      "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}

// 64 columns into r[0..63] with two loads (the caller waits once)
__device__ __forceinline__ void tmem_ld_x64(uint32_t taddr, uint32_t (&r)[64]) {
  tmem_ld_x32_at<0>(taddr, r);
  tmem_ld_x32_at<32>(taddr + 32, r);
}

// fp32 reduce-add of four consecutive floats in global memory (16-byte aligned), no return value
__device__ __forceinline__ void red_add_f32x4(float* addr, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

__device__ __forceinline__ void tmem_st_x16(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
      "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]),
      "r"(r[15])
      : "memory");
}

// ---------------------------------------------------------------------------------------
// tcgen05: MMA (kind::f16, bf16 inputs, fp32 accumulate in TMEM), issued by ONE thread
// ---------------------------------------------------------------------------------------
// Shared-memory matrix descriptor, 128-byte swizzle, for a tile stored as rows of 128 bytes
// (64 bf16) whose 16-byte chunks are XOR-swizzled by (row % 8) - exactly what a TMA box of
// {64 elements, R rows} with CU_TENSOR_MAP_SWIZZLE_128B writes. The tile base must be
// 1024-byte aligned.
//   bits [0,14)  start address >> 4
//   bits [16,30) leading-dimension byte offset >> 4
//   bits [32,46) stride-dimension byte offset >> 4
//   bits [46,48) descriptor version (1 on sm_100)
//   bits [61,64) layout type (2 = SWIZZLE_128B)
__device__ __forceinline__ uint64_t umma_smem_desc(uint32_t smem_addr, uint32_t lbo_bytes,
                                                   uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr >> 4) & 0x3fff);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3fff) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3fff) << 32;
  d |= 1ull << 46;
  d |= 2ull << 61;
  return d;
}

// K-major operand (the contraction index is the contiguous one): 8-row groups are 1024
// bytes apart; one MMA (K = 16 bf16 = 32 bytes) stays inside the 128-byte swizzle span, so
// successive K steps advance the start address by 32 bytes. LBO is unused for this layout.
__device__ __forceinline__ uint64_t umma_desc_kmajor(uint32_t smem_addr) {
  return umma_smem_desc(smem_addr, 16, 1024);
}

// MN-major operand (the non-contraction index is contiguous, e.g. V[key][d] used as B with
// N = d): a 64-element MN chunk is one swizzle span; `mn_chunk_stride` is the byte distance
// between successive 64-element chunks (LBO) and 8 contraction rows are 1024 bytes (SBO).
__device__ __forceinline__ uint64_t umma_desc_mnmajor(uint32_t smem_addr, uint32_t mn_chunk_stride) {
  return umma_smem_desc(smem_addr, mn_chunk_stride, 1024);
}

// Instruction descriptor for kind::f16 with 16-bit A/B (f16 when `f16`, else bf16) and fp32 D.
//   bits [4,6) D format (1 = f32), [7,10) A format (0 = f16, 1 = bf16), [10,13) B format (same),
//   bit 15 A major (1 = MN), bit 16 B major (1 = MN), bits [17,23) N >> 3, bits [24,29) M >> 4.
__host__ __device__ constexpr uint32_t umma_idesc_16(int M, int N, bool a_mn_major, bool b_mn_major,
                                                     bool f16) {
  return (1u << 4) | (f16 ? 0u : ((1u << 7) | (1u << 10))) | (static_cast<uint32_t>(a_mn_major) << 15) |
         (static_cast<uint32_t>(b_mn_major) << 16) | (static_cast<uint32_t>(N >> 3) << 17) |
         (static_cast<uint32_t>(M >> 4) << 24);
}

// Cheap descriptor arithmetic for issue loops. A descriptor splits into a low word
// (start address >> 4 | LBO >> 4 << 16) and a constant high word (SBO, version, swizzle); moving
// along a tile only adds (byte offset >> 4) to the low word. Shared memory is < 256 KB, so the
// 14-bit address field never carries into the LBO field.
constexpr uint32_t kDescHiSw128 = (1024u >> 4) | (1u << 14) | (2u << 29);  // SBO 1024, version 1, SWIZZLE_128B
__device__ __forceinline__ uint32_t umma_desc_lo_kmajor(uint32_t smem_addr) { return (smem_addr >> 4) | (1u << 16); }
__device__ __forceinline__ uint32_t umma_desc_lo_mnmajor(uint32_t smem_addr, uint32_t mn_chunk_stride) {
  return (smem_addr >> 4) | ((mn_chunk_stride >> 4) << 16);
}

// D[tmem] (+)= A[smem] * B[smem], descriptors given as low words (high word = kDescHiSw128)
template <uint32_t kIdesc, bool kAccumulate>
__device__ __forceinline__ void umma_ss_lo(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      ".reg .b64 da, db;\n\t"
      "mov.b64 da, {%1, %3};\n\t"
      "mov.b64 db, {%2, %3};\n\t"
      "setp.ne.b32 p, %5, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, p;\n\t"
      "}\n"
      ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(kDescHiSw128), "r"(kIdesc), "r"(kAccumulate ? 1u : 0u)
      : "memory");
}

// the same with the accumulate flag as a run-time value
template <uint32_t kIdesc>
__device__ __forceinline__ void umma_ss_lo_acc(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      ".reg .b64 da, db;\n\t"
      "mov.b64 da, {%1, %3};\n\t"
      "mov.b64 db, {%2, %3};\n\t"
      "setp.ne.b32 p, %5, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, p;\n\t"
      "}\n"
      ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(kDescHiSw128), "r"(kIdesc), "r"(accumulate)
      : "memory");
}

// D[tmem] (+)= A[tmem] * B[smem]
// The same two issue forms with the per-MMA offsets as compile-time immediates that are added INSIDE
// the asm block. Written as `a_lo + off` in C++, the sums are loop invariants the compiler hoists out
// of the issue loop - sixteen or more live registers in a thread that only has a few dozen.
template <uint32_t kIdesc, uint32_t kOffA, uint32_t kOffB, bool kAccumulate>
__device__ __forceinline__ void umma_ss_off(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      ".reg .b32 ra, rb;\n\t"
      ".reg .b64 da, db;\n\t"
      "add.u32 ra, %1, %6;\n\t"
      "add.u32 rb, %2, %7;\n\t"
      "mov.b64 da, {ra, %3};\n\t"
      "mov.b64 db, {rb, %3};\n\t"
      "setp.ne.b32 p, %5, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, p;\n\t"
      "}\n"
      ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(kDescHiSw128), "r"(kIdesc), "r"(kAccumulate ? 1u : 0u), "n"(kOffA),
      "n"(kOffB)
      : "memory");
}

template <uint32_t kIdesc, uint32_t kOffA, uint32_t kOffB>
__device__ __forceinline__ void umma_ts_off(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      ".reg .b32 ra, rb;\n\t"
      ".reg .b64 db;\n\t"
      "add.u32 ra, %1, %6;\n\t"
      "add.u32 rb, %2, %7;\n\t"
      "mov.b64 db, {rb, %3};\n\t"
      "setp.ne.b32 p, %5, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [ra], db, %4, p;\n\t"
      "}\n"
      ::"r"(d_tmem), "r"(a_tmem), "r"(b_lo), "r"(kDescHiSw128), "r"(kIdesc), "r"(accumulate), "n"(kOffA), "n"(kOffB)
      : "memory");
}

template <uint32_t kIdesc>
__device__ __forceinline__ void umma_ts_lo(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      ".reg .b64 db;\n\t"
      "mov.b64 db, {%2, %3};\n\t"
      "setp.ne.b32 p, %5, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, p;\n\t"
      "}\n"
      ::"r"(d_tmem), "r"(a_tmem), "r"(b_lo), "r"(kDescHiSw128), "r"(kIdesc), "r"(accumulate)
      : "memory");
}

// D[tmem] (+)= A[smem] * B[smem]
__device__ __forceinline__ void umma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                        uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// D[tmem] (+)= A[tmem] * B[smem]   (A: lane = row, each 32-bit column = two bf16 along K)
__device__ __forceinline__ void umma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc,
                                        uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
      "}\n"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Arrive (count 1) on an mbarrier once every tcgen05 op this thread issued so far is done.
// Implies tcgen05.fence::before_thread_sync.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   bar)
               : "memory");
}

}  // namespace sdpa_b200
