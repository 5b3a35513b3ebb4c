// Thin inline-PTX wrappers for the Blackwell (sm_100a) features the attention
// kernels use: mbarriers with bounded waits, TMA tensor loads, bulk reduce
// stores, tensor memory (TMEM) management and tcgen05 MMA / load / store.
//
// Every wait is bounded: a wait that runs out records an error code in a
// status word and lets the kernel run to its end, so a protocol bug shows up
// as a reported error and never as a GPU that stops answering.
#pragma once

#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace fal {

// ---------------------------------------------------------------------------
// Error codes written to the device status word by kernels.
// ---------------------------------------------------------------------------
enum DeviceStatus : int {
  kDevOk = 0,
  kDevWaitTimeout = 1000,     // + barrier id
  kDevAppendOverflow = 2000,  // decode: a new token did not fit the cache (length >= capacity) and was dropped
};

// Cycles a single mbarrier wait may take before it gives up (about one
// second at the boost clock; legitimate waits last microseconds).
static constexpr long long kWaitLimitCycles = 2000000000LL;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---------------------------------------------------------------------------
// mbarrier
// ---------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

// Makes generic-proxy writes to shared memory visible to the async proxy
// (TMA, tcgen05.mma operand reads).
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

__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok;
}

// Per-CTA abort state: one int in shared memory, plus the global status word.
struct WaitCtx {
  volatile int* abort_smem;  // set to 1 by the first wait that gives up
  int* status;               // device status word (may be nullptr)
};

// Slow path of mbar_wait, kept out of line: the kernels have dozens of wait sites and their hot
// loops must stay small enough for the instruction cache.
// (A kernel that re-balances registers with setmaxnreg cannot make calls: it defines
// FAL_WAIT_SLOW_PATH_INLINE before including this header.)
#ifdef FAL_WAIT_SLOW_PATH_INLINE
#define FAL_WAIT_SLOW_ATTR __forceinline__
#else
#define FAL_WAIT_SLOW_ATTR __noinline__
#endif
static __device__ FAL_WAIT_SLOW_ATTR bool mbar_wait_slow(uint32_t bar, uint32_t parity, volatile int* abort_smem,
                                            int* status, int barrier_id) {
  const long long t0 = clock64();
  uint32_t spins = 0;
  while (!mbar_try_wait(bar, parity)) {
    if ((++spins & 255u) == 0u) {
      if (*abort_smem) return false;
      if (clock64() - t0 > kWaitLimitCycles) {
        *abort_smem = 1;
        if (status) atomicCAS(status, 0, kDevWaitTimeout + barrier_id);
        return false;
      }
    }
  }
  return true;
}

// Waits for the phase with the given parity to complete.  Returns false when
// the CTA is aborting; callers carry on (results are then garbage, and the
// status word says so) so that every thread still reaches the kernel's end.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, const WaitCtx& ctx,
                                          int barrier_id) {
  if (mbar_try_wait(bar, parity)) return true;
  return mbar_wait_slow(bar, parity, ctx.abort_smem, ctx.status, barrier_id);
}

// ---------------------------------------------------------------------------
// TMA (cp.async.bulk.tensor) loads: plain single-CTA loads only.
// ---------------------------------------------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

// 4-D tiled load: coordinates are (c0 = innermost element, c1 = row, c2 = head, c3 = batch).
__device__ __forceinline__ void tma_load_4d(uint32_t dst_smem, const CUtensorMap* map, uint32_t bar,
                                            int c0, int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(dst_smem), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2),
        "r"(c3)
      : "memory");
}

__device__ __forceinline__ void bulk_commit_group() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}

// Waits until all but the N most recent bulk groups issued by this thread have finished READING
// shared memory.
template <int N>
__device__ __forceinline__ void bulk_wait_group_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}

// Waits until the bulk groups issued by this thread have completed entirely.
__device__ __forceinline__ void bulk_wait_group0() {
  asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
}

// ---------------------------------------------------------------------------
// Tensor memory (TMEM)
// ---------------------------------------------------------------------------
// Warp-collective.  Writes the base TMEM address to *dst_smem.
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

// Makes the mbarrier track completion of all tcgen05.mma issued so far by this thread.
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   bar)
               : "memory");
}

// 32 lanes x 32 consecutive 32-bit columns; thread i of the warp gets lane (base_lane + i).
__device__ __forceinline__ void tmem_ld_32x32b_x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}

__device__ __forceinline__ void tmem_st_32x32b_x32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
        "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]),
        "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]),
        "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
        "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}

__device__ __forceinline__ void tmem_st_32x32b_x16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
        "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]),
        "r"(r[14]), "r"(r[15])
      : "memory");
}

// ---------------------------------------------------------------------------
// tcgen05.mma descriptors (fp16 operands, fp32 accumulate)
// ---------------------------------------------------------------------------
// Instruction descriptor for kind::f16: D fp32 (bits 4-5 = 1), A and B fp16
// (format 0), a_major at bit 15 and b_major at bit 16 (0 = K-major, 1 =
// MN-major), N/8 at bits 17-22, M/16 at bits 24-28.
__host__ __device__ constexpr uint32_t make_idesc_f16(int m, int n, int a_mn_major, int b_mn_major) {
  return (1u << 4) | (static_cast<uint32_t>(a_mn_major) << 15) |
         (static_cast<uint32_t>(b_mn_major) << 16) | (static_cast<uint32_t>(n >> 3) << 17) |
         (static_cast<uint32_t>(m >> 4) << 24);
}

// Shared-memory operand descriptor, 128-byte swizzle, tile base 1024-byte aligned.  addr / LBO /
// SBO in bytes.  Bits: [0,14) addr>>4, [16,30) LBO>>4, [32,46) SBO>>4, [46,48) version = 1,
// [61,64) layout = 2 (SWIZZLE_128B).  It is built from its 32-bit halves, so that an issuing thread
// can keep the low word of a tile's base descriptor in a register and step through a tile with one
// 32-bit add per MMA (the address field holds addr >> 4 and shared-memory addresses never carry out
// of it).
__device__ __forceinline__ uint32_t smem_desc_lo(uint32_t addr, uint32_t lbo) {
  return ((addr & 0x3FFFFu) >> 4) | (((lbo >> 4) & 0x3FFFu) << 16);
}
__host__ __device__ constexpr uint32_t smem_desc_hi_sw128(uint32_t sbo) {
  return ((sbo >> 4) & 0x3FFFu) | (1u << 14) | (2u << 29);
}
__device__ __forceinline__ uint64_t smem_desc_join(uint32_t lo, uint32_t hi) {
  uint64_t d;
  asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "r"(lo), "r"(hi));
  return d;
}

// D[tmem] (+)= A[smem] * B[smem]; issued by one thread.
__device__ __forceinline__ void umma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                        uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// D[tmem] (+)= A[tmem] * B[smem]; issued by one thread.
__device__ __forceinline__ void umma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc,
                                        uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
      "}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Warpgroup-wide register reallocation (all four warps of a warpgroup must execute it).
template <int N>
__device__ __forceinline__ void setmaxnreg_inc() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N));
}
template <int N>
__device__ __forceinline__ void setmaxnreg_dec() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N));
}

// ---------------------------------------------------------------------------
// Small math helpers
// ---------------------------------------------------------------------------
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// exp2 on the FMA / ALU pipes instead of the special-function unit: 2^x = 2^floor(x) * 2^frac(x),
// frac part by a degree-3 polynomial (max relative error 8.6e-5, below fp16 rounding), integer
// part added into the exponent field.  Valid for x <= 127; x below -126 (masked scores are -inf)
// is clamped and yields about 1e-38.
__device__ __forceinline__ float exp2_fma(float x) {
  x = fmaxf(x, -126.f);
  float t;
  asm("add.rm.ftz.f32 %0, %1, %2;" : "=f"(t) : "f"(x), "f"(12582912.f));  // low mantissa bits = floor(x)
  const float fr = x - (t - 12582912.f);
  const float p = fmaf(fmaf(fmaf(0.07706618f, fr, 0.22764593f), fr, 0.69511657f), fr, 1.0f);
  return __int_as_float(__float_as_int(p) + (__float_as_int(t) << 23));
}

// ---- packed fp32 pairs (one instruction works on two floats held in a 64-bit register) ----
__device__ __forceinline__ uint64_t pack_f32x2(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack_f32x2(uint64_t r, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(r));
}
__device__ __forceinline__ uint64_t ffma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t fadd2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ uint64_t fsub2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ uint64_t fadd2_round_down(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rm.ftz.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}

// 2^x for a pair, on the special-function unit.
__device__ __forceinline__ uint64_t exp2_pair_mufu(uint64_t x) {
  float a, b;
  unpack_f32x2(x, a, b);
  return pack_f32x2(fast_exp2(a), fast_exp2(b));
}

// 2^x for a pair without the special-function unit: exp2_fma's arithmetic with the packed
// instructions (same polynomial, same clamp).
__device__ __forceinline__ uint64_t exp2_pair_fma(uint64_t x) {
  float a, b;
  unpack_f32x2(x, a, b);
  x = pack_f32x2(fmaxf(a, -126.f), fmaxf(b, -126.f));
  const uint64_t magic = pack_f32x2(12582912.f, 12582912.f);
  const uint64_t t = fadd2_round_down(x, magic);  // low mantissa bits = floor(x)
  const uint64_t fr = fsub2(x, fsub2(t, magic));
  uint64_t pl = ffma2(pack_f32x2(0.07706618f, 0.07706618f), fr, pack_f32x2(0.22764593f, 0.22764593f));
  pl = ffma2(pl, fr, pack_f32x2(0.69511657f, 0.69511657f));
  pl = ffma2(pl, fr, pack_f32x2(1.0f, 1.0f));
  float p0, p1, t0, t1;
  unpack_f32x2(pl, p0, p1);
  unpack_f32x2(t, t0, t1);
  return pack_f32x2(__int_as_float(__float_as_int(p0) + (__float_as_int(t0) << 23)),
                    __int_as_float(__float_as_int(p1) + (__float_as_int(t1) << 23)));
}

// Two exponentials per instruction on packed fp16 (input and result are half2 bit patterns).
__device__ __forceinline__ uint32_t exp2_f16x2(uint32_t x) {
  uint32_t y;
  asm("ex2.approx.f16x2 %0, %1;" : "=r"(y) : "r"(x));
  return y;
}

// Packed fp16 multiply on half2 bit patterns.
__device__ __forceinline__ uint32_t hmul2_bits(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}

// Three-input maximum (one instruction on sm_100).
__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
  __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}

}  // namespace fal
