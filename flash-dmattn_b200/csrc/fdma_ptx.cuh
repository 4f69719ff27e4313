// Thin inline-PTX wrappers for the sm_100a features the kernels use: mbarrier, TMA tiled copies,
// tcgen05 (TMEM allocation, UMMA issue, commit, TMEM load/store) and the shared-memory / instruction
// descriptors that tcgen05.mma consumes. Everything is cta_group::1; every TMA copy targets the issuing CTA only.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace fdma {

// ---------------------------------------------------------------------------------------------
// Bounded waits report through a per-device status word in global memory (first writer wins) and a
// CTA-wide abort flag in shared memory that makes every other wait of the CTA give up as well.
// ---------------------------------------------------------------------------------------------
constexpr uint64_t kWaitLimitNs = 2000000000ull;  // 2 s: far above any legitimate wait in these kernels

struct WaitCtl {
  volatile int* abort_flag;  // shared memory, one per CTA
  int* status;               // global memory, one per device: [0] code, [2..3] address of the host-visible mirror
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ bool elect_one() {
  uint32_t pred = 0;
  asm volatile(
      "{\n\t"
      ".reg .pred P1;\n\t"
      "elect.sync _|P1, 0xffffffff;\n\t"
      "selp.b32 %0, 1, 0, P1;\n\t"
      "}\n"
      : "=r"(pred));
  return pred != 0;
}

// ---------------------------------------------------------------------------------------------
// mbarrier
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
// Bounded wait. Returns false if the CTA-wide abort flag is (or becomes) set. A wait that lasts longer
// than the limit (`kWaitLimitNs`, or the one given to mbar_wait_limit) records `code` in the status word and in its
// host-visible mirror, sets the abort flag and returns false, so the CTA can run its tear-down (TMEM free) instead
// of hanging the device.
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t addr, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t"
      ".reg .pred P1;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 P1, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, P1;\n\t"
      "}\n"
      : "=r"(done)
      : "r"(addr), "r"(parity)
      : "memory");
  return done;
}
// Most waits in these kernels find their barrier already complete: the first attempt is straight-line code, the
// polling loop with its time limit follows only when it fails.
__device__ __forceinline__ void record_wait_timeout(int* status, int code) {
  if (atomicCAS(status, 0, code) == 0) {
    // first writer: mirror the code into page-locked host memory, where the host can see it without a sync
    int* host = *reinterpret_cast<int* volatile*>(status + 2);
    if (host) {
      *reinterpret_cast<volatile int*>(host) = code;
      __threadfence_system();
    }
  }
}
__device__ __forceinline__ bool mbar_wait_slow(uint32_t addr, uint32_t parity, volatile int* abort_flag, int* status,
                                            int code, uint64_t limit_ns) {
  uint64_t t0 = 0;
  uint32_t spins = 0;
  while (true) {
    if (mbar_try_wait(addr, parity)) return true;
    ++spins;
    if ((spins & 63u) == 0u) {
      if (*abort_flag) return false;
      uint64_t now = globaltimer_ns();
      if (t0 == 0) {
        t0 = now;
      } else if (now - t0 > limit_ns) {
        record_wait_timeout(status, code);
        *abort_flag = 1;
        return false;
      }
    }
  }
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, const WaitCtl& ctl, int code) {
  const uint32_t addr = smem_u32(bar);
  if (mbar_try_wait(addr, parity)) return true;
  return mbar_wait_slow(addr, parity, ctl.abort_flag, ctl.status, code, kWaitLimitNs);
}
// Same wait with a caller-chosen limit (the self-test uses a short one).
__device__ __forceinline__ bool mbar_wait_limit(uint64_t* bar, uint32_t parity, const WaitCtl& ctl, int code,
                                                uint64_t limit_ns) {
  const uint32_t addr = smem_u32(bar);
  if (mbar_try_wait(addr, parity)) return true;
  return mbar_wait_slow(addr, parity, ctl.abort_flag, ctl.status, code, limit_ns);
}

// ---------------------------------------------------------------------------------------------
// Optional wait-time tracing (-DFDMA_PROF): each role adds the SM clock cycles it spends inside every kind of
// wait, and its total lifetime, to a small global table that fdma_prof_read() copies out. Off by default; the
// macros then cost nothing.
// ---------------------------------------------------------------------------------------------
#ifdef FDMA_PROF
static __device__ unsigned long long g_prof[64];  // one table per translation unit
#define FDMA_PROF_BEGIN() \
  unsigned long long prof_acc_[8] = {0, 0, 0, 0, 0, 0, 0, 0}; \
  const long long prof_t0_ = clock64()
#define FDMA_PROF_WAIT(slot, expr) \
  ([&]() { const long long t_ = clock64(); const bool r_ = (expr); prof_acc_[slot] += clock64() - t_; return r_; }())
#define FDMA_PROF_END(base, active) \
  do { \
    if (active) { \
      prof_acc_[7] = clock64() - prof_t0_; \
      for (int i_ = 0; i_ < 8; ++i_) atomicAdd(&g_prof[(base) + i_], prof_acc_[i_]); \
    } \
  } while (0)
#else
#define FDMA_PROF_BEGIN() do {} while (0)
#define FDMA_PROF_WAIT(slot, expr) (expr)
#define FDMA_PROF_END(base, active) do {} while (0)
#endif

// ---------------------------------------------------------------------------------------------
// Proxy / tcgen05 fences
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// ---------------------------------------------------------------------------------------------
// TMA (tiled, single-CTA). The destination is this CTA's shared memory; completion is signalled as
// transaction bytes on an mbarrier of the same CTA.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void prefetch_tmap(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
__device__ __forceinline__ void tma_load_4d(void* smem_dst, const CUtensorMap* m, uint64_t* bar, int c0, int c1,
                                            int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], "
      "[%2];"
      :
      : "r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(c0), "r"(c1),
        "r"(c2), "r"(c3)
      : "memory");
}

// Untiled bulk copy global -> shared (both addresses 16-byte aligned, size a multiple of 16 bytes).
__device__ __forceinline__ void bulk_load_1d(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               :
               : "r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(gmem_src)), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

// ---------------------------------------------------------------------------------------------
// TMEM allocation (one warp executes these, all 32 lanes converged)
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

// ---------------------------------------------------------------------------------------------
// UMMA descriptors
// ---------------------------------------------------------------------------------------------
// Shared-memory matrix descriptor, 128-byte swizzle, tile rows of 128 bytes laid down by TMA
// (8 rows x 128 B = one 1024-byte swizzle atom; the tile base is 1024-byte aligned).
//   K-major  operand ([mn][k], k contiguous):  SBO = distance between 8-row groups along M/N (1024 B)
//   MN-major operand ([k][mn], mn contiguous): SBO = distance between 8-row groups along K (1024 B),
//                                              LBO = distance between 64-element column blocks along M/N
// Fields: start address >>4 in bits [0,14), LBO>>4 in [16,30), SBO>>4 in [32,46), version 1 in [46,48),
// layout type SWIZZLE_128B = 2 in [61,64).
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}

// Instruction descriptor for kind::f16 with fp32 accumulation.
//   bits [4,6) D format (1 = f32), [7,10) A format, [10,13) B format (0 = f16, 1 = bf16),
//   bit 15 A is MN-major, bit 16 B is MN-major, [17,23) N>>3, [24,29) M>>4.
__host__ __device__ constexpr uint32_t umma_idesc(int m, int n, bool is_bf16, bool a_mn_major, bool b_mn_major) {
  return (1u << 4) | ((is_bf16 ? 1u : 0u) << 7) | ((is_bf16 ? 1u : 0u) << 10) | ((a_mn_major ? 1u : 0u) << 15) |
         ((b_mn_major ? 1u : 0u) << 16) | (static_cast<uint32_t>(n >> 3) << 17) |
         (static_cast<uint32_t>(m >> 4) << 24);
}

// The three issue wrappers below are called by ALL lanes of a converged warp with warp-uniform arguments; one
// elected lane issues. Keeping the surrounding control flow uniform lets the compiler hold descriptors in
// uniform registers instead of moving them there one by one for every instruction.
// D[tmem] (+)= A[smem] * B[smem]
__device__ __forceinline__ void umma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                        uint32_t accumulate) {
  if (elect_one())
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n"
      :
      : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]; A holds 16-bit values packed two per 32-bit column (lane = M row).
__device__ __forceinline__ void umma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                        uint32_t accumulate) {
  if (elect_one())
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
      "}\n"
      :
      : "r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// The mbarrier receives one arrival once every tcgen05.mma issued so far by the electing warp has completed
// (elect.sync picks the same lane every time for a full, converged warp).
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  if (elect_one())
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}

// ---------------------------------------------------------------------------------------------
// TMEM <-> registers. Shape 32x32b: lane i of the warp touches TMEM lane (warp%4)*32 + i, `N` consecutive
// 32-bit columns starting at the column in `taddr` (bits [31:16] = lane, [15:0] = column).
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_ld_x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_x16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st_x32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      :
      : "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]),
        "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]),
        "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st_x16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      :
      : "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_ld_x2(uint32_t taddr, uint32_t& r0, uint32_t& r1) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x2.b32 {%0, %1}, [%2];" : "=r"(r0), "=r"(r1) : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_st_x1(uint32_t taddr, uint32_t r0) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x1.b32 [%0], {%1};" ::"r"(taddr), "r"(r0) : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// ---------------------------------------------------------------------------------------------
// Small numeric helpers
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// 16-byte read-only load (data that no thread of the grid writes)
__device__ __forceinline__ uint4 ld_nc_v4(const void* ptr) { return __ldg(reinterpret_cast<const uint4*>(ptr)); }

// 32-byte read-only load (sm_100: 256-bit global accesses); `ptr` must be 32-byte aligned. One request per sector
// where two 16-byte loads would make two.
__device__ __forceinline__ void ld_nc_v8(const void* ptr, uint32_t (&r)[8]) {
  asm volatile("ld.global.nc.L1::no_allocate.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "l"(ptr));
}

// 32-byte store; `ptr` must be 32-byte aligned.
__device__ __forceinline__ void st_v8(void* ptr, const uint32_t (&r)[8]) {
  asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"
               :
               : "l"(ptr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
               : "memory");
}

__device__ __forceinline__ void prefetch_l2(const void* ptr) {
  asm volatile("prefetch.global.L2 [%0];" ::"l"(ptr));
}
// max of three (one instruction on sm_100)
// 2^x for a pair of values on the FMA pipe instead of the transcendental unit: round-to-nearest split x = j + f with
// f in [-0.5, 0.5], cubic minimax polynomial for 2^f (relative error 7.5e-5, far below one bf16 rounding), exponent
// added through the integer bits. x is clamped at -125, so a masked (-inf) score yields 2^-125, not 0; callers must
// not rely on an exact zero. Valid for x < 100.
__device__ __forceinline__ float2 exp2_poly2(float2 x) {
  x.x = fmaxf(x.x, -125.f);
  x.y = fmaxf(x.y, -125.f);
  const float2 t = __fadd2_rn(x, make_float2(12582912.f, 12582912.f));  // 1.5 * 2^23: integer part in the low bits
  const float2 j = __fadd2_rn(t, make_float2(-12582912.f, -12582912.f));
  const float2 f = __ffma2_rn(j, make_float2(-1.f, -1.f), x);
  float2 p = __ffma2_rn(f, make_float2(0.055171460f, 0.055171460f), make_float2(0.24261086f, 0.24261086f));
  p = __ffma2_rn(p, f, make_float2(0.69326097f, 0.69326097f));
  p = __ffma2_rn(p, f, make_float2(0.99992812f, 0.99992812f));
  return make_float2(__uint_as_float(__float_as_uint(p.x) + (__float_as_uint(t.x) << 23)),
                     __uint_as_float(__float_as_uint(p.y) + (__float_as_uint(t.y) << 23)));
}

__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
__device__ __forceinline__ float fast_log2(float x) {
  float y;
  asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// Packs two floats into one 32-bit register of 16-bit values: `lo` in bits [15:0], `hi` in [31:16].
template <bool kBf16>
__device__ __forceinline__ uint32_t pack_16x2(float lo, float hi) {
  uint32_t r;
  if (kBf16) {
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  } else {
    asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  }
  return r;
}

// Named barrier over `nthreads` threads (a multiple of 32); id 0 is __syncthreads' own.
__device__ __forceinline__ void named_bar_sync(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

}  // namespace fdma
