// Shared device helpers for the sm_100a kernels: mbarrier, TMA, tcgen05/TMEM wrappers, bounded
// waits with status words, peer-memory flag primitives and small numeric utilities.
//
// Every wait in this library is bounded.  A wait that runs out records a code in a status word
// and returns false; the kernel then drains what it started, frees its TMEM and returns, so the
// context stays usable.  The reference's peer kernels follow the same abortable pattern
// (native/shared/cuda/peer_exchange.cu:190-253) but keep a trapping legacy variant; none exists here.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace cafd {

// ---- status codes written to the per-launch status word -----------------------------------
enum Status : uint32_t {
  kOk = 0,
  kTimeoutFullBarrier = 1,    // consumer waited for TMA data
  kTimeoutEmptyBarrier = 2,   // producer waited for a free stage
  kTimeoutTmemFull = 3,       // epilogue waited for the accumulator
  kTimeoutTmemEmpty = 4,      // MMA warp waited for the epilogue
  kTimeoutPeerFlag = 5,       // wait on a flag written by another GPU
  kBadArgument = 6,
  kTimeoutSoftmax = 7,
  kTimeoutTicket = 8,
};

// Wall-clock limit for any single wait (nanoseconds of %globaltimer).  Tests shorten it.
static __device__ unsigned long long g_wait_limit_ns = 2000000000ull;

__device__ __forceinline__ unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint32_t lane_id() { return threadIdx.x & 31; }

__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n.reg .pred p;\nelect.sync _|p, 0xffffffff;\nselp.u32 %0, 1, 0, p;\n}\n" : "=r"(pred));
  return pred != 0;
}

// ---- programmatic dependent launch -------------------------------------------------------------
// Every kernel of this library is launched with programmatic stream serialization: it may start
// while its predecessor in the stream is still draining, so launch latency and the prologue
// (barrier init, TMEM allocation, descriptor prefetch) overlap the predecessor's tail.  A kernel
// must not read anything a predecessor wrote, nor write anything, before pdl_wait() returns.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---- mbarrier --------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait.  Returns false (and records `code`) when the limit passes.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, uint32_t* status, uint32_t code) {
  // Fast path first: the clock (%globaltimer is slow to read) is only consulted after many failed polls, so a wait
  // that completes within microseconds never pays for it.
#pragma unroll 1
  for (int i = 0; i < 2048; ++i)
    if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = globaltimer_ns();
  const unsigned long long limit = g_wait_limit_ns;
  for (uint32_t round = 1;; ++round) {
#pragma unroll 1
    for (int i = 0; i < 64; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    // A wait that already ran out elsewhere (this CTA or another) ends every later blocked wait soon after.
    // The status word lives in global memory; it is looked at only once in a while, so that a waiter is not
    // parked on a memory load at the moment its barrier completes.
    if ((round & 255u) == 0u && status && *reinterpret_cast<volatile uint32_t*>(status) != 0u) return false;
    if (globaltimer_ns() - t0 > limit) {
      if (status) atomicCAS(status, 0u, code);
      return false;
    }
  }
}

// ---- TMA ---------------------------------------------------------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(m) : "memory");
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* m, uint64_t* bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(m), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* m, uint64_t* bar, int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(dst)), "l"(m), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
// Bring a box into L2 without touching shared memory (no barrier, no completion to wait for).
__device__ __forceinline__ void tma_prefetch_l2_3d(const CUtensorMap* m, int c0, int c1, int c2) {
  asm volatile("cp.async.bulk.prefetch.tensor.3d.L2.global.tile [%0, {%1, %2, %3}];" ::"l"(m), "r"(c0), "r"(c1), "r"(c2) : "memory");
}
__device__ __forceinline__ void tma_load_4d(void* dst, const CUtensorMap* m, uint64_t* bar, int c0, int c1, int c2,
                                            int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(smem_u32(dst)), "l"(m), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* m, const void* src, int c0, int c1) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(m),
               "r"(smem_u32(src)), "r"(c0), "r"(c1)
               : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void tma_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void tma_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// ---- tcgen05 / TMEM ----------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// D[tmem] (+)= A[smem] * B[smem], bf16/fp16 inputs, fp32 accumulate.
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                         uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Same with e4m3/e5m2 (and 6/4-bit) inputs.
__device__ __forceinline__ void umma_f8(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n}\n" ::"r"(
          d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive on an mbarrier when every MMA issued so far by this thread has finished.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}

// 32 lanes x 32 consecutive fp32 columns -> 32 registers per thread (thread = lane).
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, "
      "%23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_32x16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, "
      "%24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]),
      "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
      "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Shared-memory operand descriptor: K-major tile, rows of 128 bytes, 128-byte swizzle,
// 8-row groups 1024 bytes apart.  `addr` is the shared-space byte address of the first row
// (1024-byte aligned tile base plus a multiple of 32 bytes to step along K inside the atom).
__device__ __forceinline__ uint64_t smem_desc_k_sw128(uint32_t addr) {
  uint64_t d = static_cast<uint64_t>((addr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>(1) << 16;             // leading byte offset: unused for swizzled K-major
  d |= static_cast<uint64_t>(1024 >> 4) << 32;     // stride byte offset between 8-row groups
  d |= static_cast<uint64_t>(1) << 46;             // descriptor version (Blackwell)
  d |= static_cast<uint64_t>(2) << 61;             // SWIZZLE_128B
  return d;
}
// MN-major tile: 64-element (128-byte) runs along M/N, 128-byte swizzle; `lbo` = bytes between
// 64-element column blocks, 8-row (K) groups 1024 bytes apart.
__device__ __forceinline__ uint64_t smem_desc_mn_sw128(uint32_t addr, uint32_t lbo_bytes) {
  uint64_t d = static_cast<uint64_t>((addr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= static_cast<uint64_t>(1024 >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}
// Instruction descriptor for kind::f16 / kind::f8f6f4 with fp32 accumulation.
// fmt: f16 kinds 0 = fp16, 1 = bf16; f8 kinds 0 = e4m3, 1 = e5m2.  major: 0 = K, 1 = MN.
__host__ __device__ constexpr uint32_t make_idesc(int m, int n, int a_fmt, int b_fmt, int a_major = 0,
                                                  int b_major = 0) {
  return (1u << 4) | (static_cast<uint32_t>(a_fmt) << 7) | (static_cast<uint32_t>(b_fmt) << 10) |
         (static_cast<uint32_t>(a_major) << 15) | (static_cast<uint32_t>(b_major) << 16) |
         (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}

// ---- peer-memory flags (system scope) ----------------------------------------------------------
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t ld_relaxed_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_add_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// Wait until *flag >= want (wrap-safe signed distance).  Bounded; false on timeout.
__device__ __forceinline__ bool wait_flag_ge(const uint32_t* flag, uint32_t want, uint32_t* status) {
  // a peer usually answers within microseconds: poll without sleeping or reading the clock first
#pragma unroll 1
  for (int i = 0; i < 512; ++i)
    if (static_cast<int32_t>(ld_acquire_sys(flag) - want) >= 0) return true;
  const unsigned long long t0 = globaltimer_ns();
  const unsigned long long limit = g_wait_limit_ns;
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 32; ++i) {
      if (static_cast<int32_t>(ld_acquire_sys(flag) - want) >= 0) return true;
      __nanosleep(40);
    }
    if (globaltimer_ns() - t0 > limit) {
      if (status) atomicCAS(status, 0u, static_cast<uint32_t>(kTimeoutPeerFlag));
      return false;
    }
  }
}

// ---- numerics ----------------------------------------------------------------------------------
__device__ __forceinline__ float bf16_lo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t v) { return __uint_as_float(v & 0xffff0000u); }
__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  __nv_bfloat162 t = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&t);
}
// 2^x on the special-function unit (about 2 ulp; -inf -> 0)
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float silu(float x) { return x / (1.0f + __expf(-x)); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

}  // namespace cafd

// ---- bounds-check build ------------------------------------------------------------------------------------------
// Compiled with -DCAFD_BOUNDS_CHECK (the second library, libcuteafd_b200_chk.so), every index that addresses a buffer
// another GPU owns (slab rows, owner ranks, combine slots, gathered rows, candidate-table rows) is checked before the
// access.  A bad index is recorded (site << 48 | index, first one wins) and the access is skipped, so the run goes on
// and the record says where.  In the normal build the check compiles to `true`.  This is the in-process stand-in for
// a memory checker on the peer-store paths.
namespace cafd {
static __device__ unsigned long long g_bad_index = 0ull;
__device__ __forceinline__ bool index_ok(long long i, long long n, unsigned site) {
  if (i >= 0 && i < n) return true;
  atomicCAS(&g_bad_index, 0ull, (static_cast<unsigned long long>(site) << 48) | (static_cast<unsigned long long>(i) & 0xffffffffffffull) | (1ull << 63));
  return false;
}
}  // namespace cafd
#ifdef CAFD_BOUNDS_CHECK
#define CAFD_INDEX_OK(i, n, site) cafd::index_ok(static_cast<long long>(i), static_cast<long long>(n), site)
#define CAFD_BOUNDS_CHECK_ON 1
#else
#define CAFD_INDEX_OK(i, n, site) true
#define CAFD_BOUNDS_CHECK_ON 0
#endif
// Per translation unit: whether it was compiled with the checks, and its record (read and cleared).
#define CAFD_BOUNDS_API(prefix)                                                                     \
  extern "C" int prefix##_bounds_check_enabled(void) { return CAFD_BOUNDS_CHECK_ON; }               \
  extern "C" int prefix##_take_bad_index(unsigned long long* out) {                                 \
    unsigned long long zero = 0ull;                                                                 \
    cudaError_t e = cudaMemcpyFromSymbol(out, cafd::g_bad_index, sizeof(*out));                     \
    if (e == cudaSuccess && *out) e = cudaMemcpyToSymbol(cafd::g_bad_index, &zero, sizeof(zero));   \
    return static_cast<int>(e);                                                                     \
  }

// Each translation unit owns a copy of the wait limit; this defines its C setter.
#define CAFD_WAIT_LIMIT_SETTER(name)                                                      \
  extern "C" int name(unsigned long long ns) {                                            \
    return static_cast<int>(cudaMemcpyToSymbol(cafd::g_wait_limit_ns, &ns, sizeof(ns))); \
  }

// Launch with programmatic stream serialization (set CAFD_PDL=0 in the environment to disable).
#include <cstdlib>
#include <utility>
namespace cafd {
inline bool pdl_enabled() {
  static int v = -1;
  if (v < 0) {
    const char* e = std::getenv("CAFD_PDL");
    v = (e && e[0] == '0') ? 0 : 1;
  }
  return v != 0;
}
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                              Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, std::forward<Args>(args)...);
}
}  // namespace cafd

// Batch-invariant kv splits.  0 (default): the decode attention kernels divide a sequence's kv range evenly over as
// many splits as fill the GPU, so the summation order of a row depends on what else is in the step.  > 0: every split
// covers this many tokens counted from position 0, whatever the step holds; a row's partials and their merge order then
// depend on its own length only.  One value for the whole library (set through cafd_set_fixed_kv_split).
inline int& fixed_kv_split_tokens() {
  static int v = 0;
  return v;
}

// Host-side error plumbing shared by the C entry points.
#define CAFD_CHECK_CUDA(expr)                       \
  do {                                              \
    cudaError_t _e = (expr);                        \
    if (_e != cudaSuccess) return static_cast<int>(_e); \
  } while (0)
