// Shared device helpers for the sm_100a kernels: NVFP4 number formats, mbarrier,
// TMA (cp.async.bulk[.tensor]) and tcgen05 (tensor memory + block-scaled MMA)
// wrappers written as inline PTX. Every load is a plain (single-destination) copy.
#pragma once
#include <cstdint>
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

// ---------------------------------------------------------------------------
// Status codes returned by the C entry points / written to the status word.
// ---------------------------------------------------------------------------
enum TwStatus : int {
  TW_OK = 0,
  TW_ERR_ARGUMENT = 1,        // null pointer, non-positive size
  TW_ERR_SHAPE = 2,           // n or k not a multiple of 128, k too large, ...
  TW_ERR_ALIGNMENT = 3,       // pointer not 16-byte aligned
  TW_ERR_MISSING_SWIZZLED = 4,// a term was requested without its atom-layout scales
  TW_ERR_TENSOR_MAP = 5,      // cuTensorMapEncodeTiled failed
  TW_ERR_LAUNCH = 6,          // cudaLaunchKernel / attribute error
  TW_ERR_DRIVER = 7,          // driver entry point not found
  TW_ERR_TIMEOUT = 8,         // a bounded device-side wait ran out (status word)
  TW_ERR_TOO_LARGE = 9,       // size beyond a stated maximum
  TW_ERR_ARCH = 10,           // device is not compute capability 10.x
  TW_STATUS_COUNT
};

namespace tw {

// ---------------------------------------------------------------------------
// Number formats
// ---------------------------------------------------------------------------
__device__ __forceinline__ float bf16_bits_to_float(uint32_t bits16) { return __uint_as_float(bits16 << 16); }

// RNE float -> E4M3 byte, saturating to 448 (inputs here are already clamped).
__device__ __forceinline__ uint32_t f32_to_e4m3(float x) {
  uint16_t r;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(0.f), "f"(x));
  return r & 0xffu;
}
// E4M3 byte -> float (exact).
__device__ __forceinline__ float e4m3_to_f32(uint32_t b) {
  uint32_t h2;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"((uint16_t)b));
  return __half2float(__ushort_as_half((unsigned short)(h2 & 0xffffu)));
}
// Two floats -> one byte of E2M1 codes, `lo` in the low nibble. RNE, ties to the
// even code, saturating at +-6, sign of zero kept.
__device__ __forceinline__ uint32_t f32x2_to_e2m1x2(float lo, float hi) {
  uint32_t r;
  asm("{ .reg .b8 t; cvt.rn.satfinite.e2m1x2.f32 t, %2, %1; cvt.u32.u8 %0, t; }" : "=r"(r) : "f"(lo), "f"(hi));
  return r;
}
// tanh-form GELU in fp32 (tanh.approx), shared by the pointwise activation kernel and the GEMM epilogue so that
// both produce the same bits.
__device__ __forceinline__ float gelu_tanh(float x) {
  const float u = 0.7978845608028654f * __fmaf_rn(0.044715f * x, x * x, x);
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(u));
  return 0.5f * x * (1.f + t);
}
// ---------------------------------------------------------------------------
// Shared-memory addresses, mbarriers
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void fence_barrier_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
      : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
// Non-blocking poll of a phase: issued ahead of use so that its latency hides behind other instructions.
__device__ __forceinline__ bool mbar_test_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{ .reg .pred p; mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
      : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
// Bounded wait: polls until the phase with `parity` completes, the CTA-wide
// abort flag is raised, or about `limit_cycles` SM cycles (about half a second) have passed. On a
// timeout it raises the abort flag and returns false; it never traps.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                          long long limit_cycles = 1000000000LL) {
  if (mbar_try_wait(bar, parity)) return true;
  long long start = clock64();
  uint32_t polls = 0;
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((++polls & 255u) == 0u) {
      if (*abort_flag) return false;
      if (clock64() - start > limit_cycles) { *abort_flag = 1; return false; }
    }
  }
}

// Same contract for a whole, converged warp: every lane polls (the barrier state is the same for all
// lanes of one instruction), so control flow stays warp-uniform around the wait and the elected lane
// that issues the asynchronous operations afterwards does so from converged code.
__device__ __forceinline__ bool mbar_wait_all(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                              long long limit_cycles = 1000000000LL) {
  if (mbar_try_wait(bar, parity)) return true;     // the common case: one instruction, same answer in every lane
  bool ok = true;
  long long start = clock64();
  uint32_t polls = 0;
  while (!mbar_try_wait(bar, parity)) {
    if ((++polls & 255u) == 0u) {
      if (*abort_flag) { ok = false; break; }
      if (clock64() - start > limit_cycles) { *abort_flag = 1; ok = false; break; }
    }
  }
  __syncwarp();
  return __all_sync(0xffffffffu, ok);
}
// True in exactly one lane of a converged warp.
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile("{ .reg .pred p; elect.sync _|p, 0xffffffff; selp.u32 %0, 1, 0, p; }" : "=r"(pred));
  return pred != 0;
}

// Same contract, for warps that wait long (epilogue, table builder): only lane 0 polls, with a
// short sleep between polls, so that idle warps do not take issue slots from the single-thread
// producer and MMA roles; the other lanes block at the warp barrier.
__device__ __forceinline__ bool mbar_wait_warp(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                               long long limit_cycles = 1000000000LL) {
  int ok = 1;
  if ((threadIdx.x & 31) == 0) {
    if (!mbar_try_wait(bar, parity)) {
      long long start = clock64();
      uint32_t polls = 0;
      while (!mbar_try_wait(bar, parity)) {
        __nanosleep(64);
        if ((++polls & 63u) == 0u) {
          if (*abort_flag) { ok = 0; break; }
          if (clock64() - start > limit_cycles) { *abort_flag = 1; ok = 0; break; }
        }
      }
    }
  }
  ok = __shfl_sync(0xffffffffu, ok, 0);
  return ok != 0;
}

// ---------------------------------------------------------------------------
// TMA
// ---------------------------------------------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const void* tmap) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(tmap) : "memory");
}
__device__ __forceinline__ void tma_load_2d(void* dst, const void* tmap, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(smem_u32(dst)), "l"(tmap), "r"(x), "r"(y), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* dst, const void* tmap, int x, int y, int z, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
      ::"r"(smem_u32(dst)), "l"(tmap), "r"(x), "r"(y), "r"(z), "r"(smem_u32(bar)) : "memory");
}
// Untiled bulk copy global -> shared; both addresses 16-byte aligned, bytes % 16 == 0.
__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}

// Tiled bulk store shared -> global (x = innermost coordinate; x * element size must be a multiple of 16 bytes;
// parts of the box outside the tensor are not written). Joins the thread's current bulk group.
__device__ __forceinline__ void tma_store_2d(const void* tmap, const void* src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];\n"
               "cp.async.bulk.commit_group;"
               ::"l"(tmap), "r"(smem_u32(src)), "r"(x), "r"(y) : "memory");
}
// The issuing thread's bulk stores have finished reading shared memory / have completed.
__device__ __forceinline__ void bulk_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// ---------------------------------------------------------------------------
// tcgen05: tensor memory and block-scaled MMA (cta_group::1 only)
// ---------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* slot_in_smem, uint32_t columns) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
               ::"r"(smem_u32(slot_in_smem)), "r"(columns) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t addr, uint32_t columns) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(columns) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// Arrives once on `bar` when every tcgen05 operation issued so far by this thread has completed.
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
               ::"r"(smem_u32(bar)) : "memory");
}
// 32 rows x 16 bytes of shared memory -> 4 TMEM columns, replicated to the four lane quadrants.
__device__ __forceinline__ void tc_copy_scales(uint32_t tmem_addr, uint64_t smem_desc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(tmem_addr), "l"(smem_desc) : "memory");
}
// D[tmem] (+)= A[smem] * B[smem]^T, E2M1 operands with one UE4M3 scale per 16 elements of K; K = 64.
__device__ __forceinline__ void tc_mma_nvf4(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                            uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
  asm volatile(
      "{ .reg .pred p; setp.ne.b32 p, %4, 0;\n"
      "  tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%5], [%6], p; }"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
      : "memory");
}
// Shared-memory matrix descriptor, K-major operand.
//   bits 0-13 start address >> 4, 16-29 leading byte offset >> 4, 32-45 stride byte offset >> 4
//   (distance between 8-row groups), 46-47 descriptor version (1 on sm_100), 61-63 swizzle
//   (0 none, 2 = 128 B, 4 = 64 B, 6 = 32 B).
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes,
                                                   uint32_t swizzle) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr >> 4) & 0x3fffu);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3fffu) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3fffu) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)(swizzle & 7u) << 61;
  return d;
}
// Instruction descriptor of kind::mxf4nvf4 (E2M1 x E2M1, UE4M3 scales, fp32 accumulate, K-major A and B).
//   bits 7-9 A format (1 = E2M1), 10-12 B format, 15/16 majors (0 = K), 17-22 N >> 3, 23 scale format
//   (0 = UE4M3), 24-28 M >> 4. Scale-factor ids stay 0: with four scales per K = 64 every byte of the
//   32-bit TMEM scale column is used.
__host__ __device__ constexpr uint32_t make_idesc_nvf4(int m, int n) {
  return (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

// 32 lanes x 32 consecutive fp32 columns of TMEM -> 32 registers per thread (lane = row).
__device__ __forceinline__ void tmem_load_32x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      " %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr) : "memory");
}
// 32 lanes x 16 consecutive fp32 columns of TMEM -> 16 registers per thread.
__device__ __forceinline__ void tmem_load_32x32_x16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr) : "memory");
}
// Register budget of the calling warpgroup (all four warps execute it): the launch allocates the same
// count for every thread, warps with little state hand registers to the ones that hold tiles.
template <int N> __device__ __forceinline__ void reg_budget_shrink() { asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N)); }
template <int N> __device__ __forceinline__ void reg_budget_grow() { asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N)); }
// One 32-byte global store (32-byte aligned address).
__device__ __forceinline__ void store_256(void* ptr, const uint32_t (&w)[8]) {
  asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
               ::"l"(ptr), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]), "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7]) : "memory");
}
__device__ __forceinline__ void tmem_load_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// Load and wait for a caller that keeps a load in flight while it works on registers loaded earlier. Both are
// volatile (they keep their order among themselves and against barrier operations) but do not clobber memory,
// so the compiler may move ordinary loads, stores and arithmetic across them; the wait names the destination
// registers as operands, which keeps every use of them behind it.
__device__ __forceinline__ void tmem_load_16_async(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
}
__device__ __forceinline__ void tmem_load_wait(uint32_t (&r)[16]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
                 "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15]));
}

}  // namespace tw
