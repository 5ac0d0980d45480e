// Status strings and ABI version of libtwb200.
#include "tw_common.cuh"
#include "../../include/twb200.h"

extern "C" const char* tw_status(int status) {
  switch (status) {
    case TW_OK: return "success";
    case TW_ERR_ARGUMENT: return "invalid argument (null pointer, non-positive size or inconsistent flags)";
    case TW_ERR_SHAPE: return "unsupported shape (n and k must be multiples of 128, mp a multiple of 16 not below m)";
    case TW_ERR_ALIGNMENT: return "pointer is not 16-byte aligned";
    case TW_ERR_MISSING_SWIZZLED: return "a repair term was requested without its atom-layout scales";
    case TW_ERR_TENSOR_MAP: return "cuTensorMapEncodeTiled rejected a tensor map";
    case TW_ERR_LAUNCH: return "CUDA launch failed";
    case TW_ERR_DRIVER: return "CUDA driver entry point unavailable";
    case TW_ERR_TIMEOUT: return "a bounded device-side wait ran out";
    case TW_ERR_TOO_LARGE: return "size exceeds the stated maximum of this entry point";
    case TW_ERR_ARCH: return "device is not compute capability 10.x (sm_100a build)";
    default: return "unknown status";
  }
}

extern "C" int tw_abi_version(void) { return 3; }

// ---------------------------------------------------------------------------------------------
// Self-test of the bounded-wait protocol every kernel of this library uses: one warp waits on a barrier
// nobody ever arrives at, gives up after `limit_cycles`, and the status word reports it. Nothing is in
// flight when the CTA leaves and the context stays usable: this is how a lost signal shows up in
// production (a status code), exercised without faulting or hanging the GPU.
// ---------------------------------------------------------------------------------------------
namespace {
__global__ void bounded_wait_selftest_kernel(int* status, long long limit_cycles) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) { tw::mbar_init(&bar, 1); abort_flag = 0; tw::fence_barrier_init(); }
  __syncthreads();
  bool ok = true;
  if (threadIdx.x < 32) ok = tw::mbar_wait_all(&bar, 0, &abort_flag, limit_cycles);
  else if (threadIdx.x == 32) ok = tw::mbar_wait(&bar, 0, &abort_flag, limit_cycles);
  __syncthreads();
  if (threadIdx.x == 0 && (abort_flag || !ok)) atomicExch(status, TW_ERR_TIMEOUT);
}
}  // namespace

extern "C" int tw_selftest_bounded_wait(void* workspace, long long limit_cycles, void* stream) {
  if (!workspace || limit_cycles <= 0 || limit_cycles > 2000000000LL) return TW_ERR_ARGUMENT;
  bounded_wait_selftest_kernel<<<1, 64, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<int*>(workspace), limit_cycles);
  return cudaGetLastError() == cudaSuccess ? TW_OK : TW_ERR_LAUNCH;
}
