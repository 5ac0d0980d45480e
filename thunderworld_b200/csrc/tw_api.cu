// Status strings and ABI version of libtwb200.
#include "tw_common.cuh"
#include "../../include/twb200.h"

extern "C" const char* tw_status(int status) {
  switch (status) {
    case TW_OK: return "success";
    case TW_ERR_ARGUMENT: return "invalid argument (null pointer, non-positive size or inconsistent flags)";
    case TW_ERR_SHAPE: return "unsupported shape (n and k must be multiples of 128, mp = ceil(m/16)*16)";
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

extern "C" int tw_abi_version(void) { return 2; }
