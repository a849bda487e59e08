// Library-level entry points of the C ABI (probes and error strings).
#include <cuda_runtime.h>

#include "../../include/dw_mxfp8.h"

extern "C" DW_API int dw_mxfp8_abi_version(void) { return 1; }

extern "C" DW_API int dw_mxfp8_device_supported(int device) {
    int major = 0;
    if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return major == 10 ? 1 : 0;
}

extern "C" DW_API const char* dw_mxfp8_error_string(int code) {
    switch (code) {
        case DW_OK: return "ok";
        case DW_ERR_BAD_ARG: return "bad argument (null pointer, shape, alignment or enum)";
        case DW_ERR_ARCH: return "device is not compute capability 10.x (sm_100a required)";
        case DW_ERR_LAUNCH: return "CUDA launch or tensor-map encode failed";
        case DW_ERR_DEVICE_STATUS: return "kernel reported a non-zero status word (bounded wait expired)";
        case DW_ERR_TOO_LARGE: return "problem exceeds a fixed capacity of this entry point";
        default: return "unknown error code";
    }
}
