// Library-level entry points of the C ABI (probes and error strings) and the per-device property cache.
#include <cuda_runtime.h>

#include <atomic>
#include <mutex>

#include "dw_common.cuh"

namespace dw {

// dw_mxfp8_debug_fake_device: what current_device() reports instead of asking the runtime (cc_major < 0: off).
static std::atomic<int> g_fake_cc{-1}, g_fake_sms{0};

int current_device(DeviceInfo* out) {
    const int fake = g_fake_cc.load(std::memory_order_relaxed);
    if (fake >= 0) {
        const int sms = g_fake_sms.load(std::memory_order_relaxed);
        *out = DeviceInfo{0, sms > 0 ? sms : 148, fake};
        return fake == 10 ? DW_OK : DW_ERR_ARCH;
    }
    static std::mutex mu;
    static DeviceInfo cache[kMaxDevices];
    static bool have[kMaxDevices] = {};
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
        cudaGetLastError();
        return DW_ERR_LAUNCH;
    }
    std::lock_guard<std::mutex> lock(mu);
    if (!have[dev]) {
        DeviceInfo di{dev, 0, 0};
        if (cudaDeviceGetAttribute(&di.sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
            cudaDeviceGetAttribute(&di.cc_major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess || di.sms <= 0) {
            cudaGetLastError();
            return DW_ERR_LAUNCH;
        }
        cache[dev] = di;
        have[dev] = true;
    }
    *out = cache[dev];
    return out->cc_major == 10 ? DW_OK : DW_ERR_ARCH;
}

}  // namespace dw

extern "C" DW_API int dw_mxfp8_abi_version(void) { return 2; }

extern "C" DW_API int dw_mxfp8_device_supported(int device) {
    int major = 0;
    if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return major == 10 ? 1 : 0;
}

extern "C" DW_API int dw_mxfp8_copy_2d_async(void* dst, size_t dst_pitch, const void* src, size_t src_pitch, size_t width_bytes,
                                       size_t height, void* stream) {
    if (width_bytes == 0 || height == 0) return DW_OK;
    if (!dst || !src || dst_pitch < width_bytes || src_pitch < width_bytes) return DW_ERR_BAD_ARG;
    if (cudaMemcpy2DAsync(dst, dst_pitch, src, src_pitch, width_bytes, height, cudaMemcpyDeviceToDevice,
                          static_cast<cudaStream_t>(stream)) != cudaSuccess) {
        cudaGetLastError();
        return DW_ERR_LAUNCH;
    }
    return DW_OK;
}

extern "C" DW_API int dw_mxfp8_debug_fake_device(int cc_major, int sms) {
    dw::g_fake_sms.store(sms, std::memory_order_relaxed);
    dw::g_fake_cc.store(cc_major, std::memory_order_relaxed);
    return DW_OK;
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
