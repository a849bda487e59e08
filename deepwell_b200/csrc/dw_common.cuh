// Shared device helpers for the sm_100a MXFP8 kernels: MX arithmetic on bit patterns and
// thin inline-PTX wrappers (mbarrier, TMA, tcgen05).  No fast-math anywhere: the quantiser
// must be bit-exact.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/dw_mxfp8.h"

namespace dw {

constexpr int kBlock = 32;  // elements per scaling block

// ------------------------------------------------------------------------------------------
// host side: the current device
// ------------------------------------------------------------------------------------------
constexpr int kMaxDevices = 64;
// Programmatic dependent launch (griddepcontrol).  A kernel launched with cudaLaunchAttributeProgrammaticStreamSerialization
// may be made resident while the kernel before it on the stream is still running; pdl_wait() then blocks until that
// kernel has completed and its writes are visible, so everything before it in the kernel (parameter reads, barrier and
// tensor-memory set-up) overlaps the predecessor's tail, and nothing after it can see the predecessor half done.
// pdl_launch_dependents() lets the NEXT kernel of the stream become resident early in the same way.  Both are no-ops in
// a kernel that was launched without the attribute.  A kernel that calls pdl_launch_dependents() must call pdl_wait()
// first: the successor only waits for THIS kernel, and that covers the kernels before it only if this one waited.
#ifdef __CUDACC__
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
#endif

// Host side: launch `kernel` allowing it to become resident while its predecessor on `st` still runs (see above).
#ifdef __CUDACC__
template <typename... KArgs>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, KArgs... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, args...);
}
#endif

struct DeviceInfo { int device; int sms; int cc_major; };
// Properties of the CURRENT device (cached per device index, so one process may drive several GPUs).
// DW_OK; DW_ERR_ARCH if it is not compute capability 10.x (*out is still filled); DW_ERR_LAUNCH if no device answers.
int current_device(DeviceInfo* out);

// ------------------------------------------------------------------------------------------
// MX arithmetic
// ------------------------------------------------------------------------------------------

// E8M0 byte from the bf16 pattern of a block's amax (sign cleared, NaN elements excluded).
//   rule 0: e = floor(log2 amax) - 8
//   rule 1: e = ceil(log2(amax/448)) as the reference's kernel evaluates it when built with its own flags
//           (--use_fast_math) for sm_100a, measured on every bf16 magnitude: a quotient amax/448 below 2^-126
//           flushes to zero, which the kernel turns into scale 1.0 (amax pattern < 0x04E0 -> byte 127), and
//           amax = 1.75 * 2^k <= 224, whose quotient is exactly a power of two below 1, lands one step higher.
// byte = e + 127 clamped to [0, 254]; amax == 0 -> 127 (scale 1.0).
__device__ __forceinline__ uint32_t e8m0_from_amax(uint32_t amax, int rule) {
    const uint32_t ef = amax >> 7, m7 = amax & 0x7Fu;
    int b = static_cast<int>(ef) - 8;
    if (rule == DW_RULE_REF_CEIL) {
        if (amax < 0x04E0u) return 127u;
        if ((m7 > 0x60u || (m7 == 0x60u && ef <= 134u)) && ef < 255u) b += 1;
    }
    b = max(b, 0);
    return amax == 0u ? 127u : static_cast<uint32_t>(b);
}

// 2^(127 - byte) as fp32 (exact); byte 254 gives the subnormal 2^-127.
__device__ __forceinline__ float e8m0_inverse(uint32_t byte) {
    return __uint_as_float(byte >= 254u ? 0x00400000u : ((254u - byte) << 23));
}

// 2^(byte - 127) as fp32; byte 0 gives the subnormal 2^-127.
__device__ __forceinline__ float e8m0_value(uint32_t byte) {
    return __uint_as_float(byte == 0u ? 0x00400000u : (byte << 23));
}

// |a| max |b| on both bf16 halves at once (the sign of the result is meaningless).  A NaN operand
// is dropped in favour of the other operand, exactly as fmaxf does.
__device__ __forceinline__ uint32_t absmax_bf16x2(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("max.xorsign.abs.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}

// two fp32 -> packed E4M3 pair, RNE, saturating to +-448; `lo` lands in bits [0,8).
__device__ __forceinline__ uint32_t cvt_e4m3x2(float lo, float hi) {
    uint16_t d;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(d) : "f"(hi), "f"(lo));
    return d;
}

// 2^(127 - byte) as a bf16 pattern replicated in both halves (byte 254 -> the subnormal 2^-127).
__device__ __forceinline__ uint32_t e8m0_inverse_bf16x2(uint32_t byte) {
    const uint32_t h = byte >= 254u ? 0x0040u : ((254u - byte) << 7);
    return h | (h << 16);
}

// The two bf16 lanes of `w`, each times the bf16 power of two in the same lane of `inv2`, as fp32.  The
// mixed-precision FMA reads the bf16 halves directly, so no shift/mask unpacking is spent on the integer
// pipe; the product of a bf16 and a power of two is exact in fp32, and the -0.0 addend keeps the sign of a
// zero product (+0.0 would turn -0.0 into +0.0).
__device__ __forceinline__ void scale_pair(uint32_t w, uint32_t inv2, float& lo, float& hi) {
    asm("{\n\t.reg .b16 a0, a1, s0, s1;\n\t"
        "mov.b32 {a0, a1}, %2;\n\t"
        "mov.b32 {s0, s1}, %3;\n\t"
        "fma.rn.f32.bf16 %0, a0, s0, %4;\n\t"
        "fma.rn.f32.bf16 %1, a1, s1, %4;\n\t}"
        : "=f"(lo), "=f"(hi) : "r"(w), "r"(inv2), "f"(-0.0f));
}

// lo += low bf16 lane of w, hi += high bf16 lane of w, in fp32 with one rounding each (the mixed-precision FMA
// with a multiplier of 1.0 reads the bf16 lanes directly: no unpacking instructions).
__device__ __forceinline__ void add_bf16x2(uint32_t w, float& lo, float& hi) {
    asm("{\n\t.reg .b16 a0, a1, one;\n\t"
        "mov.b32 {a0, a1}, %2;\n\t"
        "mov.b16 one, 0x3F80;\n\t"
        "fma.rn.f32.bf16 %0, a0, one, %0;\n\t"
        "fma.rn.f32.bf16 %1, a1, one, %1;\n\t}"
        : "+f"(lo), "+f"(hi) : "r"(w));
}

// One bf16x2 word times a power of two (`inv2` from e8m0_inverse_bf16x2) -> two E4M3 codes in
// bits [0,16), element 0 in the low byte.
__device__ __forceinline__ uint32_t quant_word(uint32_t w, uint32_t inv2) {
    float lo, hi;
    scale_pair(w, inv2, lo, hi);
    return cvt_e4m3x2(lo, hi);
}

// amax pattern (15-bit magnitude) over n bf16x2 words, NaN elements dropped as fmaxf would.
template <int N>
__device__ __forceinline__ uint32_t amax_words(const uint32_t (&w)[N]) {
    uint32_t m = w[0];
#pragma unroll
    for (int i = 1; i < N; ++i) m = absmax_bf16x2(m, w[i]);
    return m;   // two candidate magnitudes, one per half; fold with fold_amax()
}

// Folds the two halves of an absmax word into one 15-bit magnitude; an all-NaN block counts as 0.
__device__ __forceinline__ uint32_t fold_amax(uint32_t m) {
    const uint32_t lo = m & 0x7FFFu, hi = (m >> 16) & 0x7FFFu;
    const uint32_t a = max(lo <= 0x7F80u ? lo : 0u, hi <= 0x7F80u ? hi : 0u);
    return a;
}

// Byte offset of (row r, k-block kb) in the tiled (tcgen05) scale layout; kt = ceil(KB/4).
__device__ __host__ __forceinline__ int64_t sf_tiled_offset(int64_t r, int64_t kb, int64_t kt) {
    return ((r >> 7) * kt + (kb >> 2)) * 512 + (r & 31) * 16 + ((r >> 5) & 3) * 4 + (kb & 3);
}

// ------------------------------------------------------------------------------------------
// memory helpers
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ uint4 ldg_nc_v4(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

__device__ __forceinline__ void ldg_nc_v8(const void* p, uint32_t (&w)[8]) {
    asm volatile("ld.global.nc.L1::no_allocate.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3]), "=r"(w[4]), "=r"(w[5]), "=r"(w[6]), "=r"(w[7])
                 : "l"(p));
}

__device__ __forceinline__ void stg_v4(void* p, uint4 v) {
    asm volatile("st.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

}  // namespace dw
