// Row-wise MX quantisation of one slab of a bf16 matrix by a few warps, many loads in flight per thread: the body of the
// kernel for large inputs (mx_quant_row_bg_kernel: 128 threads, 8 loads of 32 bytes in flight each).
#pragma once

#include "dw_common.cuh"

namespace dw {

// Division of a 32-bit index by a run-time constant without a divide instruction
// (round-up multiplier, Granlund & Montgomery): q = (t + ((n - t) >> 1)) >> shift, t = umulhi(mul, n).
struct FastDiv {
    uint32_t mul, shift, div;
    __host__ static FastDiv make(uint32_t d) {      // d >= 2
        uint32_t l = 0;
        while ((1ull << l) < d) ++l;
        FastDiv f;
        f.mul = static_cast<uint32_t>(((1ull << 32) * ((1ull << l) - d)) / d + 1);
        f.shift = l - 1;
        f.div = d;
        return f;
    }
    __device__ __forceinline__ uint32_t quot(uint32_t n) const {
        const uint32_t t = __umulhi(mul, n);
        return (t + ((n - t) >> 1)) >> shift;
    }
};

// A row-major bf16 [rows, cols] matrix (cols % 32 == 0, x and codes 16-byte aligned) seen as total_chunks chunks of 16
// elements; chunks_per_row = cols / 16.  wide: x is 32-byte aligned (one 256-bit load per chunk).  packed_sf:
// cols % 128 == 0 and scales 4-byte aligned (four scale bytes leave as one 32-bit store).
struct RowQuantJob {
    const uint16_t* x;
    uint8_t* codes;
    uint8_t* scales;
    uint32_t total_chunks;
    FastDiv cpr;
    int rule, layout, packed_sf, wide;
};

constexpr int kRowSlabThreads = 128;

// Slab `slab` = chunks [slab * kThreads * kDeep, (slab + 1) * kThreads * kDeep): thread `tid` (0..kThreads-1, whole
// warps) takes chunks first + kThreads u, u < kDeep, all kDeep loads issued before the first is used.  Lanes
// (2 i, 2 i + 1) hold the two halves of one 32-element block.
template <int kDeep, bool kWide, int kThreads>
__device__ __forceinline__ void quant_row_slab(const RowQuantJob& j, uint64_t slab, uint32_t tid) {
    const uint32_t chunks_per_row = j.cpr.div;
    const uint32_t lane = tid & 31u;
    const int64_t kt = ((chunks_per_row >> 1) + 3) >> 2;
    const uint32_t total_chunks = j.total_chunks;
    const uint32_t first = static_cast<uint32_t>(slab * (static_cast<uint32_t>(kThreads) * kDeep)) + tid;
    uint32_t w[kDeep][8];
#pragma unroll
    for (int u = 0; u < kDeep; ++u) {
        const uint32_t idx = first + static_cast<uint32_t>(kThreads) * u;
        if (idx < total_chunks && idx >= first) {        // second test guards uint32 wrap-around
            const uint16_t* p = j.x + static_cast<int64_t>(idx) * 16;
            if (kWide) {
                ldg_nc_v8(p, w[u]);
            } else {
                const uint4 a = ldg_nc_v4(p), b = ldg_nc_v4(p + 8);
                w[u][0] = a.x; w[u][1] = a.y; w[u][2] = a.z; w[u][3] = a.w;
                w[u][4] = b.x; w[u][5] = b.y; w[u][6] = b.z; w[u][7] = b.w;
            }
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) w[u][i] = 0;
        }
    }
#pragma unroll
    for (int u = 0; u < kDeep; ++u) {
        const uint32_t idx = first + static_cast<uint32_t>(kThreads) * u;
        const bool valid = idx < total_chunks && idx >= first;
        uint32_t m2 = amax_words(w[u]);
        m2 = absmax_bf16x2(m2, __shfl_xor_sync(0xFFFFFFFFu, m2, 1));
        const uint32_t sb = e8m0_from_amax(fold_amax(m2), j.rule);
        const uint32_t inv = e8m0_inverse_bf16x2(sb);
        uint4 q;
        q.x = quant_word(w[u][0], inv) | (quant_word(w[u][1], inv) << 16);
        q.y = quant_word(w[u][2], inv) | (quant_word(w[u][3], inv) << 16);
        q.z = quant_word(w[u][4], inv) | (quant_word(w[u][5], inv) << 16);
        q.w = quant_word(w[u][6], inv) | (quant_word(w[u][7], inv) << 16);
        if (valid) stg_v4(j.codes + static_cast<int64_t>(idx) * 16, q);
        auto sf_offset = [&]() -> int64_t {
            if (j.layout != DW_SF_TILED) return idx >> 1;
            const uint32_t row = j.cpr.quot(idx);
            return sf_tiled_offset(row, (idx - row * chunks_per_row) >> 1, kt);
        };
        if (j.packed_sf) {
            // cols % 128 == 0: lanes 0,2,4,6 of each group of 8 hold k-blocks kb..kb+3 of one row
            uint32_t pk = sb;
            pk |= __shfl_down_sync(0xFFFFFFFFu, sb, 2) << 8;
            pk |= __shfl_down_sync(0xFFFFFFFFu, sb, 4) << 16;
            pk |= __shfl_down_sync(0xFFFFFFFFu, sb, 6) << 24;
            if (valid && (lane & 7u) == 0u) *reinterpret_cast<uint32_t*>(j.scales + sf_offset()) = pk;
        } else if (valid && (lane & 1u) == 0u) {
            j.scales[sf_offset()] = static_cast<uint8_t>(sb);
        }
    }
}

// Slabs first, first + stride, ... of a job
template <int kDeep, int kThreads = kRowSlabThreads>
__device__ __forceinline__ void quant_row_slabs(const RowQuantJob& j, uint64_t first, uint64_t stride, uint32_t tid) {
    constexpr uint64_t kSlab = static_cast<uint64_t>(kThreads) * kDeep;
    for (uint64_t slab = first; slab * kSlab < j.total_chunks; slab += stride) {
        if (j.wide) quant_row_slab<kDeep, true, kThreads>(j, slab, tid);
        else quant_row_slab<kDeep, false, kThreads>(j, slab, tid);
    }
}

// Host side: the job for a matrix, or false if it does not meet the conditions of this path.
inline bool make_row_quant_job(RowQuantJob* j, const void* x, void* codes, void* scales, int64_t rows, int64_t cols, int rule,
                               int layout) {
    auto al = [](const void* p, uintptr_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; };
    if (rows <= 0 || cols <= 0 || cols % 32 != 0 || !al(x, 16) || !al(codes, 16) || rows * cols / 16 >= (1ll << 32)) return false;
    j->x = static_cast<const uint16_t*>(x);
    j->codes = static_cast<uint8_t*>(codes);
    j->scales = static_cast<uint8_t*>(scales);
    j->total_chunks = static_cast<uint32_t>(rows * cols / 16);
    j->cpr = FastDiv::make(static_cast<uint32_t>(cols / 16));
    j->rule = rule;
    j->layout = layout;
    j->packed_sf = (cols % 128 == 0) && al(scales, 4);
    j->wide = al(x, 32);
    return true;
}

}  // namespace dw
