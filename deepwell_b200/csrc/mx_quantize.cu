// MX quantisation kernels for sm_100a: bf16 -> E4M3 codes + E8M0 block scales.
//
// Replaces quantize_to_mxfp8_kernel / dequantize_from_mxfp8_kernel and fills in the empty
// transpose_quantize_to_mxfp8_kernel of the reference (csrc/mxfp8_quantization.cu:29-226).
// The reference launches one 256-thread CTA per 32 elements and reads the input twice; here
// every kernel is a single pass sized to keep HBM busy:
//
//   mx_quant_row_kernel   row-wise, no shared memory: 32-byte loads (16 elements per thread),
//                         block amax by one warp shuffle, 16-byte packed E4M3 stores.
//   mx_quant_tile_kernel  column-wise (transposed payload) and the fused "both directions from
//                         one read" form: a 128x128 bf16 tile is staged in shared memory, the
//                         row-wise part is computed from the registers that loaded it, the
//                         column pass reads the tile conflict-free down the rows.
//   mx_quant_generic_kernel  any shape / alignment / direction (ragged last block), one thread
//                         per scaling block.
//
// Scales are written either flat [R, K/32] or directly in the 512-byte-tile layout the
// tcgen05 block-scaled MMA reads (DW_SF_TILED), so the GEMM needs no re-layout pass.
// All arithmetic is on bit patterns; no fast-math; results are bit-exact against the oracle.

#include <algorithm>
#include <atomic>
#include <mutex>

#include "dw_common.cuh"
#include "dw_quant_row.cuh"

namespace dw {

// ------------------------------------------------------------------------------------------
// Row-wise fast path.  cols % 32 == 0.  One thread = 16 consecutive elements (half a block).
// ------------------------------------------------------------------------------------------
template <bool kWide>  // kWide: 32-byte aligned input -> one 256-bit load per chunk
__global__ void __launch_bounds__(256)
mx_quant_row_kernel(const uint16_t* __restrict__ x, uint8_t* __restrict__ codes, uint8_t* __restrict__ scales,
                    uint32_t total_chunks, FastDiv cpr, int rule, int layout, int packed_sf, int pdl) {
    // pdl: wait for the kernel before this one on the stream, then let the next one become resident (dw_common.cuh);
    // 0: DW_QUANT_OVERLAP_PREVIOUS, this kernel runs beside its predecessor and must not release its successor early
    if (pdl) { pdl_wait(); pdl_launch_dependents(); }
    const uint32_t chunks_per_row = cpr.div;
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t T = gridDim.x * blockDim.x;
    const uint32_t kb_per_row = chunks_per_row >> 1;
    const int64_t kt = (kb_per_row + 3) >> 2;

    for (uint32_t base = blockIdx.x * blockDim.x + (threadIdx.x & ~31u); base < total_chunks; base += 2u * T) {
        uint32_t idx[2] = {base + lane, base + T + lane};
        uint32_t w[2][8];
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            if (idx[u] < total_chunks && idx[u] >= base) {   // second test guards uint32 wrap-around
                const uint16_t* p = x + static_cast<int64_t>(idx[u]) * 16;
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
                idx[u] = 0xFFFFFFFFu;
            }
        }
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            uint32_t m2 = amax_words(w[u]);
            m2 = absmax_bf16x2(m2, __shfl_xor_sync(0xFFFFFFFFu, m2, 1));
            const uint32_t sb = e8m0_from_amax(fold_amax(m2), rule);
            const uint32_t inv = e8m0_inverse_bf16x2(sb);
            uint4 q;
            q.x = quant_word(w[u][0], inv) | (quant_word(w[u][1], inv) << 16);
            q.y = quant_word(w[u][2], inv) | (quant_word(w[u][3], inv) << 16);
            q.z = quant_word(w[u][4], inv) | (quant_word(w[u][5], inv) << 16);
            q.w = quant_word(w[u][6], inv) | (quant_word(w[u][7], inv) << 16);
            const bool valid = idx[u] != 0xFFFFFFFFu;
            if (valid) stg_v4(codes + static_cast<int64_t>(idx[u]) * 16, q);

            if (packed_sf) {
                // cols % 128 == 0: lanes 0,2,4,6 of each group of 8 hold k-blocks kb..kb+3 of one row
                uint32_t pk = sb;
                pk |= __shfl_down_sync(0xFFFFFFFFu, sb, 2) << 8;
                pk |= __shfl_down_sync(0xFFFFFFFFu, sb, 4) << 16;
                pk |= __shfl_down_sync(0xFFFFFFFFu, sb, 6) << 24;
                if (valid && (lane & 7u) == 0u) {
                    int64_t off;
                    if (layout == DW_SF_TILED) {
                        const uint32_t row = cpr.quot(idx[u]);
                        const uint32_t kb = (idx[u] - row * chunks_per_row) >> 1;
                        off = sf_tiled_offset(row, kb, kt);
                    } else {
                        off = idx[u] >> 1;
                    }
                    *reinterpret_cast<uint32_t*>(scales + off) = pk;
                }
            } else if (valid && (lane & 1u) == 0u) {
                int64_t off;
                if (layout == DW_SF_TILED) {
                    const uint32_t row = cpr.quot(idx[u]);
                    const uint32_t kb = (idx[u] - row * chunks_per_row) >> 1;
                    off = sf_tiled_offset(row, kb, kt);
                } else {
                    off = idx[u] >> 1;
                }
                scales[off] = static_cast<uint8_t>(sb);
            }
        }
    }
}

// The same arithmetic with kDeep 32-byte loads in flight per thread instead of two, in short-lived CTAs of 128 threads
// (one slab of 128 x kDeep chunks each; body in dw_quant_row.cuh): the kernel for large inputs.  Measured on B200 it
// runs at the copy bandwidth (16384 x 14336: 107 us against 130 us for the kernel above, 6.6 against 5.4 TB/s).
template <int kDeep>
__global__ void __maxnreg__(88)      // 128 threads x 88 registers
mx_quant_row_bg_kernel(const RowQuantJob job, int pdl) {
    if (pdl) { pdl_wait(); pdl_launch_dependents(); }
    quant_row_slabs<kDeep>(job, blockIdx.x, gridDim.x, threadIdx.x);
}

// Several matrices in one launch (dw_mxfp8_quantize_rows_batch): block b works on slab b - first_slab[j] of the job j whose
// range of slabs holds b.  For the small operands of a sharded step (a rank's row slices of the activations, its weight
// shards), where every separate launch pays its own ramp and tail.
constexpr int kMaxRowQuantJobs = DW_QUANT_BATCH_MAX;
struct RowQuantBatch {
    RowQuantJob job[kMaxRowQuantJobs];
    uint32_t first_slab[kMaxRowQuantJobs + 1];
    int count;
    int pdl;
};
template <int kDeep>
__global__ void __maxnreg__(88)
mx_quant_row_batch_kernel(const __grid_constant__ RowQuantBatch b) {
    if (b.pdl) { pdl_wait(); pdl_launch_dependents(); }
    int j = 0;
    while (j + 1 < b.count && blockIdx.x >= b.first_slab[j + 1]) ++j;
    const RowQuantJob job = b.job[j];
    const uint64_t slab = blockIdx.x - b.first_slab[j];
    if (job.wide) quant_row_slab<kDeep, true, kRowSlabThreads>(job, slab, threadIdx.x);
    else quant_row_slab<kDeep, false, kRowSlabThreads>(job, slab, threadIdx.x);
}

// Writes 127 into the padding bytes of a tiled scale buffer that mx_quant_row_kernel does not
// touch (rows beyond `rows` in the last row tile, k-blocks beyond `kb` in the last k tile).
__global__ void mx_sf_pad_kernel(uint8_t* __restrict__ scales, int64_t rows, int64_t kb, int64_t rt, int64_t kt) {
    const int64_t total = rt * kt * 512;
    for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int64_t tile = i >> 9, in = i & 511;
        const int64_t r = (tile / kt) * 128 + ((in >> 2) & 3) * 32 + (in >> 4);
        const int64_t c = (tile % kt) * 4 + (in & 3);
        if (r >= rows || c >= kb) scales[i] = 127;
    }
}

// ------------------------------------------------------------------------------------------
// Tile kernel: column-wise transposed payload, optionally fused with the row-wise form.
// rows % 32 == 0, cols % 32 == 0.  CTA = 256 threads, tile = 128 rows x 128 cols.
// ------------------------------------------------------------------------------------------
// Position of 16-byte chunk c (0..15) of tile row r in shared memory.  The XOR with the row makes the
// column pass and the row pass conflict-free: 8 lanes that read the same chunk of 8 consecutive rows,
// or the four blocks of two consecutive rows, land in 8 different 16-byte bank groups.
__device__ __forceinline__ uint32_t tile_chunk(uint32_t c, uint32_t r) { return c ^ (r & 7u) ^ ((c >> 3) << 1); }

// tile buffers of 32 KB (two, or three in the two-group form: see kSplit) + two 512-byte scale staging areas + column sums
constexpr int tile_smem_bytes(bool split) { return (split ? 3 : 2) * 128 * 16 * 16 + 1024 + 2048; }

// kColSum: also leave the fp32 sum of every column over this tile's 128 rows in colsum_partial[tile row][column]
// (the bias gradient of a linear layer is the column sum of the output gradient that is being quantised here).
// kStaged: the transposed payload of a tile (128 output rows x 128 bytes) is first collected in the tile buffer the
// column pass has just read, then written out by whole 128-byte row segments, four output rows per store instruction.
// The direct form writes each thread's 32 codes straight from registers: a warp's store then touches 32 different
// output rows, `rows` bytes apart.  Once that stride reaches the page size (rows >= 2^20 or so) every store instruction
// needs 32 address translations and the kernel falls to half its rate; staged, it needs four.
// kSplit (fused both-forms only): 512 threads, threads 0-255 run the row pass of a tile while threads 256-511 run its
// column pass, instead of 256 threads running one pass after the other: the two passes only read the tile, so they
// overlap, and a tile is done in the time of the longer one.
template <bool kDoRow, bool kDoCol, bool kColSum = false, bool kStaged = false, bool kSplit = false, bool kThree = false>
__global__ void __launch_bounds__(kSplit ? 512 : 256, kSplit ? 2 : 1)
mx_quant_tile_kernel(const uint16_t* __restrict__ x, uint8_t* __restrict__ codes_row, uint8_t* __restrict__ scales_row,
                     uint8_t* __restrict__ codes_col_t, uint8_t* __restrict__ scales_col, int64_t rows, int64_t cols,
                     uint32_t tiles_c, uint32_t num_tiles, int rule, int layout, float* __restrict__ colsum_partial = nullptr) {
    static_assert(!kSplit || (kDoRow && kDoCol), "the split form is for the fused both-forms kernel");
    pdl_wait();                      // the kernel before this one on the stream has completed (its output is this one's input)
    pdl_launch_dependents();         // the next one may become resident as SMs free up; it waits for this one in turn
    // Persistent CTA, two tile buffers: the 16-byte cp.async copies of the next tile are in flight
    // while this tile is quantised, so the SM always has loads outstanding.
    extern __shared__ __align__(16) uint8_t tile_smem[];
    typedef uint4 (*TilePtr)[16];
    // kSplit runs 2 CTAs of 512 threads per SM, which leaves room for a third tile buffer each: two tiles are then in
    // flight while one is quantised (128 KB of loads outstanding per SM instead of 64 KB)
    constexpr int kBufs = (kSplit || kThree) ? 3 : 2;
    uint8_t* sf_row = tile_smem + kBufs * 128 * 16 * 16;
    uint8_t* sf_col = sf_row + 512;
    float* cs_stage = reinterpret_cast<float*>(sf_col + 512);       // [4 row blocks][128 columns]

    constexpr uint32_t kThreads = kSplit ? 512u : 256u;
    constexpr int kCopies = kSplit ? 2 : 4;                          // 16-byte copies per thread and half tile
    constexpr uint32_t kCopyRows = kThreads / 16u;                   // rows covered by one copy of every thread
    const uint32_t tid = threadIdx.x;
    const uint32_t t = tid & 255u;                                   // index inside the pass's group of 256 threads
    const bool row_role = kDoRow && (!kSplit || tid < 256u);
    const bool col_role = kDoCol && (!kSplit || tid >= 256u);
    const uint32_t cc = tid & 15u;
    const int64_t kb_row = cols >> 5, kb_col = rows >> 5;           // k-blocks per operand row
    const int64_t kt_row = (kb_row + 3) >> 2, kt_col = (kb_col + 3) >> 2;
    const bool wide_rows = (reinterpret_cast<uintptr_t>(codes_row) & 31) == 0;   // 32-byte stores of the row payload
    const bool wide_cols = (reinterpret_cast<uintptr_t>(codes_col_t) & 31) == 0; // and of the transposed payload (rows % 32 == 0)

    // Copies rows [64 half, 64 half + 64) of tile `id` into buffer `buf` (16-byte cp.async, kCopies per thread); the
    // second half also closes the copy group.  The two halves of the next tile are issued before the row pass and
    // before the column pass of the current one, which keeps the request stream to HBM even.
    auto issue_half = [&](uint32_t id, int buf, int half) {
        const uint32_t itr = id / tiles_c, itc = id - itr * tiles_c;
        const int64_t ir0 = static_cast<int64_t>(itr) * 128, igc = static_cast<int64_t>(itc) * 128 + cc * 8;
        TilePtr dst = reinterpret_cast<TilePtr>(tile_smem + buf * (128 * 16 * 16));
        if (ir0 + 128 <= rows && static_cast<int64_t>(itc) * 128 + 128 <= cols) {
            // whole tile inside the matrix (the common case): no per-row guards; the rows of a thread are a multiple of
            // 16 rows apart, so they share the swizzled chunk position (row & 7 is the same) and differ by constant
            // strides in both address spaces
            const uint32_t row0 = (tid >> 4) + 64 * half;
            const uint16_t* src = x + (ir0 + row0) * cols + igc;
            const uint32_t d0 = smem_u32(&dst[row0][tile_chunk(cc, row0)]);
            const int64_t step = static_cast<int64_t>(kCopyRows) * cols;
#pragma unroll
            for (int j = 0; j < kCopies; ++j)
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d0 + j * (kCopyRows * 256u)), "l"(src + j * step) : "memory");
        } else {
#pragma unroll
            for (int j = 0; j < kCopies; ++j) {
                const uint32_t row = (tid >> 4) + 64 * half + kCopyRows * j;
                const int64_t gr = ir0 + row;
                const bool ok = gr < rows && igc < cols;
                const uint16_t* src = ok ? x + gr * cols + igc : x;      // out of range: zero fill, nothing read
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;"
                             ::"r"(smem_u32(&dst[row][tile_chunk(cc, row)])), "l"(src), "r"(ok ? 16 : 0) : "memory");
            }
        }
        if (half == 1) asm volatile("cp.async.commit_group;" ::: "memory");
    };

    int buf = 0;
    if (blockIdx.x < num_tiles) { issue_half(blockIdx.x, 0, 0); issue_half(blockIdx.x, 0, 1); }
    if (kBufs == 3) {                                        // the second tile of the ring (or an empty group: one group per tile)
        if (blockIdx.x + gridDim.x < num_tiles) { issue_half(blockIdx.x + gridDim.x, 1, 0); issue_half(blockIdx.x + gridDim.x, 1, 1); }
        else asm volatile("cp.async.commit_group;" ::: "memory");
    }
    for (uint32_t id = blockIdx.x; id < num_tiles; id += gridDim.x, buf = (buf + 1 == kBufs) ? 0 : buf + 1) {
    const uint32_t next = id + (kBufs - 1) * gridDim.x;      // the tile fetched during this iteration
    const int nbuf = (buf + kBufs - 1) % kBufs;              // into the buffer the previous iteration has finished with
    if (kBufs == 3) asm volatile("cp.async.wait_group 1;" ::: "memory");     // this tile; the following one may still be in flight
    else asm volatile("cp.async.wait_group 0;" ::: "memory");                // this tile (the only group in flight)
    __syncthreads();
    if (next < num_tiles) issue_half(next, nbuf, 0);
    TilePtr tile = reinterpret_cast<TilePtr>(tile_smem + buf * (128 * 16 * 16));
    const uint32_t tr = id / tiles_c, tc = id - tr * tiles_c;
    const int64_t r0 = static_cast<int64_t>(tr) * 128, c0 = static_cast<int64_t>(tc) * 128;

    if (row_role) {
        // one thread = one whole 32-element block (row r, block b): four 16-byte chunks, no shuffles;
        // four consecutive lanes cover the 128 bytes of codes of one row, so stores stay coalesced.
        const uint32_t b = t & 3u;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const uint32_t r = (t >> 2) + 64 * i;
            uint32_t w[16];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint4 v = tile[r][tile_chunk(4 * b + j, r)];
                w[4 * j] = v.x; w[4 * j + 1] = v.y; w[4 * j + 2] = v.z; w[4 * j + 3] = v.w;
            }
            const uint32_t sb = e8m0_from_amax(fold_amax(amax_words(w)), rule);
            const uint32_t inv = e8m0_inverse_bf16x2(sb);
            uint32_t q[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) q[j] = __byte_perm(quant_word(w[2 * j], inv), quant_word(w[2 * j + 1], inv), 0x5410);
            const int64_t gr = r0 + r, gcb = c0 + 32 * b;
            if (gr < rows && gcb < cols) {
                uint8_t* d = codes_row + gr * cols + gcb;
                if (wide_rows) {
                    asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(d), "r"(q[0]), "r"(q[1]), "r"(q[2]),
                                 "r"(q[3]), "r"(q[4]), "r"(q[5]), "r"(q[6]), "r"(q[7]) : "memory");
                } else {
                    stg_v4(d, make_uint4(q[0], q[1], q[2], q[3]));
                    stg_v4(d + 16, make_uint4(q[4], q[5], q[6], q[7]));
                }
            }
            sf_row[(r & 31u) * 16 + (r >> 5) * 4 + b] = static_cast<uint8_t>(sb);
        }
    }
    // Measured (one group of threads running both passes): on long runs of tiles the passes run slightly faster when
    // the warps enter the column pass together; on short runs (a few tiles per CTA) the extra barrier costs ~10 %.
    if (!kSplit && kDoRow && kDoCol && num_tiles > 8u * gridDim.x) __syncthreads();

    if (next < num_tiles) issue_half(next, nbuf, 1);
    else if (kBufs == 3) asm volatile("cp.async.commit_group;" ::: "memory");
    uint32_t qa[8], qb[8];                                // the column pass's codes: 32 rows of two columns
    const uint32_t p = t & 63u, rb = t >> 6;              // column pass: thread = (column pair p, row block rb)
    if (col_role) {
        // 32 words down the rows, two columns at once
        const uint32_t* tw = reinterpret_cast<const uint32_t*>(&tile[0][0]);
        uint32_t w[32];
#pragma unroll
        for (int i = 0; i < 32; ++i)      // chunk index XORed with the row, as written by issue_half
            w[i] = tw[(rb * 32 + i) * 64 + ((tile_chunk(p >> 2, i) << 2) | (p & 3u))];
        if (kColSum) {      // rows beyond the matrix were zero-filled, so they add nothing
            float sum_a = 0.0f, sum_b = 0.0f;
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                sum_a += __uint_as_float(w[i] << 16);
                sum_b += __uint_as_float(w[i] & 0xFFFF0000u);
            }
            cs_stage[rb * 128 + 2 * p] = sum_a;
            cs_stage[rb * 128 + 2 * p + 1] = sum_b;
        }
        uint32_t m = w[0];
#pragma unroll
        for (int i = 1; i < 32; ++i) m = absmax_bf16x2(m, w[i]);
        uint32_t amax_a = m & 0x7FFFu, amax_b = (m >> 16) & 0x7FFFu;   // one column per half
        if (amax_a > 0x7F80u) amax_a = 0;                               // column of NaNs only
        if (amax_b > 0x7F80u) amax_b = 0;
        const uint32_t sb_a = e8m0_from_amax(amax_a, rule), sb_b = e8m0_from_amax(amax_b, rule);
        const uint32_t inv2 = (e8m0_inverse_bf16x2(sb_a) & 0xFFFFu) | (e8m0_inverse_bf16x2(sb_b) & 0xFFFF0000u);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            uint32_t ca[2], cb[2];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                float a0, b0, a1, b1;   // rows 4i+2h and 4i+2h+1: column a in the low lane, column b in the high lane
                scale_pair(w[4 * i + 2 * h], inv2, a0, b0);
                scale_pair(w[4 * i + 2 * h + 1], inv2, a1, b1);
                ca[h] = cvt_e4m3x2(a0, a1);
                cb[h] = cvt_e4m3x2(b0, b1);
            }
            qa[i] = __byte_perm(ca[0], ca[1], 0x5410);
            qb[i] = __byte_perm(cb[0], cb[1], 0x5410);
        }
        const uint32_t ca = 2 * p, cb = 2 * p + 1;
        sf_col[(ca & 31u) * 16 + (ca >> 5) * 4 + rb] = static_cast<uint8_t>(sb_a);
        sf_col[(cb & 31u) * 16 + (cb >> 5) * 4 + rb] = static_cast<uint8_t>(sb_b);
    }
    if (kDoCol) {
        const int64_t gcol = c0 + 2 * p, grow = r0 + rb * 32;
        if (kStaged) {
            // stage[c][128 bytes]: the 16-byte piece j of output row c sits at piece j ^ ((c >> 1) & 7), which spreads a
            // warp's stores (32 different rows, same pieces) over all banks
            __syncthreads();                                   // every thread has read its part of the tile
            uint8_t* stage = tile_smem + buf * (128 * 16 * 16);
            if (col_role) {
                const uint32_t sw = p & 7u;
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const uint32_t piece = (2 * rb + h) ^ sw;
                    *reinterpret_cast<uint4*>(stage + (2 * p) * 128 + piece * 16) = make_uint4(qa[4 * h], qa[4 * h + 1], qa[4 * h + 2], qa[4 * h + 3]);
                    *reinterpret_cast<uint4*>(stage + (2 * p + 1) * 128 + piece * 16) = make_uint4(qb[4 * h], qb[4 * h + 1], qb[4 * h + 2], qb[4 * h + 3]);
                }
            }
            __syncthreads();
            if (col_role) {
                const uint32_t warp = t >> 5, lane = t & 31u;
                const int64_t row_bytes = (rows - r0) < 128 ? (rows - r0) : 128;      // valid bytes of every output row of this tile
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const uint32_t c = i * 32 + warp * 4 + (lane >> 3), j = lane & 7u;
                    const uint4 v = *reinterpret_cast<const uint4*>(stage + c * 128 + ((j ^ ((c >> 1) & 7u)) * 16));
                    if (c0 + c < cols && static_cast<int64_t>(j) * 16 < row_bytes)
                        stg_v4(codes_col_t + (c0 + c) * rows + r0 + j * 16, v);
                }
            }
        } else if (col_role && grow < rows) {
            // 32 codes of one column = one whole 32-byte sector: a single 256-bit store when the payload allows
            auto store32 = [&](uint8_t* d, const uint32_t (&q)[8]) {
                if (wide_cols) {
                    asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(d), "r"(q[0]), "r"(q[1]), "r"(q[2]),
                                 "r"(q[3]), "r"(q[4]), "r"(q[5]), "r"(q[6]), "r"(q[7]) : "memory");
                } else {
                    stg_v4(d, make_uint4(q[0], q[1], q[2], q[3]));
                    stg_v4(d + 16, make_uint4(q[4], q[5], q[6], q[7]));
                }
            };
            if (gcol < cols) store32(codes_col_t + gcol * rows + grow, qa);
            if (gcol + 1 < cols) store32(codes_col_t + (gcol + 1) * rows + grow, qb);
        }
    }
    // One barrier per tile after both passes: the tile buffer is free for the copy issued at the top of the
    // next iteration, and the staged scale bytes (and column sums) are complete.  The next tile's passes
    // write the staging areas only after the barrier at the top of the loop, which the threads that copy the
    // staged bytes out (below) reach only when they are done.
    __syncthreads();
    if (kDoRow) {  // scales of the row-wise operand [rows, cols/32]: the first warp (tiled) or four warps (flat) of the row group
        if (layout == DW_SF_TILED) {
            if (tid < 32) {
                uint4* dst = reinterpret_cast<uint4*>(scales_row + (static_cast<int64_t>(tr) * kt_row + tc) * 512);
                dst[tid] = reinterpret_cast<const uint4*>(sf_row)[tid];
            }
        } else if (tid < 128) {
            const int64_t gr = r0 + tid, kb0 = static_cast<int64_t>(tc) * 4;
            if (gr < rows) {
#pragma unroll
                for (int b = 0; b < 4; ++b)
                    if (kb0 + b < kb_row) scales_row[gr * kb_row + kb0 + b] = sf_row[(tid & 31u) * 16 + (tid >> 5) * 4 + b];
            }
        }
    }
    if (kDoCol) {  // scales of the column-wise operand [cols, rows/32]: the last warp (tiled) or last four warps (flat) of the CTA
        const uint32_t u = kThreads - 1u - tid;
        if (kColSum && u >= 128u && u < 256u) {
            const uint32_t c = u - 128u;
            if (c0 + c < cols)
                colsum_partial[static_cast<int64_t>(tr) * cols + c0 + c] =
                    (cs_stage[c] + cs_stage[128 + c]) + (cs_stage[256 + c] + cs_stage[384 + c]);
        }
        if (layout == DW_SF_TILED) {
            if (u < 32) {
                uint4* dst = reinterpret_cast<uint4*>(scales_col + (static_cast<int64_t>(tc) * kt_col + tr) * 512);
                dst[u] = reinterpret_cast<const uint4*>(sf_col)[u];
            }
        } else if (u < 128) {
            const int64_t gcl = c0 + u, kb0 = static_cast<int64_t>(tr) * 4;
            if (gcl < cols) {
#pragma unroll
                for (int b = 0; b < 4; ++b)
                    if (kb0 + b < kb_col) scales_col[gcl * kb_col + kb0 + b] = sf_col[(u & 31u) * 16 + (u >> 5) * 4 + b];
            }
        }
    }
    }
}

// ------------------------------------------------------------------------------------------
// Generic kernel: one thread per scaling block, element strides, ragged last block.
//   element (r, c) of the operand at x[r*xsr + c*xsc]; blocks of 32 along c; code written at
//   codes[r*csr + c*csc]; scale for (r, b) flat or tiled.
// ------------------------------------------------------------------------------------------
__global__ void mx_quant_generic_kernel(const uint16_t* __restrict__ x, uint8_t* __restrict__ codes,
                                        uint8_t* __restrict__ scales, int64_t op_rows, int64_t op_cols, int64_t xsr,
                                        int64_t xsc, int64_t csr, int64_t csc, int rule, int layout, int block_major) {
    const int64_t nb = (op_cols + 31) >> 5, kt = (nb + 3) >> 2;
    const int64_t total = op_rows * nb;
    for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        // block_major: consecutive threads take consecutive operand rows (coalesced when xsr == 1)
        const int64_t r = block_major ? i % op_rows : i / nb;
        const int64_t b = block_major ? i / op_rows : i % nb;
        const int64_t c0 = b << 5, c1 = min(c0 + 32, op_cols);
        uint32_t amax = 0;
        for (int64_t c = c0; c < c1; ++c) {
            const uint32_t a = x[r * xsr + c * xsc] & 0x7FFFu;
            if (a <= 0x7F80u) amax = max(amax, a);
        }
        const uint32_t sb = e8m0_from_amax(amax, rule);
        const float inv = e8m0_inverse(sb);          // fp32 product: exact, same codes as the bf16x2 path
        for (int64_t c = c0; c < c1; ++c) {
            const float f = __uint_as_float(static_cast<uint32_t>(x[r * xsr + c * xsc]) << 16) * inv;
            codes[r * csr + c * csc] = static_cast<uint8_t>(cvt_e4m3x2(f, 0.0f) & 0xFFu);
        }
        scales[layout == DW_SF_TILED ? sf_tiled_offset(r, b, kt) : r * nb + b] = static_cast<uint8_t>(sb);
    }
}

// ------------------------------------------------------------------------------------------
// Dequantise: codes [rows, cols] (row-wise blocks) -> bf16.  One thread = 16 codes.
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t dequant_pair(uint32_t two_codes, float s) {
    uint32_t h2;
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"(static_cast<uint16_t>(two_codes)));
    float lo, hi;
    asm("{.reg .f16 a, b; mov.b32 {a, b}, %2; cvt.f32.f16 %0, a; cvt.f32.f16 %1, b;}" : "=f"(lo), "=f"(hi) : "r"(h2));
    lo *= s; hi *= s;
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}

__global__ void __launch_bounds__(256)
mx_dequant_kernel(const uint8_t* __restrict__ codes, const uint8_t* __restrict__ scales, uint16_t* __restrict__ out,
                  int64_t rows, int64_t cols, int layout) {
    const int64_t nb = (cols + 31) >> 5, kt = (nb + 3) >> 2;
    const bool vec = (cols & 15) == 0;
    const int64_t cpr = (cols + 15) >> 4, total = rows * cpr;
    for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int64_t r = i / cpr, c = (i - r * cpr) << 4;
        const int64_t b = c >> 5;
        const float s = e8m0_value(scales[layout == DW_SF_TILED ? sf_tiled_offset(r, b, kt) : r * nb + b]);
        if (vec) {
            const uint4 q = *reinterpret_cast<const uint4*>(codes + r * cols + c);
            const uint32_t qs[4] = {q.x, q.y, q.z, q.w};
            uint32_t o[8];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                o[2 * k] = dequant_pair(qs[k] & 0xFFFFu, s);
                o[2 * k + 1] = dequant_pair(qs[k] >> 16, s);
            }
            uint4* d = reinterpret_cast<uint4*>(out + r * cols + c);
            d[0] = make_uint4(o[0], o[1], o[2], o[3]);
            d[1] = make_uint4(o[4], o[5], o[6], o[7]);
        } else {
            for (int64_t e = c; e < min(c + 16, cols); ++e)
                out[r * cols + e] = static_cast<uint16_t>(dequant_pair(codes[r * cols + e], s) & 0xFFFFu);
        }
    }
}

// ------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------
static inline bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }

static int launch_status() { return cudaGetLastError() == cudaSuccess ? DW_OK : DW_ERR_LAUNCH; }

static int quantize_generic(const uint16_t* x, uint8_t* codes, uint8_t* scales, int64_t rows, int64_t cols, int direction,
                            int rule, int layout, const DeviceInfo& di, cudaStream_t st) {
    // operand rows/cols = (rows, cols) for ROW, (cols, rows) for the column directions
    int64_t orow, ocol, xsr, xsc, csr, csc;
    int block_major;
    if (direction == DW_DIR_ROW) {
        orow = rows; ocol = cols; xsr = cols; xsc = 1; csr = cols; csc = 1; block_major = 0;
    } else {
        orow = cols; ocol = rows; xsr = 1; xsc = cols; block_major = 1;
        if (direction == DW_DIR_COL_T) { csr = rows; csc = 1; } else { csr = 1; csc = cols; }
    }
    const int64_t nb = (ocol + 31) / 32, total = orow * nb;
    const int grid = static_cast<int>(std::min<int64_t>((total + 255) / 256, static_cast<int64_t>(di.sms) * 16));
    if (layout == DW_SF_TILED) {
        const int64_t rt = (orow + 127) / 128, kt = (nb + 3) / 4;
        mx_sf_pad_kernel<<<static_cast<int>(std::min<int64_t>((rt * kt * 512 + 255) / 256, 4096)), 256, 0, st>>>(
            scales, orow, nb, rt, kt);
    }
    mx_quant_generic_kernel<<<grid, 256, 0, st>>>(x, codes, scales, orow, ocol, xsr, xsc, csr, csc, rule, layout,
                                                  block_major);
    return launch_status();
}

static int quantize_row_fast(const uint16_t* x, uint8_t* codes, uint8_t* scales, int64_t rows, int64_t cols, int rule,
                             int layout, int flags, const DeviceInfo& di, cudaStream_t st) {
    const int64_t total_chunks = rows * cols / 16;
    const FastDiv cpr = FastDiv::make(static_cast<uint32_t>(cols / 16));
    const int packed = (cols % 128 == 0) && aligned(scales, 4);
    const int64_t want = (total_chunks + 511) / 512;
    // Large inputs: mx_quant_row_bg_kernel (eight loads in flight per thread, short-lived CTAs).  Small ones: the
    // persistent grid with two loads per thread, which spreads few elements over more threads.
    const bool background = total_chunks >= (1ll << 17);
    const int grid = static_cast<int>(std::min<int64_t>(want, static_cast<int64_t>(di.sms) * 8));
    if (layout == DW_SF_TILED && (rows % 128 != 0 || (cols / 32) % 4 != 0)) {
        const int64_t nb = cols / 32, rt = (rows + 127) / 128, kt = (nb + 3) / 4;
        mx_sf_pad_kernel<<<static_cast<int>(std::min<int64_t>((rt * kt * 512 + 255) / 256, 4096)), 256, 0, st>>>(
            scales, rows, nb, rt, kt);
    }
    if (background) {
        constexpr int kDeep = 8;
        RowQuantJob job;
        if (!make_row_quant_job(&job, x, codes, scales, rows, cols, rule, layout)) return DW_ERR_BAD_ARG;
        const int64_t slabs = (total_chunks + 128 * kDeep - 1) / (128 * kDeep);
        // DW_QUANT_OVERLAP_PREVIOUS: the kernel does not wait for its predecessor (it may start once that kernel has
        // released its dependents, which the GEMM does as soon as its CTAs are resident; it reads nothing that kernel
        // writes).  Otherwise it becomes resident early, waits for the predecessor to complete and only then touches memory.
        const int pdl = (flags & DW_QUANT_OVERLAP_PREVIOUS) ? 0 : 1;
        if (launch_pdl(mx_quant_row_bg_kernel<kDeep>, dim3(static_cast<unsigned>(std::min<int64_t>(slabs, 1ll << 30))),
                       dim3(kRowSlabThreads), 0, st, job, pdl) != cudaSuccess) {
            cudaGetLastError();
            return DW_ERR_LAUNCH;
        }
        return DW_OK;
    }
    const int pdl = (flags & DW_QUANT_OVERLAP_PREVIOUS) ? 0 : 1;
    const cudaError_t rc =
        aligned(x, 32) ? launch_pdl(mx_quant_row_kernel<true>, dim3(grid), dim3(256), 0, st, x, codes, scales,
                                    static_cast<uint32_t>(total_chunks), cpr, rule, layout, packed, pdl)
                       : launch_pdl(mx_quant_row_kernel<false>, dim3(grid), dim3(256), 0, st, x, codes, scales,
                                    static_cast<uint32_t>(total_chunks), cpr, rule, layout, packed, pdl);
    if (rc != cudaSuccess) {
        cudaGetLastError();
        return DW_ERR_LAUNCH;
    }
    return DW_OK;
}

static std::atomic<int> g_quant_tuning{0};     // dw_mxfp8_quantize_set_tuning

template <bool kDoRow, bool kDoCol, bool kColSum = false, bool kStaged = false, bool kSplit = false, bool kThree = false>
static int launch_tile_kernel_impl(const uint16_t* x, uint8_t* cr, uint8_t* sr, uint8_t* ct, uint8_t* sc, int64_t rows, int64_t cols,
                                   uint32_t tiles_c, uint32_t tiles, int rule, int layout, const DeviceInfo& di, cudaStream_t st,
                                   float* colsum_partial = nullptr) {
    {   // the opt-in to more than 48 KB of dynamic shared memory is a per-device attribute of the kernel
        static std::mutex mu;
        static bool done[kMaxDevices] = {};
        std::lock_guard<std::mutex> lock(mu);
        if (!done[di.device]) {
            if (cudaFuncSetAttribute(mx_quant_tile_kernel<kDoRow, kDoCol, kColSum, kStaged, kSplit, kThree>,
                                     cudaFuncAttributeMaxDynamicSharedMemorySize, tile_smem_bytes(kSplit || kThree)) != cudaSuccess) {
                cudaGetLastError();
                return DW_ERR_LAUNCH;
            }
            done[di.device] = true;
        }
    }
    // 3 CTAs of 256 threads and 67 KB per SM, or 2 CTAs of 512 threads (kSplit)
    const uint32_t grid = std::min<uint32_t>(tiles, static_cast<uint32_t>(di.sms) * ((kSplit || kThree) ? 2u : 3u));
    if (launch_pdl(mx_quant_tile_kernel<kDoRow, kDoCol, kColSum, kStaged, kSplit, kThree>, dim3(grid), dim3(kSplit ? 512 : 256),
                   static_cast<size_t>(tile_smem_bytes(kSplit || kThree)), st, x, cr, sr, ct, sc, rows, cols, tiles_c, tiles, rule,
                   layout, colsum_partial) != cudaSuccess) {
        cudaGetLastError();
        return DW_ERR_LAUNCH;
    }
    return DW_OK;
}

// The transposed payload is written out staged (see mx_quant_tile_kernel) unless the tuning word asks for the direct form:
// measured over several B200s of this pool the staged form is 4-8 % faster on most of them and up to 5 % slower on some
// for rows <= 2^19, and 1.2-1.6x faster from 2^20 rows on everywhere.  The codes need 16-byte alignment of every output row
// (rows % 32 == 0 holds on this path).
template <bool kDoRow, bool kDoCol, bool kColSum = false>
static int launch_tile_kernel(const uint16_t* x, uint8_t* cr, uint8_t* sr, uint8_t* ct, uint8_t* sc, int64_t rows, int64_t cols,
                              uint32_t tiles_c, uint32_t tiles, int rule, int layout, const DeviceInfo& di, cudaStream_t st,
                              float* colsum_partial = nullptr) {
    const int word = g_quant_tuning.load(std::memory_order_relaxed);
    const int mode = word & 3;                                                     // 0 automatic (staged), 1 direct, 2 staged
    const bool staged = kDoCol && mode != 1;
    constexpr bool kFused = kDoRow && kDoCol;
    // two groups of threads side by side (and three tile buffers) once a CTA has several tiles to work through (measured:
    // 16384 x 4096 and larger gain 7-15 %, 8192 x 3072 5 %, 16384 x 1024 loses 9 %); bit 2 of the tuning word: always one group
    const bool split = kFused && ((word >> 2) & 1) == 0 && (tiles >= 1536u || ((word >> 3) & 1) != 0);   // bit 3: always two groups
    if (kFused && split) {
        if (staged)
            return launch_tile_kernel_impl<kDoRow, kDoCol, kColSum, true, kFused>(x, cr, sr, ct, sc, rows, cols, tiles_c, tiles, rule,
                                                                                  layout, di, st, colsum_partial);
        return launch_tile_kernel_impl<kDoRow, kDoCol, kColSum, false, kFused>(x, cr, sr, ct, sc, rows, cols, tiles_c, tiles, rule,
                                                                               layout, di, st, colsum_partial);
    }
    // Column-wise alone: 2 CTAs per SM with three tile buffers (two tiles in flight each) instead of 3 CTAs with two, up to
    // 2^28 elements (measured: 16384 x 4096 0.73 -> 0.91 of copy bandwidth, 8192 x 3072 0.75 -> 0.91, 16384 x 8192
    // 0.77 -> 0.83; from 2^30 elements on 1-2.5 % slower); bit 4 of the tuning word: always two buffers
    if (!kDoRow && kDoCol && !kColSum && staged && tiles <= 16384u && ((word >> 4) & 1) == 0)
        return launch_tile_kernel_impl<kDoRow, kDoCol, false, true, false, true>(x, cr, sr, ct, sc, rows, cols, tiles_c, tiles, rule,
                                                                                 layout, di, st, colsum_partial);
    if (staged)
        return launch_tile_kernel_impl<kDoRow, kDoCol, kColSum, true>(x, cr, sr, ct, sc, rows, cols, tiles_c, tiles, rule, layout, di,
                                                                      st, colsum_partial);
    return launch_tile_kernel_impl<kDoRow, kDoCol, kColSum, false>(x, cr, sr, ct, sc, rows, cols, tiles_c, tiles, rule, layout, di, st,
                                                                   colsum_partial);
}

// ------------------------------------------------------------------------------------------
// amax history (MicroscaleManager::update_amax_history of the reference, an empty body there)
// ------------------------------------------------------------------------------------------
// history[i] = history[i - 1] for i = len-1 .. 1, history[0] = 0: one thread, the history is a few dozen floats
__global__ void mx_amax_shift_kernel(float* __restrict__ history, int len) {
    for (int i = len - 1; i > 0; --i) history[i] = history[i - 1];
    history[0] = 0.0f;
}

// history[0] = max(history[0], max |x|) over n bf16 elements, NaN elements ignored.  Non-negative floats order like
// their bit patterns, so the final combine is an integer atomicMax.
__global__ void __launch_bounds__(256)
mx_amax_kernel(const uint16_t* __restrict__ x, int64_t n, float* __restrict__ history) {
    const int64_t tid = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x, step = static_cast<int64_t>(gridDim.x) * blockDim.x;
    uint32_t m = 0;                                            // two running magnitudes, one per bf16 lane
    const bool vec = (reinterpret_cast<uintptr_t>(x) & 31) == 0;
    const int64_t chunks = vec ? n / 16 : 0;
    for (int64_t c = tid; c < chunks; c += step) {
        uint32_t w[8];
        ldg_nc_v8(x + c * 16, w);
#pragma unroll
        for (int i = 0; i < 8; ++i) m = absmax_bf16x2(m, w[i]);
    }
    uint32_t a = fold_amax(m);
    for (int64_t i = chunks * 16 + tid; i < n; i += step) {     // tail (and everything when x is not 32-byte aligned)
        const uint32_t v = x[i] & 0x7FFFu;
        if (v <= 0x7F80u) a = max(a, v);
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) a = max(a, __shfl_xor_sync(0xFFFFFFFFu, a, off));
    if ((threadIdx.x & 31u) == 0u && a != 0u) atomicMax(reinterpret_cast<unsigned int*>(history), a << 16);
}

static bool tile_path_ok(const void* x, int64_t rows, int64_t cols) {
    const int64_t tiles = ((rows + 127) / 128) * ((cols + 127) / 128);
    return rows % 32 == 0 && cols % 32 == 0 && aligned(x, 16) && tiles < (1ll << 31);
}

}  // namespace dw

using namespace dw;

extern "C" DW_API size_t dw_mxfp8_scale_bytes(int64_t rows, int64_t k, int scale_layout) {
    if (rows <= 0 || k <= 0) return 0;
    const int64_t nb = (k + 31) / 32;
    if (scale_layout == DW_SF_TILED) return static_cast<size_t>(((rows + 127) / 128) * ((nb + 3) / 4) * 512);
    return static_cast<size_t>(rows * nb);
}

extern "C" DW_API int dw_mxfp8_quantize(const void* x_bf16, void* codes, void* scales, int64_t rows, int64_t cols, int direction,
                                 int scale_rule, int scale_layout, void* stream) {
    return dw_mxfp8_quantize_ex(x_bf16, codes, scales, rows, cols, direction, scale_rule, scale_layout, 0, stream);
}

extern "C" DW_API int dw_mxfp8_quantize_ex(const void* x_bf16, void* codes, void* scales, int64_t rows, int64_t cols, int direction,
                                    int scale_rule, int scale_layout, int flags, void* stream) {
    if (rows < 0 || cols < 0 || (flags & ~DW_QUANT_OVERLAP_PREVIOUS) != 0) return DW_ERR_BAD_ARG;
    if (direction < DW_DIR_ROW || direction > DW_DIR_COL) return DW_ERR_BAD_ARG;
    if (scale_rule != DW_RULE_OCP_FLOOR && scale_rule != DW_RULE_REF_CEIL) return DW_ERR_BAD_ARG;
    if (scale_layout != DW_SF_FLAT && scale_layout != DW_SF_TILED) return DW_ERR_BAD_ARG;
    if (rows == 0 || cols == 0) return DW_OK;  // empty input: nothing to write
    if (!x_bf16 || !codes || !scales) return DW_ERR_BAD_ARG;
    if (!aligned(x_bf16, 2)) return DW_ERR_BAD_ARG;
    if (rows * cols >= (1ll << 35)) return DW_ERR_TOO_LARGE;
    DeviceInfo di;
    const int drc = current_device(&di);
    if (drc != DW_OK) return drc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const uint16_t* x = static_cast<const uint16_t*>(x_bf16);
    uint8_t* c = static_cast<uint8_t*>(codes);
    uint8_t* s = static_cast<uint8_t*>(scales);

    if (direction == DW_DIR_ROW && cols % 32 == 0 && aligned(x, 16) && aligned(c, 16))
        return quantize_row_fast(x, c, s, rows, cols, scale_rule, scale_layout, flags, di, st);
    if (direction == DW_DIR_COL_T && tile_path_ok(x, rows, cols) && aligned(c, 16) &&
        (scale_layout == DW_SF_FLAT || aligned(s, 16))) {
        const uint32_t tiles_c = static_cast<uint32_t>((cols + 127) / 128);
        const uint32_t tiles = static_cast<uint32_t>((rows + 127) / 128) * tiles_c;
        return launch_tile_kernel<false, true>(x, nullptr, nullptr, c, s, rows, cols, tiles_c, tiles, scale_rule, scale_layout, di, st);
    }
    return quantize_generic(x, c, s, rows, cols, direction, scale_rule, scale_layout, di, st);
}

extern "C" DW_API int dw_mxfp8_quantize_rows_batch(int count, const void* const* x_bf16, void* const* codes, void* const* scales,
                                                   const int64_t* rows, const int64_t* cols, int scale_rule, int scale_layout,
                                                   int flags, void* stream) {
    if (count < 0 || count > DW_QUANT_BATCH_MAX || (flags & ~DW_QUANT_OVERLAP_PREVIOUS) != 0) return DW_ERR_BAD_ARG;
    if (scale_rule != DW_RULE_OCP_FLOOR && scale_rule != DW_RULE_REF_CEIL) return DW_ERR_BAD_ARG;
    if (scale_layout != DW_SF_FLAT && scale_layout != DW_SF_TILED) return DW_ERR_BAD_ARG;
    if (count == 0) return DW_OK;
    if (!x_bf16 || !codes || !scales || !rows || !cols) return DW_ERR_BAD_ARG;
    constexpr int kDeep = 8;
    RowQuantBatch b = {};
    uint64_t slabs = 0;
    for (int i = 0; i < count; ++i) {
        if (rows[i] < 0 || cols[i] < 0) return DW_ERR_BAD_ARG;
        if (rows[i] == 0 || cols[i] == 0) continue;                       // empty matrix: nothing to write
        if (!x_bf16[i] || !codes[i] || !scales[i]) return DW_ERR_BAD_ARG;
        if (rows[i] * cols[i] >= (1ll << 35)) return DW_ERR_TOO_LARGE;
        // whole scale tiles only: this entry point has no padding pass
        if (scale_layout == DW_SF_TILED && (rows[i] % 128 != 0 || cols[i] % 128 != 0)) return DW_ERR_BAD_ARG;
        RowQuantJob* job = &b.job[b.count];
        if (!make_row_quant_job(job, x_bf16[i], codes[i], scales[i], rows[i], cols[i], scale_rule, scale_layout)) return DW_ERR_BAD_ARG;
        b.first_slab[b.count] = static_cast<uint32_t>(slabs);
        slabs += (static_cast<uint64_t>(job->total_chunks) + kRowSlabThreads * kDeep - 1) / (kRowSlabThreads * kDeep);
        ++b.count;
    }
    if (b.count == 0) return DW_OK;
    if (slabs >= (1ull << 31)) return DW_ERR_TOO_LARGE;
    b.first_slab[b.count] = static_cast<uint32_t>(slabs);
    DeviceInfo di;
    const int drc = current_device(&di);
    if (drc != DW_OK) return drc;
    b.pdl = (flags & DW_QUANT_OVERLAP_PREVIOUS) ? 0 : 1;
    if (launch_pdl(mx_quant_row_batch_kernel<kDeep>, dim3(static_cast<unsigned>(slabs)), dim3(kRowSlabThreads), 0,
                   static_cast<cudaStream_t>(stream), b) != cudaSuccess) {
        cudaGetLastError();
        return DW_ERR_LAUNCH;
    }
    return DW_OK;
}

extern "C" DW_API int dw_mxfp8_quantize_both(const void* x_bf16, void* codes_row, void* scales_row, void* codes_col_t,
                                      void* scales_col, int64_t rows, int64_t cols, int scale_rule, int scale_layout,
                                      void* stream) {
    const bool do_row = codes_row != nullptr, do_col = codes_col_t != nullptr;
    if ((do_row && !scales_row) || (do_col && !scales_col)) return DW_ERR_BAD_ARG;
    if (!do_row && !do_col) return DW_ERR_BAD_ARG;
    if (!do_col)
        return dw_mxfp8_quantize(x_bf16, codes_row, scales_row, rows, cols, DW_DIR_ROW, scale_rule, scale_layout, stream);
    if (!do_row)
        return dw_mxfp8_quantize(x_bf16, codes_col_t, scales_col, rows, cols, DW_DIR_COL_T, scale_rule, scale_layout,
                                 stream);
    if (rows < 0 || cols < 0) return DW_ERR_BAD_ARG;
    if (scale_rule != DW_RULE_OCP_FLOOR && scale_rule != DW_RULE_REF_CEIL) return DW_ERR_BAD_ARG;
    if (scale_layout != DW_SF_FLAT && scale_layout != DW_SF_TILED) return DW_ERR_BAD_ARG;
    if (rows == 0 || cols == 0) return DW_OK;
    if (!x_bf16) return DW_ERR_BAD_ARG;
    if (rows * cols >= (1ll << 35)) return DW_ERR_TOO_LARGE;
    DeviceInfo di;
    const int drc = current_device(&di);
    if (drc != DW_OK) return drc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (tile_path_ok(x_bf16, rows, cols) && aligned(codes_row, 8) && aligned(codes_col_t, 16) &&
        (scale_layout == DW_SF_FLAT || (aligned(scales_row, 16) && aligned(scales_col, 16)))) {
        const uint32_t tiles_c = static_cast<uint32_t>((cols + 127) / 128);
        const uint32_t tiles = static_cast<uint32_t>((rows + 127) / 128) * tiles_c;
        return launch_tile_kernel<true, true>(static_cast<const uint16_t*>(x_bf16), static_cast<uint8_t*>(codes_row),
                                              static_cast<uint8_t*>(scales_row), static_cast<uint8_t*>(codes_col_t),
                                              static_cast<uint8_t*>(scales_col), rows, cols, tiles_c, tiles, scale_rule,
                                              scale_layout, di, st);
    }
    int rc = dw_mxfp8_quantize(x_bf16, codes_row, scales_row, rows, cols, DW_DIR_ROW, scale_rule, scale_layout, stream);
    if (rc != DW_OK) return rc;
    return dw_mxfp8_quantize(x_bf16, codes_col_t, scales_col, rows, cols, DW_DIR_COL_T, scale_rule, scale_layout, stream);
}

// out[c] = sum over the row tiles of partial[tile][c].  A block covers 32 columns with 8 threads per column:
// thread y adds tiles y, y+8, ... in order, then the eight sums are added in order, so the result is reproducible.
__global__ void __launch_bounds__(256)
mx_colsum_reduce_kernel(const float* __restrict__ partial, int64_t tiles_r, int64_t cols, void* __restrict__ out, int out_bf16) {
    __shared__ float part[8][32];
    pdl_wait();                      // the quantiser that wrote `partial` has completed
    pdl_launch_dependents();
    const uint32_t tx = threadIdx.x & 31u, ty = threadIdx.x >> 5;
    const int64_t c = blockIdx.x * 32ll + tx;
    float acc = 0.0f;
    if (c < cols)
        for (int64_t tr = ty; tr < tiles_r; tr += 8) acc += partial[tr * cols + c];
    part[ty][tx] = acc;
    __syncthreads();
    if (ty != 0 || c >= cols) return;
#pragma unroll
    for (int y = 1; y < 8; ++y) acc += part[y][tx];
    if (out_bf16) {
        uint32_t ob;
        asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(ob) : "f"(0.0f), "f"(acc));
        static_cast<uint16_t*>(out)[c] = static_cast<uint16_t>(ob & 0xFFFFu);
    } else {
        static_cast<float*>(out)[c] = acc;
    }
}

extern "C" DW_API int dw_mxfp8_quantize_set_tuning(int word) {
    if (word < 0 || (word & 3) == 3 || (word >> 5) != 0 || (word & 12) == 12) return DW_ERR_BAD_ARG;
    g_quant_tuning.store(word, std::memory_order_relaxed);
    return DW_OK;
}

extern "C" DW_API size_t dw_mxfp8_colsum_workspace(int64_t rows, int64_t cols) {
    if (rows <= 0 || cols <= 0) return 0;
    return static_cast<size_t>((rows + 127) / 128) * static_cast<size_t>(cols) * sizeof(float);
}

extern "C" DW_API int dw_mxfp8_quantize_both_colsum(const void* x_bf16, void* codes_row, void* scales_row, void* codes_col_t,
                                                    void* scales_col, int64_t rows, int64_t cols, int scale_rule,
                                                    int scale_layout, void* colsum_out, int colsum_is_bf16, void* workspace,
                                                    size_t workspace_bytes, void* stream) {
    if (rows <= 0 || cols <= 0) return DW_ERR_BAD_ARG;
    if (!x_bf16 || !codes_row || !scales_row || !codes_col_t || !scales_col || !colsum_out || !workspace) return DW_ERR_BAD_ARG;
    if (scale_rule != DW_RULE_OCP_FLOOR && scale_rule != DW_RULE_REF_CEIL) return DW_ERR_BAD_ARG;
    if (scale_layout != DW_SF_FLAT && scale_layout != DW_SF_TILED) return DW_ERR_BAD_ARG;
    if (rows * cols >= (1ll << 35)) return DW_ERR_TOO_LARGE;
    if (workspace_bytes < dw_mxfp8_colsum_workspace(rows, cols) || !aligned(workspace, 4) || !aligned(colsum_out, 4))
        return DW_ERR_BAD_ARG;
    // only the tiled kernel sums columns: the shapes and alignments it needs are those of a linear layer's gradients
    if (!(tile_path_ok(x_bf16, rows, cols) && aligned(codes_row, 8) && aligned(codes_col_t, 16) &&
          (scale_layout == DW_SF_FLAT || (aligned(scales_row, 16) && aligned(scales_col, 16)))))
        return DW_ERR_BAD_ARG;
    DeviceInfo di;
    const int drc = current_device(&di);
    if (drc != DW_OK) return drc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const uint32_t tiles_c = static_cast<uint32_t>((cols + 127) / 128);
    const int64_t tiles_r = (rows + 127) / 128;
    const int rc = launch_tile_kernel<true, true, true>(static_cast<const uint16_t*>(x_bf16), static_cast<uint8_t*>(codes_row),
                                                        static_cast<uint8_t*>(scales_row), static_cast<uint8_t*>(codes_col_t),
                                                        static_cast<uint8_t*>(scales_col), rows, cols, tiles_c,
                                                        static_cast<uint32_t>(tiles_r) * tiles_c, scale_rule, scale_layout, di, st,
                                                        static_cast<float*>(workspace));
    if (rc != DW_OK) return rc;
    if (launch_pdl(mx_colsum_reduce_kernel, dim3(static_cast<unsigned>((cols + 31) / 32)), dim3(256), 0, st,
                   static_cast<const float*>(workspace), tiles_r, cols, colsum_out, colsum_is_bf16) != cudaSuccess) {
        cudaGetLastError();
        return DW_ERR_LAUNCH;
    }
    return DW_OK;
}

extern "C" DW_API int dw_mxfp8_update_amax_history(const void* x_bf16, float* amax_history, int history_len, int64_t num_elements,
                                                   void* stream) {
    if (!amax_history || history_len <= 0 || num_elements < 0 || (num_elements > 0 && !x_bf16)) return DW_ERR_BAD_ARG;
    if ((reinterpret_cast<uintptr_t>(amax_history) & 3) != 0 || (reinterpret_cast<uintptr_t>(x_bf16) & 1) != 0) return DW_ERR_BAD_ARG;
    DeviceInfo di;
    const int drc = current_device(&di);
    if (drc != DW_OK) return drc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    mx_amax_shift_kernel<<<1, 1, 0, st>>>(amax_history, history_len);
    if (launch_status() != DW_OK) return DW_ERR_LAUNCH;
    if (num_elements == 0) return DW_OK;
    const int64_t want = (num_elements / 16 + 255) / 256 + 1;
    const int grid = static_cast<int>(std::min<int64_t>(want, static_cast<int64_t>(di.sms) * 8));
    mx_amax_kernel<<<grid, 256, 0, st>>>(static_cast<const uint16_t*>(x_bf16), num_elements, amax_history);
    return launch_status();
}

extern "C" DW_API int dw_mxfp8_dequantize(const void* codes, const void* scales, void* out_bf16, int64_t rows, int64_t cols,
                                   int scale_layout, void* stream) {
    if (rows < 0 || cols < 0) return DW_ERR_BAD_ARG;
    if (scale_layout != DW_SF_FLAT && scale_layout != DW_SF_TILED) return DW_ERR_BAD_ARG;
    if (rows == 0 || cols == 0) return DW_OK;
    if (!codes || !scales || !out_bf16) return DW_ERR_BAD_ARG;
    if (cols % 16 == 0 && (!aligned(codes, 16) || !aligned(out_bf16, 16))) return DW_ERR_BAD_ARG;
    DeviceInfo di;
    const int drc = current_device(&di);
    if (drc != DW_OK) return drc;
    const int64_t total = rows * ((cols + 15) / 16);
    const int grid = static_cast<int>(std::min<int64_t>((total + 255) / 256, static_cast<int64_t>(di.sms) * 16));
    mx_dequant_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint8_t*>(codes), static_cast<const uint8_t*>(scales), static_cast<uint16_t*>(out_bf16), rows,
        cols, scale_layout);
    return launch_status();
}
