// Block-scaled MXFP8 GEMM for sm_100a:  D[M,N] = bf16(alpha * A[M,K] . B[N,K]^T + beta * D + bias).
//
// Replaces launch_blackwell_mxfp8_gemm (csrc/blackwell_gemm_kernel.cu:103-156, a bf16 cuBLAS call
// that ignores its scale arguments) and the never-launched blackwell_tcgen05_mma_kernel (:171-257).
//
// A and B are E4M3 codes, K-major, with one E8M0 scale per 32 elements of K stored in the tiled
// layout of DW_SF_TILED.  The kernel is persistent and warp-specialised:
//
//   warp 0      TMA producer: per 128-wide k-block, operand tiles (128-byte swizzle) and the
//               512-byte scale tiles into a ring of shared-memory stages
//   warp 1      MMA issuer (one thread): tcgen05.cp moves the stage's scales into TMEM, then four
//               tcgen05.mma.kind::mxf8f6f4.block_scale (K = 32 each) accumulate into TMEM;
//               tcgen05.commit hands the stage back to the producer
//   warps 2-9   epilogue, two warps per TMEM lane quadrant, each on half of the columns: tcgen05.ld
//               the fp32 accumulator, alpha/beta/bias/activation, bf16, then shared memory and a TMA
//               store per 32 x 32 box (per-thread stores for ragged N, beta reads, split-K partials
//               and the fused quantised output)
//
// kCtas == 2 pairs two CTAs (a cluster of 2 along M) on one 256 x BN tile with cta_group::2: each
// CTA stages its own half of A and its own half of B; the leader CTA issues the MMAs for both.
// No load is multicast; every CTA fetches what it needs with its own TMA loads.
//
// Every wait is bounded: on expiry the CTA raises an abort flag, records a code in the status word
// and unwinds through the common exit (TMEM is always freed).

#include <algorithm>
#include <atomic>
#include <mutex>

#include "dw_common.cuh"
#include "dw_ptx.cuh"

namespace dw {

struct GemmParams {
    uint16_t* d;
    const uint16_t* bias;
    int* status;
    int64_t M, N, K;
    float alpha, beta;
    uint32_t tiles_m, tiles_n, num_tiles, num_kblocks, group_m;
    // Split-K: the k-blocks of every tile are divided among `splits` work units (unit = tile +
    // split * num_tiles); each unit leaves its raw fp32 accumulator in `partial` ([splits][M][N]) and
    // mx_splitk_reduce_kernel sums them.  splits == 1: the epilogue writes D directly.
    uint32_t splits, kb_per_split;
    float* partial;
    // Fused epilogue: activation after alpha/beta/bias, and optionally the output quantised row-wise
    // (blocks of 32 along N) as the next GEMM's A operand: codes [M, N] + tiled scales.  d may be null then.
    // act == DW_ACT_SWIGLU: the N columns are gate/up pairs interleaved in groups of 32 (columns [64 j, 64 j + 32) gate,
    // [64 j + 32, 64 j + 64) up of output columns [32 j, 32 j + 32)); the outputs (d, q_codes, q_scales) have out_n = N / 2
    // columns.  Otherwise out_n == N.
    int act, q_rule;
    uint8_t* q_codes;
    uint8_t* q_scales;
    int64_t q_kt, out_n;
    // Optional tuning counters (the caller's workspace): per CTA, SM cycles each role spent waiting
    //   [0] producer: free stage       [1] MMA issuer: accumulator drained (two tiles back)
    //   [2] MMA issuer: shared accumulator columns drained (previous tile)
    //   [3] MMA issuer: operand data   [4] epilogue warp 2: accumulator finished   [7] kernel cycles
    long long* wait_cycles;
    // 1: the bf16 output leaves through shared memory and TMA stores (tm_d is valid); 0: per-thread stores
    int tma_store;
    // Grouped GEMM (one launch over the experts of an MoE layer): A is the row-wise concatenation of the
    // groups' activations, each group padded to whole row tiles; tile_group[row tile] names the group whose
    // weight (rows [g N, (g + 1) N) of B) that tile multiplies.  nullptr: one ordinary GEMM.
    const int* tile_group;
    uint32_t num_groups;
    // 1: a unit's first k-block takes the stage after the previous unit's last one; 0: every unit starts at stage 0
    int ring_continues;
};
constexpr int kWaitCounters = 8;
// warp 0: TMA producer, warp 1: MMA issuer, warps 2-9: epilogue (two warps per TMEM lane quadrant,
// each taking half of the accumulator's columns)
constexpr int kEpilogueWarps = 8;
constexpr int kGemmThreads = 64 + 32 * kEpilogueWarps;
template <int BN, int kCtas, int kGroup>
struct GemmCfg {
    static constexpr int kBM = 128;                       // rows per CTA
    static constexpr int kBK = 128;                       // bytes (= elements) of K per stage
    static constexpr int kABytes = kBM * kBK;
    static constexpr int kBRows = BN / kCtas;             // B rows staged by one CTA
    static constexpr int kBBytes = kBRows * kBK;
    static constexpr int kSfaBytes = 512;
    // 128-row scale tiles of B that a BN-wide column tile can touch: with BN = 192 every other tile
    // starts 64 rows into its first scale tile.  (BN must be a multiple of 64: a 224-wide tile, whose
    // scales would start at an odd tensor-memory column, raised "misaligned address" on B200.)
    static_assert(BN % 64 == 0, "column tile width");
    static constexpr int kSfbTiles = (BN % 128 == 0) ? BN / 128 : (BN + 64 + 127) / 128;
    static constexpr int kSfbBytes = kSfbTiles * 512;
    static constexpr int kStageBytes = (kABytes + kBBytes + kSfaBytes + kSfbBytes + 1023) / 1024 * 1024;
    static constexpr int kFit = 212 * 1024 / kStageBytes;
    static constexpr int kStages = (kFit >= 8 ? 8 : kFit) / (kGroup % 2 ? 2 * kGroup : kGroup) * (kGroup % 2 ? 2 * kGroup : kGroup);
    // stages are handed back to the producer `kGroup` at a time: one tcgen05.commit per group
    static constexpr int kGroups = kStages / kGroup;
    static_assert(kGroup == 1, "a unit may start in the middle of the ring: stages are handed back one at a time");
    static_assert(kStages % 2 == 0 && kStages % kGroup == 0 && kGroups >= 2, "ring shape");
    // Tensor memory (512 columns): two accumulators and two sets of scale columns.  With BN = 256 the
    // two accumulators cannot both be 256 columns wide next to the scales, so they OVERLAP by 32
    // columns: acc0 = [0,256), acc1 = [224,480).  The epilogue drains the shared 32 columns of a
    // finished tile first and signals them free; the next tile's MMAs (which write the other
    // accumulator) start then, while the remaining 224 columns are drained under the mainloop.
    static constexpr int kAccStages = 2;
    static constexpr int kAccStride = (BN == 256) ? 224 : BN;
    static constexpr bool kOverlap = kAccStride < BN;
    static constexpr int kSfBase = (BN == 256) ? 480 : 2 * BN;   // first scale column
    static constexpr int kSfSetCols = 16;                  // columns per scale set (A: 4, B: up to 8)
    static constexpr int kTmemCols = 512;
    static constexpr int kBarrierBytes = 256;
    // Output staging for the TMA-store epilogue: per epilogue warp one slot of 32 rows x 32 bf16
    // columns (64-byte rows, 64-byte swizzle).
    static constexpr int kOutSlotBytes = 32 * 64;
    static constexpr int kOutBytes = 8 * kOutSlotBytes;
    static constexpr int kSmemBytes = kStages * kStageBytes + kOutBytes + kBarrierBytes + 1024;  // + alignment slack
    static_assert(kSmemBytes <= 227 * 1024, "shared memory per CTA");
    static constexpr uint32_t kTxBytes = kCtas * (kABytes + kBBytes + kSfaBytes + kSfbBytes);
    static_assert(kSfBase + 2 * kSfSetCols <= kTmemCols && 4 + 4 * kSfbTiles <= kSfSetCols, "TMEM columns");
    static_assert(kAccStride + BN <= kSfBase, "accumulators must not reach the scale columns");
    static_assert(kStages >= 2, "pipeline depth");
};

// ReLU / exact GELU / SiLU on the fp32 value before it is rounded to bf16
// (EpilogueConfig::Op::{BiasReLU, BiasGELU, BiasSwish} of the reference, csrc/cutlass_kernels.h:65-77, never applied there).
__device__ __forceinline__ float apply_activation(float x, int act) {
    if (act == DW_ACT_RELU) return fmaxf(x, 0.0f);
    if (act == DW_ACT_GELU) return 0.5f * x * (1.0f + erff(x * 0.70710678118654752f));
    if (act == DW_ACT_SILU) return x / (1.0f + expf(-x));
    return x;
}

enum : int { kErrProducer = 1, kErrMmaFull = 2, kErrMmaAcc = 3, kErrEpilogue = 4, kErrSelfTest = 5 };

template <int BN, int kCtas, int kGroup>
__global__ void __launch_bounds__(kGemmThreads, 1)
mx_gemm_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
               const __grid_constant__ CUtensorMap tm_sfa, const __grid_constant__ CUtensorMap tm_sfb,
               const __grid_constant__ CUtensorMap tm_d, const GemmParams p) {
    using Cfg = GemmCfg<BN, kCtas, kGroup>;
    constexpr int kStages = Cfg::kStages, kAcc = Cfg::kAccStages;
    extern __shared__ uint8_t smem_raw[];

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t rank = (kCtas == 2) ? ptx::cluster_ctarank() : 0u;
    const bool leader = rank == 0u;

    // ---- shared memory carve-up (1024-byte aligned for the 128-byte swizzle) ----
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    auto stage_a = [&](int s) { return smem_base + s * Cfg::kStageBytes; };
    auto stage_b = [&](int s) { return stage_a(s) + Cfg::kABytes; };
    auto stage_sfa = [&](int s) { return stage_b(s) + Cfg::kBBytes; };
    auto stage_sfb = [&](int s) { return stage_sfa(s) + Cfg::kSfaBytes; };
    const uint32_t out_base = smem_base + kStages * Cfg::kStageBytes;          // 1024-byte aligned
    const uint32_t bar_base = out_base + Cfg::kOutBytes;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int g) { return bar_base + 8u * (kStages + g); };   // one per group of stages
    auto accf_bar = [&](int a) { return bar_base + 8u * (2 * kStages + a); };
    auto acce_bar = [&](int a) { return bar_base + 8u * (2 * kStages + kAcc + a); };
    const uint32_t ovl_bar = bar_base + 8u * (2 * kStages + 2 * kAcc);   // shared accumulator columns drained
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem_gen + kStages * Cfg::kStageBytes + Cfg::kOutBytes + 8 * (2 * kStages + 2 * kAcc + 1));
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) ptx::mbar_init(full_bar(s), 1);
        for (int g = 0; g < Cfg::kGroups; ++g) ptx::mbar_init(empty_bar(g), 1);
        for (int a = 0; a < kAcc; ++a) { ptx::mbar_init(accf_bar(a), 1); ptx::mbar_init(acce_bar(a), kEpilogueWarps * kCtas); }
        ptx::mbar_init(ovl_bar, 4 * kCtas);
        *abort_flag = 0;
        ptx::fence_barrier_init();
        ptx::prefetch_tmap(&tm_a); ptx::prefetch_tmap(&tm_b); ptx::prefetch_tmap(&tm_sfa); ptx::prefetch_tmap(&tm_sfb);
        if (p.tma_store) ptx::prefetch_tmap(&tm_d);
    }
    if (warp == 1) {  // TMEM allocation: one warp, the same warp in both CTAs of a pair
        ptx::tmem_alloc<kCtas>(smem_u32(tmem_slot), Cfg::kTmemCols);
        ptx::tmem_relinquish<kCtas>();
    }
    ptx::tc_fence_before();
    __syncthreads();
    if (kCtas == 2) ptx::cluster_sync();   // peer barriers initialised before any remote arrive
    ptx::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // Every CTA of this grid is resident and set up: a kernel that was launched behind this one on the same stream with
    // programmatic stream serialisation (the quantiser of the next layer's operands, dw_mxfp8_quantize_ex with
    // DW_QUANT_OVERLAP_PREVIOUS) may start now and take the SMs this grid does not occupy.  Without such a launch
    // behind it the instruction does nothing.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    // This kernel itself is launched the same way: everything above (barriers, tensor memory, tensor-map prefetch) may have
    // run while the kernel before it on the stream (usually the quantiser of its operands) was finishing; from here on
    // that kernel has completed and its writes are visible.
    pdl_wait();

    const uint32_t num_workers = gridDim.x / kCtas, worker = blockIdx.x / kCtas;
    const uint32_t num_units = p.num_tiles * p.splits;
    int err = 0;
    const bool timed = p.wait_cycles != nullptr;
    const long long t_begin = timed ? clock64() : 0;
    long long waited[3] = {0, 0, 0};
    auto timed_wait = [&](uint32_t bar, uint32_t parity, int slot) {
        if (!timed) return ptx::mbar_wait<kCtas == 2>(bar, parity, abort_flag);
        const long long t0 = clock64();
        const bool ok = ptx::mbar_wait<kCtas == 2>(bar, parity, abort_flag);
        waited[slot] += clock64() - t0;
        return ok;
    };
    // Tile order: bands of `group_m` row tiles, column tiles outer, row tiles inner, so the CTAs
    // running at the same time share a small set of A and B tiles in L2.
    auto tile_coords = [&](uint32_t tile, uint32_t& tm, uint32_t& tn) {
        const uint32_t per_band = p.group_m * p.tiles_n;
        const uint32_t band = tile / per_band, in_band = tile - band * per_band;
        const uint32_t first = band * p.group_m;
        const uint32_t rows_in_band = min(p.group_m, p.tiles_m - first);
        tn = in_band / rows_in_band;
        tm = first + (in_band - tn * rows_in_band);
    };

    // Both pipeline roles walk the stage ring with compile-time stage indices (the k loop is unrolled
    // by the ring depth; a tile that starts in the middle of the ring skips the first stages of its
    // first pass), so addresses and descriptors are constants plus one base register and the single
    // issuing thread does almost no arithmetic.
    // Each stage's barrier parity is one bit of a mask, flipped on every use of that stage.
    if (warp == 0) {
        // ================= TMA producer (whole warp walks the ring, one elected lane issues) =================
        {
            uint32_t empty_parity = 0;   // bit g: parity of the next wait on empty_bar(g), inverted
            int ring_at = 0;             // stage of the next k-block
            const uint32_t full0 = (kCtas == 2) ? ptx::map_to_cta(full_bar(0), 0) : full_bar(0);   // leader's barrier
            const int nkb = static_cast<int>(p.num_kblocks);
            for (uint32_t unit = worker; unit < num_units && !err; unit += num_workers) {
                const uint32_t split = unit / p.num_tiles, tile = unit - split * p.num_tiles;
                uint32_t tm, tn;
                tile_coords(tile, tm, tn);
                const int row_a = static_cast<int>(tm * (128 * kCtas) + rank * 128);
                uint32_t b_first = tn * BN;                                       // first row of B for this column tile
                if (p.tile_group != nullptr)
                    b_first += min(static_cast<uint32_t>(max(p.tile_group[tm], 0)), p.num_groups - 1u) * static_cast<uint32_t>(p.N);
                const int row_b = static_cast<int>(b_first + rank * Cfg::kBRows);
                const int sfa_row = static_cast<int>(tm * kCtas + rank) * nkb;
                const int sfb_row = static_cast<int>(b_first / 128u) * nkb;       // first scale tile the column tile touches
                const int kb_first = static_cast<int>(split * p.kb_per_split);
                const int kb_end = min(nkb, kb_first + static_cast<int>(p.kb_per_split));
                // The ring runs on across tiles: this unit's first k-block takes the stage after the previous unit's last
                // one (`ring_at`), so the loads of a new tile start as soon as ANY stage is free, not when stage 0 is.  The
                // stage index stays a compile-time constant: the first pass through the unrolled body skips the stages
                // before `ring_at`.
                for (int kb0 = kb_first - ring_at; kb0 < kb_end && !err; kb0 += kStages) {
#pragma unroll
                    for (int s = 0; s < kStages; ++s) {
                        const int kb = kb0 + s;
                        if (kb >= kb_first && kb < kb_end && !err) {
                            if (s % kGroup == 0) {        // first stage of a group: wait until the group is free
                                const int g = s / kGroup;
                                if (!timed_wait(empty_bar(g), ((empty_parity >> g) & 1u) ^ 1u, 0)) { err = kErrProducer; continue; }
                                empty_parity ^= 1u << g;
                            }
                            const uint32_t bar = full0 + 8u * s;
                            if (!ptx::elect_one()) continue;
                            if (leader) ptx::mbar_arrive_expect_tx(full_bar(s), Cfg::kTxBytes);
                            if (kCtas == 2) {
                                ptx::tma_load_2d_pair(stage_a(s), &tm_a, bar, kb * Cfg::kBK, row_a);
                                ptx::tma_load_2d_pair(stage_b(s), &tm_b, bar, kb * Cfg::kBK, row_b);
                                ptx::tma_load_2d_pair(stage_sfa(s), &tm_sfa, bar, 0, sfa_row + kb);
#pragma unroll
                                for (int j = 0; j < Cfg::kSfbTiles; ++j)
                                    ptx::tma_load_2d_pair(stage_sfb(s) + 512 * j, &tm_sfb, bar, 0, sfb_row + j * nkb + kb);
                            } else {
                                ptx::tma_load_2d(stage_a(s), &tm_a, bar, kb * Cfg::kBK, row_a);
                                ptx::tma_load_2d(stage_b(s), &tm_b, bar, kb * Cfg::kBK, row_b);
                                ptx::tma_load_2d(stage_sfa(s), &tm_sfa, bar, 0, sfa_row + kb);
#pragma unroll
                                for (int j = 0; j < Cfg::kSfbTiles; ++j)
                                    ptx::tma_load_2d(stage_sfb(s) + 512 * j, &tm_sfb, bar, 0, sfb_row + j * nkb + kb);
                            }
                        }
                    }
                }
                if (p.ring_continues) ring_at = (ring_at + (kb_end - kb_first)) % kStages;
            }
        }
    } else if (warp == 1) {
        // ================= MMA issuer (leader CTA only; whole warp walks, one elected lane issues) =================
        if (leader) {
            uint32_t full_parity = 0, acc = 0, acc_phase = 0, tiles_done = 0;
            int ring_at = 0;             // stage of the next k-block (the producer counts the same way)
            constexpr uint32_t idesc = ptx::idesc_mxf8(128 * kCtas, BN);
            constexpr uint32_t kStageStep = Cfg::kStageBytes >> 4;          // descriptor units of 16 bytes
            const uint32_t a_lo0 = ptx::desc_lo_sw128(stage_a(0)), b_lo0 = ptx::desc_lo_sw128(stage_b(0));
            const uint32_t sfa_lo0 = ptx::desc_lo_sf(stage_sfa(0)), sfb_lo0 = ptx::desc_lo_sf(stage_sfb(0));
            const uint32_t sf_t0 = tmem_base + Cfg::kSfBase;
            const int nkb = static_cast<int>(p.num_kblocks);
            for (uint32_t unit = worker; unit < num_units && !err; unit += num_workers) {
                const uint32_t split = unit / p.num_tiles;
                const int kb_first = static_cast<int>(split * p.kb_per_split);
                const int kb_end = min(nkb, kb_first + static_cast<int>(p.kb_per_split));
                // A column tile that starts 32 g rows into its first scale tile reads its B scales from
                // column g of the copied tiles on (one TMEM column holds the scales of 32 rows); g is 0 or 2.
                uint32_t sfb_shift = 0;
                if (BN % 128 != 0) {
                    uint32_t tm, tn;
                    tile_coords(unit - split * p.num_tiles, tm, tn);
                    sfb_shift = ((tn * BN) % 128u) / 32u;
                }
                // this accumulator fully drained (two tiles ago) ...
                if (!timed_wait(acce_bar(acc), acc_phase ^ 1u, 0)) { err = kErrMmaAcc; break; }
                // ... and the columns it shares with the other accumulator drained (previous tile)
                if (Cfg::kOverlap && tiles_done > 0 &&
                    !timed_wait(ovl_bar, (tiles_done - 1u) & 1u, 1)) { err = kErrMmaAcc; break; }
                ptx::tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * Cfg::kAccStride;
                uint32_t accumulate = 0;
                for (int kb0 = kb_first - ring_at; kb0 < kb_end && !err; kb0 += kStages) {
#pragma unroll
                    for (int s = 0; s < kStages; ++s) {
                        if (kb0 + s >= kb_first && kb0 + s < kb_end && !err) {
                            if (!timed_wait(full_bar(s), (full_parity >> s) & 1u, 2)) { err = kErrMmaFull; continue; }
                            full_parity ^= 1u << s;
                            ptx::tc_fence_after();
                            // scales of this k-block: shared memory -> tensor memory; two column sets
                            // alternate so the copy never overwrites scales the previous MMAs still read
                            const uint32_t sfa_t = sf_t0 + (s & 1) * Cfg::kSfSetCols, sfb_t = sfa_t + 4;
                            const uint32_t acc_now = accumulate;
                            accumulate = 1;
                            if (!ptx::elect_one()) continue;
                            ptx::tc_cp_sf<kCtas>(sfa_t, sfa_lo0 + s * kStageStep);
#pragma unroll
                            for (int j = 0; j < Cfg::kSfbTiles; ++j)
                                ptx::tc_cp_sf<kCtas>(sfb_t + 4 * j, sfb_lo0 + s * kStageStep + 32 * j);
#pragma unroll
                            for (uint32_t k = 0; k < 4; ++k) {
                                // +2 descriptor units = 32 bytes along K inside the 128-byte swizzle atom
                                ptx::tc_mma_mxf8<kCtas>(d_tmem, a_lo0 + s * kStageStep + 2 * k, b_lo0 + s * kStageStep + 2 * k,
                                                        ptx::idesc_with_sf_ids(idesc, k, k), sfa_t, sfb_t + sfb_shift, acc_now | k);
                            }
                            // Last stage of a group (or of the tile): the group is free again once the MMAs
                            // issued so far have read it.  (Measured: releasing stages one at a time,
                            // kGroup = 1, is fastest; coarser groups lengthen the refill latency.)
                            if (s % kGroup == kGroup - 1 || kb0 + s == kb_end - 1) {
                                const int g = s / kGroup;
                                if (kCtas == 2) ptx::tc_commit_both(empty_bar(g)); else ptx::tc_commit(empty_bar(g));
                            }
                        }
                    }
                }
                if (err) break;
                if (p.ring_continues) ring_at = (ring_at + (kb_end - kb_first)) % kStages;
                if (ptx::elect_one()) {
                    if (kCtas == 2) ptx::tc_commit_both(accf_bar(acc)); else ptx::tc_commit(accf_bar(acc));
                }
                __syncwarp();
                ++tiles_done;
                if (++acc == kAcc) { acc = 0; acc_phase ^= 1u; }
            }
        }
    } else {
        // ================= epilogue (8 warps: 4 TMEM lane quadrants x 2 column halves) =================
        const uint32_t q = warp & 3u;                    // TMEM lane quadrant this warp may read
        const uint32_t half = (warp - 2u) >> 2;          // which half of the accumulator's columns
        uint32_t acc = 0, acc_phase = 0;
        const bool vec_ok = (p.N % 8) == 0;
        constexpr int kChunks = BN / 32, kHalfChunks = (kChunks + 1) / 2;
        const int ch_begin = static_cast<int>(half) * kHalfChunks;
        const int ch_count = min(kChunks, ch_begin + kHalfChunks) - ch_begin;
        const uint32_t slot = out_base + (warp - 2u) * Cfg::kOutSlotBytes;
        // Kernel parameters the chunk loop branches on, read once into registers: fetched from the parameter bank
        // inside the loop, the chain of dependent loads and branches took ~350 cycles per chunk (measured).
        const int64_t M_ = p.M, N_ = p.N;
        const uint16_t* const bias = p.bias;
        const int act = p.act;
        // the common epilogue: D = bf16(accumulator + bias) through the TMA store and nothing else
        const bool plain = p.splits <= 1 && vec_ok && p.tma_store != 0 && p.alpha == 1.0f && p.beta == 0.0f &&
                           p.act == DW_ACT_NONE && p.q_codes == nullptr;
        // This warp's 32 rows x 32 columns go to its staging slot (row r at 64 r, its four 16-byte pieces permuted
        // by the 64-byte swizzle so that the stores of a quarter warp cover all banks), then one TMA store writes
        // the box as whole 64-byte row segments and clips rows beyond M.  The slot is refilled only after the
        // previous store has read it.
        auto stage_and_store = [&](const uint32_t (&o)[16], bool in_rows, int64_t col, int64_t row0) {
            if (lane == 0) ptx::bulk_wait_read<0>();
            __syncwarp();
            if (in_rows) {
                const uint32_t row_addr = slot + lane * 64u, sw = (lane >> 1) & 3u;
#pragma unroll
                for (uint32_t v = 0; v < 4; ++v)
                    ptx::sts_v4(row_addr + ((v ^ sw) << 4), o[4 * v], o[4 * v + 1], o[4 * v + 2], o[4 * v + 3]);
            }
            ptx::fence_proxy_async();
            __syncwarp();
            if (lane == 0) {
                ptx::tma_store_2d(&tm_d, slot, static_cast<int>(col), static_cast<int>(row0));
                ptx::bulk_commit();
            }
        };
        for (uint32_t unit = worker; unit < num_units && !err; unit += num_workers) {
            const uint32_t split = unit / p.num_tiles, tile = unit - split * p.num_tiles;
            uint32_t tm, tn;
            tile_coords(tile, tm, tn);
            const int64_t row = static_cast<int64_t>(tm) * (128 * kCtas) + rank * 128 + q * 32 + lane;
            const int64_t col0 = static_cast<int64_t>(tn) * BN;
            if (!timed_wait(accf_bar(acc), acc_phase, 0)) { err = kErrEpilogue; break; }
            ptx::tc_fence_after();
            const uint32_t t_row = tmem_base + acc * Cfg::kAccStride + ((q * 32u) << 16);
            // The 32 columns shared with the other accumulator (the last chunk of accumulator 0, the
            // first chunk of accumulator 1) are drained first by the warps that own them.
            const bool shared_last = Cfg::kOverlap && acc == 0 && half == 1;     // shared chunk is this warp's last one
            const bool owns_shared = Cfg::kOverlap && (acc == 0 ? half == 1 : half == 0);
            // The bias of a chunk (64 bytes, the same for every lane) is fetched one chunk ahead: with nearly all of
            // the SM's L1 configured as shared memory these loads come from L2 (~350 cycles when fetched in place).
            auto chunk_of = [&](int it) { return ch_begin + (shared_last ? (it == 0 ? ch_count - 1 : it - 1) : it); };
            auto load_bias = [&](int it, uint4 (&b)[4]) {
                const int64_t bcol = col0 + chunk_of(it) * 32;
                if (bias != nullptr && vec_ok && bcol + 32 <= N_) {
#pragma unroll
                    for (int v = 0; v < 4; ++v) b[v] = *reinterpret_cast<const uint4*>(bias + bcol + 8 * v);
                }
            };
            if (act == DW_ACT_SWIGLU) {
                // Gate and up columns of the same 32 outputs sit in neighbouring chunks (2 j, 2 j + 1), both in this warp's
                // half: h = silu(gate) * up in fp32, rounded to bf16 once, then quantised as one MX block of the next
                // GEMM's A operand.  The pair that holds the shared accumulator columns goes first.
                const int npairs = ch_count / 2;
                const int64_t F_ = p.out_n;
#pragma unroll 1
                for (int ip = 0; ip < npairs; ++ip) {
                    const int pr = shared_last ? npairs - 1 - ip : ip;
                    const int cg = (ch_begin + 2 * pr) * 32;                       // gate chunk; the up chunk follows it
                    uint32_t rg[32], ru[32];
                    ptx::tc_ld_32x32b_x32(t_row + cg, rg);
                    ptx::tc_ld_32x32b_x32(t_row + cg + 32, ru);
                    ptx::tc_wait_ld();
                    if (owns_shared && ip == 0) {
                        ptx::tc_fence_before();
                        __syncwarp();
                        if (lane == 0) {
                            if (kCtas == 2) ptx::mbar_arrive_cluster(ovl_bar, 0); else ptx::mbar_arrive(ovl_bar);
                        }
                    }
                    const int64_t ocol = (col0 + cg) >> 1;                         // first of the 32 output columns
                    const bool in_rows = row < M_;
                    if (ocol + 32 <= F_) {
                        uint32_t o[16];
                        if (in_rows) {
                            float h[32];
#pragma unroll
                            for (int i = 0; i < 32; ++i) {
                                float gv = __uint_as_float(rg[i]) * p.alpha, uv = __uint_as_float(ru[i]) * p.alpha;
                                if (bias != nullptr) {
                                    gv += __uint_as_float(static_cast<uint32_t>(bias[col0 + cg + i]) << 16);
                                    uv += __uint_as_float(static_cast<uint32_t>(bias[col0 + cg + 32 + i]) << 16);
                                }
                                h[i] = apply_activation(gv, DW_ACT_SILU) * uv;
                            }
#pragma unroll
                            for (int i = 0; i < 16; ++i)
                                asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(o[i]) : "f"(h[2 * i + 1]), "f"(h[2 * i]));
                            if (p.d != nullptr && !p.tma_store) {
                                uint16_t* dst = p.d + row * F_ + ocol;
#pragma unroll
                                for (int v = 0; v < 4; ++v)
                                    *reinterpret_cast<uint4*>(dst + 8 * v) = make_uint4(o[4 * v], o[4 * v + 1], o[4 * v + 2], o[4 * v + 3]);
                            }
                        }
                        if (p.tma_store && row - lane < M_) stage_and_store(o, in_rows, ocol, row - lane);
                        if (p.q_codes != nullptr) {
                            if (in_rows) {
                                const uint32_t sb = e8m0_from_amax(fold_amax(amax_words(o)), p.q_rule);
                                const uint32_t inv = e8m0_inverse_bf16x2(sb);
                                uint32_t q[8];
#pragma unroll
                                for (int i = 0; i < 8; ++i) q[i] = quant_word(o[2 * i], inv) | (quant_word(o[2 * i + 1], inv) << 16);
                                uint8_t* qd = p.q_codes + row * F_ + ocol;
                                if ((reinterpret_cast<uintptr_t>(qd) & 31) == 0) {
                                    asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(qd), "r"(q[0]), "r"(q[1]),
                                                 "r"(q[2]), "r"(q[3]), "r"(q[4]), "r"(q[5]), "r"(q[6]), "r"(q[7]) : "memory");
                                } else {
                                    stg_v4(qd, make_uint4(q[0], q[1], q[2], q[3]));
                                    stg_v4(qd + 16, make_uint4(q[4], q[5], q[6], q[7]));
                                }
                                p.q_scales[sf_tiled_offset(row, ocol >> 5, p.q_kt)] = static_cast<uint8_t>(sb);
                            } else if (row < ((M_ + 127) & ~int64_t(127))) {
                                p.q_scales[sf_tiled_offset(row, ocol >> 5, p.q_kt)] = 127;         // padding rows of the last tile
                            }
                        }
                    } else if (p.q_codes != nullptr && ocol < ((F_ + 127) & ~int64_t(127)) && row < ((M_ + 127) & ~int64_t(127))) {
                        p.q_scales[sf_tiled_offset(row, ocol >> 5, p.q_kt)] = 127;                 // padding k-blocks of the scale tile
                    }
                }
                ptx::tc_fence_before();
                __syncwarp();
                if (lane == 0) {
                    if (kCtas == 2) ptx::mbar_arrive_cluster(acce_bar(acc), 0); else ptx::mbar_arrive(acce_bar(acc));
                }
                if (++acc == kAcc) { acc = 0; acc_phase ^= 1u; }
                continue;
            }
            uint4 bias_next[4] = {};
            load_bias(0, bias_next);
#pragma unroll 1
            for (int it = 0; it < ch_count; ++it) {
                const int ch = chunk_of(it);
                const int c = ch * 32;
                uint4 bias_now[4];
#pragma unroll
                for (int v = 0; v < 4; ++v) bias_now[v] = bias_next[v];
                if (it + 1 < ch_count) load_bias(it + 1, bias_next);
                uint32_t r[32];
                ptx::tc_ld_32x32b_x32(t_row + c, r);
                ptx::tc_wait_ld();
                if (owns_shared && it == 0) {            // shared columns are in registers: release them
                    ptx::tc_fence_before();
                    __syncwarp();
                    if (lane == 0) {
                        if (kCtas == 2) ptx::mbar_arrive_cluster(ovl_bar, 0); else ptx::mbar_arrive(ovl_bar);
                    }
                }
                const int64_t col = col0 + c;
                if (plain && col + 32 <= N_) {
                    const bool in_rows = row < M_;
                    uint32_t o[16];
                    if (in_rows) {
                        float f[32];
#pragma unroll
                        for (int i = 0; i < 32; ++i) f[i] = __uint_as_float(r[i]);
                        if (bias != nullptr) {
#pragma unroll
                            for (int v = 0; v < 4; ++v) {
                                const uint32_t ow[4] = {bias_now[v].x, bias_now[v].y, bias_now[v].z, bias_now[v].w};
#pragma unroll
                                for (int i = 0; i < 4; ++i) add_bf16x2(ow[i], f[8 * v + 2 * i], f[8 * v + 2 * i + 1]);
                            }
                        }
#pragma unroll
                        for (int i = 0; i < 16; ++i)
                            asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(o[i]) : "f"(f[2 * i + 1]), "f"(f[2 * i]));
                    }
                    if (row - lane < M_) stage_and_store(o, in_rows, col, row - lane);
                    continue;
                }
                if (p.splits > 1) {                      // split-K: raw fp32 partial sums, reduced afterwards
                    if (row < p.M && col < p.N) {
                        float* dst = p.partial + (static_cast<int64_t>(split) * p.M + row) * p.N + col;
                        if ((p.N % 4) == 0 && col + 32 <= p.N) {
#pragma unroll
                            for (int v = 0; v < 8; ++v)
                                *reinterpret_cast<uint4*>(dst + 4 * v) = make_uint4(r[4 * v], r[4 * v + 1], r[4 * v + 2], r[4 * v + 3]);
                        } else {
#pragma unroll
                            for (int i = 0; i < 32; ++i)
                                if (col + i < p.N) dst[i] = __uint_as_float(r[i]);
                        }
                    }
                } else if (vec_ok && col + 32 <= p.N) {
                    // full chunk: 32 consecutive columns of one row = exactly one MX block of the output
                    const bool in_rows = row < p.M;
                    uint32_t o[16];                      // the 32 outputs as bf16x2 words
                    if (in_rows) {
                        float f[32];
#pragma unroll
                        for (int i = 0; i < 32; ++i) f[i] = __uint_as_float(r[i]);
                        if (p.alpha != 1.0f) {
#pragma unroll
                            for (int i = 0; i < 32; ++i) f[i] *= p.alpha;
                        }
                        if (p.beta != 0.0f) {
                            const uint16_t* old = p.d + row * p.N + col;
#pragma unroll
                            for (int v = 0; v < 4; ++v) {
                                const uint4 t4 = *reinterpret_cast<const uint4*>(old + 8 * v);
                                const uint32_t ow[4] = {t4.x, t4.y, t4.z, t4.w};
#pragma unroll
                                for (int i = 0; i < 4; ++i) {
                                    f[8 * v + 2 * i] += p.beta * __uint_as_float(ow[i] << 16);
                                    f[8 * v + 2 * i + 1] += p.beta * __uint_as_float(ow[i] & 0xFFFF0000u);
                                }
                            }
                        }
                        if (p.bias != nullptr) {
#pragma unroll
                            for (int v = 0; v < 4; ++v) {
                                const uint4 t4 = bias_now[v];
                                const uint32_t ow[4] = {t4.x, t4.y, t4.z, t4.w};
#pragma unroll
                                for (int i = 0; i < 4; ++i) add_bf16x2(ow[i], f[8 * v + 2 * i], f[8 * v + 2 * i + 1]);
                            }
                        }
                        // one uniform branch per chunk, then a loop of a single function: with the selection inside
                        // the loop every element paid for all three functions (ReLU cost as much as GELU)
                        if (act == DW_ACT_RELU) {
#pragma unroll
                            for (int i = 0; i < 32; ++i) f[i] = fmaxf(f[i], 0.0f);
                        } else if (act == DW_ACT_GELU) {
#pragma unroll
                            for (int i = 0; i < 32; ++i) f[i] = apply_activation(f[i], DW_ACT_GELU);
                        } else if (act == DW_ACT_SILU) {
#pragma unroll
                            for (int i = 0; i < 32; ++i) f[i] = apply_activation(f[i], DW_ACT_SILU);
                        }
#pragma unroll
                        for (int i = 0; i < 16; ++i)
                            asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(o[i]) : "f"(f[2 * i + 1]), "f"(f[2 * i]));
                        if (p.d != nullptr && !p.tma_store) {
                            uint16_t* dst = p.d + row * p.N + col;
#pragma unroll
                            for (int v = 0; v < 4; ++v)
                                *reinterpret_cast<uint4*>(dst + 8 * v) = make_uint4(o[4 * v], o[4 * v + 1], o[4 * v + 2], o[4 * v + 3]);
                        }
                    }
                    if (p.tma_store && row - lane < p.M) stage_and_store(o, in_rows, col, row - lane);
                    if (p.q_codes != nullptr) {
                        // the bf16 outputs quantised in place as the next GEMM's row-wise operand
                        if (in_rows) {
                            const uint32_t sb = e8m0_from_amax(fold_amax(amax_words(o)), p.q_rule);
                            const uint32_t inv = e8m0_inverse_bf16x2(sb);
                            uint32_t q[8];
#pragma unroll
                            for (int i = 0; i < 8; ++i) q[i] = quant_word(o[2 * i], inv) | (quant_word(o[2 * i + 1], inv) << 16);
                            uint8_t* qd = p.q_codes + row * p.N + col;
                            // 32 codes = one whole 32-byte sector (N % 32 == 0 and a 16-byte aligned base give 16-byte
                            // alignment; a single 256-bit store needs 32)
                            if ((reinterpret_cast<uintptr_t>(qd) & 31) == 0) {
                                asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(qd), "r"(q[0]), "r"(q[1]),
                                             "r"(q[2]), "r"(q[3]), "r"(q[4]), "r"(q[5]), "r"(q[6]), "r"(q[7]) : "memory");
                            } else {
                                stg_v4(qd, make_uint4(q[0], q[1], q[2], q[3]));
                                stg_v4(qd + 16, make_uint4(q[4], q[5], q[6], q[7]));
                            }
                            p.q_scales[sf_tiled_offset(row, col >> 5, p.q_kt)] = static_cast<uint8_t>(sb);
                        } else if (row < ((p.M + 127) & ~int64_t(127))) {
                            p.q_scales[sf_tiled_offset(row, col >> 5, p.q_kt)] = 127;     // padding rows of the last tile
                        }
                    }
                } else if (row < p.M && col < p.N) {     // ragged N: scalar stores, no fused quantisation
                    uint16_t* dst = p.d + row * p.N + col;
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        if (col + i >= p.N) break;
                        float f = p.alpha * __uint_as_float(r[i]);
                        if (p.beta != 0.0f) f += p.beta * __uint_as_float(static_cast<uint32_t>(dst[i]) << 16);
                        if (p.bias != nullptr) f += __uint_as_float(static_cast<uint32_t>(p.bias[col + i]) << 16);
                        f = apply_activation(f, p.act);
                        uint32_t ob;
                        asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(ob) : "f"(0.0f), "f"(f));
                        dst[i] = static_cast<uint16_t>(ob & 0xFFFFu);
                    }
                } else if (p.q_codes != nullptr && col >= p.N && col < ((p.N + 127) & ~int64_t(127)) &&
                           row < ((p.M + 127) & ~int64_t(127))) {
                    p.q_scales[sf_tiled_offset(row, col >> 5, p.q_kt)] = 127;             // padding k-blocks of the scale tile
                }
            }
            // accumulator drained: hand it back to the MMA issuer (on the leader CTA)
            ptx::tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                if (kCtas == 2) ptx::mbar_arrive_cluster(acce_bar(acc), 0); else ptx::mbar_arrive(acce_bar(acc));
            }
            if (++acc == kAcc) { acc = 0; acc_phase ^= 1u; }
        }
        if (p.tma_store && lane == 0) ptx::bulk_wait<0>();   // staged output has left shared memory and is written
    }

    // ================= common exit =================
    if (timed && lane == 0) {
        long long* out = p.wait_cycles + static_cast<size_t>(blockIdx.x) * kWaitCounters;
        if (warp == 0) { out[0] = waited[0]; out[7] = clock64() - t_begin; }
        if (warp == 1) { out[1] = waited[0]; out[2] = waited[1]; out[3] = waited[2]; }
        if (warp == 2) out[4] = waited[0];
    }
    if (err) {
        *abort_flag = err;
        if (p.status != nullptr) atomicCAS(p.status, 0, err | (static_cast<int>(blockIdx.x) << 8));
    }
    __syncwarp();
    __syncthreads();
    if (*abort_flag != 0) __nanosleep(200000);  // let any copy still in flight land before the CTA retires
    ptx::tc_fence_before();
    if (kCtas == 2) ptx::cluster_sync();        // the peer may still read this CTA's shared memory / TMEM
    __syncthreads();
    if (warp == 1) {
        ptx::tc_fence_after();
        ptx::tmem_dealloc<kCtas>(tmem_base, Cfg::kTmemCols);
    }
}

// D = bf16(alpha * sum_s partial[s] + beta * D + bias): the second step of a split-K GEMM.
__global__ void __launch_bounds__(256)
mx_splitk_reduce_kernel(const float* __restrict__ partial, uint16_t* __restrict__ d, const uint16_t* __restrict__ bias,
                        int64_t M, int64_t N, uint32_t splits, float alpha, float beta) {
    pdl_wait();                      // the GEMM that wrote the partial sums has completed
    pdl_launch_dependents();
    const int64_t total = M * N, plane = M * N;
    const bool vec = (N % 4) == 0;
    const int64_t step = static_cast<int64_t>(gridDim.x) * blockDim.x * 4;
    for (int64_t i = (blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x) * 4; i < total; i += step) {
        float f[4] = {0.f, 0.f, 0.f, 0.f};
        const int n = vec ? 4 : static_cast<int>(total - i < 4 ? total - i : 4);
        for (uint32_t s = 0; s < splits; ++s) {
            const float* src = partial + s * plane + i;
            if (vec) {
                const float4 v = *reinterpret_cast<const float4*>(src);
                f[0] += v.x; f[1] += v.y; f[2] += v.z; f[3] += v.w;
            } else {
                for (int j = 0; j < n; ++j) f[j] += src[j];
            }
        }
        for (int j = 0; j < n; ++j) {
            float v = alpha * f[j];
            if (beta != 0.0f) v += beta * __uint_as_float(static_cast<uint32_t>(d[i + j]) << 16);
            if (bias != nullptr) v += __uint_as_float(static_cast<uint32_t>(bias[(i + j) % N]) << 16);
            uint32_t o;
            asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(o) : "f"(0.0f), "f"(v));
            d[i + j] = static_cast<uint16_t>(o & 0xFFFFu);
        }
    }
}

// Test aid for the bounded waits: one thread waits, with a caller-chosen cycle limit, on a barrier that nothing
// arrives at.  No copy and no tensor-core operation is in flight, so when the limit runs out the kernel simply
// records kErrSelfTest in the status word and returns, as the GEMM's roles do.
__global__ void mx_wait_selftest_kernel(int* status, long long limit_cycles) {
    __shared__ __align__(8) uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        abort_flag = 0;
        ptx::mbar_init(smem_u32(&bar), 1);
        ptx::fence_barrier_init();
        if (!ptx::mbar_wait<false>(smem_u32(&bar), 0, &abort_flag, limit_cycles) && status != nullptr)
            atomicCAS(status, 0, kErrSelfTest | (static_cast<int>(blockIdx.x) << 8));
    }
}

// ------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {       // a property of the driver, not of a device
        void* f = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(f);
    });
    return fn;
}

// The three kinds of tensor map the GEMM uses.  A map is a pure function of (kind, base, rows, row length, box rows),
// so encoded maps are kept in a small per-thread table and a layer that calls with the same buffers again (cached
// weight operands, a captured graph's fixed buffers, the bench loop) pays for no encode.
enum MapKind : int { kMapOperand = 0, kMapScales = 1, kMapOutput = 2 };
struct MapKey {
    const void* base; int64_t rows, inner; int box_rows, kind;
    bool operator==(const MapKey& o) const {
        return base == o.base && rows == o.rows && inner == o.inner && box_rows == o.box_rows && kind == o.kind;
    }
};

static bool encode_map(CUtensorMap* m, const MapKey& k) {
    const cuuint32_t estr[2] = {1u, 1u};
    void* base = const_cast<void*>(k.base);
    if (k.kind == kMapOperand) {
        // uint8 [rows, inner] row-major, box = box_rows x 128 bytes, 128-byte swizzle, zero fill out of bounds
        const cuuint64_t dims[2] = {static_cast<cuuint64_t>(k.inner), static_cast<cuuint64_t>(k.rows)};
        const cuuint64_t strides[1] = {static_cast<cuuint64_t>(k.inner)};
        const cuuint32_t box[2] = {128u, static_cast<cuuint32_t>(k.box_rows)};
        return encode_fn()(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                           CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
    }
    if (k.kind == kMapScales) {
        // tiled scale buffer seen as uint32 [tiles, 128]; one box = one 512-byte tile
        const cuuint64_t dims[2] = {128u, static_cast<cuuint64_t>(k.rows)};
        const cuuint64_t strides[1] = {512u};
        const cuuint32_t box[2] = {128u, 1u};
        return encode_fn()(m, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                           CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
    }
    // bf16 D [rows, inner] row-major for the epilogue's stores: box = 32 rows x 32 columns (64 bytes), 64-byte swizzle
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(k.inner), static_cast<cuuint64_t>(k.rows)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(k.inner) * 2u};
    const cuuint32_t box[2] = {32u, 32u};
    return encode_fn()(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                       CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                       CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

static std::atomic<long long> g_map_encodes{0};     // encodes actually performed (dw_mxfp8_debug_counter(0))

static bool get_map(CUtensorMap* out, const void* base, int64_t rows, int64_t inner, int box_rows, int kind) {
    constexpr int kSlots = 64;
    struct Slot { MapKey key; CUtensorMap map; bool valid; };
    static thread_local Slot table[kSlots] = {};
    const MapKey key = {base, rows, inner, box_rows, kind};
    uint64_t h = reinterpret_cast<uintptr_t>(base) >> 4;
    h ^= static_cast<uint64_t>(rows) * 0x9E3779B97F4A7C15ull + static_cast<uint64_t>(inner) * 0xC2B2AE3D27D4EB4Full +
         static_cast<uint64_t>(box_rows * 4 + kind);
    Slot& s = table[(h ^ (h >> 29)) % kSlots];
    if (!(s.valid && s.key == key)) {
        if (!encode_map(&s.map, key)) { s.valid = false; return false; }
        s.key = key; s.valid = true;
        g_map_encodes.fetch_add(1, std::memory_order_relaxed);
    }
    *out = s.map;
    return true;
}

// What a caller may fix about a launch; everything 0 = decided per problem by plan_gemm.
//   bits [0,8)   kernel variant: 1: 1 CTA, BN 128; 2: 1 CTA, BN 256; 3: CTA pair (256-row tile), BN 256;
//                4: CTA pair, BN 128; 5: CTA pair, BN 192 (two whole accumulators in tensor memory, unlike 3)
//   bits [8,16)  row tiles per raster band        bits [16,24)  split-K count
//   bit 24       D written with per-thread stores instead of TMA stores
struct PlanWord {
    int variant, group_m, splits; bool direct_stores;
    static bool valid(int w) { return w >= 0 && (w & 0xFF) <= 5 && (w >> 25) == 0; }
    explicit PlanWord(int w) : variant(w & 0xFF), group_m((w >> 8) & 0xFF), splits((w >> 16) & 0xFF), direct_stores((w >> 24) & 1) {}
};
static std::atomic<int> g_default_plan{0};          // dw_mxfp8_gemm_set_variant: the plan word of calls that pass none
static std::atomic<long long*> g_timing{nullptr};   // optional per-CTA wait counters (dw_mxfp8_gemm_set_timing_buffer)

template <int BN, int kCtas, int kGroup>
static int launch_gemm(const void* a, const void* a_sf, const void* b, const void* b_sf, GemmParams p, const PlanWord& pw,
                       const DeviceInfo& di, cudaStream_t st) {
    using Cfg = GemmCfg<BN, kCtas, kGroup>;
    CUtensorMap tm_a, tm_b, tm_sfa, tm_sfb, tm_d;
    const int64_t kt = (p.K / 32 + 3) / 4;
    const int64_t b_rows = p.tile_group != nullptr ? p.N * p.num_groups : p.N;
    if (!get_map(&tm_a, a, p.M, p.K, 128, kMapOperand) || !get_map(&tm_b, b, b_rows, p.K, Cfg::kBRows, kMapOperand) ||
        !get_map(&tm_sfa, a_sf, ((p.M + 127) / 128) * kt, 128, 1, kMapScales) ||
        !get_map(&tm_sfb, b_sf, ((b_rows + 127) / 128) * kt, 128, 1, kMapScales))
        return DW_ERR_LAUNCH;
    // D goes out by TMA when its rows are 16-byte multiples (the tensor map's stride rule) and it is
    // written by the GEMM kernel itself (not by the split-K reduction)
    p.tma_store = (p.d != nullptr && p.splits <= 1 && p.N % 8 == 0 && p.out_n % 8 == 0 && !pw.direct_stores) ? 1 : 0;
    if (p.tma_store) {
        if (!get_map(&tm_d, p.d, p.M, p.out_n, 32, kMapOutput)) return DW_ERR_LAUNCH;
    } else {
        tm_d = tm_a;                                        // unused by the kernel
    }
    p.tiles_m = static_cast<uint32_t>((p.M + 128 * kCtas - 1) / (128 * kCtas));
    p.tiles_n = static_cast<uint32_t>((p.N + BN - 1) / BN);
    p.num_tiles = p.tiles_m * p.tiles_n;
    p.num_kblocks = static_cast<uint32_t>((p.K + 127) / 128);
    // Band height (row tiles per raster band).  Inside a band the A tiles are reused by every wave of
    // CTAs while B streams through once, so DRAM reads are about A + (bands x B): when B is small it
    // stays in L2 anyway and a low band is fine; otherwise the band is made as tall as an A band of
    // ~32 MB allows (measured: L2 keeps roughly that much beside the streaming operand and D).
    {
        const int64_t tile_bytes = static_cast<int64_t>(128 * kCtas) * p.K, b_bytes = p.N * p.K;
        int64_t g = 16 / kCtas;
        if (b_bytes > (32ll << 20)) g = std::max<int64_t>(16 / kCtas, std::min<int64_t>((32ll << 20) / tile_bytes, 64 / kCtas));
        p.group_m = static_cast<uint32_t>(pw.group_m > 0 ? pw.group_m : g);
    }

    // the opt-in to more than 48 KB of dynamic shared memory is a per-device attribute of the kernel
    {
        static std::mutex mu;
        static bool done[kMaxDevices] = {};
        std::lock_guard<std::mutex> lock(mu);
        if (!done[di.device]) {
            if (cudaFuncSetAttribute(mx_gemm_kernel<BN, kCtas, kGroup>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     Cfg::kSmemBytes) != cudaSuccess) {
                cudaGetLastError();
                return DW_ERR_LAUNCH;
            }
            done[di.device] = true;
        }
    }

    // Measured in cycles per tile on B200 (6 stages): with 32 k-blocks per tile the ring that runs on across tiles is 2.3 %
    // faster than restarting every tile at stage 0 (which leaves stages idle at each tile boundary), with 8 k-blocks it
    // is 4-8 % slower and with 112 0.5 % slower.
    p.ring_continues = (p.num_kblocks % Cfg::kStages != 0 && p.num_kblocks >= 16 && p.num_kblocks <= 64) ? 1 : 0;
    p.kb_per_split = (p.num_kblocks + p.splits - 1) / p.splits;
    p.splits = (p.num_kblocks + p.kb_per_split - 1) / p.kb_per_split;      // every split owns at least one k-block
    // Work units are dealt round-robin to the workers (CTAs or CTA pairs), so the kernel lasts ceil(units / workers) units
    // whatever the remainder: the smallest worker count with that many rounds finishes at the same time and leaves the
    // other SMs to kernels of other streams (nothing is scheduled next to a GEMM CTA on its own SM).
    const int64_t units = static_cast<int64_t>(p.num_tiles) * p.splits, max_workers = di.sms / kCtas;
    const int64_t rounds = (units + max_workers - 1) / max_workers;
    const int workers = static_cast<int>(std::min<int64_t>((units + rounds - 1) / rounds, max_workers));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(workers * kCtas));
    cfg.blockDim = dim3(kGemmThreads);
    cfg.dynamicSmemBytes = Cfg::kSmemBytes;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = kCtas; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;      // see pdl_wait() in the kernel
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    if (cudaLaunchKernelEx(&cfg, mx_gemm_kernel<BN, kCtas, kGroup>, tm_a, tm_b, tm_sfa, tm_sfb, tm_d, p) != cudaSuccess) {
        cudaGetLastError();
        return DW_ERR_LAUNCH;
    }
    if (p.splits > 1) {
        const int64_t quads = (p.M * p.N + 3) / 4;
        const int grid = static_cast<int>(std::min<int64_t>((quads + 255) / 256, static_cast<int64_t>(di.sms) * 8));
        if (launch_pdl(mx_splitk_reduce_kernel, dim3(grid), dim3(256), 0, st, static_cast<const float*>(p.partial), p.d, p.bias,
                       p.M, p.N, p.splits, p.alpha, p.beta) != cudaSuccess) {
            cudaGetLastError();
            return DW_ERR_LAUNCH;
        }
    }
    return DW_OK;
}

// Kernel variant and split count for a problem.  Split-K is chosen when the output has too few
// tiles to occupy the GPU and K is long (weight-gradient GEMMs: small N x K output, contraction over
// all tokens).
struct GemmPlan { int variant; uint32_t splits; size_t ws_bytes; };

static GemmPlan plan_gemm(int64_t M, int64_t N, int64_t K, const PlanWord& pw, int sms) {
    GemmPlan pl;
    const int64_t nkb = (K + 127) / 128;
    pl.variant = pw.variant != 0 ? pw.variant : ((N <= 128) ? 1 : (M <= 128 ? 2 : 3));
    if (pw.variant == 0 && pl.variant == 3) {
        // 256 x 256 tiles on CTA pairs (3), 256 x 192 tiles on CTA pairs (5) or 128 x 256 tiles on single CTAs (2).
        // Cost of the slowest worker in units of (256 columns x one k-block) of one SM's tensor time:
        // rounds of tiles x (k-blocks x efficiency + per-tile overhead), fitted to measurements on B200.  Variant 3's
        // two accumulators share 32 tensor-memory columns, so each tile waits for the previous tile's first epilogue
        // step (about 2 k-blocks); variant 5 has whole accumulators but more tiles and 17 % more operand bytes per
        // flop; variant 2 has a shallower ring.  In practice 3 wins unless the tile count quantises badly on the
        // 74 CTA pairs (8192 x 768 x 3072: 96 tiles of 256 x 256 = 2 rounds at 65 %; 128 tiles of 256 x 192 = 2
        // rounds at 86 %: 20.7 us against 24.5).
        // Problems small enough for split-K keep variant 3, which the split heuristic below was measured with.
        const int64_t pairs = sms / 2, tm = (M + 255) / 256;
        const bool would_split = tm * ((N + 255) / 256) * 4 <= pairs && nkb >= 32;
        auto rounds = [](int64_t tiles, int64_t workers) { return static_cast<double>((tiles + workers - 1) / workers); };
        const double cost3 = rounds(tm * ((N + 255) / 256), pairs) * (nkb + 2.0);
        const double cost5 = rounds(tm * ((N + 191) / 192), pairs) * 0.75 * (nkb + 3.0) * 1.05;
        const double cost2 = rounds(((M + 127) / 128) * ((N + 255) / 256), sms) * (nkb * 1.05 + 2.7);
        if (!would_split) {
            if (cost5 < cost3 && cost5 <= cost2) pl.variant = 5;
            else if (cost2 < cost3) pl.variant = 2;
        }
    }
    const int ctas = (pl.variant >= 3) ? 2 : 1, bn = (pl.variant == 1 || pl.variant == 4) ? 128 : (pl.variant == 5 ? 192 : 256);
    const int64_t tiles = ((M + 128 * ctas - 1) / (128 * ctas)) * ((N + bn - 1) / bn);
    const int64_t workers = sms / ctas;
    int64_t splits = 1;
    if (pw.splits > 0) splits = std::min<int64_t>(pw.splits, nkb);
    // measured on B200: worth it only below a quarter of the GPU (the reduction pass costs ~10 us)
    else if (tiles * 4 <= workers && nkb >= 32) splits = std::max<int64_t>(1, std::min<int64_t>({workers / tiles, nkb / 16, 4}));
    pl.splits = static_cast<uint32_t>(splits);
    pl.ws_bytes = splits > 1 ? static_cast<size_t>(splits) * M * N * sizeof(float) : 0;
    return pl;
}

struct FusedOut {
    int act = DW_ACT_NONE; int rule = DW_RULE_OCP_FLOOR; void* codes = nullptr; void* scales = nullptr;
    const int* tile_group = nullptr; uint32_t num_groups = 0;
};

static int run_gemm(const void* a_codes, const void* a_sf, const void* b_codes, const void* b_sf, void* d_bf16,
                    const void* bias_bf16, int64_t M, int64_t N, int64_t K, float alpha, float beta, int variant,
                    uint32_t splits, float* partial, void* status_word, const PlanWord& pw, const DeviceInfo& di, cudaStream_t st,
                    const FusedOut& fo = FusedOut()) {
    GemmParams p = {};
    p.act = fo.act; p.q_rule = fo.rule;
    p.q_codes = static_cast<uint8_t*>(fo.codes); p.q_scales = static_cast<uint8_t*>(fo.scales);
    p.out_n = fo.act == DW_ACT_SWIGLU ? N / 2 : N;
    p.q_kt = (p.out_n / 32 + 3) / 4;
    p.d = static_cast<uint16_t*>(d_bf16);
    p.bias = static_cast<const uint16_t*>(bias_bf16);
    p.status = static_cast<int*>(status_word);
    p.M = M; p.N = N; p.K = K; p.alpha = alpha; p.beta = beta;
    p.splits = splits; p.partial = partial;
    p.wait_cycles = g_timing.load(std::memory_order_relaxed);
    p.tile_group = fo.tile_group; p.num_groups = fo.num_groups;
    switch (variant) {
        case 1: return launch_gemm<128, 1, 1>(a_codes, a_sf, b_codes, b_sf, p, pw, di, st);
        case 2: return launch_gemm<256, 1, 1>(a_codes, a_sf, b_codes, b_sf, p, pw, di, st);
        case 3: return launch_gemm<256, 2, 1>(a_codes, a_sf, b_codes, b_sf, p, pw, di, st);
        case 4: return launch_gemm<128, 2, 1>(a_codes, a_sf, b_codes, b_sf, p, pw, di, st);
        default: return launch_gemm<192, 2, 1>(a_codes, a_sf, b_codes, b_sf, p, pw, di, st);
    }
}

// Argument checks that need no device, then the device: DW_ERR_ARCH unless the current device is compute capability 10.x.
static int check_gemm_args(const void* a_codes, const void* a_sf, const void* b_codes, const void* b_sf, const void* d_bf16,
                           const void* bias_bf16, int64_t M, int64_t N, int64_t K, DeviceInfo* di, bool d_optional = false) {
    if (!a_codes || !a_sf || !b_codes || !b_sf || (!d_bf16 && !d_optional)) return DW_ERR_BAD_ARG;
    if (K == 0 || K % 32 != 0) return DW_ERR_BAD_ARG;
    auto al16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
    if (!al16(a_codes) || !al16(b_codes) || !al16(a_sf) || !al16(b_sf) || !al16(d_bf16)) return DW_ERR_BAD_ARG;
    if (bias_bf16 && !al16(bias_bf16)) return DW_ERR_BAD_ARG;
    if (M >= (1ll << 31) || N >= (1ll << 31) || K >= (1ll << 31)) return DW_ERR_TOO_LARGE;
    const int rc = current_device(di);
    if (rc != DW_OK) return rc;
    if (encode_fn() == nullptr) return DW_ERR_LAUNCH;
    return DW_OK;
}

}  // namespace dw

using namespace dw;

extern "C" DW_API int dw_mxfp8_gemm_set_variant(int variant) {
    if (!PlanWord::valid(variant)) return DW_ERR_BAD_ARG;
    g_default_plan.store(variant, std::memory_order_relaxed);
    return DW_OK;
}

extern "C" DW_API int dw_mxfp8_gemm_set_timing_buffer(void* device_buffer, size_t bytes) {
    if (device_buffer != nullptr && (bytes < DW_GEMM_TIMING_BYTES || (reinterpret_cast<uintptr_t>(device_buffer) & 7) != 0))
        return DW_ERR_BAD_ARG;
    g_timing.store(static_cast<long long*>(device_buffer), std::memory_order_relaxed);
    return DW_OK;
}

// SM count for planning when no device can be asked (a build machine sizing buffers): B200's
static int planning_sms() {
    DeviceInfo di;
    const int rc = current_device(&di);
    return (rc == DW_OK || rc == DW_ERR_ARCH) && di.sms > 0 ? di.sms : 148;
}

extern "C" DW_API size_t dw_mxfp8_gemm_workspace_planned(int64_t M, int64_t N, int64_t K, int plan) {
    if (M <= 0 || N <= 0 || K <= 0 || !PlanWord::valid(plan)) return 0;
    return plan_gemm(M, N, K, PlanWord(plan), planning_sms()).ws_bytes;
}

extern "C" DW_API size_t dw_mxfp8_gemm_workspace(int64_t M, int64_t N, int64_t K) {
    return dw_mxfp8_gemm_workspace_planned(M, N, K, g_default_plan.load(std::memory_order_relaxed));
}

extern "C" DW_API int dw_mxfp8_gemm_planned(const void* a_codes, const void* a_sf, const void* b_codes, const void* b_sf,
                                            void* d_bf16, const void* bias_bf16, int64_t M, int64_t N, int64_t K, float alpha,
                                            float beta, void* workspace, size_t workspace_bytes, int plan, void* status_word,
                                            void* stream) {
    if (M < 0 || N < 0 || K < 0 || !PlanWord::valid(plan)) return DW_ERR_BAD_ARG;
    if (M == 0 || N == 0) return DW_OK;
    DeviceInfo di;
    const int rc = check_gemm_args(a_codes, a_sf, b_codes, b_sf, d_bf16, bias_bf16, M, N, K, &di);
    if (rc != DW_OK) return rc;
    const PlanWord pw(plan);
    GemmPlan pl = plan_gemm(M, N, K, pw, di.sms);
    // without a large enough, 16-byte aligned workspace the GEMM runs unsplit
    if (pl.splits > 1 && (workspace == nullptr || workspace_bytes < pl.ws_bytes ||
                          (reinterpret_cast<uintptr_t>(workspace) & 15) != 0))
        pl.splits = 1;
    return run_gemm(a_codes, a_sf, b_codes, b_sf, d_bf16, bias_bf16, M, N, K, alpha, beta, pl.variant, pl.splits,
                    static_cast<float*>(workspace), status_word, pw, di, static_cast<cudaStream_t>(stream));
}

extern "C" DW_API int dw_mxfp8_gemm(const void* a_codes, const void* a_sf, const void* b_codes, const void* b_sf, void* d_bf16,
                             const void* bias_bf16, int64_t M, int64_t N, int64_t K, float alpha, float beta, void* workspace,
                             size_t workspace_bytes, void* status_word, void* stream) {
    return dw_mxfp8_gemm_planned(a_codes, a_sf, b_codes, b_sf, d_bf16, bias_bf16, M, N, K, alpha, beta, workspace,
                                 workspace_bytes, g_default_plan.load(std::memory_order_relaxed), status_word, stream);
}

extern "C" DW_API int dw_mxfp8_gemm_fused(const void* a_codes, const void* a_sf, const void* b_codes, const void* b_sf,
                                          void* d_bf16, const void* bias_bf16, int64_t M, int64_t N, int64_t K, float alpha,
                                          float beta, int activation, void* out_codes, void* out_scales, int scale_rule,
                                          void* status_word, void* stream) {
    if (M < 0 || N < 0 || K < 0) return DW_ERR_BAD_ARG;
    if (activation < DW_ACT_NONE || activation > DW_ACT_SWIGLU) return DW_ERR_BAD_ARG;
    // gate/up pairs: whole groups of 64 fused columns, and no accumulation into a previous D
    if (activation == DW_ACT_SWIGLU && (N % 64 != 0 || beta != 0.0f)) return DW_ERR_BAD_ARG;
    if (scale_rule != DW_RULE_OCP_FLOOR && scale_rule != DW_RULE_REF_CEIL) return DW_ERR_BAD_ARG;
    if ((out_codes == nullptr) != (out_scales == nullptr)) return DW_ERR_BAD_ARG;
    if (d_bf16 == nullptr && out_codes == nullptr) return DW_ERR_BAD_ARG;          // nothing to write
    if (d_bf16 == nullptr && beta != 0.0f) return DW_ERR_BAD_ARG;                  // beta reads D
    if (M == 0 || N == 0) return DW_OK;
    if (out_codes != nullptr && (N % 32 != 0 || (reinterpret_cast<uintptr_t>(out_codes) & 15) != 0)) return DW_ERR_BAD_ARG;
    if (out_codes == nullptr && N % 8 != 0 && activation != DW_ACT_NONE && d_bf16 == nullptr) return DW_ERR_BAD_ARG;
    DeviceInfo di;
    const int rc = check_gemm_args(a_codes, a_sf, b_codes, b_sf, d_bf16, bias_bf16, M, N, K, &di, true);
    if (rc != DW_OK) return rc;
    FusedOut fo;
    fo.act = activation; fo.rule = scale_rule; fo.codes = out_codes; fo.scales = out_scales;
    const PlanWord pw(g_default_plan.load(std::memory_order_relaxed));
    GemmPlan pl = plan_gemm(M, N, K, pw, di.sms);
    // the scale padding of the quantised output is written per 128-column group: keep column tiles that are multiples of 128
    if (out_codes != nullptr && pl.variant > 4) pl.variant = 3;
    // gate/up pairs must fall into one epilogue warp's half of a column tile: 128- or 256-wide tiles, and 256-wide ones
    // when the quantised output's scale tiles (128 output columns) are padded by the tile that owns them
    if (activation == DW_ACT_SWIGLU && (pl.variant == 5 || pl.variant == 1 || pl.variant == 4)) pl.variant = M <= 128 ? 2 : 3;
    return run_gemm(a_codes, a_sf, b_codes, b_sf, d_bf16, bias_bf16, M, N, K, alpha, beta, pl.variant, 1, nullptr, status_word,
                    pw, di, static_cast<cudaStream_t>(stream), fo);
}

extern "C" DW_API int dw_mxfp8_gemm_grouped(const void* a_codes, const void* a_sf, const void* b_codes, const void* b_sf,
                                            void* d_bf16, const int* tile_group, int64_t M_total, int64_t N, int64_t K,
                                            int num_groups, int rows_per_tile, float alpha, void* status_word, void* stream) {
    if (M_total < 0 || N <= 0 || K <= 0 || num_groups <= 0 || tile_group == nullptr) return DW_ERR_BAD_ARG;
    if (rows_per_tile != 128 && rows_per_tile != 256) return DW_ERR_BAD_ARG;
    if (M_total % rows_per_tile != 0 || N % 128 != 0) return DW_ERR_BAD_ARG;   // whole row tiles per group; whole scale tiles per weight
    if (M_total == 0) return DW_OK;
    if (static_cast<int64_t>(num_groups) * N >= (1ll << 31)) return DW_ERR_TOO_LARGE;
    DeviceInfo di;
    const int rc = check_gemm_args(a_codes, a_sf, b_codes, b_sf, d_bf16, nullptr, M_total, N, K, &di);
    if (rc != DW_OK) return rc;
    FusedOut fo;
    fo.tile_group = tile_group; fo.num_groups = static_cast<uint32_t>(num_groups);
    // the row tile of the kernel must be the granularity of tile_group: 1 CTA x 128 rows or a CTA pair x 256 rows
    const int variant = rows_per_tile == 128 ? 2 : 3;
    const PlanWord pw(g_default_plan.load(std::memory_order_relaxed) & (1 << 24));     // the store mode only
    return run_gemm(a_codes, a_sf, b_codes, b_sf, d_bf16, nullptr, M_total, N, K, alpha, 0.0f, variant, 1, nullptr, status_word,
                    pw, di, static_cast<cudaStream_t>(stream), fo);
}

// ------------------------------------------------------------------------------------------
// Split-K GEMM for callers that cannot allocate: the fp32 partial sums live in a fixed array that
// is part of the library image on every device that loads it (DW_GEMM_STATIC_SCRATCH_BYTES each).
// ------------------------------------------------------------------------------------------
namespace dw {
constexpr size_t kStaticScratchFloats = DW_GEMM_STATIC_SCRATCH_BYTES / sizeof(float);
static __device__ __align__(256) float g_splitk_scratch[kStaticScratchFloats];

// In host code `g_splitk_scratch` is only a handle for the runtime, not an address a kernel can use.
// The device address is looked up once per device, with that device current.
static int static_scratch_address(float** out) {
    static std::mutex mu;
    static float* cached[kMaxDevices] = {};
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return DW_ERR_LAUNCH;
    std::lock_guard<std::mutex> lock(mu);
    if (cached[dev] == nullptr) {
        void* ptr = nullptr;
        if (cudaGetSymbolAddress(&ptr, g_splitk_scratch) != cudaSuccess || ptr == nullptr) {
            cudaGetLastError();
            return DW_ERR_LAUNCH;
        }
        cached[dev] = static_cast<float*>(ptr);
    }
    *out = cached[dev];
    return DW_OK;
}
}  // namespace dw

extern "C" DW_API int dw_mxfp8_gemm_splitk_static(const void* a_codes, const void* a_sf, const void* b_codes, const void* b_sf,
                                                  void* d_bf16, const void* bias_bf16, int64_t M, int64_t N, int64_t K,
                                                  float alpha, float beta, int splits, void* status_word, void* stream) {
    if (M < 0 || N < 0 || K < 0 || splits < 2 || splits > 255) return DW_ERR_BAD_ARG;
    if (M == 0 || N == 0) return DW_OK;
    const int64_t nkb = (K + 127) / 128;
    const int64_t eff = std::min<int64_t>(splits, nkb);                        // the kernel never uses more
    if (K > 0 && static_cast<uint64_t>(eff) * static_cast<uint64_t>(M) * static_cast<uint64_t>(N) > kStaticScratchFloats)
        return DW_ERR_TOO_LARGE;
    DeviceInfo di;
    const int rc = check_gemm_args(a_codes, a_sf, b_codes, b_sf, d_bf16, bias_bf16, M, N, K, &di);
    if (rc != DW_OK) return rc;
    float* scratch = nullptr;
    const int arc = static_scratch_address(&scratch);
    if (arc != DW_OK) return arc;
    const PlanWord pw(g_default_plan.load(std::memory_order_relaxed) & 0xFF);        // the variant only
    const int variant = plan_gemm(M, N, K, pw, di.sms).variant;
    return run_gemm(a_codes, a_sf, b_codes, b_sf, d_bf16, bias_bf16, M, N, K, alpha, beta, variant,
                    static_cast<uint32_t>(eff), scratch, status_word, pw, di, static_cast<cudaStream_t>(stream));
}

extern "C" DW_API int dw_mxfp8_check_status(const void* status_word, void* stream) {
    if (!status_word) return DW_ERR_BAD_ARG;
    int host = 0;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (cudaMemcpyAsync(&host, status_word, sizeof(int), cudaMemcpyDeviceToHost, st) != cudaSuccess) return DW_ERR_LAUNCH;
    if (cudaStreamSynchronize(st) != cudaSuccess) return DW_ERR_LAUNCH;
    return host == 0 ? DW_OK : DW_ERR_DEVICE_STATUS;
}

extern "C" DW_API int dw_mxfp8_selftest_bounded_wait(long long limit_cycles, void* status_word, void* stream) {
    if (status_word == nullptr || limit_cycles < 0) return DW_ERR_BAD_ARG;
    if (limit_cycles > DW_SELFTEST_MAX_WAIT_CYCLES) return DW_ERR_TOO_LARGE;       // a test never keeps an SM longer than ~1 ms
    DeviceInfo di;
    const int rc = current_device(&di);
    if (rc != DW_OK) return rc;
    mx_wait_selftest_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<int*>(status_word), limit_cycles);
    return cudaGetLastError() == cudaSuccess ? DW_OK : DW_ERR_LAUNCH;
}

extern "C" DW_API long long dw_mxfp8_debug_counter(int which) {
    return which == 0 ? g_map_encodes.load(std::memory_order_relaxed) : -1;
}
