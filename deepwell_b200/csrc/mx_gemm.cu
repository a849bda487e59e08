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
//   warps 2-5   epilogue: tcgen05.ld the fp32 accumulator, alpha/beta/bias, bf16, global stores
//
// kCtas == 2 pairs two CTAs (a cluster of 2 along M) on one 256 x BN tile with cta_group::2: each
// CTA stages its own half of A and its own half of B; the leader CTA issues the MMAs for both.
// No load is multicast; every CTA fetches what it needs with its own TMA loads.
//
// Every wait is bounded: on expiry the CTA raises an abort flag, records a code in the status word
// and unwinds through the common exit (TMEM is always freed).

#include <algorithm>
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
    uint32_t tiles_m, tiles_n, num_tiles, num_kblocks;
};

template <int BN, int kCtas>
struct GemmCfg {
    static constexpr int kBM = 128;                       // rows per CTA
    static constexpr int kBK = 128;                       // bytes (= elements) of K per stage
    static constexpr int kABytes = kBM * kBK;
    static constexpr int kBRows = BN / kCtas;             // B rows staged by one CTA
    static constexpr int kBBytes = kBRows * kBK;
    static constexpr int kSfaBytes = 512;
    static constexpr int kSfbTiles = BN / 128;
    static constexpr int kSfbBytes = kSfbTiles * 512;
    static constexpr int kStageBytes = (kABytes + kBBytes + kSfaBytes + kSfbBytes + 1023) / 1024 * 1024;
    static constexpr int kStages = (200 * 1024 / kStageBytes) > 8 ? 8 : (200 * 1024 / kStageBytes);
    static constexpr int kAccStages = (BN == 256) ? 1 : 2;
    static constexpr int kSfaCol = kAccStages * BN;       // TMEM column of the A scales
    static constexpr int kSfbCol = kSfaCol + 4;
    static constexpr int kTmemCols = 512;
    static constexpr int kBarrierBytes = 256;
    static constexpr int kSmemBytes = kStages * kStageBytes + kBarrierBytes + 1024;  // + alignment slack
    static constexpr uint32_t kTxBytes = kCtas * (kABytes + kBBytes + kSfaBytes + kSfbBytes);
    static_assert(kSfbCol + 4 * kSfbTiles <= kTmemCols, "TMEM columns");
    static_assert(kStages >= 2, "pipeline depth");
};

enum : int { kErrProducer = 1, kErrMmaFull = 2, kErrMmaAcc = 3, kErrEpilogue = 4 };

template <int BN, int kCtas>
__global__ void __launch_bounds__(192, 1)
mx_gemm_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
               const __grid_constant__ CUtensorMap tm_sfa, const __grid_constant__ CUtensorMap tm_sfb,
               const GemmParams p) {
    using Cfg = GemmCfg<BN, kCtas>;
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
    const uint32_t bar_base = smem_base + kStages * Cfg::kStageBytes;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (kStages + s); };
    auto accf_bar = [&](int a) { return bar_base + 8u * (2 * kStages + a); };
    auto acce_bar = [&](int a) { return bar_base + 8u * (2 * kStages + kAcc + a); };
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem_gen + kStages * Cfg::kStageBytes + 8 * (2 * kStages + 2 * kAcc));
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) { ptx::mbar_init(full_bar(s), 1); ptx::mbar_init(empty_bar(s), 1); }
        for (int a = 0; a < kAcc; ++a) { ptx::mbar_init(accf_bar(a), 1); ptx::mbar_init(acce_bar(a), 4 * kCtas); }
        *abort_flag = 0;
        ptx::fence_barrier_init();
        ptx::prefetch_tmap(&tm_a); ptx::prefetch_tmap(&tm_b); ptx::prefetch_tmap(&tm_sfa); ptx::prefetch_tmap(&tm_sfb);
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

    const uint32_t num_workers = gridDim.x / kCtas, worker = blockIdx.x / kCtas;
    int err = 0;

    if (warp == 0) {
        // ================= TMA producer =================
        if (lane == 0) {
            uint32_t stage = 0, phase = 0;
            // loads of both CTAs of a pair complete on the leader's barrier
            for (uint32_t tile = worker; tile < p.num_tiles && !err; tile += num_workers) {
                const uint32_t tm = tile % p.tiles_m, tn = tile / p.tiles_m;
                const int row_a = static_cast<int>(tm * (128 * kCtas) + rank * 128);
                const int row_b = static_cast<int>(tn * BN + rank * Cfg::kBRows);
                const int sfa_tile = static_cast<int>(tm * kCtas + rank);
                const int sfb_tile = static_cast<int>(tn * Cfg::kSfbTiles);
                for (uint32_t kb = 0; kb < p.num_kblocks; ++kb) {
                    if (!ptx::mbar_wait<kCtas == 2>(empty_bar(stage), phase ^ 1u, abort_flag)) { err = kErrProducer; break; }
                    const uint32_t bar = (kCtas == 2) ? ptx::map_to_cta(full_bar(stage), 0) : full_bar(stage);
                    if (leader) ptx::mbar_arrive_expect_tx(full_bar(stage), Cfg::kTxBytes);
                    const int k0 = static_cast<int>(kb * Cfg::kBK);
                    if (kCtas == 2) {
                        ptx::tma_load_2d_pair(stage_a(stage), &tm_a, bar, k0, row_a);
                        ptx::tma_load_2d_pair(stage_b(stage), &tm_b, bar, k0, row_b);
                        ptx::tma_load_2d_pair(stage_sfa(stage), &tm_sfa, bar, 0, sfa_tile * static_cast<int>(p.num_kblocks) + static_cast<int>(kb));
                        for (int j = 0; j < Cfg::kSfbTiles; ++j)
                            ptx::tma_load_2d_pair(stage_sfb(stage) + 512 * j, &tm_sfb, bar, 0,
                                                  (sfb_tile + j) * static_cast<int>(p.num_kblocks) + static_cast<int>(kb));
                    } else {
                        ptx::tma_load_2d(stage_a(stage), &tm_a, bar, k0, row_a);
                        ptx::tma_load_2d(stage_b(stage), &tm_b, bar, k0, row_b);
                        ptx::tma_load_2d(stage_sfa(stage), &tm_sfa, bar, 0, sfa_tile * static_cast<int>(p.num_kblocks) + static_cast<int>(kb));
                        for (int j = 0; j < Cfg::kSfbTiles; ++j)
                            ptx::tma_load_2d(stage_sfb(stage) + 512 * j, &tm_sfb, bar, 0,
                                             (sfb_tile + j) * static_cast<int>(p.num_kblocks) + static_cast<int>(kb));
                    }
                    if (++stage == kStages) { stage = 0; phase ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // ================= MMA issuer (leader CTA only) =================
        if (lane == 0 && leader) {
            uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
            constexpr uint32_t idesc = ptx::idesc_mxf8(128 * kCtas, BN);
            for (uint32_t tile = worker; tile < p.num_tiles && !err; tile += num_workers) {
                if (!ptx::mbar_wait<kCtas == 2>(acce_bar(acc), acc_phase ^ 1u, abort_flag)) { err = kErrMmaAcc; break; }
                ptx::tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * BN;
                for (uint32_t kb = 0; kb < p.num_kblocks; ++kb) {
                    if (!ptx::mbar_wait<kCtas == 2>(full_bar(stage), phase, abort_flag)) { err = kErrMmaFull; break; }
                    ptx::tc_fence_after();
                    ptx::tc_cp_32x128b_warpx4<kCtas>(tmem_base + Cfg::kSfaCol, ptx::smem_desc_sf(stage_sfa(stage)));
#pragma unroll
                    for (int j = 0; j < Cfg::kSfbTiles; ++j)
                        ptx::tc_cp_32x128b_warpx4<kCtas>(tmem_base + Cfg::kSfbCol + 4 * j,
                                                         ptx::smem_desc_sf(stage_sfb(stage) + 512 * j));
                    const uint64_t a_desc = ptx::smem_desc_sw128(stage_a(stage));
                    const uint64_t b_desc = ptx::smem_desc_sw128(stage_b(stage));
#pragma unroll
                    for (uint32_t k = 0; k < 4; ++k) {
                        // advance 32 bytes along K inside the 128-byte swizzle atom: +2 in 16-byte units
                        ptx::tc_mma_mxf8_block_scale<kCtas>(d_tmem, a_desc + 2 * k, b_desc + 2 * k,
                                                            ptx::idesc_with_sf_ids(idesc, k, k),
                                                            tmem_base + Cfg::kSfaCol, tmem_base + Cfg::kSfbCol,
                                                            (kb | k) != 0u);
                    }
                    // stage free again once these MMAs have read it (in both CTAs of a pair)
                    if (kCtas == 2) {
                        ptx::tc_commit_pair(empty_bar(stage));
                        ptx::tc_commit_pair(ptx::map_to_cta(empty_bar(stage), 1));
                    } else {
                        ptx::tc_commit(empty_bar(stage));
                    }
                    if (++stage == kStages) { stage = 0; phase ^= 1u; }
                }
                if (err) break;
                if (kCtas == 2) {
                    ptx::tc_commit_pair(accf_bar(acc));
                    ptx::tc_commit_pair(ptx::map_to_cta(accf_bar(acc), 1));
                } else {
                    ptx::tc_commit(accf_bar(acc));
                }
                if (++acc == kAcc) { acc = 0; acc_phase ^= 1u; }
            }
        }
    } else {
        // ================= epilogue (4 warps = 128 TMEM lanes) =================
        const uint32_t q = warp & 3u;                    // TMEM lane quadrant this warp may read
        uint32_t acc = 0, acc_phase = 0;
        const bool vec_ok = (p.N % 8) == 0;
        for (uint32_t tile = worker; tile < p.num_tiles && !err; tile += num_workers) {
            const uint32_t tm = tile % p.tiles_m, tn = tile / p.tiles_m;
            const int64_t row = static_cast<int64_t>(tm) * (128 * kCtas) + rank * 128 + q * 32 + lane;
            const int64_t col0 = static_cast<int64_t>(tn) * BN;
            if (!ptx::mbar_wait<kCtas == 2>(accf_bar(acc), acc_phase, abort_flag)) { err = kErrEpilogue; break; }
            ptx::tc_fence_after();
            const uint32_t t_row = tmem_base + acc * BN + ((q * 32u) << 16);
#pragma unroll 1
            for (int c = 0; c < BN; c += 32) {
                uint32_t r[32];
                ptx::tc_ld_32x32b_x32(t_row + c, r);
                ptx::tc_wait_ld();
                const int64_t col = col0 + c;
                if (row < p.M && col < p.N) {
                    uint16_t* dst = p.d + row * p.N + col;
                    if (vec_ok && col + 32 <= p.N) {
#pragma unroll
                        for (int v = 0; v < 4; ++v) {
                            float f[8];
#pragma unroll
                            for (int i = 0; i < 8; ++i) f[i] = p.alpha * __uint_as_float(r[8 * v + i]);
                            if (p.beta != 0.0f) {
                                const uint4 o = *reinterpret_cast<const uint4*>(dst + 8 * v);
                                const uint32_t ow[4] = {o.x, o.y, o.z, o.w};
#pragma unroll
                                for (int i = 0; i < 4; ++i) {
                                    f[2 * i] += p.beta * __uint_as_float(ow[i] << 16);
                                    f[2 * i + 1] += p.beta * __uint_as_float(ow[i] & 0xFFFF0000u);
                                }
                            }
                            if (p.bias != nullptr) {
                                const uint4 o = *reinterpret_cast<const uint4*>(p.bias + col + 8 * v);
                                const uint32_t ow[4] = {o.x, o.y, o.z, o.w};
#pragma unroll
                                for (int i = 0; i < 4; ++i) {
                                    f[2 * i] += __uint_as_float(ow[i] << 16);
                                    f[2 * i + 1] += __uint_as_float(ow[i] & 0xFFFF0000u);
                                }
                            }
                            uint32_t o[4];
#pragma unroll
                            for (int i = 0; i < 4; ++i)
                                asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(o[i]) : "f"(f[2 * i + 1]), "f"(f[2 * i]));
                            *reinterpret_cast<uint4*>(dst + 8 * v) = make_uint4(o[0], o[1], o[2], o[3]);
                        }
                    } else {
                        for (int i = 0; i < 32 && col + i < p.N; ++i) {
                            float f = p.alpha * __uint_as_float(r[i]);
                            if (p.beta != 0.0f) f += p.beta * __uint_as_float(static_cast<uint32_t>(dst[i]) << 16);
                            if (p.bias != nullptr) f += __uint_as_float(static_cast<uint32_t>(p.bias[col + i]) << 16);
                            uint32_t o;
                            asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(o) : "f"(0.0f), "f"(f));
                            dst[i] = static_cast<uint16_t>(o & 0xFFFFu);
                        }
                    }
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
    }

    // ================= common exit =================
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

// ------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* f = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(f);
    });
    return fn;
}

// uint8 [rows, k] row-major, box = box_rows x 128 bytes, 128-byte swizzle, zero fill out of bounds
static bool make_operand_map(CUtensorMap* m, const void* base, int64_t rows, int64_t k, int box_rows) {
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(k), static_cast<cuuint64_t>(rows)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(k)};
    const cuuint32_t box[2] = {128u, static_cast<cuuint32_t>(box_rows)};
    const cuuint32_t estr[2] = {1u, 1u};
    return encode_fn()(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                       CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                       CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// tiled scale buffer seen as uint32 [tiles, 128]; one box = one 512-byte tile
static bool make_sf_map(CUtensorMap* m, const void* base, int64_t tiles) {
    const cuuint64_t dims[2] = {128u, static_cast<cuuint64_t>(tiles)};
    const cuuint64_t strides[1] = {512u};
    const cuuint32_t box[2] = {128u, 1u};
    const cuuint32_t estr[2] = {1u, 1u};
    return encode_fn()(m, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void*>(base), dims, strides, box, estr,
                       CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                       CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

static int g_variant = 0;  // 0 auto; 1: 1 CTA BN=128; 2: 1 CTA BN=256; 3: CTA pair BN=256; 4: CTA pair BN=128

static int sm_count() {
    static int sms = 0;
    if (sms == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
    }
    return sms;
}

template <int BN, int kCtas>
static int launch_gemm(const void* a, const void* a_sf, const void* b, const void* b_sf, GemmParams p, cudaStream_t st) {
    using Cfg = GemmCfg<BN, kCtas>;
    CUtensorMap tm_a, tm_b, tm_sfa, tm_sfb;
    const int64_t kt = (p.K / 32 + 3) / 4;
    if (!make_operand_map(&tm_a, a, p.M, p.K, 128) || !make_operand_map(&tm_b, b, p.N, p.K, Cfg::kBRows) ||
        !make_sf_map(&tm_sfa, a_sf, ((p.M + 127) / 128) * kt) || !make_sf_map(&tm_sfb, b_sf, ((p.N + 127) / 128) * kt))
        return DW_ERR_LAUNCH;
    p.tiles_m = static_cast<uint32_t>((p.M + 128 * kCtas - 1) / (128 * kCtas));
    p.tiles_n = static_cast<uint32_t>((p.N + BN - 1) / BN);
    p.num_tiles = p.tiles_m * p.tiles_n;
    p.num_kblocks = static_cast<uint32_t>((p.K + 127) / 128);

    static std::once_flag once;
    static cudaError_t attr_err = cudaSuccess;
    std::call_once(once, [] {
        attr_err = cudaFuncSetAttribute(mx_gemm_kernel<BN, kCtas>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        Cfg::kSmemBytes);
    });
    if (attr_err != cudaSuccess) return DW_ERR_LAUNCH;

    const int workers = std::min<int64_t>(p.num_tiles, sm_count() / kCtas);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(workers * kCtas));
    cfg.blockDim = dim3(192);
    cfg.dynamicSmemBytes = Cfg::kSmemBytes;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = kCtas; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (cudaLaunchKernelEx(&cfg, mx_gemm_kernel<BN, kCtas>, tm_a, tm_b, tm_sfa, tm_sfb, p) != cudaSuccess) {
        cudaGetLastError();
        return DW_ERR_LAUNCH;
    }
    return DW_OK;
}

}  // namespace dw

using namespace dw;

extern "C" DW_API int dw_mxfp8_gemm_set_variant(int variant) {
    if (variant < 0 || variant > 4) return DW_ERR_BAD_ARG;
    g_variant = variant;
    return DW_OK;
}

extern "C" DW_API size_t dw_mxfp8_gemm_workspace(int64_t, int64_t, int64_t) { return 0; }

extern "C" DW_API int dw_mxfp8_gemm(const void* a_codes, const void* a_sf, const void* b_codes, const void* b_sf, void* d_bf16,
                             const void* bias_bf16, int64_t M, int64_t N, int64_t K, float alpha, float beta, void* workspace,
                             size_t workspace_bytes, void* status_word, void* stream) {
    (void)workspace; (void)workspace_bytes;
    if (M < 0 || N < 0 || K < 0) return DW_ERR_BAD_ARG;
    if (M == 0 || N == 0) return DW_OK;
    if (!a_codes || !a_sf || !b_codes || !b_sf || !d_bf16) return DW_ERR_BAD_ARG;
    if (K == 0 || K % 32 != 0) return DW_ERR_BAD_ARG;
    auto al16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
    if (!al16(a_codes) || !al16(b_codes) || !al16(a_sf) || !al16(b_sf) || !al16(d_bf16)) return DW_ERR_BAD_ARG;
    if (bias_bf16 && !al16(bias_bf16)) return DW_ERR_BAD_ARG;
    if (M >= (1ll << 31) || N >= (1ll << 31) || K >= (1ll << 31)) return DW_ERR_TOO_LARGE;
    if (encode_fn() == nullptr) return DW_ERR_LAUNCH;

    GemmParams p = {};
    p.d = static_cast<uint16_t*>(d_bf16);
    p.bias = static_cast<const uint16_t*>(bias_bf16);
    p.status = static_cast<int*>(status_word);
    p.M = M; p.N = N; p.K = K; p.alpha = alpha; p.beta = beta;
    cudaStream_t st = static_cast<cudaStream_t>(stream);

    int v = g_variant;
    if (v == 0) v = (N > 128) ? 2 : 1;
    switch (v) {
        case 1: return launch_gemm<128, 1>(a_codes, a_sf, b_codes, b_sf, p, st);
        case 2: return launch_gemm<256, 1>(a_codes, a_sf, b_codes, b_sf, p, st);
        case 3: return launch_gemm<256, 2>(a_codes, a_sf, b_codes, b_sf, p, st);
        default: return launch_gemm<128, 2>(a_codes, a_sf, b_codes, b_sf, p, st);
    }
}

extern "C" DW_API int dw_mxfp8_check_status(const void* status_word, void* stream) {
    if (!status_word) return DW_ERR_BAD_ARG;
    int host = 0;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (cudaMemcpyAsync(&host, status_word, sizeof(int), cudaMemcpyDeviceToHost, st) != cudaSuccess) return DW_ERR_LAUNCH;
    if (cudaStreamSynchronize(st) != cudaSuccess) return DW_ERR_LAUNCH;
    return host == 0 ? DW_OK : DW_ERR_DEVICE_STATUS;
}
