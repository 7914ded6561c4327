// bf16 GEMM on the 5th-generation tensor cores: TMA-fed, 128B-swizzled shared-memory ring ->
// tcgen05.mma (cta_group::1, 128 x BN x 16) -> fp32 accumulators in tensor memory, double buffered
// -> tcgen05.ld epilogue with fused bias / GELU / GELU-backward.
//
// One persistent CTA per SM, warp-specialised: warp 0 issues TMA loads, warp 1 owns TMEM and issues
// the MMAs, warps 2-5 drain accumulators (each warp reads the 32 TMEM lanes of its quadrant) while
// the MMA warp already works on the next tile in the other accumulator buffer.
//
// Operand layouts (all row-major in global memory):
//   A "K-major":  A[M, K]   (forward activations, output gradients as left operand)
//   A "MN-major": A^T stored as [K, M]   (weight-gradient products: dY^T)
//   B "K-major":  B[N, K]   (weights in the forward product x W^T)
//   B "MN-major": B stored as [K, N]     (weights in the data-gradient product dY W; activations in dW)
// MN-major operands are fed to the tensor core directly through the transposing shared-memory
// descriptor; nothing is transposed in memory.
//
// In the reference every one of these products is a TransformerEngine -> cuBLASLt call
// (teletron/models/dit/dit_attention.py:65-104, dit_layerspec.py:266-298, 438-445).
#include "common.cuh"
#include "sm100.cuh"
#include "teletron_b200.h"

namespace {

using namespace sm100;

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int kThreads = 192;
constexpr int kGroupM = 16;

struct GemmParams {
    int M, N, K;
    __nv_bfloat16* C;
    long ldc;
    const __nv_bfloat16* bias;
    __nv_bfloat16* aux;     // EPI 1/2: pre-activation output; EPI 3/4: pre-activation input
    int* status;
    int tiles_m, tiles_n;
};

template <int BN>
struct Cfg {
    static constexpr int kStages = BN == 256 ? 4 : 6;
    static constexpr int kABytes = BM * BK * 2;
    static constexpr int kBBytes = BN * BK * 2;
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kTmemCols = 2 * BN;
    static constexpr int kSmemBytes = kStages * kStageBytes + 1024 /* alignment slack */ + 256 /* barriers */;
};

template <int EPI>
__device__ __forceinline__ float epi_apply(float acc, float b, float u) {
    if (EPI == 0) return acc + b;
    if (EPI == 1) return tt::gelu_erf(acc + b);
    if (EPI == 2) return tt::gelu_tanh(acc + b);
    if (EPI == 3) return acc * tt::gelu_erf_grad(u);
    return acc * tt::gelu_tanh_grad(u);
}

template <int BN, bool A_MN, bool B_MN, int EPI>
__global__ void __launch_bounds__(kThreads, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const GemmParams p) {
    using C = Cfg<BN>;
    extern __shared__ uint8_t smem_raw[];
    __shared__ volatile int abort_flag;
    __shared__ uint32_t tmem_base_slot;

    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    const uint32_t bar_base = base + C::kStages * C::kStageBytes;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (C::kStages + s); };
    auto tfull_bar = [&](int b) { return bar_base + 8u * (2 * C::kStages + b); };
    auto tempty_bar = [&](int b) { return bar_base + 8u * (2 * C::kStages + 2 + b); };

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int s = 0; s < C::kStages; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(tfull_bar(b), 1);
            mbar_init(tempty_bar(b), 4);
        }
        fence_barrier_init();
        fence_proxy_async();
        tma_prefetch_desc(&tmA);
        tma_prefetch_desc(&tmB);
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(&tmem_base_slot), C::kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_slot;

    const int num_tiles = p.tiles_m * p.tiles_n;
    const int kblocks = (p.K + BK - 1) / BK;
    auto tile_coords = [&](int t, int& m0, int& n0) {
        const int per_group = kGroupM * p.tiles_n;
        const int g = t / per_group;
        const int first_m = g * kGroupM;
        const int gm = min(kGroupM, p.tiles_m - first_m);
        const int r = t - g * per_group;
        m0 = (first_m + r % gm) * BM;
        n0 = (r / gm) * BN;
    };

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            for (int t = blockIdx.x; t < num_tiles; t += gridDim.x) {
                int m0, n0;
                tile_coords(t, m0, n0);
                for (int kb = 0; kb < kblocks; ++kb) {
                    if (!mbar_wait(empty_bar(stage), phase ^ 1u, &abort_flag)) goto done;
                    const uint32_t sa = base + stage * C::kStageBytes;
                    const uint32_t sb = sa + C::kABytes;
                    mbar_arrive_expect_tx(full_bar(stage), C::kStageBytes);
                    const int k0 = kb * BK;
                    if (!A_MN) {
                        tma_load_2d(sa, &tmA, full_bar(stage), k0, m0);
                    } else {
#pragma unroll
                        for (int j = 0; j < BM / 64; ++j) tma_load_2d(sa + j * 8192, &tmA, full_bar(stage), m0 + 64 * j, k0);
                    }
                    if (!B_MN) {
                        tma_load_2d(sb, &tmB, full_bar(stage), k0, n0);
                    } else {
#pragma unroll
                        for (int j = 0; j < BN / 64; ++j) tma_load_2d(sb + j * 8192, &tmB, full_bar(stage), n0 + 64 * j, k0);
                    }
                    if (++stage == C::kStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = idesc_bf16(BM, BN, A_MN, B_MN);
            int stage = 0;
            uint32_t phase = 0;
            int it = 0;
            for (int t = blockIdx.x; t < num_tiles; t += gridDim.x, ++it) {
                const int buf = it & 1;
                const uint32_t acc_phase = (uint32_t)(it >> 1) & 1u;
                if (!mbar_wait(tempty_bar(buf), acc_phase ^ 1u, &abort_flag)) goto done;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(buf * BN);
                for (int kb = 0; kb < kblocks; ++kb) {
                    if (!mbar_wait(full_bar(stage), phase, &abort_flag)) goto done;
                    tc_fence_after();
                    const uint32_t sa = base + stage * C::kStageBytes;
                    const uint32_t sb = sa + C::kABytes;
#pragma unroll
                    for (int kk = 0; kk < BK / 16; ++kk) {
                        const uint64_t da = A_MN ? smem_desc_sw128(sa + kk * 2048, 8192, 1024)
                                                 : smem_desc_sw128(sa + kk * 32, 16, 1024);
                        const uint64_t db = B_MN ? smem_desc_sw128(sb + kk * 2048, 8192, 1024)
                                                 : smem_desc_sw128(sb + kk * 32, 16, 1024);
                        umma_bf16_ss(d_tmem, da, db, idesc, (kb | kk) ? 1u : 0u);
                    }
                    umma_commit(empty_bar(stage));          // frees the smem stage when these MMAs retire
                    if (++stage == C::kStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                umma_commit(tfull_bar(buf));                // accumulator complete
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue (warps 2..5)
        const int quad = warp & 3;
        int it = 0;
        for (int t = blockIdx.x; t < num_tiles; t += gridDim.x, ++it) {
            int m0, n0;
            tile_coords(t, m0, n0);
            const int buf = it & 1;
            const uint32_t acc_phase = (uint32_t)(it >> 1) & 1u;
            if (!mbar_wait(tfull_bar(buf), acc_phase, &abort_flag)) goto done;
            tc_fence_after();
            const int row = m0 + quad * 32 + lane;
            const bool row_ok = row < p.M;
            __nv_bfloat16* crow = p.C + (long)row * p.ldc;
            __nv_bfloat16* arow = (EPI != 0) ? p.aux + (long)row * p.ldc : nullptr;
#pragma unroll 1
            for (int c = 0; c < BN / 32; ++c) {
                uint32_t r[32];
                tmem_ld_32x32(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(buf * BN + c * 32), r);
                tmem_ld_wait();
                const int col0 = n0 + c * 32;
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                    const int col = col0 + g * 8;
                    if (row_ok && col + 8 <= p.N) {
                        float bv[8], uv[8], o[8];
#pragma unroll
                        for (int j = 0; j < 8; ++j) bv[j] = uv[j] = 0.f;
                        if (EPI <= 2 && p.bias != nullptr) tt::unpack8(tt::ld8(p.bias + col), bv);
                        if (EPI >= 3) tt::unpack8(tt::ld8(arow + col), uv);
#pragma unroll
                        for (int j = 0; j < 8; ++j) o[j] = epi_apply<EPI>(__uint_as_float(r[g * 8 + j]), bv[j], uv[j]);
                        if (EPI == 1 || EPI == 2) {
                            float u[8];
#pragma unroll
                            for (int j = 0; j < 8; ++j) u[j] = __uint_as_float(r[g * 8 + j]) + bv[j];
                            tt::st8(arow + col, tt::pack8(u));
                        }
                        tt::st8(crow + col, tt::pack8(o));
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(tempty_bar(buf));
        }
    }

done:
    tc_fence_before();
    __syncthreads();
    if (abort_flag) {
        if (threadIdx.x == 0) atomicExch(p.status, TT_ERR_TIMEOUT);
        // give any TMA copy still in flight time to land before the CTA's shared memory goes away
        for (int i = 0; i < 200; ++i) __nanosleep(1000);
    }
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, C::kTmemCols);
    }
}

template <int BN, bool A_MN, bool B_MN, int EPI>
int launch(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmParams& p, int sms, cudaStream_t st) {
    using C = Cfg<BN>;
    auto kern = gemm_kernel<BN, A_MN, B_MN, EPI>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
        if (e != cudaSuccess) return tt_record_cuda(e);
        configured = true;
    }
    const int tiles = p.tiles_m * p.tiles_n;
    const int grid = tiles < sms ? tiles : sms;
    kern<<<grid, kThreads, C::kSmemBytes, st>>>(tmA, tmB, p);
    TT_CHECK_LAUNCH();
    return TT_OK;
}

template <int BN>
int dispatch(bool a_mn, bool b_mn, int epi, const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmParams& p, int sms,
             cudaStream_t st) {
    if (!a_mn && !b_mn) {
        if (epi == 0) return launch<BN, false, false, 0>(tmA, tmB, p, sms, st);
        if (epi == 1) return launch<BN, false, false, 1>(tmA, tmB, p, sms, st);
        if (epi == 2) return launch<BN, false, false, 2>(tmA, tmB, p, sms, st);
    } else if (!a_mn && b_mn) {
        if (epi == 0) return launch<BN, false, true, 0>(tmA, tmB, p, sms, st);
        if (epi == 3) return launch<BN, false, true, 3>(tmA, tmB, p, sms, st);
        if (epi == 4) return launch<BN, false, true, 4>(tmA, tmB, p, sms, st);
    } else if (a_mn && b_mn) {
        if (epi == 0) return launch<BN, true, true, 0>(tmA, tmB, p, sms, st);
    }
    return TT_ERR_ARG;
}

int g_sms[64] = {0};

int sm_count() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (g_sms[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        g_sms[dev] = n;
    }
    return g_sms[dev];
}

}  // namespace

// ---------------------------------------------------------------------------------------------
// tensor-map helpers (shared with the attention kernels)
// ---------------------------------------------------------------------------------------------
tt_encode_tiled_fn tt_get_encode_tiled() {
    static tt_encode_tiled_fn fn = nullptr;
    if (fn == nullptr) {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            return nullptr;
        fn = (tt_encode_tiled_fn)sym;
    }
    return fn;
}

int tt_make_tmap_2d(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows,
                    uint32_t box_cols) {
    tt_encode_tiled_fn enc = tt_get_encode_tiled();
    if (enc == nullptr) return TT_ERR_CUDA;
    if (((uintptr_t)base & 15) || ((ld * 2) & 15) || box_cols * 2 > 128 || box_rows > 256) return TT_ERR_ARG;
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {ld * 2};
    cuuint32_t box[2] = {box_cols, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? TT_OK : TT_ERR_ARG;
}

int tt_make_tmap_3d(CUtensorMap* out, const void* base, uint64_t d2, uint64_t d1, uint64_t d0, uint64_t stride1,
                    uint64_t stride2, uint32_t box1, uint32_t box0) {
    tt_encode_tiled_fn enc = tt_get_encode_tiled();
    if (enc == nullptr) return TT_ERR_CUDA;
    if (((uintptr_t)base & 15) || ((stride1 * 2) & 15) || ((stride2 * 2) & 15) || box0 * 2 > 128 || box1 > 256)
        return TT_ERR_ARG;
    cuuint64_t dims[3] = {d0, d1, d2};
    cuuint64_t strides[2] = {stride1 * 2, stride2 * 2};
    cuuint32_t box[3] = {box0, box1, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? TT_OK : TT_ERR_ARG;
}

int tt_make_tmap_bshd(CUtensorMap* out, const void* base, uint64_t B, uint64_t S, uint64_t H, uint32_t box_rows) {
    tt_encode_tiled_fn enc = tt_get_encode_tiled();
    if (enc == nullptr) return TT_ERR_CUDA;
    if (((uintptr_t)base & 15) || box_rows > 256) return TT_ERR_ARG;
    cuuint64_t dims[4] = {128, H, S, B};
    cuuint64_t strides[3] = {128 * 2, H * 128 * 2, S * H * 128 * 2};
    cuuint32_t box[4] = {64, 1, box_rows, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? TT_OK : TT_ERR_ARG;
}

// C[M, N] = epilogue(op(A) op(B)^T ...) as described at the top of this file.
//   a_mn == 0: a is A[M, K] with row pitch lda;   a_mn == 1: a is A^T stored [K, M] with row pitch lda
//   b_mn == 0: b is B[N, K] with row pitch ldb;   b_mn == 1: b is B stored [K, N] with row pitch ldb
//   epi: 0 bias (optional); 1 / 2 bias + GELU erf / tanh, pre-activation written to aux;
//        3 / 4 multiply by GELU'(aux) erf / tanh.
//   status: device int, set to TT_ERR_TIMEOUT if a bounded wait inside the kernel gave up.
extern "C" int tt_gemm_bf16(const void* a, const void* b, void* c, const void* bias, void* aux, int M, int N, int K,
                            long lda, long ldb, long ldc, int a_mn, int b_mn, int epi, int* status, void* stream) {
    if (M <= 0 || N <= 0 || K <= 0 || (N & 7) || (K & 7) || (ldc & 7) || status == nullptr) return TT_ERR_ARG;
    if (a_mn && (M & 7)) return TT_ERR_ARG;
    if (epi != 0 && aux == nullptr) return TT_ERR_ARG;
    if (((uintptr_t)c & 15) || (bias && ((uintptr_t)bias & 15)) || (aux && ((uintptr_t)aux & 15))) return TT_ERR_ARG;
    const int sms = sm_count();
    // 128 x 256 tiles unless they would leave most SMs idle or N is not a multiple of 256 but is of 128
    const long tiles256 = (long)((M + BM - 1) / BM) * ((N + 255) / 256);
    const bool use128 = (N % 256 != 0 && N % 128 == 0) || tiles256 < sms;
    const int BN = use128 ? 128 : 256;
    CUtensorMap tmA, tmB;
    int rc;
    if (!a_mn) rc = tt_make_tmap_2d(&tmA, a, (uint64_t)M, (uint64_t)K, (uint64_t)lda, BM, BK);
    else rc = tt_make_tmap_2d(&tmA, a, (uint64_t)K, (uint64_t)M, (uint64_t)lda, 64, 64);
    if (rc != TT_OK) return rc;
    if (!b_mn) rc = tt_make_tmap_2d(&tmB, b, (uint64_t)N, (uint64_t)K, (uint64_t)ldb, (uint32_t)BN, BK);
    else rc = tt_make_tmap_2d(&tmB, b, (uint64_t)K, (uint64_t)N, (uint64_t)ldb, 64, 64);
    if (rc != TT_OK) return rc;
    GemmParams p;
    p.M = M; p.N = N; p.K = K;
    p.C = (__nv_bfloat16*)c;
    p.ldc = ldc;
    p.bias = (const __nv_bfloat16*)bias;
    p.aux = (__nv_bfloat16*)aux;
    p.status = status;
    p.tiles_m = (M + BM - 1) / BM;
    p.tiles_n = (N + BN - 1) / BN;
    cudaStream_t st = (cudaStream_t)stream;
    return use128 ? dispatch<128>(a_mn != 0, b_mn != 0, epi, tmA, tmB, p, sms, st)
                  : dispatch<256>(a_mn != 0, b_mn != 0, epi, tmA, tmB, p, sms, st);
}
