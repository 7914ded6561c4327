// bf16 GEMM on CTA pairs: two CTAs of a thread-block cluster share one 256 x 256 x 64 tile and one
// tcgen05.mma.cta_group::2 instruction stream.  CTA r of the pair loads rows [128 r, 128 r + 128) of the A tile and
// rows [128 r, 128 r + 128) of the B tile (its half of N) into its own shared memory, with its own non-multicast TMA
// loads; the leader CTA (rank 0) issues every MMA, which reads both CTAs' shared memory and writes each CTA's half of
// the accumulator (128 rows x 256 fp32 columns, double buffered) into that CTA's tensor memory.  Per CTA and k-block
// 32 KB come through L2 instead of the 48 KB of the single-CTA 128 x 256 tile: the short-K products of the model
// (K = 3072: QKV, fc1, projections), which sit at the L2 / epilogue limit with the single-CTA kernel, gain the most.
//
// Synchronisation (all mbarrier waits bounded, sm100.cuh):
//   full[s]   in the leader: armed by the leader's producer with the bytes of BOTH CTAs; each CTA's TMA loads complete
//             on it (the .cta_group::2 form of the load addresses the leader's barrier);
//   empty[s]  in each CTA: the leader's tcgen05.commit multicasts the "stage consumed" arrival to both;
//   tfull[b]  in each CTA: commit multicast when an accumulator buffer is complete;
//   tempty[b] in the leader: the four epilogue warps of both CTAs arrive (8 arrivals) once a buffer has been drained.
// Tensor memory is allocated and freed by warp 1 of both CTAs (cta_group::2), the free after a cluster barrier.
//
// Layouts and epilogues are those of gemm_tcgen05.cu (nt / nn / tn; bias, GELU erf / tanh with pre-activation,
// GELU backward).  In the reference these products are TransformerEngine -> cuBLASLt calls
// (teletron/models/dit/dit_attention.py:65-104, dit_layerspec.py:266-298, 438-445).
#include "common.cuh"
#include "sm100.cuh"
#include "teletron_b200.h"

#include <string.h>

namespace {

using namespace sm100;

constexpr int BMH = 128;            // rows of A per CTA (half of the pair's 256)
constexpr int BNH = 128;            // rows of B (columns of C) loaded per CTA (half of the pair's 256)
constexpr int BN = 256;             // columns of the accumulator
constexpr int BK = 64;
constexpr int kStages = 6;
constexpr int kABytes = BMH * BK * 2;
constexpr int kBBytes = BNH * BK * 2;
constexpr int kStageBytes = kABytes + kBBytes;          // 32 KB per CTA
constexpr int kThreads = 192;
constexpr int kGroupM = 8;
constexpr int kSmemBytes = kStages * kStageBytes + 1024 + 256;
constexpr uint32_t kPeerMask = 0xFEFFFFFFu;             // clears the bit that tells the two CTAs of a pair apart

struct Params2 {
    int M, N, K;
    __nv_bfloat16* C;
    long ldc;
    const __nv_bfloat16* bias;
    __nv_bfloat16* aux;
    int* status;
    int tiles_m, tiles_n;       // in 256 x 256 tiles
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }

__device__ __forceinline__ void tmem_alloc2(uint32_t smem_result, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_result), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish2() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// 2-D tiled load (no multicast) whose completion bytes go to the LEADER CTA's mbarrier
__device__ __forceinline__ void tma_load_2d_pair(uint32_t smem_dst, const CUtensorMap* tmap, uint32_t bar, int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
            smem_dst),
        "l"((uint64_t)tmap), "r"(bar & kPeerMask), "r"(c0), "r"(c1)
        : "memory");
}
__device__ __forceinline__ void umma2_bf16_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// arrives (once the MMAs issued so far have completed) on the barrier at this shared-memory offset in BOTH CTAs of the pair
__device__ __forceinline__ void umma2_commit_both(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar),
                 "h"((uint16_t)3)
                 : "memory");
}
// plain arrival on the leader CTA's copy of a barrier (from either CTA)
__device__ __forceinline__ void mbar_arrive_leader(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(bar & kPeerMask) : "memory");
}

template <int EPI>
__device__ __forceinline__ float epi2(float acc, float b, float u) {
    if (EPI == 0) return acc + b;
    if (EPI == 1) return tt::gelu_erf(acc + b);
    if (EPI == 2) return tt::gelu_tanh(acc + b);
    if (EPI == 3) return acc * tt::gelu_erf_grad(u);
    return acc * tt::gelu_tanh_grad(u);
}

template <bool A_MN, bool B_MN, int EPI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
gemm2_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const Params2 p) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ volatile int abort_flag;
    __shared__ uint32_t tmem_base_slot;

    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t bar_base = base + kStages * kStageBytes;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (kStages + s); };
    auto tfull_bar = [&](int b) { return bar_base + 8u * (2 * kStages + b); };
    auto tempty_bar = [&](int b) { return bar_base + 8u * (2 * kStages + 2 + b); };

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();            // 0 = leader
    const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int s = 0; s < kStages; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(tfull_bar(b), 1);
            mbar_init(tempty_bar(b), 8);                  // four epilogue warps of each CTA
        }
        fence_barrier_init();
        fence_proxy_async();
        tma_prefetch_desc(&tmA);
        tma_prefetch_desc(&tmB);
    }
    if (warp == 1) {
        tmem_alloc2(smem_u32(&tmem_base_slot), 512);
        tmem_relinquish2();
    }
    tc_fence_before();
    __syncthreads();
    // nobody may signal the other CTA's barriers before they exist
    cluster_arrive();
    cluster_wait();
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
        m0 = (first_m + r % gm) * 256;
        n0 = (r / gm) * 256;
    };

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer (one per CTA: its halves of A and B)
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            for (int t = pair; t < num_tiles; t += n_pairs) {
                int m0, n0;
                tile_coords(t, m0, n0);
                const int am = m0 + (int)rank * BMH, bn = n0 + (int)rank * BNH;
                for (int kb = 0; kb < kblocks; ++kb) {
                    if (!mbar_wait(empty_bar(stage), phase ^ 1u, &abort_flag)) goto done;
                    const uint32_t sa = base + stage * kStageBytes;
                    const uint32_t sb = sa + kABytes;
                    if (rank == 0) mbar_arrive_expect_tx(full_bar(stage), 2 * kStageBytes);      // both CTAs' bytes
                    const int k0 = kb * BK;
                    if (!A_MN) {
                        tma_load_2d_pair(sa, &tmA, full_bar(stage), k0, am);
                    } else {
#pragma unroll
                        for (int j = 0; j < BMH / 64; ++j) tma_load_2d_pair(sa + j * 8192, &tmA, full_bar(stage), am + 64 * j, k0);
                    }
                    if (!B_MN) {
                        tma_load_2d_pair(sb, &tmB, full_bar(stage), k0, bn);
                    } else {
#pragma unroll
                        for (int j = 0; j < BNH / 64; ++j) tma_load_2d_pair(sb + j * 8192, &tmB, full_bar(stage), bn + 64 * j, k0);
                    }
                    if (++stage == kStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer (leader CTA only)
        if (lane == 0 && rank == 0) {
            constexpr uint32_t idesc = idesc_bf16(256, BN, A_MN, B_MN);
            int stage = 0;
            uint32_t phase = 0;
            int it = 0;
            for (int t = pair; t < num_tiles; t += n_pairs, ++it) {
                const int buf = it & 1;
                const uint32_t acc_phase = (uint32_t)(it >> 1) & 1u;
                if (!mbar_wait(tempty_bar(buf), acc_phase ^ 1u, &abort_flag)) goto done;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(buf * BN);
                for (int kb = 0; kb < kblocks; ++kb) {
                    if (!mbar_wait(full_bar(stage), phase, &abort_flag)) goto done;
                    tc_fence_after();
                    const uint32_t sa = base + stage * kStageBytes;
                    const uint32_t sb = sa + kABytes;
#pragma unroll
                    for (int kk = 0; kk < BK / 16; ++kk) {
                        const uint64_t da = A_MN ? smem_desc_sw128(sa + kk * 2048, 8192, 1024) : smem_desc_sw128(sa + kk * 32, 16, 1024);
                        const uint64_t db = B_MN ? smem_desc_sw128(sb + kk * 2048, 8192, 1024) : smem_desc_sw128(sb + kk * 32, 16, 1024);
                        umma2_bf16_ss(d_tmem, da, db, idesc, (kb | kk) ? 1u : 0u);
                    }
                    umma2_commit_both(empty_bar(stage));        // frees this stage in both CTAs when the MMAs retire
                    if (++stage == kStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                umma2_commit_both(tfull_bar(buf));              // accumulator complete, both halves
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue (warps 2..5 of each CTA: its 128 rows)
        const int quad = warp & 3;
        int it = 0;
        for (int t = pair; t < num_tiles; t += n_pairs, ++it) {
            int m0, n0;
            tile_coords(t, m0, n0);
            const int buf = it & 1;
            const uint32_t acc_phase = (uint32_t)(it >> 1) & 1u;
            if (!mbar_wait(tfull_bar(buf), acc_phase, &abort_flag)) goto done;
            tc_fence_after();
            const int row = m0 + (int)rank * BMH + quad * 32 + lane;
            const bool row_ok = row < p.M;
            const uint32_t tacc = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(buf * BN);
            __nv_bfloat16* crow = p.C + (long)row * p.ldc;
            __nv_bfloat16* arow = (EPI != 0) ? p.aux + (long)row * p.ldc : nullptr;
#pragma unroll 1
            for (int c = 0; c < BN / 32; ++c) {
                uint32_t r[32];
                tmem_ld_32x32(tacc + c * 32, r);
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
                        for (int j = 0; j < 8; ++j) o[j] = epi2<EPI>(__uint_as_float(r[g * 8 + j]), bv[j], uv[j]);
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
            if (lane == 0) mbar_arrive_leader(tempty_bar(buf));
        }
    }

done:
    tc_fence_before();
    __syncthreads();
    if (abort_flag) {
        if (threadIdx.x == 0) atomicExch(p.status, TT_ERR_TIMEOUT);
        for (int i = 0; i < 200; ++i) __nanosleep(1000);        // let TMA copies in flight land
    }
    // both CTAs are done with each other's shared and tensor memory before either frees it
    cluster_arrive();
    cluster_wait();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc2(tmem_base, 512);
    }
}

template <bool A_MN, bool B_MN, int EPI>
int launch2(const CUtensorMap& tmA, const CUtensorMap& tmB, const Params2& p, int sms, cudaStream_t st) {
    auto kern = gemm2_kernel<A_MN, B_MN, EPI>;
    static bool configured[64] = {false};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
    if (!configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
        if (e != cudaSuccess) return tt_record_cuda(e);
        configured[dev] = true;
    }
    const int tiles = p.tiles_m * p.tiles_n;
    int pairs = sms / 2;
    if (pairs > tiles) pairs = tiles;
    if (pairs < 1) pairs = 1;
    kern<<<2 * pairs, kThreads, kSmemBytes, st>>>(tmA, tmB, p);      // cluster shape comes from __cluster_dims__
    TT_CHECK_LAUNCH();
    return TT_OK;
}

}  // namespace

// Same contract as tt_gemm_bf16 (gemm_tcgen05.cu); returns TT_ERR_ARG for shapes this kernel does not take, so that the
// caller can fall back to the single-CTA kernel.
extern "C" int tt_gemm2_bf16(const void* a, const void* b, void* c, const void* bias, void* aux, int M, int N, int K,
                             long lda, long ldb, long ldc, int a_mn, int b_mn, int epi, int* status, void* stream) {
    if (M <= 0 || N <= 0 || K <= 0 || (N & 7) || (K & 7) || (ldc & 7) || status == nullptr) return TT_ERR_ARG;
    if (a_mn && (M & 7)) return TT_ERR_ARG;
    if (epi < 0 || epi > 4 || (epi != 0 && aux == nullptr)) return TT_ERR_ARG;
    if (((uintptr_t)c & 15) || (bias && ((uintptr_t)bias & 15)) || (aux && ((uintptr_t)aux & 15))) return TT_ERR_ARG;
    if (a_mn && !b_mn) return TT_ERR_ARG;
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    CUtensorMap tmA, tmB;
    int rc;
    if (!a_mn) rc = tt_make_tmap_2d(&tmA, a, (uint64_t)M, (uint64_t)K, (uint64_t)lda, BMH, BK);
    else rc = tt_make_tmap_2d(&tmA, a, (uint64_t)K, (uint64_t)M, (uint64_t)lda, 64, 64);
    if (rc != TT_OK) return rc;
    if (!b_mn) rc = tt_make_tmap_2d(&tmB, b, (uint64_t)N, (uint64_t)K, (uint64_t)ldb, BNH, BK);
    else rc = tt_make_tmap_2d(&tmB, b, (uint64_t)K, (uint64_t)N, (uint64_t)ldb, 64, 64);
    if (rc != TT_OK) return rc;
    Params2 p;
    memset(&p, 0, sizeof(p));
    p.M = M; p.N = N; p.K = K;
    p.C = (__nv_bfloat16*)c;
    p.ldc = ldc;
    p.bias = (const __nv_bfloat16*)bias;
    p.aux = (__nv_bfloat16*)aux;
    p.status = status;
    p.tiles_m = (M + 255) / 256;
    p.tiles_n = (N + 255) / 256;
    cudaStream_t st = (cudaStream_t)stream;
    const bool amn = a_mn != 0, bmn = b_mn != 0;
#define GO(A_, B_, E_) return launch2<A_, B_, E_>(tmA, tmB, p, sms, st)
    if (!amn && !bmn) {
        if (epi == 0) GO(false, false, 0);
        if (epi == 1) GO(false, false, 1);
        if (epi == 2) GO(false, false, 2);
    } else if (!amn && bmn) {
        if (epi == 0) GO(false, true, 0);
        if (epi == 3) GO(false, true, 3);
        if (epi == 4) GO(false, true, 4);
    } else if (amn && bmn) {
        if (epi == 0) GO(true, true, 0);
    }
#undef GO
    return TT_ERR_ARG;
}
