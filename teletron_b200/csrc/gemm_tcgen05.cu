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

#include <string.h>

namespace {

using namespace sm100;

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int kThreads = 192;
constexpr int kGroupM = 16;

struct TmapArray {
    CUtensorMap m[TT_MAX_PEERS + 1];     // last slot: local tensor supplying the K columns beyond the gathered ones
};

struct GemmParams {
    int M, N, K;
    __nv_bfloat16* C;
    long ldc;
    const __nv_bfloat16* bias;
    __nv_bfloat16* aux;     // EPI 1/2: pre-activation output; EPI 3/4: pre-activation input; EPI 5: raw QKV output
    int* status;
    int tiles_m, tiles_n;
    // ---- operand A gathered from several ranks (tensor maps over peer memory, plain non-multicast TMA) ----
    int a_mode;             // 0: one source; 1: source chosen by K column block (head -> owner rank);
                            // 2: source chosen by M segment (all-gather of row blocks)
    int a_span;             // mode 1: K columns held by each source
    int a_nsrc;             // mode 1: number of sources; K columns >= a_nsrc * a_span come from the local extra tensor
    int a_row_off;          // mode 0/1: row offset of this rank's rows inside the source tensor
    int n_seg, seg_rows;    // M is n_seg segments of seg_rows rows (n_seg == 1: plain)
    int seg_rot;            // first segment processed (own rank's rows first)
    int my_rank;
    // mode 2 with staging: remote row segments are copied once into `stage` (this GPU's memory) by dedicated copier
    // warps while the tensor core works on the local segment; tiles of a remote segment wait for their rows' flag
    __nv_bfloat16* stage;               // [n_seg * seg_rows, K]
    const __nv_bfloat16* peer_a[TT_MAX_PEERS];
    int* stage_flags;                   // [n_seg * tiles_per_seg], set to `stage_epoch` when the rows have landed
    int stage_epoch;
    // ---- where the output tile goes ----
    int store_mode;         // 0: C (local); 1: column block -> peer_out[col / out_span] (head -> owner);
                            // 2: row segment -> peer_out[segment] staging slot of this rank (reduce-scatter push)
    int out_span, out_row_off;
    int n_dest;             // store_mode 1: number of routed column blocks; later columns go to C
    long out_ld;
    __nv_bfloat16* peer_out[TT_MAX_PEERS];
    // ---- fused QKV epilogue (EPI 5): bias, QK-RMSNorm, RoPE, head-major scatter to the head's owner rank ----
    const __nv_bfloat16* qw;
    const __nv_bfloat16* kw;
    const float* cos_t;
    const float* sin_t;
    float eps;
    int rope_len, heads_per_rank, s_in, s_out, out_off, only_local;
    int coalesce;           // pushed tiles: stage each warp's 32 x 128 block in shared memory, store whole 256-byte rows
    __nv_bfloat16* peer_q[TT_MAX_PEERS];
    __nv_bfloat16* peer_k[TT_MAX_PEERS];
    __nv_bfloat16* peer_v[TT_MAX_PEERS];
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
    if (EPI == 0 || EPI == 6) return acc + b;
    if (EPI == 1) return tt::gelu_erf(acc + b);
    if (EPI == 2) return tt::gelu_tanh(acc + b);
    if (EPI == 3) return acc * tt::gelu_erf_grad(u);
    return acc * tt::gelu_tanh_grad(u);
}

__device__ __forceinline__ int ld_acquire(const int* p) {
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release(int* p, int v) {
    asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

template <int BN, bool A_MN, bool B_MN, int EPI, bool STAGE = false>
__global__ void __launch_bounds__(STAGE ? kThreads + 128 : kThreads, 1)
gemm_kernel(const __grid_constant__ TmapArray tmA, const __grid_constant__ CUtensorMap tmB, const GemmParams p) {
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
    const uint32_t epi_stage = bar_base + 256u;      // coalesced peer stores: 4 warps x 8 KB (only when launched with room for it)

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
        tma_prefetch_desc(&tmA.m[0]);
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
    const int tiles_per_seg = p.tiles_m / p.n_seg;
    // tile index -> (segment, first row inside the segment, first column)
    auto tile_coords = [&](int t, int& seg, int& m0, int& n0) {
        const int per_group = kGroupM * p.tiles_n;
        const int g = t / per_group;
        const int first_m = g * kGroupM;
        const int gm = min(kGroupM, p.tiles_m - first_m);
        const int r = t - g * per_group;
        const int mt = first_m + r % gm;
        const int si = mt / tiles_per_seg;
        seg = si + p.seg_rot;
        if (seg >= p.n_seg) seg -= p.n_seg;
        m0 = (mt - si * tiles_per_seg) * BM;
        n0 = (r / gm) * BN;
    };

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            for (int t = blockIdx.x; t < num_tiles; t += gridDim.x) {
                int seg, m0, n0;
                tile_coords(t, seg, m0, n0);
                for (int kb = 0; kb < kblocks; ++kb) {
                    if (!mbar_wait(empty_bar(stage), phase ^ 1u, &abort_flag)) goto done;
                    const uint32_t sa = base + stage * C::kStageBytes;
                    const uint32_t sb = sa + C::kABytes;
                    mbar_arrive_expect_tx(full_bar(stage), C::kStageBytes);
                    const int k0 = kb * BK;
                    if (!A_MN) {
                        // pick the source tensor: local, the owner of this K block (head), or the owner of this row segment
                        const CUtensorMap* ta = &tmA.m[0];
                        int ak = k0, am = p.a_row_off + seg * p.seg_rows + m0;
                        if (p.a_mode == 1) {
                            const int src = k0 / p.a_span;
                            if (src < p.a_nsrc) {
                                ta = &tmA.m[src];
                                ak = k0 - src * p.a_span;
                            } else {        // local tail (e.g. the MLP half of the single block's merged projection)
                                ta = &tmA.m[TT_MAX_PEERS];
                                ak = k0 - p.a_nsrc * p.a_span;
                                am = m0;
                            }
                        } else if (p.a_mode == 2) {
                            if (STAGE && seg != p.my_rank) {
                                if (kb == 0) {
                                    // rows of a remote segment: wait (bounded) until the copier warps have landed them
                                    const int* flag = p.stage_flags + seg * tiles_per_seg + m0 / BM;
                                    const long long t0 = clock64();
                                    while (ld_acquire(flag) != p.stage_epoch) {
                                        if (abort_flag || clock64() - t0 > kWaitCycles) {
                                            abort_flag = 1;
                                            goto done;
                                        }
                                        __nanosleep(100);
                                    }
                                    asm volatile("fence.proxy.async;" ::: "memory");    // generic-proxy writes -> TMA reads
                                }
                                ta = &tmA.m[TT_MAX_PEERS];
                                am = seg * p.seg_rows + m0;
                            } else {
                                ta = &tmA.m[seg];
                                am = m0;
                            }
                        }
                        tma_load_2d(sa, ta, full_bar(stage), ak, am);
                    } else {
#pragma unroll
                        for (int j = 0; j < BM / 64; ++j) tma_load_2d(sa + j * 8192, &tmA.m[0], full_bar(stage), m0 + 64 * j, k0);
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
    } else if (STAGE && warp >= 6) {
        // ------------------------------------------------------------ copier warps (all-gather staging)
        const int tid = threadIdx.x - 192;
        const int n_items = (p.n_seg - 1) * tiles_per_seg;
        const long row_vecs = p.K >> 3;
        for (int item = blockIdx.x; item < n_items; item += gridDim.x) {
            int seg = 1 + item / tiles_per_seg + p.seg_rot;       // segments in the order the tiles will need them
            if (seg >= p.n_seg) seg -= p.n_seg;
            const int mt = item % tiles_per_seg;
            const int r0 = mt * BM;
            const int nrows = min(BM, p.seg_rows - r0);
            const __nv_bfloat16* src = p.peer_a[seg] + (long)r0 * p.K;
            __nv_bfloat16* dst = p.stage + ((long)seg * p.seg_rows + r0) * p.K;
            const long nvec = (long)nrows * row_vecs;
            // eight 16-byte peer loads in flight per thread: one outstanding load per thread leaves NVLink mostly idle
            // (a load takes ~2 us to come back; 128 threads x 148 CTAs x 16 B per round trip is ~150 GB/s)
            long v = tid;
            for (; v + 7 * 128 < nvec; v += 8 * 128) {
                tt::bf16x8 t[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) t[u] = tt::ld8(src + (v + u * 128) * 8);
#pragma unroll
                for (int u = 0; u < 8; ++u) tt::st8(dst + (v + u * 128) * 8, t[u]);
            }
            for (; v < nvec; v += 128) tt::st8(dst + v * 8, tt::ld8(src + v * 8));
            __threadfence();
            asm volatile("bar.sync 1, 128;" ::: "memory");        // only the copier warps take part; no waits in this loop
            if (tid == 0) st_release(p.stage_flags + seg * tiles_per_seg + mt, p.stage_epoch);
        }
    } else {
        // ------------------------------------------------------------ epilogue (warps 2..5)
        const int quad = warp & 3;
        // Coalesced store of this warp's 32 rows x 128 columns (lane = row, v = the row's values, dst = where the row's 128
        // columns go, nullptr for rows that are not stored; only the first `ncols` columns are written).  The block goes
        // through shared memory, 16-byte chunks XOR-swizzled by row so that neither side has more than 2-way bank
        // conflicts, and every store instruction then covers two whole 256-byte rows.
        auto store_block_coalesced = [&](const float* v, __nv_bfloat16* dst_row, int ncols) {
            const uint32_t sst = epi_stage + (uint32_t)(warp - 2) * 8192u;
#pragma unroll
            for (int g = 0; g < 16; ++g) {
                const tt::bf16x8 pk = tt::pack8(v + g * 8);
                const uint4 u = *reinterpret_cast<const uint4*>(&pk);
                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(sst + lane * 256u + (uint32_t)((g ^ (lane & 15)) << 4)),
                             "r"(u.x), "r"(u.y), "r"(u.z), "r"(u.w)
                             : "memory");
            }
            __syncwarp();
            const unsigned long long dptr = (unsigned long long)dst_row;
#pragma unroll
            for (int t = 0; t < 16; ++t) {
                const int r = 2 * t + (lane >> 4), j = lane & 15;
                uint4 u;
                asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                             : "=r"(u.x), "=r"(u.y), "=r"(u.z), "=r"(u.w)
                             : "r"(sst + r * 256u + (uint32_t)((j ^ (r & 15)) << 4))
                             : "memory");
                const unsigned long long dst = __shfl_sync(0xffffffffu, dptr, r);
                if (dst != 0ull && j * 8 + 8 <= ncols) *reinterpret_cast<uint4*>(dst + (unsigned long long)j * 16ull) = u;
            }
            __syncwarp();       // the staging block is reused by the next call
        };
        int it = 0;
        for (int t = blockIdx.x; t < num_tiles; t += gridDim.x, ++it) {
            int seg, m0, n0;
            tile_coords(t, seg, m0, n0);
            const int buf = it & 1;
            const uint32_t acc_phase = (uint32_t)(it >> 1) & 1u;
            if (!mbar_wait(tfull_bar(buf), acc_phase, &abort_flag)) goto done;
            tc_fence_after();
            const int lrow = m0 + quad * 32 + lane;                 // row inside the segment
            const int row = seg * p.seg_rows + lrow;                // row of the logical output
            const bool row_ok = lrow < p.seg_rows && row < p.M;
            const uint32_t tacc = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(buf * BN);
            const uint32_t tacc_tile = tacc;
            const int n0_tile = n0;
            if (EPI == 5) {
              // ---- fused QKV epilogue: every 128 columns of the tile are one head's q, k or v ----
              // (256-wide tiles keep the tensor core at N = 256; the epilogue walks the two heads one after the other.)
              // Phase 1, one lane per row: accumulator + bias, rounded to bf16 (the value a separate QKV GEMM would hand to
              // the norm, and the one the backward rebuilds from), into this warp's staging block; 16-byte chunks are
              // XOR-swizzled by row so that neither phase has more than 2-way bank conflicts.
              // Phase 2, sixteen lanes per row, two rows per pass: everything that touches global or peer memory is now a
              // whole 256-byte row per half-warp - the raw copy kept for the backward, the cos / sin tables, and the
              // store into the owner rank's [head, token, 128] buffer (small scattered stores reach a peer GPU as small
              // NVLink packets).  RMSNorm sums run over the 16 lanes of a row; bias and norm weights are per-lane constants.
              const uint32_t sst = epi_stage + (uint32_t)(warp - 2) * 8192u;
              const int row_base = m0 + quad * 32;
              const int j = lane & 15, half = lane >> 4;
#pragma unroll 1
              for (int hh = 0; hh < BN / 128; ++hh) {
                const int n0 = n0_tile + hh * 128;
                if (n0 >= p.N) break;
                const uint32_t tacc = tacc_tile + hh * 128;
                const int idx = n0 / 128;
                const int head = idx / 3, which = idx - head * 3;
                const int dest = head / p.heads_per_rank, hl = head - dest * p.heads_per_rank;
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    uint32_t r[32];
                    tmem_ld_32x32(tacc + c * 32, r);
                    tmem_ld_wait();
#pragma unroll
                    for (int g = 0; g < 4; ++g) {
                        float bv[8], o[8];
#pragma unroll
                        for (int i = 0; i < 8; ++i) bv[i] = 0.f;
                        if (p.bias != nullptr) tt::unpack8(tt::ld8(p.bias + n0 + c * 32 + g * 8), bv);
#pragma unroll
                        for (int i = 0; i < 8; ++i) o[i] = __uint_as_float(r[g * 8 + i]) + bv[i];
                        const tt::bf16x8 pk = tt::pack8(o);
                        const uint4 u = *reinterpret_cast<const uint4*>(&pk);
                        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(sst + lane * 256u + (uint32_t)(((c * 4 + g) ^ (lane & 15)) << 4)),
                                     "r"(u.x), "r"(u.y), "r"(u.z), "r"(u.w)
                                     : "memory");
                    }
                }
                __syncwarp();
                float wv[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) wv[i] = 1.f;
                if (which < 2) tt::unpack8(tt::ld8((which == 0 ? p.qw : p.kw) + j * 8), wv);
                __nv_bfloat16* dbase = which == 0 ? p.peer_q[dest] : (which == 1 ? p.peer_k[dest] : p.peer_v[dest]);
                const bool head_kept = !p.only_local || dest == p.my_rank;
#pragma unroll 2
                for (int t = 0; t < 16; ++t) {
                    const int r = 2 * t + half;
                    const int row = row_base + r;
                    const bool ok = row < p.M;
                    uint4 u;
                    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                                 : "=r"(u.x), "=r"(u.y), "=r"(u.z), "=r"(u.w)
                                 : "r"(sst + r * 256u + (uint32_t)((j ^ (r & 15)) << 4))
                                 : "memory");
                    // the raw projection is kept for every head (the backward rebuilds all of them, also for replicated tokens)
                    if (ok && p.aux != nullptr) *reinterpret_cast<uint4*>(p.aux + (long)row * p.ldc + n0 + j * 8) = u;
                    float v[8];
                    tt::unpack8(*reinterpret_cast<const tt::bf16x8*>(&u), v);
                    const int b = row / p.s_in, srow = row - b * p.s_in;
                    if (which < 2) {
                        float ss = 0.f;
#pragma unroll
                        for (int i = 0; i < 8; ++i) ss += v[i] * v[i];
#pragma unroll
                        for (int o = 8; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);     // the row's 16 lanes
                        const float rstd = rsqrtf(ss * (1.f / 128.f) + p.eps);
#pragma unroll
                        for (int i = 0; i < 8; ++i) v[i] *= rstd * wv[i];
                        if (ok && srow < p.rope_len) {
                            const float4* c4 = reinterpret_cast<const float4*>(p.cos_t + (long)srow * 128 + j * 8);
                            const float4* s4 = reinterpret_cast<const float4*>(p.sin_t + (long)srow * 128 + j * 8);
#pragma unroll
                            for (int g = 0; g < 2; ++g) {
                                const float4 cc = c4[g], sn = s4[g];
                                const float a0 = v[4 * g], a1 = v[4 * g + 1], a2 = v[4 * g + 2], a3 = v[4 * g + 3];
                                v[4 * g] = a0 * cc.x - a1 * sn.x;
                                v[4 * g + 1] = a1 * cc.y + a0 * sn.y;
                                v[4 * g + 2] = a2 * cc.z - a3 * sn.z;
                                v[4 * g + 3] = a3 * cc.w + a2 * sn.w;
                            }
                        }
                    }
                    if (ok && head_kept) {
                        __nv_bfloat16* drow = dbase + (((long)b * p.heads_per_rank + hl) * p.s_out + p.out_off + srow) * 128;
                        tt::st8(drow + j * 8, tt::pack8(v));
                    }
                }
                __syncwarp();       // the staging block is reused by the next head
              }
            } else {
                // where this tile's rows land: local C, the owner rank of a column block, or an owner's staging slot
                __nv_bfloat16* crow;
                int ccol = n0;
                if (p.store_mode == 0) {
                    crow = p.C + (long)row * p.ldc;
                } else if (p.store_mode == 1) {
                    const int dest = n0 / p.out_span;
                    if (dest < p.n_dest) {
                        ccol = n0 - dest * p.out_span;
                        crow = p.peer_out[dest] + (long)(p.out_row_off + row) * p.out_ld;
                    } else {            // columns beyond the routed ones stay local
                        ccol = n0 - p.n_dest * p.out_span;
                        crow = p.C + (long)row * p.ldc;
                    }
                } else {
                    crow = p.peer_out[seg] + ((long)p.my_rank * p.seg_rows + lrow) * p.out_ld;
                }
                __nv_bfloat16* arow = (EPI != 0) ? p.aux + (long)row * p.ldc : nullptr;
                if (EPI == 6) {
                    // tiles pushed to a peer (column blocks of a dgrad, row blocks of a reduce-scatter): 128 columns at a time
                    // through the staged store, for the same reason as in the fused QKV epilogue
#pragma unroll 1
                    for (int c4 = 0; c4 < BN / 128; ++c4) {
                        const int colb = n0 + c4 * 128;
                        if (colb >= p.N) break;
                        float v[128];
#pragma unroll
                        for (int c = 0; c < 4; ++c) {
                            uint32_t r[32];
                            tmem_ld_32x32(tacc + c4 * 128 + c * 32, r);
                            tmem_ld_wait();
#pragma unroll
                            for (int g = 0; g < 4; ++g) {
                                float bv[8];
#pragma unroll
                                for (int j = 0; j < 8; ++j) bv[j] = 0.f;
                                const int col = colb + c * 32 + g * 8;
                                if (p.bias != nullptr && col + 8 <= p.N) tt::unpack8(tt::ld8(p.bias + col), bv);
#pragma unroll
                                for (int j = 0; j < 8; ++j) v[c * 32 + g * 8 + j] = __uint_as_float(r[g * 8 + j]) + bv[j];
                            }
                        }
                        __nv_bfloat16* d = nullptr;
                        if (row_ok) {
                            if (p.store_mode == 1) {
                                const int dest = colb / p.out_span;        // out_span is a multiple of 128: one owner per group
                                d = dest < p.n_dest ? p.peer_out[dest] + (long)(p.out_row_off + row) * p.out_ld + (colb - dest * p.out_span)
                                                    : p.C + (long)row * p.ldc + (colb - p.n_dest * p.out_span);
                            } else {
                                d = crow + colb;
                            }
                        }
                        store_block_coalesced(v, d, min(128, p.N - colb));
                    }
                } else
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
                            for (int j = 0; j < 8; ++j) o[j] = epi_apply<EPI>(__uint_as_float(r[g * 8 + j]), bv[j], uv[j]);
                            if (EPI == 1 || EPI == 2) {
                                float u[8];
#pragma unroll
                                for (int j = 0; j < 8; ++j) u[j] = __uint_as_float(r[g * 8 + j]) + bv[j];
                                tt::st8(arow + col, tt::pack8(u));
                            }
                            tt::st8(crow + ccol + (col - n0), tt::pack8(o));
                        }
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

template <int BN, bool A_MN, bool B_MN, int EPI, bool STAGE = false>
int launch(const TmapArray& tmA, const CUtensorMap& tmB, const GemmParams& p, int sms, cudaStream_t st) {
    using C = Cfg<BN>;
    auto kern = gemm_kernel<BN, A_MN, B_MN, EPI, STAGE>;
    // staging for the coalesced peer stores (4 epilogue warps x 8 KB), only when that variant is selected
    const bool staged_stores = EPI == 6 || EPI == 5;
    const int smem = C::kSmemBytes + (staged_stores ? 4 * 8192 : 0);
    // the attribute belongs to the device's context: remembered per device, not per process
    static int configured[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
    if (configured[dev] < smem) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return tt_record_cuda(e);
        configured[dev] = smem;
    }
    const int tiles = p.tiles_m * p.tiles_n;
    const int grid = tiles < sms ? tiles : sms;
    kern<<<grid, STAGE ? kThreads + 128 : kThreads, smem, st>>>(tmA, tmB, p);
    TT_CHECK_LAUNCH();
    return TT_OK;
}

template <int BN>
int dispatch(bool a_mn, bool b_mn, int epi, const TmapArray& tmA, const CUtensorMap& tmB, const GemmParams& p, int sms,
             cudaStream_t st) {
    if (!a_mn && !b_mn) {
        if (epi == 0) return launch<BN, false, false, 0>(tmA, tmB, p, sms, st);
        if (epi == 1) return launch<BN, false, false, 1>(tmA, tmB, p, sms, st);
        if (epi == 2) return launch<BN, false, false, 2>(tmA, tmB, p, sms, st);
        if (epi == 5) return launch<BN, false, false, 5>(tmA, tmB, p, sms, st);
        if (epi == 6) return launch<BN, false, false, 6>(tmA, tmB, p, sms, st);
    } else if (!a_mn && b_mn) {
        if (epi == 0) return launch<BN, false, true, 0>(tmA, tmB, p, sms, st);
        if (epi == 6) return launch<BN, false, true, 6>(tmA, tmB, p, sms, st);
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

namespace {

void default_params(GemmParams& p) {
    memset(&p, 0, sizeof(p));
    p.n_seg = 1;
}

// Epilogues that push tiles to a peer (column blocks of a data gradient, row blocks of a reduce-scatter) can stage each
// warp's 32 x 128 block in shared memory and store whole 256-byte rows per instruction instead of 16 bytes per thread
// and row.  Chosen by tt_set_coalesced_peer_stores(), else by TELETRON_B200_COALESCED_PEER_STORES (default on).
int g_coalesce = -1;

int coalesced_peer_stores() {
    if (g_coalesce < 0) {
        const char* v = getenv("TELETRON_B200_COALESCED_PEER_STORES");
        g_coalesce = (v != nullptr && v[0] == '0') ? 0 : 1;
    }
    return g_coalesce;
}

int pick_bn(int M, int N, int sms, bool force128) {
    // 128 x 256 tiles unless they would leave most SMs idle or N is not a multiple of 256 but is of 128
    const long tiles256 = (long)((M + BM - 1) / BM) * ((N + 255) / 256);
    return (force128 || (N % 256 != 0 && N % 128 == 0) || tiles256 < sms) ? 128 : 256;
}

}  // namespace

extern "C" void tt_set_coalesced_peer_stores(int on) { g_coalesce = on ? 1 : 0; }

// C[M, N] = epilogue(op(A) op(B)^T ...) as described at the top of this file.
//   a_mn == 0: a is A[M, K] with row pitch lda;   a_mn == 1: a is A^T stored [K, M] with row pitch lda
//   b_mn == 0: b is B[N, K] with row pitch ldb;   b_mn == 1: b is B stored [K, N] with row pitch ldb
//   epi: 0 bias (optional); 1 / 2 bias + GELU erf / tanh, pre-activation written to aux;
//        3 / 4 multiply by GELU'(aux) erf / tanh.  (Internal codes: 5 = the fused QKV epilogue of tt_qkv_gemm_fused,
//        6 = bias with staged, coalesced stores for tiles pushed to a peer by tt_gemm_comm_bf16.)
//   status: device int, set to TT_ERR_TIMEOUT if a bounded wait inside the kernel gave up.
extern "C" int tt_gemm_bf16(const void* a, const void* b, void* c, const void* bias, void* aux, int M, int N, int K,
                            long lda, long ldb, long ldc, int a_mn, int b_mn, int epi, int* status, void* stream) {
    if (M <= 0 || N <= 0 || K <= 0 || (N & 7) || (K & 7) || (ldc & 7) || status == nullptr) return TT_ERR_ARG;
    if (a_mn && (M & 7)) return TT_ERR_ARG;
    if (epi < 0 || epi > 4 || (epi != 0 && aux == nullptr)) return TT_ERR_ARG;
    if (((uintptr_t)c & 15) || (bias && ((uintptr_t)bias & 15)) || (aux && ((uintptr_t)aux & 15))) return TT_ERR_ARG;
    const int sms = sm_count();
    const int BN = pick_bn(M, N, sms, false);
    TmapArray tmA;
    CUtensorMap tmB;
    int rc;
    if (!a_mn) rc = tt_make_tmap_2d(&tmA.m[0], a, (uint64_t)M, (uint64_t)K, (uint64_t)lda, BM, BK);
    else rc = tt_make_tmap_2d(&tmA.m[0], a, (uint64_t)K, (uint64_t)M, (uint64_t)lda, 64, 64);
    if (rc != TT_OK) return rc;
    if (!b_mn) rc = tt_make_tmap_2d(&tmB, b, (uint64_t)N, (uint64_t)K, (uint64_t)ldb, (uint32_t)BN, BK);
    else rc = tt_make_tmap_2d(&tmB, b, (uint64_t)K, (uint64_t)N, (uint64_t)ldb, 64, 64);
    if (rc != TT_OK) return rc;
    GemmParams p;
    default_params(p);
    p.M = M; p.N = N; p.K = K;
    p.C = (__nv_bfloat16*)c;
    p.ldc = ldc;
    p.bias = (const __nv_bfloat16*)bias;
    p.aux = (__nv_bfloat16*)aux;
    p.status = status;
    p.seg_rows = M;
    p.tiles_m = (M + BM - 1) / BM;
    p.tiles_n = (N + BN - 1) / BN;
    cudaStream_t st = (cudaStream_t)stream;
    return BN == 128 ? dispatch<128>(a_mn != 0, b_mn != 0, epi, tmA, tmB, p, sms, st)
                     : dispatch<256>(a_mn != 0, b_mn != 0, epi, tmA, tmB, p, sms, st);
}

// GEMM fused with a collective over peer memory (n ranks of one NVLink domain).  A is K-major.
//   a_mode 0: a_ptrs[0] is A[a_rows, K] (local), this rank's rows start at a_row_off.
//   a_mode 1: head -> sequence all-to-all fused into the operand fetch: a_ptrs[r] is rank r's
//             [a_rows, a_span] tensor holding K columns [r*a_span, (r+1)*a_span) for all rows; this rank's M rows
//             start at a_row_off in each of them (K == n * a_span).
//   a_mode 2: all-gather fused into the operand fetch: a_ptrs[r] is rank r's [seg_rows, K] row block; M == n * seg_rows.
//   b is B[N, K] (b_mn 0) or [K, N] (b_mn 1), always local.
//             With `stage` ([M, K], this GPU's memory) and `stage_flags` ([n * ceil(seg_rows / 128)] ints, zero at first
//             use) and a per-launch increasing `stage_epoch`, remote row blocks are copied into `stage` once by
//             dedicated warps and TMA-loaded from there, instead of crossing NVLink again for every N tile.
//   store_mode 0: C local.  1: column block j of width out_span goes to out_ptrs[j] (token rows out_row_off + row,
//             row pitch out_ld): the sequence -> head all-to-all of a data gradient.  2: row segment i goes to
//             out_ptrs[i] + my_rank * seg_rows * N: partial sums pushed to their owner (reduce-scatter; sum with
//             tt_partial_sum after a barrier).
//   a_extra (a_mode 1, optional): local [M, K - n * a_span] tensor (row pitch lda_extra) supplying the remaining K
//             columns.  With store_mode 1, output columns beyond n * out_span are stored to c (row pitch ldc).
extern "C" int tt_gemm_comm_bf16(void* const* a_ptrs, int n, int a_mode, long a_rows, int a_span, int a_row_off,
                                 const void* a_extra, long lda_extra, const void* b, int b_mn, long ldb, void* c,
                                 long ldc, const void* bias, int M, int N, int K, int seg_rows, int my_rank,
                                 int store_mode, void* const* out_ptrs, int out_span, int out_row_off, long out_ld,
                                 void* stage, int* stage_flags, int stage_epoch, int* status, void* stream) {
    if (n < 1 || n > TT_MAX_PEERS || M <= 0 || N <= 0 || K <= 0 || (N & 7) || (K & 7) || status == nullptr) return TT_ERR_ARG;
    if (a_mode < 0 || a_mode > 2 || store_mode < 0 || store_mode > 2 || my_rank < 0 || my_rank >= n) return TT_ERR_ARG;
    if (a_mode == 1 && ((a_span % BK) || (long)a_span * n > K)) return TT_ERR_ARG;
    if (a_mode == 1 && (long)a_span * n != K && a_extra == nullptr) return TT_ERR_ARG;
    const bool segmented = a_mode == 2 || store_mode == 2;
    if (segmented && (seg_rows <= 0 || (long)seg_rows * n != M)) return TT_ERR_ARG;
    if (store_mode == 0 && (c == nullptr || (ldc & 7))) return TT_ERR_ARG;
    if (store_mode != 0 && (out_ptrs == nullptr || (out_ld & 7))) return TT_ERR_ARG;
    if (store_mode == 1 && (out_span <= 0 || (out_span % 128) || (long)out_span * n > N)) return TT_ERR_ARG;
    if (store_mode == 1 && (long)out_span * n != N && (c == nullptr || (ldc & 7))) return TT_ERR_ARG;
    const int sms = sm_count();
    // a column block routed to one peer must not straddle two tiles' owners: 128-wide tiles when spans are 128-multiples
    const int BN = pick_bn(M, N, sms, store_mode == 1 && (out_span % 256) != 0);
    TmapArray tmA;
    CUtensorMap tmB;
    int rc;
    const int n_src = a_mode == 0 ? 1 : n;
    for (int r = 0; r < n_src; ++r) {
        const uint64_t rows = a_mode == 2 ? (uint64_t)seg_rows : (uint64_t)a_rows;
        const uint64_t cols = a_mode == 1 ? (uint64_t)a_span : (uint64_t)K;
        if ((rc = tt_make_tmap_2d(&tmA.m[r], a_ptrs[r], rows, cols, cols, BM, BK)) != TT_OK) return rc;
    }
    const bool staged = a_mode == 2 && stage != nullptr && stage_flags != nullptr && n > 1 && store_mode == 0 && !b_mn;
    if (staged) {
        if ((rc = tt_make_tmap_2d(&tmA.m[TT_MAX_PEERS], stage, (uint64_t)M, (uint64_t)K, (uint64_t)K, BM, BK)) != TT_OK) return rc;
    }
    if (a_mode == 1 && a_extra != nullptr) {
        const uint64_t cols = (uint64_t)K - (uint64_t)a_span * n;
        if ((rc = tt_make_tmap_2d(&tmA.m[TT_MAX_PEERS], a_extra, (uint64_t)M, cols, (uint64_t)lda_extra, BM, BK)) != TT_OK)
            return rc;
    }
    if (!b_mn) rc = tt_make_tmap_2d(&tmB, b, (uint64_t)N, (uint64_t)K, (uint64_t)ldb, (uint32_t)BN, BK);
    else rc = tt_make_tmap_2d(&tmB, b, (uint64_t)K, (uint64_t)N, (uint64_t)ldb, 64, 64);
    if (rc != TT_OK) return rc;
    GemmParams p;
    default_params(p);
    p.M = M; p.N = N; p.K = K;
    p.C = (__nv_bfloat16*)c;
    p.ldc = ldc;
    p.bias = (const __nv_bfloat16*)bias;
    p.status = status;
    p.a_mode = a_mode;
    p.a_span = a_span;
    p.a_nsrc = n;
    p.a_row_off = a_row_off;
    p.n_dest = n;
    p.n_seg = segmented ? n : 1;
    p.seg_rows = segmented ? seg_rows : M;
    p.seg_rot = segmented ? my_rank : 0;       // own rows first: they need no peer traffic
    p.my_rank = my_rank;
    p.store_mode = store_mode;
    p.coalesce = (store_mode != 0 && bias == nullptr) ? coalesced_peer_stores() : 0;
    p.out_span = out_span;
    p.out_row_off = out_row_off;
    p.out_ld = out_ld;
    if (store_mode != 0)
        for (int r = 0; r < n; ++r) p.peer_out[r] = (__nv_bfloat16*)out_ptrs[r];
    p.tiles_m = p.n_seg * ((p.seg_rows + BM - 1) / BM);
    p.tiles_n = (N + BN - 1) / BN;
    cudaStream_t st = (cudaStream_t)stream;
    if (staged) {
        p.stage = (__nv_bfloat16*)stage;
        p.stage_flags = stage_flags;
        p.stage_epoch = stage_epoch;
        for (int r = 0; r < n; ++r) p.peer_a[r] = (const __nv_bfloat16*)a_ptrs[r];
        return BN == 128 ? launch<128, false, false, 0, true>(tmA, tmB, p, sms, st)
                         : launch<256, false, false, 0, true>(tmA, tmB, p, sms, st);
    }
    const int epi = p.coalesce ? 6 : 0;          // 6 = bias epilogue with staged, coalesced peer stores
    return BN == 128 ? dispatch<128>(false, b_mn != 0, epi, tmA, tmB, p, sms, st)
                     : dispatch<256>(false, b_mn != 0, epi, tmA, tmB, p, sms, st);
}

// Tensor-parallel all-gather -> GEMM with the epilogues of the plain GEMM: C[n * seg_rows, N] = epi(gather_r(A_r) op(B) + bias).
//   a_ptrs[r]: rank r's [seg_rows, K] row block (peer memory); stage [n * seg_rows, K]: local buffer that receives the
//   gathered operand (filled by the kernel's copier warps, one crossing of NVLink per remote row block) and stays valid
//   after the call, so the caller can keep it for the weight gradient;  stage_flags [n * ceil(seg_rows / 128)] ints,
//   zero before the first call; stage_epoch: a value that differs from every earlier call on the same flags.
//   b_mn = 0: B is [N, K] (y = x W^T; epi 0 bias, 1 / 2 GELU erf / tanh with the pre-activation kept in aux);
//   b_mn = 1: B is [K, N] (dgrad of a row-parallel linear; epi 0 only).
extern "C" int tt_gemm_ag_bf16(void* const* a_ptrs, int n, int my_rank, int seg_rows, const void* b, int b_mn, long ldb,
                               void* c, long ldc, const void* bias, void* aux, int N, int K, int epi, void* stage,
                               int* stage_flags, int stage_epoch, int* status, void* stream) {
    if (n < 2 || n > TT_MAX_PEERS || my_rank < 0 || my_rank >= n || seg_rows <= 0 || N <= 0 || K <= 0 || (N & 7) || (K & 7))
        return TT_ERR_ARG;
    if (status == nullptr || stage == nullptr || stage_flags == nullptr || c == nullptr || (ldc & 7)) return TT_ERR_ARG;
    if (epi < 0 || epi > 2 || (epi != 0 && (aux == nullptr || b_mn))) return TT_ERR_ARG;
    const long M = (long)seg_rows * n;
    if (M > 0x7fffffffL) return TT_ERR_ARG;
    const int sms = sm_count();
    const int BN = pick_bn((int)M, N, sms, false);
    TmapArray tmA;
    CUtensorMap tmB;
    int rc;
    for (int r = 0; r < n; ++r)
        if ((rc = tt_make_tmap_2d(&tmA.m[r], a_ptrs[r], (uint64_t)seg_rows, (uint64_t)K, (uint64_t)K, BM, BK)) != TT_OK) return rc;
    if ((rc = tt_make_tmap_2d(&tmA.m[TT_MAX_PEERS], stage, (uint64_t)M, (uint64_t)K, (uint64_t)K, BM, BK)) != TT_OK) return rc;
    if (!b_mn) rc = tt_make_tmap_2d(&tmB, b, (uint64_t)N, (uint64_t)K, (uint64_t)ldb, (uint32_t)BN, BK);
    else rc = tt_make_tmap_2d(&tmB, b, (uint64_t)K, (uint64_t)N, (uint64_t)ldb, 64, 64);
    if (rc != TT_OK) return rc;
    GemmParams p;
    default_params(p);
    p.M = (int)M; p.N = N; p.K = K;
    p.C = (__nv_bfloat16*)c;
    p.ldc = ldc;
    p.bias = (const __nv_bfloat16*)bias;
    p.aux = (__nv_bfloat16*)aux;
    p.status = status;
    p.a_mode = 2;
    p.a_nsrc = n;
    p.n_dest = n;
    p.n_seg = n;
    p.seg_rows = seg_rows;
    p.seg_rot = my_rank;                       // own rows first: they need no peer traffic
    p.my_rank = my_rank;
    p.tiles_m = n * ((seg_rows + BM - 1) / BM);
    p.tiles_n = (N + BN - 1) / BN;
    p.stage = (__nv_bfloat16*)stage;
    p.stage_flags = stage_flags;
    p.stage_epoch = stage_epoch;
    for (int r = 0; r < n; ++r) p.peer_a[r] = (const __nv_bfloat16*)a_ptrs[r];
    cudaStream_t st = (cudaStream_t)stream;
    if (b_mn) return BN == 128 ? launch<128, false, true, 0, true>(tmA, tmB, p, sms, st)
                               : launch<256, false, true, 0, true>(tmA, tmB, p, sms, st);
    if (epi == 1) return BN == 128 ? launch<128, false, false, 1, true>(tmA, tmB, p, sms, st)
                                   : launch<256, false, false, 1, true>(tmA, tmB, p, sms, st);
    if (epi == 2) return BN == 128 ? launch<128, false, false, 2, true>(tmA, tmB, p, sms, st)
                                   : launch<256, false, false, 2, true>(tmA, tmB, p, sms, st);
    return BN == 128 ? launch<128, false, false, 0, true>(tmA, tmB, p, sms, st)
                     : launch<256, false, false, 0, true>(tmA, tmB, p, sms, st);
}

// QKV projection with everything after it fused into the epilogue: bias, QK-RMSNorm, RoPE, and the Ulysses
// sequence -> head all-to-all (each 128-column tile is one head's q, k or v and is stored straight into the
// [batch, heads_per_rank, s_out, 128] buffer of the rank that owns the head, at token offset out_off).
//   x [M, K] local tokens (M = batch * s_in), w [heads*384, K] with rows ordered [head][q|k|v][128];
//   q_ptrs / k_ptrs / v_ptrs [n]: destination buffers per owner rank (n = 1: local only);
//   only_local != 0: compute every head but store only the heads this rank owns (replicated text tokens);
//   aux (optional) [M, heads*384]: raw projection output, kept for the backward pass.
extern "C" int tt_qkv_gemm_fused(const void* x, const void* w, const void* bias, const void* qw, const void* kw,
                                 const float* cos_t, const float* sin_t, void* const* q_ptrs, void* const* k_ptrs,
                                 void* const* v_ptrs, int n, int my_rank, void* aux, int M, int heads, int K, int s_in,
                                 int s_out, int out_off, int rope_len, int only_local, float eps, int* status,
                                 void* stream) {
    if (n < 1 || n > TT_MAX_PEERS || my_rank < 0 || my_rank >= n || M <= 0 || heads <= 0 || heads % n || (K & 7)) return TT_ERR_ARG;
    if (s_in <= 0 || M % s_in || out_off < 0 || out_off + s_in > s_out || status == nullptr) return TT_ERR_ARG;
    if (rope_len > 0 && (cos_t == nullptr || sin_t == nullptr)) return TT_ERR_ARG;
    const int N = heads * 384;
    TmapArray tmA;
    CUtensorMap tmB;
    int rc;
    if ((rc = tt_make_tmap_2d(&tmA.m[0], x, (uint64_t)M, (uint64_t)K, (uint64_t)K, BM, BK)) != TT_OK) return rc;
    // 256-wide tiles (two heads per tile) run the tensor core at full rate; 128-wide ones only pay off when the
    // problem has too few tiles to fill the SMs otherwise
    const int BN = pick_bn(M, N, sm_count(), false);
    if ((rc = tt_make_tmap_2d(&tmB, w, (uint64_t)N, (uint64_t)K, (uint64_t)K, (uint32_t)BN, BK)) != TT_OK) return rc;
    GemmParams p;
    default_params(p);
    p.M = M; p.N = N; p.K = K;
    p.ldc = N;
    p.bias = (const __nv_bfloat16*)bias;
    p.aux = (__nv_bfloat16*)aux;
    p.status = status;
    p.seg_rows = M;
    p.my_rank = my_rank;
    p.qw = (const __nv_bfloat16*)qw;
    p.kw = (const __nv_bfloat16*)kw;
    p.cos_t = cos_t;
    p.sin_t = sin_t;
    p.eps = eps;
    p.rope_len = rope_len;
    p.heads_per_rank = heads / n;
    p.s_in = s_in;
    p.s_out = s_out;
    p.out_off = out_off;
    p.only_local = only_local;
    for (int r = 0; r < n; ++r) {
        p.peer_q[r] = (__nv_bfloat16*)q_ptrs[r];
        p.peer_k[r] = (__nv_bfloat16*)k_ptrs[r];
        p.peer_v[r] = (__nv_bfloat16*)v_ptrs[r];
    }
    p.tiles_m = (M + BM - 1) / BM;
    p.tiles_n = (N + BN - 1) / BN;
    return BN == 128 ? dispatch<128>(false, false, 5, tmA, tmB, p, sm_count(), (cudaStream_t)stream)
                     : dispatch<256>(false, false, 5, tmA, tmB, p, sm_count(), (cudaStream_t)stream);
}
