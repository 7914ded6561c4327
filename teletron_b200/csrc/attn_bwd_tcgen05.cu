// Flash attention backward on tcgen05 / TMEM (head dim 128, non-causal, key-length mask), split into two
// atomics-free, deterministic kernels built from one template:
//
//   KV-stationary (dK, dV): a CTA owns 128 keys (K, V tiles resident in shared memory) and streams the
//     queries in chunks of 64 rows (Q, dO).   T1 = K Q^T = S^T,  T2 = V dO^T = dP^T,
//     P^T = exp2(S^T * c - lse[q]),  dS^T = P^T * (dP^T - delta[q]),  dV += P^T dO,  dK += dS^T Q.
//   Q-stationary (dQ): a CTA owns 128 queries (Q, dO resident) and streams the keys in chunks of 64
//     (K, V).   T1 = Q K^T = S,  T2 = dO V^T = dP,  dS = exp2(S * c - lse[row]) * (dP - delta[row]),
//     dQ += dS K.
//
// Both run the same pipeline.  Stationary operands [128 x 128] are loaded once; streamed chunks
// [64 x 128] x 2 go through a 4-stage TMA ring.  T1 / T2 (128 x 64 fp32 each) are double buffered in
// tensor memory, so the tensor core computes the next chunk's T products and the previous chunk's
// accumulator updates while the eight softmax warps (one stationary row x 32 streamed columns per thread) turn the current
// T1 / T2 into bf16 P / dS, written back over T1 / T2 in tensor memory and consumed from there as the
// A operand of the accumulator MMAs.  The streamed chunk is used twice from the same shared-memory bytes:
// as a K-major B operand for the T products and as an MN-major B operand for the accumulator updates.
//
//   TMEM columns: [0,64) T1 buf0 (P0 aliases [0,32)), [64,128) T2 buf0 (dS0 aliases [64,96)),
//                 [128,192) T1 buf1, [192,256) T2 buf1, [256,384) accumulator 1, [384,512) accumulator 2.
//
// q, k, v, dq, dk, dv: [B*H, S, 128] bf16 head-major; dout: [B, S, H*128] bf16 token-major;
// lse, delta: [B*H, pitch] fp32 (delta = rowsum(dO * O), computed by the preprocess kernel below).
// The reference gets this from torch SDPA's backward (teletron/models/dit/dit_attention.py:313).
#include "common.cuh"
#include "sm100.cuh"
#include "teletron_b200.h"

namespace {

using namespace sm100;

constexpr int D = 128;
constexpr int BS = 128;            // stationary rows
constexpr int BC = 64;             // streamed rows per chunk
constexpr int kStages = 4;
constexpr int kThreads = 320;      // warp 0 TMA, warp 1 MMA, warps 2-9 softmax / epilogue (two warpgroups)
constexpr int kStatSlab = BS * 128;        // [128 x 64] slab: 16 KB
constexpr int kStatTile = 2 * kStatSlab;   // [128 x 128]: 32 KB
constexpr int kChunkSlab = BC * 128;       // [64 x 64] slab: 8 KB
constexpr int kChunkTile = 2 * kChunkSlab; // [64 x 128]: 16 KB
constexpr int kStageBytes = 2 * kChunkTile;   // two streamed operands per stage: 32 KB
constexpr int kSmemBytes = 2 * kStatTile + kStages * kStageBytes + 1024 /* stats */ + 256 /* barriers */ + 1024;
constexpr float kLog2e = 1.4426950408889634f;

struct BwdParams {
    __nv_bfloat16* out1;    // KV-stationary: dV; Q-stationary: dQ
    __nv_bfloat16* out2;    // KV-stationary: dK
    const float* lse;       // [BH, pitch]; entries at and beyond S hold +inf
    const float* delta;     // [BH, pitch]; entries at and beyond S hold 0
    int S, kv_len, H;
    int pitch;              // multiple of 64, so every 64-query chunk of statistics is 16-byte aligned
    float scale;            // softmax scale
    int* status;
};

// delta[bh, s] = sum_d dO[b, s, h, d] * O[b, s, h, d]; one warp per (token, head)
__global__ void __launch_bounds__(256) delta_kernel(const __nv_bfloat16* __restrict__ dout, const __nv_bfloat16* __restrict__ out,
                                                   float* __restrict__ delta, int B, int S, int H, int pitch) {
    const int lane = threadIdx.x & 31;
    const long nwork = (long)B * S * H;
    for (long w = (long)blockIdx.x * 8 + (threadIdx.x >> 5); w < nwork; w += (long)gridDim.x * 8) {
        const long tok = w / H;
        const int h = (int)(w - tok * H);
        const long b = tok / S, s = tok - b * S;
        const uint2 a = *reinterpret_cast<const uint2*>(dout + w * D + lane * 4);
        const uint2 o = *reinterpret_cast<const uint2*>(out + w * D + lane * 4);
        const float2 a0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&a.x));
        const float2 a1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&a.y));
        const float2 o0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&o.x));
        const float2 o1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&o.y));
        float v = a0.x * o0.x + a0.y * o0.y + a1.x * o1.x + a1.y * o1.y;
        v = tt::warp_sum(v);
        if (lane == 0) delta[(b * H + h) * pitch + s] = v;
    }
}

template <bool KVS>
__global__ void __launch_bounds__(kThreads, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO, const BwdParams p) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ volatile int abort_flag;
    __shared__ uint32_t tmem_base_slot;

    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t sA1 = base;                       // stationary operand 1 (K or Q)
    const uint32_t sA2 = base + kStatTile;           // stationary operand 2 (V or dO)
    const uint32_t sRing = base + 2 * kStatTile;     // stage: [B1 chunk (Q or K) | B2 chunk (dO or V)]
    const uint32_t bars = base + 2 * kStatTile + kStages * kStageBytes + 1024;
    const uint32_t a_full = bars;
    auto b_full = [&](int s) { return bars + 8u * (1 + s); };
    auto b_empty = [&](int s) { return bars + 8u * (1 + kStages + s); };
    auto t_full = [&](int u) { return bars + 8u * (1 + 2 * kStages + u); };
    auto p_full = [&](int u) { return bars + 8u * (3 + 2 * kStages + u); };
    const uint32_t acc_final = bars + 8u * (5 + 2 * kStages);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int bh = blockIdx.y;
    const int b = bh / p.H, head = bh - b * p.H;
    const int r0 = blockIdx.x * BS;                                     // first stationary row
    const int stream_len = KVS ? p.S : p.kv_len;                        // rows streamed (queries / keys)
    const int n_chunks = (stream_len + BC - 1) / BC;

    if (threadIdx.x == 0) {
        abort_flag = 0;
        mbar_init(a_full, 1);
        for (int s = 0; s < kStages; ++s) {
            mbar_init(b_full(s), 1);
            mbar_init(b_empty(s), 1);
        }
        for (int u = 0; u < 2; ++u) {
            mbar_init(t_full(u), 1);
            mbar_init(p_full(u), 8);
        }
        mbar_init(acc_final, 1);
        fence_barrier_init();
        fence_proxy_async();
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(&tmem_base_slot), 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_base_slot;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            mbar_arrive_expect_tx(a_full, 2 * kStatTile);
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                if (KVS) {
                    tma_load_3d(sA1 + h * kStatSlab, &tmK, a_full, h * 64, r0, bh);
                    tma_load_3d(sA2 + h * kStatSlab, &tmV, a_full, h * 64, r0, bh);
                } else {
                    tma_load_3d(sA1 + h * kStatSlab, &tmQ, a_full, h * 64, r0, bh);
                    tma_load_4d(sA2 + h * kStatSlab, &tmDO, a_full, h * 64, head, r0, b);
                }
            }
            for (int c = 0; c < n_chunks; ++c) {
                const int s = c % kStages;
                const uint32_t ph = (uint32_t)(c / kStages) & 1u;
                if (!mbar_wait(b_empty(s), ph ^ 1u, &abort_flag)) goto done;
                mbar_arrive_expect_tx(b_full(s), kStageBytes);
                const uint32_t dst = sRing + s * kStageBytes;
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    if (KVS) {
                        tma_load_3d(dst + h * kChunkSlab, &tmQ, b_full(s), h * 64, c * BC, bh);
                        tma_load_4d(dst + kChunkTile + h * kChunkSlab, &tmDO, b_full(s), h * 64, head, c * BC, b);
                    } else {
                        tma_load_3d(dst + h * kChunkSlab, &tmK, b_full(s), h * 64, c * BC, bh);
                        tma_load_3d(dst + kChunkTile + h * kChunkSlab, &tmV, b_full(s), h * 64, c * BC, bh);
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc_t = idesc_bf16(BS, BC, false, false);   // T = A B^T, both K-major, N = 64
            constexpr uint32_t idesc_a = idesc_bf16(BS, D, false, true);     // acc += P B, B MN-major, N = 128
            auto issue_t = [&](int c) {
                const int u = c & 1;
                const uint32_t sb = sRing + (c % kStages) * kStageBytes;
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) {
                    const uint32_t oa = (kk >> 2) * kStatSlab + (kk & 3) * 32;
                    const uint32_t ob = (kk >> 2) * kChunkSlab + (kk & 3) * 32;
                    umma_bf16_ss(tmem + u * 128, smem_desc_sw128(sA1 + oa, 16, 1024), smem_desc_sw128(sb + ob, 16, 1024),
                                 idesc_t, kk ? 1u : 0u);
                }
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) {
                    const uint32_t oa = (kk >> 2) * kStatSlab + (kk & 3) * 32;
                    const uint32_t ob = (kk >> 2) * kChunkSlab + (kk & 3) * 32;
                    umma_bf16_ss(tmem + u * 128 + 64, smem_desc_sw128(sA2 + oa, 16, 1024),
                                 smem_desc_sw128(sb + kChunkTile + ob, 16, 1024), idesc_t, kk ? 1u : 0u);
                }
                umma_commit(t_full(u));
            };
            auto issue_acc = [&](int c) {
                const int u = c & 1;
                const uint32_t sb = sRing + (c % kStages) * kStageBytes;
                if (KVS) {
                    // dV += P^T dO  (P at T1 columns, B = dO chunk)
#pragma unroll
                    for (int kk = 0; kk < BC / 16; ++kk)
                        umma_bf16_ts(tmem + 256, tmem + u * 128 + kk * 8,
                                     smem_desc_sw128(sb + kChunkTile + kk * 2048, kChunkSlab, 1024), idesc_a, (c | kk) ? 1u : 0u);
                }
                // dK += dS^T Q   /   dQ += dS K   (dS at T2 columns, B = first streamed operand)
#pragma unroll
                for (int kk = 0; kk < BC / 16; ++kk)
                    umma_bf16_ts(tmem + (KVS ? 384 : 256), tmem + u * 128 + 64 + kk * 8,
                                 smem_desc_sw128(sb + kk * 2048, kChunkSlab, 1024), idesc_a, (c | kk) ? 1u : 0u);
                umma_commit(b_empty(c % kStages));
            };
            if (!mbar_wait(a_full, 0, &abort_flag)) goto done;
            for (int c = 0; c < 2 && c < n_chunks; ++c) {
                if (!mbar_wait(b_full(c % kStages), 0, &abort_flag)) goto done;
                tc_fence_after();
                issue_t(c);
            }
            for (int c = 0; c < n_chunks; ++c) {
                if (!mbar_wait(p_full(c & 1), (uint32_t)(c >> 1) & 1u, &abort_flag)) goto done;
                tc_fence_after();
                issue_acc(c);
                if (c + 2 < n_chunks) {
                    const int c2 = c + 2;
                    if (!mbar_wait(b_full(c2 % kStages), (uint32_t)(c2 / kStages) & 1u, &abort_flag)) goto done;
                    tc_fence_after();
                    issue_t(c2);
                }
            }
            umma_commit(acc_final);
        }
    } else {
        // ------------------------------------------------------------ softmax / dS
        // Two warpgroups share every chunk: a thread owns one stationary row and 32 of the chunk's 64 streamed
        // columns (warpgroup 0: columns [0, 32), warpgroup 1: [32, 64)), so two warps per scheduler hide each
        // other's tcgen05.ld / exp2 latency.
        const int half = (warp - 2) >> 2;
        const int quad = warp & 3;
        const int srow = quad * 32 + lane;                 // row within the stationary tile
        const int row = r0 + srow;                         // key (KVS) or query index
        const uint32_t lane_sel = (uint32_t)(quad * 32) << 16;
        const float c_log2 = p.scale * kLog2e;
        float my_lse = 0.f, my_delta = 0.f;
        bool row_live;
        if (KVS) {
            row_live = row < p.kv_len;
        } else {
            row_live = row < p.S;
            my_lse = row_live ? p.lse[(long)bh * p.pitch + row] * kLog2e : INFINITY;
            my_delta = row_live ? p.delta[(long)bh * p.pitch + row] : 0.f;
        }
        for (int c = 0; c < n_chunks; ++c) {
            const int u = c & 1;
            const int col0 = c * BC;
            // KV-stationary: the chunk's 64 queries each have their own lse / delta; every thread reads them
            // straight from global memory (same addresses across the warp, so each load is one broadcast)
            const float4* lse4 = reinterpret_cast<const float4*>(p.lse + (long)bh * p.pitch + col0);
            const float4* del4 = reinterpret_cast<const float4*>(p.delta + (long)bh * p.pitch + col0);
            if (!mbar_wait(t_full(u), (uint32_t)(c >> 1) & 1u, &abort_flag)) goto done;
            tc_fence_after();
            const uint32_t t1 = tmem + lane_sel + u * 128, t2 = t1 + 64;
            uint32_t pk[16], dk[16];
            {
                uint32_t a[32], g[32];
                tmem_ld_32x32(t1 + half * 32, a);
                tmem_ld_32x32(t2 + half * 32, g);
                tmem_ld_wait();
                float4 lq[8], dq4[8];
                if (KVS) {
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        lq[i] = __ldg(lse4 + half * 8 + i);
                        dq4[i] = __ldg(del4 + half * 8 + i);
                    }
                }
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const int cc = half * 32 + 2 * i;
                    float2 l2, d2;
                    if (KVS) {
                        const float4 lv = lq[i >> 1], dv = dq4[i >> 1];
                        l2 = (i & 1) ? make_float2(lv.z * kLog2e, lv.w * kLog2e) : make_float2(lv.x * kLog2e, lv.y * kLog2e);
                        d2 = (i & 1) ? make_float2(dv.z, dv.w) : make_float2(dv.x, dv.y);
                    } else {
                        l2 = make_float2(my_lse, my_lse);
                        d2 = make_float2(my_delta, my_delta);
                    }
                    const float2 x = __ffma2_rn(make_float2(__uint_as_float(a[2 * i]), __uint_as_float(a[2 * i + 1])),
                                                make_float2(c_log2, c_log2), make_float2(-l2.x, -l2.y));
                    float2 pr = make_float2(exp2f(x.x), exp2f(x.y));
                    if (KVS) {
                        if (!row_live) pr = make_float2(0.f, 0.f);
                    } else {
                        if (col0 + cc >= p.kv_len) pr.x = 0.f;
                        if (col0 + cc + 1 >= p.kv_len) pr.y = 0.f;
                    }
                    const float2 dp = make_float2(__uint_as_float(g[2 * i]) - d2.x, __uint_as_float(g[2 * i + 1]) - d2.y);
                    const float2 ds = __fmul2_rn(pr, dp);
                    const __nv_bfloat162 pb = __floats2bfloat162_rn(pr.x, pr.y);
                    const __nv_bfloat162 db = __floats2bfloat162_rn(ds.x, ds.y);
                    pk[i] = *reinterpret_cast<const uint32_t*>(&pb);
                    dk[i] = *reinterpret_cast<const uint32_t*>(&db);
                }
            }
            if (KVS) tmem_st_32x16(t1 + half * 16, pk);
            tmem_st_32x16(t2 + half * 16, dk);
            tmem_st_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(p_full(u));
        }
        // ------------------------------------------------------------ epilogue
        if (!mbar_wait(acc_final, 0, &abort_flag)) goto done;
        tc_fence_after();
        const bool store = row < p.S;
        const long orow = ((long)bh * p.S + row) * D;
#pragma unroll 1
        for (int which = 0; which < (KVS ? 2 : 1); ++which) {
            __nv_bfloat16* dst = (which == 0 ? p.out1 : p.out2) + orow;
            // dV is unscaled; dK and dQ carry the softmax scale
            const float mul = (KVS && which == 0) ? 1.f : p.scale;
            const uint32_t tacc = tmem + lane_sel + 256 + which * 128;
#pragma unroll 1
            for (int cch = half * 2; cch < half * 2 + 2; ++cch) {      // each warpgroup stores half of the columns
                uint32_t r[32];
                tmem_ld_32x32(tacc + cch * 32, r);
                tmem_ld_wait();
                if (store) {
#pragma unroll
                    for (int g = 0; g < 4; ++g) {
                        float o[8];
#pragma unroll
                        for (int i = 0; i < 8; ++i) o[i] = __uint_as_float(r[g * 8 + i]) * mul;
                        tt::st8(dst + cch * 32 + g * 8, tt::pack8(o));
                    }
                }
            }
        }
    }

done:
    tc_fence_before();
    __syncthreads();
    if (abort_flag) {
        if (threadIdx.x == 0) atomicExch(p.status, TT_ERR_TIMEOUT);
        for (int i = 0; i < 200; ++i) __nanosleep(1000);
    }
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem, 512);
    }
}

}  // namespace

// lse, delta: [B*H, pitch] fp32 with pitch a multiple of 64; lse holds +inf and delta 0 at positions >= S
// (delta is scratch owned by the caller, zero-initialised; this call fills positions < S).
extern "C" int tt_attn_bwd(const void* q, const void* k, const void* v, const void* out, const void* dout,
                           const float* lse, float* delta, void* dq, void* dk, void* dv, int B, int H, int S, int kv_len,
                           int pitch, float scale, int* status, void* stream) {
    if (B <= 0 || H <= 0 || S <= 0 || kv_len <= 0 || kv_len > S || status == nullptr || delta == nullptr) return TT_ERR_ARG;
    if (pitch < S || (pitch & 63) || ((uintptr_t)lse & 15) || ((uintptr_t)delta & 15)) return TT_ERR_ARG;
    cudaStream_t st = (cudaStream_t)stream;
    const uint64_t BH = (uint64_t)B * H;
    CUtensorMap tq_s, tk_s, tv_s, tdo_s;     // 128-row boxes (stationary operands)
    CUtensorMap tq_c, tk_c, tv_c, tdo_c;     // 64-row boxes (streamed chunks)
    int rc;
    if ((rc = tt_make_tmap_3d(&tq_s, q, BH, (uint64_t)S, D, D, (uint64_t)S * D, BS, 64)) != TT_OK) return rc;
    if ((rc = tt_make_tmap_3d(&tk_s, k, BH, (uint64_t)S, D, D, (uint64_t)S * D, BS, 64)) != TT_OK) return rc;
    if ((rc = tt_make_tmap_3d(&tv_s, v, BH, (uint64_t)S, D, D, (uint64_t)S * D, BS, 64)) != TT_OK) return rc;
    if ((rc = tt_make_tmap_bshd(&tdo_s, dout, (uint64_t)B, (uint64_t)S, (uint64_t)H, BS)) != TT_OK) return rc;
    if ((rc = tt_make_tmap_3d(&tq_c, q, BH, (uint64_t)S, D, D, (uint64_t)S * D, BC, 64)) != TT_OK) return rc;
    if ((rc = tt_make_tmap_3d(&tk_c, k, BH, (uint64_t)S, D, D, (uint64_t)S * D, BC, 64)) != TT_OK) return rc;
    if ((rc = tt_make_tmap_3d(&tv_c, v, BH, (uint64_t)S, D, D, (uint64_t)S * D, BC, 64)) != TT_OK) return rc;
    if ((rc = tt_make_tmap_bshd(&tdo_c, dout, (uint64_t)B, (uint64_t)S, (uint64_t)H, BC)) != TT_OK) return rc;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attn_bwd_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute(attn_bwd_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
        if (e != cudaSuccess) return tt_record_cuda(e);
        configured = true;
    }
    const long nwork = (long)B * S * H;
    long want = (nwork + 7) / 8;
    delta_kernel<<<(int)(want < 148L * 16 ? want : 148L * 16), 256, 0, st>>>((const __nv_bfloat16*)dout,
                                                                            (const __nv_bfloat16*)out, delta, B, S, H, pitch);
    TT_CHECK_LAUNCH();
    BwdParams p;
    p.lse = lse;
    p.delta = delta;
    p.S = S;
    p.kv_len = kv_len;
    p.H = H;
    p.pitch = pitch;
    p.scale = scale;
    p.status = status;
    // dK, dV: stationary keys (K, V resident), streamed queries (Q, dO)
    p.out1 = (__nv_bfloat16*)dv;
    p.out2 = (__nv_bfloat16*)dk;
    attn_bwd_kernel<true><<<dim3((S + BS - 1) / BS, (unsigned)BH), kThreads, kSmemBytes, st>>>(tq_c, tk_s, tv_s, tdo_c, p);
    TT_CHECK_LAUNCH();
    // dQ: stationary queries (Q, dO resident), streamed keys (K, V)
    p.out1 = (__nv_bfloat16*)dq;
    p.out2 = nullptr;
    attn_bwd_kernel<false><<<dim3((S + BS - 1) / BS, (unsigned)BH), kThreads, kSmemBytes, st>>>(tq_s, tk_c, tv_c, tdo_s, p);
    TT_CHECK_LAUNCH();
    return TT_OK;
}
