// Flash attention backward on tcgen05 / TMEM (head dim 128, non-causal, key-length mask).  Two variants share this file:
// the one-pass kernel further down (attn_bwd_fused_kernel: five products per tile pair, dQ reduced in fp32 by the TMA
// unit; what the Python layer calls by default) and, described first, the split into two atomics-free, deterministic
// kernels built from one template (seven products per tile pair):
//
//   KV-stationary (dK, dV): a CTA owns 128 keys (K, V tiles resident in shared memory) and streams the
//     queries in chunks of 128 rows (Q, dO).   T1 = K Q^T = S^T,  T2 = V dO^T = dP^T,
//     P^T = exp2(S^T * c - lse[q]),  dS^T = P^T * (dP^T - delta[q]),  dV += P^T dO,  dK += dS^T Q.
//   Q-stationary (dQ): a CTA owns 128 queries (Q, dO resident) and streams the keys in chunks of 128
//     (K, V).   T1 = Q K^T = S,  T2 = dO V^T = dP,  dS = exp2(S * c - lse[row]) * (dP - delta[row]),
//     dQ += dS K.
//
// Both run the same pipeline.  Stationary operands [128 x 128] are loaded once; streamed chunks are 128 rows,
// held in two TMA rings (three slots for the operand that the score product needs early and dK / dQ needs last,
// two for the other).  Chunks of 128 keep every MMA at N = 128: an N = 64 instruction was measured to take as long
// as an N = 128 one on this part.  T1 and T2 are single-buffered in tensor memory; the overlap comes from keeping P
// in registers between the two softmax passes, so that T1 is free for the next chunk's scores while dS is formed:
//
//   tensor core:  S(c+1) ......... | dK(c) dV(c) dP(c+1) | S(c+2) ........ | dK(c+1) ...
//   softmax:      dS(c) .......... | P(c+1) ............ | dS(c+1) ....... | P(c+2) ...
//
// The sixteen softmax warps (one stationary row x 32 streamed columns per thread) read S from T1 and keep bf16 P in
// registers (the special-function unit's 16 exp2 per clock make this pass ~1250 clocks per chunk), then read dP from
// T2 and write bf16 P and dS back over the dP columns they have just read; both are consumed from tensor memory as
// the A operand of the accumulator MMAs.  dP(c+1) may overwrite T2 as soon as dK(c) / dV(c) have consumed it; the
// tensor core executes in issue order, so that hazard needs no extra barrier.  A streamed chunk is used twice from
// the same shared-memory bytes: as a K-major B operand for the T products and as an MN-major B operand for the
// accumulator updates.
//
//   TMEM columns: [0,128) T1 = S, [128,256) T2 = dP (of every 32 columns, P aliases the first 16 and dS the last 16),
//                 [256,384) accumulator 1, [384,512) accumulator 2.
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
constexpr int BC = 128;            // streamed rows per chunk
constexpr int kRing1 = 3;           // slots of the first streamed operand (Q or K): used by the score product and, last, by dK / dQ
constexpr int kRing2 = 2;           // slots of the second streamed operand (dO or V)
constexpr int kGroups = 4;         // softmax warpgroups: each owns 128 / kGroups streamed columns of every chunk
constexpr int kCols = BC / kGroups; // 32: one tcgen05.ld per pass and thread
constexpr int kThreads = 64 + 128 * kGroups;   // warp 0 TMA, warp 1 MMA, then the softmax / epilogue warpgroups
constexpr int kSlab = 128 * 128;           // [128 rows x 64 columns] bf16 slab, 128-byte rows: 16 KB
constexpr int kTile = 2 * kSlab;           // [128 x 128]: 32 KB
constexpr int kSmemBytes = (2 + kRing1 + kRing2) * kTile + 256 /* barriers */ + 1024 /* alignment */;   // 225.3 KB
constexpr float kLog2e = 1.4426950408889634f;

struct BwdParams {
    __nv_bfloat16* out1;    // KV-stationary: dV; Q-stationary: dQ
    __nv_bfloat16* out2;    // KV-stationary: dK
    const float* lse;       // [BH, pitch]; entries at and beyond S hold +inf
    const float* delta;     // [BH, pitch]; entries at and beyond S hold 0
    int S, kv_len, H;
    int mask_lo, mask_hi;   // keys in [mask_lo, mask_hi) are masked in addition to those at and beyond kv_len
    int pitch;              // multiple of 64, so every 64-query chunk of statistics is 16-byte aligned
    float scale;            // softmax scale
    int* status;
    const __nv_bfloat16* q_raw;     // q [BH, S, 128] and dout [B, S, H * 128] as plain pointers: the variant that keeps the
    const __nv_bfloat16* do_raw;    // stationary operands in tensor memory loads them with ordinary loads
    float* dq_acc;                  // one-pass variant: fp32 [B*H, s_pad, 128] accumulator for dQ (zeroed by the launcher)
    int s_pad;                      // rows per head in dq_acc: S rounded up to a multiple of 128
#ifdef TT_ATTN_STAMPS
    long long* stamps;              // scratch builds only: clock64() of CTA (0, 0)'s pipeline events, [chunk][10]
#endif
};

#ifdef TT_ATTN_STAMPS
#define TT_STAMP(slot) do { if (p.stamps != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && c < 256) p.stamps[c * 10 + (slot)] = clock64(); } while (0)
#define TT_STAMPF(slot) do { if (p.stamps != nullptr && blockIdx.x == 0 && blockIdx.y == 0 && c < 256) p.stamps[c * 16 + (slot)] = clock64(); } while (0)
#else
#define TT_STAMP(slot) do { } while (0)
#define TT_STAMPF(slot) do { } while (0)
#endif

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

// TSA (query-stationary only): the stationary operands Q and dO live in tensor memory (bf16 pairs, columns [384, 512),
// free in that kernel) instead of shared memory, so the score-type products become TS instructions.  An SS instruction
// with N = 128 was measured at ~128 clocks on this part, a TS one at ~84.
template <bool KVS, bool TSA = false>
__global__ void __launch_bounds__(kThreads, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO, const BwdParams p) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ volatile int abort_flag;
    __shared__ uint32_t tmem_base_slot;

    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t sA1 = base;                       // stationary operand 1 (K or Q)
    const uint32_t sA2 = base + kTile;               // stationary operand 2 (V or dO)
    const uint32_t sRing1 = base + 2 * kTile;                        // slots of streamed operand 1 (Q or K)
    const uint32_t sRing2 = sRing1 + kRing1 * kTile;                 // slots of streamed operand 2 (dO or V)
    const uint32_t bars = sRing2 + kRing2 * kTile;
    const uint32_t a_full = bars;
    auto b1_full = [&](int s) { return bars + 8u * (1 + s); };
    auto b1_empty = [&](int s) { return bars + 8u * (1 + kRing1 + s); };
    auto b2_full = [&](int s) { return bars + 8u * (1 + 2 * kRing1 + s); };
    auto b2_empty = [&](int s) { return bars + 8u * (1 + 2 * kRing1 + kRing2 + s); };
    const uint32_t s_full = bars + 8u * (1 + 2 * kRing1 + 2 * kRing2);   // T1 = S holds this chunk's scores
    const uint32_t dp_full = s_full + 8u;                      // T2 = dP holds this chunk's products
    const uint32_t p_ready = s_full + 16u;                     // every softmax warp has read S (P is in registers)
    const uint32_t ds_ready = s_full + 24u;                    // P and dS have been written over dP
    const uint32_t acc_final = s_full + 32u;

    static_assert(!(KVS && TSA), "the key-stationary kernel has no free tensor-memory columns");
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int bh = blockIdx.y;
    const int b = bh / p.H, head = bh - b * p.H;
    const int r0 = blockIdx.x * BS;                                     // first stationary row
    const int stream_len = KVS ? p.S : p.kv_len;                        // rows streamed (queries / keys)
    const int n_chunks = (stream_len + BC - 1) / BC;

    if (threadIdx.x == 0) {
        abort_flag = 0;
        mbar_init(a_full, TSA ? 4 * kGroups : 1);
        for (int s = 0; s < kRing1; ++s) {
            mbar_init(b1_full(s), 1);
            mbar_init(b1_empty(s), 1);
        }
        for (int s = 0; s < kRing2; ++s) {
            mbar_init(b2_full(s), 1);
            mbar_init(b2_empty(s), 1);
        }
        mbar_init(s_full, 1);
        mbar_init(dp_full, 1);
        mbar_init(p_ready, 4 * kGroups);
        mbar_init(ds_ready, 4 * kGroups);
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
    constexpr uint32_t kT1 = 0, kT2 = 128, kAcc1 = 256, kAcc2 = 384;
    constexpr uint32_t kA1 = 384, kA2 = 448;          // TSA: Q and dO as bf16 pairs, 64 columns each

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            if (!TSA) mbar_arrive_expect_tx(a_full, 2 * kTile);
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                if (TSA) break;
                if (KVS) {
                    tma_load_3d(sA1 + h * kSlab, &tmK, a_full, h * 64, r0, bh);
                    tma_load_3d(sA2 + h * kSlab, &tmV, a_full, h * 64, r0, bh);
                } else {
                    tma_load_3d(sA1 + h * kSlab, &tmQ, a_full, h * 64, r0, bh);
                    tma_load_4d(sA2 + h * kSlab, &tmDO, a_full, h * 64, head, r0, b);
                }
            }
            for (int c = 0; c < n_chunks; ++c) {
                const int s1 = c % kRing1, s2 = c % kRing2;
                if (!mbar_wait(b1_empty(s1), ((uint32_t)(c / kRing1) & 1u) ^ 1u, &abort_flag)) goto done;
                mbar_arrive_expect_tx(b1_full(s1), kTile);
                const uint32_t d1 = sRing1 + s1 * kTile;
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    if (KVS) tma_load_3d(d1 + h * kSlab, &tmQ, b1_full(s1), h * 64, c * BC, bh);
                    else tma_load_3d(d1 + h * kSlab, &tmK, b1_full(s1), h * 64, c * BC, bh);
                }
                if (!mbar_wait(b2_empty(s2), ((uint32_t)(c / kRing2) & 1u) ^ 1u, &abort_flag)) goto done;
                mbar_arrive_expect_tx(b2_full(s2), kTile);
                const uint32_t d2 = sRing2 + s2 * kTile;
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    if (KVS) tma_load_4d(d2 + h * kSlab, &tmDO, b2_full(s2), h * 64, head, c * BC, b);
                    else tma_load_3d(d2 + h * kSlab, &tmV, b2_full(s2), h * 64, c * BC, bh);
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc_t = idesc_bf16(BS, BC, false, false);   // T = A B^T, both K-major
            constexpr uint32_t idesc_a = idesc_bf16(BS, D, false, true);     // acc += P B, B MN-major
            // T[128 x 128] = stationary (K-major) x chunk^T (K-major): eight K = 16 steps over the head dim
            auto issue_t = [&](uint32_t t_col, uint32_t sa, uint32_t sb) {
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) {
                    const uint32_t o = (kk >> 2) * kSlab + (kk & 3) * 32;
                    if (TSA)        // A from tensor memory: eight 32-bit columns per K = 16 step
                        umma_bf16_ts(tmem + t_col, tmem + (t_col == kT1 ? kA1 : kA2) + kk * 8,
                                     smem_desc_sw128(sb + o, 16, 1024), idesc_t, kk ? 1u : 0u);
                    else
                        umma_bf16_ss(tmem + t_col, smem_desc_sw128(sa + o, 16, 1024), smem_desc_sw128(sb + o, 16, 1024),
                                     idesc_t, kk ? 1u : 0u);
                }
            };
            // acc[128 x 128] += A (bf16 pairs in tensor memory, 128 x 128 chunk rows) x chunk (MN-major B)
            auto issue_acc = [&](uint32_t acc_col, uint32_t a_col, uint32_t sb, bool first) {
#pragma unroll
                for (int kk = 0; kk < BC / 16; ++kk)
                    umma_bf16_ts(tmem + acc_col, tmem + a_col + (kk >> 1) * kCols + (kk & 1) * 8,
                                 smem_desc_sw128(sb + kk * 2048, kSlab, 1024), idesc_a, (first && kk == 0) ? 0u : 1u);
            };
            if (!mbar_wait(a_full, 0, &abort_flag)) goto done;
            if (!mbar_wait(b1_full(0), 0, &abort_flag)) goto done;
            tc_fence_after();
            issue_t(kT1, sA1, sRing1);
            umma_commit(s_full);
            if (!mbar_wait(b2_full(0), 0, &abort_flag)) goto done;
            tc_fence_after();
            issue_t(kT2, sA2, sRing2);
            umma_commit(dp_full);
            for (int c = 0; c < n_chunks; ++c) {
                const uint32_t par = (uint32_t)c & 1u;
                const bool more = c + 1 < n_chunks;
                // T1 is free as soon as every softmax warp has read S(c): the next chunk's scores overlap the dS pass
                TT_STAMP(0);
                if (!mbar_wait(p_ready, par, &abort_flag)) goto done;
                TT_STAMP(1);
                tc_fence_after();
                if (more) {
                    const int n1 = (c + 1) % kRing1;
                    if (!mbar_wait(b1_full(n1), (uint32_t)((c + 1) / kRing1) & 1u, &abort_flag)) goto done;
                    tc_fence_after();
                    issue_t(kT1, sA1, sRing1 + n1 * kTile);
                    umma_commit(s_full);
                }
                TT_STAMP(2);
                // T2 now holds bf16 P (first 16 columns of every 32) and dS (last 16) of this chunk
                if (!mbar_wait(ds_ready, par, &abort_flag)) goto done;
                TT_STAMP(3);
                tc_fence_after();
                issue_acc(KVS ? kAcc2 : kAcc1, kT2 + 16, sRing1 + (c % kRing1) * kTile, c == 0);   // dK += dS^T Q  /  dQ += dS K
                umma_commit(b1_empty(c % kRing1));
                if (KVS) issue_acc(kAcc1, kT2, sRing2 + (c % kRing2) * kTile, c == 0);             // dV += P^T dO
                umma_commit(b2_empty(c % kRing2));
                TT_STAMP(4);
                if (more) {
                    const int n2 = (c + 1) % kRing2;
                    if (!mbar_wait(b2_full(n2), (uint32_t)((c + 1) / kRing2) & 1u, &abort_flag)) goto done;
                    tc_fence_after();
                    issue_t(kT2, sA2, sRing2 + n2 * kTile);                                        // next chunk's dP
                    umma_commit(dp_full);
                }
                TT_STAMP(5);
            }
            umma_commit(acc_final);
        }
    } else {
        // ------------------------------------------------------------ softmax / dS
        // The warpgroups share every chunk: a thread owns one stationary row and kCols = 32 of the chunk's 128
        // streamed rows (columns of T1 / T2; warpgroup g: [32 g, 32 g + 32)), so four warps per scheduler hide each
        // other's tcgen05.ld / exp2 / tcgen05.st latency.  Each chunk has two passes:
        // P from the scores (runs while the tensor core forms dP), then dS from dP (runs while it forms the
        // next chunk's scores and, KV-stationary, dV).
        const int part = (warp - 2) >> 2;
        const int quad = warp & 3;
        const int srow = quad * 32 + lane;                 // row within the stationary tile
        const int row = r0 + srow;                         // key (KVS) or query index
        const uint32_t lane_sel = (uint32_t)(quad * 32) << 16;
        const float c_log2 = p.scale * kLog2e;
        float my_lse = 0.f, my_delta = 0.f;
        bool row_live;
        if (KVS) {
            row_live = row < p.kv_len && !(row >= p.mask_lo && row < p.mask_hi);
        } else {
            row_live = row < p.S;
            my_lse = row_live ? p.lse[(long)bh * p.pitch + row] * kLog2e : INFINITY;
            my_delta = row_live ? p.delta[(long)bh * p.pitch + row] : 0.f;
        }
        const uint32_t t1 = tmem + lane_sel + kT1 + part * kCols, t2 = tmem + lane_sel + kT2 + part * kCols;
        if (TSA) {
            // stationary operands into tensor memory: this thread owns row `srow` and 32 of its 128 elements (16 columns
            // of bf16 pairs, in memory order: element 2j in the low half of column j)
            uint32_t qv[16], dv[16];
            if (row_live) {
                const uint4* qp = reinterpret_cast<const uint4*>(p.q_raw + ((long)bh * p.S + row) * D + part * 32);
                const uint4* dp = reinterpret_cast<const uint4*>(p.do_raw + (((long)b * p.S + row) * p.H + head) * D + part * 32);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const uint4 a = __ldg(qp + i), g = __ldg(dp + i);
                    qv[4 * i] = a.x; qv[4 * i + 1] = a.y; qv[4 * i + 2] = a.z; qv[4 * i + 3] = a.w;
                    dv[4 * i] = g.x; dv[4 * i + 1] = g.y; dv[4 * i + 2] = g.z; dv[4 * i + 3] = g.w;
                }
            } else {
#pragma unroll
                for (int i = 0; i < 16; ++i) qv[i] = dv[i] = 0u;
            }
            tmem_st_32x16(tmem + lane_sel + kA1 + part * 16, qv);
            tmem_st_32x16(tmem + lane_sel + kA2 + part * 16, dv);
            tmem_st_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(a_full);
        }
        for (int c = 0; c < n_chunks; ++c) {
            const uint32_t par = (uint32_t)c & 1u;
            const int col0 = c * BC + part * kCols;         // first streamed row of this thread's 32 columns
            // KV-stationary: the streamed queries each have their own lse / delta; every thread reads them straight
            // from global memory (same addresses across the warp, so each load is one broadcast).  The statistics
            // rows are `pitch` long (a multiple of 64): a 32-column group past the end has no live query.
            const bool cols_ok = !KVS || col0 < p.pitch;
            const float4* lse4 = reinterpret_cast<const float4*>(p.lse + (long)bh * p.pitch + col0);
            const float4* del4 = reinterpret_cast<const float4*>(p.delta + (long)bh * p.pitch + col0);
            uint32_t pk[16];
            // query-stationary: only a chunk that straddles the key length or the masked key range needs per-key tests
#ifdef TT_ATTN_NO_RANGE_MASK
            const bool chunk_clean = false;
#else
            const bool chunk_clean = KVS || ((c + 1) * BC <= p.kv_len &&
                                             (p.mask_lo >= p.mask_hi || p.mask_hi <= c * BC || p.mask_lo >= (c + 1) * BC));
#endif
            if (!mbar_wait(s_full, par, &abort_flag)) goto done;
            if (threadIdx.x == 64) TT_STAMP(6);
            tc_fence_after();
            {
                constexpr int pass = 0;
                uint32_t a[32];
                tmem_ld_32x32(t1, a);
                float4 lq[8];
                if (KVS) {
#pragma unroll
                    for (int i = 0; i < 8; ++i)
                        lq[i] = cols_ok ? __ldg(lse4 + pass * 8 + i) : make_float4(INFINITY, INFINITY, INFINITY, INFINITY);
                }
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    float2 l2;
                    if (KVS) {
                        const float4 lv = lq[i >> 1];
                        l2 = (i & 1) ? make_float2(lv.z * kLog2e, lv.w * kLog2e) : make_float2(lv.x * kLog2e, lv.y * kLog2e);
                    } else {
                        l2 = make_float2(my_lse, my_lse);
                    }
                    const float2 x = __ffma2_rn(make_float2(__uint_as_float(a[2 * i]), __uint_as_float(a[2 * i + 1])),
                                                make_float2(c_log2, c_log2), make_float2(-l2.x, -l2.y));
                    float2 pr = make_float2(exp2f(x.x), exp2f(x.y));
                    if (KVS) {
                        if (!row_live) pr = make_float2(0.f, 0.f);
                    } else if (!chunk_clean) {
                        const int cc = col0 + pass * 32 + 2 * i;
#ifdef TT_ATTN_NO_RANGE_MASK
                        if (cc >= p.kv_len) pr.x = 0.f;
                        if (cc + 1 >= p.kv_len) pr.y = 0.f;
#else
                        if (cc >= p.kv_len || (cc >= p.mask_lo && cc < p.mask_hi)) pr.x = 0.f;
                        if (cc + 1 >= p.kv_len || (cc + 1 >= p.mask_lo && cc + 1 < p.mask_hi)) pr.y = 0.f;
#endif
                    }
                    const __nv_bfloat162 pb = __floats2bfloat162_rn(pr.x, pr.y);
                    pk[pass * 16 + i] = *reinterpret_cast<const uint32_t*>(&pb);
                }
            }
            // P stays in registers: T1 is released to the next chunk's score product right away
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(p_ready);
            if (threadIdx.x == 64) TT_STAMP(7);

            if (!mbar_wait(dp_full, par, &abort_flag)) goto done;
            if (threadIdx.x == 64) TT_STAMP(8);
            tc_fence_after();
            uint32_t dk[16];
            {
                constexpr int pass = 0;
                uint32_t g[32];
                tmem_ld_32x32(t2, g);
                float4 dq4[8];
                if (KVS) {
#pragma unroll
                    for (int i = 0; i < 8; ++i)
                        dq4[i] = cols_ok ? __ldg(del4 + pass * 8 + i) : make_float4(0.f, 0.f, 0.f, 0.f);
                }
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    float2 d2;
                    if (KVS) {
                        const float4 dv = dq4[i >> 1];
                        d2 = (i & 1) ? make_float2(dv.z, dv.w) : make_float2(dv.x, dv.y);
                    } else {
                        d2 = make_float2(my_delta, my_delta);
                    }
                    const float2 pr = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&pk[pass * 16 + i]));
                    const float2 dp = make_float2(__uint_as_float(g[2 * i]) - d2.x, __uint_as_float(g[2 * i + 1]) - d2.y);
                    const float2 ds = __fmul2_rn(pr, dp);
                    const __nv_bfloat162 db = __floats2bfloat162_rn(ds.x, ds.y);
                    dk[pass * 16 + i] = *reinterpret_cast<const uint32_t*>(&db);
                }
            }
            // bf16 pairs over the 32 dP columns this thread has just read: P in the first 16, dS in the last 16
            if (KVS) tmem_st_32x16(t2, pk);
            tmem_st_32x16(t2 + 16, dk);
            tmem_st_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(ds_ready);
            if (threadIdx.x == 64) TT_STAMP(9);
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
            const uint32_t tacc = tmem + lane_sel + kAcc1 + which * 128;
#pragma unroll 1
            for (int cch = part; cch < D / 32; cch += kGroups) {        // the warpgroups share the accumulator's columns
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


// ---------------------------------------------------------------------------------------------------------------
// One-pass variant: the key-stationary kernel also forms this chunk's dQ contribution, so S and dP are computed once
// (five products per [128 x 128] tile pair instead of seven).  dS is written twice by the softmax warps: as bf16 pairs
// into tensor memory (the A operand of dK += dS^T Q, as above) and into a shared-memory tile laid out [key][query]
// with 128-byte swizzle, which the tensor core reads MN-major as the A operand of dQ(c) = dS(c) K.  That product lands
// in T2 once dK(c) / dV(c) have consumed the bf16 P / dS there (the tensor core executes in issue order); the softmax
// warps read it back and add it to an fp32 [B*H, s_pad, 128] accumulator in global memory with vector reductions
// (every key tile of a head adds into the same rows: the order of those additions is not fixed, so dQ is reproducible
// only to fp32 rounding).  A last elementwise kernel scales and rounds the accumulator to bf16.
//
//   tensor core:  dP(c) S(c+1) ............ | dK(c) dV(c) dQ(c) | dP(c+1) S(c+2) ...
//   softmax:      readout(c-1) | dS(c) .... | P(c+1) .......... | readout(c) | dS(c+1) ...
//
// Shared memory: K, V resident; two slots each for the streamed Q and dO; one dS tile (same 225 KB as above).
constexpr int kFRing = 2;
constexpr int kFSmemBytes = (2 + 2 * kFRing + 1) * kTile + 256 + 1024;

// TMA reduction shared -> global: adds the [32 x 32] fp32 box at `smem_src` (128-byte swizzle) into the tensor at (x, y)
__device__ __forceinline__ void tma_reduce_add_2d(const CUtensorMap* tmap, uint32_t smem_src, int x, int y) {
    asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
                     (uint64_t)tmap),
                 "r"(smem_src), "r"(x), "r"(y)
                 : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read_but_last() { asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

constexpr int kFThreads = kThreads + 32;     // one more warp: issues the dQ reductions and waits for them
__global__ void __launch_bounds__(kFThreads, 1)
attn_bwd_fused_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                      const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
                      const __grid_constant__ CUtensorMap tmDQ, const BwdParams p) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ volatile int abort_flag;
    __shared__ uint32_t tmem_base_slot;

    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t sA1 = base;                       // K tile
    const uint32_t sA2 = base + kTile;               // V tile
    const uint32_t sRing1 = base + 2 * kTile;        // Q chunks
    const uint32_t sRing2 = sRing1 + kFRing * kTile; // dO chunks
    const uint32_t sDS = sRing2 + kFRing * kTile;    // dS of the current chunk, [key][query] bf16
    const uint32_t bars = sDS + kTile;
    const uint32_t a_full = bars;
    auto b1_full = [&](int s) { return bars + 8u * (1 + s); };
    auto b1_empty = [&](int s) { return bars + 8u * (1 + kFRing + s); };
    auto b2_full = [&](int s) { return bars + 8u * (1 + 2 * kFRing + s); };
    auto b2_empty = [&](int s) { return bars + 8u * (1 + 3 * kFRing + s); };
    const uint32_t s_full = bars + 8u * (1 + 4 * kFRing);
    const uint32_t dp_full = s_full + 8u;
    const uint32_t p_ready = s_full + 16u;
    const uint32_t ds_ready = s_full + 24u;
    const uint32_t dq_full = s_full + 32u;           // T2 holds dQ(c)
    const uint32_t dq_read = s_full + 40u;           // every softmax warp has read dQ(c) out of T2
    const uint32_t acc_final = s_full + 48u;
    const uint32_t stage_done = s_full + 56u;        // the dQ(c) half staged in the dS tile has been read by the TMA unit
    const uint32_t staged_a = s_full + 64u;          // column groups 0, 1 of dQ(c) are in the dS tile
    const uint32_t staged_b = s_full + 72u;          // column groups 2, 3 of dQ(c) are in chunk c's dO slot

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int bh = blockIdx.y;
    const int b = bh / p.H, head = bh - b * p.H;
    const int r0 = blockIdx.x * BS;                  // first key of this CTA
    const int n_chunks = (p.S + BC - 1) / BC;        // query chunks
    // Key tile x starts at query chunk x and wraps around: at any moment the CTAs of a head work on different chunks, so
    // their dQ reductions land on different lines of the accumulator instead of queueing up on the same 64 KB.
    const int c0 = (int)blockIdx.x % n_chunks;
    auto chunk_of = [&](int c) { const int e = c + c0; return e >= n_chunks ? e - n_chunks : e; };

    if (threadIdx.x == 0) {
        abort_flag = 0;
        mbar_init(a_full, 1);
        for (int s = 0; s < kFRing; ++s) {
            mbar_init(b1_full(s), 1);
            mbar_init(b1_empty(s), 1);
            mbar_init(b2_full(s), 1);
            mbar_init(b2_empty(s), 2);     // dV(c) has read the slot + the dQ half staged in it afterwards has left
        }
        mbar_init(s_full, 1);
        mbar_init(dp_full, 1);
        mbar_init(p_ready, 4 * kGroups);
        mbar_init(ds_ready, 4 * kGroups);
        mbar_init(dq_full, 1);
        mbar_init(dq_read, 4 * kGroups);
        mbar_init(acc_final, 1);
        mbar_init(stage_done, 1);
        mbar_init(staged_a, 2 * kGroups);
        mbar_init(staged_b, 2 * kGroups);
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
    constexpr uint32_t kT1 = 0, kT2 = 128, kAccV = 256, kAccK = 384;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            mbar_arrive_expect_tx(a_full, 2 * kTile);
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                tma_load_3d(sA1 + h * kSlab, &tmK, a_full, h * 64, r0, bh);
                tma_load_3d(sA2 + h * kSlab, &tmV, a_full, h * 64, r0, bh);
            }
            for (int c = 0; c < n_chunks; ++c) {
                const int s = c % kFRing;
                const uint32_t wpar = ((uint32_t)(c / kFRing) & 1u) ^ 1u;
                if (!mbar_wait(b1_empty(s), wpar, &abort_flag)) goto done;
                TT_STAMPF(15);
                mbar_arrive_expect_tx(b1_full(s), kTile);
#pragma unroll
                for (int h = 0; h < 2; ++h) tma_load_3d(sRing1 + s * kTile + h * kSlab, &tmQ, b1_full(s), h * 64, chunk_of(c) * BC, bh);
                if (!mbar_wait(b2_empty(s), wpar, &abort_flag)) goto done;
                TT_STAMPF(14);
                mbar_arrive_expect_tx(b2_full(s), kTile);
#pragma unroll
                for (int h = 0; h < 2; ++h)
                    tma_load_4d(sRing2 + s * kTile + h * kSlab, &tmDO, b2_full(s), h * 64, head, chunk_of(c) * BC, b);
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc_t = idesc_bf16(BS, BC, false, false);   // T = A B^T, both K-major
            constexpr uint32_t idesc_a = idesc_bf16(BS, D, false, true);     // acc += (tensor-memory A) B, B MN-major
            constexpr uint32_t idesc_q = idesc_bf16(BC, D, true, true);      // dQ = dS K: both operands MN-major
            auto issue_t = [&](uint32_t t_col, uint32_t sa, uint32_t sb) {
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) {
                    const uint32_t o = (kk >> 2) * kSlab + (kk & 3) * 32;
                    umma_bf16_ss(tmem + t_col, smem_desc_sw128(sa + o, 16, 1024), smem_desc_sw128(sb + o, 16, 1024), idesc_t,
                                 kk ? 1u : 0u);
                }
            };
            auto issue_acc = [&](uint32_t acc_col, uint32_t a_col, uint32_t sb, bool first) {
#pragma unroll
                for (int kk = 0; kk < BC / 16; ++kk)
                    umma_bf16_ts(tmem + acc_col, tmem + a_col + (kk >> 1) * kCols + (kk & 1) * 8,
                                 smem_desc_sw128(sb + kk * 2048, kSlab, 1024), idesc_a, (first && kk == 0) ? 0u : 1u);
            };
            if (!mbar_wait(a_full, 0, &abort_flag)) goto done;
            if (!mbar_wait(b1_full(0), 0, &abort_flag)) goto done;
            tc_fence_after();
            issue_t(kT1, sA1, sRing1);
            umma_commit(s_full);
            if (!mbar_wait(b2_full(0), 0, &abort_flag)) goto done;
            tc_fence_after();
            issue_t(kT2, sA2, sRing2);
            umma_commit(dp_full);
            for (int c = 0; c < n_chunks; ++c) {
                const uint32_t par = (uint32_t)c & 1u;
                const bool more = c + 1 < n_chunks;
                const int slot = c % kFRing, nslot = (c + 1) % kFRing;
                const uint32_t npar = (uint32_t)((c + 1) / kFRing) & 1u;
                TT_STAMPF(0);
                if (!mbar_wait(p_ready, par, &abort_flag)) goto done;              // S(c) has been read: T1 is free
                TT_STAMPF(1);
                tc_fence_after();
                if (more) {
                    if (!mbar_wait(b1_full(nslot), npar, &abort_flag)) goto done;
                    tc_fence_after();
                    issue_t(kT1, sA1, sRing1 + nslot * kTile);                     // S(c+1)
                    umma_commit(s_full);
                }
                if (!mbar_wait(ds_ready, par, &abort_flag)) goto done;             // P, dS in T2; dS in shared memory
                TT_STAMPF(2);
                tc_fence_after();
                issue_acc(kAccK, kT2 + 16, sRing1 + slot * kTile, c == 0);          // dK += dS^T Q
                umma_commit(b1_empty(slot));
                issue_acc(kAccV, kT2, sRing2 + slot * kTile, c == 0);               // dV += P^T dO
                umma_commit(b2_empty(slot));
#pragma unroll
                for (int kk = 0; kk < BS / 16; ++kk)                                // dQ(c) = dS K over the 128 keys, into T2
                    umma_bf16_ss(tmem + kT2, smem_desc_sw128(sDS + kk * 2048, kSlab, 1024),
                                 smem_desc_sw128(sA1 + kk * 2048, kSlab, 1024), idesc_q, kk ? 1u : 0u);
                umma_commit(dq_full);
                TT_STAMPF(3);
                if (more) {
                    if (!mbar_wait(dq_read, par, &abort_flag)) goto done;          // dQ(c) is in registers: T2 is free
                    TT_STAMPF(4);
                    if (!mbar_wait(b2_full(nslot), npar, &abort_flag)) goto done;
                    TT_STAMPF(10);
                    tc_fence_after();
                    issue_t(kT2, sA2, sRing2 + nslot * kTile);                     // dP(c+1)
                    umma_commit(dp_full);
                }
            }
            umma_commit(acc_final);
        }
    } else if (warp == 2 + 4 * kGroups) {
        // ------------------------------------------------------------ dQ reductions
        // dQ(c) is staged by the softmax warps in two halves of eight [32 x 32] fp32 boxes: column groups 0, 1 in the dS
        // tile (idle until the next chunk's dS is stored), groups 2, 3 in chunk c's dO slot (dV(c) has consumed it; the
        // producer refills it only after this thread has released it).  The first half is issued first, so it leaves
        // first; both drain while the next chunk is computed.  A thread of its own waits for the TMA unit, so that no
        // softmax warp ever does.
        if (lane == 0) {
            for (int c = 0; c < n_chunks; ++c) {
                const uint32_t par = (uint32_t)c & 1u;
                const int yrow = bh * p.s_pad + chunk_of(c) * BC;
                if (!mbar_wait(staged_a, par, &abort_flag)) goto done;
                TT_STAMPF(11);
#ifndef TT_FUSED_NO_RED
#pragma unroll
                for (int g = 0; g < 8; ++g) tma_reduce_add_2d(&tmDQ, sDS + ((uint32_t)g << 12), (g & 1) * kCols, yrow + (g >> 1) * 32);
#endif
                bulk_commit();
                if (!mbar_wait(staged_b, par, &abort_flag)) goto done;
#ifndef TT_FUSED_NO_RED
                const uint32_t slot = sRing2 + (uint32_t)(c % kFRing) * kTile;
#pragma unroll
                for (int g = 0; g < 8; ++g)
                    tma_reduce_add_2d(&tmDQ, slot + ((uint32_t)g << 12), (2 + (g & 1)) * kCols, yrow + (g >> 1) * 32);
#endif
                bulk_commit();
                bulk_wait_read_but_last();
                TT_STAMPF(12);
                mbar_arrive(stage_done);
                bulk_wait_read();
                TT_STAMPF(13);
                mbar_arrive(b2_empty(c % kFRing));
            }
            bulk_wait_all();
        }
    } else {
        // ------------------------------------------------------------ softmax / dS / dQ read-out
        const int part = (warp - 2) >> 2;
        const int quad = warp & 3;
        const int srow = quad * 32 + lane;                 // key row within the tile; also the query row of a dQ read-out
        const int row = r0 + srow;
        const uint32_t lane_sel = (uint32_t)(quad * 32) << 16;
        const float c_log2 = p.scale * kLog2e;
        const bool row_live = row < p.kv_len && !(row >= p.mask_lo && row < p.mask_hi);
        const uint32_t t1 = tmem + lane_sel + kT1 + part * kCols, t2 = tmem + lane_sel + kT2 + part * kCols;
        // this thread's 64 bytes of the dS tile: row srow of slab (part >> 1), 16-byte chunks 4 (part & 1) + 0..3, swizzled
        const uint32_t ds_row = sDS + (uint32_t)(part >> 1) * kSlab + (uint32_t)srow * 128u;
        const uint32_t ds_chunk0 = (uint32_t)(part & 1) * 4u, ds_xor = (uint32_t)srow & 7u;
        uint32_t pk[16];
        // this warp's 4 KB of the dQ staging: groups 0, 1 in the dS tile, groups 2, 3 in the chunk's dO slot
        const uint32_t stage_off = ((uint32_t)(quad * 2 + (part & 1)) << 12) + (uint32_t)lane * 128u;

        auto p_pass = [&](int c) -> bool {
            const int col0 = chunk_of(c) * BC + part * kCols;
            const bool cols_ok = col0 < p.pitch;
            const float4* lse4 = reinterpret_cast<const float4*>(p.lse + (long)bh * p.pitch + col0);
            if (!mbar_wait(s_full, (uint32_t)c & 1u, &abort_flag)) return false;
            tc_fence_after();
            uint32_t a[32];
            tmem_ld_32x32(t1, a);
            float4 lq[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) lq[i] = cols_ok ? __ldg(lse4 + i) : make_float4(INFINITY, INFINITY, INFINITY, INFINITY);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const float4 lv = lq[i >> 1];
                const float2 l2 = (i & 1) ? make_float2(lv.z * kLog2e, lv.w * kLog2e) : make_float2(lv.x * kLog2e, lv.y * kLog2e);
                const float2 x = __ffma2_rn(make_float2(__uint_as_float(a[2 * i]), __uint_as_float(a[2 * i + 1])),
                                            make_float2(c_log2, c_log2), make_float2(-l2.x, -l2.y));
                float2 pr = make_float2(exp2f(x.x), exp2f(x.y));
                if (!row_live) pr = make_float2(0.f, 0.f);
                const __nv_bfloat162 pb = __floats2bfloat162_rn(pr.x, pr.y);
                pk[i] = *reinterpret_cast<const uint32_t*>(&pb);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(p_ready);
            return true;
        };

        if (!p_pass(0)) goto done;
        for (int c = 0; c < n_chunks; ++c) {
            const uint32_t par = (uint32_t)c & 1u;
            const int col0 = chunk_of(c) * BC + part * kCols;
            const bool cols_ok = col0 < p.pitch;
            const float4* del4 = reinterpret_cast<const float4*>(p.delta + (long)bh * p.pitch + col0);
            // ---- dS(c) from dP(c) and the P kept in registers
            if (!mbar_wait(dp_full, par, &abort_flag)) goto done;
            if (threadIdx.x == 64) TT_STAMPF(5);
            tc_fence_after();
            uint32_t dk[16];
            {
                uint32_t g[32];
                tmem_ld_32x32(t2, g);
                float4 dq4[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) dq4[i] = cols_ok ? __ldg(del4 + i) : make_float4(0.f, 0.f, 0.f, 0.f);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const float4 dv = dq4[i >> 1];
                    const float2 d2 = (i & 1) ? make_float2(dv.z, dv.w) : make_float2(dv.x, dv.y);
                    const float2 pr = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&pk[i]));
                    const float2 dp = make_float2(__uint_as_float(g[2 * i]) - d2.x, __uint_as_float(g[2 * i + 1]) - d2.y);
                    const float2 ds = __fmul2_rn(pr, dp);
                    const __nv_bfloat162 db = __floats2bfloat162_rn(ds.x, ds.y);
                    dk[i] = *reinterpret_cast<const uint32_t*>(&db);
                }
            }
            tmem_st_32x16(t2, pk);
            tmem_st_32x16(t2 + 16, dk);
            // the dS tile doubles as a staging buffer of the previous chunk's dQ read-out: wait until that has left
            if (c > 0 && !mbar_wait(stage_done, (uint32_t)(c - 1) & 1u, &abort_flag)) goto done;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint32_t addr = ds_row + (((ds_chunk0 + (uint32_t)j) ^ ds_xor) << 4);
                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(dk[4 * j]), "r"(dk[4 * j + 1]),
                             "r"(dk[4 * j + 2]), "r"(dk[4 * j + 3])
                             : "memory");
            }
            tmem_st_wait();
            fence_proxy_async();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(ds_ready);
            if (threadIdx.x == 64) TT_STAMPF(6);
            // ---- P(c+1): runs while the tensor core forms dK(c), dV(c), dQ(c)
            if (c + 1 < n_chunks && !p_pass(c + 1)) goto done;
            if (threadIdx.x == 64) TT_STAMPF(7);
            // ---- dQ(c) out of T2 and into the global accumulator
            if (!mbar_wait(dq_full, par, &abort_flag)) goto done;
            if (threadIdx.x == 64) TT_STAMPF(8);
            tc_fence_after();
            uint32_t r[32];
            tmem_ld_32x32(t2, r);
            tmem_ld_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(dq_read);
            {
                const uint32_t mine = (part < 2 ? sDS : sRing2 + (uint32_t)(c % kFRing) * kTile) + stage_off;
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(mine + ((((uint32_t)j) ^ ((uint32_t)lane & 7u)) << 4)),
                                 "r"(r[4 * j]), "r"(r[4 * j + 1]), "r"(r[4 * j + 2]), "r"(r[4 * j + 3])
                                 : "memory");
                fence_proxy_async();
                __syncwarp();
                if (lane == 0) mbar_arrive(part < 2 ? staged_a : staged_b);
            }
            if (threadIdx.x == 64) TT_STAMPF(9);
        }
        // ------------------------------------------------------------ epilogue: dV (unscaled), dK (x softmax scale)
        if (!mbar_wait(acc_final, 0, &abort_flag)) goto done;
        tc_fence_after();
        const bool store = row < p.S;
        const long orow = ((long)bh * p.S + row) * D;
#pragma unroll 1
        for (int which = 0; which < 2; ++which) {
            __nv_bfloat16* dst = (which == 0 ? p.out1 : p.out2) + orow;
            const float mul = which == 0 ? 1.f : p.scale;
            const uint32_t tacc = tmem + lane_sel + kAccV + which * 128;
            uint32_t r[32];
            tmem_ld_32x32(tacc + part * 32, r);
            tmem_ld_wait();
            if (store) {
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                    float o[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) o[i] = __uint_as_float(r[g * 8 + i]) * mul;
                    tt::st8(dst + part * 32 + g * 8, tt::pack8(o));
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

// dq[bh, s, :] = bf16(scale * acc[bh, s, :]); eight elements per thread
__global__ void __launch_bounds__(256) dq_finish_kernel(const float* __restrict__ acc, __nv_bfloat16* __restrict__ dq, long BH, int S,
                                                       int s_pad, float scale) {
    const long n8 = BH * S * (D / 8);
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (long)gridDim.x * blockDim.x) {
        const long rowi = i / (D / 8);
        const int c8 = (int)(i - rowi * (D / 8));
        const long bhi = rowi / S, s = rowi - bhi * S;
        const float4* src = reinterpret_cast<const float4*>(acc + (bhi * s_pad + s) * D + c8 * 8);
        const float4 x = __ldg(src), y = __ldg(src + 1);
        float o[8] = {x.x * scale, x.y * scale, x.z * scale, x.w * scale, y.x * scale, y.y * scale, y.z * scale, y.w * scale};
        tt::st8(dq + rowi * D + c8 * 8, tt::pack8(o));
    }
}

}  // namespace

// lse, delta: [B*H, pitch] fp32 with pitch a multiple of 64; lse holds +inf and delta 0 at positions >= S
// (delta is scratch owned by the caller, zero-initialised; this call fills positions < S).
#ifdef TT_ATTN_STAMPS
static long long* g_attn_stamps = nullptr;
extern "C" void tt_attn_set_stamps(long long* ptr) { g_attn_stamps = ptr; }
#endif

extern "C" int tt_attn_bwd(const void* q, const void* k, const void* v, const void* out, const void* dout,
                           const float* lse, float* delta, void* dq, void* dk, void* dv, int B, int H, int S, int kv_len,
                           int mask_lo, int mask_hi, int pitch, float scale, int* status, void* stream) {
    if (B <= 0 || H <= 0 || S <= 0 || kv_len <= 0 || kv_len > S || status == nullptr || delta == nullptr) return TT_ERR_ARG;
    if (mask_lo < mask_hi && (mask_lo < 0 || (mask_lo == 0 && mask_hi >= kv_len))) return TT_ERR_ARG;
    if (pitch < S || (pitch & 63) || ((uintptr_t)lse & 15) || ((uintptr_t)delta & 15)) return TT_ERR_ARG;
    cudaStream_t st = (cudaStream_t)stream;
    const uint64_t BH = (uint64_t)B * H;
    CUtensorMap tq_s, tk_s, tv_s, tdo_s;     // 128-row x 64-column boxes (stationary operands and streamed chunks)
    int rc;
    if ((rc = tt_make_tmap_3d(&tq_s, q, BH, (uint64_t)S, D, D, (uint64_t)S * D, BS, 64)) != TT_OK) return rc;
    if ((rc = tt_make_tmap_3d(&tk_s, k, BH, (uint64_t)S, D, D, (uint64_t)S * D, BS, 64)) != TT_OK) return rc;
    if ((rc = tt_make_tmap_3d(&tv_s, v, BH, (uint64_t)S, D, D, (uint64_t)S * D, BS, 64)) != TT_OK) return rc;
    if ((rc = tt_make_tmap_bshd(&tdo_s, dout, (uint64_t)B, (uint64_t)S, (uint64_t)H, BS)) != TT_OK) return rc;
    static bool configured_dev[64] = {false};   // per device: the attribute belongs to the device's context
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
    bool& configured = configured_dev[dev];
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attn_bwd_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute(attn_bwd_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute(attn_bwd_kernel<false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
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
    p.mask_lo = mask_lo;
    p.mask_hi = mask_lo < mask_hi ? mask_hi : mask_lo;
    p.H = H;
    p.pitch = pitch;
    p.scale = scale;
    p.status = status;
    p.q_raw = (const __nv_bfloat16*)q;
    p.do_raw = (const __nv_bfloat16*)dout;
    p.dq_acc = nullptr;
    p.s_pad = 0;
#ifdef TT_ATTN_STAMPS
    p.stamps = g_attn_stamps;
#endif
    // dK, dV: stationary keys (K, V resident), streamed queries (Q, dO)
    p.out1 = (__nv_bfloat16*)dv;
    p.out2 = (__nv_bfloat16*)dk;
    attn_bwd_kernel<true><<<dim3((S + BS - 1) / BS, (unsigned)BH), kThreads, kSmemBytes, st>>>(tq_s, tk_s, tv_s, tdo_s, p);
    TT_CHECK_LAUNCH();
    // dQ: stationary queries (Q, dO resident), streamed keys (K, V)
    p.out1 = (__nv_bfloat16*)dq;
    p.out2 = nullptr;
#ifdef TT_ATTN_STAMPS
    if (p.stamps != nullptr) p.stamps += 2560;      // second half of the buffer: the query-stationary kernel
#endif
    // TELETRON_B200_ATTN_BWD_TSA=1 selects the variant with Q / dO in tensor memory (off by default)
    static const bool tsa = [] { const char* v = getenv("TELETRON_B200_ATTN_BWD_TSA"); return v != nullptr && v[0] == '1'; }();
    if (tsa)
        attn_bwd_kernel<false, true><<<dim3((S + BS - 1) / BS, (unsigned)BH), kThreads, kSmemBytes, st>>>(tq_s, tk_s, tv_s, tdo_s, p);
    else
        attn_bwd_kernel<false><<<dim3((S + BS - 1) / BS, (unsigned)BH), kThreads, kSmemBytes, st>>>(tq_s, tk_s, tv_s, tdo_s, p);
    TT_CHECK_LAUNCH();
    return TT_OK;
}

// One-pass backward: delta preprocess, the fused key-stationary kernel (dK, dV written, dQ accumulated in fp32 into
// `dq_acc`), then the scale-and-round pass into `dq`.  dq_acc: fp32 scratch of B * H * s_pad * 128 elements with
// s_pad = S rounded up to a multiple of 128; it is zeroed here.
extern "C" int tt_attn_bwd_fused(const void* q, const void* k, const void* v, const void* out, const void* dout,
                                 const float* lse, float* delta, float* dq_acc, void* dq, void* dk, void* dv, int B, int H,
                                 int S, int kv_len, int mask_lo, int mask_hi, int pitch, float scale, int* status,
                                 void* stream) {
    if (B <= 0 || H <= 0 || S <= 0 || kv_len <= 0 || kv_len > S || status == nullptr || delta == nullptr || dq_acc == nullptr)
        return TT_ERR_ARG;
    if (mask_lo < mask_hi && (mask_lo < 0 || (mask_lo == 0 && mask_hi >= kv_len))) return TT_ERR_ARG;
    if (pitch < S || (pitch & 63) || ((uintptr_t)lse & 15) || ((uintptr_t)delta & 15) || ((uintptr_t)dq_acc & 15)) return TT_ERR_ARG;
    cudaStream_t st = (cudaStream_t)stream;
    const uint64_t BH = (uint64_t)B * H;
    const int s_pad = (S + BC - 1) / BC * BC;
    CUtensorMap tq_s, tk_s, tv_s, tdo_s;
    int rc;
    if ((rc = tt_make_tmap_3d(&tq_s, q, BH, (uint64_t)S, D, D, (uint64_t)S * D, BS, 64)) != TT_OK) return rc;
    if ((rc = tt_make_tmap_3d(&tk_s, k, BH, (uint64_t)S, D, D, (uint64_t)S * D, BS, 64)) != TT_OK) return rc;
    if ((rc = tt_make_tmap_3d(&tv_s, v, BH, (uint64_t)S, D, D, (uint64_t)S * D, BS, 64)) != TT_OK) return rc;
    if ((rc = tt_make_tmap_bshd(&tdo_s, dout, (uint64_t)B, (uint64_t)S, (uint64_t)H, BS)) != TT_OK) return rc;
    static bool configured_dev[64] = {false};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
    if (!configured_dev[dev]) {
        cudaError_t e = cudaFuncSetAttribute(attn_bwd_fused_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kFSmemBytes);
        if (e != cudaSuccess) return tt_record_cuda(e);
        configured_dev[dev] = true;
    }
    CUtensorMap tdq;      // fp32 [B*H*s_pad, 128], boxes of 32 rows x 32 columns (128 bytes), 128-byte swizzle
    {
        tt_encode_tiled_fn enc = tt_get_encode_tiled();
        if (enc == nullptr) return TT_ERR_CUDA;
        cuuint64_t dims[2] = {(cuuint64_t)D, (cuuint64_t)(BH * (uint64_t)s_pad)};
        cuuint64_t strides[1] = {(cuuint64_t)D * sizeof(float)};
        cuuint32_t box[2] = {32, 32};
        cuuint32_t estr[2] = {1, 1};
        if (enc(&tdq, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, dq_acc, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return TT_ERR_ARG;
    }
    cudaError_t e = cudaMemsetAsync(dq_acc, 0, BH * (uint64_t)s_pad * D * sizeof(float), st);
    if (e != cudaSuccess) return tt_record_cuda(e);
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
    p.mask_lo = mask_lo;
    p.mask_hi = mask_lo < mask_hi ? mask_hi : mask_lo;
    p.H = H;
    p.pitch = pitch;
    p.scale = scale;
    p.status = status;
    p.q_raw = (const __nv_bfloat16*)q;
    p.do_raw = (const __nv_bfloat16*)dout;
    p.dq_acc = dq_acc;
    p.s_pad = s_pad;
#ifdef TT_ATTN_STAMPS
    p.stamps = g_attn_stamps;
#endif
    p.out1 = (__nv_bfloat16*)dv;
    p.out2 = (__nv_bfloat16*)dk;
    attn_bwd_fused_kernel<<<dim3((S + BS - 1) / BS, (unsigned)BH), kFThreads, kFSmemBytes, st>>>(tq_s, tk_s, tv_s, tdo_s, tdq, p);
    TT_CHECK_LAUNCH();
    const long n8 = (long)BH * S * (D / 8);
    long blocks = (n8 + 255) / 256;
    dq_finish_kernel<<<(int)(blocks < 148L * 16 ? blocks : 148L * 16), 256, 0, st>>>(dq_acc, (__nv_bfloat16*)dq, (long)BH, S, s_pad,
                                                                                   scale);
    TT_CHECK_LAUNCH();
    return TT_OK;
}
