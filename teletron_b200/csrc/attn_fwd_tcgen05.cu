// Flash attention forward on tcgen05 / TMEM for head dim 128, non-causal, with a key-length mask.
//
// One CTA owns 256 query rows of one (batch, head) as two 128-row tiles that ping-pong through the
// tensor core: while the softmax warps of tile 0 turn S0 into P0, the tensor core computes S1 = Q1 K^T
// or O1 += P1 V, and vice versa.  Accumulators never leave tensor memory:
//   TMEM columns [0,128) S0 / P0 (bf16 P overwrites S in place), [128,256) S1 / P1,
//                [256,384) O0, [384,512) O1.
// Warp roles: warp 0 TMA loads (Q once, K / V double buffered), warp 1 issues every MMA
// (S = Q K^T with both operands from shared memory; O += P V with P read from tensor memory and V fed
// as an MN-major shared-memory operand, so V is never transposed), warps 2-5 softmax of tile 0,
// warps 6-9 softmax of tile 1 (one query row per thread).
// The running row maximum is only raised when it grows by more than 2^8 ("lazy rescale"), so O is
// corrected in tensor memory on rare iterations only.
//
// q, k, v: [B * H, S, 128] bf16 (head-major, as written by the QKV kernel); out: [B, S, H * 128] bf16
// (token-major, as read by the output projection); lse: [B * H, S] fp32 (natural log).
// The reference calls torch SDPA here (teletron/models/dit/dit_attention.py:311-313, 483-485).
#include "common.cuh"
#include "sm100.cuh"
#include "teletron_b200.h"

namespace {

using namespace sm100;

constexpr int D = 128;          // head dim
constexpr int BQ = 128;         // rows per query tile (two tiles per CTA)
constexpr int BKV = 128;        // keys per iteration
constexpr int kThreads = 320;   // 10 warps
constexpr int kSlab = BQ * 128; // bytes of one [128 rows x 64 cols] swizzled slab (16 KB)
constexpr int kTileBytes = 2 * kSlab;   // a [128 x 128] bf16 tile = two slabs (32 KB)
// smem: Q0, Q1, K[2], V[2] = 6 tiles = 192 KB
constexpr int kSmemBytes = 6 * kTileBytes + 1024 + 256;
constexpr float kRescaleThreshold = 8.0f;   // log2 units

__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

struct AttnParams {
    __nv_bfloat16* out;   // [B, S, H*128]
    float* lse;           // [B*H, lse_pitch]
    int lse_pitch;
    int S;                // query / key sequence length
    int kv_len;           // keys >= kv_len are masked
    int mask_lo, mask_hi; // keys in [mask_lo, mask_hi) are masked as well (padded text tokens that are not the sequence tail)
    int H;                // heads (for the output layout)
    float scale_log2;     // softmax scale * log2(e)
    int* status;
    // Ulysses head -> sequence all-to-all fused into the epilogue (batch 1): besides the local copy, every output row
    // is stored into the gathered buffer [text_len + s_local, dest_ld] of the rank that owns that token (text rows,
    // which come first in the sequence, go to every rank), at this rank's head columns.
    int push, n_peers, my_rank, text_len, s_local;
    long dest_ld;
    __nv_bfloat16* peer_out[TT_MAX_PEERS];
};

__global__ void __launch_bounds__(kThreads, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const AttnParams p) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ volatile int abort_flag;
    __shared__ uint32_t tmem_base_slot;

    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t sQ = base;                          // Q0 at +0, Q1 at +kTileBytes
    const uint32_t sK = base + 2 * kTileBytes;         // two stages
    const uint32_t sV = base + 4 * kTileBytes;         // two stages
    const uint32_t bars = base + 6 * kTileBytes;
    const uint32_t q_full = bars;
    auto k_full = [&](int s) { return bars + 8u * (1 + s); };
    auto k_empty = [&](int s) { return bars + 8u * (3 + s); };
    auto v_full = [&](int s) { return bars + 8u * (5 + s); };
    auto v_empty = [&](int s) { return bars + 8u * (7 + s); };
    auto s_full = [&](int t) { return bars + 8u * (9 + t); };
    auto p_full = [&](int t) { return bars + 8u * (11 + t); };
    const uint32_t o_final = bars + 8u * 13;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int bh = blockIdx.y;                  // batch * H + head
    const int q0 = blockIdx.x * (2 * BQ);       // first query row of this CTA
    const int n_kv = (p.kv_len + BKV - 1) / BKV;

    if (threadIdx.x == 0) {
        abort_flag = 0;
        mbar_init(q_full, 1);
        for (int s = 0; s < 2; ++s) {
            mbar_init(k_full(s), 1);
            mbar_init(k_empty(s), 1);
            mbar_init(v_full(s), 1);
            mbar_init(v_empty(s), 1);
            mbar_init(s_full(s), 1);
            mbar_init(p_full(s), 4);
        }
        mbar_init(o_final, 1);
        fence_barrier_init();
        fence_proxy_async();
        tma_prefetch_desc(&tmQ);
        tma_prefetch_desc(&tmK);
        tma_prefetch_desc(&tmV);
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
            mbar_arrive_expect_tx(q_full, 2 * kTileBytes);
#pragma unroll
            for (int t = 0; t < 2; ++t)
#pragma unroll
                for (int h = 0; h < 2; ++h) tma_load_3d(sQ + t * kTileBytes + h * kSlab, &tmQ, q_full, h * 64, q0 + t * BQ, bh);
            for (int j = 0; j < n_kv; ++j) {
                const int s = j & 1;
                const uint32_t ph = (uint32_t)(j >> 1) & 1u;
                if (!mbar_wait(k_empty(s), ph ^ 1u, &abort_flag)) goto done;
                mbar_arrive_expect_tx(k_full(s), kTileBytes);
#pragma unroll
                for (int h = 0; h < 2; ++h) tma_load_3d(sK + s * kTileBytes + h * kSlab, &tmK, k_full(s), h * 64, j * BKV, bh);
                if (!mbar_wait(v_empty(s), ph ^ 1u, &abort_flag)) goto done;
                mbar_arrive_expect_tx(v_full(s), kTileBytes);
#pragma unroll
                for (int h = 0; h < 2; ++h) tma_load_3d(sV + s * kTileBytes + h * kSlab, &tmV, v_full(s), h * 64, j * BKV, bh);
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc_s = idesc_bf16(BQ, BKV, false, false);   // S = Q K^T: both K-major
            constexpr uint32_t idesc_o = idesc_bf16(BQ, D, false, true);      // O += P V: V is MN-major
            auto issue_s = [&](int t, int stage) {
                const uint32_t a = sQ + t * kTileBytes, b = sK + stage * kTileBytes;
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) {
                    const uint32_t off = (kk >> 2) * kSlab + (kk & 3) * 32;
                    umma_bf16_ss(tmem + t * 128, smem_desc_sw128(a + off, 16, 1024), smem_desc_sw128(b + off, 16, 1024),
                                 idesc_s, kk ? 1u : 0u);
                }
                umma_commit(s_full(t));
            };
            auto issue_o = [&](int t, int stage, bool accumulate) {
                const uint32_t b = sV + stage * kTileBytes;
#pragma unroll
                for (int kk = 0; kk < BKV / 16; ++kk) {
                    // P: 16 bf16 keys = 8 TMEM columns per step; V: 16 key rows = 2048 B per step, dims slabs 16 KB apart
                    umma_bf16_ts(tmem + 256 + t * 128, tmem + t * 128 + kk * 8, smem_desc_sw128(b + kk * 2048, kSlab, 1024),
                                 idesc_o, (accumulate || kk) ? 1u : 0u);
                }
            };
            if (!mbar_wait(q_full, 0, &abort_flag)) goto done;
            if (!mbar_wait(k_full(0), 0, &abort_flag)) goto done;
            tc_fence_after();
            issue_s(0, 0);
            issue_s(1, 0);
            umma_commit(k_empty(0));
            for (int j = 0; j < n_kv; ++j) {
                const int s = j & 1;
                const uint32_t ph = (uint32_t)(j >> 1) & 1u;
                const uint32_t pph = (uint32_t)j & 1u;
                const bool more = j + 1 < n_kv;
                const int s1 = (j + 1) & 1;
                const uint32_t ph1 = (uint32_t)((j + 1) >> 1) & 1u;
                if (!mbar_wait(v_full(s), ph, &abort_flag)) goto done;
                if (!mbar_wait(p_full(0), pph, &abort_flag)) goto done;
                tc_fence_after();
                issue_o(0, s, j > 0);
                if (more) {
                    if (!mbar_wait(k_full(s1), ph1, &abort_flag)) goto done;
                    tc_fence_after();
                    issue_s(0, s1);
                }
                if (!mbar_wait(p_full(1), pph, &abort_flag)) goto done;
                tc_fence_after();
                issue_o(1, s, j > 0);
                umma_commit(v_empty(s));
                if (more) {
                    issue_s(1, s1);
                    umma_commit(k_empty(s1));
                }
            }
            umma_commit(o_final);
        }
    } else {
        // ------------------------------------------------------------ softmax + epilogue (one row per thread)
        const int t = (warp - 2) >> 2;             // query tile 0 / 1
        const int quad = warp & 3;                 // TMEM lane quadrant this warp may touch
        const int row_in_tile = quad * 32 + lane;
        const int row = q0 + t * BQ + row_in_tile;
        const uint32_t lane_sel = (uint32_t)(quad * 32) << 16;
        const uint32_t tS = tmem + lane_sel + t * 128;
        const uint32_t tO = tmem + lane_sel + 256 + t * 128;
        float m = -INFINITY, l = 0.f;
        for (int j = 0; j < n_kv; ++j) {
            if (!mbar_wait(s_full(t), (uint32_t)j & 1u, &abort_flag)) goto done;
            tc_fence_after();
            const int valid = p.kv_len - j * BKV;      // columns >= valid are masked (only in the last tile)
#ifdef TT_ATTN_NO_RANGE_MASK
            const int lo = 0, hi = 0;
            const bool full_tile = valid >= BKV;
#else
            const int lo = p.mask_lo - j * BKV, hi = p.mask_hi - j * BKV;      // and columns [lo, hi) of this tile
            const bool full_tile = valid >= BKV && (lo >= hi || hi <= 0 || lo >= BKV);
#endif
            // pass 1: row maximum (3-input max, four independent chains)
            float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
            for (int c = 0; c < BKV / 32; ++c) {
                uint32_t r[32];
                tmem_ld_32x32(tS + c * 32, r);
                tmem_ld_wait();
                if (!full_tile) {
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        if (c * 32 + i >= valid || (c * 32 + i >= lo && c * 32 + i < hi)) r[i] = 0xff800000u;      // -inf
                }
#pragma unroll
                for (int i = 0; i < 32; i += 8) {
                    mx0 = max3(mx0, __uint_as_float(r[i]), __uint_as_float(r[i + 1]));
                    mx1 = max3(mx1, __uint_as_float(r[i + 2]), __uint_as_float(r[i + 3]));
                    mx2 = max3(mx2, __uint_as_float(r[i + 4]), __uint_as_float(r[i + 5]));
                    mx3 = max3(mx3, __uint_as_float(r[i + 6]), __uint_as_float(r[i + 7]));
                }
            }
            const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * p.scale_log2;
            // lazy rescale of the accumulator
            const bool grow = mx > m + kRescaleThreshold || j == 0;
            if (j > 0 && __any_sync(0xffffffffu, grow)) {
                const float alpha = grow ? exp2f(m - mx) : 1.f;
                l *= alpha;
#pragma unroll 1
                for (int c = 0; c < D / 16; ++c) {
                    uint32_t r[16];
                    tmem_ld_32x16(tO + c * 16, r);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 16; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
                    tmem_st_32x16(tO + c * 16, r);
                }
                tmem_st_wait();
            }
            if (grow) m = mx;
            // pass 2: P = exp2(s * scale - m) with packed fp32x2 arithmetic, row sum, bf16 pack, store over S
            const float2 sc2 = make_float2(p.scale_log2, p.scale_log2);
            const float2 nm2 = make_float2(-m, -m);
            float2 sum2a = make_float2(0.f, 0.f), sum2b = make_float2(0.f, 0.f);
#pragma unroll
            for (int c = 0; c < BKV / 32; ++c) {
                uint32_t r[32];
                tmem_ld_32x32(tS + c * 32, r);
                tmem_ld_wait();
                uint32_t pk[16];
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const float2 x = __ffma2_rn(make_float2(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1])), sc2, nm2);
                    float2 e = make_float2(exp2f(x.x), exp2f(x.y));
                    if (!full_tile) {
                        const int c0 = c * 32 + 2 * i;
                        if (c0 >= valid || (c0 >= lo && c0 < hi)) e.x = 0.f;
                        if (c0 + 1 >= valid || (c0 + 1 >= lo && c0 + 1 < hi)) e.y = 0.f;
                    }
                    if (i & 1) sum2b = __fadd2_rn(sum2b, e);
                    else sum2a = __fadd2_rn(sum2a, e);
                    const __nv_bfloat162 b2 = __floats2bfloat162_rn(e.x, e.y);
                    pk[i] = *reinterpret_cast<const uint32_t*>(&b2);
                }
                tmem_st_32x16(tS + c * 16, pk);
            }
            const float sum = (sum2a.x + sum2a.y) + (sum2b.x + sum2b.y);
            l += sum;
            tmem_st_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(p_full(t));
        }
        // epilogue: O / l -> bf16, token-major store; log-sum-exp for the backward pass
        if (!mbar_wait(o_final, 0, &abort_flag)) goto done;
        tc_fence_after();
        const float inv = 1.f / l;
        const int b = bh / p.H, head = bh - b * p.H;
        __nv_bfloat16* orow = p.out + ((long)b * p.S + row) * ((long)p.H * D) + head * D;
        // remote destinations of this row (none, the token's owner, or everybody for a text row)
        int first_dst = 0, n_dst = 0;
        long drow = 0;
        if (p.push && row < p.S) {
            if (row < p.text_len) {
                n_dst = p.n_peers;
                drow = row;
            } else {
                const int v = row - p.text_len;
                first_dst = v / p.s_local;
                n_dst = first_dst < p.n_peers ? 1 : 0;
                drow = p.text_len + (v - first_dst * p.s_local);
            }
        }
        const long dcol = ((long)p.my_rank * p.H + head) * D;
#pragma unroll 1
        for (int c = 0; c < D / 32; ++c) {
            uint32_t r[32];
            tmem_ld_32x32(tO + c * 32, r);
            tmem_ld_wait();
            if (row < p.S) {
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                    float o[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) o[i] = __uint_as_float(r[g * 8 + i]) * inv;
                    const tt::bf16x8 pk = tt::pack8(o);
                    tt::st8(orow + c * 32 + g * 8, pk);
                    for (int d = 0; d < n_dst; ++d)
                        tt::st8(p.peer_out[first_dst + d] + drow * p.dest_ld + dcol + c * 32 + g * 8, pk);
                }
            }
        }
        if (row < p.S) p.lse[(long)bh * p.lse_pitch + row] = (m + log2f(l)) * 0.6931471805599453f;
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

// q, k, v: [BH, S, 128] bf16 contiguous; out [B, S, H*128] bf16; lse [BH, lse_pitch] fp32 (rows < S written).
static int attn_fwd_launch(const void* q, const void* k, const void* v, void* out, float* lse, int B, int H, int S,
                           int kv_len, int mask_lo, int mask_hi, int lse_pitch, float scale, int* status, void* stream,
                           void* const* peer_out, int n_peers, int my_rank, int text_len, int s_local, long dest_ld);

// Keys at and beyond kv_len are masked, and so are keys in [mask_lo, mask_hi) (pass mask_lo >= mask_hi for none); at least
// one key must stay visible.
extern "C" int tt_attn_fwd(const void* q, const void* k, const void* v, void* out, float* lse, int B, int H, int S,
                           int kv_len, int mask_lo, int mask_hi, int lse_pitch, float scale, int* status, void* stream) {
    return attn_fwd_launch(q, k, v, out, lse, B, H, S, kv_len, mask_lo, mask_hi, lse_pitch, scale, status, stream, nullptr,
                           0, 0, 0, 0, 0);
}

// Forward with the Ulysses head -> sequence all-to-all fused into the epilogue (batch 1).  The sequence is
// [text_len text tokens | n_peers * s_local video tokens]; peer_out[r] is rank r's gathered buffer
// [text_len + s_local, dest_ld] (dest_ld = n_peers * H * 128) and receives this rank's H heads at columns
// [my_rank * H * 128, (my_rank + 1) * H * 128).  `out` still receives the local head-sharded copy for the backward.
extern "C" int tt_attn_fwd_push(const void* q, const void* k, const void* v, void* out, float* lse, int H, int S,
                                int kv_len, int mask_lo, int mask_hi, int lse_pitch, float scale, int* status, void* stream,
                                void* const* peer_out, int n_peers, int my_rank, int text_len, int s_local, long dest_ld) {
    if (peer_out == nullptr || n_peers < 1 || n_peers > TT_MAX_PEERS || my_rank < 0 || my_rank >= n_peers) return TT_ERR_ARG;
    if (text_len < 0 || s_local <= 0 || text_len + (long)n_peers * s_local != S || (dest_ld & 7)) return TT_ERR_ARG;
    return attn_fwd_launch(q, k, v, out, lse, 1, H, S, kv_len, mask_lo, mask_hi, lse_pitch, scale, status, stream, peer_out,
                           n_peers, my_rank, text_len, s_local, dest_ld);
}

static int attn_fwd_launch(const void* q, const void* k, const void* v, void* out, float* lse, int B, int H, int S,
                           int kv_len, int mask_lo, int mask_hi, int lse_pitch, float scale, int* status, void* stream,
                           void* const* peer_out, int n_peers, int my_rank, int text_len, int s_local, long dest_ld) {
    if (B <= 0 || H <= 0 || S <= 0 || kv_len <= 0 || kv_len > S || lse_pitch < S || status == nullptr) return TT_ERR_ARG;
    if (mask_lo < mask_hi && (mask_lo < 0 || (mask_lo == 0 && mask_hi >= kv_len))) return TT_ERR_ARG;
    CUtensorMap tq, tk, tv;
    int rc;
    const uint64_t BH = (uint64_t)B * H;
    if ((rc = tt_make_tmap_3d(&tq, q, BH, (uint64_t)S, D, D, (uint64_t)S * D, BQ, 64)) != TT_OK) return rc;
    if ((rc = tt_make_tmap_3d(&tk, k, BH, (uint64_t)S, D, D, (uint64_t)S * D, BKV, 64)) != TT_OK) return rc;
    if ((rc = tt_make_tmap_3d(&tv, v, BH, (uint64_t)S, D, D, (uint64_t)S * D, BKV, 64)) != TT_OK) return rc;
    static bool configured[64] = {false};       // per device: the attribute belongs to the device's context
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
    if (!configured[dev]) {
        cudaError_t e = cudaFuncSetAttribute(attn_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
        if (e != cudaSuccess) return tt_record_cuda(e);
        configured[dev] = true;
    }
    AttnParams p;
    p.out = (__nv_bfloat16*)out;
    p.lse = lse;
    p.lse_pitch = lse_pitch;
    p.S = S;
    p.kv_len = kv_len;
    p.mask_lo = mask_lo;
    p.mask_hi = mask_lo < mask_hi ? mask_hi : mask_lo;
    p.H = H;
    p.scale_log2 = scale * 1.4426950408889634f;
    p.status = status;
    p.push = peer_out != nullptr ? 1 : 0;
    p.n_peers = n_peers;
    p.my_rank = my_rank;
    p.text_len = text_len;
    p.s_local = s_local;
    p.dest_ld = dest_ld;
    for (int r = 0; r < TT_MAX_PEERS; ++r) p.peer_out[r] = (peer_out != nullptr && r < n_peers) ? (__nv_bfloat16*)peer_out[r] : nullptr;
    dim3 grid((S + 2 * BQ - 1) / (2 * BQ), (unsigned)BH);
    attn_fwd_kernel<<<grid, kThreads, kSmemBytes, (cudaStream_t)stream>>>(tq, tk, tv, p);
    TT_CHECK_LAUNCH();
    return TT_OK;
}
