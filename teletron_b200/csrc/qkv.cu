// QKV post-processing: per-head split of the packed QKV GEMM output, QK-RMSNorm, rotary embedding
// and the change to head-major layout, forward and backward, in one pass each.
//
// The reference runs this as view/split/transpose + two RMSNorm launches + two diffusers
// `apply_rotary_emb` calls + permute/contiguous copies + torch.cat with the text tokens
// (teletron/models/dit/dit_attention.py:191-212, 260-273, 295-297).  Here one kernel reads the GEMM
// output `[rows, heads*3*128]` (row layout `[head][q|k|v][128]`) once and writes q, k, v straight
// into `[batch, heads, seq_out, 128]` buffers at a token offset, so the video and the text stream
// land in one concatenated sequence without a copy.
#include "common.cuh"
#include "teletron_b200.h"

namespace {

using namespace tt;

constexpr int D = 128;   // head dim: one warp covers a head vector with 4 elements per lane

struct alignas(8) bf16x4 {
    __nv_bfloat162 a, b;
};

__device__ __forceinline__ void ld4(const __nv_bfloat16* p, float* f) {
    bf16x4 r;
    *reinterpret_cast<uint2*>(&r) = *reinterpret_cast<const uint2*>(p);
    float2 t0 = __bfloat1622float2(r.a), t1 = __bfloat1622float2(r.b);
    f[0] = t0.x; f[1] = t0.y; f[2] = t1.x; f[3] = t1.y;
}

__device__ __forceinline__ void st4(__nv_bfloat16* p, const float* f) {
    bf16x4 r;
    r.a = __floats2bfloat162_rn(f[0], f[1]);
    r.b = __floats2bfloat162_rn(f[2], f[3]);
    *reinterpret_cast<uint2*>(p) = *reinterpret_cast<const uint2*>(&r);
}

// Sum over the 16 lanes that share one (token, head) item.
__device__ __forceinline__ float half_warp_sum(float v) {
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// RoPE on 8 consecutive elements (4 interleaved pairs) with per-element tables; `t` = +1 forward, -1 transpose.
__device__ __forceinline__ void rope8(float* v, const float* c, const float* s) {
#pragma unroll
    for (int i = 0; i < 8; i += 2) {
        const float a0 = v[i], a1 = v[i + 1];
        v[i] = a0 * c[i] - a1 * s[i];
        v[i + 1] = a1 * c[i + 1] + a0 * s[i + 1];
    }
}
__device__ __forceinline__ void rope8_transpose(float* v, const float* c, const float* s) {
#pragma unroll
    for (int i = 0; i < 8; i += 2) {
        const float a0 = v[i], a1 = v[i + 1];
        v[i] = a0 * c[i] + a1 * s[i + 1];
        v[i + 1] = a1 * c[i + 1] - a0 * s[i];
    }
}
__device__ __forceinline__ void ldf8(const float* p, float* f) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}

// Sixteen lanes per (token, head) item, 16-byte accesses, two items per warp and two such pairs per iteration: every
// lane keeps six 16-byte loads in flight.  (With one warp per item and 8-byte accesses the kernel reached 0.6 of the
// copy bandwidth forward and 0.3 backward.)
__global__ void __launch_bounds__(256, 3) qkv_post_fwd_kernel(
    const __nv_bfloat16* __restrict__ qkv, const __nv_bfloat16* __restrict__ qw, const __nv_bfloat16* __restrict__ kw,
    const float* __restrict__ cos_t, const float* __restrict__ sin_t, __nv_bfloat16* __restrict__ q,
    __nv_bfloat16* __restrict__ k, __nv_bfloat16* __restrict__ v, long rows, int heads, long seq_in, long seq_out,
    long out_offset, long rope_len, float eps) {
    constexpr int U = 2;
    const int lane = threadIdx.x & 31, sub = lane >> 4, l = lane & 15;
    const long nwork = rows * heads;
    const long warp_id = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const long stride = (long)gridDim.x * (blockDim.x >> 5) * (2 * U);
    float wq[8], wk[8];
    unpack8(ld8(qw + l * 8), wq);
    unpack8(ld8(kw + l * 8), wk);
    for (long w0 = warp_id * (2 * U); w0 < nwork; w0 += stride) {
        bf16x8 pq[U], pk[U], pv[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const long w = w0 + u * 2 + sub;
            if (w < nwork) {
                const __nv_bfloat16* src = qkv + w * (3L * D) + l * 8;
                pq[u] = ld8(src);
                pk[u] = ld8(src + D);
                pv[u] = ld8(src + 2 * D);
            } else {
                pq[u] = pk[u] = pv[u] = bf16x8{};
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const long w = w0 + u * 2 + sub;
            const bool ok = w < nwork;
            const long row = ok ? w / heads : 0;
            const int h = ok ? (int)(w - row * heads) : 0;
            const long b = row / seq_in, s = row - b * seq_in;
            const long dst = ((b * heads + h) * seq_out + out_offset + s) * D + l * 8;
            float xq[8], xk[8];
            unpack8(pq[u], xq);
            unpack8(pk[u], xk);
            float sq = 0.f, sk = 0.f;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                sq += xq[j] * xq[j];
                sk += xk[j] * xk[j];
            }
            const float rq = rsqrtf(half_warp_sum(sq) * (1.f / D) + eps);
            const float rk = rsqrtf(half_warp_sum(sk) * (1.f / D) + eps);
            if (ok) {
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    // the reference rounds the normalised value to bf16 before the rotation; keep fp32 instead
                    xq[j] *= rq * wq[j];
                    xk[j] *= rk * wk[j];
                }
                if (s < rope_len) {
                    float c[8], sn[8];
                    ldf8(cos_t + s * D + l * 8, c);
                    ldf8(sin_t + s * D + l * 8, sn);
                    rope8(xq, c, sn);
                    rope8(xk, c, sn);
                }
                st8(q + dst, pack8(xq));
                st8(k + dst, pack8(xk));
                st8(v + dst, pv[u]);
            }
        }
    }
}

struct PeerTable3 {
    const __nv_bfloat16* q[TT_MAX_PEERS];
    const __nv_bfloat16* k[TT_MAX_PEERS];
    const __nv_bfloat16* v[TT_MAX_PEERS];
};

// partials: [gridDim.x * warps][2][128] fp32 (dq-norm weight, dk-norm weight)
// dq / dk / dv live head-sharded on the rank that owns each head ([batch, heads_per_rank, seq_out, 128]); with
// more than one rank this kernel reads them over NVLink, which is the head -> sequence all-to-all of the
// Ulysses backward fused with the RoPE transpose and the RMSNorm backward.  Same lane layout as the forward kernel:
// sixteen lanes per (token, head) item, whole 256-byte rows per half-warp on the peer side.
__global__ void __launch_bounds__(256, 3) qkv_post_bwd_kernel(
    const PeerTable3 src, const int heads_per_rank, const __nv_bfloat16* __restrict__ qkv,
    const __nv_bfloat16* __restrict__ qw, const __nv_bfloat16* __restrict__ kw,
    const float* __restrict__ cos_t, const float* __restrict__ sin_t, __nv_bfloat16* __restrict__ dqkv,
    float* __restrict__ partials, long rows, int heads, long seq_in, long seq_out, long out_offset, long rope_len,
    float eps) {
    constexpr int U = 1;      // with two items per lane the kernel needed 156 registers: one CTA per SM
    const int lane = threadIdx.x & 31, sub = lane >> 4, l = lane & 15;
    const long nwork = rows * heads;
    const long gw = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const long stride = (long)gridDim.x * (blockDim.x >> 5) * (2 * U);
    float wq[8], wk[8], aq[8], ak[8];
    unpack8(ld8(qw + l * 8), wq);
    unpack8(ld8(kw + l * 8), wk);
#pragma unroll
    for (int j = 0; j < 8; ++j) aq[j] = ak[j] = 0.f;
    for (long w0 = gw * (2 * U); w0 < nwork; w0 += stride) {
        bf16x8 pgq[U], pgk[U], pgv[U], pxq[U], pxk[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const long w = w0 + u * 2 + sub;
            if (w < nwork) {
                const long row = w / heads;
                const int h = (int)(w - row * heads);
                const long b = row / seq_in, s = row - b * seq_in;
                const int owner = h / heads_per_rank, hl = h - owner * heads_per_rank;
                const long so = ((b * heads_per_rank + hl) * seq_out + out_offset + s) * D + l * 8;
                pgq[u] = ld8(src.q[owner] + so);
                pgk[u] = ld8(src.k[owner] + so);
                pgv[u] = ld8(src.v[owner] + so);
                pxq[u] = ld8(qkv + w * (3L * D) + l * 8);
                pxk[u] = ld8(qkv + w * (3L * D) + D + l * 8);
            } else {
                pgq[u] = pgk[u] = pgv[u] = pxq[u] = pxk[u] = bf16x8{};
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const long w = w0 + u * 2 + sub;
            const bool ok = w < nwork;
            const long row = ok ? w / heads : 0;
            const long b = row / seq_in, s = row - b * seq_in;
            float gq[8], gk[8], xq[8], xk[8];
            unpack8(pgq[u], gq);
            unpack8(pgk[u], gk);
            unpack8(pxq[u], xq);
            unpack8(pxk[u], xk);
            if (ok && s < rope_len) {        // transpose of the rotation
                float c[8], sn[8];
                ldf8(cos_t + s * D + l * 8, c);
                ldf8(sin_t + s * D + l * 8, sn);
                rope8_transpose(gq, c, sn);
                rope8_transpose(gk, c, sn);
            }
            float sq = 0.f, sk = 0.f;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                sq += xq[j] * xq[j];
                sk += xk[j] * xk[j];
            }
            const float rq = rsqrtf(half_warp_sum(sq) * (1.f / D) + eps);
            const float rk = rsqrtf(half_warp_sum(sk) * (1.f / D) + eps);
            float cq = 0.f, ck = 0.f;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                xq[j] *= rq;                 // x_hat
                xk[j] *= rk;
                aq[j] += gq[j] * xq[j];
                ak[j] += gk[j] * xk[j];
                gq[j] *= wq[j];
                gk[j] *= wk[j];
                cq += gq[j] * xq[j];
                ck += gk[j] * xk[j];
            }
            cq = half_warp_sum(cq) * (1.f / D);
            ck = half_warp_sum(ck) * (1.f / D);
            if (ok) {
                float oq[8], okk[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    oq[j] = rq * (gq[j] - xq[j] * cq);
                    okk[j] = rk * (gk[j] - xk[j] * ck);
                }
                __nv_bfloat16* dst = dqkv + w * (3L * D) + l * 8;
                st8(dst, pack8(oq));
                st8(dst + D, pack8(okk));
                st8(dst + 2 * D, pgv[u]);
            }
        }
    }
    // the two halves of the warp own the same columns
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        aq[j] += __shfl_xor_sync(0xffffffffu, aq[j], 16);
        ak[j] += __shfl_xor_sync(0xffffffffu, ak[j], 16);
    }
    if (sub == 0) {
        float* p = partials + gw * (2L * D) + l * 8;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            p[j] = aq[j];
            p[D + j] = ak[j];
        }
    }
}

__global__ void __launch_bounds__(1024) qkv_weight_finalize_kernel(const float* __restrict__ partials,
                                                                   __nv_bfloat16* __restrict__ dqw,
                                                                   __nv_bfloat16* __restrict__ dkw, int nparts) {
    // One block (fixed summation order => deterministic).  1024 threads = 4 row groups x 256 columns; every thread
    // keeps 8 independent loads in flight, then the 4 groups are folded through shared memory in a fixed order.
    __shared__ float fold[4][256];
    const int c = threadIdx.x & 255, g = threadIdx.x >> 8;
    float acc[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) acc[u] = 0.f;
    int i = g;
    for (; i + 28 < nparts; i += 32) {
#pragma unroll
        for (int u = 0; u < 8; ++u) acc[u] += partials[(long)(i + 4 * u) * 256 + c];
    }
    for (; i < nparts; i += 4) acc[0] += partials[(long)i * 256 + c];
    fold[g][c] = ((acc[0] + acc[1]) + (acc[2] + acc[3])) + ((acc[4] + acc[5]) + (acc[6] + acc[7]));
    __syncthreads();
    if (g == 0) {
        const float s = (fold[0][c] + fold[1][c]) + (fold[2][c] + fold[3][c]);
        if (c < D) dqw[c] = __float2bfloat16(s);
        else dkw[c - D] = __float2bfloat16(s);
    }
}

inline int pick_grid(long nwork) {
    long want = (nwork + 7) / 8;
    long cap = TT_QKV_MAX_PARTIAL_WARPS / 8;
    return (int)(want < cap ? want : cap);
}

}  // namespace

extern "C" int tt_qkv_partial_warps(long rows, int heads) { return pick_grid(rows * heads) * 8; }

extern "C" int tt_qkv_post_fwd(const void* qkv, const void* qw, const void* kw, const float* cos_t, const float* sin_t,
                               void* q, void* k, void* v, long rows, int heads, long seq_in, long seq_out,
                               long out_offset, long rope_len, float eps, void* stream) {
    if (rows <= 0 || heads <= 0 || seq_in <= 0 || rows % seq_in || out_offset < 0 || out_offset + seq_in > seq_out)
        return TT_ERR_ARG;
    if (rope_len > 0 && (cos_t == nullptr || sin_t == nullptr)) return TT_ERR_ARG;
    qkv_post_fwd_kernel<<<pick_grid(rows * heads), 256, 0, (cudaStream_t)stream>>>(
        (const __nv_bfloat16*)qkv, (const __nv_bfloat16*)qw, (const __nv_bfloat16*)kw, cos_t, sin_t, (__nv_bfloat16*)q,
        (__nv_bfloat16*)k, (__nv_bfloat16*)v, rows, heads, seq_in, seq_out, out_offset, rope_len, eps);
    TT_CHECK_LAUNCH();
    return TT_OK;
}

// dq_ptrs / dk_ptrs / dv_ptrs [n]: rank r's [batch, heads / n, seq_out, 128] gradient buffers (n = 1: local).
extern "C" int tt_qkv_post_bwd_peer(void* const* dq_ptrs, void* const* dk_ptrs, void* const* dv_ptrs, int n,
                                    const void* qkv, const void* qw, const void* kw, const float* cos_t,
                                    const float* sin_t, void* dqkv, float* partials, void* dqw, void* dkw, long rows,
                                    int heads, long seq_in, long seq_out, long out_offset, long rope_len, float eps,
                                    void* stream) {
    if (rows <= 0 || heads <= 0 || seq_in <= 0 || rows % seq_in || out_offset < 0 || out_offset + seq_in > seq_out)
        return TT_ERR_ARG;
    if (n < 1 || n > TT_MAX_PEERS || heads % n) return TT_ERR_ARG;
    if (rope_len > 0 && (cos_t == nullptr || sin_t == nullptr)) return TT_ERR_ARG;
    PeerTable3 t;
    for (int r = 0; r < TT_MAX_PEERS; ++r) {
        t.q[r] = (const __nv_bfloat16*)(r < n ? dq_ptrs[r] : nullptr);
        t.k[r] = (const __nv_bfloat16*)(r < n ? dk_ptrs[r] : nullptr);
        t.v[r] = (const __nv_bfloat16*)(r < n ? dv_ptrs[r] : nullptr);
    }
    cudaStream_t st = (cudaStream_t)stream;
    const int grid = pick_grid(rows * heads);
    qkv_post_bwd_kernel<<<grid, 256, 0, st>>>(t, heads / n, (const __nv_bfloat16*)qkv, (const __nv_bfloat16*)qw,
                                              (const __nv_bfloat16*)kw, cos_t, sin_t, (__nv_bfloat16*)dqkv, partials,
                                              rows, heads, seq_in, seq_out, out_offset, rope_len, eps);
    TT_CHECK_LAUNCH();
    qkv_weight_finalize_kernel<<<1, 1024, 0, st>>>(partials, (__nv_bfloat16*)dqw, (__nv_bfloat16*)dkw, grid * 8);
    TT_CHECK_LAUNCH();
    return TT_OK;
}

extern "C" int tt_qkv_post_bwd(const void* dq, const void* dk, const void* dv, const void* qkv, const void* qw,
                               const void* kw, const float* cos_t, const float* sin_t, void* dqkv, float* partials,
                               void* dqw, void* dkw, long rows, int heads, long seq_in, long seq_out, long out_offset,
                               long rope_len, float eps, void* stream) {
    void* q1[1] = {const_cast<void*>(dq)};
    void* k1[1] = {const_cast<void*>(dk)};
    void* v1[1] = {const_cast<void*>(dv)};
    return tt_qkv_post_bwd_peer(q1, k1, v1, 1, qkv, qw, kw, cos_t, sin_t, dqkv, partials, dqw, dkw, rows, heads, seq_in,
                                seq_out, out_offset, rope_len, eps, stream);
}
