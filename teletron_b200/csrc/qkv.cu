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

__global__ void __launch_bounds__(256) qkv_post_fwd_kernel(
    const __nv_bfloat16* __restrict__ qkv, const __nv_bfloat16* __restrict__ qw, const __nv_bfloat16* __restrict__ kw,
    const float* __restrict__ cos_t, const float* __restrict__ sin_t, __nv_bfloat16* __restrict__ q,
    __nv_bfloat16* __restrict__ k, __nv_bfloat16* __restrict__ v, long rows, int heads, long seq_in, long seq_out,
    long out_offset, long rope_len, float eps) {
    const int lane = threadIdx.x & 31;
    const long nwork = rows * heads;
    const long stride = (long)gridDim.x * (blockDim.x >> 5);
    float wq[4], wk[4];
    ld4(qw + lane * 4, wq);
    ld4(kw + lane * 4, wk);
    for (long w = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); w < nwork; w += stride) {
        const long row = w / heads;
        const int h = (int)(w - row * heads);
        const long b = row / seq_in, s = row - b * seq_in;
        const __nv_bfloat16* src = qkv + (row * heads + h) * (3L * D) + lane * 4;
        const long dst = ((b * heads + h) * seq_out + out_offset + s) * D + lane * 4;
        float xq[4], xk[4];
        ld4(src, xq);
        ld4(src + D, xk);
        // v: plain copy
        *reinterpret_cast<uint2*>(v + dst) = *reinterpret_cast<const uint2*>(src + 2 * D);
        float sq = xq[0] * xq[0] + xq[1] * xq[1] + xq[2] * xq[2] + xq[3] * xq[3];
        float sk = xk[0] * xk[0] + xk[1] * xk[1] + xk[2] * xk[2] + xk[3] * xk[3];
        const float rq = rsqrtf(warp_sum(sq) * (1.f / D) + eps);
        const float rk = rsqrtf(warp_sum(sk) * (1.f / D) + eps);
        float nq[4], nk[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            // the reference rounds the normalised value to bf16 before the rotation; keep fp32 instead
            nq[j] = xq[j] * rq * wq[j];
            nk[j] = xk[j] * rk * wk[j];
        }
        if (s < rope_len) {
            const float4 c = *reinterpret_cast<const float4*>(cos_t + s * D + lane * 4);
            const float4 sn = *reinterpret_cast<const float4*>(sin_t + s * D + lane * 4);
            float oq[4], ok[4];
            oq[0] = nq[0] * c.x - nq[1] * sn.x;
            oq[1] = nq[1] * c.y + nq[0] * sn.y;
            oq[2] = nq[2] * c.z - nq[3] * sn.z;
            oq[3] = nq[3] * c.w + nq[2] * sn.w;
            ok[0] = nk[0] * c.x - nk[1] * sn.x;
            ok[1] = nk[1] * c.y + nk[0] * sn.y;
            ok[2] = nk[2] * c.z - nk[3] * sn.z;
            ok[3] = nk[3] * c.w + nk[2] * sn.w;
            st4(q + dst, oq);
            st4(k + dst, ok);
        } else {
            st4(q + dst, nq);
            st4(k + dst, nk);
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
// Ulysses backward fused with the RoPE transpose and the RMSNorm backward.
__global__ void __launch_bounds__(256) qkv_post_bwd_kernel(
    const PeerTable3 src, const int heads_per_rank, const __nv_bfloat16* __restrict__ qkv,
    const __nv_bfloat16* __restrict__ qw, const __nv_bfloat16* __restrict__ kw,
    const float* __restrict__ cos_t, const float* __restrict__ sin_t, __nv_bfloat16* __restrict__ dqkv,
    float* __restrict__ partials, long rows, int heads, long seq_in, long seq_out, long out_offset, long rope_len,
    float eps) {
    const int lane = threadIdx.x & 31;
    const long nwork = rows * heads;
    const long gw = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const long stride = (long)gridDim.x * (blockDim.x >> 5);
    float wq[4], wk[4], aq[4] = {0.f, 0.f, 0.f, 0.f}, ak[4] = {0.f, 0.f, 0.f, 0.f};
    ld4(qw + lane * 4, wq);
    ld4(kw + lane * 4, wk);
    for (long w = gw; w < nwork; w += stride) {
        const long row = w / heads;
        const int h = (int)(w - row * heads);
        const long b = row / seq_in, s = row - b * seq_in;
        const long off_in = (row * heads + h) * (3L * D) + lane * 4;
        const int owner = h / heads_per_rank, hl = h - owner * heads_per_rank;
        const long so = ((b * heads_per_rank + hl) * seq_out + out_offset + s) * D + lane * 4;
        float gq[4], gk[4], xq[4], xk[4];
        ld4(src.q[owner] + so, gq);
        ld4(src.k[owner] + so, gk);
        ld4(qkv + off_in, xq);
        ld4(qkv + off_in + D, xk);
        *reinterpret_cast<uint2*>(dqkv + off_in + 2 * D) = *reinterpret_cast<const uint2*>(src.v[owner] + so);
        if (s < rope_len) {        // transpose of the rotation
            const float4 c = *reinterpret_cast<const float4*>(cos_t + s * D + lane * 4);
            const float4 sn = *reinterpret_cast<const float4*>(sin_t + s * D + lane * 4);
            float t[4];
            t[0] = gq[0] * c.x + gq[1] * sn.y;
            t[1] = gq[1] * c.y - gq[0] * sn.x;
            t[2] = gq[2] * c.z + gq[3] * sn.w;
            t[3] = gq[3] * c.w - gq[2] * sn.z;
#pragma unroll
            for (int j = 0; j < 4; ++j) gq[j] = t[j];
            t[0] = gk[0] * c.x + gk[1] * sn.y;
            t[1] = gk[1] * c.y - gk[0] * sn.x;
            t[2] = gk[2] * c.z + gk[3] * sn.w;
            t[3] = gk[3] * c.w - gk[2] * sn.z;
#pragma unroll
            for (int j = 0; j < 4; ++j) gk[j] = t[j];
        }
        float sq = 0.f, sk = 0.f;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            sq += xq[j] * xq[j];
            sk += xk[j] * xk[j];
        }
        const float rq = rsqrtf(warp_sum(sq) * (1.f / D) + eps);
        const float rk = rsqrtf(warp_sum(sk) * (1.f / D) + eps);
        float hq[4], hk[4], cq = 0.f, ck = 0.f;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            hq[j] = xq[j] * rq;
            hk[j] = xk[j] * rk;
            aq[j] += gq[j] * hq[j];
            ak[j] += gk[j] * hk[j];
            gq[j] *= wq[j];
            gk[j] *= wk[j];
            cq += gq[j] * hq[j];
            ck += gk[j] * hk[j];
        }
        cq = warp_sum(cq) * (1.f / D);
        ck = warp_sum(ck) * (1.f / D);
        float oq[4], ok[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            oq[j] = rq * (gq[j] - hq[j] * cq);
            ok[j] = rk * (gk[j] - hk[j] * ck);
        }
        st4(dqkv + off_in, oq);
        st4(dqkv + off_in + D, ok);
    }
    float* p = partials + gw * (2L * D) + lane * 4;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        p[j] = aq[j];
        p[D + j] = ak[j];
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
