// Fused AdamW on flat ranges: bf16 weights and gradients, fp32 or bf16 moments, and either an fp32
// master copy or a 16-bit remainder that together with the bf16 weight reconstructs the fp32 master
// exactly (master_bits = (bf16_bits << 16) + int16 remainder).
//
// Plays the role of apex / TransformerEngine FusedAdam under Megatron's DistributedOptimizer in the
// reference (teletron/core/training.py:36-43), with the gradient scale (1/(dp*cp) or the clip
// coefficient) folded in so no separate cast / scale pass over the gradients is needed.
#include "common.cuh"
#include "teletron_b200.h"

namespace {
using namespace tt;

template <typename T>
__device__ __forceinline__ void load8f(const T* p, float* f);
template <>
__device__ __forceinline__ void load8f<float>(const float* p, float* f) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}
template <>
__device__ __forceinline__ void load8f<__nv_bfloat16>(const __nv_bfloat16* p, float* f) {
    unpack8(ld8(p), f);
}
template <typename T>
__device__ __forceinline__ void store8f(T* p, const float* f);
template <>
__device__ __forceinline__ void store8f<float>(float* p, const float* f) {
    *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(f[4], f[5], f[6], f[7]);
}
template <>
__device__ __forceinline__ void store8f<__nv_bfloat16>(__nv_bfloat16* p, const float* f) {
    st8(p, pack8(f));
}

// MODE 0: fp32 master; 1: split16 remainder; 2: bf16 weights only
template <typename ST, int MODE>
__global__ void __launch_bounds__(256) adamw_kernel(__nv_bfloat16* __restrict__ param, const __nv_bfloat16* __restrict__ grad,
                                                   ST* __restrict__ m, ST* __restrict__ v, float* __restrict__ master,
                                                   int16_t* __restrict__ lo, long nvec, float lr, float beta1, float beta2,
                                                   float eps, float wd, float bc1, float bc2, float gscale) {
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (long)gridDim.x * blockDim.x) {
        const long o = i * 8;
        float g[8], mm[8], vv[8], w[8];
        unpack8(ld8(grad + o), g);
        load8f<ST>(m + o, mm);
        load8f<ST>(v + o, vv);
        if (MODE == 0) {
            load8f<float>(master + o, w);
        } else if (MODE == 1) {
            const uint4 pb = *reinterpret_cast<const uint4*>(param + o);
            const uint4 lb = *reinterpret_cast<const uint4*>(lo + o);
            const unsigned short* ps = reinterpret_cast<const unsigned short*>(&pb);
            const short* ls = reinterpret_cast<const short*>(&lb);
#pragma unroll
            for (int j = 0; j < 8; ++j) w[j] = __int_as_float((int)((unsigned)ps[j] << 16) + (int)ls[j]);
        } else {
            unpack8(ld8(param + o), w);
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float gj = g[j] * gscale;
            mm[j] = beta1 * mm[j] + (1.f - beta1) * gj;
            vv[j] = beta2 * vv[j] + (1.f - beta2) * gj * gj;
            const float upd = (mm[j] / bc1) / (sqrtf(vv[j] / bc2) + eps);
            w[j] = w[j] * (1.f - lr * wd) - lr * upd;
        }
        store8f<ST>(m + o, mm);
        store8f<ST>(v + o, vv);
        if (MODE == 1) {
            // weight = fp32 bits rounded half-up in magnitude to 16 bits; the remainder always fits int16
            uint4 pb, lb;
            unsigned short* ps = reinterpret_cast<unsigned short*>(&pb);
            short* ls = reinterpret_cast<short*>(&lb);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const unsigned bits = __float_as_uint(w[j]);
                const unsigned hi = (bits + 0x8000u) >> 16;
                ps[j] = (unsigned short)hi;
                ls[j] = (short)(int)(bits - (hi << 16));
            }
            *reinterpret_cast<uint4*>(param + o) = pb;
            *reinterpret_cast<uint4*>(lo + o) = lb;
        } else {
            st8(param + o, pack8(w));
            if (MODE == 0) store8f<float>(master + o, w);
        }
    }
}
struct PeerTable {
    void* ptr[TT_MAX_PEERS];
};

// Gradient reduce-scatter + AdamW + parameter all-gather in one pass over this rank's shard [offset, offset + 8 nvec) of the
// flat buffers: the bf16 gradients of all n_g sources are read (peer loads over NVLink, all issued before the first is
// used), summed in fp32 and scaled; the moments and the master weight of the shard are updated; the new bf16 weight is
// stored into all n_p parameter buffers (peer stores).  NVLink carries the gradient reads in one direction and the
// parameter writes in the other at the same time.  n_g = 1 with the local buffer gives AdamW + all-gather on an already
// reduced shard; n_g = n_p = 1 is the plain update.
template <typename ST, int MODE>
__global__ void __launch_bounds__(256) rs_adamw_ag_kernel(PeerTable grads, int n_g, PeerTable params, int n_p, int my_p,
                                                         long offset, ST* __restrict__ m, ST* __restrict__ v,
                                                         float* __restrict__ master, int16_t* __restrict__ lo, long nvec,
                                                         float lr, float beta1, float beta2, float eps, float wd, float bc1,
                                                         float bc2, float gscale) {
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (long)gridDim.x * blockDim.x) {
        const long o = i * 8;
        bf16x8 t[TT_MAX_PEERS];
#pragma unroll
        for (int r = 0; r < TT_MAX_PEERS; ++r)
            if (r < n_g) t[r] = ld8(reinterpret_cast<const __nv_bfloat16*>(grads.ptr[r]) + offset + o);
        float g[8], mm[8], vv[8], w[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) g[j] = 0.f;
#pragma unroll
        for (int r = 0; r < TT_MAX_PEERS; ++r) {
            if (r < n_g) {
                float f[8];
                unpack8(t[r], f);
#pragma unroll
                for (int j = 0; j < 8; ++j) g[j] += f[j];
            }
        }
        load8f<ST>(m + o, mm);
        load8f<ST>(v + o, vv);
        const __nv_bfloat16* own = reinterpret_cast<const __nv_bfloat16*>(params.ptr[my_p]) + offset + o;
        if (MODE == 0) {
            load8f<float>(master + o, w);
        } else if (MODE == 1) {
            const uint4 pb = *reinterpret_cast<const uint4*>(own);
            const uint4 lb = *reinterpret_cast<const uint4*>(lo + o);
            const unsigned short* ps = reinterpret_cast<const unsigned short*>(&pb);
            const short* ls = reinterpret_cast<const short*>(&lb);
#pragma unroll
            for (int j = 0; j < 8; ++j) w[j] = __int_as_float((int)((unsigned)ps[j] << 16) + (int)ls[j]);
        } else {
            unpack8(ld8(own), w);
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float gj = g[j] * gscale;
            mm[j] = beta1 * mm[j] + (1.f - beta1) * gj;
            vv[j] = beta2 * vv[j] + (1.f - beta2) * gj * gj;
            const float upd = (mm[j] / bc1) / (sqrtf(vv[j] / bc2) + eps);
            w[j] = w[j] * (1.f - lr * wd) - lr * upd;
        }
        store8f<ST>(m + o, mm);
        store8f<ST>(v + o, vv);
        uint4 pb;
        if (MODE == 1) {
            uint4 lb;
            unsigned short* ps = reinterpret_cast<unsigned short*>(&pb);
            short* ls = reinterpret_cast<short*>(&lb);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const unsigned bits = __float_as_uint(w[j]);
                const unsigned hi = (bits + 0x8000u) >> 16;
                ps[j] = (unsigned short)hi;
                ls[j] = (short)(int)(bits - (hi << 16));
            }
            *reinterpret_cast<uint4*>(lo + o) = lb;
        } else {
            const bf16x8 pk = pack8(w);
            pb = *reinterpret_cast<const uint4*>(&pk);
            if (MODE == 0) store8f<float>(master + o, w);
        }
        for (int r = 0; r < n_p; ++r) *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(params.ptr[r]) + offset + o) = pb;
    }
}
}  // namespace

// Fused gradient reduce-scatter + AdamW + parameter all-gather on this rank's shard of the flat buffers (see the kernel).
//   grad_ptrs [n_g]: every source's bf16 gradient buffer base (peers' buffers, or only the local one when the shard is
//   already reduced); param_ptrs [n_p]: every destination's bf16 parameter buffer base, this rank's own at index my_p;
//   offset / n: the shard in elements of those buffers (multiples of 8); m, v, master / master_lo: shard-local state.
// The caller brackets the call with barriers of the heap that holds the buffers: all gradients complete before, all
// reads and stores done after.
extern "C" int tt_rs_adamw_ag(void* const* grad_ptrs, int n_g, void* const* param_ptrs, int n_p, int my_p, long offset,
                              void* m, void* v, float* master, void* master_lo, long n, int state_is_bf16, float lr,
                              float beta1, float beta2, float eps, float wd, int step, float grad_scale, void* stream) {
    if (n <= 0 || (n & 7) || (offset & 7) || offset < 0 || step < 1) return TT_ERR_ARG;
    if (n_g < 1 || n_g > TT_MAX_PEERS || n_p < 1 || n_p > TT_MAX_PEERS || my_p < 0 || my_p >= n_p) return TT_ERR_ARG;
    if (master != nullptr && master_lo != nullptr) return TT_ERR_ARG;
    PeerTable tg, tp;
    for (int r = 0; r < TT_MAX_PEERS; ++r) {
        tg.ptr[r] = r < n_g ? grad_ptrs[r] : nullptr;
        tp.ptr[r] = r < n_p ? param_ptrs[r] : nullptr;
    }
    const long nvec = n >> 3;
    long want = (nvec + 255) / 256;
    const int grid = (int)(want < 148L * 8 ? want : 148L * 8);
    const float bc1 = 1.f - powf(beta1, (float)step), bc2 = 1.f - powf(beta2, (float)step);
    cudaStream_t st = (cudaStream_t)stream;
    const int mode = master != nullptr ? 0 : (master_lo != nullptr ? 1 : 2);
#define FUSED(ST, MODE)                                                                                             \
    rs_adamw_ag_kernel<ST, MODE><<<grid, 256, 0, st>>>(tg, n_g, tp, n_p, my_p, offset, (ST*)m, (ST*)v, master,      \
                                                       (int16_t*)master_lo, nvec, lr, beta1, beta2, eps, wd, bc1,   \
                                                       bc2, grad_scale)
    if (state_is_bf16) {
        if (mode == 0) FUSED(__nv_bfloat16, 0);
        else if (mode == 1) FUSED(__nv_bfloat16, 1);
        else FUSED(__nv_bfloat16, 2);
    } else {
        if (mode == 0) FUSED(float, 0);
        else if (mode == 1) FUSED(float, 1);
        else FUSED(float, 2);
    }
#undef FUSED
    TT_CHECK_LAUNCH();
    return TT_OK;
}

extern "C" int tt_adamw(void* param, const void* grad, void* m, void* v, float* master, void* master_lo, long n,
                        int state_is_bf16, float lr, float beta1, float beta2, float eps, float wd, int step,
                        float grad_scale, void* stream) {
    if (n <= 0 || (n & 7) || step < 1) return TT_ERR_ARG;
    if (master != nullptr && master_lo != nullptr) return TT_ERR_ARG;
    const long nvec = n >> 3;
    long want = (nvec + 255) / 256;
    const int grid = (int)(want < 148L * 16 ? want : 148L * 16);
    const float bc1 = 1.f - powf(beta1, (float)step), bc2 = 1.f - powf(beta2, (float)step);
    cudaStream_t st = (cudaStream_t)stream;
    const int mode = master != nullptr ? 0 : (master_lo != nullptr ? 1 : 2);
#define ADAM(ST, MODE)                                                                                               \
    adamw_kernel<ST, MODE><<<grid, 256, 0, st>>>((__nv_bfloat16*)param, (const __nv_bfloat16*)grad, (ST*)m, (ST*)v, \
                                                 master, (int16_t*)master_lo, nvec, lr, beta1, beta2, eps, wd, bc1,  \
                                                 bc2, grad_scale)
    if (state_is_bf16) {
        if (mode == 0) ADAM(__nv_bfloat16, 0);
        else if (mode == 1) ADAM(__nv_bfloat16, 1);
        else ADAM(__nv_bfloat16, 2);
    } else {
        if (mode == 0) ADAM(float, 0);
        else if (mode == 1) ADAM(float, 1);
        else ADAM(float, 2);
    }
    TT_CHECK_LAUNCH();
    return TT_OK;
}
