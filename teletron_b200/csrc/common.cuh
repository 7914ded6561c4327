// Shared device helpers for the teletron_b200 kernels (sm_100a).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define TT_OK 0
#define TT_ERR_ARG 1        // bad shape / alignment / size
#define TT_ERR_CUDA 2       // a CUDA runtime call failed (see tt_last_cuda_error)
#define TT_ERR_TIMEOUT 3    // a bounded device-side wait ran out
#define TT_ERR_LIMIT 4      // size beyond a compiled-in maximum

namespace tt {

struct alignas(16) bf16x8 {
    __nv_bfloat162 v[4];
};

__device__ __forceinline__ bf16x8 ld8(const __nv_bfloat16* p) {
    bf16x8 r;
    *reinterpret_cast<uint4*>(&r) = *reinterpret_cast<const uint4*>(p);
    return r;
}

__device__ __forceinline__ void st8(__nv_bfloat16* p, const bf16x8& r) {
    *reinterpret_cast<uint4*>(p) = *reinterpret_cast<const uint4*>(&r);
}

__device__ __forceinline__ void unpack8(const bf16x8& r, float* f) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float2 t = __bfloat1622float2(r.v[i]);
        f[2 * i] = t.x;
        f[2 * i + 1] = t.y;
    }
}

__device__ __forceinline__ bf16x8 pack8(const float* f) {
    bf16x8 r;
#pragma unroll
    for (int i = 0; i < 4; ++i) r.v[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    return r;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Sum of `v` over the whole CTA; every thread gets the result. `smem` needs 32 floats.
__device__ __forceinline__ float block_sum(float v, float* smem) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();            // protect smem from the previous use
    if (lane == 0) smem[warp] = v;
    __syncthreads();
    float r = (lane < nwarps) ? smem[lane] : 0.f;
    return warp_sum(r);
}

// Two sums at once (saves a barrier pair). `smem` needs 64 floats.
__device__ __forceinline__ float2 block_sum2(float a, float b, float* smem) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    a = warp_sum(a);
    b = warp_sum(b);
    __syncthreads();
    if (lane == 0) {
        smem[warp] = a;
        smem[32 + warp] = b;
    }
    __syncthreads();
    float ra = (lane < nwarps) ? smem[lane] : 0.f;
    float rb = (lane < nwarps) ? smem[32 + lane] : 0.f;
    return make_float2(warp_sum(ra), warp_sum(rb));
}

__device__ __forceinline__ float gelu_erf(float x) { return 0.5f * x * (1.f + erff(x * 0.70710678118654752f)); }

__device__ __forceinline__ float gelu_erf_grad(float x) {
    const float cdf = 0.5f * (1.f + erff(x * 0.70710678118654752f));
    const float pdf = 0.3989422804014327f * __expf(-0.5f * x * x);
    return cdf + x * pdf;
}

__device__ __forceinline__ float gelu_tanh(float x) {
    const float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
    return 0.5f * x * (1.f + tanhf(u));
}

__device__ __forceinline__ float gelu_tanh_grad(float x) {
    const float x2 = x * x;
    const float u = 0.7978845608028654f * (x + 0.044715f * x * x2);
    const float t = tanhf(u);
    const float du = 0.7978845608028654f * (1.f + 3.f * 0.044715f * x2);
    return 0.5f * (1.f + t) + 0.5f * x * (1.f - t * t) * du;
}

}  // namespace tt

// Host-side: remember the last CUDA error for diagnostics.
extern "C" const char* tt_last_cuda_error();
int tt_record_cuda(cudaError_t e);

#define TT_CHECK_LAUNCH()                                   \
    do {                                                    \
        cudaError_t _e = cudaGetLastError();                \
        if (_e != cudaSuccess) return tt_record_cuda(_e);   \
    } while (0)
