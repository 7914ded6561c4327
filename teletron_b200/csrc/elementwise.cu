// GELU (erf / tanh) forward and backward on flat bf16 buffers; used where the activation is not
// already folded into a GEMM epilogue.
#include "common.cuh"
#include "teletron_b200.h"

namespace {
using namespace tt;

template <int KIND>
__global__ void __launch_bounds__(256) gelu_fwd_kernel(const __nv_bfloat16* __restrict__ u, __nv_bfloat16* __restrict__ y,
                                                      long nvec) {
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (long)gridDim.x * blockDim.x) {
        float f[8];
        unpack8(ld8(u + i * 8), f);
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] = KIND == 0 ? gelu_erf(f[j]) : gelu_tanh(f[j]);
        st8(y + i * 8, pack8(f));
    }
}

template <int KIND>
__global__ void __launch_bounds__(256) gelu_bwd_kernel(const __nv_bfloat16* __restrict__ dy,
                                                      const __nv_bfloat16* __restrict__ u, __nv_bfloat16* __restrict__ du,
                                                      long nvec) {
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (long)gridDim.x * blockDim.x) {
        float f[8], g[8];
        unpack8(ld8(u + i * 8), f);
        unpack8(ld8(dy + i * 8), g);
#pragma unroll
        for (int j = 0; j < 8; ++j) g[j] *= KIND == 0 ? gelu_erf_grad(f[j]) : gelu_tanh_grad(f[j]);
        st8(du + i * 8, pack8(g));
    }
}

inline int grid_for(long nvec) {
    long want = (nvec + 255) / 256;
    return (int)(want < 148L * 32 ? want : 148L * 32);
}
}  // namespace

extern "C" int tt_gelu_fwd(const void* u, void* y, long n, int kind, void* stream) {
    if (n <= 0 || (n & 7) || (kind != 0 && kind != 1)) return TT_ERR_ARG;
    const long nvec = n >> 3;
    if (kind == 0)
        gelu_fwd_kernel<0><<<grid_for(nvec), 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)u, (__nv_bfloat16*)y, nvec);
    else
        gelu_fwd_kernel<1><<<grid_for(nvec), 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)u, (__nv_bfloat16*)y, nvec);
    TT_CHECK_LAUNCH();
    return TT_OK;
}

extern "C" int tt_gelu_bwd(const void* dy, const void* u, void* du, long n, int kind, void* stream) {
    if (n <= 0 || (n & 7) || (kind != 0 && kind != 1)) return TT_ERR_ARG;
    const long nvec = n >> 3;
    if (kind == 0)
        gelu_bwd_kernel<0><<<grid_for(nvec), 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)dy, (const __nv_bfloat16*)u, (__nv_bfloat16*)du, nvec);
    else
        gelu_bwd_kernel<1><<<grid_for(nvec), 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)dy, (const __nv_bfloat16*)u, (__nv_bfloat16*)du, nvec);
    TT_CHECK_LAUNCH();
    return TT_OK;
}
