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

// ---------------------------------------------------------------------------------------------
// Flow matching: the noise mix that builds the model input and the weighted MSE loss with its gradient, one kernel each.
// The reference runs these as a handful of PyTorch elementwise ops (teletron/models/hunyuanvideo/pipeline.py:118-129, 215-224).
// ---------------------------------------------------------------------------------------------
namespace {
using namespace tt;

// out = (1 - sigma[b]) * latents + sigma[b] * noise
__global__ void __launch_bounds__(256) noise_mix_kernel(const __nv_bfloat16* __restrict__ latents,
                                                       const __nv_bfloat16* __restrict__ noise, const float* __restrict__ sigma,
                                                       __nv_bfloat16* __restrict__ out, long nvec, long vec_per_batch) {
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (long)gridDim.x * blockDim.x) {
        const float s = sigma[i / vec_per_batch];
        float a[8], n[8];
        unpack8(ld8(latents + i * 8), a);
        unpack8(ld8(noise + i * 8), n);
#pragma unroll
        for (int j = 0; j < 8; ++j) a[j] = __bfloat162float(__float2bfloat16((1.f - s))) * a[j] + __bfloat162float(__float2bfloat16(s)) * n[j];
        st8(out + i * 8, pack8(a));
    }
}

// diff = pred - (noise - latents); partial[block] = sum w[b] * diff^2; dpred = 2 * w[b] * diff * inv_total (bf16)
__global__ void __launch_bounds__(256) flow_loss_kernel(const __nv_bfloat16* __restrict__ pred,
                                                       const __nv_bfloat16* __restrict__ noise,
                                                       const __nv_bfloat16* __restrict__ latents, const float* __restrict__ weight,
                                                       float* __restrict__ partials, __nv_bfloat16* __restrict__ dpred, long nvec,
                                                       long vec_per_batch, float inv_total) {
    __shared__ float red[32];
    float acc = 0.f;
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (long)gridDim.x * blockDim.x) {
        const float w = weight[i / vec_per_batch];
        float p[8], n[8], l[8], g[8];
        unpack8(ld8(pred + i * 8), p);
        unpack8(ld8(noise + i * 8), n);
        unpack8(ld8(latents + i * 8), l);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float d = p[j] - (n[j] - l[j]);
            acc += w * d * d;
            g[j] = 2.f * w * d * inv_total;
        }
        if (dpred != nullptr) st8(dpred + i * 8, pack8(g));
    }
    const float s = block_sum(acc, red);
    if (threadIdx.x == 0) partials[blockIdx.x] = s;
}

// fixed-order sum of the block partials (deterministic), scaled to the mean
__global__ void flow_loss_finalize_kernel(const float* __restrict__ partials, int n, float inv_total, float* __restrict__ loss) {
    __shared__ float red[32];
    float acc = 0.f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) acc += partials[i];
    const float s = block_sum(acc, red);
    if (threadIdx.x == 0) *loss = s * inv_total;
}
}  // namespace

#define TT_FLOW_MAX_BLOCKS 1184

extern "C" int tt_flow_loss_blocks(void) { return TT_FLOW_MAX_BLOCKS; }

// latents, noise, out: [batch, n_per_batch] bf16 (n_per_batch a multiple of 8); sigma [batch] fp32
extern "C" int tt_noise_mix(const void* latents, const void* noise, const float* sigma, void* out, long n_per_batch, int batch,
                            void* stream) {
    if (n_per_batch <= 0 || (n_per_batch & 7) || batch <= 0) return TT_ERR_ARG;
    const long nvec = n_per_batch / 8 * batch;
    noise_mix_kernel<<<grid_for(nvec), 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)latents, (const __nv_bfloat16*)noise, sigma,
                                                                      (__nv_bfloat16*)out, nvec, n_per_batch / 8);
    TT_CHECK_LAUNCH();
    return TT_OK;
}

// loss = mean_b,i weight[b] * (pred - (noise - latents))^2 (fp32 scalar); dpred (optional) = d loss / d pred in bf16.
// partials: fp32 scratch of tt_flow_loss_blocks() entries.
extern "C" int tt_flow_loss(const void* pred, const void* noise, const void* latents, const float* weight, float* partials,
                            void* dpred, float* loss, long n_per_batch, int batch, void* stream) {
    if (n_per_batch <= 0 || (n_per_batch & 7) || batch <= 0 || partials == nullptr || loss == nullptr) return TT_ERR_ARG;
    const long nvec = n_per_batch / 8 * batch;
    long want = (nvec + 255) / 256;
    const int grid = (int)(want < TT_FLOW_MAX_BLOCKS ? want : TT_FLOW_MAX_BLOCKS);
    const float inv_total = 1.f / ((float)n_per_batch * (float)batch);
    cudaStream_t st = (cudaStream_t)stream;
    flow_loss_kernel<<<grid, 256, 0, st>>>((const __nv_bfloat16*)pred, (const __nv_bfloat16*)noise, (const __nv_bfloat16*)latents, weight,
                                           partials, (__nv_bfloat16*)dpred, nvec, n_per_batch / 8, inv_total);
    TT_CHECK_LAUNCH();
    flow_loss_finalize_kernel<<<1, 256, 0, st>>>(partials, grid, inv_total, loss);
    TT_CHECK_LAUNCH();
    return TT_OK;
}
