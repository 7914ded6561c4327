// Symmetric-heap plumbing for the in-kernel NVLink collectives: plain device allocations shared between
// the ranks of one node through CUDA IPC handles, a device-side barrier over per-rank flag words, and
// the peer-reading reduction kernels (gradient reduce-scatter with cast / scale, partial-sum reduction
// after a row-parallel GEMM).
//
// Nothing here uses NVLS multicast objects or TMA multicast: peers are reached with ordinary loads and
// stores on IPC-mapped pointers.  Every wait is bounded and reports through a status word; a rank that
// never arrives makes its peers return TT_ERR_TIMEOUT instead of spinning.
//
// The reference has no counterpart: all of its collectives are NCCL calls through torch.distributed
// (teletron/core/parallel_state.py:279-515, teletron/core/distributed/distributed_data_parallel.py:220-242).
#include "common.cuh"
#include "teletron_b200.h"

#include <string.h>

namespace {

using namespace tt;

struct PeerTable {
    void* ptr[TT_MAX_PEERS];
};

// Every rank: publish `epoch` into slot [my_rank] of every peer's flag array, then wait until every slot of
// the local array has reached `epoch`.  flags are 64-bit, monotonically increasing.
__global__ void barrier_kernel(PeerTable flags, int my_rank, int n, unsigned long long epoch, long long timeout_cycles,
                               int* status) {
    const int t = threadIdx.x;
    if (t < n) {
        __threadfence_system();     // order this GPU's earlier writes (kernel boundary already did) before the flag
        volatile unsigned long long* dst = reinterpret_cast<unsigned long long*>(flags.ptr[t]) + my_rank;
        *dst = epoch;
    }
    __threadfence_system();
    if (t < n) {
        volatile unsigned long long* mine = reinterpret_cast<unsigned long long*>(flags.ptr[my_rank]) + t;
        const long long t0 = clock64();
        bool ok = false;
        while (true) {
            if (*mine >= epoch) {
                ok = true;
                break;
            }
            if (clock64() - t0 > timeout_cycles) break;
            __nanosleep(64);
        }
        if (!ok) atomicExch(status, TT_ERR_TIMEOUT);
    }
    __threadfence_system();
}

// out[i] = scale * sum_r src_r[offset + i]   (bf16 in, bf16 out, fp32 accumulate); src_r = peers' gradient buckets
__global__ void __launch_bounds__(256) reduce_scatter_kernel(PeerTable src, int n, long offset, __nv_bfloat16* __restrict__ out,
                                                            long nvec, float scale) {
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (long)gridDim.x * blockDim.x) {
        // all peers' loads are issued before the first one is consumed: a peer load takes ~2 us to come back, so the
        // number of loads in flight per thread sets the NVLink bandwidth this kernel reaches
        bf16x8 t[TT_MAX_PEERS];
#pragma unroll
        for (int r = 0; r < TT_MAX_PEERS; ++r)
            if (r < n) t[r] = ld8(reinterpret_cast<const __nv_bfloat16*>(src.ptr[r]) + offset + i * 8);
        float acc[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = 0.f;
#pragma unroll
        for (int r = 0; r < TT_MAX_PEERS; ++r) {
            if (r < n) {
                float v[8];
                unpack8(t[r], v);
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[j] += v[j];
            }
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] *= scale;
        st8(out + i * 8, pack8(acc));
    }
}

// dst_r[offset + i] = src[i] for every peer r (all-gather of an updated parameter shard by stores)
__global__ void __launch_bounds__(256) all_gather_push_kernel(PeerTable dst, int n, long offset,
                                                             const __nv_bfloat16* __restrict__ src, long nvec) {
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (long)gridDim.x * blockDim.x) {
        const bf16x8 v = ld8(src + i * 8);
        for (int r = 0; r < n; ++r) st8(reinterpret_cast<__nv_bfloat16*>(dst.ptr[r]) + offset + i * 8, v);
    }
}

// out[row, :] = sum over n staged partials + bias   (row-parallel GEMM partial sums landed by peers in `stage`,
// laid out [n][rows][cols]); optional fused gated residual: out = res + gate * (sum + bias)
__global__ void __launch_bounds__(256) partial_sum_kernel(const __nv_bfloat16* __restrict__ stage, int n, long rows, int cols,
                                                         const __nv_bfloat16* __restrict__ bias,
                                                         const __nv_bfloat16* __restrict__ res,
                                                         const __nv_bfloat16* __restrict__ gate, long rows_per_batch,
                                                         __nv_bfloat16* __restrict__ out) {
    const int nvec = cols >> 3;
    const long total = rows * nvec;
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
        const long row = i / nvec;
        const int c = (int)(i - row * nvec);
        float acc[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = 0.f;
        for (int r = 0; r < n; ++r) {
            float v[8];
            unpack8(ld8(stage + ((long)r * rows + row) * cols + c * 8), v);
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] += v[j];
        }
        if (bias != nullptr) {
            float b[8];
            unpack8(ld8(bias + c * 8), b);
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] += b[j];
        }
        if (res != nullptr) {
            float rr[8], g[8];
            unpack8(ld8(res + row * cols + c * 8), rr);
            unpack8(ld8(gate + (row / rows_per_batch) * cols + c * 8), g);
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] = rr[j] + g[j] * acc[j];
        }
        st8(out + row * cols + c * 8, pack8(acc));
    }
}

// dst[row, r*span + c] = src_r[(row_off + row) * span + c]: the head -> sequence all-to-all as a plain copy
// (each rank holds `span` columns for all rows; this rank collects its own rows from everyone)
__global__ void __launch_bounds__(256) gather_cols_kernel(PeerTable src, int n, long rows, int span, long row_off,
                                                         __nv_bfloat16* __restrict__ dst) {
    const int nvec = span >> 3;
    const long total = rows * n * nvec;
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
        const long row = i / ((long)n * nvec);
        const int rem = (int)(i - row * n * nvec);
        const int r = rem / nvec, c = rem - r * nvec;
        const bf16x8 v = ld8(reinterpret_cast<const __nv_bfloat16*>(src.ptr[r]) + (row_off + row) * span + c * 8);
        st8(dst + (row * n + r) * span + c * 8, v);
    }
}

int fill_table(PeerTable& t, void* const* ptrs, int n) {
    if (n < 1 || n > TT_MAX_PEERS) return TT_ERR_ARG;
    for (int i = 0; i < TT_MAX_PEERS; ++i) t.ptr[i] = i < n ? ptrs[i] : nullptr;
    return TT_OK;
}

}  // namespace

extern "C" int tt_symm_alloc(size_t bytes, void** out) {
    cudaError_t e = cudaMalloc(out, bytes);
    if (e != cudaSuccess) return tt_record_cuda(e);
    e = cudaMemset(*out, 0, bytes);
    if (e != cudaSuccess) return tt_record_cuda(e);
    return TT_OK;
}

extern "C" int tt_symm_free(void* p) {
    cudaError_t e = cudaFree(p);
    return e == cudaSuccess ? TT_OK : tt_record_cuda(e);
}

extern "C" int tt_ipc_get_handle(void* p, void* handle64) {
    cudaIpcMemHandle_t h;
    cudaError_t e = cudaIpcGetMemHandle(&h, p);
    if (e != cudaSuccess) return tt_record_cuda(e);
    memcpy(handle64, &h, sizeof(h));
    return TT_OK;
}

extern "C" int tt_ipc_open(const void* handle64, void** out) {
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, sizeof(h));
    cudaError_t e = cudaIpcOpenMemHandle(out, h, cudaIpcMemLazyEnablePeerAccess);
    return e == cudaSuccess ? TT_OK : tt_record_cuda(e);
}

extern "C" int tt_ipc_close(void* p) {
    cudaError_t e = cudaIpcCloseMemHandle(p);
    return e == cudaSuccess ? TT_OK : tt_record_cuda(e);
}

extern "C" int tt_comm_barrier(void* const* flag_ptrs, int my_rank, int n, unsigned long long epoch,
                               long long timeout_cycles, int* status, void* stream) {
    PeerTable t;
    int rc = fill_table(t, flag_ptrs, n);
    if (rc != TT_OK || my_rank < 0 || my_rank >= n || status == nullptr) return TT_ERR_ARG;
    barrier_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(t, my_rank, n, epoch, timeout_cycles, status);
    TT_CHECK_LAUNCH();
    return TT_OK;
}

extern "C" int tt_reduce_scatter_bf16(void* const* src_ptrs, int n, long offset, void* out, long count, float scale,
                                      void* stream) {
    PeerTable t;
    int rc = fill_table(t, src_ptrs, n);
    if (rc != TT_OK || count <= 0 || (count & 7) || (offset & 7)) return TT_ERR_ARG;
    const long nvec = count >> 3;
    long want = (nvec + 255) / 256;
    const int grid = (int)(want < 148L * 8 ? want : 148L * 8);
    reduce_scatter_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(t, n, offset, (__nv_bfloat16*)out, nvec, scale);
    TT_CHECK_LAUNCH();
    return TT_OK;
}

extern "C" int tt_all_gather_push_bf16(void* const* dst_ptrs, int n, long offset, const void* src, long count,
                                       void* stream) {
    PeerTable t;
    int rc = fill_table(t, dst_ptrs, n);
    if (rc != TT_OK || count <= 0 || (count & 7) || (offset & 7)) return TT_ERR_ARG;
    const long nvec = count >> 3;
    long want = (nvec + 255) / 256;
    const int grid = (int)(want < 148L * 8 ? want : 148L * 8);
    all_gather_push_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(t, n, offset, (const __nv_bfloat16*)src, nvec);
    TT_CHECK_LAUNCH();
    return TT_OK;
}

extern "C" int tt_partial_sum(const void* stage, int n, long rows, int cols, const void* bias, const void* res,
                              const void* gate, long rows_per_batch, void* out, void* stream) {
    if (n < 1 || n > TT_MAX_PEERS || rows <= 0 || cols <= 0 || (cols & 7)) return TT_ERR_ARG;
    if ((res == nullptr) != (gate == nullptr)) return TT_ERR_ARG;
    if (res != nullptr && (rows_per_batch <= 0 || rows % rows_per_batch)) return TT_ERR_ARG;
    const long total = rows * (cols >> 3);
    long want = (total + 255) / 256;
    const int grid = (int)(want < 148L * 16 ? want : 148L * 16);
    partial_sum_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(
        (const __nv_bfloat16*)stage, n, rows, cols, (const __nv_bfloat16*)bias, (const __nv_bfloat16*)res,
        (const __nv_bfloat16*)gate, rows_per_batch > 0 ? rows_per_batch : rows, (__nv_bfloat16*)out);
    TT_CHECK_LAUNCH();
    return TT_OK;
}

extern "C" int tt_gather_cols_bf16(void* const* src_ptrs, int n, long rows, int span, long row_off, void* dst,
                                   void* stream) {
    PeerTable t;
    int rc = fill_table(t, src_ptrs, n);
    if (rc != TT_OK || rows <= 0 || span <= 0 || (span & 7) || row_off < 0) return TT_ERR_ARG;
    const long total = rows * n * (span >> 3);
    long want = (total + 255) / 256;
    const int grid = (int)(want < 148L * 8 ? want : 148L * 8);
    gather_cols_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(t, n, rows, span, row_off, (__nv_bfloat16*)dst);
    TT_CHECK_LAUNCH();
    return TT_OK;
}
