// LayerNorm(no affine) + AdaLN modulation, optionally fused with the gated residual update,
// forward and backward; plain RMSNorm forward and backward.
//
// Covers what the reference's `teletron_op/fused_adaln` (adaln_forward.cu:111-196,
// adaln_backward.cu:62-127, scale_shift_backward.cu:49-126) and `fused_rmsnorm` extensions do,
// without their restrictions: any column count that is a multiple of 8 up to 8192, any row
// count, per-batch modulation vectors, fp32 arithmetic throughout, (mean, rstd) saved instead of
// a normalised copy of the activations, and every launch on the caller's stream.
#include "common.cuh"
#include "sm100.cuh"
#include "teletron_b200.h"
#include "teletron_b200_noalloc.h"

namespace {

using namespace tt;

constexpr int kMaxCols = 8192;

// ---------------------------------------------------------------------------------------------
// forward: one warp per row, the row lives in registers
// ---------------------------------------------------------------------------------------------
template <int VPL, bool GATE>
__global__ void __launch_bounds__(256, (VPL <= 12 ? 3 : 1)) ln_mod_fwd_kernel(
    const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ branch,
    const __nv_bfloat16* __restrict__ gate, const __nv_bfloat16* __restrict__ scale,
    const __nv_bfloat16* __restrict__ shift, __nv_bfloat16* __restrict__ new_res,
    __nv_bfloat16* __restrict__ y, float* __restrict__ mean_out, float* __restrict__ rstd_out,
    long rows, int cols, long rows_per_batch, float eps) {
    // The row stays in registers as packed bf16 (4 registers per 8 elements) and is unpacked in each of the three
    // passes: that keeps the kernel under 85 registers, so three CTAs (24 warps, each with a whole row of loads in
    // flight) share an SM.  With the fp32 copy it needed 150 registers and ran one CTA per SM at 0.47 of the copy
    // bandwidth.
    const int lane = threadIdx.x & 31;
    const int warps_per_cta = blockDim.x >> 5;
    const int nvec = cols >> 3;
    const float inv_cols = 1.f / (float)cols;
    for (long row = (long)blockIdx.x * warps_per_cta + (threadIdx.x >> 5); row < rows;
         row += (long)gridDim.x * warps_per_cta) {
        const long b = row / rows_per_batch;
        const __nv_bfloat16* xr = x + row * cols;
        bf16x8 pk[VPL];
#pragma unroll
        for (int i = 0; i < VPL; ++i) {
            const int c = lane + i * 32;
            if (c < nvec) pk[i] = ld8(xr + c * 8);
        }
        float sum = 0.f;
#pragma unroll
        for (int i = 0; i < VPL; ++i) {
            const int c = lane + i * 32;
            if (c < nvec) {
                float v[8];
                unpack8(pk[i], v);
                if (GATE) {
                    float br[8], g[8];
                    unpack8(ld8(branch + row * cols + c * 8), br);
                    unpack8(ld8(gate + b * cols + c * 8), g);
#pragma unroll
                    for (int j = 0; j < 8; ++j) v[j] = v[j] + g[j] * br[j];
                    // the residual stream is stored in bf16: normalise exactly what is stored
                    pk[i] = pack8(v);
                    st8(new_res + row * cols + c * 8, pk[i]);
                    unpack8(pk[i], v);
                }
#pragma unroll
                for (int j = 0; j < 8; ++j) sum += v[j];
            }
        }
        const float mean = warp_sum(sum) * inv_cols;
        float sq = 0.f;
#pragma unroll
        for (int i = 0; i < VPL; ++i) {
            if (lane + i * 32 < nvec) {
                float v[8];
                unpack8(pk[i], v);
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const float d = v[j] - mean;
                    sq += d * d;
                }
            }
        }
        const float rstd = rsqrtf(warp_sum(sq) * inv_cols + eps);
        if (lane == 0) {
            mean_out[row] = mean;
            rstd_out[row] = rstd;
        }
#pragma unroll
        for (int i = 0; i < VPL; ++i) {
            const int c = lane + i * 32;
            if (c < nvec) {
                float v[8], sc[8], sh[8], o[8];
                unpack8(pk[i], v);
                unpack8(ld8(scale + b * cols + c * 8), sc);
                unpack8(ld8(shift + b * cols + c * 8), sh);
#pragma unroll
                for (int j = 0; j < 8; ++j) o[j] = (v[j] - mean) * rstd * (1.f + sc[j]) + sh[j];
                st8(y + row * cols + c * 8, pack8(o));
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------
// backward: one CTA walks rows, thread t owns columns [8t, 8t+8); column sums stay in registers
// ---------------------------------------------------------------------------------------------
// partials layout: [batch][blocks_per_batch][K][cols] fp32 with K = 2 (dscale, dshift) or 3 (+dgate)
//
// kRowBatch rows go through one block-wide reduction together: a thread first issues the loads of all of them (8 x 16 bytes in
// flight instead of 2) and the CTA pays one barrier pair per batch instead of per row.
constexpr int kRowBatch = 4;

// Sums of 8 values (2 per row of the batch) over the CTA; every thread gets all of them.  Shuffles are the scarce resource
// here (one warp-wide shuffle per clock and SM), so the eight warp sums are formed together: in each of the first three
// butterfly steps a lane hands half of its values to its partner and keeps the other half (4 + 2 + 1 shuffles), two more
// steps finish the one value left (lane 4q ends up with value q): 9 shuffles instead of 40.  `red` holds [2][8][32]
// floats and is used alternately (parity), so one barrier per call is enough.
static_assert(kRowBatch == 4, "block_sum_batch reduces exactly eight values");
__device__ __forceinline__ void block_sum_batch(float* v, float* red, int parity) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    float* r = red + parity * (8 * 32);
    float a[4], b2[2];
    const bool h16 = lane & 16, h8 = lane & 8, h4 = lane & 4;
#pragma unroll
    for (int i = 0; i < 4; ++i) a[i] = (h16 ? v[i + 4] : v[i]) + __shfl_xor_sync(0xffffffffu, h16 ? v[i] : v[i + 4], 16);
#pragma unroll
    for (int i = 0; i < 2; ++i) b2[i] = (h8 ? a[i + 2] : a[i]) + __shfl_xor_sync(0xffffffffu, h8 ? a[i] : a[i + 2], 8);
    float c = (h4 ? b2[1] : b2[0]) + __shfl_xor_sync(0xffffffffu, h4 ? b2[0] : b2[1], 4);
    c += __shfl_xor_sync(0xffffffffu, c, 2);
    c += __shfl_xor_sync(0xffffffffu, c, 1);
    if ((lane & 3) == 0) r[(lane >> 2) * 32 + warp] = c;        // value q = 4 * bit4 + 2 * bit3 + bit2 = lane >> 2
    __syncthreads();
    // lane L sums the warps w = L / 8, L / 8 + 4, ... of value L % 8, the four parts meet by two shuffles
    float t = 0.f;
    for (int w = lane >> 3; w < nwarps; w += 4) t += r[(lane & 7) * 32 + w];
    t += __shfl_xor_sync(0xffffffffu, t, 8);
    t += __shfl_xor_sync(0xffffffffu, t, 16);
#pragma unroll
    for (int q = 0; q < 8; ++q) v[q] = __shfl_sync(0xffffffffu, t, q);
}

template <bool GATE, int MAXT>
__global__ void __launch_bounds__(MAXT) ln_mod_bwd_kernel(
    const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ dres_in,
    const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ branch,
    const __nv_bfloat16* __restrict__ gate, const __nv_bfloat16* __restrict__ scale,
    const float* __restrict__ mean, const float* __restrict__ rstd, __nv_bfloat16* __restrict__ dx,
    __nv_bfloat16* __restrict__ dbranch, float* __restrict__ partials, int cols, long rows_per_batch) {
    __shared__ float red[2 * 8 * 32];
    const int nvec = cols >> 3;
    const int t = threadIdx.x;
    const bool active = t < nvec;
    const long b = blockIdx.y;
    const float inv_cols = 1.f / (float)cols;
    float sc1[8], gt[8];
    float acc_scale[8], acc_shift[8], acc_gate[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        sc1[j] = 0.f;
        gt[j] = 0.f;
        acc_scale[j] = acc_shift[j] = acc_gate[j] = 0.f;
    }
    if (active) {
        unpack8(ld8(scale + b * cols + t * 8), sc1);
#pragma unroll
        for (int j = 0; j < 8; ++j) sc1[j] += 1.f;
        if (GATE) unpack8(ld8(gate + b * cols + t * 8), gt);
    }
    int parity = 0;
    for (long r0 = (long)blockIdx.x * kRowBatch; r0 < rows_per_batch; r0 += (long)gridDim.x * kRowBatch, parity ^= 1) {
        bf16x8 pdy[kRowBatch], px[kRowBatch];
        float mu[kRowBatch], rs[kRowBatch], sums[2 * kRowBatch];
#pragma unroll
        for (int k = 0; k < kRowBatch; ++k) {
            const bool live = r0 + k < rows_per_batch;
            const long row = b * rows_per_batch + (live ? r0 + k : r0);
            mu[k] = mean[row];
            rs[k] = rstd[row];
            if (active && live) {
                pdy[k] = ld8(dy + row * cols + t * 8);
                px[k] = ld8(x + row * cols + t * 8);
            } else {
                const float z[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
                pdy[k] = pack8(z);
                px[k] = pack8(z);
                if (!live) mu[k] = 0.f;      // padded row: x - mu = 0, dy = 0, nothing accumulates
            }
        }
#pragma unroll
        for (int k = 0; k < kRowBatch; ++k) {
            float dyv[8], xv[8];
            unpack8(pdy[k], dyv);
            unpack8(px[k], xv);
            float s1 = 0.f, s2 = 0.f;
            if (active) {
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const float xh = (xv[j] - mu[k]) * rs[k];
                    const float g = dyv[j] * sc1[j];
                    s1 += g;
                    s2 += g * xh;
                    acc_scale[j] += dyv[j] * xh;
                    acc_shift[j] += dyv[j];
                }
            }
            sums[2 * k] = s1;
            sums[2 * k + 1] = s2;
        }
        block_sum_batch(sums, red, parity);
#pragma unroll
        for (int k = 0; k < kRowBatch; ++k) {
            if (active && r0 + k < rows_per_batch) {
                const long row = b * rows_per_batch + r0 + k;
                const float m1 = sums[2 * k] * inv_cols, m2 = sums[2 * k + 1] * inv_cols;
                float dyv[8], xv[8], d[8];
                unpack8(pdy[k], dyv);
                unpack8(px[k], xv);
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const float xh = (xv[j] - mu[k]) * rs[k];
                    d[j] = rs[k] * (dyv[j] * sc1[j] - m1 - xh * m2);
                }
                if (dres_in != nullptr) {
                    float up[8];
                    unpack8(ld8(dres_in + row * cols + t * 8), up);
#pragma unroll
                    for (int j = 0; j < 8; ++j) d[j] += up[j];
                }
                st8(dx + row * cols + t * 8, pack8(d));
                if (GATE) {
                    float br[8], db[8];
                    unpack8(ld8(branch + row * cols + t * 8), br);
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        acc_gate[j] += d[j] * br[j];
                        db[j] = d[j] * gt[j];
                    }
                    st8(dbranch + row * cols + t * 8, pack8(db));
                }
            }
        }
    }
    if (active) {
        constexpr int K = GATE ? 3 : 2;
        float* p = partials + ((b * gridDim.x + blockIdx.x) * K) * (long)cols + t * 8;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            p[j] = acc_scale[j];
            p[cols + j] = acc_shift[j];
            if (GATE) p[2 * cols + j] = acc_gate[j];
        }
    }
}

// ---------------------------------------------------------------------------------------------
// backward, bulk-copy fed: the same arithmetic as ln_mod_bwd_kernel, but dy and x rows arrive through a shared-memory ring
// filled by one producer warp with untiled bulk copies (cp.async.bulk, completion on an mbarrier).  What is in flight
// is then set by the ring (up to ~190 KB per SM) instead of by the registers a thread can spare for pending loads, which
// kept the register version at a third of the copy bandwidth.  Consumer thread t owns columns [8t, 8t + 8) as before;
// branch / upstream-gradient rows are fetched with ordinary loads issued before the block reduction.
// ---------------------------------------------------------------------------------------------
__device__ int g_norm_status = 0;       // TT_ERR_TIMEOUT when a bounded wait of the ring ran out (read by tt_norm_status)

__device__ __forceinline__ void consumer_sum_batch(float* v, float* red, int parity, int nthreads) {
    // block_sum_batch for the consumer threads only (named barrier 1: the producer warp never joins it)
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = nthreads >> 5;
    float* r = red + parity * (8 * 32);
    float a[4], b2[2];
    const bool h16 = lane & 16, h8 = lane & 8, h4 = lane & 4;
#pragma unroll
    for (int i = 0; i < 4; ++i) a[i] = (h16 ? v[i + 4] : v[i]) + __shfl_xor_sync(0xffffffffu, h16 ? v[i] : v[i + 4], 16);
#pragma unroll
    for (int i = 0; i < 2; ++i) b2[i] = (h8 ? a[i + 2] : a[i]) + __shfl_xor_sync(0xffffffffu, h8 ? a[i] : a[i + 2], 8);
    float c = (h4 ? b2[1] : b2[0]) + __shfl_xor_sync(0xffffffffu, h4 ? b2[0] : b2[1], 4);
    c += __shfl_xor_sync(0xffffffffu, c, 2);
    c += __shfl_xor_sync(0xffffffffu, c, 1);
    if ((lane & 3) == 0) r[(lane >> 2) * 32 + warp] = c;
    asm volatile("bar.sync 1, %0;" ::"r"(nthreads) : "memory");
    float t = 0.f;
    for (int w = lane >> 3; w < nwarps; w += 4) t += r[(lane & 7) * 32 + w];
    t += __shfl_xor_sync(0xffffffffu, t, 8);
    t += __shfl_xor_sync(0xffffffffu, t, 16);
#pragma unroll
    for (int q = 0; q < 8; ++q) v[q] = __shfl_sync(0xffffffffu, t, q);
}

template <bool GATE, int MAXT>
__global__ void __launch_bounds__(MAXT + 32) ln_mod_bwd_ring_kernel(
    const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ dres_in,
    const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ branch,
    const __nv_bfloat16* __restrict__ gate, const __nv_bfloat16* __restrict__ scale,
    const float* __restrict__ mean, const float* __restrict__ rstd, __nv_bfloat16* __restrict__ dx,
    __nv_bfloat16* __restrict__ dbranch, float* __restrict__ partials, int cols, long rows_per_batch, int stages) {
    extern __shared__ uint8_t ring_raw[];
    __shared__ float red[2 * 8 * 32];
    __shared__ volatile int abort_flag;
    using namespace sm100;
    const uint32_t base = (smem_u32(ring_raw) + 127u) & ~127u;
    const uint32_t row_bytes = (uint32_t)cols * 2u;
    const uint32_t stage_bytes = 2u * kRowBatch * row_bytes;              // dy rows then x rows
    const uint32_t bars = base + (uint32_t)stages * stage_bytes;
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (stages + s); };
    const int n_cons = blockDim.x - 32;                                     // consumer threads (a multiple of 32)
    const int t = threadIdx.x;
    const bool producer = t >= n_cons;
    const long b = blockIdx.y;
    if (t == 0) {
        abort_flag = 0;
        for (int s = 0; s < stages; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), n_cons >> 5);
        }
        fence_barrier_init();
        fence_proxy_async();
    }
    __syncthreads();
    const long first = (long)blockIdx.x * kRowBatch, step = (long)gridDim.x * kRowBatch;
    if (producer) {
        if (t == n_cons) {
            int s = 0;
            uint32_t phase = 0;
            for (long r0 = first; r0 < rows_per_batch; r0 += step) {
                if (!mbar_wait(empty_bar(s), phase ^ 1u, &abort_flag)) break;
                const int live = (int)min((long)kRowBatch, rows_per_batch - r0);
                mbar_arrive_expect_tx(full_bar(s), 2u * live * row_bytes);
                const uint32_t dst = base + (uint32_t)s * stage_bytes;
                for (int k = 0; k < live; ++k) {
                    const long row = b * rows_per_batch + r0 + k;
                    bulk_load_1d(dst + k * row_bytes, dy + row * cols, row_bytes, full_bar(s));
                    bulk_load_1d(dst + (kRowBatch + k) * row_bytes, x + row * cols, row_bytes, full_bar(s));
                }
                if (++s == stages) {
                    s = 0;
                    phase ^= 1u;
                }
            }
        }
    } else {
        const int nvec = cols >> 3;
        const bool active = t < nvec;
        const float inv_cols = 1.f / (float)cols;
        float sc1[8], gt[8], acc_scale[8], acc_shift[8], acc_gate[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            sc1[j] = 0.f;
            gt[j] = 0.f;
            acc_scale[j] = acc_shift[j] = acc_gate[j] = 0.f;
        }
        if (active) {
            unpack8(ld8(scale + b * cols + t * 8), sc1);
#pragma unroll
            for (int j = 0; j < 8; ++j) sc1[j] += 1.f;
            if (GATE) unpack8(ld8(gate + b * cols + t * 8), gt);
        }
        int s = 0, parity = 0;
        uint32_t phase = 0;
        for (long r0 = first; r0 < rows_per_batch; r0 += step, parity ^= 1) {
            const int live = (int)min((long)kRowBatch, rows_per_batch - r0);
            // rows that do not come through the ring: issue their loads now, they land while the ring data is reduced
            bf16x8 pup[kRowBatch], pbr[kRowBatch];
            float mu[kRowBatch], rs[kRowBatch];
#pragma unroll
            for (int k = 0; k < kRowBatch; ++k) {
                const long row = b * rows_per_batch + (k < live ? r0 + k : r0);
                mu[k] = mean[row];
                rs[k] = rstd[row];
                if (active && k < live) {
                    if (dres_in != nullptr) pup[k] = ld8(dres_in + row * cols + t * 8);
                    if (GATE) pbr[k] = ld8(branch + row * cols + t * 8);
                }
            }
            if (!mbar_wait(full_bar(s), phase, &abort_flag)) break;
            // the rows are read from the ring twice (before and after the block reduction) instead of being held in
            // registers across it; the slot is released after the second read
            const uint32_t src = base + (uint32_t)s * stage_bytes + (uint32_t)t * 16u;
            auto ring_row = [&](int which, int k) {
                uint4 a;
                asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(a.x), "=r"(a.y), "=r"(a.z), "=r"(a.w)
                             : "r"(src + (uint32_t)(which * kRowBatch + k) * row_bytes) : "memory");
                return *reinterpret_cast<bf16x8*>(&a);
            };
            float sums[2 * kRowBatch];
#pragma unroll
            for (int k = 0; k < kRowBatch; ++k) {
                float s1 = 0.f, s2 = 0.f;
                if (active && k < live) {
                    float dyv[8], xv[8];
                    unpack8(ring_row(0, k), dyv);
                    unpack8(ring_row(1, k), xv);
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const float xh = (xv[j] - mu[k]) * rs[k];
                        const float g = dyv[j] * sc1[j];
                        s1 += g;
                        s2 += g * xh;
                        acc_scale[j] += dyv[j] * xh;
                        acc_shift[j] += dyv[j];
                    }
                }
                sums[2 * k] = s1;
                sums[2 * k + 1] = s2;
            }
            consumer_sum_batch(sums, red, parity, n_cons);
#pragma unroll
            for (int k = 0; k < kRowBatch; ++k) {
                if (active && k < live) {
                    const long row = b * rows_per_batch + r0 + k;
                    const float m1 = sums[2 * k] * inv_cols, m2 = sums[2 * k + 1] * inv_cols;
                    float dyv[8], xv[8], d[8];
                    unpack8(ring_row(0, k), dyv);
                    unpack8(ring_row(1, k), xv);
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const float xh = (xv[j] - mu[k]) * rs[k];
                        d[j] = rs[k] * (dyv[j] * sc1[j] - m1 - xh * m2);
                    }
                    if (dres_in != nullptr) {
                        float up[8];
                        unpack8(pup[k], up);
#pragma unroll
                        for (int j = 0; j < 8; ++j) d[j] += up[j];
                    }
                    st8(dx + row * cols + t * 8, pack8(d));
                    if (GATE) {
                        float br[8], db[8];
                        unpack8(pbr[k], br);
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            acc_gate[j] += d[j] * br[j];
                            db[j] = d[j] * gt[j];
                        }
                        st8(dbranch + row * cols + t * 8, pack8(db));
                    }
                }
            }
            // every consumer warp has finished with the slot: it can be refilled
            __syncwarp();
            if ((t & 31) == 0) mbar_arrive(empty_bar(s));
            if (++s == stages) {
                s = 0;
                phase ^= 1u;
            }
        }
        if (active) {
            constexpr int K = GATE ? 3 : 2;
            float* p = partials + ((b * gridDim.x + blockIdx.x) * K) * (long)cols + t * 8;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                p[j] = acc_scale[j];
                p[cols + j] = acc_shift[j];
                if (GATE) p[2 * cols + j] = acc_gate[j];
            }
        }
    }
    __syncthreads();
    if (abort_flag) {
        if (t == 0) atomicExch(&g_norm_status, TT_ERR_TIMEOUT);
        for (int i = 0; i < 200; ++i) __nanosleep(1000);      // let bulk copies in flight land before the ring goes away
    }
}

// out[k][b][c] (bf16) = sum over blocks of partials[b][blk][k][c]
__global__ void column_finalize_kernel(const float* __restrict__ partials, __nv_bfloat16* __restrict__ out0,
                                       __nv_bfloat16* __restrict__ out1, __nv_bfloat16* __restrict__ out2, int K,
                                       int nblk, int cols) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int k = blockIdx.y;
    const long b = blockIdx.z;
    if (c >= cols) return;
    // four independent chains keep several loads in flight; the order is fixed, so the sum is deterministic
    float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
    const float* p = partials + (b * nblk * K + k) * (long)cols + c;
    const long step = (long)K * cols;
    int i = 0;
    for (; i + 3 < nblk; i += 4) {
        s0 += p[(i + 0) * step];
        s1 += p[(i + 1) * step];
        s2 += p[(i + 2) * step];
        s3 += p[(i + 3) * step];
    }
    for (; i < nblk; ++i) s0 += p[i * step];
    const float s = (s0 + s1) + (s2 + s3);
    __nv_bfloat16* o = k == 0 ? out0 : (k == 1 ? out1 : out2);
    if (o != nullptr) o[b * cols + c] = __float2bfloat16(s);
}

// ---------------------------------------------------------------------------------------------
// gated residual: out = res + gate[b] * branch (+ backward with the gate's column sums)
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) gate_residual_fwd_kernel(const __nv_bfloat16* __restrict__ res,
                                                               const __nv_bfloat16* __restrict__ branch,
                                                               const __nv_bfloat16* __restrict__ gate,
                                                               __nv_bfloat16* __restrict__ out, long rows, int cols,
                                                               long rows_per_batch) {
    const int nvec = cols >> 3;
    const long total = rows * nvec;
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
        const long row = i / nvec;
        const int c = (int)(i - row * nvec);
        const long b = row / rows_per_batch;
        float r[8], br[8], g[8];
        unpack8(ld8(res + i * 8), r);
        unpack8(ld8(branch + i * 8), br);
        unpack8(ld8(gate + b * cols + c * 8), g);
#pragma unroll
        for (int j = 0; j < 8; ++j) r[j] += g[j] * br[j];
        st8(out + i * 8, pack8(r));
    }
}

// dbranch = gate * dout; partial dgate column sums of dout * branch (K = 1 partial layout)
__global__ void __launch_bounds__(1024) gate_residual_bwd_kernel(const __nv_bfloat16* __restrict__ dout,
                                                                const __nv_bfloat16* __restrict__ branch,
                                                                const __nv_bfloat16* __restrict__ gate,
                                                                __nv_bfloat16* __restrict__ dbranch,
                                                                float* __restrict__ partials, int cols,
                                                                long rows_per_batch) {
    const int nvec = cols >> 3;
    const int t = threadIdx.x;
    if (t >= nvec) return;
    const long b = blockIdx.y;
    float gt[8], acc[8];
    unpack8(ld8(gate + b * cols + t * 8), gt);
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    // four rows per iteration: eight 16-byte loads in flight per thread
    for (long r0 = (long)blockIdx.x * 4; r0 < rows_per_batch; r0 += (long)gridDim.x * 4) {
        bf16x8 pd[4], pb[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            if (r0 + k < rows_per_batch) {
                const long row = b * rows_per_batch + r0 + k;
                pd[k] = ld8(dout + row * cols + t * 8);
                pb[k] = ld8(branch + row * cols + t * 8);
            }
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            if (r0 + k < rows_per_batch) {
                const long row = b * rows_per_batch + r0 + k;
                float d[8], br[8], db[8];
                unpack8(pd[k], d);
                unpack8(pb[k], br);
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    acc[j] += d[j] * br[j];
                    db[j] = d[j] * gt[j];
                }
                st8(dbranch + row * cols + t * 8, pack8(db));
            }
        }
    }
    float* p = partials + (b * gridDim.x + blockIdx.x) * (long)cols + t * 8;
#pragma unroll
    for (int j = 0; j < 8; ++j) p[j] = acc[j];
}

// ---------------------------------------------------------------------------------------------
// RMSNorm over the last dimension (any cols % 8 == 0 up to 8192): y = x * rstd * w
// ---------------------------------------------------------------------------------------------
template <int VPL>
__global__ void __launch_bounds__(256) rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x,
                                                         const __nv_bfloat16* __restrict__ w,
                                                         __nv_bfloat16* __restrict__ y, float* __restrict__ rstd_out,
                                                         long rows, int cols, float eps) {
    const int lane = threadIdx.x & 31;
    const int wpc = blockDim.x >> 5;
    const int nvec = cols >> 3;
    for (long row = (long)blockIdx.x * wpc + (threadIdx.x >> 5); row < rows; row += (long)gridDim.x * wpc) {
        float v[VPL][8];
        float sq = 0.f;
#pragma unroll
        for (int i = 0; i < VPL; ++i) {
            const int c = lane + i * 32;
            if (c < nvec) {
                unpack8(ld8(x + row * cols + c * 8), v[i]);
#pragma unroll
                for (int j = 0; j < 8; ++j) sq += v[i][j] * v[i][j];
            }
        }
        const float rstd = rsqrtf(warp_sum(sq) / (float)cols + eps);
        if (lane == 0) rstd_out[row] = rstd;
#pragma unroll
        for (int i = 0; i < VPL; ++i) {
            const int c = lane + i * 32;
            if (c < nvec) {
                float wv[8], o[8];
                unpack8(ld8(w + c * 8), wv);
#pragma unroll
                for (int j = 0; j < 8; ++j) o[j] = v[i][j] * rstd * wv[j];
                st8(y + row * cols + c * 8, pack8(o));
            }
        }
    }
}

// dx = rstd * (dy*w - xhat * mean(dy*w*xhat)); partial dw[c] = sum_rows dy * xhat  (uses the saved INPUT,
// not y / w as the reference does, so zero weights are harmless)
__global__ void __launch_bounds__(1024) rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy,
                                                          const __nv_bfloat16* __restrict__ x,
                                                          const __nv_bfloat16* __restrict__ w,
                                                          const float* __restrict__ rstd,
                                                          __nv_bfloat16* __restrict__ dx, float* __restrict__ partials,
                                                          long rows, int cols) {
    __shared__ float red[64];
    const int nvec = cols >> 3;
    const int t = threadIdx.x;
    const bool active = t < nvec;
    float wv[8], acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        wv[j] = 0.f;
        acc[j] = 0.f;
    }
    if (active) unpack8(ld8(w + t * 8), wv);
    for (long row = blockIdx.x; row < rows; row += gridDim.x) {
        float g[8], xh[8];
        float s = 0.f;
        const float rs = rstd[row];
        if (active) {
            float d[8], xv[8];
            unpack8(ld8(dy + row * cols + t * 8), d);
            unpack8(ld8(x + row * cols + t * 8), xv);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                xh[j] = xv[j] * rs;
                g[j] = d[j] * wv[j];
                s += g[j] * xh[j];
                acc[j] += d[j] * xh[j];
            }
        }
        const float m = block_sum(s, red) / (float)cols;
        if (active) {
            float o[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) o[j] = rs * (g[j] - xh[j] * m);
            st8(dx + row * cols + t * 8, pack8(o));
        }
    }
    if (active) {
        float* p = partials + (long)blockIdx.x * cols + t * 8;
#pragma unroll
        for (int j = 0; j < 8; ++j) p[j] = acc[j];
    }
}

// ---------------------------------------------------------------------------------------------
// RMSNorm for short rows (cols <= 256, e.g. the per-head norm with cols = 128): LPR lanes per row, 32 / LPR rows per
// warp and two such groups per iteration, so that every lane has work and several 16-byte loads in flight.  With one
// warp per row half of the lanes idled (forward) and the backward ran 32-thread CTAs.
// ---------------------------------------------------------------------------------------------
template <int LPR>
__device__ __forceinline__ float row_sum(float v) {
#pragma unroll
    for (int o = LPR / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

template <int LPR>
__global__ void __launch_bounds__(256) rmsnorm_fwd_small_kernel(const __nv_bfloat16* __restrict__ x,
                                                               const __nv_bfloat16* __restrict__ w,
                                                               __nv_bfloat16* __restrict__ y, float* __restrict__ rstd_out,
                                                               long rows, int cols, float eps) {
    constexpr int RPW = 32 / LPR, U = 4;
    const int lane = threadIdx.x & 31, sub = lane / LPR, l = lane % LPR;
    const int nvec = cols >> 3;
    const bool col_ok = l < nvec;
    const long warp_id = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const long nwarps = (long)gridDim.x * (blockDim.x >> 5);
    float wv[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) wv[j] = 0.f;
    if (col_ok) unpack8(ld8(w + l * 8), wv);
    const float inv_cols = 1.f / (float)cols;
    for (long base = warp_id * (RPW * U); base < rows; base += nwarps * (RPW * U)) {
        bf16x8 pk[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const long row = base + u * RPW + sub;
            if (row < rows && col_ok) pk[u] = ld8(x + row * cols + l * 8);
            else pk[u] = bf16x8{};
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const long row = base + u * RPW + sub;
            float v[8], o[8];
            unpack8(pk[u], v);
            float sq = 0.f;
#pragma unroll
            for (int j = 0; j < 8; ++j) sq += v[j] * v[j];
            const float rstd = rsqrtf(row_sum<LPR>(sq) * inv_cols + eps);
            if (row < rows) {
                if (l == 0) rstd_out[row] = rstd;
                if (col_ok) {
#pragma unroll
                    for (int j = 0; j < 8; ++j) o[j] = v[j] * rstd * wv[j];
                    st8(y + row * cols + l * 8, pack8(o));
                }
            }
        }
    }
}

// partials [gridDim.x][cols]: per-CTA column sums of dy * xhat (summed by column_finalize_kernel)
template <int LPR>
__global__ void __launch_bounds__(256) rmsnorm_bwd_small_kernel(const __nv_bfloat16* __restrict__ dy,
                                                               const __nv_bfloat16* __restrict__ x,
                                                               const __nv_bfloat16* __restrict__ w,
                                                               const float* __restrict__ rstd,
                                                               __nv_bfloat16* __restrict__ dx, float* __restrict__ partials,
                                                               long rows, int cols) {
    constexpr int RPW = 32 / LPR, U = 4;
    __shared__ float fold[8][LPR * 8];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, sub = lane / LPR, l = lane % LPR;
    const int nvec = cols >> 3;
    const bool col_ok = l < nvec;
    const long warp_id = (long)blockIdx.x * (blockDim.x >> 5) + warp;
    const long nwarps = (long)gridDim.x * (blockDim.x >> 5);
    float wv[8], acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        wv[j] = 0.f;
        acc[j] = 0.f;
    }
    if (col_ok) unpack8(ld8(w + l * 8), wv);
    const float inv_cols = 1.f / (float)cols;
    for (long base = warp_id * (RPW * U); base < rows; base += nwarps * (RPW * U)) {
        bf16x8 pd[U], px[U];
        float rs[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const long row = base + u * RPW + sub;
            const bool ok = row < rows && col_ok;
            pd[u] = ok ? ld8(dy + row * cols + l * 8) : bf16x8{};
            px[u] = ok ? ld8(x + row * cols + l * 8) : bf16x8{};
            rs[u] = row < rows ? rstd[row] : 0.f;
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const long row = base + u * RPW + sub;
            float d[8], xv[8], g[8], xh[8], o[8];
            unpack8(pd[u], d);
            unpack8(px[u], xv);
            float sdot = 0.f;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                xh[j] = xv[j] * rs[u];
                g[j] = d[j] * wv[j];
                sdot += g[j] * xh[j];
                acc[j] += d[j] * xh[j];
            }
            const float m = row_sum<LPR>(sdot) * inv_cols;
            if (row < rows && col_ok) {
#pragma unroll
                for (int j = 0; j < 8; ++j) o[j] = rs[u] * (g[j] - xh[j] * m);
                st8(dx + row * cols + l * 8, pack8(o));
            }
        }
    }
    // fold the RPW row groups of the warp (lanes l, l + LPR, ... own the same columns), then the warps of the CTA
#pragma unroll
    for (int j = 0; j < 8; ++j) {
#pragma unroll
        for (int o = LPR; o < 32; o <<= 1) acc[j] += __shfl_xor_sync(0xffffffffu, acc[j], o);
    }
    if (sub == 0) {
#pragma unroll
        for (int j = 0; j < 8; ++j) fold[warp][l * 8 + j] = acc[j];
    }
    __syncthreads();
    const int nw = blockDim.x >> 5;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) {
        float sacc = 0.f;
        for (int q = 0; q < nw; ++q) sacc += fold[q][c];
        partials[(long)blockIdx.x * cols + c] = sacc;
    }
}

inline int pick_blocks(long rows_per_batch, int batch) {
    long want = (148L * 4) / (batch > 0 ? batch : 1);
    if (want < 1) want = 1;
    if (want > rows_per_batch) want = rows_per_batch;
    if (want > TT_NORM_MAX_PARTIAL_BLOCKS) want = TT_NORM_MAX_PARTIAL_BLOCKS;
    return (int)want;
}

inline bool bad_cols(int cols) { return cols <= 0 || (cols & 7) || cols > kMaxCols; }

}  // namespace

extern "C" int tt_norm_partial_blocks(long rows_per_batch, int batch) { return pick_blocks(rows_per_batch, batch); }

// TT_OK, or TT_ERR_TIMEOUT if a bounded wait inside a norm kernel's shared-memory ring ran out since the last call
// (synchronises the device; the word is cleared).
extern "C" int tt_norm_status(void) {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_norm_status, sizeof(int)) != cudaSuccess) return TT_ERR_CUDA;
    if (v != 0) cudaMemcpyToSymbol(g_norm_status, &zero, sizeof(int));
    return v;
}

#define LAUNCH_FWD(VPL)                                                                                         \
    do {                                                                                                        \
        if (has_gate)                                                                                           \
            ln_mod_fwd_kernel<VPL, true><<<grid, 256, 0, st>>>(X, BR, G, SC, SH, NR, Y, mean, rstd, rows, cols, \
                                                               rows_per_batch, eps);                            \
        else                                                                                                    \
            ln_mod_fwd_kernel<VPL, false><<<grid, 256, 0, st>>>(X, BR, G, SC, SH, NR, Y, mean, rstd, rows,      \
                                                                cols, rows_per_batch, eps);                     \
    } while (0)

extern "C" int tt_ln_mod_fwd(const void* x, const void* branch, const void* gate, const void* scale,
                             const void* shift, void* new_res, void* y, float* mean, float* rstd, long rows,
                             int cols, long rows_per_batch, float eps, void* stream) {
    if (bad_cols(cols) || rows <= 0 || rows_per_batch <= 0 || rows % rows_per_batch) return TT_ERR_ARG;
    const bool has_gate = branch != nullptr;
    if (has_gate && (gate == nullptr || new_res == nullptr)) return TT_ERR_ARG;
    auto X = (const __nv_bfloat16*)x;
    auto BR = (const __nv_bfloat16*)branch;
    auto G = (const __nv_bfloat16*)gate;
    auto SC = (const __nv_bfloat16*)scale;
    auto SH = (const __nv_bfloat16*)shift;
    auto NR = (__nv_bfloat16*)new_res;
    auto Y = (__nv_bfloat16*)y;
    cudaStream_t st = (cudaStream_t)stream;
    long want = (rows + 7) / 8;
    const int grid = (int)(want < 148L * 16 ? want : 148L * 16);
    const int vpl = ((cols >> 3) + 31) / 32;
    if (vpl <= 4) LAUNCH_FWD(4);
    else if (vpl <= 8) LAUNCH_FWD(8);
    else if (vpl <= 12) LAUNCH_FWD(12);
    else if (vpl <= 16) LAUNCH_FWD(16);
    else LAUNCH_FWD(32);
    TT_CHECK_LAUNCH();
    return TT_OK;
}

extern "C" int tt_ln_mod_bwd(const void* dy, const void* dres_in, const void* x, const void* branch,
                             const void* gate, const void* scale, const float* mean, const float* rstd, void* dx,
                             void* dbranch, float* partials, void* dscale, void* dshift, void* dgate, long rows,
                             int cols, long rows_per_batch, void* stream) {
    if (bad_cols(cols) || rows <= 0 || rows_per_batch <= 0 || rows % rows_per_batch) return TT_ERR_ARG;
    const bool has_gate = branch != nullptr;
    if (has_gate && (gate == nullptr || dbranch == nullptr || dgate == nullptr)) return TT_ERR_ARG;
    const int batch = (int)(rows / rows_per_batch);
    const int nblk = pick_blocks(rows_per_batch, batch);
    cudaStream_t st = (cudaStream_t)stream;
    const int threads = (((cols >> 3) + 31) / 32) * 32;
    int nblk_used = nblk;
    // Bulk-copy fed ring kernel when at least two stages of four dy + four x rows fit in shared memory (cols <= 6144):
    // one persistent CTA per SM (fewer partial rows than the register kernel, never more than the caller allocated).
    const long stage_bytes = 2L * kRowBatch * cols * 2;
    const int stages = (int)((200 * 1024) / stage_bytes) > 8 ? 8 : (int)((200 * 1024) / stage_bytes);
    static const bool ring_off = [] { const char* v = getenv("TELETRON_B200_NORM_RING"); return v != nullptr && v[0] == '0'; }();
    if (stages >= 2 && !ring_off) {
        int dev = 0, sms = 148;
        if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        int g = sms / batch;
        if (g < 1) g = 1;
        if (g > nblk) g = nblk;
        nblk_used = g;
        const int smem = (int)(stages * stage_bytes) + 16 * stages + 256;
        const bool wide = threads > 512;
        auto kern = has_gate ? (wide ? ln_mod_bwd_ring_kernel<true, 1024> : ln_mod_bwd_ring_kernel<true, 512>)
                             : (wide ? ln_mod_bwd_ring_kernel<false, 1024> : ln_mod_bwd_ring_kernel<false, 512>);
        static int configured[4][64] = {{0}};
        if (dev < 0 || dev >= 64) dev = 0;
        const int which = (has_gate ? 2 : 0) + (wide ? 1 : 0);
        if (configured[which][dev] < smem) {
            cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
            if (e != cudaSuccess) return tt_record_cuda(e);
            configured[which][dev] = smem;
        }
        dim3 rgrid(g, batch);
        kern<<<rgrid, threads + 32, smem, st>>>(
            (const __nv_bfloat16*)dy, (const __nv_bfloat16*)dres_in, (const __nv_bfloat16*)x, (const __nv_bfloat16*)branch,
            (const __nv_bfloat16*)gate, (const __nv_bfloat16*)scale, mean, rstd, (__nv_bfloat16*)dx, (__nv_bfloat16*)dbranch,
            partials, cols, rows_per_batch, stages);
        TT_CHECK_LAUNCH();
    } else {
    dim3 grid(nblk, batch);
#define LN_BWD(G_, T_)                                                                                          \
    ln_mod_bwd_kernel<G_, T_><<<grid, threads, 0, st>>>(                                                        \
        (const __nv_bfloat16*)dy, (const __nv_bfloat16*)dres_in, (const __nv_bfloat16*)x,                       \
        (const __nv_bfloat16*)branch, (const __nv_bfloat16*)gate, (const __nv_bfloat16*)scale, mean, rstd,      \
        (__nv_bfloat16*)dx, (__nv_bfloat16*)dbranch, partials, cols, rows_per_batch)
    if (has_gate) {
        if (threads <= 512) LN_BWD(true, 512);
        else LN_BWD(true, 1024);
    } else {
        if (threads <= 512) LN_BWD(false, 512);
        else LN_BWD(false, 1024);
    }
    TT_CHECK_LAUNCH();
    }
    const int K = has_gate ? 3 : 2;
    dim3 fgrid((cols + 255) / 256, K, batch);
    column_finalize_kernel<<<fgrid, 256, 0, st>>>(partials, (__nv_bfloat16*)dscale, (__nv_bfloat16*)dshift,
                                                  (__nv_bfloat16*)dgate, K, nblk_used, cols);
    TT_CHECK_LAUNCH();
    return TT_OK;
}

extern "C" int tt_gate_residual_fwd(const void* res, const void* branch, const void* gate, void* out, long rows,
                                    int cols, long rows_per_batch, void* stream) {
    if (bad_cols(cols) || rows <= 0 || rows_per_batch <= 0 || rows % rows_per_batch) return TT_ERR_ARG;
    const long total = rows * (cols >> 3);
    long want = (total + 255) / 256;
    const int grid = (int)(want < 148L * 32 ? want : 148L * 32);
    gate_residual_fwd_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(
        (const __nv_bfloat16*)res, (const __nv_bfloat16*)branch, (const __nv_bfloat16*)gate, (__nv_bfloat16*)out, rows,
        cols, rows_per_batch);
    TT_CHECK_LAUNCH();
    return TT_OK;
}

extern "C" int tt_gate_residual_bwd(const void* dout, const void* branch, const void* gate, void* dbranch,
                                    float* partials, void* dgate, long rows, int cols, long rows_per_batch,
                                    void* stream) {
    if (bad_cols(cols) || rows <= 0 || rows_per_batch <= 0 || rows % rows_per_batch) return TT_ERR_ARG;
    const int batch = (int)(rows / rows_per_batch);
    const int nblk = pick_blocks(rows_per_batch, batch);
    cudaStream_t st = (cudaStream_t)stream;
    const int threads = (((cols >> 3) + 31) / 32) * 32;
    gate_residual_bwd_kernel<<<dim3(nblk, batch), threads, 0, st>>>(
        (const __nv_bfloat16*)dout, (const __nv_bfloat16*)branch, (const __nv_bfloat16*)gate, (__nv_bfloat16*)dbranch,
        partials, cols, rows_per_batch);
    TT_CHECK_LAUNCH();
    column_finalize_kernel<<<dim3((cols + 255) / 256, 1, batch), 256, 0, st>>>(partials, (__nv_bfloat16*)dgate, nullptr,
                                                                             nullptr, 1, nblk, cols);
    TT_CHECK_LAUNCH();
    return TT_OK;
}

#define LAUNCH_RMS(VPL) \
    rmsnorm_fwd_kernel<VPL><<<grid, 256, 0, st>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)w, (__nv_bfloat16*)y, rstd, rows, cols, eps)

extern "C" int tt_rmsnorm_fwd(const void* x, const void* w, void* y, float* rstd, long rows, int cols, float eps,
                              void* stream) {
    if (bad_cols(cols) || rows <= 0) return TT_ERR_ARG;
    cudaStream_t st = (cudaStream_t)stream;
    long want = (rows + 7) / 8;
    const int grid = (int)(want < 148L * 16 ? want : 148L * 16);
    const int vpl = ((cols >> 3) + 31) / 32;
    if (cols <= 256) {
        // short rows: several rows per warp
        const int nvec = cols >> 3;
        long need = (rows + 63) / 64;
        const int g2 = (int)(need < 148L * 8 ? need : 148L * 8);
#define RMS_SMALL(LPR) rmsnorm_fwd_small_kernel<LPR><<<g2, 256, 0, st>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)w, (__nv_bfloat16*)y, rstd, rows, cols, eps)
        if (nvec <= 4) RMS_SMALL(4);
        else if (nvec <= 8) RMS_SMALL(8);
        else if (nvec <= 16) RMS_SMALL(16);
        else RMS_SMALL(32);
#undef RMS_SMALL
        TT_CHECK_LAUNCH();
        return TT_OK;
    }
    if (vpl <= 1) LAUNCH_RMS(1);
    else if (vpl <= 4) LAUNCH_RMS(4);
    else if (vpl <= 12) LAUNCH_RMS(12);
    else if (vpl <= 16) LAUNCH_RMS(16);
    else LAUNCH_RMS(32);
    TT_CHECK_LAUNCH();
    return TT_OK;
}

namespace {
// first pass of the RMSNorm backward into `nblk` partial rows: rows-per-warp kernel for short rows, CTA-per-row otherwise
void launch_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, void* dx, float* partials,
                        long rows, int cols, int nblk, cudaStream_t st) {
    if (cols <= 256) {
        const int nvec = cols >> 3;
#define RMS_BWD_SMALL(LPR) rmsnorm_bwd_small_kernel<LPR><<<nblk, 256, 0, st>>>((const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, rstd, (__nv_bfloat16*)dx, partials, rows, cols)
        if (nvec <= 4) RMS_BWD_SMALL(4);
        else if (nvec <= 8) RMS_BWD_SMALL(8);
        else if (nvec <= 16) RMS_BWD_SMALL(16);
        else RMS_BWD_SMALL(32);
#undef RMS_BWD_SMALL
        return;
    }
    const int threads = (((cols >> 3) + 31) / 32) * 32;
    rmsnorm_bwd_kernel<<<nblk, threads, 0, st>>>((const __nv_bfloat16*)dy, (const __nv_bfloat16*)x,
                                                 (const __nv_bfloat16*)w, rstd, (__nv_bfloat16*)dx, partials, rows, cols);
}
}  // namespace

extern "C" int tt_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, void* dx,
                              float* partials, void* dw, long rows, int cols, void* stream) {
    if (bad_cols(cols) || rows <= 0) return TT_ERR_ARG;
    cudaStream_t st = (cudaStream_t)stream;
    const int nblk = pick_blocks(rows, 1);
    launch_rmsnorm_bwd(dy, x, w, rstd, dx, partials, rows, cols, nblk, st);
    TT_CHECK_LAUNCH();
    column_finalize_kernel<<<dim3((cols + 255) / 256, 1, 1), 256, 0, st>>>(partials, (__nv_bfloat16*)dw, nullptr, nullptr,
                                                                         1, nblk, cols);
    TT_CHECK_LAUNCH();
    return TT_OK;
}

// ---------------------------------------------------------------------------------------------
// RMSNorm backward for callers that cannot allocate device memory (declared in teletron_b200_noalloc.h)
// ---------------------------------------------------------------------------------------------
// The partial column sums that tt_rmsnorm_bwd takes from its caller live here instead, in a fixed array that
// is part of the library image: every GPU that loads the library carries these 2 MiB until the process exits.
static __device__ __align__(256) float g_rmsnorm_noalloc_partials[TT_NOALLOC_MAX_BLOCKS * TT_NOALLOC_MAX_COLS];

namespace {
// Device address of the array above, per device.  In host code the array's name is only a handle for the
// runtime's symbol table, never something a kernel can dereference, so the address is looked up once per device.
float* g_noalloc_ptr[64] = {nullptr};

int noalloc_scratch(float** out) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return tt_record_cuda(e);
    if (dev < 0 || dev >= 64) return TT_ERR_LIMIT;
    if (g_noalloc_ptr[dev] == nullptr) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_rmsnorm_noalloc_partials);     // resolves against the current device
        if (e != cudaSuccess) return tt_record_cuda(e);
        g_noalloc_ptr[dev] = static_cast<float*>(p);
    }
    *out = g_noalloc_ptr[dev];
    return TT_OK;
}
}  // namespace

extern "C" int tt_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* rstd, void* dx, void* dw,
                                      long rows, int cols, void* stream) {
    if (bad_cols(cols) || rows <= 0) return TT_ERR_ARG;
    if (cols > TT_NOALLOC_MAX_COLS) return TT_ERR_LIMIT;
    float* partials = nullptr;
    const int rc = noalloc_scratch(&partials);
    if (rc != TT_OK) return rc;
    int nblk = pick_blocks(rows, 1);
    if (nblk > TT_NOALLOC_MAX_BLOCKS) nblk = TT_NOALLOC_MAX_BLOCKS;
    cudaStream_t st = (cudaStream_t)stream;
    // every one of the nblk partial rows is fully rewritten by its block before the finalize pass reads it,
    // so nothing left behind by an earlier call can leak into this one
    launch_rmsnorm_bwd(dy, x, w, rstd, dx, partials, rows, cols, nblk, st);
    TT_CHECK_LAUNCH();
    column_finalize_kernel<<<dim3((cols + 255) / 256, 1, 1), 256, 0, st>>>(partials, (__nv_bfloat16*)dw, nullptr, nullptr,
                                                                         1, nblk, cols);
    TT_CHECK_LAUNCH();
    return TT_OK;
}
