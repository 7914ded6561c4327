/* C ABI of libteletron_b200.so: hand-written sm_100a kernels reached from Python through ctypes.
 *
 * Conventions: every pointer is a device pointer unless stated; bf16 buffers are passed as void*;
 * `stream` is a cudaStream_t; every function returns TT_OK (0) or a TT_ERR_* code and never
 * allocates device memory (scratch buffers are passed in by the caller, who sizes them with the
 * *_partial_* helpers). */
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

#include <stddef.h>

#define TT_MAX_PEERS 8
#define TT_NORM_MAX_PARTIAL_BLOCKS 1024
#define TT_QKV_MAX_PARTIAL_WARPS 4736

const char* tt_last_cuda_error(void);
int tt_version(void);

/* ---- LayerNorm + AdaLN modulation (optionally fused with the gated residual update) ---- */
int tt_norm_partial_blocks(long rows_per_batch, int batch);
int tt_norm_status(void);      /* TT_ERR_TIMEOUT once if a bounded wait inside a norm kernel ran out; synchronises */
int tt_ln_mod_fwd(const void* x, const void* branch, const void* gate, const void* scale, const void* shift,
                  void* new_res, void* y, float* mean, float* rstd, long rows, int cols, long rows_per_batch,
                  float eps, void* stream);
/* partials: fp32 [batch][tt_norm_partial_blocks][2 or 3][cols] */
int tt_ln_mod_bwd(const void* dy, const void* dres_in, const void* x, const void* branch, const void* gate,
                  const void* scale, const float* mean, const float* rstd, void* dx, void* dbranch, float* partials,
                  void* dscale, void* dshift, void* dgate, long rows, int cols, long rows_per_batch, void* stream);
int tt_gate_residual_fwd(const void* res, const void* branch, const void* gate, void* out, long rows, int cols,
                         long rows_per_batch, void* stream);
int tt_gate_residual_bwd(const void* dout, const void* branch, const void* gate, void* dbranch, float* partials,
                         void* dgate, long rows, int cols, long rows_per_batch, void* stream);
int tt_rmsnorm_fwd(const void* x, const void* w, void* y, float* rstd, long rows, int cols, float eps, void* stream);
int tt_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, void* dx, float* partials,
                   void* dw, long rows, int cols, void* stream);

/* ---- QKV post-processing: split + QK-RMSNorm + RoPE + head-major layout ---- */
int tt_qkv_partial_warps(long rows, int heads);
int tt_qkv_post_fwd(const void* qkv, const void* qw, const void* kw, const float* cos_t, const float* sin_t, void* q,
                    void* k, void* v, long rows, int heads, long seq_in, long seq_out, long out_offset, long rope_len,
                    float eps, void* stream);
/* partials: fp32 [tt_qkv_partial_warps][2][128] */
int tt_qkv_post_bwd(const void* dq, const void* dk, const void* dv, const void* qkv, const void* qw, const void* kw,
                    const float* cos_t, const float* sin_t, void* dqkv, float* partials, void* dqw, void* dkw,
                    long rows, int heads, long seq_in, long seq_out, long out_offset, long rope_len, float eps,
                    void* stream);

int tt_qkv_post_bwd_peer(void* const* dq_ptrs, void* const* dk_ptrs, void* const* dv_ptrs, int n, const void* qkv,
                         const void* qw, const void* kw, const float* cos_t, const float* sin_t, void* dqkv,
                         float* partials, void* dqw, void* dkw, long rows, int heads, long seq_in, long seq_out,
                         long out_offset, long rope_len, float eps, void* stream);

/* ---- activations ---- */
int tt_gelu_fwd(const void* u, void* y, long n, int kind, void* stream);   /* kind 0 = erf, 1 = tanh */
int tt_gelu_bwd(const void* dy, const void* u, void* du, long n, int kind, void* stream);

/* ---- flow matching: noise mix and weighted MSE loss (+ its gradient) ---- */
int tt_flow_loss_blocks(void);
int tt_noise_mix(const void* latents, const void* noise, const float* sigma, void* out, long n_per_batch, int batch,
                 void* stream);
int tt_flow_loss(const void* pred, const void* noise, const void* latents, const float* weight, float* partials,
                 void* dpred, float* loss, long n_per_batch, int batch, void* stream);

/* ---- optimizer ---- */
int tt_adamw(void* param, const void* grad, void* m, void* v, float* master, void* master_lo, long n,
             int state_is_bf16, float lr, float beta1, float beta2, float eps, float wd, int step, float grad_scale,
             void* stream);

/* gradient reduce-scatter + AdamW + parameter all-gather on one shard of flat buffers that live in peer-mapped memory
 * (grad_ptrs [n_g] sources, param_ptrs [n_p] destinations, this rank's own at my_p; see optim.cu) */
int tt_rs_adamw_ag(void* const* grad_ptrs, int n_g, void* const* param_ptrs, int n_p, int my_p, long offset, void* m,
                   void* v, float* master, void* master_lo, long n, int state_is_bf16, float lr, float beta1,
                   float beta2, float eps, float wd, int step, float grad_scale, void* stream);

/* ---- tcgen05 GEMM (see gemm_tcgen05.cu for the layout / epilogue codes) ---- */
int tt_gemm_bf16(const void* a, const void* b, void* c, const void* bias, void* aux, int M, int N, int K, long lda,
                 long ldb, long ldc, int a_mn, int b_mn, int epi, int* status, void* stream);

/* the same product on CTA pairs (thread-block cluster of 2, tcgen05.mma.cta_group::2, 256 x 256 tiles; gemm2_tcgen05.cu) */
int tt_gemm2_bf16(const void* a, const void* b, void* c, const void* bias, void* aux, int M, int N, int K, long lda,
                  long ldb, long ldc, int a_mn, int b_mn, int epi, int* status, void* stream);

/* pushed tiles (tt_gemm_comm_bf16 store modes 1 / 2): 1 = staged stores of whole 256-byte rows (default), 0 = 16 bytes per thread */
void tt_set_coalesced_peer_stores(int on);

/* GEMM fused with a collective over peer memory, and the fused QKV projection (see gemm_tcgen05.cu) */
int tt_gemm_comm_bf16(void* const* a_ptrs, int n, int a_mode, long a_rows, int a_span, int a_row_off,
                      const void* a_extra, long lda_extra, const void* b, int b_mn, long ldb, void* c, long ldc,
                      const void* bias, int M, int N, int K, int seg_rows, int my_rank, int store_mode,
                      void* const* out_ptrs, int out_span, int out_row_off, long out_ld, void* stage, int* stage_flags,
                      int stage_epoch, int* status, void* stream);
int tt_qkv_gemm_fused(const void* x, const void* w, const void* bias, const void* qw, const void* kw, const float* cos_t,
                      const float* sin_t, void* const* q_ptrs, void* const* k_ptrs, void* const* v_ptrs, int n,
                      int my_rank, void* aux, int M, int heads, int K, int s_in, int s_out, int out_off, int rope_len,
                      int only_local, float eps, int* status, void* stream);

/* ---- tcgen05 flash attention: q, k, v, dq, dk, dv [B*H, S, 128]; out, dout [B, S, H*128];
 *      lse, delta [B*H, pitch] fp32, pitch % 64 == 0, lse = +inf and delta = 0 at positions >= S ---- */
/* masked keys: those at and beyond kv_len, and those in [mask_lo, mask_hi) (mask_lo >= mask_hi: no such range) */
int tt_attn_fwd(const void* q, const void* k, const void* v, void* out, float* lse, int B, int H, int S, int kv_len,
                int mask_lo, int mask_hi, int lse_pitch, float scale, int* status, void* stream);
int tt_attn_fwd_push(const void* q, const void* k, const void* v, void* out, float* lse, int H, int S, int kv_len,
                     int mask_lo, int mask_hi, int lse_pitch, float scale, int* status, void* stream,
                     void* const* peer_out, int n_peers, int my_rank, int text_len, int s_local, long dest_ld);
int tt_attn_bwd(const void* q, const void* k, const void* v, const void* out, const void* dout, const float* lse,
                float* delta, void* dq, void* dk, void* dv, int B, int H, int S, int kv_len, int mask_lo, int mask_hi,
                int pitch, float scale, int* status, void* stream);
/* one pass over the scores: dQ accumulated in fp32 scratch dq_acc [B*H, roundup(S,128), 128] with vector reductions */
int tt_attn_bwd_fused(const void* q, const void* k, const void* v, const void* out, const void* dout, const float* lse,
                      float* delta, float* dq_acc, void* dq, void* dk, void* dv, int B, int H, int S, int kv_len,
                      int mask_lo, int mask_hi, int pitch, float scale, int* status, void* stream);

/* ---- symmetric heap + in-kernel collectives over IPC-mapped peer memory (comm.cu) ---- */
int tt_symm_alloc(size_t bytes, void** out);                 /* cudaMalloc + zero */
int tt_symm_free(void* p);
int tt_ipc_get_handle(void* p, void* handle64);              /* 64-byte CUDA IPC handle */
int tt_ipc_open(const void* handle64, void** out);
int tt_ipc_close(void* p);
/* flag_ptrs[r] = rank r's array of n 64-bit flags (peer-mapped); sets TT_ERR_TIMEOUT in *status on expiry */
int tt_comm_barrier(void* const* flag_ptrs, int my_rank, int n, unsigned long long epoch, long long timeout_cycles,
                    int* status, void* stream);
int tt_reduce_scatter_bf16(void* const* src_ptrs, int n, long offset, void* out, long count, float scale, void* stream);
int tt_all_gather_push_bf16(void* const* dst_ptrs, int n, long offset, const void* src, long count, void* stream);
int tt_gather_cols_bf16(void* const* src_ptrs, int n, long rows, int span, long row_off, void* dst, void* stream);
int tt_partial_sum(const void* stage, int n, long rows, int cols, const void* bias, const void* res, const void* gate,
                   long rows_per_batch, void* out, void* stream);

#ifdef __cplusplus
}
#endif
