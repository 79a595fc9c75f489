// C entry points of libtspipe_b200.so (all kernels are compiled for sm_100a only).
// Every function enqueues on `stream` and returns 0 on success, a cudaError_t value, or a negative
// code for rejected arguments (-2 misaligned pointer, -3 unsupported shape).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// ---- flat_optim.cu ---------------------------------------------------------------------------------------------
int tsp_ema_update(float* teacher, const float* student, int64_t n, float momentum, void* bf16_shadow,
                   cudaStream_t stream);
int tsp_lars_step(float* p, const float* g, float* mu, const int64_t* chunks, int n_chunks, const float* seg_hp,
                  float grad_scale, float* norms, int n_seg, float* teacher, int64_t teacher_n, float ema_m,
                  cudaStream_t stream);
int tsp_lars_norms(const float* p, const float* g, const int64_t* chunks, int n_chunks, const float* seg_hp,
                   float grad_scale, float* norms, int n_seg, cudaStream_t stream);
int tsp_lars_apply(float* p, const float* g, float* mu, const int64_t* chunks, int n_chunks, const float* seg_hp,
                   float grad_scale, const float* norms, float* teacher, int64_t teacher_n, float ema_m,
                   cudaStream_t stream);
int tsp_adamw_step(float* p, const float* g, float* m, float* v, const int64_t* chunks, int n_chunks,
                   const float* seg_hp, float grad_scale, float* teacher, int64_t teacher_n, float ema_m,
                   cudaStream_t stream);
int tsp_sgd_step(float* p, const float* g, float* buf, const int64_t* chunks, int n_chunks, const float* seg_hp,
                 float grad_scale, float* teacher, int64_t teacher_n, float ema_m, cudaStream_t stream);

// ---- losses.cu ---------------------------------------------------------------------------------------------------
int tsp_byol_loss(const void* x, const void* y, int n, int d, int dtype, float scale, float* loss, void* gx,
                  cudaStream_t stream);
int tsp_cosine_loss(const void* x, const void* y, const uint8_t* row_mask, int n, int d, int dtype, float scale,
                    float* loss, void* gx, cudaStream_t stream);
int tsp_kd_ce_loss(const void* s, const void* t, const int64_t* labels, const uint8_t* row_mask, int n, int c,
                   int s_dtype, int t_dtype, float temp, float w_ce, float w_kd, float* loss, void* gs,
                   cudaStream_t stream);

// ---- norms.cu ----------------------------------------------------------------------------------------------------
int tsp_layernorm_fwd(const void* x, const float* w, const float* b, void* y, float* mean, float* rstd, int rows, int d,
                      float eps, int dtype, cudaStream_t stream);
int tsp_layernorm_bwd_blocks(int rows);
int tsp_layernorm_bwd(const void* dy, const void* x, const float* w, const float* mean, const float* rstd, void* dx,
                      float* dw, float* db, float* partial, int rows, int d, int dtype, cudaStream_t stream);
int tsp_gelu_fwd(const void* x, const float* bias, void* y, int64_t n, int d, int dtype, cudaStream_t stream);
int tsp_gelu_bwd(const void* dy, const void* x, const float* bias, void* dx, int64_t n, int d, int dtype,
                 cudaStream_t stream);

// ---- batchnorm.cu -----------------------------------------------------------------------------------------------
int tsp_bn_stats(const void* x, int64_t m, int c, int dtype, float* sums, int segs, cudaStream_t stream);
int tsp_bn_stream_status(int reset);
int tsp_bn_apply(const void* x, const void* res, void* y, const float* sums, const float* fixed_mean_var,
                 const float* w, const float* b, float* save_mean_rstd, float* acc_sum, float* acc_sumsq,
                 float* acc_count, int64_t acc_seg_stride, int64_t m, int c, float eps, int relu, int dtype, int segs,
                 cudaStream_t stream);
int tsp_bn_bwd_reduce(const void* dy, const void* x, const void* y, void* dres, const float* mean_rstd, const float* w,
                      const float* bias, int relu, int64_t m, int c, int dtype, float* sums, int segs,
                      cudaStream_t stream);
int tsp_bn_bwd_apply(const void* dy, const void* x, const void* y, const float* mean_rstd, const float* w,
                     const float* bias, int relu, const float* sums, void* dx, int64_t m, int c, int dtype, int segs,
                     cudaStream_t stream);

// ---- peer.cu ------------------------------------------------------------------------------------------------------
int tsp_enable_peer_access(int peer_device);
int tsp_ipc_import(const unsigned char* handle64, void** base);
int tsp_ipc_close(void* base);
int tsp_gather_blocks(void* const* srcs, int n_peers, int64_t bytes_each, void* dst, cudaStream_t stream);
int tsp_dp_reduce_norms(void* const* grads, int n_peers, float scale, float* g_out, const float* p,
                        const int64_t* chunks, int n_chunks, const float* seg_hp, float* norms, int n_seg,
                        cudaStream_t stream);
int tsp_dp_lars_apply(void* const* params, int n_peers, int self, const float* g, float* mu, const int64_t* chunks,
                      int n_chunks, const float* seg_hp, const float* norms, cudaStream_t stream);
int tsp_dp_adamw_step(void* const* grads, void* const* params, int n_peers, int self, float scale, float* m, float* v,
                      const int64_t* chunks, int n_chunks, const float* seg_hp, cudaStream_t stream);

// ---- pool.cu ------------------------------------------------------------------------------------------------------
int tsp_maxpool3x3s2_fwd(const void* x, void* y, uint8_t* idx, int n, int h, int w, int c, int dtype,
                         cudaStream_t stream);
int tsp_maxpool3x3s2_bwd(const void* dy, const uint8_t* idx, void* dx, int n, int h, int w, int c, int dtype,
                         cudaStream_t stream);
int tsp_avgpool_fwd(const void* x, void* y, int n, int hw, int c, int dtype, cudaStream_t stream);
int tsp_avgpool_bwd(const void* dy, void* dx, int n, int hw, int c, int dtype, cudaStream_t stream);

// ---- gemm_tcgen05.cu ------------------------------------------------------------------------------------------
int tsp_gemm_bf16_tn(const void* a, const void* b, void* c, const float* bias, int m, int n, int k, int lda, int ldb,
                     int ldc, int out_dtype, int epi, int* status, cudaStream_t stream);
int tsp_gemm_bf16_tn_gathered_b(const void* a, void* const* b_srcs, int n_src, int rows_per_b, void* c, int m, int k,
                                int lda, int ldb, int ldc, int out_dtype, int* status, cudaStream_t stream);

// ---- attn_tcgen05.cu ----------------------------------------------------------------------------------------------
int tsp_attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse, int batch, int heads, int nq, int nk,
                 int d, int dv, const int64_t* q_strides, const int64_t* k_strides, const int64_t* v_strides,
                 const int64_t* o_strides, float scale, float fixed_max, int use_fixed_max, int out_dtype, int* status,
                 cudaStream_t stream);

int tsp_attn_nce_gathered(const void* q, void* const* k_srcs, int n_src, int rows_per_src, void* o, float* lse, int nq,
                          float scale, float fixed_max, int* status, cudaStream_t stream);

// ---- conv_stem_tcgen05.cu -----------------------------------------------------------------------------------------
int tsp_conv_stem_fwd(const void* x, const void* wmat, void* y, float* sums, int n, int h, int w, int segs,
                      int* status, cudaStream_t stream);

int tsp_gemm_bf16_tn_stats(const void* a, const void* b, void* c, int m, int n, int k, int lda, int ldb, int ldc,
                           float* col_sums, int segs, int* status, cudaStream_t stream);

// ---- gemm_tcgen05_2cta.cu -----------------------------------------------------------------------------------------
int tsp_gemm_bf16_tn_2cta(const void* a, const void* b, void* c, const float* bias, int m, int n, int k, int lda,
                          int ldb, int ldc, int out_dtype, int epi, int* status, cudaStream_t stream);
int tsp_gemm_bf16_tn_2cta_stats(const void* a, const void* b, void* c, int m, int n, int k, int lda, int ldb, int ldc,
                                float* col_sums, int segs, int* status, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
