// The C interface of the janas_b200 kernel library.
//
// Every function takes device pointers and the stream to launch on, allocates
// nothing and returns 0 or a negative code (JB_EINVAL: a size or type the
// kernel does not take; JB_ELAUNCH: the launch failed).  The Python side
// (janas_b200/csrc/ops.py) checks shapes and types before it calls in here.
//
// The kernels are launched so that their CTAs may start while the kernel before
// them in the stream still runs, and they read what cannot depend on it before
// they wait for it: weights, norm weights, rotation tables, and the index arrays
// row_pos, row_seq and block_table.  None of these may be the output of another of
// this library's kernels launched just before (a copy, or any kernel launched in
// the ordinary way, is fine: nothing starts before those have finished).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

// element types of buffers
#define JB_F32 0
#define JB_BF16 1

#ifdef __cplusplus
extern "C" {
#endif

int jb_page(void);
int jb_embed(const void *table, int table_dt, const int32_t *tokens, float *x, int n, int dm,
             cudaStream_t st);
int jb_rmsnorm(float *x, const float *delta, int S, long long delta_stride,
               const int32_t *row_idx, const void *w, int w_dt, void *out, int out_dt, int n_out,
               int dm, float eps, cudaStream_t st);
int jb_swiglu(const float *gu, int S, long long stride, void *out, int out_dt, int n, int ff,
              cudaStream_t st);
int jb_rope_table(float *cs, float *sn, const float *inv_freq, int n_pos, int half,
                  cudaStream_t st);
int jb_qk_norm_rope_append(const float *qkv, int S, long long split_stride, const void *q_w,
                           const void *k_w, int w_dt, float eps, const float *cs, const float *sn,
                           int rot_half, const int32_t *row_pos, const int32_t *row_seq,
                           const int32_t *block_table, int bt_stride, void *q_out, void *k_cache,
                           void *v_cache, int cache_dt, int n, int nh, int nkv, int hd,
                           cudaStream_t st);
int jb_attention_chunk(void);
long long jb_attention_scratch(int n_rows, int nh, int hd, int max_chunks);
int jb_attention(const void *q, const void *k_cache, const void *v_cache, int dt,
                 const int32_t *row_pos, const int32_t *row_seq, const int32_t *block_table,
                 int bt_stride, float *scratch, void *out, int row0, int n_rows, int nh, int nkv,
                 int hd, int window, float scale, int max_chunks, cudaStream_t st);
int jb_attention_merge(const float *scratch, const int32_t *row_pos, void *out, int dt, int row0,
                       int n_rows, int nh, int hd, int window, int max_parts, int chunks_per_part,
                       cudaStream_t st);
int jb_attn_tc_decode_runs(int nh, int nkv, int hd);
int jb_attn_tc_ok(int nh, int nkv, int hd);
int jb_attn_tc_block_positions(int nh, int nkv);
int jb_attn_tc_prefill(const void *q, const void *k_cache, const void *v_cache, long long n_pages,
                       const int32_t *qblk, int n_blocks, const int32_t *block_table,
                       int bt_stride, void *out, int n, int nh, int nkv, int hd, int window,
                       float scale, cudaStream_t st);
int jb_attn_tc_decode(const void *q, const void *k_cache, const void *v_cache, long long n_pages,
                      const int32_t *row_pos, const int32_t *row_seq, const int32_t *block_table,
                      int bt_stride, float *part, int n, int row0, int n_rows, int nh, int nkv,
                      int hd, int window, float scale, int max_chunks, int chunks_per_cta,
                      cudaStream_t st);
int jb_attn_tc_decode_qkv(const float *qkv, int S, long long split_stride, const void *q_w,
                          const void *k_w, int w_dt, float eps, const float *cs, const float *sn,
                          void *k_cache, void *v_cache, int append, long long n_pages,
                          const int32_t *row_pos, const int32_t *row_seq,
                          const int32_t *block_table, int bt_stride, float *part, int n, int row0,
                          int n_rows, int nh, int nkv, int hd, int window, float scale,
                          int max_chunks, int chunks_per_cta, cudaStream_t st);
int jb_attn_tc_error(void);
long long jb_gemm_simt_scratch(int n, int m, int k);
int jb_gemm_simt(const void *A, int a_dt, const void *W, int w_dt, float *out, int n, int m, int k,
                 float *scratch, cudaStream_t st);
int jb_gemm_tc_ok(const void *A, const void *W, int n, int m, int k);
int jb_gemm_tc_splits(int n, int m, int k);
int jb_gemm_tc(const void *A, const void *W, float *out, int n, int m, int k, int splits,
               cudaStream_t st);
int jb_gemm_tc_swiglu(const void *A, const void *W, void *out_act, int n, int ff, int k,
                      cudaStream_t st);
int jb_gemm_tc_error(void);
int jb_gemm_tc_force_tile(int tokens);
int jb_gemm_tc_last_tile(void);
int jb_wait_selftest(long long limit_cycles);
int jb_sample_small_cap(void);
int jb_sample_needs_big(int V, int top_k);
int jb_sampler_set(const int32_t *slots, int n, const unsigned long long *seeds,
                   const float *temperature, const int32_t *top_k, const float *top_p,
                   const float *min_p, unsigned long long *rng_out, float *temperature_out,
                   int32_t *top_k_out, float *top_p_out, float *min_p_out, cudaStream_t st);
long long jb_sample_scratch(int rows, int V);
int jb_sample_launches(int V, long long big_cap, int sampled);
int jb_sample(const float *logits, int rows, int V, const int32_t *row_slot,
              const float *temperature, const int32_t *top_k, const float *top_p,
              const float *min_p, unsigned long long *rng, unsigned long long *big_keys,
              float *big_probs, long long big_cap, unsigned long long *chunk_keys, int32_t *out,
              int32_t *forced, cudaStream_t st);

#ifdef __cplusplus
}
#endif
