// Declarations of the launchers a layer's parts call, for the code that calls them from C++
// (layer_replay.cu). Every source file that defines one of them includes this header, so a
// declaration that drifts from its definition stops the build instead of passing wrong arguments.
#pragma once

#include <cuda_runtime.h>

#include "common.cuh"

TIE_API int tie_add_rmsnorm(int dtype, float* x, const void* delta, const float* part, long long part_stride,
                            int splits, const int* rows, const float* w, float eps, void* out, int n, int dim,
                            cudaStream_t s);
TIE_API int tie_rmsnorm_rows(int dtype, const void* x, long long x_stride, const float* w, float eps, void* out,
                             long long out_stride, int size, long long n, cudaStream_t s);
TIE_API int tie_silu_mul(int dtype, const void* gu, void* out, int tokens, int inter, cudaStream_t s);
TIE_API int tie_rope(int dtype, void* x, long long stride, const int* pos, const float* inv_freq, int tokens,
                     int heads, int head_dim, int rot, cudaStream_t s);
TIE_API int tie_kv_append(int dtype, const void* k, const void* v, long long k_stride, long long v_stride,
                          const int* slots, void* k_cache, void* v_cache, int tokens, int kv_heads, int head_dim,
                          int page_size, cudaStream_t s);
TIE_API int tie_qk_norm_rope_append(int dtype, void* qkv, long long stride, const float* part, long long part_stride,
                                    int splits, long long part_ld, const float* qw, const float* kw,
                                    float q_eps, float k_eps, const float* inv_freq, int rot, const int* pos,
                                    const int* slots, void* k_cache, void* v_cache, int tokens, int q_heads,
                                    int kv_heads, int head_dim, int page_size, int write_kv, cudaStream_t s);

TIE_API int tie_gemm_simt(int in_dtype, int out_dtype, const void* a, const void* w, void* out, int M, int N, int K,
                          long long lda, long long ldw, long long ldo, cudaStream_t s);
TIE_API int tie_gemm_tc(int out_dtype, const void* a, const void* w, void* out, int M, int N, int K, long long lda,
                        long long ldw, long long ldo, int transposed, int bn, int splits, float* scratch, int silu,
                        int reduce, int deep, int w_rows, int w_row0, cudaStream_t s);
TIE_API int tie_gemm_tc2(int out_dtype, const void* a, const void* w, void* out, int M, int N, int K, long long lda,
                         long long ldw, long long ldo, int silu, int w_rows, int w_row0, int bn, cudaStream_t s);

TIE_API int tie_attention_rows(int dtype, const void* q, long long q_stride, const void* k_cache, const void* v_cache,
                               void* out, const int* seq_of_row, const int* query_start, const int* context_lens,
                               const int* block_tables, int max_blocks, int rows, int seqs, int q_heads, int kv_heads,
                               int head_dim, int page_size, int window, float scale, cudaStream_t s);
TIE_API int tie_attention_split(int dtype, const void* q, long long q_stride, const void* k_cache, const void* v_cache,
                                void* out, const int* query_start, const int* context_lens, const int* block_tables,
                                int max_blocks, int seqs, int q_heads, int kv_heads, int head_dim, int page_size,
                                int window, float scale, const int* seq_list, int n_list, int split_keys,
                                int max_splits, float* scratch, cudaStream_t s);
TIE_API int tie_attention_merge(int dtype, void* out, const int* query_start, const int* context_lens, int q_heads,
                                int head_dim, int window, const int* seq_list, int n_list, int split_keys, int max_splits,
                                const float* scratch, cudaStream_t s);
TIE_API int tie_attention_prompt_tc(const void* q, long long q_stride, const void* k_cache, const void* v_cache, void* out,
                                    const int* query_start, const int* context_lens, const int* block_tables,
                                    int max_blocks, int n_seqs, int max_queries, int q_heads, int kv_heads, int head_dim,
                                    int page_size, int window, float scale, cudaStream_t s);
TIE_API int tie_attention_decode_tc(const void* q, long long q_stride, const void* k_cache, const void* v_cache,
                                    const int* query_start, const int* context_lens, const int* block_tables,
                                    int max_blocks, int q_heads, int kv_heads, int head_dim, int page_size, int window,
                                    float scale, const int* seq_list, int n_list, int split_keys, int max_splits,
                                    float* scratch, cudaStream_t s);
TIE_API int tie_attention_prompt_tma(const void* q, long long q_stride, const void* k_cache, const void* v_cache, void* out,
                                     const int* query_start, const int* context_lens, const int* block_tables,
                                     int max_blocks, int n_seqs, int max_queries, int q_heads, int kv_heads, int head_dim,
                                     int page_size, int pages, int window, float scale, cudaStream_t s);
TIE_API int tie_attention_decode_tma(const void* q, long long q_stride, const void* k_cache, const void* v_cache, void* out,
                                     const int* query_start, const int* context_lens, const int* block_tables,
                                     int max_blocks, int q_heads, int kv_heads, int head_dim, int page_size, int pages,
                                     int window, float scale, const int* seq_list, int seq_first, int n_list,
                                     int split_keys, int max_splits, float* scratch, int* counters, int cluster,
                                     cudaStream_t s);
TIE_API int tie_attention_decode_prep(const void* qkv, long long qkv_stride, const float* part, long long part_stride,
                                      int part_splits, long long part_ld, const float* qw, const float* kw, float q_eps,
                                      float k_eps, const float* inv_freq, const int* positions, int append, void* k_cache,
                                      void* v_cache, void* out, const int* query_start, const int* context_lens,
                                      const int* block_tables, int max_blocks, int q_heads, int kv_heads, int head_dim,
                                      int page_size, int pages, int window, float scale, const int* seq_list, int seq_first,
                                      int n_list,
                                      int split_keys, int max_splits, float* scratch, int* counters, int cluster,
                                      cudaStream_t s);
TIE_API int tie_attention_prompt_umma(const void* q, long long q_stride, const void* k_cache, const void* v_cache, void* out,
                                      const int* query_start, const int* context_lens, const int* block_tables,
                                      int max_blocks, int n_seqs, int max_queries, int q_heads, int kv_heads, int head_dim,
                                      int page_size, int pages, int window, float scale, cudaStream_t s);
