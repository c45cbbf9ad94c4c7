// Prototypes of the kernel launchers that the native prompt-step executor (prompt_exec.cu) calls
// through pointers.  The libraries that define them include this file as well, so that a definition
// that drifts from its prototype does not compile.
#pragma once
#include <cuda_runtime.h>

extern "C" {
int qd_add_rmsnorm(float* x, const void* delta, int delta_dtype, const float* w, void* out, int out_dtype,
                   const int* rows, int n_rows, int D, float eps, int write_back, int n_parts,
                   long long part_stride, cudaStream_t stream);
int qd_rope_kv_write_biased(void* qkv, const float* bias, int T, int H, int G, int d, int rotary_dim, int pairing,
                            const float* cos_t, const float* sin_t, const int* positions, void* kv,
                            const int* slot_map, int page_size, int write_kv, cudaStream_t stream);
int qd_swiglu(const void* gate_up, void* out, int dtype, int T, int F, cudaStream_t stream);
void qd_elementwise_plain_next();
int qd_decode_attention(const void* q, long long q_stride, void* out, const void* kv, const int* block_table,
                        int max_blocks, const int* token_req, const int* positions, int T, int H, int G, int d,
                        int page_size, float scale, int window, int splits, float* part_o, float* part_ml,
                        unsigned* tickets, cudaStream_t stream);
int qd_prefill_attention(const void* q, long long q_stride, void* out, const void* kv, const int* block_table,
                         int max_blocks, const int* cu_tokens, const int* start_pos, int R, int T, int H, int G,
                         int d, int page_size, float scale, int window, cudaStream_t stream);
int qd_prefill_attention_tc5(const void* q, long long q_stride, void* out, const void* kv, long long n_pages,
                             const int* block_table, int max_blocks, const int* cu_tokens, const int* start_pos,
                             int R, int T, int H, int G, int d, int page_size, float scale, int window,
                             long long* timeline, cudaStream_t stream);
}
