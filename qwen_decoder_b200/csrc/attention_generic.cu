// Generic paged attention on CUDA cores, float32 arithmetic: any head size that is a
// multiple of 2 up to 512, any number of heads and groups, any page size, optional
// window.  One warp owns one (token, query head): it walks the keys 0..pos of the
// token's request through the request's block table in tiles of 32 keys, with the
// online softmax of the reference's kernels (gpu_kernels.cu:262-311: running max m,
// denominator, rescaled output).  Tiles start at multiples of 32 counted from key 0,
// so the order of every sum depends only on the token's own position: the result
// does not depend on how the prompt was cut or on what else is in the batch.
// It serves the whole float32 path, and the bfloat16 path for sizes the tensor-core
// kernels refuse.  Prefill portions and decode tokens take the same code: a portion's
// K/V were written to the pages before this kernel runs (gpu_decoder.cu:377-397).
#include "common.cuh"
#include <math.h>

#define AG_WARPS 4
#define AG_MAX_D 512

template <typename T>
__global__ void __launch_bounds__(AG_WARPS * 32)
paged_attention_generic_kernel(const T* __restrict__ q, long long q_stride, T* __restrict__ out,
                               long long out_stride, const T* __restrict__ kv,
                               const int* __restrict__ block_table, int max_blocks,
                               const int* __restrict__ token_req, const int* __restrict__ positions,
                               int n_tokens, int H, int G, int d, int page_size, float scale,
                               int window) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float smem[];
  int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  long long item = (long long)blockIdx.x * AG_WARPS + warp;
  if (item >= (long long)n_tokens * H) return;
  int t = (int)(item / H), h = (int)(item - (long long)t * H);
  int g = h / (H / G);
  float* qs = smem + (size_t)warp * d;
  const T* qr = q + (size_t)t * q_stride + (size_t)h * d;
  for (int i = lane; i < d; i += 32) qs[i] = to_float(qr[i]);
  __syncwarp();

  int pos = positions[t];
  const int* bt = block_table + (size_t)token_req[t] * max_blocks;
  int key_lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  size_t page_elems = (size_t)2 * G * page_size * d;
  size_t head_off = (size_t)g * page_size * d;
  size_t v_off = (size_t)G * page_size * d;

  float m = -INFINITY, l = 0.0f;
  float o[AG_MAX_D / 32];
#pragma unroll
  for (int i = 0; i < AG_MAX_D / 32; i++) o[i] = 0.0f;

  for (int base = key_lo & ~31; base <= pos; base += 32) {
    int key = base + lane;
    bool valid = key >= key_lo && key <= pos;
    float s = -INFINITY;
    if (valid) {
      int page = bt[key / page_size];
      const T* kr = kv + (size_t)page * page_elems + head_off + (size_t)(key % page_size) * d;
      float acc = 0.0f;
      for (int i = 0; i < d; i++) acc = fmaf(qs[i], to_float(kr[i]), acc);
      s = acc * scale;
    }
    float m_new = fmaxf(m, warp_max(s));
    float c = expf(m - m_new);  // m = -inf on the first tile gives 0
    float p = valid ? expf(s - m_new) : 0.0f;
    l = l * c + warp_sum(p);
    m = m_new;
#pragma unroll
    for (int i = 0; i < AG_MAX_D / 32; i++) o[i] *= c;
    int jend = pos - base + 1 < 32 ? pos - base + 1 : 32;
    for (int j = 0; j < jend; j++) {
      float pj = __shfl_sync(0xffffffffu, p, j);
      int kj = base + j;
      if (kj < key_lo) continue;
      int page = bt[kj / page_size];
      const T* vr = kv + (size_t)page * page_elems + v_off + head_off + (size_t)(kj % page_size) * d;
#pragma unroll
      for (int i = 0; i < AG_MAX_D / 32; i++) {
        int idx = lane + 32 * i;
        if (idx < d) o[i] = fmaf(pj, to_float(vr[idx]), o[i]);
      }
    }
  }
  T* orow = out + (size_t)t * out_stride + (size_t)h * d;
  float inv = 1.0f / l;
#pragma unroll
  for (int i = 0; i < AG_MAX_D / 32; i++) {
    int idx = lane + 32 * i;
    if (idx < d) orow[idx] = from_float<T>(o[i] * inv);
  }
}

extern "C" int qd_paged_attention_generic(const void* q, long long q_stride, void* out,
                                          long long out_stride, const void* kv, int dtype,
                                          const int* block_table, int max_blocks,
                                          const int* token_req, const int* positions, int n_tokens,
                                          int H, int G, int d, int page_size, float scale, int window,
                                          cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (d <= 0 || d > AG_MAX_D || G <= 0 || H % G != 0 || page_size <= 0) return QD_ERR_UNSUPPORTED;
  long long items = (long long)n_tokens * H;
  unsigned blocks = (unsigned)((items + AG_WARPS - 1) / AG_WARPS);
  size_t smem = (size_t)AG_WARPS * d * sizeof(float);
  if (dtype == QD_F32)
    qd_launch(paged_attention_generic_kernel<float>, dim3(blocks), dim3(AG_WARPS * 32), smem, stream, 
        (const float*)q, q_stride, (float*)out, out_stride, (const float*)kv, block_table, max_blocks,
        token_req, positions, n_tokens, H, G, d, page_size, scale, window);
  else if (dtype == QD_BF16)
    qd_launch(paged_attention_generic_kernel<bf16>, dim3(blocks), dim3(AG_WARPS * 32), smem, stream, 
        (const bf16*)q, q_stride, (bf16*)out, out_stride, (const bf16*)kv, block_table, max_blocks,
        token_req, positions, n_tokens, H, G, d, page_size, scale, window);
  else
    return QD_ERR_UNSUPPORTED;
  return qd_last_error();
}
