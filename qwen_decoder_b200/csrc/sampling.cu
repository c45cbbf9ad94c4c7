// Sampling over float32 logits on the device: greedy, temperature, top-k.
//
// Semantics of the reference's host sampler (common.cpp:564-629): temperature 0 is
// argmax with the lowest index winning ties (common.cpp:564-574); otherwise
// p_i = exp((l_i - max) / T) over the kept entries, normalised, and the first index
// whose running sum reaches the uniform draw r is returned (common.cpp:590-598);
// with 0 < k < V only entries >= the k-th largest logit are kept, ties included
// (common.cpp:600-618).  The draw r is given per row by the caller, so that a request's
// draws do not depend on the batch it is in.
#include "common.cuh"
#include <math.h>

#define SB 1024

__device__ __forceinline__ unsigned order_key(float f) {
  unsigned u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);  // ascending in float order
}
__device__ __forceinline__ float key_to_float(unsigned k) {
  unsigned u = (k & 0x80000000u) ? (k & 0x7fffffffu) : ~k;
  return __uint_as_float(u);
}

__global__ void __launch_bounds__(SB)
sample_kernel(const float* __restrict__ logits, int V, const float* __restrict__ temperature,
              const int* __restrict__ top_k, const float* __restrict__ draws, int* __restrict__ out) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float s_val[SB];
  __shared__ int s_idx[SB];
  __shared__ unsigned s_hist[256];
  __shared__ float s_scratch[40];
  __shared__ unsigned s_prefix, s_remaining;
  __shared__ int s_result;
  int r = blockIdx.x, tid = threadIdx.x;
  const float* row = logits + (size_t)r * V;

  // 1. maximum and its lowest index
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = tid; i < V; i += SB) {
    float v = row[i];
    if (v > best || bi == 0x7fffffff) { best = v; bi = i; }
  }
  s_val[tid] = best; s_idx[tid] = bi;
  __syncthreads();
  for (int s = SB / 2; s > 0; s >>= 1) {
    if (tid < s) {
      float ov = s_val[tid + s]; int oi = s_idx[tid + s];
      if (oi != 0x7fffffff && (s_idx[tid] == 0x7fffffff || ov > s_val[tid] ||
                               (ov == s_val[tid] && oi < s_idx[tid]))) {
        s_val[tid] = ov; s_idx[tid] = oi;
      }
    }
    __syncthreads();
  }
  float mx = s_val[0];
  int amax = s_idx[0];
  float temp = temperature[r];
  if (temp == 0.0f) {
    if (tid == 0) out[r] = amax;
    return;
  }

  // 2. threshold = k-th largest logit (radix select on order-preserving keys)
  int k = top_k[r];
  float threshold = -INFINITY;
  if (k > 0 && k < V) {
    if (tid == 0) { s_prefix = 0; s_remaining = (unsigned)k; }
    __syncthreads();
    for (int shift = 24; shift >= 0; shift -= 8) {
      if (tid < 256) s_hist[tid] = 0;
      __syncthreads();
      unsigned prefix = s_prefix;
      unsigned mask = shift == 24 ? 0u : (0xffffffffu << (shift + 8));
      for (int i = tid; i < V; i += SB) {
        unsigned key = order_key(row[i]);
        if ((key & mask) == prefix) atomicAdd(&s_hist[(key >> shift) & 255u], 1u);
      }
      __syncthreads();
      if (tid == 0) {
        unsigned rem = s_remaining;
        int dgt = 255;
        for (; dgt > 0; dgt--) {
          unsigned c = s_hist[dgt];
          if (c >= rem) break;
          rem -= c;
        }
        s_prefix = prefix | ((unsigned)dgt << shift);
        s_remaining = rem;
      }
      __syncthreads();
    }
    threshold = key_to_float(s_prefix);
  }

  // 3. each thread owns a contiguous segment; segment sums of the kept probabilities
  int seg = (V + SB - 1) / SB;
  int lo = tid * seg, hi = lo + seg < V ? lo + seg : V;
  float part = 0.0f;
  for (int i = lo; i < hi; i++) {
    float v = row[i];
    if (v >= threshold) part += expf((v - mx) / temp);
  }
  s_val[tid] = part;
  __syncthreads();
  float total = block_sum(part, s_scratch);
  // 4. first index whose running sum reaches r * total
  if (tid == 0) {
    float target = draws[r] * total;
    float cum = 0.0f;
    int found = -1;
    for (int sgi = 0; sgi < SB && found < 0; sgi++) {
      float next = cum + s_val[sgi];
      if (target <= next && s_val[sgi] > 0.0f) {
        int a = sgi * seg, b = a + seg < V ? a + seg : V;
        for (int i = a; i < b; i++) {
          float v = row[i];
          if (v >= threshold) {
            cum += expf((v - mx) / temp);
            if (target <= cum) { found = i; break; }
          }
        }
        if (found < 0) cum = next;  // rounding: go on with the next segment
      } else {
        cum = next;
      }
    }
    s_result = found >= 0 ? found : amax;
  }
  __syncthreads();
  if (tid == 0) out[r] = s_result;
}

extern "C" int qd_sample(const float* logits, int R, int V, const float* temperature, const int* top_k,
                         const float* draws, int* out, cudaStream_t stream) {
  if (R <= 0) return 0;
  if (V <= 0) return QD_ERR_UNSUPPORTED;
  qd_launch(sample_kernel, dim3(R), dim3(SB), 0, stream, logits, V, temperature, top_k, draws, out);
  return qd_last_error();
}
