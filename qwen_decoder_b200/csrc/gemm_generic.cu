// Generic contraction Y[T, N] = X[T, K] * W[N, K]^T (+ bias[N]) on CUDA cores with
// float32 FMA: any T, N, K.  It is the whole float32 path's matrix product (no
// TF32, no tensor cores) and the bfloat16 path's fallback for sizes the tensor-core
// kernels refuse.  Each output element is one FMA chain over k = 0..K-1 in order,
// so a row's result does not depend on the other rows of the batch.
//
// The reference calls cublasHgemm for these products (gpu_kernels.cu:431-436) and
// adds the bias in a separate kernel (gpu_kernels.cu:70-79).
#include "common.cuh"

#define GBM 64
#define GBN 64
#define GBK 16

template <typename TI, typename TO>
__global__ void __launch_bounds__(256)
gemm_generic_kernel(const TI* __restrict__ X, const TI* __restrict__ W, const float* __restrict__ bias,
                    TO* __restrict__ Y, int T, int N, int K, long long ldx, long long ldy) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float As[GBK][GBM + 4];
  __shared__ float Bs[GBK][GBN + 4];
  int tid = threadIdx.x;
  int ty = tid >> 4, tx = tid & 15;
  int m0 = blockIdx.y * GBM, n0 = blockIdx.x * GBN;
  int lr = tid >> 2, lk = (tid & 3) * 4;  // load row, first k of four
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; i++)
#pragma unroll
    for (int j = 0; j < 4; j++) acc[i][j] = 0.0f;

  for (int k0 = 0; k0 < K; k0 += GBK) {
    int gm = m0 + lr, gn = n0 + lr;
#pragma unroll
    for (int j = 0; j < 4; j++) {
      int gk = k0 + lk + j;
      As[lk + j][lr] = (gm < T && gk < K) ? to_float(X[(size_t)gm * ldx + gk]) : 0.0f;
      Bs[lk + j][lr] = (gn < N && gk < K) ? to_float(W[(size_t)gn * K + gk]) : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < GBK; kk++) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; i++) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; j++) b[j] = Bs[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; i++) {
    int gm = m0 + ty * 4 + i;
    if (gm >= T) continue;
#pragma unroll
    for (int j = 0; j < 4; j++) {
      int gn = n0 + tx * 4 + j;
      if (gn >= N) continue;
      float v = acc[i][j];
      if (bias) v += bias[gn];
      Y[(size_t)gm * ldy + gn] = from_float<TO>(v);
    }
  }
}

// x_dtype is the type of X and W; y_dtype the type of Y.  ldx / ldy are row strides in
// elements (X and Y may be column slices of wider buffers).
extern "C" int qd_gemm_generic(const void* X, const void* W, int x_dtype, const float* bias, void* Y,
                               int y_dtype, int T, int N, int K, long long ldx, long long ldy,
                               cudaStream_t stream) {
  if (T <= 0 || N <= 0) return 0;
  if (K <= 0) return QD_ERR_UNSUPPORTED;
  dim3 grid((N + GBN - 1) / GBN, (T + GBM - 1) / GBM);
  if (grid.y > 65535) return QD_ERR_UNSUPPORTED;
  if (x_dtype == QD_F32 && y_dtype == QD_F32)
    qd_launch(gemm_generic_kernel<float, float>, dim3(grid), dim3(256), 0, stream, (const float*)X, (const float*)W, bias,
                                                                (float*)Y, T, N, K, ldx, ldy);
  else if (x_dtype == QD_BF16 && y_dtype == QD_BF16)
    qd_launch(gemm_generic_kernel<bf16, bf16>, dim3(grid), dim3(256), 0, stream, (const bf16*)X, (const bf16*)W, bias,
                                                              (bf16*)Y, T, N, K, ldx, ldy);
  else if (x_dtype == QD_BF16 && y_dtype == QD_F32)
    qd_launch(gemm_generic_kernel<bf16, float>, dim3(grid), dim3(256), 0, stream, (const bf16*)X, (const bf16*)W, bias,
                                                               (float*)Y, T, N, K, ldx, ldy);
  else
    return QD_ERR_UNSUPPORTED;
  return qd_last_error();
}
