// Contractions with few tokens (decode steps): Y[T, N] = X[T, K] * W[N, K]^T for T <= 64,
// bfloat16 in, float32 accumulation.  The product is bound by reading W once from HBM, so
// the kernel is a weight streamer: every warp owns 16 rows of W and a share of K, pulls its
// rows with 16-byte non-allocating loads straight into registers (eight loads in flight per
// thread), and feeds them to mma.sync m16n8k16 with the tokens as the N dimension.
//
// Operand layout trick: a 16-byte load holds 8 consecutive k of one row.  Within one MMA a
// thread supplies k slots (2j, 2j+1) and (2j+8, 2j+9); since a dot product does not care about
// the order of k as long as both operands agree, the 8 loaded values feed two MMAs as
// slots (2j,2j+1),(2j+8,2j+9) <- k (8j+0,1),(8j+2,3) and then (8j+4,5),(8j+6,7), and the token
// operand is loaded the same way.  No shared-memory staging of W, no ldmatrix.
//
// The four warps of a CTA split K and sum in shared memory; the grid may split K further
// (``splits``), then float32 partial sums [splits, T, N] are written and the consumer kernel
// adds them up.  Epilogues: store (+ float32 bias) as bfloat16 or float32; partial sums;
// SwiGLU (a CTA holds 8 gate rows and the 8 matching up rows: out = silu(gate) * up).
// The reference runs these products as separate cublasHgemm calls with separate bias and
// SwiGLU kernels (gpu_decoder.cu:334-349, 457-476).
#include "common.cuh"

#define SK_WARPS 4
#define SK_U 4          // k-steps of 32 per load group

#define EPI_STORE 0
#define EPI_PARTIAL 1
#define EPI_SWIGLU 2

__device__ __forceinline__ uint4 ldg_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ void mma16816(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                         unsigned b0, unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <int TN, int EPI, typename TO>
__global__ void __launch_bounds__(SK_WARPS * 32)
gemm_skinny_kernel(const bf16* __restrict__ W, const bf16* __restrict__ X, long long ldx,
                   const float* __restrict__ bias, TO* __restrict__ out, long long ldo,
                   float* __restrict__ part, int T, int N, int K, int splits) {
  __shared__ float red[SK_WARPS][16][TN * 8 + 1];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int j = lane & 3, r = lane >> 2;
  const int tile = blockIdx.x, split = blockIdx.y;
  // rows of W this thread loads
  int row_lo, row_hi;
  if (EPI == EPI_SWIGLU) {
    int F = N >> 1;
    int f = tile * 8 + r;
    if (f >= F) f = F - 1;
    row_lo = f; row_hi = F + f;
  } else {
    row_lo = tile * 16 + r; row_hi = row_lo + 8;
    if (row_lo >= N) row_lo = N - 1;
    if (row_hi >= N) row_hi = N - 1;
  }
  const bf16* w_lo = W + (size_t)row_lo * K + 8 * j;
  const bf16* w_hi = W + (size_t)row_hi * K + 8 * j;
  // token rows of X this thread loads (one per n-tile); tokens past T read row 0 and are never stored
  const bf16* xp[TN];
#pragma unroll
  for (int n = 0; n < TN; n++) {
    int tok = n * 8 + r;
    xp[n] = X + (size_t)(tok < T ? tok : 0) * ldx + 8 * j;
  }
  // groups of SK_U k-steps: this split's range, dealt round-robin to the warps
  const int n_groups = (K + 32 * SK_U - 1) / (32 * SK_U);
  const int g_begin = (int)((long long)n_groups * split / splits);
  const int g_end = (int)((long long)n_groups * (split + 1) / splits);

  float acc[TN][4];
#pragma unroll
  for (int n = 0; n < TN; n++) acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.f;

  // two register buffers of SK_U k-steps each, named apart so that nothing is indexed at run time
  uint4 lo0[SK_U], hi0[SK_U], lo1[SK_U], hi1[SK_U];
  auto load_group = [&](int g, uint4 (&lo)[SK_U], uint4 (&hi)[SK_U]) {
#pragma unroll
    for (int u = 0; u < SK_U; u++) {
      int k = (g * SK_U + u) * 32;
      if (k + 8 * j < K) {
        lo[u] = ldg_stream(w_lo + k);
        hi[u] = ldg_stream(w_hi + k);
      } else {
        lo[u] = make_uint4(0, 0, 0, 0);
        hi[u] = make_uint4(0, 0, 0, 0);
      }
    }
  };
  auto compute_group = [&](int g, const uint4 (&lo)[SK_U], const uint4 (&hi)[SK_U]) {
#pragma unroll
    for (int u = 0; u < SK_U; u++) {
      int k = (g * SK_U + u) * 32;
      bool in = k + 8 * j < K;
#pragma unroll
      for (int n = 0; n < TN; n++) {
        uint4 b = in ? __ldg(reinterpret_cast<const uint4*>(xp[n] + k)) : make_uint4(0, 0, 0, 0);
        mma16816(acc[n], lo[u].x, hi[u].x, lo[u].y, hi[u].y, b.x, b.y);
        mma16816(acc[n], lo[u].z, hi[u].z, lo[u].w, hi[u].w, b.z, b.w);
      }
    }
  };
  int g = g_begin + warp;
  if (g < g_end) load_group(g, lo0, hi0);   // weights: no kernel of the step writes them
  pdl_wait();                               // the tokens come from the kernel before this one
  for (; g < g_end; g += 2 * SK_WARPS) {
    if (g + SK_WARPS < g_end) load_group(g + SK_WARPS, lo1, hi1);
    compute_group(g, lo0, hi0);
    if (g + 2 * SK_WARPS < g_end) load_group(g + 2 * SK_WARPS, lo0, hi0);
    if (g + SK_WARPS < g_end) compute_group(g + SK_WARPS, lo1, hi1);
  }
  pdl_launch_dependents();   // the next kernel may start its prologue while this one reduces
  // sum the four warps' shares of K
#pragma unroll
  for (int n = 0; n < TN; n++) {
    red[warp][r][n * 8 + 2 * j] = acc[n][0];
    red[warp][r][n * 8 + 2 * j + 1] = acc[n][1];
    red[warp][r + 8][n * 8 + 2 * j] = acc[n][2];
    red[warp][r + 8][n * 8 + 2 * j + 1] = acc[n][3];
  }
  __syncthreads();
  if (EPI == EPI_SWIGLU) {
    int F = N >> 1;
    for (int idx = threadIdx.x; idx < 8 * TN * 8; idx += SK_WARPS * 32) {
      int row = idx & 7, tok = idx >> 3;
      int f = tile * 8 + row;
      if (tok >= T || f >= F) continue;
      float gate = 0.f, up = 0.f;
#pragma unroll
      for (int w = 0; w < SK_WARPS; w++) { gate += red[w][row][tok]; up += red[w][row + 8][tok]; }
      out[(size_t)tok * ldo + f] = from_float<TO>(gate / (1.0f + expf(-gate)) * up);
    }
  } else {
    for (int idx = threadIdx.x; idx < 16 * TN * 8; idx += SK_WARPS * 32) {
      int row = idx & 15, tok = idx >> 4;
      int n = tile * 16 + row;
      if (tok >= T || n >= N) continue;
      float v = 0.f;
#pragma unroll
      for (int w = 0; w < SK_WARPS; w++) v += red[w][row][tok];
      if (EPI == EPI_PARTIAL) {
        part[((size_t)split * T + tok) * N + n] = v;
      } else {
        if (bias) v += bias[n];
        out[(size_t)tok * ldo + n] = from_float<TO>(v);
      }
    }
  }
}

template <int TN>
static int launch_skinny(const bf16* W, const bf16* X, long long ldx, const float* bias, void* out,
                         int out_dtype, long long ldo, float* part, int T, int N, int K, int splits, int epi,
                         cudaStream_t stream) {
  dim3 block(SK_WARPS * 32);
  if (epi == EPI_SWIGLU) {
    dim3 grid((N / 2 + 7) / 8, 1);
    if (out_dtype != QD_BF16) return QD_ERR_UNSUPPORTED;
    qd_launch(gemm_skinny_kernel<TN, EPI_SWIGLU, bf16>, dim3(grid), dim3(block), 0, stream, W, X, ldx, nullptr, (bf16*)out, ldo,
                                                                         nullptr, T, N, K, 1);
  } else if (epi == EPI_PARTIAL) {
    dim3 grid((N + 15) / 16, splits);
    qd_launch(gemm_skinny_kernel<TN, EPI_PARTIAL, float>, dim3(grid), dim3(block), 0, stream, W, X, ldx, nullptr, nullptr, 0, part,
                                                                           T, N, K, splits);
  } else {
    dim3 grid((N + 15) / 16, 1);
    if (out_dtype == QD_BF16)
      qd_launch(gemm_skinny_kernel<TN, EPI_STORE, bf16>, dim3(grid), dim3(block), 0, stream, W, X, ldx, bias, (bf16*)out, ldo,
                                                                          nullptr, T, N, K, 1);
    else if (out_dtype == QD_F32)
      qd_launch(gemm_skinny_kernel<TN, EPI_STORE, float>, dim3(grid), dim3(block), 0, stream, W, X, ldx, bias, (float*)out, ldo,
                                                                           nullptr, T, N, K, 1);
    else
      return QD_ERR_UNSUPPORTED;
  }
  return qd_last_error();
}

// epi 0: out[T, N] = X W^T + bias (out_dtype bf16 or f32).  epi 1: part[splits, T, N] float32 partial
// sums over ``splits`` shares of K (no bias).  epi 2: W is [2F, K] = gate rows then up rows, N = 2F,
// out[T, F] = silu(X Wg^T) * (X Wu^T), bfloat16.  X rows are ldx elements apart, out rows ldo.
extern "C" int qd_gemm_skinny(const void* W, const void* X, long long ldx, const float* bias, void* out,
                              int out_dtype, long long ldo, float* part, int T, int N, int K, int splits,
                              int epi, cudaStream_t stream) {
  if (T <= 0 || N <= 0) return 0;
  if (T > 64 || K <= 0 || K % 8 != 0 || ldx % 8 != 0 || splits < 1 || splits > 65535) return QD_ERR_UNSUPPORTED;
  if (((uintptr_t)W & 15) || ((uintptr_t)X & 15)) return QD_ERR_UNSUPPORTED;
  if (epi == EPI_SWIGLU && (N & 1)) return QD_ERR_UNSUPPORTED;
  if (epi == EPI_PARTIAL && !part) return QD_ERR_UNSUPPORTED;
  if (epi != EPI_PARTIAL && splits != 1) return QD_ERR_UNSUPPORTED;
  const bf16* w = (const bf16*)W;
  const bf16* x = (const bf16*)X;
  if (T <= 8) return launch_skinny<1>(w, x, ldx, bias, out, out_dtype, ldo, part, T, N, K, splits, epi, stream);
  if (T <= 16) return launch_skinny<2>(w, x, ldx, bias, out, out_dtype, ldo, part, T, N, K, splits, epi, stream);
  if (T <= 32) return launch_skinny<4>(w, x, ldx, bias, out, out_dtype, ldo, part, T, N, K, splits, epi, stream);
  return launch_skinny<8>(w, x, ldx, bias, out, out_dtype, ldo, part, T, N, K, splits, epi, stream);
}
