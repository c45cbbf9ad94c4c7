// The layers of a prompt step launched from native code.
//
// A step with a prompt portion is no replayed graph: its kernels are launched one by one, about nine
// per layer, and from Python each launch costs some 15 us of interpreter, argument conversion and
// tensor bookkeeping -- more than the device needs for portions of a few hundred tokens.  For a model
// whose layers are all the common composition (pre-norm block, grouped-query attention with one
// rotary table, SwiGLU, RMSNorm; bfloat16) this file runs the same kernels, in the same order, with
// the same arguments as the parts do, from one C++ loop:
//
//   per layer:  h = rmsnorm(x += delta) ; qkv = h Wqkv^T ; bias, rotation, cache write ; attention over
//               the pages (the decode kernel for the single tokens of a mixed step, a prompt kernel for the
//               rest) ; delta = attn Wo^T ; h = rmsnorm(x += delta) ; gu = h Wgu^T ; act = silu(gate) * up ;
//               delta = act Wd^T
//   at the end: hrows = rmsnorm(x += delta) at the wanted rows          (the output projection stays outside)
//
// It holds no kernel of its own.  The launchers live in the other libraries of this directory and the
// matrix products in cuBLAS (as the reference's do, gpu_kernels.cu:431-436); the caller hands over their
// addresses, so this library links against none of them and uses whatever cuBLAS the process has loaded.
// The reference launches its layers from C++ as well (gpu_decoder.cu:321-497).
#include "common.cuh"
#include "entry_points.h"
#include <cublas_v2.h>

struct PeLayer {
  const float* norm1_w; const float* norm2_w;
  const void* wqkv; const float* bqkv; const void* wo; const void* wgu; const void* wd;
  void* kv;                        // this layer's pages [pages, 2, G, page_size, d]
  float eps1, eps2;
  int write_kv, pad;
};

// cublasGemmEx (the 32-bit form; the header overloads the name for C++)
typedef cublasStatus_t (*PeGemmEx)(cublasHandle_t, cublasOperation_t, cublasOperation_t, int, int, int, const void*,
                                   const void*, cudaDataType, int, const void*, cudaDataType, int, const void*, void*,
                                   cudaDataType, int, cublasComputeType_t, cublasGemmAlgo_t);

// cublasGemmStridedBatchedEx (32-bit form)
typedef cublasStatus_t (*PeGemmBatched)(cublasHandle_t, cublasOperation_t, cublasOperation_t, int, int, int, const void*,
                                        const void*, cudaDataType, int, long long, const void*, cudaDataType, int,
                                        long long, const void*, void*, cudaDataType, int, long long, int,
                                        cublasComputeType_t, cublasGemmAlgo_t);

struct PeFns {
  decltype(&qd_add_rmsnorm) add_rmsnorm;
  decltype(&qd_rope_kv_write_biased) rope_kv_write;
  decltype(&qd_swiglu) swiglu;
  decltype(&qd_prefill_attention) attention_regs;       // mma.sync, any supported head size
  decltype(&qd_prefill_attention_tc5) attention_tc5;    // tcgen05, head size 64 or 128
  decltype(&qd_decode_attention) attention_decode;      // split-KV, for the single tokens of a mixed step
  PeGemmEx gemm_ex;
  cublasHandle_t blas;             // the caller's handle, bound to ``stream``
  PeGemmBatched gemm_batched;
  decltype(&qd_elementwise_plain_next) plain_next;      // the elementwise library's next launch without the attribute
};

struct PeParams {
  PeFns fn;
  const PeLayer* layers; int n_layers;
  int T, R, D, H, G, d, F, page_size, window, rotary_dim, pairing, max_blocks, use_tc5, n_wanted;
  float scale, final_eps;
  long long n_pages;
  const int* positions; const int* slot_map; const int* block_table; const int* cu_tokens; const int* start_pos;
  const int* logit_rows;
  const float* cos_t; const float* sin_t; const float* final_w;
  float* x;                        // [T, D] residual sum, float32
  const void* delta0;              // null: nothing pending on entry
  void* h; void* qkv; void* attn; void* delta; void* gu; void* act;   // bfloat16 scratch: [T,D] [T,(H+2G)d] [T,Hd] [T,D] [T,2F] [T,F]
  void* hrows;                     // [n_wanted, D] bfloat16
  // a mixed step: requests and tokens 0 .. n_decode-1 are single tokens and go to the decode kernel
  int n_decode, decode_splits;
  const int* token_req; float* part_o; float* part_ml; unsigned* tickets;
  // the down projection over ``down_shares`` equal shares of F as one batched product that leaves float32 partial
  // sums [down_shares, T, D] in ``down_part`` for the next norm's kernel (0: the plain product into ``delta``).
  // With few tokens, a long K and few output features the plain product fills the GPU with too few CTAs.
  float* down_part; int down_shares, pad2;
};

extern "C" int qd_prompt_exec_struct_sizes(int* layer_bytes, int* params_bytes) {
  *layer_bytes = (int)sizeof(PeLayer);
  *params_bytes = (int)sizeof(PeParams);
  return 0;
}

// Y[T, N] = X[T, K] W[N, K]^T, all bfloat16 row-major, float32 accumulation
static int product(const PeParams& p, const void* W, const void* X, void* Y, int T, int N, int K) {
  const float one = 1.f, zero = 0.f;
  cublasStatus_t st = p.fn.gemm_ex(p.fn.blas, CUBLAS_OP_T, CUBLAS_OP_N, N, T, K, &one, W, CUDA_R_16BF, K, X, CUDA_R_16BF,
                                   K, &zero, Y, CUDA_R_16BF, N, CUBLAS_COMPUTE_32F, CUBLAS_GEMM_DEFAULT);
  return st == CUBLAS_STATUS_SUCCESS ? 0 : 20000 + (int)st;
}

// part[s][T, N] = X[T, share s of K] W[N, share s of K]^T in float32, for `shares` equal shares of K
static int product_shares(const PeParams& p, const void* W, const void* X, float* part, int T, int N, int K, int shares) {
  const float one = 1.f, zero = 0.f;
  const int kc = K / shares;
  cublasStatus_t st = p.fn.gemm_batched(p.fn.blas, CUBLAS_OP_T, CUBLAS_OP_N, N, T, kc, &one, W, CUDA_R_16BF, K, kc, X,
                                        CUDA_R_16BF, K, kc, &zero, part, CUDA_R_32F, N, (long long)T * N, shares,
                                        CUBLAS_COMPUTE_32F, CUBLAS_GEMM_DEFAULT);
  return st == CUBLAS_STATUS_SUCCESS ? 0 : 20000 + (int)st;
}

#define PE_TRY(call)            \
  do {                          \
    int rc_ = (call);           \
    if (rc_ != 0) return rc_;   \
  } while (0)

extern "C" int qd_prompt_exec(const PeParams* pp, cudaStream_t stream) {
  const PeParams& p = *pp;
  if (p.T <= 0 || p.n_layers < 0 || p.n_decode < 0 || p.n_decode >= p.R) return QD_ERR_UNSUPPORTED;
  const int shares = p.down_shares;
  if (shares < 0 || shares == 1 ||
      (shares > 1 && (!p.down_part || !p.fn.gemm_batched || !p.fn.plain_next || p.F % (8 * shares))))
    return QD_ERR_UNSUPPORTED;
  const int T = p.T, D = p.D, H = p.H, G = p.G, d = p.d, F = p.F;
  const int n_qkv = (H + 2 * G) * d;
  const long long xn = (long long)T * D;
  const void* delta = p.delta0;
  int delta_dtype = QD_BF16, delta_parts = 1;          // what the previous layer's down projection left
  for (int l = 0; l < p.n_layers; l++) {
    const PeLayer& L = p.layers[l];
    if (delta_parts > 1) p.fn.plain_next();            // the norm that reads the batched product waits for all of it
    PE_TRY(p.fn.add_rmsnorm(p.x, delta, delta ? delta_dtype : -1, L.norm1_w, p.h, QD_BF16, nullptr, T, D, L.eps1, 1,
                            delta_parts, xn, stream));
    PE_TRY(product(p, L.wqkv, p.h, p.qkv, T, n_qkv, D));
    PE_TRY(p.fn.rope_kv_write(p.qkv, L.bqkv, T, H, G, d, p.rotary_dim, p.pairing, p.cos_t, p.sin_t, p.positions, L.kv,
                              p.slot_map, p.page_size, L.write_kv, stream));
    const int nd = p.n_decode;
    if (nd > 0)
      PE_TRY(p.fn.attention_decode(p.qkv, n_qkv, p.attn, L.kv, p.block_table, p.max_blocks, p.token_req, p.positions,
                                   nd, H, G, d, p.page_size, p.scale, p.window, p.decode_splits, p.part_o, p.part_ml,
                                   p.tickets, stream));
    const int* bt = p.block_table + (size_t)nd * p.max_blocks;
    if (p.use_tc5)
      PE_TRY(p.fn.attention_tc5(p.qkv, n_qkv, p.attn, L.kv, p.n_pages, bt, p.max_blocks, p.cu_tokens + nd,
                                p.start_pos + nd, p.R - nd, T - nd, H, G, d, p.page_size, p.scale, p.window, nullptr,
                                stream));
    else
      PE_TRY(p.fn.attention_regs(p.qkv, n_qkv, p.attn, L.kv, bt, p.max_blocks, p.cu_tokens + nd, p.start_pos + nd,
                                 p.R - nd, T - nd, H, G, d, p.page_size, p.scale, p.window, stream));
    PE_TRY(product(p, L.wo, p.attn, p.delta, T, D, H * d));
    PE_TRY(p.fn.add_rmsnorm(p.x, p.delta, QD_BF16, L.norm2_w, p.h, QD_BF16, nullptr, T, D, L.eps2, 1, 1, xn, stream));
    PE_TRY(product(p, L.wgu, p.h, p.gu, T, 2 * F, D));
    PE_TRY(p.fn.swiglu(p.gu, p.act, QD_BF16, T, F, stream));
    if (shares > 1) {
      PE_TRY(product_shares(p, L.wd, p.act, p.down_part, T, D, F, shares));
      delta = p.down_part; delta_dtype = QD_F32; delta_parts = shares;
    } else {
      PE_TRY(product(p, L.wd, p.act, p.delta, T, D, F));
      delta = p.delta;
    }
  }
  if (p.n_wanted > 0 && delta_parts > 1) p.fn.plain_next();
  if (p.n_wanted > 0)
    PE_TRY(p.fn.add_rmsnorm(p.x, delta, delta ? delta_dtype : -1, p.final_w, p.hrows, QD_BF16, p.logit_rows, p.n_wanted,
                            D, p.final_eps, 0, delta_parts, xn, stream));     // only the wanted rows: x itself stays as it is
  return 0;
}
