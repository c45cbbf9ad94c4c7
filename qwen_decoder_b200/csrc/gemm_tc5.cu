// Contraction Y[T, N] = X[T, K] * W[N, K]^T on the fifth-generation tensor cores:
// tcgen05.mma with the accumulator in tensor memory (TMEM), operands staged in shared
// memory by TMA tensor copies (cp.async.bulk.tensor, 128-byte swizzle), bfloat16 in,
// float32 accumulation.
//
// Orientation: the weights are the MMA's A operand (128 rows of W = 128 output features per
// tile, K-major as stored) and the tokens its B operand (BN = 16..256 tokens per tile,
// K-major as stored), so D[feature, token] lives in TMEM with one feature per lane and one
// token per column.  A few tokens (decode) and many tokens (prefill) are the same kernel with
// another BN; the epilogue thread that owns a feature's lane adds that feature's bias, or
// combines the gate and the up accumulator of its feature (SwiGLU), without any exchange.
//
// Roles in a CTA of 192 threads (one CTA per SM, persistent over work items = feature tile x
// token tile x share of K):
//   warp 0   producer: one lane issues the TMA copies of a stage (A: 128 x 64 box, or two of
//            them for SwiGLU; B: BN x 64 box) onto the stage's "full" mbarrier;
//   warp 1   allocates TMEM; one lane issues four tcgen05.mma (K = 16 each) per stage and
//            commits them to the stage's "empty" mbarrier, and after an item's last stage
//            to the accumulator's "ready" mbarrier;
//   warps 2-5  epilogue: tcgen05.ld of their 32 lanes, bias / SwiGLU / conversion, stores;
//            the accumulator is double-buffered in TMEM so that the epilogue of one item runs
//            under the MMAs of the next.
// The producer requests the first stages' weights before the programmatic-dependency wait and
// the tokens after it.  Every mbarrier wait is bounded (see `dead` below).
//
// The reference calls cublasHgemm for these products (gpu_kernels.cu:431-436) and adds bias
// and SwiGLU in separate kernels (gpu_kernels.cu:70-79, 149-160).
#include "common.cuh"
#include <cuda.h>

#define TC_THREADS 192
#define TC_BM 128
#define TC_BK 64
#define TC_MAX_STAGES 8
#define TC_SPIN_LIMIT (1u << 24)

#define EPI_STORE 0
#define EPI_PARTIAL 1
#define EPI_SWIGLU 2

__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(unsigned long long* bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(unsigned long long* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(unsigned long long* bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// true when the phase with this parity has completed; false after TC_SPIN_LIMIT polls, or at once
// when a wait of this CTA has already run out (*dead set): then nobody spins again, every role runs
// on to its end without leaving early, the kernel ends and the host sees a non-zero status.
__device__ __forceinline__ bool mbar_wait(unsigned long long* bar, unsigned parity, volatile int* dead,
                                          unsigned backoff_ns = 0, unsigned poll_limit = TC_SPIN_LIMIT) {
  return qd_mbar_wait_bounded(smem_u32(bar), parity, dead, poll_limit, 2000000000ull, backoff_ns);
}
// x = innermost coordinate (k, in elements; always a multiple of 64 here: 128 bytes), y = row
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, unsigned long long* bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
               ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y) : "memory");
}
// plain bulk copy of ``bytes`` contiguous bytes (16-byte aligned) onto the same kind of mbarrier
__device__ __forceinline__ void bulk_load(void* dst, const void* src, unsigned bytes, unsigned long long* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes with the 128-byte
// swizzle, as the TMA copies above leave it: rows of 8 form groups 1024 bytes apart.
__device__ __forceinline__ unsigned long long smem_desc_sw128(unsigned addr) {
  unsigned long long d = 0;
  d |= (unsigned long long)((addr & 0x3FFFF) >> 4);        // start address, 16-byte units
  d |= (unsigned long long)1 << 16;                        // leading byte offset (unused with swizzle)
  d |= (unsigned long long)(1024 >> 4) << 32;              // stride byte offset: 8 rows x 128 bytes
  d |= (unsigned long long)1 << 46;                        // descriptor version of this architecture
  d |= (unsigned long long)2 << 61;                        // layout: 128-byte swizzle
  return d;
}
__device__ __forceinline__ void umma_bf16(unsigned tmem_d, unsigned long long desc_a, unsigned long long desc_b,
                                          unsigned idesc, unsigned accumulate) {
  asm volatile(
      "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
      " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n}\n"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}
__device__ __forceinline__ void umma_commit(unsigned long long* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld16(unsigned taddr, unsigned (&v)[16]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"
               : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
                 "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
               : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

struct TcParams {
  int T, N, K;            // tokens, output features (for SwiGLU: 2F rows of W), contraction
  int BN;                 // tokens per tile: 16, 32, 64, 128 or 256
  int splits;             // shares of K (partial sums) or 1
  int n_ftiles, n_ttiles; // feature tiles of 128, token tiles of BN
  int stages;             // shared-memory stages in the ring
  int kbs;                // 64-wide k blocks per stage (several: long contiguous reads of each weight row)
  int acc_cols;           // TMEM columns of one accumulator buffer
  int nacc;               // independent accumulators per buffer, used round-robin over the k-steps and added in
                          // the epilogue: back-to-back MMAs into one accumulator wait for each other (about 220
                          // cycles each at N = 16), MMAs into different accumulators overlap
  int set_cols;           // TMEM columns of one accumulator set (BN, or 2 BN for SwiGLU)
  int tmem_cols;          // TMEM columns allocated (power of two >= 32)
  long long ldo;          // row stride of out, elements
  int w_tiled;            // W is stored tile by tile: [feature tile][k block][128][64], each tile one 16 KB run
  int w_up_tile0;         // SwiGLU with tiled W: index of the first feature tile of the up half
};

template <int EPI, typename TO>
__global__ void __launch_bounds__(TC_THREADS)
gemm_tc5_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                const bf16* __restrict__ w_tiles, const float* __restrict__ bias, TO* __restrict__ out,
                float* __restrict__ part, const TcParams p, int* __restrict__ status) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  __shared__ unsigned long long full_bar[TC_MAX_STAGES], empty_bar[TC_MAX_STAGES], acc_ready[2], acc_free[2];
  __shared__ unsigned tmem_base_slot;
  __shared__ int dead;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int A_TILES = EPI == EPI_SWIGLU ? 2 : 1;
  const int a_bytes = TC_BM * TC_BK * 2;                       // one 128 x 64 box
  const int b_bytes = p.BN * TC_BK * 2;
  const int blk_bytes = A_TILES * a_bytes + b_bytes;           // one k block: multiples of 1024, tiles stay 1024-aligned
  const int stage_bytes = p.kbs * blk_bytes;
  // dynamic shared memory is only guaranteed 16-byte aligned: round the base up to 1024
  unsigned char* tiles = smem_raw + ((1024 - (smem_u32(smem_raw) & 1023)) & 1023);

  if (threadIdx.x == 0) {
    dead = 0;
    for (int s = 0; s < p.stages; s++) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int b = 0; b < 2; b++) { mbar_init(&acc_ready[b], 1); mbar_init(&acc_free[b], 4); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)),
                 "r"((unsigned)p.tmem_cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const unsigned tmem_base = tmem_base_slot;

  const int kb_total = (p.K + TC_BK - 1) / TC_BK;
  const int n_items = p.n_ftiles * p.n_ttiles * p.splits;
  const int F = p.N >> 1;                                      // SwiGLU: features per half

  // item -> (feature tile, token tile, share of K); neighbouring CTAs take neighbouring feature
  // tiles of the same token tile, so the token tile is shared through L2
  auto decode = [&](int item, int& ft, int& tt, int& kb0, int& kb1) {
    int sp = item % p.splits;
    int rest = item / p.splits;
    ft = rest % p.n_ftiles;
    tt = rest / p.n_ftiles;
    kb0 = (int)((long long)kb_total * sp / p.splits);
    kb1 = (int)((long long)kb_total * (sp + 1) / p.splits);
    return sp;
  };

  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    if (lane == 0) {
      unsigned it = 0;
      bool waited = false;
      // sub-block j of stage s holds k block kb: [A (gate) | A (up, SwiGLU only) | B]
      auto load_a = [&](unsigned s, int j, int ft, int kb) {
        unsigned char* st = tiles + (size_t)s * stage_bytes + (size_t)j * blk_bytes;
        if (p.w_tiled) {
          // the tile is stored as its shared-memory image (swizzle applied): one contiguous 16 KB copy
          const unsigned char* wt = reinterpret_cast<const unsigned char*>(w_tiles);
          bulk_load(st, wt + (size_t)(ft * kb_total + kb) * a_bytes, a_bytes, &full_bar[s]);
          if (EPI == EPI_SWIGLU)
            bulk_load(st + a_bytes, wt + (size_t)((p.w_up_tile0 + ft) * kb_total + kb) * a_bytes, a_bytes, &full_bar[s]);
        } else {
          tma_load_2d(st, &map_w, kb * TC_BK, ft * TC_BM, &full_bar[s]);
          if (EPI == EPI_SWIGLU) tma_load_2d(st + a_bytes, &map_w, kb * TC_BK, F + ft * TC_BM, &full_bar[s]);
        }
      };
      auto load_b = [&](unsigned s, int j, int tt, int kb) {
        tma_load_2d(tiles + (size_t)s * stage_bytes + (size_t)j * blk_bytes + A_TILES * a_bytes, &map_x, kb * TC_BK,
                    tt * p.BN, &full_bar[s]);
      };
      auto tokens_of_first_stages = [&]() {       // the B boxes of the stages whose A boxes went out before the wait
        pdl_wait();
        waited = true;
        unsigned jt = 0;
        for (int item2 = blockIdx.x; item2 < n_items && jt < it; item2 += gridDim.x) {
          int ft2, tt2, k0, k1;
          decode(item2, ft2, tt2, k0, k1);
          for (int kb = k0; kb < k1 && jt < it; kb += p.kbs, jt++)
            for (int j = 0; j < p.kbs && kb + j < k1; j++) load_b(jt % p.stages, j, tt2, kb + j);
        }
      };
      for (int item = blockIdx.x; item < n_items; item += gridDim.x) {
        int ft, tt, kb0, kb1;
        decode(item, ft, tt, kb0, kb1);
        for (int kb = kb0; kb < kb1; kb += p.kbs, it++) {
          const unsigned s = it % p.stages, ph = (it / p.stages) & 1;
          if (it == (unsigned)p.stages && !waited) tokens_of_first_stages();
          if (!mbar_wait(&empty_bar[s], ph ^ 1, &dead)) atomicExch(status, 1);
          const int nb = min(p.kbs, kb1 - kb);
          mbar_expect_tx(&full_bar[s], (unsigned)(nb * blk_bytes));
          for (int j = 0; j < nb; j++) load_a(s, j, ft, kb + j);     // back to back: each weight row is read in one run
          if (waited) for (int j = 0; j < nb; j++) load_b(s, j, tt, kb + j);
        }
      }
      if (!waited) tokens_of_first_stages();
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    // One thread issues every MMA of the CTA, so its instruction count per MMA bounds the tensor rate:
    // descriptors are one 64-bit add apart (32 bytes of k = 2 units of 16 bytes), nothing is divided.
    if (lane == 0) {
      const unsigned idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(p.BN >> 3) << 17) | ((unsigned)(TC_BM >> 4) << 24);
      const unsigned long long desc_hi = smem_desc_sw128(0);       // everything but the start address
      const unsigned tiles_addr = smem_u32(tiles);
      const unsigned set_cols = p.set_cols, nacc = p.nacc;
      unsigned it = 0, n_done = 0;
      for (int item = blockIdx.x; item < n_items; item += gridDim.x, n_done++) {
        int ft, tt, kb0, kb1;
        decode(item, ft, tt, kb0, kb1);
        const unsigned buf = n_done & 1, use = n_done >> 1;
        if (!mbar_wait(&acc_free[buf], (use & 1) ^ 1, &dead)) atomicExch(status, 3);   // epilogue has drained it
        tc_fence_after();
        const unsigned d0 = tmem_base + buf * p.acc_cols;
        unsigned d = d0, acc_i = 0, fresh = nacc;     // accumulators still unwritten in this item
        for (int kb = kb0; kb < kb1; kb += p.kbs, it++) {
          const unsigned s = it % p.stages, ph = (it / p.stages) & 1;
          if (!mbar_wait(&full_bar[s], ph, &dead)) atomicExch(status, 2);
          tc_fence_after();
          const int nb = min(p.kbs, kb1 - kb);
          unsigned a_addr = tiles_addr + s * (unsigned)stage_bytes;
          for (int j = 0; j < nb; j++, a_addr += (unsigned)blk_bytes) {
            const unsigned long long da = desc_hi | (unsigned long long)((a_addr & 0x3FFFF) >> 4);
            const unsigned long long du = desc_hi | (unsigned long long)(((a_addr + a_bytes) & 0x3FFFF) >> 4);
            const unsigned long long db = desc_hi | (unsigned long long)(((a_addr + A_TILES * a_bytes) & 0x3FFFF) >> 4);
#pragma unroll
            for (int k = 0; k < TC_BK / 16; k++) {
              const unsigned accf = fresh ? 0u : 1u;            // the first use of an accumulator overwrites it
              umma_bf16(d, da + 2 * k, db + 2 * k, idesc, accf);
              if (EPI == EPI_SWIGLU) umma_bf16(d + p.BN, du + 2 * k, db + 2 * k, idesc, accf);
              if (fresh) fresh--;
              d += set_cols;
              if (++acc_i == nacc) { acc_i = 0; d = d0; }
            }
          }
          umma_commit(&empty_bar[s]);        // the stage is free once these MMAs have read it
        }
        umma_commit(&acc_ready[buf]);        // the accumulator is complete once all MMAs so far are done
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    const int lane_base = (warp & 3) * 32;   // the TMEM lanes this warp may read
    unsigned n_done = 0;
    for (int item = blockIdx.x; item < n_items; item += gridDim.x, n_done++) {
      int ft, tt, kb0, kb1;
      const int sp = decode(item, ft, tt, kb0, kb1);
      const unsigned buf = n_done & 1, use = n_done >> 1;
      if (!mbar_wait(&acc_ready[buf], use & 1, &dead, 256) && lane == 0) atomicExch(status, 4);
      tc_fence_after();
      const int feature = ft * TC_BM + lane_base + lane;           // within a half for SwiGLU
      const int n_feat = EPI == EPI_SWIGLU ? F : p.N;
      const float bv = (EPI == EPI_STORE && bias && feature < n_feat) ? bias[feature] : 0.f;
      const unsigned t0 = tmem_base + ((unsigned)lane_base << 16) + buf * p.acc_cols;
      const int n_used = min(p.nacc, (kb1 - kb0) * (TC_BK / 16));    // accumulators this item wrote
      for (int c = 0; c < p.BN; c += 16) {
        float v[16], u[16];
#pragma unroll
        for (int i = 0; i < 16; i++) { v[i] = 0.f; u[i] = 0.f; }
        for (int a = 0; a < n_used; a++) {
          unsigned r[16], q[16];
          tmem_ld16(t0 + a * p.set_cols + c, r);
          if (EPI == EPI_SWIGLU) tmem_ld16(t0 + a * p.set_cols + p.BN + c, q);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 16; i++) {
            v[i] += __uint_as_float(r[i]);
            if (EPI == EPI_SWIGLU) u[i] += __uint_as_float(q[i]);
          }
        }
        if (feature < n_feat) {
#pragma unroll
          for (int i = 0; i < 16; i++) {
            const int tok = tt * p.BN + c + i;
            if (tok < p.T) {
              float a = v[i];
              if (EPI == EPI_SWIGLU) {
                out[(size_t)tok * p.ldo + feature] = from_float<TO>(a / (1.0f + expf(-a)) * u[i]);
              } else if (EPI == EPI_PARTIAL) {
                part[((size_t)sp * p.T + tok) * p.N + feature] = a;
              } else {
                out[(size_t)tok * p.ldo + feature] = from_float<TO>(a + bv);
              }
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_free[buf]);
    }
  }
  pdl_launch_dependents();
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((unsigned)p.tmem_cols) : "memory");
  }
}

// ------------------------------------------------------------------------------------ host
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  }
  return fn;
}

// rows x cols bfloat16, row stride ld elements; box = box_rows x 64 columns, 128-byte swizzle, zero fill
static bool make_map(CUtensorMap* map, const void* base, long long rows, long long cols, long long ld, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {TC_BK, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

static int* g_status[64];
static int* status_word() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  if (!g_status[dev]) {
    int* ptr = nullptr;
    if (cudaMalloc(&ptr, sizeof(int)) != cudaSuccess) return nullptr;
    cudaMemset(ptr, 0, sizeof(int));
    g_status[dev] = ptr;
  }
  return g_status[dev];
}

// epi 0: out[T, N] = X W^T + bias (out_dtype bf16 or f32); epi 1: part[splits, T, N] float32 partial sums
// over ``splits`` shares of K; epi 2: W = [gate rows; up rows] of shape [2F, K] (F a multiple of 128 is not
// required), out[T, F] = silu(X Wg^T) * (X Wu^T) in bfloat16.  X rows are ldx elements apart, out rows ldo.
// K a multiple of 8, ldx a multiple of 8, W and X 16-byte aligned.  max_ctas bounds the persistent grid.
// w_tiled: W is given tile by tile, [ceil(N/128)][ceil(K/64)][128][64] zero-padded, each tile stored as its
// shared-memory image with the 128-byte swizzle applied (see ``tile_weight`` in kernels.py): a tile then arrives
// with one contiguous 16 KB bulk copy instead of a TMA box of 128 rows x 128 bytes.
extern "C" int qd_gemm_tc5(const void* W, const void* X, long long ldx, const float* bias, void* out, int out_dtype,
                           long long ldo, float* part, int T, int N, int K, int splits, int epi, int max_ctas,
                           int w_tiled, cudaStream_t stream) {
  if (T <= 0 || N <= 0) return 0;
  if (K <= 0 || K % 8 != 0 || ldx % 8 != 0 || splits < 1 || max_ctas < 1) return QD_ERR_UNSUPPORTED;
  if (((uintptr_t)W & 15) || ((uintptr_t)X & 15)) return QD_ERR_UNSUPPORTED;
  if (epi == EPI_SWIGLU && (N & 1)) return QD_ERR_UNSUPPORTED;
  if (epi == EPI_PARTIAL && !part) return QD_ERR_UNSUPPORTED;
  if (epi != EPI_PARTIAL && splits != 1) return QD_ERR_UNSUPPORTED;
  const int kb_total = (K + TC_BK - 1) / TC_BK;
  if (splits > kb_total) return QD_ERR_UNSUPPORTED;
  int* status = status_word();
  if (!status) return QD_ERR_UNSUPPORTED;

  TcParams p;
  p.T = T; p.N = N; p.K = K; p.splits = splits; p.ldo = ldo;
  p.BN = T <= 16 ? 16 : T <= 32 ? 32 : T <= 64 ? 64 : T <= 128 ? 128 : 256;
  if (epi == EPI_SWIGLU && p.BN > 128) p.BN = 128;       // two accumulators x two buffers must fit 512 columns
  const int feats = epi == EPI_SWIGLU ? N / 2 : N;
  p.n_ftiles = (feats + TC_BM - 1) / TC_BM;
  p.n_ttiles = (T + p.BN - 1) / p.BN;
  const int a_tiles = epi == EPI_SWIGLU ? 2 : 1;
  const int blk_bytes = a_tiles * TC_BM * TC_BK * 2 + p.BN * TC_BK * 2;
  // few tokens: the product is bound by reading W, and DRAM likes long runs: four k blocks (512 bytes
  // of every weight row) per stage; many tokens: one k block per stage, more stages
  p.kbs = T <= 64 ? 4 : 1;
  int min_stages = 3;
  int smem_budget = 200 * 1024;
  if (p.kbs > (kb_total + splits - 1) / splits) p.kbs = (kb_total + splits - 1) / splits;
  while (p.kbs > 1 && smem_budget / (p.kbs * blk_bytes) < min_stages) p.kbs /= 2;     // keep at least three stages
  const int stage_bytes = p.kbs * blk_bytes;
  p.stages = smem_budget / stage_bytes;
  if (p.stages > TC_MAX_STAGES) p.stages = TC_MAX_STAGES;
  if (p.stages < 1) return QD_ERR_UNSUPPORTED;
  p.set_cols = a_tiles * p.BN;
  p.nacc = 4;
  while (p.nacc > 1 && 2 * p.nacc * p.set_cols > 512) p.nacc /= 2;
  if (p.nacc < 1) p.nacc = 1;
  p.acc_cols = p.nacc * p.set_cols < 32 ? 32 : p.nacc * p.set_cols;
  int cols = 2 * p.acc_cols;
  p.tmem_cols = 32;
  while (p.tmem_cols < cols) p.tmem_cols *= 2;
  if (p.tmem_cols > 512) return QD_ERR_UNSUPPORTED;

  CUtensorMap map_w, map_x;
  p.w_tiled = w_tiled;
  p.w_up_tile0 = p.n_ftiles;
  // tiled W: tile (ft, kb) is the 16 KB at ((ft * kb_total + kb) * 16 KB); SwiGLU: the gate half's tiles, then the
  // up half's (each half padded to whole tiles); no tensor map is needed for it (map_w then describes X as well)
  bool ok_w = w_tiled ? make_map(&map_w, X, T, K, ldx, p.BN) : make_map(&map_w, W, N, K, K, TC_BM);
  if (!ok_w || !make_map(&map_x, X, T, K, ldx, p.BN)) return QD_ERR_UNSUPPORTED;
  const long long n_items = (long long)p.n_ftiles * p.n_ttiles * splits;
  const int grid = (int)(n_items < max_ctas ? n_items : max_ctas);
  const size_t smem = (size_t)p.stages * stage_bytes + 1024;
#define LAUNCH(E, TO)                                                                                        \
  do {                                                                                                       \
    cudaFuncSetAttribute(gemm_tc5_kernel<E, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);    \
    qd_launch(gemm_tc5_kernel<E, TO>, dim3(grid), dim3(TC_THREADS), smem, stream, map_w, map_x,               \
              (const bf16*)W, bias, (TO*)out, part, p, status);                                              \
  } while (0)
  if (epi == EPI_SWIGLU) {
    if (out_dtype != QD_BF16) return QD_ERR_UNSUPPORTED;
    LAUNCH(EPI_SWIGLU, bf16);
  } else if (epi == EPI_PARTIAL) {
    LAUNCH(EPI_PARTIAL, float);
  } else if (out_dtype == QD_BF16) {
    LAUNCH(EPI_STORE, bf16);
  } else if (out_dtype == QD_F32) {
    LAUNCH(EPI_STORE, float);
  } else {
    return QD_ERR_UNSUPPORTED;
  }
#undef LAUNCH
  return qd_last_error();
}

// 0 if no bounded wait of this library's kernels has run out on the current device (1: producer waiting
// for a free stage, 2: MMA issuer waiting for data, 3: MMA issuer waiting for a drained accumulator,
// 4: epilogue waiting for a complete accumulator).  Synchronises the device.
QD_DEFINE_WAIT_PROBE(qd_gemm_tc5_wait_probe, mbar_wait(bar, 0, dead, 0, poll_limit), status_word, 99)

extern "C" int qd_gemm_tc5_status() {
  int* status = status_word();
  if (!status) return -1;
  int v = 0;
  if (cudaMemcpy(&v, status, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
  if (v) cudaMemset(status, 0, sizeof(int));      // reported once
  return v;
}
