// Paged prefill attention on the fifth-generation tensor cores: S = Q K^T and O = P V by tcgen05.mma with
// the accumulators in tensor memory, K and V tiles fetched from the cache pages by TMA tensor copies
// (128-byte swizzle), float32 online softmax by one thread per row.
//
// A CTA takes 128 rows = (128 / gs) tokens x the gs query heads of one KV head (as attention_flash.cu
// does with 64 or 128 rows), and walks key tiles of 128 through the request's block table.  Warps:
//   4        producer: per key tile, 16-key boxes of K and of V (two 64-column halves each) from the pages
//   5        issues the MMAs (one thread): S = Q K^T (both operands K-major), O' = P V (V is MN-major:
//            its rows are keys, the contraction dimension)
//   0..3     softmax: thread r owns row r (= TMEM lane r): loads S from tensor memory, scales, masks,
//            keeps the running maximum and sum, writes P as bfloat16 into shared memory in the layout
//            the MMA reads, then adds O' into its output row (held in registers, rescaled when the
//            maximum moves).
// Formulas: gpu_kernels.cu:223-311 of the reference (scores q.k / sqrt(d), causal, softmax, weighted sum).
// Keys past a row's position are masked on the scores; their V rows are whatever finite values the
// pages hold (the cache starts as zeros and is only ever written with finite numbers), times zero.
//
// Every wait on an mbarrier is bounded in polls and in time; a wait that runs out marks the CTA dead:
// nobody waits again, all roles run to their end, tensor memory is freed, and the host reads a status.
#include "common.cuh"
#include <cuda.h>
#include <cudaTypedefs.h>

#define AT_THREADS 192
#define AT_ROWS 128
#define AT_KEYS 128
#define AT_SPIN_LIMIT (1u << 24)

__device__ __forceinline__ unsigned at_smem(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void at_mbar_init(unsigned long long* bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(at_smem(bar)), "r"(count));
}
__device__ __forceinline__ void at_mbar_arrive(unsigned long long* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(at_smem(bar)) : "memory");
}
__device__ __forceinline__ void at_mbar_expect_tx(unsigned long long* bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(at_smem(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool at_mbar_wait(unsigned long long* bar, unsigned parity, volatile int* dead) {
  unsigned addr = at_smem(bar);
  if (*dead) return false;
  unsigned long long start = 0;
  for (unsigned spin = 0; spin < AT_SPIN_LIMIT; spin++) {
    unsigned ok;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(ok) : "r"(addr), "r"(parity) : "memory");
    if (ok) return true;
    if ((spin & 255) == 255) {              // also bounded in time: two seconds
      unsigned long long now;
      asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
      if (start == 0) start = now;
      else if (now - start > 2000000000ull) break;
    }
  }
  *dead = 1;
  return false;
}
// x = column in elements (0 or 64 here: a multiple of 128 bytes), y = row of the cache seen as [rows][d]
__device__ __forceinline__ void at_tma_2d(void* dst, const CUtensorMap* map, int x, int y, unsigned long long* bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
               ::"r"(at_smem(dst)), "l"(map), "r"(at_smem(bar)), "r"(x), "r"(y) : "memory");
}
// Shared-memory matrix descriptors, 128-byte swizzle, rows of 128 bytes, groups of 8 rows 1024 bytes apart.
// K-major (the contraction runs along a row): stride offset = 1024 (next 8 rows), leading offset unused.
__device__ __forceinline__ unsigned long long at_desc_kmajor(unsigned addr) {
  unsigned long long d = 0;
  d |= (unsigned long long)((addr & 0x3FFFF) >> 4);
  d |= (unsigned long long)1 << 16;
  d |= (unsigned long long)(1024 >> 4) << 32;
  d |= (unsigned long long)1 << 46;
  d |= (unsigned long long)2 << 61;
  return d;
}
// MN-major (a row holds 64 consecutive N elements of ONE contraction index; 8 contraction indices per group):
// stride offset = 1024 (next 8 contraction indices), leading offset = distance to the next 64 N elements.
__device__ __forceinline__ unsigned long long at_desc_mnmajor(unsigned addr, unsigned lbo_bytes) {
  unsigned long long d = 0;
  d |= (unsigned long long)((addr & 0x3FFFF) >> 4);
  d |= (unsigned long long)((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= (unsigned long long)(1024 >> 4) << 32;
  d |= (unsigned long long)1 << 46;
  d |= (unsigned long long)2 << 61;
  return d;
}
__device__ __forceinline__ void at_umma(unsigned tmem_d, unsigned long long desc_a, unsigned long long desc_b,
                                        unsigned idesc, unsigned accumulate) {
  asm volatile(
      "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
      " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n}\n"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}
__device__ __forceinline__ void at_commit(unsigned long long* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(at_smem(bar)) : "memory");
}
__device__ __forceinline__ void at_tmem_ld16(unsigned taddr, float (&v)[16]) {
  unsigned r[16];
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                 "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
               : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 16; i++) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void at_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void at_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void at_fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ float at_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ unsigned at_pack(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<unsigned*>(&v);
}
// Byte offset of the 16-byte piece `c` (of 64-column block c / 8) of row r in a [128 rows][HD] K-major tile
// stored as HD / 64 blocks of [128 rows][128 bytes] with the 128-byte swizzle.
__device__ __forceinline__ unsigned at_swz(int r, int c) {
  return (unsigned)((c >> 3) * (AT_ROWS * 128) + (r >> 3) * 1024 + (r & 7) * 128 + (((c & 7) ^ (r & 7)) << 4));
}

struct AtParams {
  const bf16* q; long long q_stride; bf16* out;
  const int* block_table; int max_blocks;
  const int* cu_tokens; const int* start_pos;
  int R, H, G, page_size, window, tok_tile;
  float scale_log2e;
  int* status;
};

template <int HD>
__global__ void __launch_bounds__(AT_THREADS, 1)
prefill_attention_tc5_kernel(const __grid_constant__ CUtensorMap kv_map, const AtParams p) {
  constexpr int NB = HD / 64;                       // 64-column blocks of a row
  constexpr int TILE_BYTES = AT_ROWS * HD * 2;      // one [128][HD] bfloat16 tile
  extern __shared__ __align__(16) unsigned char smem_raw[];
  unsigned char* base = smem_raw + ((1024 - (at_smem(smem_raw) & 1023)) & 1023);
  unsigned char* q_s = base;                        // Q tile, K-major
  unsigned char* p_s = q_s + TILE_BYTES;            // P tile [128 rows][128 keys], K-major
  unsigned char* k_s = p_s + AT_ROWS * AT_KEYS * 2; // 2 stages of K [128 keys][HD], K-major
  unsigned char* v_s = k_s + 2 * TILE_BYTES;        // 2 stages of V [128 keys][HD], MN-major for the product
  __shared__ unsigned long long k_full[2], v_full[2], k_empty[2], v_empty[2], s_full, p_full, o_full, o_free, q_full;
  __shared__ unsigned tmem_slot;
  __shared__ int dead;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    dead = 0;
    for (int s = 0; s < 2; s++) {
      at_mbar_init(&k_full[s], 1); at_mbar_init(&v_full[s], 1); at_mbar_init(&k_empty[s], 1); at_mbar_init(&v_empty[s], 1);
    }
    at_mbar_init(&s_full, 1); at_mbar_init(&o_full, 1);
    at_mbar_init(&p_full, AT_ROWS); at_mbar_init(&o_free, AT_ROWS); at_mbar_init(&q_full, AT_ROWS);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 5) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(at_smem(&tmem_slot)), "r"(256u)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  at_fence_before();
  __syncthreads();
  at_fence_after();
  const unsigned tmem = tmem_slot;                  // S: columns 0..127, O': columns 128..128+HD-1
  pdl_wait();

  // ---- which request and which tokens (tiles numbered request by request, the longest histories first)
  const int g = blockIdx.y;
  const int gs = p.H / p.G;
  int b = gridDim.x - 1 - blockIdx.x;
  int r = 0, before = 0;
  for (; r < p.R; r++) {
    int n = p.cu_tokens[r + 1] - p.cu_tokens[r];
    int nt = (n + p.tok_tile - 1) / p.tok_tile;
    if (b < before + nt) break;
    before += nt;
  }
  const bool idle = r == p.R;
  int tok0 = 0, n_tok = 0, pos0 = 0;
  if (!idle) {
    tok0 = p.cu_tokens[r] + (b - before) * p.tok_tile;
    n_tok = min(p.tok_tile, p.cu_tokens[r + 1] - tok0);
    pos0 = p.start_pos[r] + (tok0 - p.cu_tokens[r]);
  }
  const int key_hi = pos0 + n_tok;
  const int key_lo_tile = (p.window > 0 && pos0 - p.window + 1 > 0) ? pos0 - p.window + 1 : 0;
  const int kt_lo = key_lo_tile / AT_KEYS, kt_hi = idle ? kt_lo : (key_hi + AT_KEYS - 1) / AT_KEYS;
  const int n_kt = kt_hi - kt_lo;

  if (warp == 4) {
    // ------------------------------------------------------------------ producer
    if (!idle) {
      const int* bt = p.block_table + (size_t)r * p.max_blocks;
      for (int j = 0; j < n_kt; j++) {
        const int s = j & 1;
        const unsigned ph = (j >> 1) & 1;
        if (!at_mbar_wait(&k_empty[s], ph ^ 1, &dead) && lane == 0) atomicExch(p.status, 1);
        if (!at_mbar_wait(&v_empty[s], ph ^ 1, &dead) && lane == 0) atomicExch(p.status, 1);
        if (lane == 0) {
          at_mbar_expect_tx(&k_full[s], TILE_BYTES);
          at_mbar_expect_tx(&v_full[s], TILE_BYTES);
        }
        __syncwarp();
        if (lane < AT_KEYS / 16) {                    // one 16-key box row per lane
          const int key0 = (kt_lo + j) * AT_KEYS + lane * 16;
          int page = key0 < key_hi ? bt[key0 / p.page_size] : -1;
          if (page < 0) page = 0;                     // no such keys: any page will do, the scores are masked
          const int row_k = ((page * 2 + 0) * p.G + g) * p.page_size + key0 % p.page_size;
          const int row_v = ((page * 2 + 1) * p.G + g) * p.page_size + key0 % p.page_size;
#pragma unroll
          for (int cb = 0; cb < NB; cb++) {
            const unsigned off = (unsigned)(cb * (AT_KEYS * 128) + lane * 2048);     // 16 keys = two groups of 8 rows
            at_tma_2d(k_s + s * TILE_BYTES + off, &kv_map, cb * 64, row_k, &k_full[s]);
            at_tma_2d(v_s + s * TILE_BYTES + off, &kv_map, cb * 64, row_v, &v_full[s]);
          }
        }
      }
    }
  } else if (warp == 5) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0 && !idle) {
      const unsigned idesc_qk = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(AT_KEYS >> 3) << 17) | ((unsigned)(AT_ROWS >> 4) << 24);
      const unsigned idesc_pv = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((unsigned)(HD >> 3) << 17) |
                                ((unsigned)(AT_ROWS >> 4) << 24);
      const unsigned long long dq = at_desc_kmajor(at_smem(q_s));
      const unsigned long long dp = at_desc_kmajor(at_smem(p_s));
      auto issue_qk = [&](int j) {
        const int s = j & 1;
        if (!at_mbar_wait(&k_full[s], (j >> 1) & 1, &dead)) atomicExch(p.status, 2);
        at_fence_after();
        const unsigned long long dk = at_desc_kmajor(at_smem(k_s + s * TILE_BYTES));
#pragma unroll
        for (int k = 0; k < HD / 16; k++) {
          // 16 columns = 32 bytes inside a 64-column block; the next block is 128 rows x 128 bytes further
          const unsigned long long adv = (unsigned long long)(((k >> 2) * (AT_ROWS * 128) + (k & 3) * 32) >> 4);
          at_umma(tmem, dq + adv, dk + adv, idesc_qk, k ? 1u : 0u);
        }
        at_commit(&k_empty[s]);
        at_commit(&s_full);
      };
      if (!at_mbar_wait(&q_full, 0, &dead)) atomicExch(p.status, 3);
      if (n_kt > 0) issue_qk(0);
      for (int j = 0; j < n_kt; j++) {
        const int s = j & 1;
        if (!at_mbar_wait(&p_full, j & 1, &dead)) atomicExch(p.status, 4);
        if (!at_mbar_wait(&v_full[s], (j >> 1) & 1, &dead)) atomicExch(p.status, 5);
        if (j > 0 && !at_mbar_wait(&o_free, (j - 1) & 1, &dead)) atomicExch(p.status, 6);
        at_fence_after();
        const unsigned v_addr = at_smem(v_s + s * TILE_BYTES);
#pragma unroll
        for (int k = 0; k < AT_KEYS / 16; k++) {
          const unsigned long long adv_p = (unsigned long long)(((k >> 2) * (AT_ROWS * 128) + (k & 3) * 32) >> 4);
          // 16 keys = two groups of 8 rows of V; the d columns 64.. lie one [128 keys][128 bytes] block further
          const unsigned long long dv = at_desc_mnmajor(v_addr + k * 2048, AT_KEYS * 128);
          at_umma(tmem + 128, dp + adv_p, dv, idesc_pv, k ? 1u : 0u);
        }
        at_commit(&v_empty[s]);
        at_commit(&o_full);
        if (j + 1 < n_kt) issue_qk(j + 1);
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax: thread = row
    const int row = threadIdx.x;                                   // 0..127, also the TMEM lane
    const int t = row / gs, hh = row - t * gs;
    const bool ok = !idle && t < n_tok;
    const int pos = pos0 + t;
    const int lo = (p.window > 0 && pos - p.window + 1 > 0) ? pos - p.window + 1 : 0;
    // Q row into shared memory, in the layout the MMA reads
    {
      const bf16* qr = p.q + (size_t)(tok0 + t) * p.q_stride + (size_t)(g * gs + hh) * HD;
#pragma unroll
      for (int c = 0; c < HD / 8; c++) {
        uint4 v = make_uint4(0, 0, 0, 0);
        if (ok) v = *reinterpret_cast<const uint4*>(qr + c * 8);
        *reinterpret_cast<uint4*>(q_s + at_swz(row, c)) = v;
      }
      at_fence_async_smem();
      at_mbar_arrive(&q_full);
    }
    float o[HD];
#pragma unroll
    for (int i = 0; i < HD; i++) o[i] = 0.f;
    float m = -INFINITY, l = 0.f;
    const unsigned t_row = tmem + ((unsigned)(warp * 32) << 16);   // this warp's 32 lanes
    for (int j = 0; j < n_kt; j++) {
      const int key_base = (kt_lo + j) * AT_KEYS;
      if (!at_mbar_wait(&s_full, j & 1, &dead) && lane == 0) atomicExch(p.status, 7);
      at_fence_after();
      // pass 1: the row's maximum over this tile
      float mx = -INFINITY;
#pragma unroll 1
      for (int c = 0; c < AT_KEYS; c += 16) {
        float sv[16];
        at_tmem_ld16(t_row + c, sv);
#pragma unroll
        for (int i = 0; i < 16; i++) {
          const int key = key_base + c + i;
          const bool vis = ok && key <= pos && key >= lo;
          mx = fmaxf(mx, vis ? sv[i] * p.scale_log2e : -INFINITY);
        }
      }
      const float m_new = fmaxf(m, mx);
      const float ref = m_new == -INFINITY ? 0.f : m_new;
      const float alpha = at_exp2(m - ref);
      m = m_new;
      // pass 2: p = exp2(s - max), as bfloat16 into the P tile; the sum
      float sum = 0.f;
#pragma unroll 1
      for (int c = 0; c < AT_KEYS; c += 16) {
        float sv[16];
        at_tmem_ld16(t_row + c, sv);
        unsigned pk[8];
#pragma unroll
        for (int i = 0; i < 16; i += 2) {
          const int key = key_base + c + i;
          const bool v0 = ok && key <= pos && key >= lo, v1 = ok && key + 1 <= pos && key + 1 >= lo;
          const float p0 = v0 ? at_exp2(sv[i] * p.scale_log2e - ref) : 0.f;
          const float p1 = v1 ? at_exp2(sv[i + 1] * p.scale_log2e - ref) : 0.f;
          sum += p0 + p1;
          pk[i >> 1] = at_pack(p0, p1);
        }
        *reinterpret_cast<uint4*>(p_s + at_swz(row, c >> 3)) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
        *reinterpret_cast<uint4*>(p_s + at_swz(row, (c >> 3) + 1)) = make_uint4(pk[4], pk[5], pk[6], pk[7]);
      }
      l = l * alpha + sum;
      at_fence_before();
      at_fence_async_smem();
      at_mbar_arrive(&p_full);
      // the output of the tiles so far moves to the new maximum while the tensor cores multiply P and V
#pragma unroll
      for (int i = 0; i < HD; i++) o[i] *= alpha;
      if (!at_mbar_wait(&o_full, j & 1, &dead) && lane == 0) atomicExch(p.status, 8);
      at_fence_after();
#pragma unroll
      for (int c = 0; c < HD; c += 16) {
        float ov[16];
        at_tmem_ld16(t_row + 128 + c, ov);
#pragma unroll
        for (int i = 0; i < 16; i++) o[c + i] += ov[i];
      }
      at_fence_before();
      at_mbar_arrive(&o_free);
    }
    if (ok) {
      const float inv = 1.f / l;
      bf16* d = p.out + (size_t)(tok0 + t) * p.H * HD + (size_t)(g * gs + hh) * HD;
#pragma unroll
      for (int c = 0; c < HD; c += 8) {
        uint4 v;
        v.x = at_pack(o[c] * inv, o[c + 1] * inv);
        v.y = at_pack(o[c + 2] * inv, o[c + 3] * inv);
        v.z = at_pack(o[c + 4] * inv, o[c + 5] * inv);
        v.w = at_pack(o[c + 6] * inv, o[c + 7] * inv);
        *reinterpret_cast<uint4*>(d + c) = v;
      }
    }
  }
  pdl_launch_dependents();
  at_fence_before();
  __syncthreads();
  if (warp == 5) {
    at_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(256u) : "memory");
  }
}

// ------------------------------------------------------------------------------------ host
typedef CUresult (*AtEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                               const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                               CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static AtEncodeFn at_encode_fn() {
  static AtEncodeFn fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (AtEncodeFn)ptr;
  }
  return fn;
}

static int* at_status_word() {
  static int* words[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  if (!words[dev]) {
    int* w = nullptr;
    if (cudaMalloc(&w, sizeof(int)) != cudaSuccess) return nullptr;
    cudaMemset(w, 0, sizeof(int));
    words[dev] = w;
  }
  return words[dev];
}

template <int HD>
static int at_launch(const CUtensorMap& map, const AtParams& p, int tiles, cudaStream_t stream) {
  size_t smem = 1024 + (size_t)AT_ROWS * HD * 2 + (size_t)AT_ROWS * AT_KEYS * 2 + (size_t)4 * AT_ROWS * HD * 2;
  auto kernel = prefill_attention_tc5_kernel<HD>;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
    cudaGetLastError();
    return QD_ERR_UNSUPPORTED;
  }
  qd_launch(kernel, dim3((unsigned)tiles, (unsigned)p.G), dim3(AT_THREADS), smem, stream, map, p);
  return (int)cudaGetLastError();
}

// Arguments as qd_prefill_attention (attention_flash.cu) plus the number of pages of `kv`
// ([pages, 2, G, page_size, d], bfloat16).  Takes head sizes 64 and 128, groups of 1, 2, 4, 8 or 16 query
// heads per KV head, page sizes that are multiples of 16; refuses the rest (the caller has another kernel).
extern "C" int qd_prefill_attention_tc5(const void* q, long long q_stride, void* out, const void* kv, long long n_pages,
                                        const int* block_table, int max_blocks, const int* cu_tokens,
                                        const int* start_pos, int R, int T, int H, int G, int d, int page_size,
                                        float scale, int window, cudaStream_t stream) {
  if (T <= 0 || R <= 0) return 0;
  if (G < 1 || H % G != 0 || page_size % 16 != 0 || (d != 64 && d != 128) || n_pages < 1) return QD_ERR_UNSUPPORTED;
  const int gs = H / G;
  if (AT_ROWS % gs != 0 || gs > 16) return QD_ERR_UNSUPPORTED;
  if (((uintptr_t)q & 15) || ((uintptr_t)kv & 15) || ((uintptr_t)out & 15) || q_stride % 8 != 0) return QD_ERR_UNSUPPORTED;
  AtEncodeFn fn = at_encode_fn();
  int* status = at_status_word();
  if (!fn || !status) return QD_ERR_UNSUPPORTED;
  // the cache as rows of d: [pages * 2 * G * page_size][d]; a box is 16 rows x 64 columns
  CUtensorMap map;
  cuuint64_t dims[2] = {(cuuint64_t)d, (cuuint64_t)(n_pages * 2 * G * page_size)};
  cuuint64_t strides[1] = {(cuuint64_t)d * 2};
  cuuint32_t box[2] = {64, 16};
  cuuint32_t estr[2] = {1, 1};
  if (fn(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(kv), dims, strides, box, estr,
         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return QD_ERR_UNSUPPORTED;
  AtParams p;
  p.q = (const bf16*)q; p.q_stride = q_stride; p.out = (bf16*)out;
  p.block_table = block_table; p.max_blocks = max_blocks; p.cu_tokens = cu_tokens; p.start_pos = start_pos;
  p.R = R; p.H = H; p.G = G; p.page_size = page_size; p.window = window; p.tok_tile = AT_ROWS / gs;
  p.scale_log2e = scale * 1.4426950408889634f;
  p.status = status;
  const int tiles = (T + p.tok_tile - 1) / p.tok_tile + R;      // upper bound on the tiles of R requests
  return d == 64 ? at_launch<64>(map, p, tiles, stream) : at_launch<128>(map, p, tiles, stream);
}

// 0 if no kernel of this library has recorded a bounded-wait expiry on the current device.  Synchronises.
extern "C" int qd_prefill_attention_tc5_status() {
  int* status = at_status_word();
  if (!status) return -1;
  int v = 0;
  if (cudaMemcpy(&v, status, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
  if (v) cudaMemset(status, 0, sizeof(int));
  return v;
}
