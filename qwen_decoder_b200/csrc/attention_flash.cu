// Paged attention on tensor cores for the bfloat16 path: a prefill kernel (portions of any
// length, causal over the cached history plus the portion itself) and a decode kernel
// (one query token per request, keys split over CTAs and warps, partial results merged).
// Scores, softmax and the output accumulators are float32; Q K^T and P V are
// mma.sync m16n8k16 bf16 products.  K and V tiles are fetched page by page through the
// block table with cp.async; all query heads of a KV head's group share each tile, where
// the reference's kernels re-read K and V for every (head, token) pair
// (gpu_kernels.cu:197-312, 320-429) and run the dot products on CUDA cores.
//
// Rows of a tile are (token, head within the group) pairs, so a group of 8 heads fills a
// 64-row tile with 8 tokens: short portions still fill tiles and a decode token's group is
// one 16-row tile.  Head sizes 16..128 in steps of 16 (instantiated: 16, 32, 48, 64, 96,
// 128); page sizes that are multiples of 16; groups of up to 16 heads (decode) / 64 heads
// (prefill).  Anything else is refused and the caller takes the generic kernel.
#include "common.cuh"
#include "entry_points.h"
#include <cuda.h>
#include <math.h>
#include <stdint.h>
#include <stdlib.h>

#define FA_PAD 8  // bf16 elements of padding per smem row: 16 bytes, keeps ldmatrix conflict-free

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, int src_bytes) {
  unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(src_bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}
__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], const void* smem) {
  unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned (&r)[4], const void* smem) {
  unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<unsigned*>(&v);
}
__device__ __forceinline__ float quad_max(float v) {
  v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 1));
  return fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 2));
}
__device__ __forceinline__ float quad_sum(float v) {
  v += __shfl_xor_sync(0xffffffffu, v, 1);
  return v + __shfl_xor_sync(0xffffffffu, v, 2);
}

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// ===================================================================== decode
#define DEC_WARPS 4
#define DEC_STAGES 3
#define DEC_CHUNK 16  // keys per warp iteration; a chunk never straddles a page

// The end of a decode attention CTA, shared by the kernels below: the warps' partial results (o, running
// maxima m and denominators l of 16 rows each) are merged in shared memory; with one split the result is
// written, otherwise it goes to scratch and the CTA that finishes last for its (token, kv head) adds up all
// splits.  Every warp must be done with the stage buffers that start at smem_raw.
template <int HD>
__device__ __forceinline__ void dec_finish(float (&o)[HD / 8][4], float m0, float m1, float l0, float l1,
                                           unsigned char* smem_raw, int warp, int lane, int gs, int g, int t, int s,
                                           int H, int G, int splits, bf16* __restrict__ out,
                                           float* __restrict__ part_o, float* __restrict__ part_ml,
                                           unsigned* __restrict__ tickets) {
  l0 = quad_sum(l0);
  l1 = quad_sum(l1);
  __syncthreads();  // every warp is done with its stage buffers: reuse them for the merge

  // rows HD + 8 floats apart: the eight rows a store instruction touches fall on different banks (two by two)
  constexpr int OLD = HD + 8;
  float* mo = reinterpret_cast<float*>(smem_raw);             // [warps][16][HD + 8]
  float* mm = mo + DEC_WARPS * 16 * OLD;                      // [warps][16]
  float* ml = mm + DEC_WARPS * 16;                            // [warps][16]
  {
    const int r0 = lane >> 2, r1 = r0 + 8, cq = (lane & 3) * 2;
#pragma unroll
    for (int n = 0; n < HD / 8; n++) {
      *reinterpret_cast<float2*>(mo + ((size_t)warp * 16 + r0) * OLD + n * 8 + cq) = make_float2(o[n][0], o[n][1]);
      *reinterpret_cast<float2*>(mo + ((size_t)warp * 16 + r1) * OLD + n * 8 + cq) = make_float2(o[n][2], o[n][3]);
    }
    if ((lane & 3) == 0) {
      mm[warp * 16 + r0] = m0; mm[warp * 16 + r1] = m1;
      ml[warp * 16 + r0] = l0; ml[warp * 16 + r1] = l1;
    }
  }
  __syncthreads();
  // a thread takes four columns of a head: the warps' factors once, the sums as float4
  for (int idx = threadIdx.x; idx < gs * (HD / 4); idx += DEC_WARPS * 32) {
    const int row = idx / (HD / 4), dim = (idx - row * (HD / 4)) * 4;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < DEC_WARPS; w++) M = fmaxf(M, mm[w * 16 + row]);
    float L = 0.f;
    float4 O = make_float4(0.f, 0.f, 0.f, 0.f);
    if (M != -INFINITY) {
#pragma unroll
      for (int w = 0; w < DEC_WARPS; w++) {
        const float f = exp2f(mm[w * 16 + row] - M);
        L += ml[w * 16 + row] * f;
        const float4 v = *reinterpret_cast<const float4*>(mo + ((size_t)w * 16 + row) * OLD + dim);
        O.x += v.x * f; O.y += v.y * f; O.z += v.z * f; O.w += v.w * f;
      }
    }
    const int h = g * gs + row;
    if (splits == 1) {
      const float inv = 1.f / L;
      uint2 raw;
      raw.x = pack_bf16(O.x * inv, O.y * inv);
      raw.y = pack_bf16(O.z * inv, O.w * inv);
      *reinterpret_cast<uint2*>(out + (size_t)t * H * HD + (size_t)h * HD + dim) = raw;
    } else {
      const size_t pi = ((size_t)t * H + h) * splits + s;
      *reinterpret_cast<float4*>(part_o + pi * HD + dim) = O;
      if (dim == 0) { part_ml[pi * 2] = M; part_ml[pi * 2 + 1] = L; }
    }
  }
  if (splits == 1 || tickets == nullptr) return;   // without tickets a combine kernel follows
  // The CTA that finishes last for this (token, kv head) adds up all partial results.  The partial results are
  // written by all threads; they meet, then one thread takes the ticket with release and acquire at GPU scope:
  // the barrier before it puts the others' writes before the release, the barrier after it the others' reads
  // after the acquire.
  __shared__ unsigned s_ticket;
  __syncthreads();
  if (threadIdx.x == 0) {
    unsigned old;
    asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;" : "=r"(old) : "l"(tickets + (size_t)t * G + g) : "memory");
    s_ticket = old;
  }
  __syncthreads();
  if (s_ticket != (unsigned)splits - 1) return;
  // A thread takes four output columns of one head.  It asks for the maxima and sums of all splits of its head
  // and for its columns of the first 16 partial outputs in one go, makes the weights 2^(m_sp - M) itself (the
  // lanes of a warp that share a head read the same words: one access) and adds up: one trip through L2, no
  // exchange through shared memory, no barrier.
  constexpr int PB = 16;
  for (int idx = threadIdx.x; idx < gs * (HD / 4); idx += DEC_WARPS * 32) {
    const int row = idx / (HD / 4), d4 = idx - row * (HD / 4);
    const size_t base = ((size_t)t * H + (size_t)g * gs + row) * splits;
    const float2* ml_g = reinterpret_cast<const float2*>(part_ml) + base;
    float2 mlv[PB];
    float4 pv[PB];
#pragma unroll
    for (int u = 0; u < PB; u++) {
      mlv[u] = u < splits ? __ldcg(ml_g + u) : make_float2(-INFINITY, 0.f);
      pv[u] = u < splits ? __ldcg(reinterpret_cast<const float4*>(part_o + (base + u) * HD) + d4)
                         : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    float M = -INFINITY;
#pragma unroll
    for (int u = 0; u < PB; u++) M = fmaxf(M, mlv[u].x);
    for (int sp = PB; sp < splits; sp++) M = fmaxf(M, __ldcg(ml_g + sp).x);      // more than 16 splits
    float L = 0.f;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int u = 0; u < PB; u++) {
      const float f = u < splits ? exp2f(mlv[u].x - M) : 0.f;
      L += mlv[u].y * f;
      acc.x += pv[u].x * f; acc.y += pv[u].y * f; acc.z += pv[u].z * f; acc.w += pv[u].w * f;
    }
    for (int sp = PB; sp < splits; sp++) {
      const float2 v = __ldcg(ml_g + sp);
      const float4 o4 = __ldcg(reinterpret_cast<const float4*>(part_o + (base + sp) * HD) + d4);
      const float f = exp2f(v.x - M);
      L += v.y * f;
      acc.x += o4.x * f; acc.y += o4.y * f; acc.z += o4.z * f; acc.w += o4.w * f;
    }
    const float invL = 1.f / L;
    bf16* dst = out + (size_t)t * H * HD + ((size_t)g * gs + row) * HD + 4 * d4;
    uint2 raw;
    raw.x = pack_bf16(acc.x * invL, acc.y * invL);
    raw.y = pack_bf16(acc.z * invL, acc.w * invL);
    *reinterpret_cast<uint2*>(dst) = raw;
  }
  if (threadIdx.x == 0) tickets[(size_t)t * G + g] = 0;   // ready for the next launch
}

template <int HD>
__global__ void __launch_bounds__(DEC_WARPS * 32)
decode_attention_kernel(const bf16* __restrict__ q, long long q_stride, bf16* __restrict__ out,
                        const bf16* __restrict__ kv, const int* __restrict__ block_table, int max_blocks,
                        const int* __restrict__ token_req, const int* __restrict__ positions, int H, int G,
                        int page_size, float scale_log2e, int window, int splits,
                        float* __restrict__ part_o, float* __restrict__ part_ml,
                        unsigned* __restrict__ tickets) {
  // Before pdl_wait() only data that no kernel of this step writes is touched: positions and block
  // table (copied in before the step's first kernel) and cache chunks of *earlier* tokens.  The
  // query and the chunk that holds this step's own key are read after the wait.
  constexpr int LD = HD + FA_PAD;
  constexpr int TILE = DEC_CHUNK * LD;            // elements of one K or V chunk in smem
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* smem = reinterpret_cast<bf16*>(smem_raw);
  const int s = blockIdx.x, g = blockIdx.y, t = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int gs = H / G;
  const int pos = positions[t];
  const int n_keys = pos + 1;
  const int key_lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  const int chunk_lo = key_lo / DEC_CHUNK, chunk_hi = (n_keys + DEC_CHUNK - 1) / DEC_CHUNK;
  const int per = (chunk_hi - chunk_lo + splits - 1) / splits;
  const int c0 = chunk_lo + s * per;
  const int c1 = min(chunk_hi, c0 + per);
  const int* bt = block_table + (size_t)token_req[t] * max_blocks;
  const size_t page_elems = (size_t)2 * G * page_size * HD;
  const size_t k_off = (size_t)g * page_size * HD, v_off = ((size_t)G + g) * page_size * HD;

  bf16* wbuf = smem + (size_t)warp * DEC_STAGES * 2 * TILE;
  constexpr int CPR = HD / 8;                        // 16-byte pieces per row
  constexpr int ROWS_PER_IT = 32 / CPR > 0 ? 32 / CPR : 1;
  const int l_row = lane / CPR, l_col = (lane % CPR) * 8;
  // Page ids of this warp's chunks go through a ring of 64 entries in shared memory that is
  // filled 32 chunks ahead, so that no cache load waits for a block-table load.
  __shared__ int page_ring[DEC_WARPS][64];
  const int first = c0 + warp;
  const int n_my = first < c1 ? (c1 - first + DEC_WARPS - 1) / DEC_WARPS : 0;
  auto fill_ring = [&](int from) {      // entries [from, from + 32) of this warp's chunk sequence
    int i = from + lane;
    if (i < n_my) page_ring[warp][i & 63] = bt[((first + i * DEC_WARPS) * DEC_CHUNK) / page_size];
  };
  fill_ring(0);
  fill_ring(32);
  __syncwarp();
  auto load_chunk = [&](int i, int stage) {          // i-th chunk of this warp
    bf16* ks = wbuf + (size_t)stage * 2 * TILE;
    bf16* vs = ks + TILE;
    int key0 = (first + i * DEC_WARPS) * DEC_CHUNK;
    int page = page_ring[warp][i & 63];
    int in_page = key0 % page_size;
    const bf16* kg = kv + (page < 0 ? 0 : (size_t)page * page_elems) + k_off + (size_t)in_page * HD;
    const bf16* vg = kv + (page < 0 ? 0 : (size_t)page * page_elems) + v_off + (size_t)in_page * HD;
    const int rows_ok = page < 0 ? 0 : n_keys - key0;           // rows past the end are zero-filled
#pragma unroll
    for (int row = l_row; row < DEC_CHUNK; row += ROWS_PER_IT) {
      int bytes = row < rows_ok ? 16 : 0;
      cp_async16(ks + row * LD + l_col, kg + (bytes ? row * HD + l_col : 0), bytes);
      cp_async16(vs + row * LD + l_col, vg + (bytes ? row * HD + l_col : 0), bytes);
    }
  };

  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
  float o[HD / 8][4];
#pragma unroll
  for (int i = 0; i < HD / 8; i++) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;

  const int hot = chunk_hi - 1;        // the chunk this step's own key was just written to
  int deferred = -1;
#pragma unroll
  for (int p = 0; p < DEC_STAGES - 1; p++) {
    if (p < n_my) {
      if (first + p * DEC_WARPS == hot) deferred = p; else load_chunk(p, p);
    }
    cp_async_commit();
  }
  pdl_wait();
  if (deferred >= 0) { load_chunk(deferred, deferred); cp_async_commit(); }
  // Q fragments: rows are the heads of this KV head's group (rows >= gs are zero)
  unsigned qa[HD / 16][4];
  {
    const int r0 = lane >> 2, r1 = r0 + 8, cq = (lane & 3) * 2;
    const bf16* q0 = q + (size_t)t * q_stride + (size_t)(g * gs + r0) * HD + cq;
    const bf16* q1 = q + (size_t)t * q_stride + (size_t)(g * gs + r1) * HD + cq;
#pragma unroll
    for (int kk = 0; kk < HD / 16; kk++) {
      qa[kk][0] = r0 < gs ? *reinterpret_cast<const unsigned*>(q0 + kk * 16) : 0u;
      qa[kk][1] = r1 < gs ? *reinterpret_cast<const unsigned*>(q1 + kk * 16) : 0u;
      qa[kk][2] = r0 < gs ? *reinterpret_cast<const unsigned*>(q0 + kk * 16 + 8) : 0u;
      qa[kk][3] = r1 < gs ? *reinterpret_cast<const unsigned*>(q1 + kk * 16 + 8) : 0u;
    }
  }
  for (int i = 0; i < n_my; i++) {
    int nx = i + DEC_STAGES - 1;
    if ((i & 31) == 0 && i > 0) fill_ring(i + 32);     // entries [i, i+32) are in place; refill the other half
    if (nx < n_my) load_chunk(nx, nx % DEC_STAGES);
    cp_async_commit();
    if (i == n_my - 1) cp_async_wait<0>(); else cp_async_wait<DEC_STAGES - 1>();
    __syncwarp();
    const bf16* ks = wbuf + (size_t)(i % DEC_STAGES) * 2 * TILE;
    const bf16* vs = ks + TILE;
    const int c = first + i * DEC_WARPS;
    float sc[2][4];
#pragma unroll
    for (int n = 0; n < 2; n++) sc[n][0] = sc[n][1] = sc[n][2] = sc[n][3] = 0.f;
#pragma unroll
    for (int kk = 0; kk < HD / 16; kk++) {
      unsigned b[4];
      ldmatrix_x4(b, ks + ((lane & 7) + 8 * (lane >> 4)) * LD + kk * 16 + 8 * ((lane >> 3) & 1));
      mma_bf16(sc[0], qa[kk], b[0], b[1]);
      mma_bf16(sc[1], qa[kk], b[2], b[3]);
    }
#pragma unroll
    for (int n = 0; n < 2; n++)
#pragma unroll
      for (int j = 0; j < 4; j++) {
        int key = c * DEC_CHUNK + n * 8 + (lane & 3) * 2 + (j & 1);
        bool ok = key >= key_lo && key < n_keys;
        sc[n][j] = ok ? sc[n][j] * scale_log2e : -INFINITY;
      }
    float mx0 = quad_max(fmaxf(fmaxf(sc[0][0], sc[0][1]), fmaxf(sc[1][0], sc[1][1])));
    float mx1 = quad_max(fmaxf(fmaxf(sc[0][2], sc[0][3]), fmaxf(sc[1][2], sc[1][3])));
    float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
    float ref0 = mn0 == -INFINITY ? 0.f : mn0, ref1 = mn1 == -INFINITY ? 0.f : mn1;
    float a0 = fast_exp2(m0 - ref0), a1 = fast_exp2(m1 - ref1);
    m0 = mn0; m1 = mn1;
    float p[2][4];
#pragma unroll
    for (int n = 0; n < 2; n++) {
      p[n][0] = fast_exp2(sc[n][0] - ref0); p[n][1] = fast_exp2(sc[n][1] - ref0);
      p[n][2] = fast_exp2(sc[n][2] - ref1); p[n][3] = fast_exp2(sc[n][3] - ref1);
    }
    l0 = l0 * a0 + p[0][0] + p[0][1] + p[1][0] + p[1][1];
    l1 = l1 * a1 + p[0][2] + p[0][3] + p[1][2] + p[1][3];
    unsigned pa[4] = {pack_bf16(p[0][0], p[0][1]), pack_bf16(p[0][2], p[0][3]),
                      pack_bf16(p[1][0], p[1][1]), pack_bf16(p[1][2], p[1][3])};
    // the running maxima rarely move after the first chunks: rescale only when one did
    if (__any_sync(0xffffffffu, a0 != 1.f || a1 != 1.f)) {
#pragma unroll
      for (int n = 0; n < HD / 8; n++) { o[n][0] *= a0; o[n][1] *= a0; o[n][2] *= a1; o[n][3] *= a1; }
    }
#pragma unroll
    for (int dn = 0; dn < HD / 16; dn++) {
      unsigned b[4];
      ldmatrix_x4_trans(b, vs + ((lane & 7) + 8 * ((lane >> 3) & 1)) * LD + dn * 16 + 8 * (lane >> 4));
      mma_bf16(o[2 * dn], pa, b[0], b[1]);
      mma_bf16(o[2 * dn + 1], pa, b[2], b[3]);
    }
    __syncwarp();
  }
  cp_async_wait<0>();
  pdl_launch_dependents();
  dec_finish<HD>(o, m0, m1, l0, l1, smem_raw, warp, lane, gs, g, t, s, H, G, splits, out, part_o, part_ml, tickets);
}

// ------------------------------------------------------------------ the same with K/V through TMA
// Head sizes 64 and 128.  A chunk's K and V arrive as TMA tensor copies (boxes of 16 keys x 64 columns,
// 128-byte swizzle: the 16-byte unit u of row r lies at unit u ^ (r & 7)) onto an mbarrier per (warp, stage);
// one lane issues them, nobody computes addresses per row.  Waits are bounded: a wait that runs out sets the
// status word and the CTA runs on to its end.
#define DEC_SPIN_LIMIT (1u << 22)
__device__ __forceinline__ unsigned fa_smem(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ bool fa_mbar_wait(unsigned long long* bar, unsigned parity, volatile int* dead,
                                             unsigned poll_limit = DEC_SPIN_LIMIT) {
  return qd_mbar_wait_bounded(fa_smem(bar), parity, dead, poll_limit, 1000000000ull);
}

template <int HD>
__global__ void __launch_bounds__(DEC_WARPS * 32)
decode_attention_tma_kernel(const __grid_constant__ CUtensorMap kv_map, const bf16* __restrict__ q, long long q_stride,
                            bf16* __restrict__ out, const int* __restrict__ block_table, int max_blocks,
                            const int* __restrict__ token_req, const int* __restrict__ positions, int H, int G,
                            int page_size, float scale_log2e, int window, int splits,
                            float* __restrict__ part_o, float* __restrict__ part_ml,
                            unsigned* __restrict__ tickets, int* __restrict__ status) {
  static_assert(HD % 64 == 0, "boxes of 64 columns");
  constexpr int NB = HD / 64;                      // boxes per K or V chunk
  constexpr int BOX = 16 * 64;                     // elements of a box (2 KB)
  constexpr int STAGE = 2 * NB * BOX;              // elements of a stage: K boxes, then V boxes
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __shared__ unsigned long long bars[DEC_WARPS][DEC_STAGES];
  __shared__ int dead;
  __shared__ int page_ring[DEC_WARPS][64];
  // the swizzle pattern follows address bits 7-9: stages start on 1024-byte boundaries
  bf16* smem = reinterpret_cast<bf16*>(smem_raw + ((1024 - (fa_smem(smem_raw) & 1023)) & 1023));
  const int s = blockIdx.x, g = blockIdx.y, t = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int gs = H / G;
  if (threadIdx.x == 0) {
    dead = 0;
    for (int w = 0; w < DEC_WARPS; w++)
      for (int st = 0; st < DEC_STAGES; st++)
        asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(fa_smem(&bars[w][st])), "r"(1));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  const int pos = positions[t];
  const int n_keys = pos + 1;
  const int key_lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  const int chunk_lo = key_lo / DEC_CHUNK, chunk_hi = (n_keys + DEC_CHUNK - 1) / DEC_CHUNK;
  const int per = (chunk_hi - chunk_lo + splits - 1) / splits;
  const int c0 = chunk_lo + s * per;
  const int c1 = min(chunk_hi, c0 + per);
  const int* bt = block_table + (size_t)token_req[t] * max_blocks;
  bf16* wbuf = smem + (size_t)warp * DEC_STAGES * STAGE;
  const int first = c0 + warp;
  const int n_my = first < c1 ? (c1 - first + DEC_WARPS - 1) / DEC_WARPS : 0;
  auto fill_ring = [&](int from) {      // page ids of chunks [from, from + 32) of this warp's sequence
    int i = from + lane;
    if (i < n_my) page_ring[warp][i & 63] = bt[((first + i * DEC_WARPS) * DEC_CHUNK) / page_size];
  };
  fill_ring(0);
  fill_ring(32);
  __syncwarp();
  auto load_chunk = [&](int i, int stage) {          // i-th chunk of this warp; one lane asks for its four boxes
    if (lane != 0) return;
    unsigned long long* bar = &bars[warp][stage];
    const int key0 = (first + i * DEC_WARPS) * DEC_CHUNK;
    int page = page_ring[warp][i & 63];
    if (page < 0) page = 0;                          // no such keys: any page will do, the scores are masked
    const int in_page = key0 % page_size;
    const int row_k = ((page * 2 + 0) * G + g) * page_size + in_page;
    const int row_v = ((page * 2 + 1) * G + g) * page_size + in_page;
    bf16* ks = wbuf + (size_t)stage * STAGE;
    bf16* vs = ks + NB * BOX;
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(fa_smem(bar)),
                 "r"((unsigned)(STAGE * sizeof(bf16))) : "memory");
#pragma unroll
    for (int b = 0; b < NB; b++) {
      asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                   ::"r"(fa_smem(ks + b * BOX)), "l"(&kv_map), "r"(fa_smem(bar)), "r"(b * 64), "r"(row_k) : "memory");
      asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                   ::"r"(fa_smem(vs + b * BOX)), "l"(&kv_map), "r"(fa_smem(bar)), "r"(b * 64), "r"(row_v) : "memory");
    }
  };

  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
  float o[HD / 8][4];
#pragma unroll
  for (int i = 0; i < HD / 8; i++) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;

  // before the dependency wait only chunks of earlier steps' keys; the chunk that holds this step's own key after it
  const int hot = chunk_hi - 1;
  int deferred = -1;
#pragma unroll
  for (int p = 0; p < DEC_STAGES - 1; p++) {
    if (p < n_my) {
      if (first + p * DEC_WARPS == hot) deferred = p; else load_chunk(p, p);
    }
  }
  pdl_wait();
  if (deferred >= 0) load_chunk(deferred, deferred);
  unsigned qa[HD / 16][4];
  {
    const int r0 = lane >> 2, r1 = r0 + 8, cq = (lane & 3) * 2;
    const bf16* q0 = q + (size_t)t * q_stride + (size_t)(g * gs + r0) * HD + cq;
    const bf16* q1 = q + (size_t)t * q_stride + (size_t)(g * gs + r1) * HD + cq;
#pragma unroll
    for (int kk = 0; kk < HD / 16; kk++) {
      qa[kk][0] = r0 < gs ? *reinterpret_cast<const unsigned*>(q0 + kk * 16) : 0u;
      qa[kk][1] = r1 < gs ? *reinterpret_cast<const unsigned*>(q1 + kk * 16) : 0u;
      qa[kk][2] = r0 < gs ? *reinterpret_cast<const unsigned*>(q0 + kk * 16 + 8) : 0u;
      qa[kk][3] = r1 < gs ? *reinterpret_cast<const unsigned*>(q1 + kk * 16 + 8) : 0u;
    }
  }
  // element offset of the 16-byte unit `unit` (0 .. HD/8-1) of row r inside a K or V chunk
  auto sw = [](int r, int unit) { return (unit >> 3) * BOX + r * 64 + (((unit & 7) ^ (r & 7)) << 3); };
  for (int i = 0; i < n_my; i++) {
    const int nx = i + DEC_STAGES - 1;
    if ((i & 31) == 0 && i > 0) { fill_ring(i + 32); __syncwarp(); }
    if (nx < n_my) load_chunk(nx, nx % DEC_STAGES);      // its stage was read in iteration i - 1 (syncwarp below)
    const int stage = i % DEC_STAGES;
    if (!fa_mbar_wait(&bars[warp][stage], (i / DEC_STAGES) & 1, &dead) && lane == 0) atomicExch(status, 1);
    __syncwarp();
    bf16* ks = wbuf + (size_t)stage * STAGE;
    bf16* vs = ks + NB * BOX;
    const int c = first + i * DEC_WARPS;
    const int rows_ok = n_keys - c * DEC_CHUNK;
    if (rows_ok < DEC_CHUNK) {        // a request's last chunk: rows past its keys hold whatever the page held
      for (int idx = lane; idx < (DEC_CHUNK - rows_ok) * (HD / 8); idx += 32) {
        const int r = rows_ok + idx / (HD / 8), unit = idx % (HD / 8);
        *reinterpret_cast<uint4*>(vs + sw(r, unit)) = make_uint4(0u, 0u, 0u, 0u);
      }
      __syncwarp();
    }
    float sc[2][4];
#pragma unroll
    for (int n = 0; n < 2; n++) sc[n][0] = sc[n][1] = sc[n][2] = sc[n][3] = 0.f;
#pragma unroll
    for (int kk = 0; kk < HD / 16; kk++) {
      unsigned b[4];
      ldmatrix_x4(b, ks + sw((lane & 7) + 8 * (lane >> 4), kk * 2 + ((lane >> 3) & 1)));
      mma_bf16(sc[0], qa[kk], b[0], b[1]);
      mma_bf16(sc[1], qa[kk], b[2], b[3]);
    }
#pragma unroll
    for (int n = 0; n < 2; n++)
#pragma unroll
      for (int j = 0; j < 4; j++) {
        int key = c * DEC_CHUNK + n * 8 + (lane & 3) * 2 + (j & 1);
        bool ok = key >= key_lo && key < n_keys;
        sc[n][j] = ok ? sc[n][j] * scale_log2e : -INFINITY;
      }
    float mx0 = quad_max(fmaxf(fmaxf(sc[0][0], sc[0][1]), fmaxf(sc[1][0], sc[1][1])));
    float mx1 = quad_max(fmaxf(fmaxf(sc[0][2], sc[0][3]), fmaxf(sc[1][2], sc[1][3])));
    float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
    float ref0 = mn0 == -INFINITY ? 0.f : mn0, ref1 = mn1 == -INFINITY ? 0.f : mn1;
    float a0 = fast_exp2(m0 - ref0), a1 = fast_exp2(m1 - ref1);
    m0 = mn0; m1 = mn1;
    float p[2][4];
#pragma unroll
    for (int n = 0; n < 2; n++) {
      p[n][0] = fast_exp2(sc[n][0] - ref0); p[n][1] = fast_exp2(sc[n][1] - ref0);
      p[n][2] = fast_exp2(sc[n][2] - ref1); p[n][3] = fast_exp2(sc[n][3] - ref1);
    }
    l0 = l0 * a0 + p[0][0] + p[0][1] + p[1][0] + p[1][1];
    l1 = l1 * a1 + p[0][2] + p[0][3] + p[1][2] + p[1][3];
    unsigned pa[4] = {pack_bf16(p[0][0], p[0][1]), pack_bf16(p[0][2], p[0][3]),
                      pack_bf16(p[1][0], p[1][1]), pack_bf16(p[1][2], p[1][3])};
    if (__any_sync(0xffffffffu, a0 != 1.f || a1 != 1.f)) {
#pragma unroll
      for (int n = 0; n < HD / 8; n++) { o[n][0] *= a0; o[n][1] *= a0; o[n][2] *= a1; o[n][3] *= a1; }
    }
#pragma unroll
    for (int dn = 0; dn < HD / 16; dn++) {
      unsigned b[4];
      ldmatrix_x4_trans(b, vs + sw((lane & 7) + 8 * ((lane >> 3) & 1), dn * 2 + (lane >> 4)));
      mma_bf16(o[2 * dn], pa, b[0], b[1]);
      mma_bf16(o[2 * dn + 1], pa, b[2], b[3]);
    }
    __syncwarp();
  }
  pdl_launch_dependents();
  dec_finish<HD>(o, m0, m1, l0, l1, smem_raw, warp, lane, gs, g, t, s, H, G, splits, out, part_o, part_ml, tickets);
}

// out[t, h, :] = sum_s O_s * 2^(m_s - M) / sum_s l_s * 2^(m_s - M)
__global__ void decode_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                      bf16* __restrict__ out, int HD, int splits) {
  pdl_launch_dependents();
  pdl_wait();
  size_t th = blockIdx.x;
  float M = -INFINITY;
  for (int s = 0; s < splits; s++) M = fmaxf(M, part_ml[(th * splits + s) * 2]);
  float L = 0.f;
  for (int s = 0; s < splits; s++) L += part_ml[(th * splits + s) * 2 + 1] * exp2f(part_ml[(th * splits + s) * 2] - M);
  for (int dim = threadIdx.x; dim < HD; dim += blockDim.x) {
    float O = 0.f;
    for (int s = 0; s < splits; s++)
      O += part_o[(th * splits + s) * HD + dim] * exp2f(part_ml[(th * splits + s) * 2] - M);
    out[th * HD + dim] = __float2bfloat16_rn(O / L);
  }
}

template <int HD>
static int launch_decode(const bf16* q, long long q_stride, bf16* out, const bf16* kv, const int* block_table,
                         int max_blocks, const int* token_req, const int* positions, int T, int H, int G,
                         int page_size, float scale, int window, int splits, float* part_o, float* part_ml,
                         unsigned* tickets, cudaStream_t stream) {
  constexpr int LD = HD + FA_PAD;
  size_t smem = (size_t)DEC_WARPS * DEC_STAGES * 2 * DEC_CHUNK * LD * sizeof(bf16);
  size_t merge = (size_t)DEC_WARPS * 16 * (HD + 8 + 2) * sizeof(float);         // the warps' outputs, maxima and sums
  if (merge > smem) smem = merge;
  if (smem > 48 * 1024)
    cudaFuncSetAttribute(decode_attention_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  dim3 grid(splits, G, T);
  qd_launch(decode_attention_kernel<HD>, dim3(grid), dim3(DEC_WARPS * 32), smem, stream, 
      q, q_stride, out, kv, block_table, max_blocks, token_req, positions, H, G, page_size,
      scale * 1.4426950408889634f, window, splits, part_o, part_ml, tickets);
  int e = qd_last_error();
  if (e) return e;
  if (splits > 1 && !tickets) {
    qd_launch(decode_combine_kernel, dim3((unsigned)((size_t)T * H)), dim3(HD < 32 ? 32 : (HD > 128 ? 128 : HD)), 0, stream, 
        part_o, part_ml, out, HD, splits);
    e = qd_last_error();
  }
  return e;
}

// One query token per entry of positions/token_req.  part_o must hold T*H*splits*HD floats and
// part_ml T*H*splits*2 floats when splits > 1 (scratch; contents need not be initialised).
// tickets: T*G unsigned counters that are ZERO on entry (the kernel leaves them zero again); with
// them the last CTA of each (token, kv head) adds up the partial results itself; with a null
// pointer a second small kernel does it.
extern "C" int qd_decode_attention(const void* q, long long q_stride, void* out, const void* kv,
                                   const int* block_table, int max_blocks, const int* token_req,
                                   const int* positions, int T, int H, int G, int d, int page_size,
                                   float scale, int window, int splits, float* part_o, float* part_ml,
                                   unsigned* tickets, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (G <= 0 || H % G != 0 || H / G > 16 || page_size % DEC_CHUNK != 0 || splits < 1 || T > 65535 || G > 65535)
    return QD_ERR_UNSUPPORTED;
  if (splits > 1 && (!part_o || !part_ml)) return QD_ERR_UNSUPPORTED;
  if (splits > 64 && tickets) return QD_ERR_UNSUPPORTED;
#define CASE(HD)                                                                                          \
  case HD:                                                                                                \
    return launch_decode<HD>((const bf16*)q, q_stride, (bf16*)out, (const bf16*)kv, block_table, max_blocks, \
                             token_req, positions, T, H, G, page_size, scale, window, splits, part_o,     \
                             part_ml, tickets, stream);
  switch (d) {
    CASE(16) CASE(32) CASE(48) CASE(64) CASE(96) CASE(128)
    default: return QD_ERR_UNSUPPORTED;
  }
#undef CASE
}

// ---- host side of the TMA variant
typedef CUresult (*FaEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                               const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                               CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static FaEncodeFn fa_encode_fn() {
  static FaEncodeFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (FaEncodeFn)p;
  }
  return fn;
}
static int* fa_status_word() {
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
static int launch_decode_tma(const CUtensorMap& map, const bf16* q, long long q_stride, bf16* out, const int* block_table,
                             int max_blocks, const int* token_req, const int* positions, int T, int H, int G,
                             int page_size, float scale, int window, int splits, float* part_o, float* part_ml,
                             unsigned* tickets, int* status, cudaStream_t stream) {
  size_t smem = (size_t)DEC_WARPS * DEC_STAGES * 2 * DEC_CHUNK * HD * sizeof(bf16) + 1024;
  if (cudaFuncSetAttribute(decode_attention_tma_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
      cudaSuccess) {
    cudaGetLastError();
    return QD_ERR_UNSUPPORTED;
  }
  dim3 grid(splits, G, T);
  qd_launch(decode_attention_tma_kernel<HD>, dim3(grid), dim3(DEC_WARPS * 32), smem, stream, map, q, q_stride, out,
            block_table, max_blocks, token_req, positions, H, G, page_size, scale * 1.4426950408889634f, window, splits,
            part_o, part_ml, tickets, status);
  return qd_last_error();
}

// As qd_decode_attention with K/V fetched by TMA tensor copies: head size 64 or 128, tickets required when
// splits > 1, the cache 16-byte aligned; ``n_pages`` = pages of ``kv``.  Anything else is refused.
extern "C" int qd_decode_attention_tma(const void* q, long long q_stride, void* out, const void* kv, long long n_pages,
                                       const int* block_table, int max_blocks, const int* token_req,
                                       const int* positions, int T, int H, int G, int d, int page_size, float scale,
                                       int window, int splits, float* part_o, float* part_ml, unsigned* tickets,
                                       cudaStream_t stream) {
  if (T <= 0) return 0;
  if (G <= 0 || H % G != 0 || H / G > 16 || page_size % DEC_CHUNK != 0 || splits < 1 || splits > 64 || T > 65535 ||
      G > 65535 || (d != 64 && d != 128) || n_pages < 1)
    return QD_ERR_UNSUPPORTED;
  if (splits > 1 && (!part_o || !part_ml || !tickets)) return QD_ERR_UNSUPPORTED;
  if (((uintptr_t)kv & 15) || q_stride % 2 != 0) return QD_ERR_UNSUPPORTED;
  FaEncodeFn fn = fa_encode_fn();
  int* status = fa_status_word();
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
  if (d == 64)
    return launch_decode_tma<64>(map, (const bf16*)q, q_stride, (bf16*)out, block_table, max_blocks, token_req, positions,
                                 T, H, G, page_size, scale, window, splits, part_o, part_ml, tickets, status, stream);
  return launch_decode_tma<128>(map, (const bf16*)q, q_stride, (bf16*)out, block_table, max_blocks, token_req, positions,
                                T, H, G, page_size, scale, window, splits, part_o, part_ml, tickets, status, stream);
}

// 0 if no bounded wait of the TMA decode kernel has run out on the current device (reported once).  Synchronises.
QD_DEFINE_WAIT_PROBE(qd_decode_attention_tma_wait_probe, fa_mbar_wait(bar, 0, dead, poll_limit), fa_status_word, 99)

extern "C" int qd_decode_attention_tma_status() {
  int* status = fa_status_word();
  if (!status) return -1;
  int v = 0;
  if (cudaMemcpy(&v, status, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
  if (v) cudaMemset(status, 0, sizeof(int));
  return v;
}

// ==================================================================== prefill
#define PF_KEYS 64  // keys per tile

// NW warps of 16 rows each; NST cp.async stages of one K tile + one V tile.
template <int HD, int NW, int NST>
__global__ void __launch_bounds__(NW * 32)
prefill_attention_kernel(const bf16* __restrict__ q, long long q_stride, bf16* __restrict__ out,
                         const bf16* __restrict__ kv, const int* __restrict__ block_table, int max_blocks,
                         const int* __restrict__ cu_tokens, const int* __restrict__ start_pos, int R, int H,
                         int G, int page_size, float scale_log2e, int window, int tok_tile) {
  pdl_wait();
  constexpr int LD = HD + FA_PAD;
  constexpr int TILE = PF_KEYS * LD;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* smem = reinterpret_cast<bf16*>(smem_raw);    // [NST stages][K tile, V tile]
  const int g = blockIdx.y;
  const int gs = H / G;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // which request and which tokens: tiles are numbered request by request; the last tiles
  // (longest histories within a request) are taken first
  int b = gridDim.x - 1 - blockIdx.x;
  int r = 0, before = 0;
  for (; r < R; r++) {
    int n = cu_tokens[r + 1] - cu_tokens[r];
    int nt = (n + tok_tile - 1) / tok_tile;
    if (b < before + nt) break;
    before += nt;
  }
  if (r == R) return;
  const int tok0 = cu_tokens[r] + (b - before) * tok_tile;
  const int n_tok = min(tok_tile, cu_tokens[r + 1] - tok0);
  const int pos0 = start_pos[r] + (tok0 - cu_tokens[r]);
  const int key_hi = pos0 + n_tok;                                  // keys [.., key_hi) may be read
  const int key_lo_tile = (window > 0 && pos0 - window + 1 > 0) ? pos0 - window + 1 : 0;
  const int* bt = block_table + (size_t)r * max_blocks;
  const size_t page_elems = (size_t)2 * G * page_size * HD;
  const size_t k_off = (size_t)g * page_size * HD, v_off = ((size_t)G + g) * page_size * HD;

  // this thread's two rows
  const int row0 = warp * 16 + (lane >> 2), row1 = row0 + 8;
  const int t0 = row0 / gs, h0 = row0 - t0 * gs, t1 = row1 / gs, h1 = row1 - t1 * gs;
  const bool ok0 = t0 < n_tok, ok1 = t1 < n_tok;
  const int p0 = pos0 + t0, p1 = pos0 + t1;                          // positions of the rows
  const int lo0 = (window > 0 && p0 - window + 1 > 0) ? p0 - window + 1 : 0;
  const int lo1 = (window > 0 && p1 - window + 1 > 0) ? p1 - window + 1 : 0;
  // keys in [full_lo, full_hi) are visible to every valid row of the tile: no masking there
  const int full_hi = pos0 + 1;
  const int full_lo = (window > 0 && key_hi - 1 - window + 1 > 0) ? key_hi - window : 0;

  unsigned qa[HD / 16][4];
  {
    const int cq = (lane & 3) * 2;
    const bf16* q0 = q + (size_t)(tok0 + t0) * q_stride + (size_t)(g * gs + h0) * HD + cq;
    const bf16* q1 = q + (size_t)(tok0 + t1) * q_stride + (size_t)(g * gs + h1) * HD + cq;
#pragma unroll
    for (int kk = 0; kk < HD / 16; kk++) {
      qa[kk][0] = ok0 ? *reinterpret_cast<const unsigned*>(q0 + kk * 16) : 0u;
      qa[kk][1] = ok1 ? *reinterpret_cast<const unsigned*>(q1 + kk * 16) : 0u;
      qa[kk][2] = ok0 ? *reinterpret_cast<const unsigned*>(q0 + kk * 16 + 8) : 0u;
      qa[kk][3] = ok1 ? *reinterpret_cast<const unsigned*>(q1 + kk * 16 + 8) : 0u;
    }
  }

  // Each thread copies PIECES 16-byte pieces of K and of V per tile; the page ids of a tile's
  // rows are fetched one tile ahead, so that no cache load waits for a block-table load.
  constexpr int CPR = HD / 8;
  constexpr int PIECES = (PF_KEYS * CPR + NW * 32 - 1) / (NW * 32);
  int pg_next[PIECES];
  auto fetch_pages = [&](int kt) {
#pragma unroll
    for (int j = 0; j < PIECES; j++) {
      int i = threadIdx.x + j * NW * 32;
      int key = kt * PF_KEYS + i / CPR;
      pg_next[j] = (i < PF_KEYS * CPR && key < key_hi) ? bt[key / page_size] : -1;
    }
  };
  auto load_tile = [&](int kt, int stage) {          // uses pg_next fetched for this kt
    bf16* ks = smem + (size_t)stage * 2 * TILE;
    bf16* vs = ks + TILE;
    const int key_base = kt * PF_KEYS;
#pragma unroll
    for (int j = 0; j < PIECES; j++) {
      int i = threadIdx.x + j * NW * 32;
      if (i < PF_KEYS * CPR) {
        int row = i / CPR, col = (i % CPR) * 8;
        int key = key_base + row;
        int page = pg_next[j];
        int bytes = page >= 0 ? 16 : 0;
        size_t base = page >= 0 ? (size_t)page * page_elems + (size_t)(key % page_size) * HD + col : 0;
        cp_async16(ks + row * LD + col, kv + base + (page >= 0 ? k_off : 0), bytes);
        cp_async16(vs + row * LD + col, kv + base + (page >= 0 ? v_off : 0), bytes);
      }
    }
  };

  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
  float o[HD / 8][4];
#pragma unroll
  for (int i = 0; i < HD / 8; i++) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;

  const int kt_lo = key_lo_tile / PF_KEYS, kt_hi = (key_hi + PF_KEYS - 1) / PF_KEYS;
#pragma unroll
  for (int p = 0; p < NST - 1; p++) {
    if (kt_lo + p < kt_hi) { fetch_pages(kt_lo + p); load_tile(kt_lo + p, p); }
    cp_async_commit();
  }
  if (kt_lo + NST - 1 < kt_hi) fetch_pages(kt_lo + NST - 1);
  for (int kt = kt_lo; kt < kt_hi; kt++) {
    const int it = kt - kt_lo;
    const int stage = it % NST;
    if (kt + NST - 1 < kt_hi) load_tile(kt + NST - 1, (it + NST - 1) % NST);
    cp_async_commit();
    if (kt + NST < kt_hi) fetch_pages(kt + NST);      // for the load of the next iteration
    cp_async_wait<NST - 1>();
    __syncthreads();
    const bf16* ks = smem + (size_t)stage * 2 * TILE;
    const bf16* vs = ks + TILE;
    float sc[PF_KEYS / 8][4];
#pragma unroll
    for (int n = 0; n < PF_KEYS / 8; n++) sc[n][0] = sc[n][1] = sc[n][2] = sc[n][3] = 0.f;
    // K fragments of the next 16 dims are fetched while the MMAs of the current 16 run
    {
      const bf16* kfrag = ks + ((lane & 7) + 8 * (lane >> 4)) * LD + 8 * ((lane >> 3) & 1);
      unsigned bq[2][PF_KEYS / 16][4];
#pragma unroll
      for (int kb = 0; kb < PF_KEYS / 16; kb++) ldmatrix_x4(bq[0][kb], kfrag + kb * 16 * LD);
#pragma unroll
      for (int kk = 0; kk < HD / 16; kk++) {
        if (kk + 1 < HD / 16) {
#pragma unroll
          for (int kb = 0; kb < PF_KEYS / 16; kb++)
            ldmatrix_x4(bq[(kk + 1) & 1][kb], kfrag + kb * 16 * LD + (kk + 1) * 16);
        }
#pragma unroll
        for (int kb = 0; kb < PF_KEYS / 16; kb++) {
          mma_bf16(sc[2 * kb], qa[kk], bq[kk & 1][kb][0], bq[kk & 1][kb][1]);
          mma_bf16(sc[2 * kb + 1], qa[kk], bq[kk & 1][kb][2], bq[kk & 1][kb][3]);
        }
      }
    }
    const int key_base = kt * PF_KEYS + (lane & 3) * 2;
    float mx0 = -INFINITY, mx1 = -INFINITY;
    const bool interior = kt * PF_KEYS >= full_lo && kt * PF_KEYS + PF_KEYS <= full_hi;
    if (interior) {
#pragma unroll
      for (int n = 0; n < PF_KEYS / 8; n++) {
#pragma unroll
        for (int j = 0; j < 2; j++) {
          sc[n][j] = ok0 ? sc[n][j] * scale_log2e : -INFINITY;
          sc[n][2 + j] = ok1 ? sc[n][2 + j] * scale_log2e : -INFINITY;
          mx0 = fmaxf(mx0, sc[n][j]);
          mx1 = fmaxf(mx1, sc[n][2 + j]);
        }
      }
    } else {
#pragma unroll
      for (int n = 0; n < PF_KEYS / 8; n++) {
#pragma unroll
        for (int j = 0; j < 2; j++) {
          int key = key_base + n * 8 + j;
          bool a = ok0 && key <= p0 && key >= lo0;
          bool c = ok1 && key <= p1 && key >= lo1;
          sc[n][j] = a ? sc[n][j] * scale_log2e : -INFINITY;
          sc[n][2 + j] = c ? sc[n][2 + j] * scale_log2e : -INFINITY;
          mx0 = fmaxf(mx0, sc[n][j]);
          mx1 = fmaxf(mx1, sc[n][2 + j]);
        }
      }
    }
    mx0 = quad_max(mx0);
    mx1 = quad_max(mx1);
    float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
    float ref0 = mn0 == -INFINITY ? 0.f : mn0, ref1 = mn1 == -INFINITY ? 0.f : mn1;
    float a0 = fast_exp2(m0 - ref0), a1 = fast_exp2(m1 - ref1);
    m0 = mn0; m1 = mn1;
    float s0 = 0.f, s1 = 0.f;
#pragma unroll
    for (int n = 0; n < PF_KEYS / 8; n++) {
      sc[n][0] = fast_exp2(sc[n][0] - ref0); sc[n][1] = fast_exp2(sc[n][1] - ref0);
      sc[n][2] = fast_exp2(sc[n][2] - ref1); sc[n][3] = fast_exp2(sc[n][3] - ref1);
      s0 += sc[n][0] + sc[n][1];
      s1 += sc[n][2] + sc[n][3];
    }
    l0 = l0 * a0 + s0;
    l1 = l1 * a1 + s1;
#pragma unroll
    for (int n = 0; n < HD / 8; n++) { o[n][0] *= a0; o[n][1] *= a0; o[n][2] *= a1; o[n][3] *= a1; }
    {
      // V fragments: four 16-dim groups are fetched ahead of the MMAs that use them
      const bf16* vfrag = vs + ((lane & 7) + 8 * ((lane >> 3) & 1)) * LD + 8 * (lane >> 4);
      constexpr int DG = HD / 16;               // 16-dim groups
      constexpr int STEPS = (PF_KEYS / 16) * DG;
      constexpr int AHEAD = DG < 4 ? DG : 4;
      unsigned bv[AHEAD][4];
#pragma unroll
      for (int st = 0; st < AHEAD; st++)
        ldmatrix_x4_trans(bv[st], vfrag + (st / DG) * 16 * LD + (st % DG) * 16);
#pragma unroll
      for (int st = 0; st < STEPS; st++) {
        const int kb = st / DG, dn = st % DG;
        unsigned pa[4] = {pack_bf16(sc[2 * kb][0], sc[2 * kb][1]), pack_bf16(sc[2 * kb][2], sc[2 * kb][3]),
                          pack_bf16(sc[2 * kb + 1][0], sc[2 * kb + 1][1]),
                          pack_bf16(sc[2 * kb + 1][2], sc[2 * kb + 1][3])};
        unsigned b0 = bv[st % AHEAD][0], b1 = bv[st % AHEAD][1], b2 = bv[st % AHEAD][2], b3 = bv[st % AHEAD][3];
        if (st + AHEAD < STEPS) {
          const int nx = st + AHEAD;
          ldmatrix_x4_trans(bv[st % AHEAD], vfrag + (nx / DG) * 16 * LD + (nx % DG) * 16);
        }
        mma_bf16(o[2 * dn], pa, b0, b1);
        mma_bf16(o[2 * dn + 1], pa, b2, b3);
      }
    }
    __syncthreads();  // all warps are done with this stage before a later load overwrites it
  }
  cp_async_wait<0>();
  pdl_launch_dependents();
  l0 = quad_sum(l0);
  l1 = quad_sum(l1);
  const int cq = (lane & 3) * 2;
  if (ok0) {
    float inv = 1.f / l0;
    bf16* d = out + (size_t)(tok0 + t0) * H * HD + (size_t)(g * gs + h0) * HD + cq;
#pragma unroll
    for (int n = 0; n < HD / 8; n++)
      *reinterpret_cast<unsigned*>(d + n * 8) = pack_bf16(o[n][0] * inv, o[n][1] * inv);
  }
  if (ok1) {
    float inv = 1.f / l1;
    bf16* d = out + (size_t)(tok0 + t1) * H * HD + (size_t)(g * gs + h1) * HD + cq;
#pragma unroll
    for (int n = 0; n < HD / 8; n++)
      *reinterpret_cast<unsigned*>(d + n * 8) = pack_bf16(o[n][2] * inv, o[n][3] * inv);
  }
}

template <int HD, int NW, int NST>
static int launch_prefill_v(const bf16* q, long long q_stride, bf16* out, const bf16* kv, const int* block_table,
                            int max_blocks, const int* cu_tokens, const int* start_pos, int R, int T, int H, int G,
                            int page_size, float scale, int window, cudaStream_t stream) {
  constexpr int LD = HD + FA_PAD;
  size_t smem = (size_t)NST * 2 * PF_KEYS * LD * sizeof(bf16);
  if (smem > 48 * 1024)
    cudaFuncSetAttribute(prefill_attention_kernel<HD, NW, NST>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  int gs = H / G;
  int tok_tile = (NW * 16) / gs;
  int tiles = (T + tok_tile - 1) / tok_tile + R;   // upper bound on the tiles of R requests
  dim3 grid(tiles, G);
  qd_launch(prefill_attention_kernel<HD, NW, NST>, dim3(grid), dim3(NW * 32), smem, stream,
      q, q_stride, out, kv, block_table, max_blocks, cu_tokens, start_pos, R, H, G, page_size,
      scale * 1.4426950408889634f, window, tok_tile);
  return qd_last_error();
}

template <int HD>
static int launch_prefill(const bf16* q, long long q_stride, bf16* out, const bf16* kv, const int* block_table,
                          int max_blocks, const int* cu_tokens, const int* start_pos, int R, int T, int H, int G,
                          int page_size, float scale, int window, cudaStream_t stream) {
#define PFV(NW, NST) launch_prefill_v<HD, NW, NST>(q, q_stride, out, kv, block_table, max_blocks, cu_tokens, \
                                                   start_pos, R, T, H, G, page_size, scale, window, stream)
  int gs = H / G;
  // eight warps (128 rows) halve the K/V traffic per row, but only pay with enough tokens per request
  bool big = T / R >= 128 && gs <= 128;
  return big && gs <= 64 ? PFV(8, 2) : PFV(4, 2);       // three stages measured no better with either
#undef PFV
}

// Portions of R requests: tokens cu_tokens[r]..cu_tokens[r+1]-1 of the flat batch sit at positions
// start_pos[r].. of request r (block-table row r).  Their K/V are already in the pages.
extern "C" int qd_prefill_attention(const void* q, long long q_stride, void* out, const void* kv,
                                    const int* block_table, int max_blocks, const int* cu_tokens,
                                    const int* start_pos, int R, int T, int H, int G, int d, int page_size,
                                    float scale, int window, cudaStream_t stream) {
  if (T <= 0 || R <= 0) return 0;
  if (G <= 0 || H % G != 0 || H / G > 64 || page_size <= 0 || G > 65535) return QD_ERR_UNSUPPORTED;
#define CASE(HD)                                                                                           \
  case HD:                                                                                                 \
    return launch_prefill<HD>((const bf16*)q, q_stride, (bf16*)out, (const bf16*)kv, block_table, max_blocks, \
                              cu_tokens, start_pos, R, T, H, G, page_size, scale, window, stream);
  switch (d) {
    CASE(16) CASE(32) CASE(48) CASE(64) CASE(96) CASE(128)
    default: return QD_ERR_UNSUPPORTED;
  }
#undef CASE
}
