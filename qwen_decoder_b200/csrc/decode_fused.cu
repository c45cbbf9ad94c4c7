// A whole decode step of up to 16 tokens in ONE cooperative kernel: all layers, the final norm
// and the output projection.  The unfused path runs about nine kernels per layer; here the CTAs
// stay resident (cudaLaunchCooperativeKernel, two per SM) and meet at a grid barrier between phases:
//
//   per layer   P1  x -> RMSNorm -> q, k, v sums        (float32)
//               P2  bias + rotary + cache write + paged attention over the block table
//               P3  attention output -> o projection    (added into the residual x)
//               P4  x -> RMSNorm -> gate/up -> SwiGLU   (h written as bfloat16)
//               P5  h -> down projection                (added into the residual x)
//   at the end  P6  x -> final RMSNorm -> output projection -> float32 logits
//
// The kernel body is an interpreter over phases, so that each phase's code exists once.
// Contractions stream the weights with 16-byte non-allocating loads into registers and run
// mma.sync m16n8k16 with the tokens as the N dimension (the scheme of gemm_skinny.cu).  A CTA
// takes units of 16 weight rows x 1024 k (its 8 warps take 128 k each and add up in shared
// memory) and keeps one k range for a whole phase; one phase ahead it asks for its first weights to
// be brought into L2, so that a barrier's latency hides under the fetch.  Where several CTAs share
// one tile's k range they leave partial sums in scratch and the last to arrive (a ticket per tile)
// adds them in a fixed order, so results do not depend on timing.  Attention is the split-KV scheme
// of attention_flash.cu with 8 warps per (token, kv head, split).
//
// It computes what the unfused kernels compute (same formulas: gpu_decoder.cu:311-540 of the
// reference, with the fusions named above).  Every spin (grid barrier) is bounded in polls and in
// time; when a wait runs out the kernel records it in `status`, goes on without waiting and ends.
//
// Measured on a B200 (8 tokens, context 2048, 3B layer sizes): 105 us per layer against 61 us of
// the unfused path with programmatic dependent launch.  A grid barrier with the skew between CTAs
// costs 4-7 us, five times per layer -- no less than the kernel boundaries it replaces -- and every
// CTA normalises the whole residual for itself (7 us, twice per layer).  So this path is off by
// default (QD_FUSED_DECODE=1 turns it on); `timeline` shows where a step's time goes.
#include "common.cuh"
#include <cooperative_groups.h>
#include <math.h>

#define FD_WARPS 8
#define FD_THREADS (FD_WARPS * 32)
#define FD_U 4                       // k-steps of 32 per warp and unit: 128 k per warp, 1024 per CTA
#define FD_KCTA (FD_WARPS * FD_U * 32)
#define FD_PAD 8
#define FD_XPAD 32                   // row padding of the staged activations: rows 64 bytes apart mod 128
#define FD_SPIN_LIMIT (1u << 26)

struct FdLayer {
  const float* norm1_w; float eps1;
  const bf16* wqkv; const float* bqkv;     // [(H + 2G) d, D], bias or null
  const bf16* wo;                          // [D, H d]
  const float* norm2_w; float eps2;
  const bf16* wgu;                         // [2F, D]: gate rows then up rows
  const bf16* wd;                          // [D, F]
  bf16* kv;                                // this layer's cache: [pages, 2, G, page_size, d]
};

struct FdParams {
  int T, D, H, G, d, F, V, L;
  float* x;                  // [T, D] residual, float32 (holds the embeddings on entry)
  float* qkv;                // [T, (H + 2G) d] float32: q, k, v before bias and rotation
  bf16* attn_out;            // [T, H d]
  bf16* h;                   // [T, F]
  float* part_o; float* part_ml; unsigned* tickets;   // attention partial results; tickets zero on entry and exit
  float* scratch; unsigned* gemm_tickets;             // partial sums of shared k ranges; tickets zero on entry and exit
  int scratch_floats, n_gemm_tickets;
  const int* positions; const int* token_req; const int* block_table; const int* slot_map;
  int max_blocks, page_size, splits, window;
  const float* cos_t; const float* sin_t; int rotary_dim, pairing; float scale_log2e;
  const FdLayer* layers;
  const float* final_w; float final_eps; const bf16* lm_head; float* logits;   // [T, V]
  unsigned* barrier;         // two words, zero on first use: arrivals, generation
  int* status;               // device word: set when a wait ran out
  int* host_status;          // the same in pinned host memory, written only then (the host reads it without a sync)
  long long* timeline;       // null, or [(L + 1) * 16] nanosecond stamps of CTA 0: per phase its start, the end of
                             // its preparation and the end of its work (before the barrier)
};

// ------------------------------------------------------------------------------ small helpers
__device__ __forceinline__ uint4 fd_ldg_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ void fd_mma(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                       unsigned b0, unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void fd_cp_async16(void* smem, const void* gmem, int src_bytes) {
  unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(src_bytes));
}
__device__ __forceinline__ void fd_ldmatrix_x4(unsigned (&r)[4], const void* smem) {
  unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void fd_ldmatrix_x4_trans(unsigned (&r)[4], const void* smem) {
  unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ unsigned fd_pack(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<unsigned*>(&v);
}
__device__ __forceinline__ float fd_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Row length of the staged activations: the widest of x, the attention output and one k range of h.
__host__ __device__ inline int fd_ldxs(int D, int Hd, int F) {
  int w = D > Hd ? D : Hd;
  int kf = F < FD_KCTA ? F : FD_KCTA;
  return (w > kf ? w : kf) + FD_XPAD;
}

// Grid barrier: every CTA arrives, the last one opens the next generation.  Bounded: after
// FD_SPIN_LIMIT polls or two seconds a CTA records the failure and goes on.
__device__ __noinline__ void fd_grid_sync(unsigned* bar, int* status, int* host_status) {
  __syncthreads();
  if (threadIdx.x == 0 && *reinterpret_cast<volatile int*>(status) == 0) {   // after a failure nobody waits again
    volatile unsigned* gen_p = bar + 1;
    unsigned gen = *gen_p;
    __threadfence();
    unsigned arrived = atomicAdd(bar, 1u);
    if (arrived == gridDim.x - 1) {
      bar[0] = 0;
      __threadfence();
      atomicAdd(bar + 1, 1u);
    } else {
      unsigned long long start = 0;
      bool ok = false;
      for (unsigned spin = 0; spin < FD_SPIN_LIMIT; spin++) {
        if (*gen_p != gen) { ok = true; break; }
        if ((spin & 1023) == 1023) {
          unsigned long long now;
          asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
          if (start == 0) start = now;
          else if (now - start > 2000000000ull) break;
        }
      }
      if (!ok) {
        atomicExch(status, 1);
        *reinterpret_cast<volatile int*>(host_status) = 1;
        __threadfence_system();
      }
    }
    __threadfence();
  }
  __syncthreads();
}

__device__ __forceinline__ void fd_stamp(const FdParams& p, int slot) {
  if (p.timeline && blockIdx.x == 0 && threadIdx.x == 0) {
    long long now;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
    p.timeline[slot] = now;
  }
}

// xs[t, :] = bfloat16(rmsnorm(x[t, :]) * w) for t < T, zero rows up to TP (one warp per row).  Every CTA
// does this for itself; a row of up to 2048 values is read once, with all of a lane's loads in flight
// together, and kept in registers for the second pass.
__device__ __forceinline__ void fd_norm_to_smem(const float* __restrict__ x, const float* __restrict__ w, float eps, bf16* xs,
                                                int ldxs, int T, int TP, int D) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int D4 = D >> 2;
  const float4* wr = reinterpret_cast<const float4*>(w);
  for (int t = warp; t < TP; t += FD_WARPS) {
    uint2* row = reinterpret_cast<uint2*>(xs + (size_t)t * ldxs);
    if (t >= T) {
      for (int i = lane; i < D4; i += 32) row[i] = make_uint2(0, 0);
      continue;
    }
    const float4* xr = reinterpret_cast<const float4*>(x + (size_t)t * D);
    float ss = 0.f;
    if (D4 <= 32 * 16) {
      float4 v[16];
#pragma unroll
      for (int u = 0; u < 16; u++) {
        int i = lane + 32 * u;
        v[u] = i < D4 ? __ldcg(xr + i) : make_float4(0.f, 0.f, 0.f, 0.f);
      }
#pragma unroll
      for (int u = 0; u < 16; u++) ss += v[u].x * v[u].x + v[u].y * v[u].y + v[u].z * v[u].z + v[u].w * v[u].w;
      ss = warp_sum(ss);
      const float inv = 1.0f / sqrtf(ss / (float)D + eps);
#pragma unroll
      for (int h = 0; h < 2; h++) {          // the scales in two batches of 8 loads, each batch in flight together
        float4 g[8];
#pragma unroll
        for (int u = 0; u < 8; u++) {
          int i = lane + 32 * (8 * h + u);
          g[u] = i < D4 ? __ldg(wr + i) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int u = 0; u < 8; u++) {
          int i = lane + 32 * (8 * h + u);
          const float4 a = v[8 * h + u];
          if (i < D4)
            row[i] = make_uint2(fd_pack(a.x * inv * g[u].x, a.y * inv * g[u].y),
                                fd_pack(a.z * inv * g[u].z, a.w * inv * g[u].w));
        }
      }
      continue;
    }
    for (int i0 = lane; i0 < D4; i0 += 32 * 4) {
      float4 v[4];
#pragma unroll
      for (int u = 0; u < 4; u++) {
        int i = i0 + 32 * u;
        v[u] = i < D4 ? __ldcg(xr + i) : make_float4(0.f, 0.f, 0.f, 0.f);
      }
#pragma unroll
      for (int u = 0; u < 4; u++) ss += v[u].x * v[u].x + v[u].y * v[u].y + v[u].z * v[u].z + v[u].w * v[u].w;
    }
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)D + eps);
    for (int i0 = lane; i0 < D4; i0 += 32 * 4) {
      float4 v[4], g[4];
#pragma unroll
      for (int u = 0; u < 4; u++) {
        int i = i0 + 32 * u;
        if (i < D4) { v[u] = __ldcg(xr + i); g[u] = __ldg(wr + i); }
      }
#pragma unroll
      for (int u = 0; u < 4; u++) {
        int i = i0 + 32 * u;
        if (i < D4)
          row[i] = make_uint2(fd_pack(v[u].x * inv * g[u].x, v[u].y * inv * g[u].y),
                              fd_pack(v[u].z * inv * g[u].z, v[u].w * inv * g[u].w));
      }
    }
  }
}

// ------------------------------------------------------------------------------ contraction
// What a CTA does in a contraction phase: units = (16 rows of W) x (k range of FD_KCTA).  A CTA keeps one k
// range for the whole phase (CTA b: range b % n_kc) and walks the tiles first, first + stride, ...; CTAs
// beyond n_kc * stride have nothing to do.  `lo`/`hi` hold this warp's share of the unit's weights.
struct FdGemm {
  const bf16* W; int n_rows; int K;        // W [n_rows (or 2F for SwiGLU), K]
  int swiglu_F;                            // > 0: rows f and F + f pair up (8 + 8 rows per unit)
  int n_tiles, n_kc, n_units;
  int kc, first, stride;                   // this CTA's k range, first tile and step over tiles
};

__device__ __forceinline__ FdGemm fd_gemm_desc(const bf16* W, int n_rows, int K, int swiglu_F, bool full_k) {
  FdGemm g;
  g.W = W; g.n_rows = n_rows; g.K = K; g.swiglu_F = swiglu_F;
  g.n_tiles = swiglu_F > 0 ? (swiglu_F + 7) / 8 : (n_rows + 15) / 16;
  g.n_kc = full_k ? 1 : (K + FD_KCTA - 1) / FD_KCTA;
  g.n_units = g.n_tiles * g.n_kc;
  g.stride = (int)gridDim.x / g.n_kc;
  g.kc = (int)blockIdx.x % g.n_kc;
  g.first = (int)blockIdx.x / g.n_kc;
  if (g.stride < 1 || g.first >= g.stride) { g.first = g.n_tiles; g.stride = 1; }      // idle
  return g;
}

// Where this lane reads in unit u: pointers to its 16 bytes of rows r and r + 8 at the warp's first k, and
// how many k are left from there (its s-th load of a group is inside while (group * FD_U + s) * 32 < left).
struct FdLane { const bf16* lo; const bf16* hi; int k0; int left; int tile; };

__device__ __forceinline__ FdLane fd_lane(const FdGemm& g, int tile) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, j = lane & 3, r = lane >> 2;
  FdLane L;
  L.tile = tile;
  const int kc = g.kc;
  int kw0, kw1;                                  // the warp's k range
  if (g.n_kc == 1) {                             // the whole K, split evenly over the warps in multiples of 32
    int per = (((g.K + 31) >> 5) + FD_WARPS - 1) / FD_WARPS * 32;
    kw0 = warp * per; kw1 = min(g.K, kw0 + per);
  } else {
    kw0 = kc * FD_KCTA + warp * FD_U * 32; kw1 = min(g.K, kw0 + FD_U * 32);
  }
  L.k0 = kw0 + 8 * j;
  L.left = kw1 - L.k0;
  long long row_lo, row_hi;
  if (g.swiglu_F > 0) {
    int f = min(L.tile * 8 + r, g.swiglu_F - 1);
    row_lo = f; row_hi = (long long)g.swiglu_F + f;
  } else {
    row_lo = min(L.tile * 16 + r, g.n_rows - 1);
    row_hi = min(L.tile * 16 + r + 8, g.n_rows - 1);
  }
  L.lo = g.W + row_lo * g.K + L.k0;
  L.hi = g.W + row_hi * g.K + L.k0;
  return L;
}

__device__ __forceinline__ void fd_load_group(const FdLane& L, int group, uint4 (&lo)[FD_U], uint4 (&hi)[FD_U]) {
#pragma unroll
  for (int s = 0; s < FD_U; s++) {
    const int off = (group * FD_U + s) * 32;
    if (off < L.left) {
      lo[s] = fd_ldg_stream(L.lo + off);
      hi[s] = fd_ldg_stream(L.hi + off);
    } else {
      lo[s] = make_uint4(0, 0, 0, 0);
      hi[s] = make_uint4(0, 0, 0, 0);
    }
  }
}

#define FD_EPI_STORE 0     // out[t * ld + n] = sum             (float32)
#define FD_EPI_ADD 1       // out[t * ld + n] += sum            (float32; one CTA per tile does it)
#define FD_EPI_SWIGLU 2    // out[t * ld + f] = silu(gate) * up (bfloat16)

struct FdOut {
  float* f; bf16* b; int ld;
  float* scratch; unsigned* tickets;       // for k ranges shared by several CTAs
};

__device__ __forceinline__ void fd_epilogue(const FdGemm& g, const FdOut& out, int EPI, int tile, int idx, float v, int T) {
  const int row = idx & 15, tok = idx >> 4;
  const int n = tile * 16 + row;
  if (tok >= T || n >= g.n_rows) return;
  float* dst = out.f + (size_t)tok * out.ld + n;
  if (EPI == FD_EPI_ADD) *dst = __ldcg(dst) + v;
  else *dst = v;
}

// Ask for ALL the weights this CTA will read in a phase to be brought into L2 (fire and forget, no
// registers held).  Called one phase ahead, so that the memory system streams the next weights while
// the present phase computes, waits at its barrier, or -- attention -- reads little.
__device__ __forceinline__ void fd_prefetch_phase(const FdGemm& g) {
  if (g.n_units == 0) return;
  const int k_lo = g.n_kc == 1 ? 0 : g.kc * FD_KCTA;
  const int k_hi = g.n_kc == 1 ? g.K : min(g.K, k_lo + FD_KCTA);
  const int lines = ((k_hi - k_lo) * 2 + 127) / 128;                 // 128-byte lines per row
  int left = 2;                         // two units ahead: more did not pay (measured), and the output projection has far more
  for (int tile = g.first; tile < g.n_tiles && left > 0; tile += g.stride, left--) {
    for (int i = threadIdx.x; i < 16 * lines; i += FD_THREADS) {
      int r = i / lines, c = i - r * lines;
      long long row;
      if (g.swiglu_F > 0) row = (r & 8 ? (long long)g.swiglu_F : 0) + min(tile * 8 + (r & 7), g.swiglu_F - 1);
      else row = min(tile * 16 + r, g.n_rows - 1);
      const bf16* src = g.W + row * g.K + k_lo + c * 64;
      asm volatile("prefetch.global.L2 [%0];\n" ::"l"(src));
    }
  }
}

// Run this CTA's units of a phase.  B operand: bfloat16 rows [TP][ldb] in shared memory, holding the
// activations' columns from k_base on.
template <int TN>
__device__ __forceinline__ void fd_gemm_run(const FdGemm& g, const int EPI, const bf16* xs, int ldb, int k_base,
                                            const FdOut& out, int T, float* red) {
  uint4 lo[FD_U], hi[FD_U];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, j = lane & 3, r = lane >> 2;
  constexpr int TP = TN * 8;
  constexpr int RED_LD = TP + 1;
  __shared__ unsigned s_last;
  if (g.first >= g.n_tiles) return;
  FdLane L = fd_lane(g, g.first);
  fd_load_group(L, 0, lo, hi);
  const int n_groups = L.left > 0 ? (L.left + FD_U * 32 - 1) / (FD_U * 32) : 0;   // the same for the lanes of a warp
  const bf16* bs = xs + (size_t)r * ldb + (L.k0 - k_base);
  for (int tile = g.first; tile < g.n_tiles; tile += g.stride) {
    // lo/hi hold group 0 of this unit; the next group, or group 0 of this CTA's next unit, is
    // requested before the tensor cores take the present one
    const bool more_units = tile + g.stride < g.n_tiles;
    FdLane Ln = L;
    if (more_units) Ln = fd_lane(g, tile + g.stride);
    float acc[TN][4];
#pragma unroll
    for (int n = 0; n < TN; n++) acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.f;
    const int n_iter = n_groups > 0 ? n_groups : 1;      // a warp without k in this range still fetches for the next
    for (int grp = 0; grp < n_iter; grp++) {
      uint4 nlo[FD_U], nhi[FD_U];
      if (grp + 1 < n_groups) fd_load_group(L, grp + 1, nlo, nhi);
      else if (more_units) fd_load_group(Ln, 0, nlo, nhi);
#pragma unroll
      for (int s = 0; s < FD_U; s++) {
        const int off = (grp * FD_U + s) * 32;
        const bool in = off < L.left;
#pragma unroll
        for (int n = 0; n < TN; n++) {
          uint4 b = make_uint4(0, 0, 0, 0);
          if (in) b = *reinterpret_cast<const uint4*>(bs + (size_t)n * 8 * ldb + off);
          fd_mma(acc[n], lo[s].x, hi[s].x, lo[s].y, hi[s].y, b.x, b.y);
          fd_mma(acc[n], lo[s].z, hi[s].z, lo[s].w, hi[s].w, b.z, b.w);
        }
      }
      if (grp + 1 < n_groups || more_units) {
#pragma unroll
        for (int s = 0; s < FD_U; s++) { lo[s] = nlo[s]; hi[s] = nhi[s]; }
      }
    }
    L = Ln;
    // add the warps' shares of k
    float* mine = red + (size_t)warp * 16 * RED_LD;
#pragma unroll
    for (int n = 0; n < TN; n++) {
      mine[r * RED_LD + n * 8 + 2 * j] = acc[n][0];
      mine[r * RED_LD + n * 8 + 2 * j + 1] = acc[n][1];
      mine[(r + 8) * RED_LD + n * 8 + 2 * j] = acc[n][2];
      mine[(r + 8) * RED_LD + n * 8 + 2 * j + 1] = acc[n][3];
    }
    __syncthreads();
    if (EPI == FD_EPI_SWIGLU) {
      for (int idx = threadIdx.x; idx < 8 * TP; idx += FD_THREADS) {
        int row = idx & 7, tok = idx >> 3;
        int f = tile * 8 + row;
        if (tok >= T || f >= g.swiglu_F) continue;
        float gate = 0.f, up = 0.f;
#pragma unroll
        for (int w = 0; w < FD_WARPS; w++) {
          gate += red[((size_t)w * 16 + row) * RED_LD + tok];
          up += red[((size_t)w * 16 + row + 8) * RED_LD + tok];
        }
        out.b[(size_t)tok * out.ld + f] = __float2bfloat16_rn(gate / (1.0f + expf(-gate)) * up);
      }
    } else {
      for (int idx = threadIdx.x; idx < 16 * TP; idx += FD_THREADS) {
        int row = idx & 15, tok = idx >> 4;
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < FD_WARPS; w++) v += red[((size_t)w * 16 + row) * RED_LD + tok];
        if (g.n_kc == 1) fd_epilogue(g, out, EPI, tile, idx, v, T);
        else __stcg(out.scratch + ((size_t)tile * g.n_kc + g.kc) * (16 * TP) + idx, v);
      }
      if (g.n_kc > 1) {
        // the last CTA of this tile to arrive adds the partial sums, always in the order of k
        __syncthreads();
        if (threadIdx.x == 0) {
          __threadfence();
          s_last = atomicAdd(&out.tickets[tile], 1u) == (unsigned)g.n_kc - 1;
          __threadfence();
        }
        __syncthreads();
        if (s_last) {
          for (int idx = threadIdx.x; idx < 16 * TP; idx += FD_THREADS) {
            float v = 0.f;
            for (int c = 0; c < g.n_kc; c++) v += __ldcg(out.scratch + ((size_t)tile * g.n_kc + c) * (16 * TP) + idx);
            fd_epilogue(g, out, EPI, tile, idx, v, T);
          }
          if (threadIdx.x == 0) out.tickets[tile] = 0;
        }
      }
    }
    __syncthreads();
  }
}

// ------------------------------------------------------------------------------ attention phase
// Work item = (token t, kv head g, split s); item i goes to CTA i % gridDim.x.  The item builds q (and,
// if it owns the chunk of the token's own position, k and v) from the q/k/v sums: bias, rotation, cache
// write; then its 8 warps walk 16-key chunks; partial results go to scratch and the last item of a
// (t, g) to finish combines them into attn_out.
template <int HD>
__device__ __forceinline__ void fd_attention(const FdParams& p, const FdLayer& L, unsigned char* smem_raw) {
  constexpr int LD = HD + FD_PAD;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int H = p.H, G = p.G, gs = H / G, Nqkv = (H + 2 * G) * HD;
  bf16* qs = reinterpret_cast<bf16*>(smem_raw);                       // [16][LD] rotated q of the group
  bf16* kvs = qs + 16 * LD;                                           // per warp: K chunk, V chunk [16][LD] each
  float* mm = reinterpret_cast<float*>(kvs + (size_t)FD_WARPS * 2 * 16 * LD);   // merge: [warps][16]
  float* ml = mm + FD_WARPS * 16;                                     // [warps][16]
  float* fac = ml + FD_WARPS * 16;                                    // combine: [16][64] x 3
  __shared__ unsigned s_ticket;
  const int n_items = p.T * G * p.splits;
  const size_t page_elems = (size_t)2 * G * p.page_size * HD;
  const int half = p.rotary_dim >> 1;

  for (int item = blockIdx.x; item < n_items; item += gridDim.x) {
    const int s = item % p.splits, g = (item / p.splits) % G, t = item / (p.splits * G);
    const int pos = p.positions[t];
    const int n_keys = pos + 1;
    const int key_lo = (p.window > 0 && pos - p.window + 1 > 0) ? pos - p.window + 1 : 0;
    const int chunk_lo = key_lo / 16, chunk_hi = (n_keys + 15) / 16;
    const int per = (chunk_hi - chunk_lo + p.splits - 1) / p.splits;
    const int c0 = chunk_lo + s * per, c1 = min(chunk_hi, c0 + per);
    const int* bt = p.block_table + (size_t)p.token_req[t] * p.max_blocks;
    const float* acc = p.qkv + (size_t)t * Nqkv;
    const size_t k_off = (size_t)g * p.page_size * HD, v_off = ((size_t)G + g) * p.page_size * HD;

    // ---- q of the group (gs heads), rotated, as bfloat16 rows in shared memory (rows >= gs zero)
    for (int w = threadIdx.x; w < 16 * (HD / 2); w += FD_THREADS) {
      int row = w / (HD / 2), pp = w - row * (HD / 2);
      int i0, i1;
      bool rot = pp < half;
      if (p.pairing == 0) { i0 = 2 * pp; i1 = 2 * pp + 1; }
      else if (rot) { i0 = pp; i1 = pp + half; }
      else { int jj = 2 * (pp - half) + p.rotary_dim; i0 = jj; i1 = jj + 1; }
      float a = 0.f, b = 0.f;
      if (row < gs) {
        int e = (g * gs + row) * HD;
        a = __ldcg(acc + e + i0) + (L.bqkv ? L.bqkv[e + i0] : 0.f);
        b = __ldcg(acc + e + i1) + (L.bqkv ? L.bqkv[e + i1] : 0.f);
        if (rot && p.cos_t) {
          float cv = p.cos_t[(size_t)pos * half + pp], sv = p.sin_t[(size_t)pos * half + pp];
          float ra = a * cv - b * sv, rb = a * sv + b * cv;
          a = ra; b = rb;
        }
      }
      qs[row * LD + i0] = __float2bfloat16_rn(a);
      qs[row * LD + i1] = __float2bfloat16_rn(b);
    }
    // ---- the token's own k and v: written to the cache by the item that owns their chunk
    const bool owns_new = (chunk_hi - 1 >= c0 && chunk_hi - 1 < c1);
    if (owns_new) {
      const int slot = p.slot_map[t];
      const int page = slot / p.page_size, off = slot - page * p.page_size;
      bf16* kdst = L.kv + (size_t)page * page_elems + k_off + (size_t)off * HD;
      bf16* vdst = L.kv + (size_t)page * page_elems + v_off + (size_t)off * HD;
      for (int w = threadIdx.x; w < HD; w += FD_THREADS) {           // HD/2 pairs of k, then HD/2 pairs of v
        bool is_v = w >= HD / 2;
        int pp = is_v ? w - HD / 2 : w;
        int i0, i1;
        bool rot = pp < half && !is_v;
        if (is_v || p.pairing == 0) { i0 = 2 * pp; i1 = 2 * pp + 1; }
        else if (pp < half) { i0 = pp; i1 = pp + half; }
        else { int jj = 2 * (pp - half) + p.rotary_dim; i0 = jj; i1 = jj + 1; }
        int e = ((is_v ? H + G : H) + g) * HD;
        float a = __ldcg(acc + e + i0) + (L.bqkv ? L.bqkv[e + i0] : 0.f);
        float b = __ldcg(acc + e + i1) + (L.bqkv ? L.bqkv[e + i1] : 0.f);
        if (rot && p.cos_t) {
          float cv = p.cos_t[(size_t)pos * half + pp], sv = p.sin_t[(size_t)pos * half + pp];
          float ra = a * cv - b * sv, rb = a * sv + b * cv;
          a = ra; b = rb;
        }
        bf16* dst = is_v ? vdst : kdst;
        dst[i0] = __float2bfloat16_rn(a);
        dst[i1] = __float2bfloat16_rn(b);
      }
      __threadfence();       // the chunk loads below read these through L2
    }
    __syncthreads();

    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
    float o[HD / 8][4];
#pragma unroll
    for (int i = 0; i < HD / 8; i++) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    bf16* ks = kvs + (size_t)warp * 2 * 16 * LD;
    bf16* vs = ks + 16 * LD;
    constexpr int CPR = HD / 8;
    constexpr int ROWS_PER_IT = 32 / CPR > 0 ? 32 / CPR : 1;
    const int l_row = lane / CPR, l_col = (lane % CPR) * 8;
    for (int c = c0 + warp; c < c1; c += FD_WARPS) {
      const int key0 = c * 16;
      const int page = bt[key0 / p.page_size];
      const int in_page = key0 % p.page_size;
      const bf16* kg = L.kv + (page < 0 ? 0 : (size_t)page * page_elems) + k_off + (size_t)in_page * HD;
      const bf16* vg = L.kv + (page < 0 ? 0 : (size_t)page * page_elems) + v_off + (size_t)in_page * HD;
      const int rows_ok = page < 0 ? 0 : n_keys - key0;
      for (int row = l_row; row < 16; row += ROWS_PER_IT) {
        int bytes = row < rows_ok ? 16 : 0;
        fd_cp_async16(ks + row * LD + l_col, kg + (bytes ? row * HD + l_col : 0), bytes);
        fd_cp_async16(vs + row * LD + l_col, vg + (bytes ? row * HD + l_col : 0), bytes);
      }
      asm volatile("cp.async.commit_group;\n" ::);
      asm volatile("cp.async.wait_group 0;\n" ::);
      __syncwarp();
      float sc[2][4];
#pragma unroll
      for (int n = 0; n < 2; n++) sc[n][0] = sc[n][1] = sc[n][2] = sc[n][3] = 0.f;
#pragma unroll
      for (int kk = 0; kk < HD / 16; kk++) {
        unsigned qa[4], b[4];
        // q fragment: matrices (rows 0-7 | 8-15) x (k 0-7 | 8-15) in the order a0..a3 of the mma
        fd_ldmatrix_x4(qa, qs + ((lane & 7) + 8 * ((lane >> 3) & 1)) * LD + kk * 16 + 8 * (lane >> 4));
        fd_ldmatrix_x4(b, ks + ((lane & 7) + 8 * (lane >> 4)) * LD + kk * 16 + 8 * ((lane >> 3) & 1));
        fd_mma(sc[0], qa[0], qa[1], qa[2], qa[3], b[0], b[1]);
        fd_mma(sc[1], qa[0], qa[1], qa[2], qa[3], b[2], b[3]);
      }
#pragma unroll
      for (int n = 0; n < 2; n++)
#pragma unroll
        for (int jx = 0; jx < 4; jx++) {
          int key = key0 + n * 8 + (lane & 3) * 2 + (jx & 1);
          bool ok = key >= key_lo && key < n_keys;
          sc[n][jx] = ok ? sc[n][jx] * p.scale_log2e : -INFINITY;
        }
      float mx0 = fmaxf(fmaxf(sc[0][0], sc[0][1]), fmaxf(sc[1][0], sc[1][1]));
      float mx1 = fmaxf(fmaxf(sc[0][2], sc[0][3]), fmaxf(sc[1][2], sc[1][3]));
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
      float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
      float ref0 = mn0 == -INFINITY ? 0.f : mn0, ref1 = mn1 == -INFINITY ? 0.f : mn1;
      float a0 = fd_exp2(m0 - ref0), a1 = fd_exp2(m1 - ref1);
      m0 = mn0; m1 = mn1;
      float pr[2][4];
#pragma unroll
      for (int n = 0; n < 2; n++) {
        pr[n][0] = fd_exp2(sc[n][0] - ref0); pr[n][1] = fd_exp2(sc[n][1] - ref0);
        pr[n][2] = fd_exp2(sc[n][2] - ref1); pr[n][3] = fd_exp2(sc[n][3] - ref1);
      }
      l0 = l0 * a0 + pr[0][0] + pr[0][1] + pr[1][0] + pr[1][1];
      l1 = l1 * a1 + pr[0][2] + pr[0][3] + pr[1][2] + pr[1][3];
      unsigned pa0 = fd_pack(pr[0][0], pr[0][1]), pa1 = fd_pack(pr[0][2], pr[0][3]);
      unsigned pa2 = fd_pack(pr[1][0], pr[1][1]), pa3 = fd_pack(pr[1][2], pr[1][3]);
#pragma unroll
      for (int n = 0; n < HD / 8; n++) { o[n][0] *= a0; o[n][1] *= a0; o[n][2] *= a1; o[n][3] *= a1; }
#pragma unroll
      for (int dn = 0; dn < HD / 16; dn++) {
        unsigned b[4];
        fd_ldmatrix_x4_trans(b, vs + ((lane & 7) + 8 * ((lane >> 3) & 1)) * LD + dn * 16 + 8 * (lane >> 4));
        fd_mma(o[2 * dn], pa0, pa1, pa2, pa3, b[0], b[1]);
        fd_mma(o[2 * dn + 1], pa0, pa1, pa2, pa3, b[2], b[3]);
      }
      __syncwarp();
    }
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    // ---- merge the 8 warps; a warp's partial output [16][HD] float32 lies over its own K/V chunk buffers
    // (2 * 16 * LD bfloat16 = 16 * (HD + 8) floats), which it no longer reads
    {
      const int r0 = lane >> 2, r1 = r0 + 8, cq = (lane & 3) * 2;
      __syncwarp();
#pragma unroll
      for (int n = 0; n < HD / 8; n++) {
        float* d0 = reinterpret_cast<float*>(ks) + (size_t)r0 * HD + n * 8 + cq;
        float* d1 = reinterpret_cast<float*>(ks) + (size_t)r1 * HD + n * 8 + cq;
        d0[0] = o[n][0]; d0[1] = o[n][1]; d1[0] = o[n][2]; d1[1] = o[n][3];
      }
      if ((lane & 3) == 0) {
        mm[warp * 16 + r0] = m0; mm[warp * 16 + r1] = m1;
        ml[warp * 16 + r0] = l0; ml[warp * 16 + r1] = l1;
      }
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < gs * HD; idx += FD_THREADS) {
      int row = idx / HD, dim = idx - row * HD;
      float M = -INFINITY;
#pragma unroll
      for (int w = 0; w < FD_WARPS; w++) M = fmaxf(M, mm[w * 16 + row]);
      float Lsum = 0.f, O = 0.f;
      if (M != -INFINITY) {
#pragma unroll
        for (int w = 0; w < FD_WARPS; w++) {
          float f = fd_exp2(mm[w * 16 + row] - M);
          Lsum += ml[w * 16 + row] * f;
          O += reinterpret_cast<const float*>(kvs + (size_t)w * 2 * 16 * LD)[(size_t)row * HD + dim] * f;
        }
      }
      int hd = g * gs + row;
      if (p.splits == 1) {
        p.attn_out[(size_t)t * H * HD + (size_t)hd * HD + dim] = __float2bfloat16_rn(O / Lsum);
      } else {
        size_t pi = ((size_t)t * H + hd) * p.splits + s;
        p.part_o[pi * HD + dim] = O;
        if (dim == 0) { p.part_ml[pi * 2] = M; p.part_ml[pi * 2 + 1] = Lsum; }
      }
    }
    if (p.splits > 1) {
      __threadfence();
      __syncthreads();
      if (threadIdx.x == 0) s_ticket = atomicAdd(&p.tickets[(size_t)t * G + g], 1u);
      __syncthreads();
      if (s_ticket == (unsigned)p.splits - 1) {          // the last item of this (t, g) combines
        __threadfence();
        float* pm = fac + 16 * 64;
        float* pl = pm + 16 * 64;
        for (int idx = threadIdx.x; idx < gs * p.splits; idx += FD_THREADS) {
          int row = idx / p.splits, sp = idx - row * p.splits;
          size_t pi = ((size_t)t * H + (size_t)g * gs + row) * p.splits + sp;
          float2 v = __ldcg(reinterpret_cast<const float2*>(p.part_ml) + pi);
          pm[row * 64 + sp] = v.x;
          pl[row * 64 + sp] = v.y;
        }
        __syncthreads();
        if (threadIdx.x < gs) {
          int row = threadIdx.x;
          float M = -INFINITY;
          for (int sp = 0; sp < p.splits; sp++) M = fmaxf(M, pm[row * 64 + sp]);
          float Lsum = 0.f;
          for (int sp = 0; sp < p.splits; sp++) Lsum += pl[row * 64 + sp] * fd_exp2(pm[row * 64 + sp] - M);
          float inv = 1.f / Lsum;
          for (int sp = 0; sp < p.splits; sp++) fac[row * 64 + sp] = fd_exp2(pm[row * 64 + sp] - M) * inv;
        }
        __syncthreads();
        for (int idx = threadIdx.x; idx < gs * (HD / 4); idx += FD_THREADS) {
          int row = idx / (HD / 4), d4 = idx - row * (HD / 4);
          size_t base = ((size_t)t * H + (size_t)g * gs + row) * p.splits;
          float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 8
          for (int sp = 0; sp < p.splits; sp++) {
            float4 v = __ldcg(reinterpret_cast<const float4*>(p.part_o + (base + sp) * HD) + d4);
            float f = fac[row * 64 + sp];
            a.x += v.x * f; a.y += v.y * f; a.z += v.z * f; a.w += v.w * f;
          }
          bf16* dst = p.attn_out + (size_t)t * H * HD + ((size_t)g * gs + row) * HD + 4 * d4;
          uint2 raw;
          raw.x = fd_pack(a.x, a.y);
          raw.y = fd_pack(a.z, a.w);
          *reinterpret_cast<uint2*>(dst) = raw;
        }
        if (threadIdx.x == 0) p.tickets[(size_t)t * G + g] = 0;
      }
    }
    __syncthreads();
  }
}

// ------------------------------------------------------------------------------ the kernel
// Phase ph of the step: 5 per layer (q/k/v, attention, o, gate/up, down) and the output projection at the
// end.  The loop below is an interpreter over phases, so that each phase's code exists once.
__device__ __forceinline__ FdGemm fd_phase_gemm(const FdParams& p, int ph, int HD) {
  const int l = ph / 5, k = ph - 5 * l;
  if (l >= p.L) return fd_gemm_desc(p.lm_head, p.V, p.D, 0, true);
  const FdLayer& L = p.layers[l];
  if (k == 0) return fd_gemm_desc(L.wqkv, (p.H + 2 * p.G) * HD, p.D, 0, false);
  if (k == 2) return fd_gemm_desc(L.wo, p.D, p.H * HD, 0, false);
  if (k == 3) return fd_gemm_desc(L.wgu, 2 * p.F, p.D, p.F, true);
  if (k == 4) return fd_gemm_desc(L.wd, p.D, p.F, 0, false);
  FdGemm none = fd_gemm_desc(nullptr, 0, 0, 0, true);     // attention: no weights
  none.n_units = 0;
  return none;
}

template <int TN, int HD>
__global__ void __launch_bounds__(FD_THREADS, 2)
decode_fused_kernel(const __grid_constant__ FdParams p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  constexpr int TP = TN * 8;
  const int D = p.D, Hd = p.H * HD, Nqkv = (p.H + 2 * p.G) * HD;
  const int ldxs = fd_ldxs(D, Hd, p.F);
  bf16* xs = reinterpret_cast<bf16*>(smem_raw);                              // [TP][ldxs]
  float* red = reinterpret_cast<float*>(smem_raw + (size_t)TP * ldxs * sizeof(bf16));   // [8][16][TP+1]
  const int n_phases = 5 * p.L + 1;
  for (int ph = 0; ph < n_phases; ph++) {
    const int l = ph / 5, k = ph - 5 * l;
    const bool last = l >= p.L;
    const FdLayer& L = p.layers[last ? p.L - 1 : l];
    const int slot = (last ? p.L : l) * 16 + 3 * k;
    fd_stamp(p, slot);
    // one phase ahead: the weights of the next contraction start coming into L2 now (the attention
    // phase, which reads few bytes itself, brings in gate/up; the o phase then has nothing to ask for)
    if (!last && k != 2) {
      const int ahead = k == 0 ? ph + 2 : (k == 1 ? ph + 2 : ph + 1);
      fd_prefetch_phase(fd_phase_gemm(p, ahead, HD));
    }
    if (k == 1 && !last) {
      fd_attention<HD>(p, L, smem_raw);
    } else {
      const FdGemm g = fd_phase_gemm(p, ph, HD);
      int epi = FD_EPI_STORE;
      FdOut out = {p.logits, nullptr, p.V, p.scratch, p.gemm_tickets};
      int ldb = ldxs, k_base = 0;
      if (last || k == 0 || k == 3) {           // the contraction reads the normalised residual
        const float* w = last ? p.final_w : (k == 0 ? L.norm1_w : L.norm2_w);
        const float eps = last ? p.final_eps : (k == 0 ? L.eps1 : L.eps2);
        fd_norm_to_smem(p.x, w, eps, xs, ldxs, p.T, TP, D);
        if (!last && k == 0) { out.f = p.qkv; out.ld = Nqkv; }
        if (!last && k == 3) { epi = FD_EPI_SWIGLU; out.b = p.h; out.ld = p.F; }
      } else if (k == 2) {                      // ... the attention output
        for (int i = threadIdx.x; i < TP * (Hd / 8); i += FD_THREADS) {
          int t = i / (Hd / 8), c = i - t * (Hd / 8);
          uint4 v = make_uint4(0, 0, 0, 0);
          if (t < p.T) v = __ldcg(reinterpret_cast<const uint4*>(p.attn_out + (size_t)t * Hd) + c);
          *reinterpret_cast<uint4*>(xs + (size_t)t * ldxs + c * 8) = v;
        }
        epi = FD_EPI_ADD; out.f = p.x; out.ld = D;
      } else {                                  // ... this CTA's k range of h
        const int kb = g.kc * FD_KCTA, kn = min(FD_KCTA, p.F - kb);
        const int kw = min(FD_KCTA, p.F);             // columns staged per row (a multiple of 8)
        ldb = kw + FD_XPAD; k_base = kb;
        if (g.first < g.n_tiles) {
          for (int i = threadIdx.x; i < TP * (kw / 8); i += FD_THREADS) {
            int t = i / (kw / 8), c = i - t * (kw / 8);
            uint4 v = make_uint4(0, 0, 0, 0);
            if (t < p.T && c * 8 < kn) v = __ldcg(reinterpret_cast<const uint4*>(p.h + (size_t)t * p.F + kb) + c);
            *reinterpret_cast<uint4*>(xs + (size_t)t * ldb + c * 8) = v;
          }
        }
        epi = FD_EPI_ADD; out.f = p.x; out.ld = D;
      }
      __syncthreads();
      fd_stamp(p, slot + 1);
      fd_gemm_run<TN>(g, epi, xs, ldb, k_base, out, p.T, red);
    }
    fd_stamp(p, slot + 2);
    if (ph + 1 < n_phases) fd_grid_sync(p.barrier, p.status, p.host_status);
  }
}

// ------------------------------------------------------------------------------ host
template <int TN, int HD>
static int fd_launch(const FdParams& p, int max_ctas, cudaStream_t stream) {
  const int TP = TN * 8;
  const int Hd = p.H * HD;
  const int ldxs = fd_ldxs(p.D, Hd, p.F);
  size_t gemm_smem = (size_t)TP * ldxs * sizeof(bf16) + (size_t)FD_WARPS * 16 * (TP + 1) * sizeof(float);
  size_t attn_smem = (size_t)16 * (HD + FD_PAD) * sizeof(bf16) + (size_t)FD_WARPS * 2 * 16 * (HD + FD_PAD) * sizeof(bf16) +
                     (size_t)FD_WARPS * 16 * 2 * sizeof(float) + (size_t)3 * 16 * 64 * sizeof(float);
  size_t smem = gemm_smem > attn_smem ? gemm_smem : attn_smem;
  if (smem > 200 * 1024) return QD_ERR_UNSUPPORTED;
  auto kernel = decode_fused_kernel<TN, HD>;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
    cudaGetLastError();
    return QD_ERR_UNSUPPORTED;
  }
  int per_sm = 0, dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, FD_THREADS, smem) != cudaSuccess || per_sm < 1) {
    cudaGetLastError();
    return QD_ERR_UNSUPPORTED;
  }
  if (per_sm > 2) per_sm = 2;
  int grid = per_sm * sms;
  if (grid > max_ctas) grid = max_ctas;
  void* args[] = {(void*)&p};
  cudaError_t e = cudaLaunchCooperativeKernel((void*)kernel, dim3(grid), dim3(FD_THREADS), args, smem, stream);
  return (int)e;
}

// A decode step of T <= 16 tokens (one per request): see FdParams.  Refuses what it does not take
// (head size not in 16..128 by 16, more than 16 query heads per kv head, page size not a multiple of 16,
// widths that are no multiple of 8, more than 64 splits).
extern "C" int qd_decode_step_fused(const FdParams* params, int max_ctas, cudaStream_t stream) {
  const FdParams& p = *params;
  if (p.T < 1 || p.T > 16 || p.L < 1) return QD_ERR_UNSUPPORTED;
  if (p.G < 1 || p.H % p.G != 0 || p.H / p.G > 16 || p.page_size % 16 != 0 || p.splits < 1 || p.splits > 64)
    return QD_ERR_UNSUPPORTED;
  if (p.D % 8 != 0 || p.F % 8 != 0 || (p.H * p.d) % 8 != 0 || (p.rotary_dim & 1) || p.rotary_dim > p.d)
    return QD_ERR_UNSUPPORTED;
  {
    // scratch and tickets of the contractions whose k range several CTAs share
    const int TP = p.T <= 8 ? 8 : 16;
    const long long Nqkv = (long long)(p.H + 2 * p.G) * p.d;
    auto units = [](long long rows, long long K) { return ((rows + 15) / 16) * ((K + FD_KCTA - 1) / FD_KCTA); };
    long long most = units(Nqkv, p.D);
    if (units(p.D, (long long)p.H * p.d) > most) most = units(p.D, (long long)p.H * p.d);
    if (units(p.D, p.F) > most) most = units(p.D, p.F);
    long long tiles = (Nqkv > p.D ? Nqkv : p.D) / 16 + 1;
    if (most * 16 * TP > p.scratch_floats || tiles > p.n_gemm_tickets) return QD_ERR_UNSUPPORTED;
  }
#define FD_CASE(HD)                                                                         \
  case HD:                                                                                  \
    return p.T <= 8 ? fd_launch<1, HD>(p, max_ctas, stream) : fd_launch<2, HD>(p, max_ctas, stream);
  switch (p.d) {
    FD_CASE(16) FD_CASE(32) FD_CASE(48) FD_CASE(64) FD_CASE(96) FD_CASE(128)
    default: return QD_ERR_UNSUPPORTED;
  }
#undef FD_CASE
}

extern "C" int qd_decode_fused_param_bytes() { return (int)sizeof(FdParams); }
extern "C" int qd_decode_fused_layer_bytes() { return (int)sizeof(FdLayer); }
