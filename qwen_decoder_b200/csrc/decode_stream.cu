// The products of a decode step of up to 8 tokens, each with the work before and after it folded in, so
// that a layer is four launches (q/k/v, attention, output projection, feed-forward) instead of six and no
// launch exists only to add partial sums or to normalise eight rows:
//
//   ds_gemm<PRO, EPI>   Y = X W^T as a persistent weight streamer (producer warp, ring of stages filled by
//                       cp.async.bulk, four consumer warps on mma.sync, tokens resident in shared memory)
//     prologue  PRO_ROWS  the tokens' bfloat16 rows are copied in
//               PRO_NORM  the tokens are rows of the float32 residual sum: every CTA normalises them itself
//                         (RMSNorm in float32: gpu_kernels.cu:32-67 of the reference) into its resident rows
//     epilogue  EPI_STORE     (+ bias) -> out, bfloat16 or float32 (the output projection's logits)
//               EPI_PARTIAL   float32 partial sums per share of K
//               EPI_ADD       the residual sum += Y: with K shared among CTAs the last CTA to finish a tile
//                             (a ticket per tile) adds the shares in their fixed order, so the sum does not
//                             depend on which CTA came last
//               EPI_QKV       + bias, rotation of q and k by position (gpu_kernels.cu:82-112), k and v to the
//                             token's cache slot (gpu_kernels.cu:116-133), q out as bfloat16: what the
//                             attention kernel then starts from
//   ds_ffn              PRO_NORM, gate/up with SwiGLU (gpu_kernels.cu:149-160), a grid barrier, the down
//                       projection with EPI_ADD; the producer warp fetches the down projection's first
//                       weights while the barrier is waited for
//
// A CTA keeps ONE share of K for a whole product (CTA b: share b % splits, tiles b / splits, + grid / splits,
// ...).  The number of stages and the width of the resident rows are launch parameters: hidden sizes beyond
// 2,048 take one CTA per SM with more stages instead of two with two.  Every wait is bounded (common.cuh).
#include "common.cuh"
#include <cstdlib>

#define DS_CONSUMERS 4
#define DS_THREADS ((DS_CONSUMERS + 1) * 32)
#define DS_KC 1024                           // k per stage
#define DS_ROW_BYTES (DS_KC * 2 + 64)        // padded row of a stage: 16-byte reads of 8 rows x 4 lanes hit 32 banks once
#define DS_STAGE_BYTES (16 * DS_ROW_BYTES)   // 16 rows of W
#define DS_MAX_STAGES 6
#define DS_SPIN_LIMIT (1u << 24)
#define DS_RED_LD 9

#define PRO_ROWS 0
#define PRO_NORM 1
#define EPI_STORE 0
#define EPI_PARTIAL 1
#define EPI_ADD 3
#define EPI_QKV 4

struct DsArgs {
  const bf16* W; int N, K, n_tiles, splits, T;
  // prologue
  const bf16* X; long long ldx;                               // PRO_ROWS: [T, K] bfloat16
  const float* xf; const float* norm_w; float eps; const int* rows;   // PRO_NORM: residual sum [*, K], row t = rows[t] or t
  // epilogue
  const float* bias; void* out; long long ldo; int out_f32;   // EPI_STORE
  float* part;                                                // EPI_PARTIAL, EPI_ADD: [splits, T, N]
  float* resid; unsigned* tickets;                            // EPI_ADD: [T, N] float32; one ticket per tile, zero between launches
  // EPI_QKV
  bf16* q_out; bf16* kv; const int* positions; const int* slot_map; const float* cos_t; const float* sin_t;
  int H, G, d, page_size, rotary_half, pairing, write_kv;
  // the second product of ds_ffn (down projection), its intermediate and its barrier
  const bf16* W2; int N2, K2, n_tiles2, splits2; bf16* h; long long ldh; unsigned* gbar;
  // shared memory
  int n_stages, xr_row_bytes;
  int* status;
};

__device__ __forceinline__ unsigned ds_smem(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void ds_mbar_init(unsigned long long* bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(ds_smem(bar)), "r"(count));
}
__device__ __forceinline__ void ds_mbar_arrive(unsigned long long* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(ds_smem(bar)) : "memory");
}
__device__ __forceinline__ void ds_mbar_expect_tx(unsigned long long* bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(ds_smem(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool ds_mbar_wait(unsigned long long* bar, unsigned parity, volatile int* dead,
                                             unsigned poll_limit = DS_SPIN_LIMIT) {
  return qd_mbar_wait_bounded(ds_smem(bar), parity, dead, poll_limit, 2000000000ull);
}
__device__ __forceinline__ void ds_bulk_copy(void* dst, const void* src, unsigned bytes, unsigned long long* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(ds_smem(dst)), "l"(src), "r"(bytes), "r"(ds_smem(bar)) : "memory");
}
__device__ __forceinline__ void ds_mma(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0,
                                       unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ds_consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(DS_CONSUMERS * 32) : "memory"); }

// The row of W that row r of a tile holds.  With half-split rotary pairs (p, p + d/2) a tile of a q or k head
// takes 8 elements of the first half and their 8 partners, so that both elements of a pair meet in one epilogue.
template <int EPI>
__device__ __forceinline__ long long ds_row(const DsArgs& a, int tile, int r) {
  if (EPI == EPI_QKV && a.pairing == 1) {
    const int tph = a.d >> 4;
    const int head = tile / tph, i = tile - head * tph;
    if (head < a.H + a.G) return (long long)head * a.d + 8 * i + (r & 7) + ((r & 8) ? (a.d >> 1) : 0);
  }
  const long long row = (long long)tile * 16 + r;
  return row < a.N ? row : a.N - 1;
}

// RMSNorm of the tokens' rows of the float32 residual sum into the resident rows (bfloat16): columns
// [k_begin, k_end) of out = x / sqrt(mean(x^2) + eps) * w; rows >= T are zero.  Called by the consumer warps.
__device__ __forceinline__ void ds_norm_rows(const DsArgs& a, unsigned char* xres, int k_begin, int k_end, int warp,
                                             int lane) {
  const int D = a.K;
  for (int t = warp; t < 8; t += DS_CONSUMERS) {
    bf16* dst = reinterpret_cast<bf16*>(xres + (size_t)t * a.xr_row_bytes);
    if (t >= a.T) {
      for (int k = k_begin + lane * 2; k < k_end; k += 64) *reinterpret_cast<unsigned*>(dst + (k - k_begin)) = 0u;
      continue;
    }
    const float* src = a.xf + (size_t)(a.rows ? a.rows[t] : t) * D;
    float ss = 0.f;
    if ((D & 3) == 0) {
      for (int k = lane * 4; k < D; k += 128) {
        const float4 v = *reinterpret_cast<const float4*>(src + k);
        ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
      }
    } else {
      for (int k = lane; k < D; k += 32) ss += src[k] * src[k];
    }
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)D + a.eps);
    for (int k = k_begin + lane * 2; k < k_end; k += 64) {        // k_begin and k_end are even (multiples of DS_KC, or K)
      const float2 v = *reinterpret_cast<const float2*>(src + k);
      const float2 w = *reinterpret_cast<const float2*>(a.norm_w + k);
      __nv_bfloat162 o = __floats2bfloat162_rn(v.x * inv * w.x, v.y * inv * w.y);
      *reinterpret_cast<unsigned*>(dst + (k - k_begin)) = *reinterpret_cast<unsigned*>(&o);
    }
  }
}

// One stage through the tensor cores: this warp's quarter of the stage's k against the resident rows.
__device__ __forceinline__ void ds_stage_mma(float (&acc)[4], const unsigned char* st, const unsigned char* xs,
                                             int xr_row_bytes, int K, int c, int warp, int lane) {
  const int j = lane & 3, r = lane >> 2;
#pragma unroll
  for (int u = 0; u < DS_KC / 32 / DS_CONSUMERS; u++) {
    const int kq = warp * (DS_KC / DS_CONSUMERS) + u * 32;
    if (c * DS_KC + kq >= K) break;                 // the whole k-step lies past K (same for all lanes)
    const bool in = c * DS_KC + kq + 8 * j < K;     // lanes past K feed zeros; every lane runs the MMAs
    const uint4 zero = make_uint4(0, 0, 0, 0);
    const size_t col = (size_t)(kq + 8 * j) * 2;
    const uint4 lo = in ? *reinterpret_cast<const uint4*>(st + (size_t)r * DS_ROW_BYTES + col) : zero;
    const uint4 hi = in ? *reinterpret_cast<const uint4*>(st + (size_t)(r + 8) * DS_ROW_BYTES + col) : zero;
    const uint4 b = in ? *reinterpret_cast<const uint4*>(xs + (size_t)r * xr_row_bytes + col) : zero;
    ds_mma(acc, lo.x, hi.x, lo.y, hi.y, b.x, b.y);
    ds_mma(acc, lo.z, hi.z, lo.w, hi.w, b.z, b.w);
  }
}

// The four warps' shares of a stage's k, side by side in shared memory; the epilogues add them up.
__device__ __forceinline__ void ds_to_red(float* red, const float (&acc)[4], int warp, int lane) {
  const int j = lane & 3, r = lane >> 2;
  float* base = red + (size_t)warp * 16 * DS_RED_LD;
  base[r * DS_RED_LD + 2 * j] = acc[0];
  base[r * DS_RED_LD + 2 * j + 1] = acc[1];
  base[(r + 8) * DS_RED_LD + 2 * j] = acc[2];
  base[(r + 8) * DS_RED_LD + 2 * j + 1] = acc[3];
  ds_consumer_sync();
}
__device__ __forceinline__ float ds_red_sum(const float* red, int row, int tok) {
  float v = 0.f;
#pragma unroll
  for (int w = 0; w < DS_CONSUMERS; w++) v += red[((size_t)w * 16 + row) * DS_RED_LD + tok];
  return v;
}

// residual sum += this tile's result.  With one share of K: directly.  With several: every share leaves its
// partial sums, takes a ticket, and the last one adds all shares in the order of the shares.
__device__ __forceinline__ void ds_epilogue_add(float* resid, float* part, unsigned* tickets, unsigned* s_ticket,
                                                const float* red, int tile, int sp, int splits, int T, int N) {
  if (splits == 1) {
    for (int idx = threadIdx.x; idx < 16 * 8; idx += DS_CONSUMERS * 32) {
      const int row = idx & 15, tok = idx >> 4, n = tile * 16 + row;
      if (tok < T && n < N) resid[(size_t)tok * N + n] += ds_red_sum(red, row, tok);
    }
    return;
  }
  for (int idx = threadIdx.x; idx < 16 * 8; idx += DS_CONSUMERS * 32) {
    const int row = idx & 15, tok = idx >> 4, n = tile * 16 + row;
    if (tok < T && n < N) part[((size_t)sp * T + tok) * N + n] = ds_red_sum(red, row, tok);
  }
  __threadfence();
  ds_consumer_sync();
  if (threadIdx.x == 0) *s_ticket = atomicAdd(&tickets[tile], 1u);
  ds_consumer_sync();
  if (*s_ticket == (unsigned)splits - 1) {
    __threadfence();
    for (int idx = threadIdx.x; idx < 16 * 8; idx += DS_CONSUMERS * 32) {
      const int row = idx & 15, tok = idx >> 4, n = tile * 16 + row;
      if (tok >= T || n >= N) continue;
      float v = resid[(size_t)tok * N + n];
      for (int q = 0; q < splits; q++) v += __ldcg(part + ((size_t)q * T + tok) * N + n);
      resid[(size_t)tok * N + n] = v;
    }
    if (threadIdx.x == 0) tickets[tile] = 0;          // as found: the next launch counts from zero again
  }
}

template <int PRO, int EPI>
__global__ void __launch_bounds__(DS_THREADS) ds_gemm_kernel(const DsArgs a) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  const int NST = a.n_stages;
  unsigned char* stages = smem_raw;                                                  // NST x 16 rows of W
  unsigned char* xres = smem_raw + (size_t)NST * DS_STAGE_BYTES;                     // 8 token rows
  float* red = reinterpret_cast<float*>(xres + (size_t)8 * a.xr_row_bytes);          // [4][16][9]
  __shared__ unsigned long long full_bar[DS_MAX_STAGES], empty_bar[DS_MAX_STAGES], x_bar;
  __shared__ int dead;
  __shared__ unsigned s_ticket;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    dead = 0;
    for (int s = 0; s < NST; s++) { ds_mbar_init(&full_bar[s], 1); ds_mbar_init(&empty_bar[s], DS_CONSUMERS); }
    ds_mbar_init(&x_bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  const int T = a.T, K = a.K, splits = a.splits;
  const int n_chunks = (K + DS_KC - 1) / DS_KC;
  const int stride = (int)gridDim.x / splits;                 // CTAs per share of K (the host made it >= 1)
  const int sp = (int)blockIdx.x % splits;
  const int first = (int)blockIdx.x / splits;
  const bool idle = first >= stride;
  const int c_begin = (int)((long long)n_chunks * sp / splits), c_end = (int)((long long)n_chunks * (sp + 1) / splits);
  const int k_begin = c_begin * DS_KC, k_end = min(K, c_end * DS_KC);

  if (warp == DS_CONSUMERS) {
    // ------------------------------------------------------------ producer
    // weights are written by no kernel of the step: they are asked for at once; PRO_ROWS copies the tokens'
    // rows after the dependency wait, PRO_NORM leaves the tokens to the consumers
    if (idle) return;
    unsigned it = 0;
    bool waited = PRO != PRO_ROWS;
    auto tokens = [&]() {
      pdl_wait();
      waited = true;
      const unsigned xb = (unsigned)((k_end - k_begin) * 2);
      if (lane == 0) ds_mbar_expect_tx(&x_bar, xb * T);
      __syncwarp();
      for (int t = lane; t < T; t += 32)
        ds_bulk_copy(xres + (size_t)t * a.xr_row_bytes, a.X + (size_t)t * a.ldx + k_begin, xb, &x_bar);
    };
    for (int tile = first; tile < a.n_tiles; tile += stride) {
      const long long row = ds_row<EPI>(a, tile, lane & 15);
      for (int c = c_begin; c < c_end; c++, it++) {
        const int s = it % NST;
        const unsigned ph = (it / NST) & 1;
        if (it >= (unsigned)NST && !waited) tokens();        // the ring is full of W requests
        if (!ds_mbar_wait(&empty_bar[s], ph ^ 1, &dead) && lane == 0) atomicExch(a.status, 1);
        const int k0 = c * DS_KC;
        const unsigned row_bytes = (unsigned)(min(DS_KC, K - k0) * 2);
        if (lane == 0) ds_mbar_expect_tx(&full_bar[s], row_bytes * 16);
        __syncwarp();
        if (lane < 16)
          ds_bulk_copy(stages + (size_t)s * DS_STAGE_BYTES + (size_t)lane * DS_ROW_BYTES, a.W + row * K + k0, row_bytes,
                       &full_bar[s]);
      }
    }
    if (!waited) tokens();
    return;
  }

  // -------------------------------------------------------------- consumers
  if (idle) { pdl_launch_dependents(); return; }
  if (PRO == PRO_NORM) {
    pdl_wait();
    ds_norm_rows(a, xres, k_begin, k_end, warp, lane);
    ds_consumer_sync();
  } else if (EPI == EPI_ADD) {
    pdl_wait();                                   // the residual sum is read and written in the epilogue
  }
  unsigned it = 0;
  bool have_x = PRO != PRO_ROWS;
  for (int tile = first; tile < a.n_tiles; tile += stride) {
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int c = c_begin; c < c_end; c++, it++) {
      const int s = it % NST;
      const unsigned ph = (it / NST) & 1;
      if (!ds_mbar_wait(&full_bar[s], ph, &dead) && lane == 0) atomicExch(a.status, 2);
      if (!have_x) {
        if (!ds_mbar_wait(&x_bar, 0, &dead) && lane == 0) atomicExch(a.status, 2);
        have_x = true;
      }
      ds_stage_mma(acc, stages + (size_t)s * DS_STAGE_BYTES, xres + (size_t)(c - c_begin) * DS_KC * 2, a.xr_row_bytes, K, c,
                   warp, lane);
      __syncwarp();
      if (lane == 0) ds_mbar_arrive(&empty_bar[s]);
    }
    ds_to_red(red, acc, warp, lane);
    if (EPI == EPI_ADD) {
      ds_epilogue_add(a.resid, a.part, a.tickets, &s_ticket, red, tile, sp, splits, T, a.N);
    } else if (EPI == EPI_QKV) {
      // 8 pairs x 8 tokens: pair pp of the tile is rows (2pp, 2pp+1), or (pp, pp+8) with half-split pairs
      const int idx = threadIdx.x;
      const int pp = idx & 7, tok = idx >> 3;
      if (idx < 64 && tok < T) {
        const int tph = a.d >> 4;
        const int head = tile / tph, i = tile - head * tph;
        const bool is_v = head >= a.H + a.G;
        const bool half_pairs = a.pairing == 1 && !is_v;
        const int ra = half_pairs ? pp : 2 * pp, rb = half_pairs ? pp + 8 : 2 * pp + 1;
        const int fa = half_pairs ? 8 * i + pp : 16 * i + 2 * pp;                   // element of the head
        const int fb = half_pairs ? fa + (a.d >> 1) : fa + 1;
        float va = ds_red_sum(red, ra, tok), vb = ds_red_sum(red, rb, tok);
        if (a.bias) { va += a.bias[(size_t)head * a.d + fa]; vb += a.bias[(size_t)head * a.d + fb]; }
        const int p = 8 * i + pp;                                                    // the pair's index in its head
        if (!is_v && a.cos_t && p < a.rotary_half) {
          const int pos = a.positions[tok];
          const float cs = a.cos_t[(size_t)pos * a.rotary_half + p], sn = a.sin_t[(size_t)pos * a.rotary_half + p];
          const float xa = va * cs - vb * sn, xb = va * sn + vb * cs;
          va = xa; vb = xb;
        }
        const bf16 ha = __float2bfloat16_rn(va), hb = __float2bfloat16_rn(vb);
        if (head < a.H) {
          bf16* q = a.q_out + (size_t)tok * a.H * a.d + (size_t)head * a.d;
          q[fa] = ha; q[fb] = hb;
        } else if (a.write_kv) {
          const int g = is_v ? head - a.H - a.G : head - a.H;
          const int slot = a.slot_map[tok];
          const int page = slot / a.page_size, off = slot - page * a.page_size;
          bf16* dst = a.kv + (((size_t)page * 2 + (is_v ? 1 : 0)) * a.G + g) * a.page_size * a.d + (size_t)off * a.d;
          dst[fa] = ha; dst[fb] = hb;
        }
      }
    } else {
      for (int idx = threadIdx.x; idx < 16 * 8; idx += DS_CONSUMERS * 32) {
        const int row = idx & 15, tok = idx >> 4, n = tile * 16 + row;
        if (tok >= T || n >= a.N) continue;
        float v = ds_red_sum(red, row, tok);
        if (EPI == EPI_PARTIAL) {
          a.part[((size_t)sp * T + tok) * a.N + n] = v;
        } else {
          if (a.bias) v += a.bias[n];
          if (a.out_f32) reinterpret_cast<float*>(a.out)[(size_t)tok * a.ldo + n] = v;
          else reinterpret_cast<bf16*>(a.out)[(size_t)tok * a.ldo + n] = __float2bfloat16_rn(v);
        }
      }
    }
    ds_consumer_sync();                                       // red is reused by the next tile
  }
  pdl_launch_dependents();
}

// ---------------------------------------------------------------------------------------------
// The feed-forward: rmsnorm, gate/up with SwiGLU, a grid barrier, the down projection added to the residual
// sum.  Phase 1 shares no K (every CTA walks tiles b, b + grid, ... over the whole hidden size); phase 2 shares
// K2 = the intermediate size among splits2 CTAs per tile.  All CTAs are resident (the host launches no more
// than fit); the barrier's spin is bounded like every other wait.
__global__ void __launch_bounds__(DS_THREADS) ds_ffn_kernel(const DsArgs a) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  const int NST = a.n_stages;
  unsigned char* stages = smem_raw;
  unsigned char* xres = smem_raw + (size_t)NST * DS_STAGE_BYTES;
  float* red = reinterpret_cast<float*>(xres + (size_t)8 * a.xr_row_bytes);
  __shared__ unsigned long long full_bar[DS_MAX_STAGES], empty_bar[DS_MAX_STAGES], x_bar, go_bar;
  __shared__ int dead;
  __shared__ unsigned s_ticket;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    dead = 0;
    for (int s = 0; s < NST; s++) { ds_mbar_init(&full_bar[s], 1); ds_mbar_init(&empty_bar[s], DS_CONSUMERS); }
    ds_mbar_init(&x_bar, 1);
    ds_mbar_init(&go_bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  const int T = a.T;
  const int F = a.N >> 1;                                    // W = [gate; up] of [2F, K]
  const int chunks1 = (a.K + DS_KC - 1) / DS_KC;
  const int chunks2 = (a.K2 + DS_KC - 1) / DS_KC;
  const int stride2 = (int)gridDim.x / a.splits2;
  const int sp2 = (int)blockIdx.x % a.splits2;
  const int first2 = (int)blockIdx.x / a.splits2;
  const bool idle2 = first2 >= stride2;
  const int cb2 = (int)((long long)chunks2 * sp2 / a.splits2), ce2 = (int)((long long)chunks2 * (sp2 + 1) / a.splits2);
  const int k2_begin = cb2 * DS_KC, k2_end = min(a.K2, ce2 * DS_KC);

  if (warp == DS_CONSUMERS) {
    // ------------------------------------------------------------ producer: weights only, never waits for a kernel
    unsigned it = 0;
    auto weights = [&](const bf16* W, long long row, int K, int c) {
      const int s = it % NST;
      const unsigned ph = (it / NST) & 1;
      if (!ds_mbar_wait(&empty_bar[s], ph ^ 1, &dead) && lane == 0) atomicExch(a.status, 1);
      const int k0 = c * DS_KC;
      const unsigned row_bytes = (unsigned)(min(DS_KC, K - k0) * 2);
      if (lane == 0) ds_mbar_expect_tx(&full_bar[s], row_bytes * 16);
      __syncwarp();
      if (lane < 16)
        ds_bulk_copy(stages + (size_t)s * DS_STAGE_BYTES + (size_t)lane * DS_ROW_BYTES, W + row * K + k0, row_bytes, &full_bar[s]);
      it++;
    };
    for (int tile = blockIdx.x; tile < a.n_tiles; tile += gridDim.x) {
      int f = tile * 8 + (lane & 7);
      if (f >= F) f = F - 1;
      const long long row = (lane & 8) ? (long long)F + f : f;
      for (int c = 0; c < chunks1; c++) weights(a.W, row, a.K, c);
    }
    // the down projection's weights follow at once; its tokens (h) only when every CTA has written its part
    unsigned issued2 = 0;
    bool have_h = false;
    auto tokens2 = [&]() {
      have_h = true;
      if (!ds_mbar_wait(&go_bar, 0, &dead) && lane == 0) atomicExch(a.status, 3);
      asm volatile("fence.proxy.async;" ::: "memory");        // h was written by ordinary stores of other CTAs
      if (idle2) return;
      const unsigned xb = (unsigned)((k2_end - k2_begin) * 2);
      if (lane == 0) ds_mbar_expect_tx(&x_bar, xb * T);
      __syncwarp();
      for (int t = lane; t < T; t += 32)
        ds_bulk_copy(xres + (size_t)t * a.xr_row_bytes, a.h + (size_t)t * a.ldh + k2_begin, xb, &x_bar);
    };
    if (!idle2) {
      for (int tile = first2; tile < a.n_tiles2; tile += stride2) {
        long long row = (long long)tile * 16 + (lane & 15);
        if (row >= a.N2) row = a.N2 - 1;
        for (int c = cb2; c < ce2; c++) {
          if (issued2 >= (unsigned)NST && !have_h) tokens2();
          weights(a.W2, row, a.K2, c);
          issued2++;
        }
      }
    }
    if (!have_h) tokens2();
    return;
  }

  // -------------------------------------------------------------- consumers
  pdl_wait();
  ds_norm_rows(a, xres, 0, a.K, warp, lane);
  ds_consumer_sync();
  unsigned it = 0;
  auto stage = [&](float (&acc)[4], int K, int c, int c_first) {
    const int s = it % NST;
    const unsigned ph = (it / NST) & 1;
    if (!ds_mbar_wait(&full_bar[s], ph, &dead) && lane == 0) atomicExch(a.status, 2);
    ds_stage_mma(acc, stages + (size_t)s * DS_STAGE_BYTES, xres + (size_t)(c - c_first) * DS_KC * 2, a.xr_row_bytes, K, c,
                 warp, lane);
    __syncwarp();
    if (lane == 0) ds_mbar_arrive(&empty_bar[s]);
    it++;
  };
  // ---- phase 1: gate, up, SwiGLU
  for (int tile = blockIdx.x; tile < a.n_tiles; tile += gridDim.x) {
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int c = 0; c < chunks1; c++) stage(acc, a.K, c, 0);
    ds_to_red(red, acc, warp, lane);
    for (int idx = threadIdx.x; idx < 8 * 8; idx += DS_CONSUMERS * 32) {
      const int row = idx & 7, tok = idx >> 3;
      const int f = tile * 8 + row;
      if (tok >= T || f >= F) continue;
      const float gate = ds_red_sum(red, row, tok), up = ds_red_sum(red, row + 8, tok);
      a.h[(size_t)tok * a.ldh + f] = __float2bfloat16_rn(gate / (1.0f + expf(-gate)) * up);
    }
    ds_consumer_sync();
  }
  // ---- every CTA's part of h is written: meet the others
  ds_consumer_sync();
  if (threadIdx.x == 0) {
    volatile unsigned* gen_p = a.gbar + 1;
    const unsigned gen = *gen_p;
    __threadfence();
    const unsigned arrived = atomicAdd(a.gbar, 1u);
    if (arrived == gridDim.x - 1) {
      a.gbar[0] = 0;
      __threadfence();
      atomicAdd(a.gbar + 1, 1u);
    } else if (!dead) {
      unsigned long long start = 0;
      bool ok = false;
      for (unsigned spin = 0; spin < (1u << 26); spin++) {
        if (*gen_p != gen) { ok = true; break; }
        if ((spin & 1023) == 1023) {
          unsigned long long now;
          asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
          if (start == 0) start = now;
          else if (now - start > 2000000000ull) break;
        }
      }
      if (!ok) { dead = 1; atomicExch(a.status, 4); }
    }
    __threadfence();
    ds_mbar_arrive(&go_bar);
  }
  // ---- phase 2: down projection, added to the residual sum
  if (!idle2) {
    if (!ds_mbar_wait(&x_bar, 0, &dead) && lane == 0) atomicExch(a.status, 2);
    for (int tile = first2; tile < a.n_tiles2; tile += stride2) {
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
      for (int c = cb2; c < ce2; c++) stage(acc, a.K2, c, cb2);
      ds_to_red(red, acc, warp, lane);
      ds_epilogue_add(a.resid, a.part, a.tickets, &s_ticket, red, tile, sp2, a.splits2, T, a.N2);
      ds_consumer_sync();
    }
  }
  pdl_launch_dependents();
}

// ------------------------------------------------------------------------------------------------ host side
static int* g_ds_status[64];   // per device: one int of device memory for the kernels' error status
static int* ds_status_word() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  if (!g_ds_status[dev]) {
    int* p = nullptr;
    if (cudaMalloc(&p, sizeof(int)) != cudaSuccess) return nullptr;
    cudaMemset(p, 0, sizeof(int));
    g_ds_status[dev] = p;
  }
  return g_ds_status[dev];
}
static int ds_sm_count() {
  static int sms[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 1;
  if (!sms[dev]) cudaDeviceGetAttribute(&sms[dev], cudaDevAttrMultiProcessorCount, dev);
  return sms[dev] > 0 ? sms[dev] : 1;
}
static int ds_smem_limit() {
  static int lim[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 48 * 1024;
  if (!lim[dev]) cudaDeviceGetAttribute(&lim[dev], cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
  return lim[dev];
}

// Shared memory of a CTA whose resident rows are ``k_res`` elements wide: two CTAs per SM with two stages each
// if that fits, else one CTA with as many stages as fit (at most DS_MAX_STAGES, at least two).
struct DsShape { int n_stages, xr_row_bytes, ctas_per_sm; size_t smem; };
static bool ds_shape(int k_res, DsShape* out) {
  const int xr_row_bytes = k_res * 2 + 64;
  const size_t fixed = (size_t)8 * xr_row_bytes + (size_t)DS_CONSUMERS * 16 * DS_RED_LD * sizeof(float);
  const size_t limit = (size_t)ds_smem_limit();
  const size_t per_sm = limit + 1024;                  // what an SM has: the per-CTA limit and its reserve
  const size_t two = fixed + (size_t)2 * DS_STAGE_BYTES;
  if (2 * (two + 1024) <= per_sm) { *out = {2, xr_row_bytes, 2, two}; return true; }
  int n = (int)((limit - fixed) / DS_STAGE_BYTES);
  if (fixed > limit || n < 2) return false;
  if (n > DS_MAX_STAGES) n = DS_MAX_STAGES;
  *out = {n, xr_row_bytes, 1, fixed + (size_t)n * DS_STAGE_BYTES};
  return true;
}

extern "C" int qd_decode_stream_ctas(int k_res) {
  DsShape s;
  if (!ds_shape(k_res, &s)) return 0;
  return s.ctas_per_sm * ds_sm_count();
}

template <typename Kernel>
static int ds_launch(Kernel kernel, DsArgs& a, const DsShape& s, int grid, cudaStream_t stream) {
  a.n_stages = s.n_stages;
  a.xr_row_bytes = s.xr_row_bytes;
  a.status = ds_status_word();
  if (!a.status) return QD_ERR_UNSUPPORTED;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)s.smem) != cudaSuccess) {
    cudaGetLastError();
    return QD_ERR_UNSUPPORTED;
  }
  qd_launch(kernel, dim3((unsigned)grid), dim3(DS_THREADS), s.smem, stream, a);
  return qd_last_error();
}

static bool ds_aligned(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// The widest share of K when ``n_chunks`` stages are dealt to ``splits`` shares, in elements.
static int ds_widest_share(int K, int splits) {
  const int n_chunks = (K + DS_KC - 1) / DS_KC;
  int widest = 0;
  for (int sp = 0; sp < splits; sp++) {
    const int cb = (int)((long long)n_chunks * sp / splits), ce = (int)((long long)n_chunks * (sp + 1) / splits);
    const int w = (ce * DS_KC < K ? ce * DS_KC : K) - cb * DS_KC;
    if (w > widest) widest = w;
  }
  return widest;
}

// Y = X W^T for T <= 8 tokens.  pro: 0 rows of X (bfloat16 [T, K], ldx), 1 rmsnorm of xf[rows[t] or t, :K] (float32)
// with norm_w and eps.  epi: 0 store (+ bias) to out (out_f32 or bfloat16, ldo), 1 partial sums [splits, T, N],
// 3 resid[T, N] += Y (part and tickets needed when splits > 1).
extern "C" int qd_ds_gemm(const void* W, int N, int K, int T, int splits, int pro, const void* X, long long ldx,
                          const float* xf, const float* norm_w, float eps, const int* rows, int epi, const float* bias,
                          void* out, long long ldo, int out_f32, float* part, float* resid, unsigned* tickets,
                          cudaStream_t stream) {
  if (T < 1 || T > 8 || N < 1 || K < 8 || (K & 7) || splits < 1 || !ds_aligned(W)) return QD_ERR_UNSUPPORTED;
  if (pro == PRO_ROWS && (!X || !ds_aligned(X) || (ldx & 7))) return QD_ERR_UNSUPPORTED;
  if (pro == PRO_NORM && (!xf || !norm_w)) return QD_ERR_UNSUPPORTED;
  if (epi == EPI_PARTIAL && !part) return QD_ERR_UNSUPPORTED;
  if (epi == EPI_ADD && (!resid || (splits > 1 && (!part || !tickets)))) return QD_ERR_UNSUPPORTED;
  if (epi == EPI_STORE && (!out || splits != 1)) return QD_ERR_UNSUPPORTED;
  DsShape s;
  if (!ds_shape(ds_widest_share(K, splits), &s)) return QD_ERR_UNSUPPORTED;
  const int max_ctas = s.ctas_per_sm * ds_sm_count();
  if (splits > max_ctas) return QD_ERR_UNSUPPORTED;
  DsArgs a = {};
  a.W = (const bf16*)W; a.N = N; a.K = K; a.n_tiles = (N + 15) / 16; a.splits = splits; a.T = T;
  a.X = (const bf16*)X; a.ldx = ldx; a.xf = xf; a.norm_w = norm_w; a.eps = eps; a.rows = rows;
  a.bias = bias; a.out = out; a.ldo = ldo; a.out_f32 = out_f32; a.part = part; a.resid = resid; a.tickets = tickets;
  const int per_share = a.n_tiles < max_ctas / splits ? a.n_tiles : max_ctas / splits;
  const int grid = per_share * splits;
#define DS_PICK(P, E) return ds_launch(ds_gemm_kernel<P, E>, a, s, grid, stream)
  if (pro == PRO_ROWS) {
    if (epi == EPI_STORE) DS_PICK(PRO_ROWS, EPI_STORE);
    if (epi == EPI_PARTIAL) DS_PICK(PRO_ROWS, EPI_PARTIAL);
    if (epi == EPI_ADD) DS_PICK(PRO_ROWS, EPI_ADD);
  } else if (pro == PRO_NORM) {
    if (epi == EPI_STORE) DS_PICK(PRO_NORM, EPI_STORE);
    if (epi == EPI_PARTIAL) DS_PICK(PRO_NORM, EPI_PARTIAL);
    if (epi == EPI_ADD) DS_PICK(PRO_NORM, EPI_ADD);
  }
  return QD_ERR_UNSUPPORTED;
}

// q, k, v of T <= 8 tokens from the residual sum: rmsnorm, the product with Wqkv [(H + 2G) d, K], bias, rotation
// of q and k (table rows of ``positions``; pairing 0: elements (2p, 2p+1), 1: (p, p + d/2), then rotary_dim
// must be d), k and v to their cache slots (kv [pages, 2, G, page_size, d]) when write_kv, q to q_out [T, H d].
extern "C" int qd_ds_qkv(const void* W, int K, int T, const float* xf, const float* norm_w, float eps, const float* bias,
                         void* q_out, void* kv, const int* positions, const int* slot_map, const float* cos_t,
                         const float* sin_t, int H, int G, int d, int page_size, int rotary_dim, int pairing,
                         int write_kv, cudaStream_t stream) {
  if (T < 1 || T > 8 || K < 8 || (K & 7) || H < 1 || G < 1 || d < 16 || (d & 15) || !ds_aligned(W)) return QD_ERR_UNSUPPORTED;
  if ((rotary_dim & 1) || rotary_dim > d || (rotary_dim > 0 && (!cos_t || !sin_t || !positions))) return QD_ERR_UNSUPPORTED;
  if (pairing != 0 && pairing != 1) return QD_ERR_UNSUPPORTED;
  if (pairing == 1 && rotary_dim != 0 && rotary_dim != d) return QD_ERR_UNSUPPORTED;
  if (!xf || !norm_w || !q_out || (write_kv && (!kv || !slot_map || page_size < 1))) return QD_ERR_UNSUPPORTED;
  DsShape s;
  if (!ds_shape(K, &s)) return QD_ERR_UNSUPPORTED;
  DsArgs a = {};
  a.W = (const bf16*)W; a.N = (H + 2 * G) * d; a.K = K; a.n_tiles = a.N / 16; a.splits = 1; a.T = T;
  a.xf = xf; a.norm_w = norm_w; a.eps = eps; a.bias = bias;
  a.q_out = (bf16*)q_out; a.kv = (bf16*)kv; a.positions = positions; a.slot_map = slot_map;
  a.cos_t = rotary_dim > 0 ? cos_t : nullptr; a.sin_t = sin_t;
  a.H = H; a.G = G; a.d = d; a.page_size = page_size; a.rotary_half = rotary_dim >> 1;
  a.pairing = rotary_dim > 0 ? pairing : 0; a.write_kv = write_kv;
  const int max_ctas = s.ctas_per_sm * ds_sm_count();
  const int grid = a.n_tiles < max_ctas ? a.n_tiles : max_ctas;
  return ds_launch(ds_gemm_kernel<PRO_NORM, EPI_QKV>, a, s, grid, stream);
}

// The feed-forward of T <= 8 tokens on the residual sum, in place: resid += (silu(h Wg^T) * (h Wu^T)) Wd^T with
// h = rmsnorm(resid).  w_gate_up = [Wg; Wu] of [2F, D], w_down [D, F]; act [T, F] bfloat16, part [splits, T, D]
// float32 and tickets [ceil(D/16)] (zero between launches) are scratch; barrier: two words, zero before first use.
extern "C" int qd_ds_ffn(const void* w_gate_up, const void* w_down, int D, int F, int T, float* resid,
                         const float* norm_w, float eps, void* act, float* part, int splits, unsigned* tickets,
                         unsigned* barrier, cudaStream_t stream) {
  if (T < 1 || T > 8 || D < 8 || (D & 7) || F < 8 || (F & 7) || splits < 1) return QD_ERR_UNSUPPORTED;
  if (!ds_aligned(w_gate_up) || !ds_aligned(w_down) || !ds_aligned(act) || !resid || !norm_w || !barrier) return QD_ERR_UNSUPPORTED;
  if (splits > 1 && (!part || !tickets)) return QD_ERR_UNSUPPORTED;
  const int widest2 = ds_widest_share(F, splits);
  DsShape s;
  if (!ds_shape(D > widest2 ? D : widest2, &s)) return QD_ERR_UNSUPPORTED;
  const int max_ctas = s.ctas_per_sm * ds_sm_count();
  if (splits > max_ctas) return QD_ERR_UNSUPPORTED;
  // every CTA must be resident at the barrier: ask the occupancy calculator, not only the arithmetic above
  if (cudaFuncSetAttribute(ds_ffn_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)s.smem) != cudaSuccess) {
    cudaGetLastError();
    return QD_ERR_UNSUPPORTED;
  }
  int per_sm = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, ds_ffn_kernel, DS_THREADS, s.smem) != cudaSuccess || per_sm < 1) {
    cudaGetLastError();
    return QD_ERR_UNSUPPORTED;
  }
  int grid = (per_sm < s.ctas_per_sm ? per_sm : s.ctas_per_sm) * ds_sm_count();
  const int n_tiles1 = (F + 7) / 8, n_tiles2 = (D + 15) / 16;
  const int useful = n_tiles1 > n_tiles2 * splits ? n_tiles1 : n_tiles2 * splits;
  if (grid > useful) grid = useful;
  if (grid < splits) return QD_ERR_UNSUPPORTED;
  DsArgs a = {};
  a.W = (const bf16*)w_gate_up; a.N = 2 * F; a.K = D; a.n_tiles = n_tiles1; a.splits = 1; a.T = T;
  a.xf = resid; a.norm_w = norm_w; a.eps = eps;
  a.W2 = (const bf16*)w_down; a.N2 = D; a.K2 = F; a.n_tiles2 = n_tiles2; a.splits2 = splits;
  a.h = (bf16*)act; a.ldh = F; a.gbar = barrier;
  a.part = part; a.resid = resid; a.tickets = tickets;
  return ds_launch(ds_ffn_kernel, a, s, grid, stream);
}

QD_DEFINE_WAIT_PROBE(qd_decode_stream_wait_probe, ds_mbar_wait(bar, 0, dead, poll_limit), ds_status_word, 99)

extern "C" int qd_decode_stream_status() {
  int* status = ds_status_word();
  if (!status) return -1;
  int v = 0;
  if (cudaMemcpy(&v, status, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
  if (v) cudaMemset(status, 0, sizeof(int));      // reported once
  return v;
}
