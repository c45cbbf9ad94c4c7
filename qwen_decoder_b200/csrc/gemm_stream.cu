// Few-token contraction as a persistent weight streamer: Y[T, N] = X[T, K] * W[N, K]^T for
// T <= 64 (decode steps), bfloat16 in, float32 accumulation.
//
// A decode step is bound by reading every weight once.  Here a CTA stays on its SM and walks
// a list of work items (16 rows of W x a share of K).  One producer warp keeps a ring of
// shared-memory stages full with bulk asynchronous copies (cp.async.bulk, completion counted
// on an mbarrier per stage): 16 rows of W and the tokens' rows of X for 1024 k per stage (copies of 2 KB: the copy engine is
// bound by the number of copies, 1 KB rows ran a quarter slower), several
// stages in flight per CTA, no registers tied up, and the stream runs on across item boundaries.  Four consumer warps read
// a stage (each a quarter of its k range) with 16-byte shared loads and feed mma.sync
// m16n8k16 with the tokens as the N dimension; the 16-byte operand trick is the one of
// gemm_skinny.cu.  After an item's last stage the four partial sums are added in shared
// memory and the epilogue runs: store (+ bias), split-K partial sums, or SwiGLU.
// The producer starts before the programmatic-dependency wait (weights are written by no
// kernel of the step); the consumers wait before they read the tokens.
//
// Every wait on an mbarrier is bounded: after ST_SPIN_LIMIT polls a warp records an error in
// `status`, marks the CTA dead (no wait of it spins again) and runs on to the end without
// leaving early, so that all warps still meet at every barrier; the host turns a non-zero
// status into an error.
#include "common.cuh"
#include <cstdlib>

#define ST_CONSUMERS 4
#define ST_THREADS ((ST_CONSUMERS + 1) * 32)
#define ST_KC 1024                        // k per stage
#define ST_ROW_BYTES (ST_KC * 2 + 64)     // padded row: 16-byte reads of 8 rows x 4 lanes hit 32 banks once
// a stage holds 16 rows of W and TN*8 token rows of X for the same ST_KC k; stages per CTA are
// chosen so that two CTAs fit on an SM (about 104 KB each) and the L1 keeps nothing it needs
template <int TN> struct StageCfg {
  static constexpr int ROWS = 16 + TN * 8;
  static constexpr int BYTES = ROWS * ST_ROW_BYTES;
  static constexpr int STAGES = TN == 1 ? 2 : (TN == 2 ? 2 : 1);
};
#define ST_SPIN_LIMIT (1u << 24)

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
// true when the phase with the given parity has completed; false after ST_SPIN_LIMIT polls or two seconds (or at
// once when a wait of this CTA has already run out: *dead is then set and nobody waits any more)
__device__ __forceinline__ bool mbar_wait(unsigned long long* bar, unsigned parity, volatile int* dead,
                                          unsigned poll_limit = ST_SPIN_LIMIT) {
  return qd_mbar_wait_bounded(smem_u32(bar), parity, dead, poll_limit, 2000000000ull);
}
__device__ __forceinline__ void bulk_copy(void* dst, const void* src, unsigned bytes, unsigned long long* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mma16816(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                         unsigned b0, unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <int TN, int EPI, typename TO>
__global__ void __launch_bounds__(ST_THREADS)
gemm_stream_kernel(const bf16* __restrict__ W, const bf16* __restrict__ X, long long ldx,
                   const float* __restrict__ bias, TO* __restrict__ out, long long ldo,
                   float* __restrict__ part, int T, int N, int K, int splits, int n_tiles,
                   int* __restrict__ status) {
  constexpr int NST = StageCfg<TN>::STAGES;
  constexpr int STAGE_BYTES = StageCfg<TN>::BYTES;
  extern __shared__ __align__(128) unsigned char smem_raw[];
  unsigned char* stages = smem_raw;                                         // NST x stage
  float* red = reinterpret_cast<float*>(smem_raw + NST * STAGE_BYTES);      // [4][16][TN*8+1]
  __shared__ unsigned long long full_bar[NST], empty_bar[NST];
  __shared__ int dead;   // set when a bounded wait ran out: every warp then runs on without waiting, so that
                         // all of them still meet at every barrier and the kernel ends; the result is void
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    dead = 0;
    for (int s = 0; s < NST; s++) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], ST_CONSUMERS); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  const int n_chunks = (K + ST_KC - 1) / ST_KC;
  const int n_items = n_tiles * splits;
  constexpr int RED_LD = TN * 8 + 1;

  if (warp == ST_CONSUMERS) {
    // ------------------------------------------------------------ producer
    // Weights are written by no kernel of the step: the first NST stages' W rows are requested
    // before the dependency wait, their X rows after it.
    unsigned it = 0;                      // stages issued so far
    bool waited = false;
    for (int item = blockIdx.x; item < n_items; item += gridDim.x) {
      const int tile = item / splits, sp = item - tile * splits;
      const int c_begin = (int)((long long)n_chunks * sp / splits), c_end = (int)((long long)n_chunks * (sp + 1) / splits);
      long long row;                      // the row of W this lane copies (lanes 0..15)
      if (EPI == EPI_SWIGLU) {
        int F = N >> 1, f = tile * 8 + (lane & 7);
        if (f >= F) f = F - 1;
        row = (lane & 8) ? (long long)F + f : f;
      } else {
        row = (long long)tile * 16 + (lane & 15);
        if (row >= N) row = N - 1;
      }
      for (int c = c_begin; c < c_end; c++, it++) {
        const int s = it % NST;
        const unsigned ph = (it / NST) & 1;
        if (it >= (unsigned)NST && !waited) {
          // the ring is full of W requests: now the tokens of the first stages
          pdl_wait();
          waited = true;
          unsigned jt = 0;
          for (int item2 = blockIdx.x; item2 < n_items && jt < (unsigned)NST; item2 += gridDim.x) {
            const int sp2 = item2 % splits;
            const int cb = (int)((long long)n_chunks * sp2 / splits), ce = (int)((long long)n_chunks * (sp2 + 1) / splits);
            for (int c2 = cb; c2 < ce && jt < (unsigned)NST; c2++, jt++) {
              const int k2 = c2 * ST_KC;
              const unsigned rb = (unsigned)(min(ST_KC, K - k2) * 2);
              for (int t = lane; t < T; t += 32)
                bulk_copy(stages + (size_t)jt * STAGE_BYTES + (size_t)(16 + t) * ST_ROW_BYTES, X + (size_t)t * ldx + k2,
                          rb, &full_bar[jt]);
            }
          }
        }
        if (!mbar_wait(&empty_bar[s], ph ^ 1, &dead) && lane == 0) atomicExch(status, 1);
        const int k0 = c * ST_KC;
        const unsigned row_bytes = (unsigned)(min(ST_KC, K - k0) * 2);
        if (lane == 0) mbar_expect_tx(&full_bar[s], row_bytes * (16 + T));
        __syncwarp();
        unsigned char* st = stages + (size_t)s * STAGE_BYTES;
        if (lane < 16) bulk_copy(st + (size_t)lane * ST_ROW_BYTES, W + row * K + k0, row_bytes, &full_bar[s]);
        if (waited)
          for (int t = lane; t < T; t += 32)
            bulk_copy(st + (size_t)(16 + t) * ST_ROW_BYTES, X + (size_t)t * ldx + k0, row_bytes, &full_bar[s]);
      }
    }
    if (!waited) {
      // fewer stages than the ring holds: all W requests are out, now the tokens
      pdl_wait();
      unsigned jt = 0;
      for (int item2 = blockIdx.x; item2 < n_items; item2 += gridDim.x) {
        const int sp2 = item2 % splits;
        const int cb = (int)((long long)n_chunks * sp2 / splits), ce = (int)((long long)n_chunks * (sp2 + 1) / splits);
        for (int c2 = cb; c2 < ce; c2++, jt++) {
          const int k2 = c2 * ST_KC;
          const unsigned rb = (unsigned)(min(ST_KC, K - k2) * 2);
          for (int t = lane; t < T; t += 32)
            bulk_copy(stages + (size_t)jt * STAGE_BYTES + (size_t)(16 + t) * ST_ROW_BYTES, X + (size_t)t * ldx + k2, rb,
                      &full_bar[jt]);
        }
      }
    }
    return;
  }

  // -------------------------------------------------------------- consumers
  const int j = lane & 3, r = lane >> 2;
  unsigned it = 0;
  for (int item = blockIdx.x; item < n_items; item += gridDim.x) {
    const int tile = item / splits, sp = item - tile * splits;
    const int c_begin = (int)((long long)n_chunks * sp / splits), c_end = (int)((long long)n_chunks * (sp + 1) / splits);
    float acc[TN][4];
#pragma unroll
    for (int n = 0; n < TN; n++) acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.f;
    for (int c = c_begin; c < c_end; c++, it++) {
      const int s = it % NST;
      const unsigned ph = (it / NST) & 1;
      if (!mbar_wait(&full_bar[s], ph, &dead) && lane == 0) atomicExch(status, 2);
      const unsigned char* st = stages + (size_t)s * STAGE_BYTES;
      // this warp's quarter of the stage: k-steps of 32 at kq = warp * (ST_KC / 4) + u * 32
      if (TN == 1) {
        // one tile of tokens: every load from shared memory before the first MMA, two chains of MMAs (as
        // xr_stage_mma does it; the token rows lie below the 16 weight rows of the stage)
        constexpr int NU = ST_KC / 32 / ST_CONSUMERS;
        uint4 lo[NU], hi[NU], b[NU];
#pragma unroll
        for (int u = 0; u < NU; u++) {
          const int kq = warp * (ST_KC / ST_CONSUMERS) + u * 32;
          const bool in = c * ST_KC + kq + 8 * j < K;
          const uint4 zero = make_uint4(0, 0, 0, 0);
          const size_t col = (size_t)(kq + 8 * j) * 2;
          lo[u] = in ? *reinterpret_cast<const uint4*>(st + (size_t)r * ST_ROW_BYTES + col) : zero;
          hi[u] = in ? *reinterpret_cast<const uint4*>(st + (size_t)(r + 8) * ST_ROW_BYTES + col) : zero;
          b[u] = in ? *reinterpret_cast<const uint4*>(st + (size_t)(16 + r) * ST_ROW_BYTES + col) : zero;
        }
        float acc2[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int u = 0; u < NU; u += 2) {
          mma16816(acc[0], lo[u].x, hi[u].x, lo[u].y, hi[u].y, b[u].x, b[u].y);
          mma16816(acc2, lo[u + 1].x, hi[u + 1].x, lo[u + 1].y, hi[u + 1].y, b[u + 1].x, b[u + 1].y);
          mma16816(acc[0], lo[u].z, hi[u].z, lo[u].w, hi[u].w, b[u].z, b[u].w);
          mma16816(acc2, lo[u + 1].z, hi[u + 1].z, lo[u + 1].w, hi[u + 1].w, b[u + 1].z, b[u + 1].w);
        }
#pragma unroll
        for (int i = 0; i < 4; i++) acc[0][i] += acc2[i];
      } else
#pragma unroll
      for (int u = 0; u < ST_KC / 32 / ST_CONSUMERS; u++) {
        const int kq = warp * (ST_KC / ST_CONSUMERS) + u * 32;
        if (c * ST_KC + kq >= K) break;                 // the whole k-step lies past K (same for all lanes)
        const bool in = c * ST_KC + kq + 8 * j < K;     // lanes past K feed zeros; every lane runs the MMAs
        const uint4 zero = make_uint4(0, 0, 0, 0);
        const size_t col = (size_t)(kq + 8 * j) * 2;
        uint4 lo = in ? *reinterpret_cast<const uint4*>(st + (size_t)r * ST_ROW_BYTES + col) : zero;
        uint4 hi = in ? *reinterpret_cast<const uint4*>(st + (size_t)(r + 8) * ST_ROW_BYTES + col) : zero;
#pragma unroll
        for (int n = 0; n < TN; n++) {
          // token rows past T were never copied: whatever is there only reaches columns that are not stored
          uint4 b = in ? *reinterpret_cast<const uint4*>(st + (size_t)(16 + n * 8 + r) * ST_ROW_BYTES + col) : zero;
          mma16816(acc[n], lo.x, hi.x, lo.y, hi.y, b.x, b.y);
          mma16816(acc[n], lo.z, hi.z, lo.w, hi.w, b.z, b.w);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty_bar[s]);
    }
    // add the four warps' shares of K and write the item's result
#pragma unroll
    for (int n = 0; n < TN; n++) {
      float* base = red + (size_t)warp * 16 * RED_LD;
      base[r * RED_LD + n * 8 + 2 * j] = acc[n][0];
      base[r * RED_LD + n * 8 + 2 * j + 1] = acc[n][1];
      base[(r + 8) * RED_LD + n * 8 + 2 * j] = acc[n][2];
      base[(r + 8) * RED_LD + n * 8 + 2 * j + 1] = acc[n][3];
    }
    asm volatile("bar.sync 1, %0;" ::"n"(ST_CONSUMERS * 32) : "memory");
    if (EPI == EPI_SWIGLU) {
      const int F = N >> 1;
      for (int idx = threadIdx.x; idx < 8 * TN * 8; idx += ST_CONSUMERS * 32) {
        int row = idx & 7, tok = idx >> 3;
        int f = tile * 8 + row;
        if (tok >= T || f >= F) continue;
        float gate = 0.f, up = 0.f;
#pragma unroll
        for (int w = 0; w < ST_CONSUMERS; w++) {
          gate += red[((size_t)w * 16 + row) * RED_LD + tok];
          up += red[((size_t)w * 16 + row + 8) * RED_LD + tok];
        }
        out[(size_t)tok * ldo + f] = from_float<TO>(gate / (1.0f + expf(-gate)) * up);
      }
    } else {
      for (int idx = threadIdx.x; idx < 16 * TN * 8; idx += ST_CONSUMERS * 32) {
        int row = idx & 15, tok = idx >> 4;
        int n = tile * 16 + row;
        if (tok >= T || n >= N) continue;
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < ST_CONSUMERS; w++) v += red[((size_t)w * 16 + row) * RED_LD + tok];
        if (EPI == EPI_PARTIAL) {
          part[((size_t)sp * T + tok) * N + n] = v;
        } else {
          if (bias) v += bias[n];
          out[(size_t)tok * ldo + n] = from_float<TO>(v);
        }
      }
    }
    asm volatile("bar.sync 1, %0;" ::"n"(ST_CONSUMERS * 32) : "memory");   // red is reused by the next item
  }
  pdl_launch_dependents();
}

// ---------------------------------------------------------------------------------------------
// The same streamer with the tokens RESIDENT in shared memory: for up to 8 tokens and a k range per
// CTA of at most XR_KMAX, or 9 to 16 tokens and a k range of at most XR_KMAX / 2 (TN = 2).  Above, every stage carries the tokens' rows for its k beside the 16 rows
// of W -- half as many bytes again through the copy engine, which is what bounds the stream.  Here a
// CTA keeps ONE share of K for the whole launch (CTA b: share b % splits, tiles b / splits,
// b / splits + grid / splits, ...), copies the tokens' rows for that share once, and its stages
// carry weights only.
#define XR_KMAX 2048
#define XR_ROW_BYTES (XR_KMAX * 2 + 64)
#define XR_STAGES 2
#define XR_STAGE_BYTES (16 * ST_ROW_BYTES)

// One stage of the resident-token kernels for one consumer warp: its quarter of the stage's k (ST_KC / 4), in
// steps of 32.  All loads from shared memory are issued before the first MMA, and the MMAs run as two chains
// that are added at the end: a warp that has its data already (the first stage of a launch, a small product)
// spends its time on latencies, not on arithmetic.  k-steps past K feed zeros.
__device__ __forceinline__ void xr_stage_mma(float (&acc)[4], const unsigned char* st, const unsigned char* xs,
                                             int k_stage, int K, int warp, int j, int r) {
  constexpr int NU = ST_KC / 32 / ST_CONSUMERS;
  uint4 lo[NU], hi[NU], b[NU];
#pragma unroll
  for (int u = 0; u < NU; u++) {
    const int kq = warp * (ST_KC / ST_CONSUMERS) + u * 32;
    const bool in = k_stage + kq + 8 * j < K;
    const uint4 zero = make_uint4(0, 0, 0, 0);
    const size_t col = (size_t)(kq + 8 * j) * 2;
    lo[u] = in ? *reinterpret_cast<const uint4*>(st + (size_t)r * ST_ROW_BYTES + col) : zero;
    hi[u] = in ? *reinterpret_cast<const uint4*>(st + (size_t)(r + 8) * ST_ROW_BYTES + col) : zero;
    // token rows past T were never copied: whatever is there only reaches columns that are not stored
    b[u] = in ? *reinterpret_cast<const uint4*>(xs + (size_t)r * XR_ROW_BYTES + col) : zero;
  }
  float acc2[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int u = 0; u < NU; u += 2) {
    mma16816(acc, lo[u].x, hi[u].x, lo[u].y, hi[u].y, b[u].x, b[u].y);
    mma16816(acc2, lo[u + 1].x, hi[u + 1].x, lo[u + 1].y, hi[u + 1].y, b[u + 1].x, b[u + 1].y);
    mma16816(acc, lo[u].z, hi[u].z, lo[u].w, hi[u].w, b[u].z, b[u].w);
    mma16816(acc2, lo[u + 1].z, hi[u + 1].z, lo[u + 1].w, hi[u + 1].w, b[u + 1].z, b[u + 1].w);
  }
#pragma unroll
  for (int i = 0; i < 4; i++) acc[i] += acc2[i];
}


// The same for 9 to 16 tokens (two token tiles of the MMA): the resident rows are half as long (a share of K of
// at most XR_KMAX / 2), so that the tokens take the same shared memory and two CTAs still fit on an SM.  The
// loads go out in two halves of the warp's k range (registers); each half feeds two chains per token tile.
#define XR_ROW_BYTES2 (XR_KMAX / 2 * 2 + 64)
__device__ __forceinline__ void xr_stage_mma2(float (&acc)[2][4], const unsigned char* st, const unsigned char* xs,
                                              int k_stage, int K, int warp, int j, int r) {
  constexpr int NU = ST_KC / 32 / ST_CONSUMERS, NH = NU / 2;
  float acc2[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
  for (int h = 0; h < 2; h++) {
    uint4 lo[NH], hi[NH], b0[NH], b1[NH];
#pragma unroll
    for (int u = 0; u < NH; u++) {
      const int kq = warp * (ST_KC / ST_CONSUMERS) + (h * NH + u) * 32;
      const bool in = k_stage + kq + 8 * j < K;
      const uint4 zero = make_uint4(0, 0, 0, 0);
      const size_t col = (size_t)(kq + 8 * j) * 2;
      lo[u] = in ? *reinterpret_cast<const uint4*>(st + (size_t)r * ST_ROW_BYTES + col) : zero;
      hi[u] = in ? *reinterpret_cast<const uint4*>(st + (size_t)(r + 8) * ST_ROW_BYTES + col) : zero;
      b0[u] = in ? *reinterpret_cast<const uint4*>(xs + (size_t)r * XR_ROW_BYTES2 + col) : zero;
      b1[u] = in ? *reinterpret_cast<const uint4*>(xs + (size_t)(r + 8) * XR_ROW_BYTES2 + col) : zero;
    }
#pragma unroll
    for (int u = 0; u < NH; u += 2) {
      mma16816(acc[0], lo[u].x, hi[u].x, lo[u].y, hi[u].y, b0[u].x, b0[u].y);
      mma16816(acc[1], lo[u].x, hi[u].x, lo[u].y, hi[u].y, b1[u].x, b1[u].y);
      mma16816(acc2[0], lo[u + 1].x, hi[u + 1].x, lo[u + 1].y, hi[u + 1].y, b0[u + 1].x, b0[u + 1].y);
      mma16816(acc2[1], lo[u + 1].x, hi[u + 1].x, lo[u + 1].y, hi[u + 1].y, b1[u + 1].x, b1[u + 1].y);
      mma16816(acc[0], lo[u].z, hi[u].z, lo[u].w, hi[u].w, b0[u].z, b0[u].w);
      mma16816(acc[1], lo[u].z, hi[u].z, lo[u].w, hi[u].w, b1[u].z, b1[u].w);
      mma16816(acc2[0], lo[u + 1].z, hi[u + 1].z, lo[u + 1].w, hi[u + 1].w, b0[u + 1].z, b0[u + 1].w);
      mma16816(acc2[1], lo[u + 1].z, hi[u + 1].z, lo[u + 1].w, hi[u + 1].w, b1[u + 1].z, b1[u + 1].w);
    }
  }
#pragma unroll
  for (int n = 0; n < 2; n++)
#pragma unroll
    for (int i = 0; i < 4; i++) acc[n][i] += acc2[n][i];
}

template <int TN, int EPI, typename TO>
__global__ void __launch_bounds__(ST_THREADS, 2)
gemm_stream_xres_kernel(const bf16* __restrict__ W, const bf16* __restrict__ X, long long ldx,
                        const float* __restrict__ bias, TO* __restrict__ out, long long ldo,
                        float* __restrict__ part, int T, int N, int K, int splits, int n_tiles,
                        int* __restrict__ status) {
  constexpr int NST = XR_STAGES;
  extern __shared__ __align__(128) unsigned char smem_raw[];
  unsigned char* stages = smem_raw;                                               // NST x 16 rows of W
  constexpr int XROW = TN == 1 ? XR_ROW_BYTES : XR_ROW_BYTES2;
  unsigned char* xres = smem_raw + NST * XR_STAGE_BYTES;                          // TN * 8 token rows
  float* red = reinterpret_cast<float*>(xres + TN * 8 * XROW);                    // [4][16][TN * 8 + 1]
  __shared__ unsigned long long full_bar[NST], empty_bar[NST], x_bar;
  __shared__ int dead;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    dead = 0;
    for (int s = 0; s < NST; s++) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], ST_CONSUMERS); }
    mbar_init(&x_bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  pdl_launch_dependents();      // the next kernel's CTAs may start where there is room; they wait for this grid's end
  const int n_chunks = (K + ST_KC - 1) / ST_KC;
  const int stride = (int)gridDim.x / splits;                 // CTAs per share of K (the host made it >= 1)
  const int sp = (int)blockIdx.x % splits;
  const int first = (int)blockIdx.x / splits;
  const bool idle = first >= stride;
  const int c_begin = (int)((long long)n_chunks * sp / splits), c_end = (int)((long long)n_chunks * (sp + 1) / splits);
  const int k_begin = c_begin * ST_KC, k_end = min(K, c_end * ST_KC);
  constexpr int RED_LD = TN * 8 + 1;

  if (warp == ST_CONSUMERS) {
    // ------------------------------------------------------------ producer
    if (idle) { pdl_wait(); return; }
    unsigned it = 0;
    bool waited = false;
    auto tokens = [&]() {
      // after the dependency wait: the tokens' rows for this CTA's share of K, once
      pdl_wait();
      waited = true;
      const unsigned xb = (unsigned)((k_end - k_begin) * 2);
      if (lane == 0) mbar_expect_tx(&x_bar, xb * T);
      __syncwarp();
      for (int t = lane; t < T; t += 32)
        bulk_copy(xres + (size_t)t * XROW, X + (size_t)t * ldx + k_begin, xb, &x_bar);
    };
    for (int tile = first; tile < n_tiles; tile += stride) {
      long long row;                      // the row of W this lane copies (lanes 0..15)
      if (EPI == EPI_SWIGLU) {
        int F = N >> 1, f = tile * 8 + (lane & 7);
        if (f >= F) f = F - 1;
        row = (lane & 8) ? (long long)F + f : f;
      } else {
        row = (long long)tile * 16 + (lane & 15);
        if (row >= N) row = N - 1;
      }
      for (int c = c_begin; c < c_end; c++, it++) {
        const int s = it % NST;
        const unsigned ph = (it / NST) & 1;
        if (it >= (unsigned)NST && !waited) tokens();        // the ring is full of W requests
        if (!mbar_wait(&empty_bar[s], ph ^ 1, &dead) && lane == 0) atomicExch(status, 1);
        const int k0 = c * ST_KC;
        const unsigned row_bytes = (unsigned)(min(ST_KC, K - k0) * 2);
        if (lane == 0) mbar_expect_tx(&full_bar[s], row_bytes * 16);
        __syncwarp();
        if (lane < 16)
          bulk_copy(stages + (size_t)s * XR_STAGE_BYTES + (size_t)lane * ST_ROW_BYTES, W + row * K + k0, row_bytes,
                    &full_bar[s]);
      }
    }
    if (!waited) tokens();
    return;
  }

  // -------------------------------------------------------------- consumers
  if (idle) { pdl_launch_dependents(); return; }
  const int j = lane & 3, r = lane >> 2;
  unsigned it = 0;
  bool have_x = false;
  for (int tile = first; tile < n_tiles; tile += stride) {
    float acc[TN][4];
#pragma unroll
    for (int n = 0; n < TN; n++) acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.f;
    for (int c = c_begin; c < c_end; c++, it++) {
      const int s = it % NST;
      const unsigned ph = (it / NST) & 1;
      if (!mbar_wait(&full_bar[s], ph, &dead) && lane == 0) atomicExch(status, 2);
      if (!have_x) {
        if (!mbar_wait(&x_bar, 0, &dead) && lane == 0) atomicExch(status, 2);
        have_x = true;
      }
      const unsigned char* st = stages + (size_t)s * XR_STAGE_BYTES;
      const unsigned char* xs = xres + (size_t)(c - c_begin) * ST_KC * 2;
      if constexpr (TN == 1) xr_stage_mma(acc[0], st, xs, c * ST_KC, K, warp, j, r);
      else xr_stage_mma2(acc, st, xs, c * ST_KC, K, warp, j, r);
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty_bar[s]);
    }
    float* base = red + (size_t)warp * 16 * RED_LD;
#pragma unroll
    for (int n = 0; n < TN; n++) {
      base[r * RED_LD + n * 8 + 2 * j] = acc[n][0];
      base[r * RED_LD + n * 8 + 2 * j + 1] = acc[n][1];
      base[(r + 8) * RED_LD + n * 8 + 2 * j] = acc[n][2];
      base[(r + 8) * RED_LD + n * 8 + 2 * j + 1] = acc[n][3];
    }
    asm volatile("bar.sync 1, %0;" ::"n"(ST_CONSUMERS * 32) : "memory");
    if (EPI == EPI_SWIGLU) {
      const int F = N >> 1;
      for (int idx = threadIdx.x; idx < 8 * TN * 8; idx += ST_CONSUMERS * 32) {
        int row = idx & 7, tok = idx >> 3;
        int f = tile * 8 + row;
        if (tok >= T || f >= F) continue;
        float gate = 0.f, up = 0.f;
#pragma unroll
        for (int w = 0; w < ST_CONSUMERS; w++) {
          gate += red[((size_t)w * 16 + row) * RED_LD + tok];
          up += red[((size_t)w * 16 + row + 8) * RED_LD + tok];
        }
        out[(size_t)tok * ldo + f] = from_float<TO>(gate / (1.0f + expf(-gate)) * up);
      }
    } else {
      for (int idx = threadIdx.x; idx < 16 * TN * 8; idx += ST_CONSUMERS * 32) {
        int row = idx & 15, tok = idx >> 4;
        int n = tile * 16 + row;
        if (tok >= T || n >= N) continue;
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < ST_CONSUMERS; w++) v += red[((size_t)w * 16 + row) * RED_LD + tok];
        if (EPI == EPI_PARTIAL) {
          part[((size_t)sp * T + tok) * N + n] = v;
        } else {
          if (bias) v += bias[n];
          out[(size_t)tok * ldo + n] = from_float<TO>(v);
        }
      }
    }
    asm volatile("bar.sync 1, %0;" ::"n"(ST_CONSUMERS * 32) : "memory");   // red is reused by the next tile
  }
  pdl_launch_dependents();
}

// ---------------------------------------------------------------------------------------------
// The feed-forward of a few tokens as ONE launch of the resident-token streamer: gate/up with the SwiGLU
// epilogue, then the down projection as split-K partial sums.  A CTA's share of the down projection's K needs
// those columns of h, so it waits until the row tiles that write them are counted (a counter per chunk of
// ST_KC columns) -- but its producer warp does not: it goes on filling the stages with the down projection's
// first weights meanwhile, so the second product starts with its pipeline full.  All CTAs are resident (the
// host launches no more than fit); the wait's spin is bounded like every other wait.
#define FFN_SYNC_WORDS 64
struct FfnArgs {
  const bf16* w1; const bf16* x1; long long ldx1; int N1, K1, n_tiles1;        // [2F, D], tokens [T, D]
  bf16* h; long long ldh;                                                       // [T, F]
  const bf16* w2; int N2, K2, n_tiles2, splits2; float* part;                   // [D, F] -> [splits2, T, D]
  int T;
  unsigned* gbar;            // FFN_SYNC_WORDS words, zero before first use: per chunk of ST_KC columns of h the
                             // row tiles of the first product that are written; last word: CTAs past their wait
  int* status;
  long long* timeline;       // null, or 8 nanosecond stamps per CTA (for measurements): start, tokens there, first tile
                             // done, first product done, wait for h over, h there, second product done
};

__device__ __forceinline__ void ffn_stamp(const FfnArgs& a, int i) {
  if (a.timeline) {
    long long now;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
    a.timeline[(size_t)blockIdx.x * 8 + i] = now;
  }
}

#define FFN_THREADS (ST_THREADS + 32)       // consumers, the producer warp, and a warp that tells and waits
__global__ void __launch_bounds__(FFN_THREADS)
ffn_stream_kernel(const FfnArgs a) {
  constexpr int NST = XR_STAGES;
  extern __shared__ __align__(128) unsigned char smem_raw[];
  unsigned char* stages = smem_raw;
  unsigned char* xres = smem_raw + NST * XR_STAGE_BYTES;
  float* red = reinterpret_cast<float*>(xres + 8 * XR_ROW_BYTES);
  __shared__ unsigned long long full_bar[NST], empty_bar[NST], x_bar;
  __shared__ int dead;
  __shared__ unsigned tiles_written;       // row tiles of the first product whose columns of h this CTA has written
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    dead = 0;
    for (int s = 0; s < NST; s++) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], ST_CONSUMERS); }
    mbar_init(&x_bar, 1);
    tiles_written = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  if (threadIdx.x == 0) ffn_stamp(a, 0);

  const int T = a.T;
  const int F = a.N1 >> 1;
  // phase 1: every CTA walks tiles b, b + grid, ... over the whole K1 (at most XR_KMAX)
  const int chunks1 = (a.K1 + ST_KC - 1) / ST_KC;
  // phase 2: CTA b keeps share b % splits2 of K2 and walks tiles b / splits2, + grid / splits2, ...
  const int chunks2 = (a.K2 + ST_KC - 1) / ST_KC;
  const int stride2 = (int)gridDim.x / a.splits2;
  const int sp2 = (int)blockIdx.x % a.splits2;
  const int first2 = (int)blockIdx.x / a.splits2;
  const bool idle2 = first2 >= stride2;
  const int cb2 = (int)((long long)chunks2 * sp2 / a.splits2), ce2 = (int)((long long)chunks2 * (sp2 + 1) / a.splits2);
  const int k2_begin = cb2 * ST_KC, k2_end = min(a.K2, ce2 * ST_KC);
  constexpr int RED_LD = 9;

  if (warp == ST_CONSUMERS) {
    // ------------------------------------------------------------ producer
    unsigned it = 0;
    bool waited = false;
    auto tokens1 = [&]() {
      pdl_wait();
      waited = true;
      const unsigned xb = (unsigned)(a.K1 * 2);
      if (lane == 0) mbar_expect_tx(&x_bar, xb * T);
      __syncwarp();
      for (int t = lane; t < T; t += 32) bulk_copy(xres + (size_t)t * XR_ROW_BYTES, a.x1 + (size_t)t * a.ldx1, xb, &x_bar);
    };
    auto weights = [&](const bf16* W, long long row, int K, int c) {
      const int s = it % NST;
      const unsigned ph = (it / NST) & 1;
      if (!mbar_wait(&empty_bar[s], ph ^ 1, &dead) && lane == 0) atomicExch(a.status, 1);
      const int k0 = c * ST_KC;
      const unsigned row_bytes = (unsigned)(min(ST_KC, K - k0) * 2);
      if (lane == 0) mbar_expect_tx(&full_bar[s], row_bytes * 16);
      __syncwarp();
      if (lane < 16)
        bulk_copy(stages + (size_t)s * XR_STAGE_BYTES + (size_t)lane * ST_ROW_BYTES, W + row * K + k0, row_bytes, &full_bar[s]);
      it++;
    };
    for (int tile = blockIdx.x; tile < a.n_tiles1; tile += gridDim.x) {
      int f = tile * 8 + (lane & 7);
      if (f >= F) f = F - 1;
      const long long row = (lane & 8) ? (long long)F + f : f;
      for (int c = 0; c < chunks1; c++) {
        if (it >= (unsigned)NST && !waited) tokens1();
        weights(a.w1, row, a.K1, c);
      }
    }
    if (!waited) tokens1();
    // the down projection's weights follow at once (the stages fill while the consumers wait for its tokens, h:
    // the warp below fetches those as soon as they are written)
    if (!idle2) {
      for (int tile = first2; tile < a.n_tiles2; tile += stride2) {
        long long row = (long long)tile * 16 + (lane & 15);
        if (row >= a.N2) row = a.N2 - 1;
        for (int c = cb2; c < ce2; c++) weights(a.w2, row, a.K2, c);
      }
    }
    return;
  }

  if (warp == ST_CONSUMERS + 1) {
    // ------------------------------------------------------------ the warp that tells and waits
    // After each row tile of the first product it counts the tile for the chunk of ST_KC columns of h it lies in
    // (a fence, then a reduction: no consumer waits for either).  The second product needs columns [k2_begin,
    // k2_end) of h: the warp waits until every tile that writes into them is counted -- not for the whole grid:
    // tiles are walked in the order of h's columns, so all but the last chunks are complete while some CTAs still
    // work on their last tile -- and lets the producer fetch them.
    if (lane != 0) return;
    unsigned n = 0;
    for (int tile = blockIdx.x; tile < a.n_tiles1; tile += gridDim.x, n++) {
      // wait for the consumers' count in shared memory (it may be several tiles ahead); bounded like every wait
      bool seen = false;
      for (unsigned spin = 0; spin < (1u << 24) && !dead; spin++) {
        if (*(volatile unsigned*)&tiles_written > n) { seen = true; break; }
        __nanosleep(64);
      }
      if (!seen && !dead) { dead = 1; atomicExch(a.status, 5); }
      __threadfence();
      asm volatile("red.relaxed.gpu.global.add.u32 [%0], 1;" ::"l"(a.gbar + (tile * 8) / ST_KC) : "memory");
    }
    if (!idle2 && !dead) {
      unsigned long long start = 0;
      for (int c = cb2; c < ce2 && !dead; c++) {
        const unsigned target = (unsigned)(min(ST_KC, a.K2 - c * ST_KC) / 8);
        bool ok = false;
        for (unsigned spin = 0; spin < (1u << 26); spin++) {
          unsigned v;
          asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(a.gbar + c) : "memory");
          if (v == target) { ok = true; break; }
          if ((spin & 1023) == 1023) {
            unsigned long long now;
            asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
            if (start == 0) start = now;
            else if (now - start > 2000000000ull) break;
          }
        }
        if (!ok) { dead = 1; atomicExch(a.status, 4); }
      }
    }
    ffn_stamp(a, 4);
    if (!idle2) {
      // this CTA's consumers are done with the first product's tokens (their last tile is counted above): h takes
      // their place.  h was written by ordinary stores of other CTAs, the copy reads it through the async proxy
      asm volatile("fence.proxy.async;" ::: "memory");
      const unsigned xb = (unsigned)((k2_end - k2_begin) * 2);
      mbar_expect_tx(&x_bar, xb * T);
      for (int t = 0; t < T; t++)
        bulk_copy(xres + (size_t)t * XR_ROW_BYTES, a.h + (size_t)t * a.ldh + k2_begin, xb, &x_bar);
    }
    __threadfence();
    // the last CTA past its wait puts the words back to zero for the next launch: every CTA has counted its
    // tiles before it waited, and counts itself here after a fence
    if (atomicAdd(a.gbar + FFN_SYNC_WORDS - 1, 1u) == gridDim.x - 1) {
      __threadfence();
      for (int c = 0; c < FFN_SYNC_WORDS; c++) a.gbar[c] = 0;
    }
    return;
  }

  // -------------------------------------------------------------- consumers
  const int j = lane & 3, r = lane >> 2;
  unsigned it = 0;
  auto stage_mma = [&](float (&acc)[4], int K, int c, int c_first) {
    const int s = it % NST;
    const unsigned ph = (it / NST) & 1;
    if (!mbar_wait(&full_bar[s], ph, &dead) && lane == 0) atomicExch(a.status, 2);
    const unsigned char* st = stages + (size_t)s * XR_STAGE_BYTES;
    const unsigned char* xs = xres + (size_t)(c - c_first) * ST_KC * 2;
    xr_stage_mma(acc, st, xs, c * ST_KC, K, warp, j, r);
    __syncwarp();
    if (lane == 0) mbar_arrive(&empty_bar[s]);
    it++;
  };
  auto to_red = [&](const float (&acc)[4]) {
    float* base = red + (size_t)warp * 16 * RED_LD;
    base[r * RED_LD + 2 * j] = acc[0];
    base[r * RED_LD + 2 * j + 1] = acc[1];
    base[(r + 8) * RED_LD + 2 * j] = acc[2];
    base[(r + 8) * RED_LD + 2 * j + 1] = acc[3];
    asm volatile("bar.sync 1, %0;" ::"n"(ST_CONSUMERS * 32) : "memory");
  };
  // ---- phase 1: gate, up, SwiGLU
  bool have_x = false;
  for (int tile = blockIdx.x; tile < a.n_tiles1; tile += gridDim.x) {
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int c = 0; c < chunks1; c++) {
      if (!have_x) {
        if (!mbar_wait(&x_bar, 0, &dead) && lane == 0) atomicExch(a.status, 2);
        have_x = true;
        if (threadIdx.x == 0) ffn_stamp(a, 1);
      }
      stage_mma(acc, a.K1, c, 0);
    }
    to_red(acc);
    for (int idx = threadIdx.x; idx < 8 * 8; idx += ST_CONSUMERS * 32) {
      int row = idx & 7, tok = idx >> 3;
      int f = tile * 8 + row;
      if (tok >= T || f >= F) continue;
      float gate = 0.f, up = 0.f;
#pragma unroll
      for (int w = 0; w < ST_CONSUMERS; w++) {
        gate += red[((size_t)w * 16 + row) * RED_LD + tok];
        up += red[((size_t)w * 16 + row + 8) * RED_LD + tok];
      }
      a.h[(size_t)tok * a.ldh + f] = __float2bfloat16_rn(gate / (1.0f + expf(-gate)) * up);
    }
    asm volatile("bar.sync 1, %0;" ::"n"(ST_CONSUMERS * 32) : "memory");
    // this tile's 8 columns of h are written (by the threads that met at the barrier above): the telling warp
    // makes that known to the other CTAs, so that no consumer waits for a fence
    if (threadIdx.x == 0) {
      __threadfence_block();
      *(volatile unsigned*)&tiles_written = tiles_written + 1;
      if (tile == (int)blockIdx.x) ffn_stamp(a, 2);
    }
  }
  if (threadIdx.x == 0) ffn_stamp(a, 3);
  // ---- phase 2: down projection, partial sums of this CTA's share of K
  if (!idle2) {
    if (!mbar_wait(&x_bar, 1, &dead) && lane == 0) atomicExch(a.status, 2);
    if (threadIdx.x == 0) ffn_stamp(a, 5);
    for (int tile = first2; tile < a.n_tiles2; tile += stride2) {
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
      for (int c = cb2; c < ce2; c++) stage_mma(acc, a.K2, c, cb2);
      to_red(acc);
      for (int idx = threadIdx.x; idx < 16 * 8; idx += ST_CONSUMERS * 32) {
        int row = idx & 15, tok = idx >> 4;
        int n = tile * 16 + row;
        if (tok >= T || n >= a.N2) continue;
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < ST_CONSUMERS; w++) v += red[((size_t)w * 16 + row) * RED_LD + tok];
        a.part[((size_t)sp2 * T + tok) * a.N2 + n] = v;
      }
      asm volatile("bar.sync 1, %0;" ::"n"(ST_CONSUMERS * 32) : "memory");
    }
  }
  if (threadIdx.x == 0) ffn_stamp(a, 6);
  pdl_launch_dependents();
}

static int* g_status[64];   // per device: one int of device memory for the kernels' error status

static int* status_word() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  if (!g_status[dev]) {
    int* p = nullptr;
    if (cudaMalloc(&p, sizeof(int)) != cudaSuccess) return nullptr;
    cudaMemset(p, 0, sizeof(int));
    g_status[dev] = p;
  }
  return g_status[dev];
}

// The resident-token form: up to 8 tokens with every share of K at most XR_KMAX wide, or 9 to 16 tokens with
// shares of at most XR_KMAX / 2; at least one CTA per share.
static bool xres_fits(int T, int K, int splits, int max_ctas) {
  if (T > 16 || splits > max_ctas) return false;
  const int widest = T <= 8 ? XR_KMAX : XR_KMAX / 2;
  const int n_chunks = (K + ST_KC - 1) / ST_KC;
  for (int sp = 0; sp < splits; sp++) {
    int cb = (int)((long long)n_chunks * sp / splits), ce = (int)((long long)n_chunks * (sp + 1) / splits);
    if ((ce - cb) * ST_KC > widest) return false;
  }
  return true;
}

template <int TN>
static int launch_stream_xres(const bf16* W, const bf16* X, long long ldx, const float* bias, void* out, int out_dtype,
                              long long ldo, float* part, int T, int N, int K, int splits, int epi, int max_ctas,
                              cudaStream_t stream) {
  int* status = status_word();
  if (!status) return QD_ERR_UNSUPPORTED;
  int n_tiles = epi == EPI_SWIGLU ? (N / 2 + 7) / 8 : (N + 15) / 16;
  // CTAs per share of K: no more than there are tiles, a multiple of `splits` in all
  int per_share = max_ctas / splits;
  if (per_share > n_tiles) per_share = n_tiles;
  int grid = per_share * splits;
  size_t smem = (size_t)XR_STAGES * XR_STAGE_BYTES + (size_t)TN * 8 * (TN == 1 ? XR_ROW_BYTES : XR_ROW_BYTES2) +
                (size_t)ST_CONSUMERS * 16 * (TN * 8 + 1) * sizeof(float);
#define LAUNCH(E, TO)                                                                                            \
  do {                                                                                                           \
    cudaFuncSetAttribute(gemm_stream_xres_kernel<TN, E, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    qd_launch(gemm_stream_xres_kernel<TN, E, TO>, dim3(grid), dim3(ST_THREADS), smem, stream, W, X, ldx, bias,       \
              (TO*)out, ldo, part, T, N, K, splits, n_tiles, status);                                            \
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

template <int TN>
static int launch_stream(const bf16* W, const bf16* X, long long ldx, const float* bias, void* out, int out_dtype,
                         long long ldo, float* part, int T, int N, int K, int splits, int epi, int max_ctas,
                         cudaStream_t stream) {
  int* status = status_word();
  if (!status) return QD_ERR_UNSUPPORTED;
  int n_tiles = epi == EPI_SWIGLU ? (N / 2 + 7) / 8 : (N + 15) / 16;
  int n_items = n_tiles * splits;
  int grid = n_items < max_ctas ? n_items : max_ctas;
  size_t smem = (size_t)StageCfg<TN>::STAGES * StageCfg<TN>::BYTES + (size_t)ST_CONSUMERS * 16 * (TN * 8 + 1) * sizeof(float);
#define LAUNCH(E, TO)                                                                                       \
  do {                                                                                                      \
    cudaFuncSetAttribute(gemm_stream_kernel<TN, E, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    qd_launch(gemm_stream_kernel<TN, E, TO>, dim3(grid), dim3(ST_THREADS), smem, stream, W, X, ldx, bias,   \
              (TO*)out, ldo, part, T, N, K, splits, n_tiles, status);                                       \
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

// Arguments as qd_gemm_skinny (gemm_skinny.cu); max_ctas bounds the persistent grid (two per SM is
// a good value).  K a multiple of 8, W and X 16-byte aligned, ldx a multiple of 8, splits <= ceil(K / 1024).
extern "C" int qd_gemm_stream(const void* W, const void* X, long long ldx, const float* bias, void* out,
                              int out_dtype, long long ldo, float* part, int T, int N, int K, int splits,
                              int epi, int max_ctas, cudaStream_t stream) {
  if (T <= 0 || N <= 0) return 0;
  if (T > 64 || K <= 0 || K % 8 != 0 || ldx % 8 != 0 || splits < 1 || max_ctas < 1) return QD_ERR_UNSUPPORTED;
  if (splits > (K + ST_KC - 1) / ST_KC) return QD_ERR_UNSUPPORTED;
  if (((uintptr_t)W & 15) || ((uintptr_t)X & 15)) return QD_ERR_UNSUPPORTED;
  if (epi == EPI_SWIGLU && (N & 1)) return QD_ERR_UNSUPPORTED;
  if (epi == EPI_PARTIAL && !part) return QD_ERR_UNSUPPORTED;
  if (epi != EPI_PARTIAL && splits != 1) return QD_ERR_UNSUPPORTED;
  const bf16* w = (const bf16*)W;
  const bf16* x = (const bf16*)X;
  if (xres_fits(T, K, splits, max_ctas))
    return T <= 8 ? launch_stream_xres<1>(w, x, ldx, bias, out, out_dtype, ldo, part, T, N, K, splits, epi, max_ctas, stream)
                  : launch_stream_xres<2>(w, x, ldx, bias, out, out_dtype, ldo, part, T, N, K, splits, epi, max_ctas, stream);
  if (T <= 8) return launch_stream<1>(w, x, ldx, bias, out, out_dtype, ldo, part, T, N, K, splits, epi, max_ctas, stream);
  if (T <= 16) return launch_stream<2>(w, x, ldx, bias, out, out_dtype, ldo, part, T, N, K, splits, epi, max_ctas, stream);
  if (T <= 32) return launch_stream<4>(w, x, ldx, bias, out, out_dtype, ldo, part, T, N, K, splits, epi, max_ctas, stream);
  return launch_stream<8>(w, x, ldx, bias, out, out_dtype, ldo, part, T, N, K, splits, epi, max_ctas, stream);
}

// The feed-forward of up to 8 tokens in one launch: h = silu(x Wg^T) * (x Wu^T) (w1 = [Wg; Wu], [2F, D]) and
// part[s] = partial sums of h W2^T over `splits2` shares of F.  `gbar`: 64 zeroed words of device memory that
// stay with the caller (the kernel leaves them zero for the next launch).  Refuses what it cannot take
// (more than 8 tokens, D above 2,048, a share of F wider than 2,048, more CTAs than fit on the device at once).
extern "C" int qd_ffn_stream(const void* w1, const void* x, long long ldx, void* h, long long ldh, const void* w2,
                             float* part, int T, int D, int F, int splits2, unsigned* gbar, int max_ctas,
                             long long* timeline, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (T > 8 || D <= 0 || F <= 0 || D % 8 != 0 || F % 8 != 0 || ldx % 8 != 0 || ldh % 8 != 0 || D > XR_KMAX ||
      splits2 < 1 || !gbar || !part || (F + ST_KC - 1) / ST_KC > FFN_SYNC_WORDS - 1)
    return QD_ERR_UNSUPPORTED;
  if (((uintptr_t)w1 & 15) || ((uintptr_t)w2 & 15) || ((uintptr_t)x & 15) || ((uintptr_t)h & 15)) return QD_ERR_UNSUPPORTED;
  if (!xres_fits(T, F, splits2, max_ctas)) return QD_ERR_UNSUPPORTED;
  int* status = status_word();
  if (!status) return QD_ERR_UNSUPPORTED;
  const size_t smem = (size_t)XR_STAGES * XR_STAGE_BYTES + (size_t)8 * XR_ROW_BYTES + (size_t)ST_CONSUMERS * 16 * 9 * sizeof(float);
  if (cudaFuncSetAttribute(ffn_stream_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
    cudaGetLastError();
    return QD_ERR_UNSUPPORTED;
  }
  // every CTA waits for every other one: no more CTAs than the device holds at once
  int per_sm = 0, dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, ffn_stream_kernel, FFN_THREADS, smem) != cudaSuccess || per_sm < 1) {
    cudaGetLastError();
    return QD_ERR_UNSUPPORTED;
  }
  FfnArgs a;
  a.w1 = (const bf16*)w1; a.x1 = (const bf16*)x; a.ldx1 = ldx; a.N1 = 2 * F; a.K1 = D; a.n_tiles1 = (F + 7) / 8;
  a.h = (bf16*)h; a.ldh = ldh;
  a.w2 = (const bf16*)w2; a.N2 = D; a.K2 = F; a.n_tiles2 = (D + 15) / 16; a.splits2 = splits2; a.part = part;
  a.T = T; a.gbar = gbar; a.status = status; a.timeline = timeline;
  int grid = per_sm * sms;
  if (grid > max_ctas) grid = max_ctas;
  if (grid > a.n_tiles1) grid = a.n_tiles1;
  if (grid < splits2) return QD_ERR_UNSUPPORTED;
  qd_launch(ffn_stream_kernel, dim3(grid), dim3(FFN_THREADS), smem, stream, a);
  return qd_last_error();
}

// 0 if no kernel of this library has recorded a bounded-wait expiry on the current device
// (1: producer gave up waiting for a free stage, 2: a consumer gave up waiting for data).  Synchronises.
QD_DEFINE_WAIT_PROBE(qd_gemm_stream_wait_probe, mbar_wait(bar, 0, dead, poll_limit), status_word, 99)

extern "C" int qd_gemm_stream_status() {
  int* status = status_word();
  if (!status) return -1;
  int v = 0;
  if (cudaMemcpy(&v, status, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
  if (v) cudaMemset(status, 0, sizeof(int));      // reported once
  return v;
}
