// Paged prefill attention on the fifth-generation tensor cores: S = Q K^T and O = P V by tcgen05.mma with
// the accumulators in tensor memory, K and V tiles fetched from the cache pages by TMA tensor copies
// (128-byte swizzle), float32 online softmax by one thread per row.
//
// A CTA takes 128 rows = (128 / gs) tokens x the gs query heads of one KV head (as attention_flash.cu
// does with 64 or 128 rows), and walks key tiles of 128 through the request's block table.  With TPR softmax
// threads per row (2 here; 4 was measured 4 % slower at head size 128) the warps are:
//   0..4 TPR-1  softmax: TPR threads per row (= TMEM lane), each for 128 / TPR keys and d / TPR output columns:
//            each writes its share of the Q row into tensor memory once, then per key tile loads its share of S
//            from tensor memory in one go, scales, masks, shares the row maximum through shared memory and
//            writes P as bfloat16 back into tensor memory over the scores it has just read (two bfloat16 per
//            column).  The output rows stay in tensor memory, where the products accumulate; a row's sum and
//            output are scaled down only when its maximum has grown by more than 2^8 since the reference of its
//            exponentials (then the thread waits for the product in flight first), and once at the end by 1/sum
//   4 TPR    producer of K, 4 TPR + 1 producer of V: per key tile, 16-key boxes (two 64-column halves each)
//            from the pages; each reads the page numbers of the next tile while this one's copies fly.  A stage
//            holds K of tile j + 2 and V of tile j under one barrier: what the MMA thread reads in its step j
//   4 TPR+2  issues the MMAs (one thread): O += P V of tile j (P is the A operand from tensor memory, V MN-major
//            in shared memory: its rows are keys, the contraction dimension), then S = Q K^T of tile j + 2 (Q the
//            A operand from tensor memory, K K-major in shared memory) into the columns P of tile j was read
//            from: the tensor cores run a thread's MMAs in the order it issued them.  The scores of tile j + 1
//            are complete by then, so the softmax threads never wait for them.  With both A operands in tensor
//            memory an MMA reads 4 KB of shared memory, not 8
// Tensor memory: columns 0..255 the two S/P buffers, 256..383 O, 384..447 Q.  Shared memory: 3 stages of K and V.
// Formulas: gpu_kernels.cu:223-311 of the reference (scores q.k / sqrt(d), causal, softmax, weighted sum).
// Keys past a row's position are masked on the scores; their V rows are whatever finite values the
// pages hold (the cache starts as zeros and is only ever written with finite numbers), times zero.
//
// Every wait on an mbarrier is bounded in polls and in time; a wait that runs out marks the CTA dead:
// nobody waits again, all roles run to their end, tensor memory is freed, and the host reads a status
// (the number of the wait that gave up first).
#include "common.cuh"
#include "entry_points.h"
#include <cuda.h>
#include <cudaTypedefs.h>

// softmax threads per row (TPR): 2 or 4; the softmax warps come first, then the two producers and the MMA warp
#define AT_SOFTMAX_THREADS_OF(TPR) ((TPR) * 128)
#define AT_THREADS_OF(TPR) ((TPR) * 128 + 96)
#define AT_STAGES 3        // a stage holds K of tile j + 2 and V of tile j: what the MMA thread's step j reads
#define AT_META 256        // requests whose token ranges are staged in shared memory
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
__device__ __forceinline__ bool at_mbar_wait(unsigned long long* bar, unsigned parity, volatile int* dead,
                                             unsigned poll_limit = AT_SPIN_LIMIT) {
  return qd_mbar_wait_bounded(at_smem(bar), parity, dead, poll_limit, 2000000000ull);
}
// x = column in elements (0 or 64 here: a multiple of 128 bytes), y = row of the cache seen as [rows][d]
__device__ __forceinline__ void at_tma_2d(void* dst, const CUtensorMap* map, int x, int y, unsigned long long* bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
               ::"r"(at_smem(dst)), "l"(map), "r"(at_smem(bar)), "r"(x), "r"(y) : "memory");
}
// Shared-memory matrix descriptors (64 bits), 128-byte swizzle, rows of 128 bytes, groups of 8 rows 1024 bytes
// apart.  Low word: bits 0-13 the start address in 16-byte units, bits 16-29 the leading offset in 16-byte units.
// High word: bits 0-13 the stride offset (1024 bytes: the next group of 8 rows) in 16-byte units, bit 14 the
// descriptor version of this architecture, bits 29-31 the layout (2 = 128-byte swizzle).
//   K-major (the contraction runs along a row; K tiles): leading offset unused (1).
//   MN-major (a row holds 64 consecutive N elements of ONE contraction index, 8 contraction indices per group;
//   V tiles): leading offset = distance to the next 64 N elements.
// The high word is the same for all tiles, so a step along a tile is one 32-bit addition to the low word.
#define AT_DESC_HI ((unsigned)(1024 >> 4) | (1u << 14) | (2u << 29))
__device__ __forceinline__ unsigned at_desc_lo(unsigned smem_addr, unsigned leading_bytes) {
  return ((smem_addr & 0x3FFFF) >> 4) | (leading_bytes ? ((leading_bytes >> 4) & 0x3FFF) << 16 : 1u << 16);
}
// D[128 x N] (+)= A[128 x 16] B[N x 16]^T with A in tensor memory: rows = lanes, the contraction index along the
// columns, two bfloat16 per 32-bit column (element 2c in the low half of column c); B in shared memory.
__device__ __forceinline__ void at_umma_ta(unsigned tmem_d, unsigned tmem_a, unsigned desc_lo, unsigned desc_hi,
                                           unsigned idesc, unsigned accumulate) {
  asm volatile(
      "{\n .reg .pred p;\n .reg .b64 d;\n setp.ne.b32 p, %5, 0;\n mov.b64 d, {%2, %3};\n"
      " tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], d, %4, {%6, %6, %6, %6}, p;\n}\n"
      ::"r"(tmem_d), "r"(tmem_a), "r"(desc_lo), "r"(desc_hi), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}
// N consecutive 32-bit columns of this thread's TMEM lane from registers (N = 16 or 32)
template <int N>
__device__ __forceinline__ void at_tmem_st(unsigned taddr, const unsigned (&r)[N]) {
  static_assert(N == 16 || N == 32, "16 or 32 columns");
  if (N == 16) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};\n"
                 ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
                   "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]) : "memory");
  } else {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,"
        "%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};\n"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
          "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
          "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
          "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31]) : "memory");
  }
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void at_commit(unsigned long long* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(at_smem(bar)) : "memory");
}
// N consecutive columns of this thread's TMEM lane (N = 16, 32 or 64) in one request
template <int N>
__device__ __forceinline__ void at_tmem_ld(unsigned taddr, float (&v)[N]) {
  static_assert(N == 16 || N == 32 || N == 64, "16, 32 or 64 columns");
  unsigned r[N];
  if (N == 16) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr));
  } else if (N == 32) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,"
        "%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
  } else {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x64.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,"
        "%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32,%33,%34,%35,%36,%37,%38,%39,%40,%41,%42,%43,%44,%45,%46,"
        "%47,%48,%49,%50,%51,%52,%53,%54,%55,%56,%57,%58,%59,%60,%61,%62,%63}, [%64];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31]), "=r"(r[32]),
          "=r"(r[33]), "=r"(r[34]), "=r"(r[35]), "=r"(r[36]), "=r"(r[37]), "=r"(r[38]), "=r"(r[39]), "=r"(r[40]),
          "=r"(r[41]), "=r"(r[42]), "=r"(r[43]), "=r"(r[44]), "=r"(r[45]), "=r"(r[46]), "=r"(r[47]), "=r"(r[48]),
          "=r"(r[49]), "=r"(r[50]), "=r"(r[51]), "=r"(r[52]), "=r"(r[53]), "=r"(r[54]), "=r"(r[55]), "=r"(r[56]),
          "=r"(r[57]), "=r"(r[58]), "=r"(r[59]), "=r"(r[60]), "=r"(r[61]), "=r"(r[62]), "=r"(r[63])
        : "r"(taddr));
  }
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < N; i++) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void at_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void at_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ float at_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ unsigned at_pack(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<unsigned*>(&v);
}
__device__ __forceinline__ long long at_now() {
  long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// A row's sum and output are rescaled only when its maximum has grown by more than this (in powers of two) since
// the value its exponentials refer to: P stays below 2^8, which loses nothing in bfloat16 or in the float32
// sums, and the final division by the row sum, taken against the same reference, gives the same result.
#define AT_RESCALE_STEP 8.0f

struct AtParams {
  const bf16* q; long long q_stride; bf16* out;
  const int* block_table; int max_blocks;
  const int* cu_tokens; const int* start_pos;
  int R, H, G, page_size, window, tok_tile;
  float scale_log2e;
  int* status;
  // null, or nanosecond stamps for measurements: [0, 128) 16 x 8 of row 0's softmax thread and [128, 192) 16 x 4
  // of the MMA thread of the CTA of KV head 0 whose rows end at key 2047 (16 key tiles; slot 7 of the first seven
  // tiles holds the CTA's own phases: start, tensor memory allocated, request found, Q stored, last P stored, last
  // product complete, end); from 192 on four words per CTA: start, end, SM, key tiles
  long long* timeline;
};

template <int HD, int TPR>
__global__ void __launch_bounds__(AT_THREADS_OF(TPR), 1)
prefill_attention_tc5_kernel(const __grid_constant__ CUtensorMap kv_map, const AtParams p) {
  constexpr int AT_SOFTMAX_THREADS = AT_SOFTMAX_THREADS_OF(TPR);
  constexpr int W_PRODUCER = TPR * 4, W_MMA = TPR * 4 + 2;      // warps of the two producers (K, V) and of the MMA issuer
  constexpr int KQ = AT_KEYS / TPR;                 // keys of a tile per softmax thread
  constexpr int NS = AT_STAGES;
  constexpr int NB = HD / 64;                       // 64-column blocks of a row
  constexpr int DH = HD / TPR;                      // output columns per softmax thread
  constexpr int TILE_BYTES = AT_ROWS * HD * 2;      // one [128][HD] bfloat16 tile
  // tensor memory: two S/P buffers of 128 columns, the output rows O (HD columns), the query rows Q (HD / 2
  // columns of bfloat16 pairs)
  constexpr unsigned TMEM_COLS = 512, T_O = 2 * AT_KEYS, T_Q = 3 * AT_KEYS;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  unsigned char* base = smem_raw + ((1024 - (at_smem(smem_raw) & 1023)) & 1023);
  unsigned char* k_s = base;                        // NS stages of K [128 keys][HD], K-major
  unsigned char* v_s = k_s + NS * TILE_BYTES;       // NS stages of V [128 keys][HD], MN-major for the product
  // Slot i (i = -2 .. n_kt - 1, stage (i + 2) % NS) holds K of tile i + 2 and V of tile i, the two tiles the MMA
  // thread reads in its step i, under one pair of barriers: each wait of that one thread is time in which no
  // MMA is issued.  Both producers arrive at kv_full (with their bytes, or bare where a slot lacks their tile).
  __shared__ unsigned long long kv_full[NS], kv_empty[NS], s_full[2], p_full[2], o_done, q_full;
  __shared__ float mx_s[2][TPR][AT_ROWS];           // [tile parity][share of the keys][row]: the shares' maxima
  __shared__ float l_s[TPR][AT_ROWS];               // the shares' sums, at the end
  __shared__ unsigned tmem_slot;
  __shared__ int dead;
  __shared__ int cu_s[AT_META + 1], sp_s[AT_META + 1];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long cta_t0 = p.timeline ? at_now() : 0;

  if (threadIdx.x == 0) {
    dead = 0;
    for (int s = 0; s < NS; s++) { at_mbar_init(&kv_full[s], 2); at_mbar_init(&kv_empty[s], 1); }
    for (int s = 0; s < 2; s++) at_mbar_init(&s_full[s], 1);
    at_mbar_init(&o_done, 1);
    // P of tile j + 1 may be ready before the MMA thread has looked at tile j's barrier (the softmax threads
    // hand P over before they wait for the product of the tile before): two barriers, used in turn
    at_mbar_init(&p_full[0], AT_SOFTMAX_THREADS); at_mbar_init(&p_full[1], AT_SOFTMAX_THREADS);
    at_mbar_init(&q_full, AT_SOFTMAX_THREADS);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == W_MMA) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(at_smem(&tmem_slot)),
                 "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  // the requests' token ranges and start positions (the step's metadata, not the work of the kernel before) go to
  // shared memory in one trip: the search below would otherwise wait for a load per request it passes
  const bool meta_staged = p.R < AT_META;
  if (meta_staged) {
    for (int i = threadIdx.x; i <= p.R; i += AT_THREADS_OF(TPR)) {
      cu_s[i] = p.cu_tokens[i];
      sp_s[i] = i < p.R ? p.start_pos[i] : 0;
    }
  }
  at_fence_before();
  __syncthreads();
  at_fence_after();
  const unsigned tmem = tmem_slot;
  const long long cta_t1 = p.timeline ? at_now() : 0;

  // ---- which request and which tokens (tiles numbered request by request, the longest histories first)
  const int g = blockIdx.y;
  const int gs = p.H / p.G;
  const int* cu = meta_staged ? cu_s : p.cu_tokens;
  const int* sp = meta_staged ? sp_s : p.start_pos;
  int b = gridDim.x - 1 - blockIdx.x;
  int r = 0, before = 0;
  for (; r < p.R; r++) {
    int n = cu[r + 1] - cu[r];
    int nt = (n + p.tok_tile - 1) / p.tok_tile;
    if (b < before + nt) break;
    before += nt;
  }
  const bool idle = r == p.R;
  const long long cta_t2 = p.timeline ? at_now() : 0;
  int tok0 = 0, n_tok = 0, pos0 = 0;
  if (!idle) {
    tok0 = cu[r] + (b - before) * p.tok_tile;
    n_tok = min(p.tok_tile, cu[r + 1] - tok0);
    pos0 = sp[r] + (tok0 - cu[r]);
  }
  pdl_wait();
  const int key_hi = pos0 + n_tok;
  const int key_lo_tile = (p.window > 0 && pos0 - p.window + 1 > 0) ? pos0 - p.window + 1 : 0;
  const int kt_lo = key_lo_tile / AT_KEYS, kt_hi = idle ? kt_lo : (key_hi + AT_KEYS - 1) / AT_KEYS;
  const int n_kt = kt_hi - kt_lo;

  if (warp == W_PRODUCER || warp == W_PRODUCER + 1) {
    // ------------------------------------------------------------------ producers: one warp for K, one for V
    // Each walks its own tiles and is held back only by its own stages' barriers, so a K stage is refilled as
    // soon as its scores are done and a V stage as soon as its product is.  A tile is eight 16-key boxes (two
    // 64-column halves each) from eight pages; the page numbers of the next tile are read from the block
    // table while this tile's stage is waited for, so no copy waits for a load of its own address.
    if (!idle) {
      const int which = warp - W_PRODUCER;            // 0 = K, 1 = V
      const int shift = which ? 0 : 2;                // slot i holds this producer's tile i + shift
      const int* bt = p.block_table + (size_t)r * p.max_blocks;
      auto page_of = [&](int j) {                     // page of this lane's box row of tile j (lanes 0..7)
        const int key0 = (kt_lo + j) * AT_KEYS + lane * 16;
        return (lane < AT_KEYS / 16 && j >= 0 && j < n_kt && key0 < key_hi) ? bt[key0 / p.page_size] : -1;
      };
      int page_next = page_of(-2 + shift);
      for (int i = -2; i < n_kt; i++) {
        const int j = i + shift;                      // this producer's tile of the slot, if 0 <= j < n_kt
        int page = page_next;
        page_next = page_of(j + 1);
        const int s = (i + 2) % NS;
        const unsigned ph = ((i + 2) / NS) & 1;
        if (!at_mbar_wait(&kv_empty[s], ph ^ 1, &dead) && lane == 0) atomicCAS(p.status, 0, 1);
        const bool have = j >= 0 && j < n_kt;
        if (lane == 0) {
          if (have) at_mbar_expect_tx(&kv_full[s], TILE_BYTES);
          else at_mbar_arrive(&kv_full[s]);
        }
        __syncwarp();
        if (have && lane < AT_KEYS / 16) {            // one 16-key box row per lane
          const int key0 = (kt_lo + j) * AT_KEYS + lane * 16;
          if (page < 0) page = 0;                     // no such keys: any page will do, the scores are masked
          const int row0 = ((page * 2 + which) * p.G + g) * p.page_size + key0 % p.page_size;
          unsigned char* dst = (which ? v_s : k_s) + s * TILE_BYTES + lane * 2048;     // 16 keys = two groups of 8 rows
#pragma unroll
          for (int cb = 0; cb < NB; cb++) at_tma_2d(dst + cb * (AT_KEYS * 128), &kv_map, cb * 64, row0, &kv_full[s]);
        }
      }
    }
  } else if (warp == W_MMA) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0 && !idle) {
      const unsigned idesc_qk = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(AT_KEYS >> 3) << 17) | ((unsigned)(AT_ROWS >> 4) << 24);
      const unsigned idesc_pv = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((unsigned)(HD >> 3) << 17) |
                                ((unsigned)(AT_ROWS >> 4) << 24);
      // Q is the A operand from tensor memory (16 columns of the contraction = 8 columns of bfloat16 pairs per
      // step), so the scores read only K from shared memory; P likewise for the product, which reads only V.
      // Scores of tile j + 2 go where P of tile j lies and are issued after the product of tile j (the tensor
      // cores run a thread's MMAs in the order it issued them); the scores of tile j + 1 are complete by then,
      // so the softmax threads never wait for them.
      const unsigned desc_hi = AT_DESC_HI;
      const unsigned k_lo0 = at_desc_lo(at_smem(k_s), 0);                  // K-major
      const unsigned v_lo0 = at_desc_lo(at_smem(v_s), AT_KEYS * 128);      // MN-major: the d columns 64.. lie one
                                                                           // [128 keys][128 bytes] block further
      auto slot_ready = [&](int i) {                    // K of tile i + 2 and V of tile i are in shared memory
        if (!at_mbar_wait(&kv_full[(i + 2) % NS], ((i + 2) / NS) & 1, &dead)) atomicCAS(p.status, 0, 2);
      };
      auto scores = [&](int j) {                        // S of tile j from the stage of slot j - 2
        const unsigned k_lo = k_lo0 + (unsigned)(j % NS) * (TILE_BYTES >> 4);
#pragma unroll
        for (int k = 0; k < HD / 16; k++) {
          // 16 columns = 32 bytes inside a 64-column block; the next block is 128 rows x 128 bytes further
          const unsigned adv = (unsigned)(((k >> 2) * (AT_ROWS * 128) + (k & 3) * 32) >> 4);
          at_umma_ta(tmem + (unsigned)(j & 1) * AT_KEYS, tmem + T_Q + (unsigned)k * 8, k_lo + adv, desc_hi, idesc_qk, k ? 1u : 0u);
        }
      };
      const bool mstamp = p.timeline && blockIdx.y == 0 && n_kt >= 16 && pos0 + n_tok == n_kt * AT_KEYS;
      if (!at_mbar_wait(&q_full, 0, &dead)) atomicCAS(p.status, 0, 3);
      for (int j = 0; j < 2; j++) {                     // slots -2 and -1: the first two tiles' scores
        slot_ready(j - 2);
        at_fence_after();
        if (j < n_kt) scores(j);
        at_commit(&kv_empty[j % NS]);
        if (j < n_kt) at_commit(&s_full[j & 1]);
      }
      for (int j = 0; j < n_kt; j++) {
        const int s = (j + 2) % NS;
        if (mstamp) p.timeline[128 + j * 4 + 0] = at_now();
        if (!at_mbar_wait(&p_full[j & 1], (j >> 1) & 1, &dead)) atomicCAS(p.status, 0, 4);
        if (mstamp) p.timeline[128 + j * 4 + 1] = at_now();
        slot_ready(j);
        at_fence_after();
        const unsigned v_lo = v_lo0 + (unsigned)s * (TILE_BYTES >> 4);
#pragma unroll
        for (int k = 0; k < AT_KEYS / 16; k++) {
          // 16 keys = two groups of 8 rows of V (2,048 bytes); P of this tile lies where its scores were: 16 keys
          // = 8 columns of bfloat16 pairs per step
          at_umma_ta(tmem + T_O, tmem + (unsigned)(j & 1) * AT_KEYS + (unsigned)k * 8, v_lo + (unsigned)k * (2048 >> 4), desc_hi,
                      idesc_pv, (j > 0 || k > 0) ? 1u : 0u);
        }
        if (mstamp) p.timeline[128 + j * 4 + 2] = at_now();
        at_commit(&o_done);
        if (j + 2 < n_kt) scores(j + 2);
        at_commit(&kv_empty[s]);
        if (j + 2 < n_kt) at_commit(&s_full[j & 1]);
        if (mstamp) p.timeline[128 + j * 4 + 3] = at_now();
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax: TPR threads per row
    const int row = (warp & 3) * 32 + lane;                        // 0..127, also the TMEM lane
    const int h = warp >> 2;                                       // which share of the keys and of the columns
    const int t = row / gs, hh = row - t * gs;
    const bool ok = !idle && t < n_tok;
    const int pos = pos0 + t;
    const int lo = (p.window > 0 && pos - p.window + 1 > 0) ? pos - p.window + 1 : 0;
    const unsigned t_lane = tmem + ((unsigned)((warp & 3) * 32) << 16);      // this warp's 32 lanes
    // this thread's share of the Q row into tensor memory: bfloat16 pairs as they lie in memory, a pair a column
    {
      constexpr int QC = HD / 2 / TPR;                               // columns of this share
      static_assert(QC == 16 || QC == 32, "a share of Q is 16 or 32 columns");
      const bf16* qr = p.q + (size_t)(tok0 + t) * p.q_stride + (size_t)(g * gs + hh) * HD + h * (HD / TPR);
      unsigned qv[QC];
#pragma unroll
      for (int c = 0; c < QC / 4; c++) {
        uint4 v = make_uint4(0, 0, 0, 0);
        if (ok) v = *reinterpret_cast<const uint4*>(qr + c * 8);
        qv[4 * c] = v.x; qv[4 * c + 1] = v.y; qv[4 * c + 2] = v.z; qv[4 * c + 3] = v.w;
      }
      at_tmem_st<QC>(t_lane + T_Q + h * QC, qv);
      at_fence_before();
      at_mbar_arrive(&q_full);
    }
    float m = -INFINITY, l = 0.f;        // m: the maximum that this row's exponentials, sum and output refer to
    const bool stamp = p.timeline && threadIdx.x == 0 && blockIdx.y == 0 && n_kt >= 16 && pos0 + n_tok == n_kt * AT_KEYS;
    if (stamp) { p.timeline[7] = cta_t0; p.timeline[8 + 7] = cta_t1; p.timeline[16 + 7] = cta_t2; p.timeline[24 + 7] = at_now(); }
    // keys every valid row of the tile sees need no test: all up to the first row's position and, with a
    // window, from the last row's first visible key on
    const int free_hi = pos0 + 1;
    const int free_lo = (p.window > 0 && key_hi - p.window > 0) ? key_hi - p.window : 0;
    for (int j = 0; j < n_kt; j++) {
      const int tile_base = (kt_lo + j) * AT_KEYS;
      const int key_base = tile_base + h * KQ;
      if (stamp) p.timeline[j * 8 + 0] = at_now();
      if (!at_mbar_wait(&s_full[j & 1], (j >> 1) & 1, &dead) && lane == 0) atomicCAS(p.status, 0, 7);
      at_fence_after();
      if (stamp) p.timeline[j * 8 + 1] = at_now();
      float sv[KQ];
      at_tmem_ld<KQ>(t_lane + (unsigned)(j & 1) * AT_KEYS + h * KQ, sv);
      if (stamp) p.timeline[j * 8 + 2] = at_now();
      const bool interior = tile_base >= free_lo && tile_base + AT_KEYS <= free_hi && p.scale_log2e > 0.f;
      float mx = -INFINITY;
      if (interior) {
#pragma unroll
        for (int i = 0; i < KQ; i++) mx = fmaxf(mx, sv[i]);
        mx *= p.scale_log2e;
      } else {
#pragma unroll
        for (int i = 0; i < KQ; i++) {
          const int key = key_base + i;
          const bool vis = ok && key <= pos && key >= lo;
          sv[i] = vis ? sv[i] * p.scale_log2e : -INFINITY;
          mx = fmaxf(mx, sv[i]);
        }
      }
      mx_s[j & 1][h][row] = mx;
      asm volatile("bar.sync 1, %0;" ::"n"(AT_SOFTMAX_THREADS) : "memory");
      if (stamp) p.timeline[j * 8 + 3] = at_now();
      float m_tile = mx;
#pragma unroll
      for (int o2 = 1; o2 < TPR; o2++) m_tile = fmaxf(m_tile, mx_s[j & 1][(h + o2) % TPR][row]);
      // The row moves to a new reference only when its maximum has grown by more than AT_RESCALE_STEP (always
      // from "no key yet"): then its sum and its output in tensor memory are scaled down, once the product of
      // the tile before is complete.  All threads of a row decide alike; the warp acts together, since the
      // tensor-memory accesses are the warp's.
      const bool grow = m_tile > m + AT_RESCALE_STEP;
      if (__any_sync(0xffffffffu, grow)) {
        const float alpha = grow ? at_exp2(m - m_tile) : 1.0f;     // m = -inf: 0, and sum and output are 0 so far
        if (grow) m = m_tile;
        l *= alpha;
        if (j > 0) {
          if (!at_mbar_wait(&o_done, (j - 1) & 1, &dead) && lane == 0) atomicCAS(p.status, 0, 8);
          at_fence_after();
#pragma unroll
          for (int c = 0; c < DH; c += 32) {
            float ov[32];
            at_tmem_ld<32>(t_lane + T_O + h * DH + c, ov);
            unsigned ob[32];
#pragma unroll
            for (int i = 0; i < 32; i++) ob[i] = __float_as_uint(ov[i] * alpha);
            at_tmem_st<32>(t_lane + T_O + h * DH + c, ob);
          }
        }
      }
      const float ref = m == -INFINITY ? 0.f : m;
      // p = exp2(score - max) as bfloat16 pairs, kept in registers until the P tile is free
      unsigned pk[KQ / 2];
      float sum = 0.f;
      const float mul = interior ? p.scale_log2e : 1.0f;
#pragma unroll
      for (int i = 0; i < KQ / 2; i++) {
        const float p0 = at_exp2(fmaf(sv[2 * i], mul, -ref)), p1 = at_exp2(fmaf(sv[2 * i + 1], mul, -ref));
        sum += p0 + p1;
        pk[i] = at_pack(p0, p1);
      }
      l += sum;
      if (stamp) p.timeline[j * 8 + 4] = at_now();
      // P goes into tensor memory, over the first half of this tile's own scores (every thread of the row has
      // its scores in registers since the barrier above): the product reads it from there as its A operand and
      // nothing passes through shared memory
      at_tmem_st<KQ / 2>(t_lane + (unsigned)(j & 1) * AT_KEYS + h * (KQ / 2), pk);
      at_fence_before();
      at_mbar_arrive(&p_full[j & 1]);
      if (stamp) p.timeline[j * 8 + 5] = at_now();
    }
    if (n_kt > 0) {
      if (stamp) p.timeline[32 + 7] = at_now();
      if (!at_mbar_wait(&o_done, (n_kt - 1) & 1, &dead) && lane == 0) atomicCAS(p.status, 0, 9);
      if (stamp) p.timeline[40 + 7] = at_now();
      at_fence_after();
    }
    l_s[h][row] = l;
    asm volatile("bar.sync 1, %0;" ::"n"(AT_SOFTMAX_THREADS) : "memory");
    if (n_kt > 0) {
      float l_all = l;
#pragma unroll
      for (int o2 = 1; o2 < TPR; o2++) l_all += l_s[(h + o2) % TPR][row];
      const float inv = l_all > 0.f ? 1.f / l_all : 0.f;
      bf16* d = p.out + (size_t)(tok0 + t) * p.H * HD + (size_t)(g * gs + hh) * HD + h * DH;
#pragma unroll
      for (int c = 0; c < DH; c += 32) {
        float ov[32];
        at_tmem_ld<32>(t_lane + T_O + h * DH + c, ov);      // the warp's access: rows without a token take part too
        if (ok) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint4 v;
            v.x = at_pack(ov[i] * inv, ov[i + 1] * inv);
            v.y = at_pack(ov[i + 2] * inv, ov[i + 3] * inv);
            v.z = at_pack(ov[i + 4] * inv, ov[i + 5] * inv);
            v.w = at_pack(ov[i + 6] * inv, ov[i + 7] * inv);
            *reinterpret_cast<uint4*>(d + c + i) = v;
          }
        }
      }
      if (stamp) p.timeline[(n_kt - 1) * 8 + 6] = at_now();
    }
  }
  pdl_launch_dependents();
  at_fence_before();
  __syncthreads();
  if (p.timeline && threadIdx.x == 0) {
    unsigned smid;
    asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
    long long* e = p.timeline + 192 + (size_t)(blockIdx.y * gridDim.x + blockIdx.x) * 4;
    e[0] = cta_t0; e[1] = at_now(); e[2] = smid; e[3] = n_kt;
    if (blockIdx.y == 0 && n_kt >= 16 && pos0 + n_tok == n_kt * AT_KEYS) p.timeline[48 + 7] = e[1];
  }
  if (warp == W_MMA) {
    at_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
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

template <int HD, int TPR>
static int at_launch(const CUtensorMap& map, const AtParams& p, int tiles, cudaStream_t stream) {
  size_t smem = 1024 + (size_t)(2 * AT_STAGES) * AT_ROWS * HD * 2;
  auto kernel = prefill_attention_tc5_kernel<HD, TPR>;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
    cudaGetLastError();
    return QD_ERR_UNSUPPORTED;
  }
  qd_launch(kernel, dim3((unsigned)tiles, (unsigned)p.G), dim3(AT_THREADS_OF(TPR)), smem, stream, map, p);
  return (int)cudaGetLastError();
}

// Arguments as qd_prefill_attention (attention_flash.cu) plus the number of pages of `kv`
// ([pages, 2, G, page_size, d], bfloat16).  Takes head sizes 64 and 128, groups of 1 to 16 query heads per KV
// head (a tile's 128 rows hold floor(128 / group) tokens x the group's heads; with a group that does not
// divide 128 the last rows of a tile stay empty: 2 of 128 at 7 heads, 3 at 5), page sizes that are multiples
// of 16; refuses the rest (the caller has another kernel).
extern "C" int qd_prefill_attention_tc5(const void* q, long long q_stride, void* out, const void* kv, long long n_pages,
                                        const int* block_table, int max_blocks, const int* cu_tokens,
                                        const int* start_pos, int R, int T, int H, int G, int d, int page_size,
                                        float scale, int window, long long* timeline, cudaStream_t stream) {
  if (T <= 0 || R <= 0) return 0;
  if (G < 1 || H % G != 0 || page_size % 16 != 0 || (d != 64 && d != 128) || n_pages < 1) return QD_ERR_UNSUPPORTED;
  const int gs = H / G;
  if (gs > 16) return QD_ERR_UNSUPPORTED;
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
  p.timeline = timeline;
  const int tiles = (T + p.tok_tile - 1) / p.tok_tile + R;      // upper bound on the tiles of R requests
  return d == 64 ? at_launch<64, 2>(map, p, tiles, stream) : at_launch<128, 2>(map, p, tiles, stream);
}

// 0 if no kernel of this library has recorded a bounded-wait expiry on the current device.  Synchronises.
QD_DEFINE_WAIT_PROBE(qd_prefill_attention_tc5_wait_probe, at_mbar_wait(bar, 0, dead, poll_limit), at_status_word, 99)

extern "C" int qd_prefill_attention_tc5_status() {
  int* status = at_status_word();
  if (!status) return -1;
  int v = 0;
  if (cudaMemcpy(&v, status, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
  if (v) cudaMemset(status, 0, sizeof(int));
  return v;
}
