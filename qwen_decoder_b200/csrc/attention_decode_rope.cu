// Decode attention for a few tokens that starts from what the few-token contraction leaves: float32
// partial sums of q, k and v.  One kernel adds them up with the bias, rotates q and k by position,
// writes the token's k and v to its cache slot and attends over the paged cache -- the work of
// rope_kv_write_partial (elementwise.cu) and decode_attention (attention_flash.cu) in one launch, with
// one CTA of 8 warps per (token, kv head, split) and every warp's first 16-key chunk requested before
// the kernel waits for its predecessor.  Formulas: gpu_kernels.cu:82-133 (rotation, cache write) and
// :223-311 (attention) of the reference; softmax, rotation and sums in float32.
#include "common.cuh"
#include <math.h>
#include <stdlib.h>

#define AR_WARPS 8
#define AR_THREADS (AR_WARPS * 32)
#define AR_PAD 8

struct ArParams {
  const float* part; int n_parts;      // [n_parts, T, (H + 2G) d] float32
  const float* bias;                   // [(H + 2G) d] or null
  bf16* out;                           // [T, H d]
  bf16* kv;                            // [pages, 2, G, page_size, d]
  const int* block_table; int max_blocks;
  const int* token_req; const int* positions; const int* slot_map;
  int T, H, G, page_size, window, splits, write_kv;
  const float* cos_t; const float* sin_t; int rotary_dim, pairing; float scale_log2e;
  float* part_o; float* part_ml; unsigned* tickets;
  long long* timeline;                 // null, or 16 nanosecond stamps per CTA (for measurements)
};

__device__ __forceinline__ void ar_stamp(const ArParams& p, int i) {
  if (p.timeline && threadIdx.x == 0) {
    long long now;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
    p.timeline[(size_t)blockIdx.x * 16 + i] = now;
  }
}
__device__ __forceinline__ void ar_mma(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                       unsigned b0, unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ar_cp_async16(void* smem, const void* gmem, int src_bytes) {
  unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(src_bytes));
}
__device__ __forceinline__ void ar_ldmatrix_x4(unsigned (&r)[4], const void* smem) {
  unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void ar_ldmatrix_x4_trans(unsigned (&r)[4], const void* smem) {
  unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ unsigned ar_pack(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<unsigned*>(&v);
}
__device__ __forceinline__ float ar_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// NS: chunks a warp keeps in flight (stages of its own K/V ring).  With 3 a CTA needs nearly all of an SM's
// shared memory, which costs nothing while the grid has no more CTAs than the GPU has SMs; 1 leaves room for
// two CTAs per SM.
template <int HD, int NS>
__global__ void __launch_bounds__(AR_THREADS, NS == 1 ? 2 : 1) decode_attention_rope_kernel(const ArParams p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  constexpr int LD = HD + AR_PAD;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int H = p.H, G = p.G, gs = H / G, Nqkv = (H + 2 * G) * HD;
  bf16* qs = reinterpret_cast<bf16*>(smem_raw);                       // [16][LD] rotated q of the group
  bf16* kvs = qs + 16 * LD;                                           // per warp: K chunk, V chunk [16][LD] each
  constexpr int STAGE = 2 * 16 * LD;                                  // elements of a stage: K chunk, V chunk
  float* mm = reinterpret_cast<float*>(kvs + (size_t)AR_WARPS * NS * STAGE);     // merge: [warps][16]
  float* ml = mm + AR_WARPS * 16;                                     // [warps][16]
  bf16* newkv = reinterpret_cast<bf16*>(ml + AR_WARPS * 16);         // the token's own k and v: [2][HD]
  __shared__ unsigned s_ticket;
  const size_t page_elems = (size_t)2 * G * p.page_size * HD;
  const int half = p.rotary_dim >> 1;

  {
    ar_stamp(p, 0);
    pdl_launch_dependents();      // the next kernel's CTAs may start beside these and fetch their weights; they wait for this grid's end
    const int item = blockIdx.x;
    const int s = item % p.splits, g = (item / p.splits) % G, t = item / (p.splits * G);
    const int pos = p.positions[t];
    const int n_keys = pos + 1;
    const int key_lo = (p.window > 0 && pos - p.window + 1 > 0) ? pos - p.window + 1 : 0;
    const int chunk_lo = key_lo / 16, chunk_hi = (n_keys + 15) / 16;
    const int per = (chunk_hi - chunk_lo + p.splits - 1) / p.splits;
    const int c0 = chunk_lo + s * per, c1 = min(chunk_hi, c0 + per);
    const int* bt = p.block_table + (size_t)p.token_req[t] * p.max_blocks;
    const float* acc = p.part + (size_t)t * Nqkv;
    const size_t part_stride = (size_t)p.T * Nqkv;
    const size_t k_off = (size_t)g * p.page_size * HD, v_off = ((size_t)G + g) * p.page_size * HD;

    // ---- before waiting for the kernel that makes q, k, v: ask for this warp's first chunk of old keys
    bf16* wbuf = kvs + (size_t)warp * NS * STAGE;
    constexpr int CPR = HD / 8;
    constexpr int ROWS_PER_IT = 32 / CPR > 0 ? 32 / CPR : 1;
    const int l_row = lane / CPR, l_col = (lane % CPR) * 8;
    auto request_chunk = [&](int c, int stage) {
      bf16* ks = wbuf + (size_t)stage * STAGE;
      bf16* vs = ks + 16 * LD;
      const int key0 = c * 16;
      const int page = bt[key0 / p.page_size];
      const int in_page = key0 % p.page_size;
      const bf16* kg = p.kv + (page < 0 ? 0 : (size_t)page * page_elems) + k_off + (size_t)in_page * HD;
      const bf16* vg = p.kv + (page < 0 ? 0 : (size_t)page * page_elems) + v_off + (size_t)in_page * HD;
      // keys already in the cache: all of them, but not the token's own when this kernel writes it
      const int rows_ok = page < 0 ? 0 : (n_keys - (p.write_kv ? 1 : 0)) - key0;
      for (int row = l_row; row < 16; row += ROWS_PER_IT) {
        int bytes = row < rows_ok ? 16 : 0;
        ar_cp_async16(ks + row * LD + l_col, kg + (bytes ? row * HD + l_col : 0), bytes);
        ar_cp_async16(vs + row * LD + l_col, vg + (bytes ? row * HD + l_col : 0), bytes);
      }
    };
    // The first NS chunks of this warp hold keys of earlier steps only -- except, when this run reads another
    // run's cache (write_kv = 0), the chunk with the token's own position: its owner wrote that key earlier in
    // this very step, so it is asked for only after the wait.
    const int c_first = c0 + warp;
    int deferred = -1;
#pragma unroll
    for (int j = 0; j < NS; j++) {
      const int c = c_first + j * AR_WARPS;
      if (c < c1) {
        if (!p.write_kv && c == chunk_hi - 1) deferred = j;
        else request_chunk(c, j);
      }
      asm volatile("cp.async.commit_group;\n" ::);
    }
    ar_stamp(p, 1);
    pdl_wait();
    if (deferred >= 0) {
      request_chunk(chunk_hi - 1, deferred);
      asm volatile("cp.async.commit_group;\n" ::);
    }
    ar_stamp(p, 2);

    // ---- q of the group (gs heads) and, in the CTA that holds the chunk of the token's own position, its
    // k and v: sums of the parts + bias, rotated; q as bfloat16 rows in shared memory (rows >= gs zero),
    // k and v to the cache slot and to a staging row.  A task is one rotation pair; a thread takes up to
    // four tasks at a time and issues all their loads before it uses any.
    const bool owns_new = p.write_kv && (chunk_hi - 1 >= c0 && chunk_hi - 1 < c1);
    bf16* kdst = nullptr;
    bf16* vdst = nullptr;
    if (owns_new) {
      const int slot = p.slot_map[t];
      const int page = slot / p.page_size, off = slot - page * p.page_size;
      kdst = p.kv + (size_t)page * page_elems + k_off + (size_t)off * HD;
      vdst = p.kv + (size_t)page * page_elems + v_off + (size_t)off * HD;
    }
    for (int w = threadIdx.x; w < (16 - gs) * (HD / 2); w += AR_THREADS)
      reinterpret_cast<unsigned*>(qs + (size_t)gs * LD)[(w / (HD / 2)) * (LD / 2) + (w % (HD / 2))] = 0u;
    const int n_tasks = (gs + (owns_new ? 2 : 0)) * (HD / 2);
    constexpr int NB = 4;
    constexpr int NP = 4;          // shares of the sums whose loads are all in flight before any is used
    for (int base = threadIdx.x; base < n_tasks; base += AR_THREADS * NB) {
      float a[NB], b[NB], cv[NB], sv[NB];
      float pa[NB][NP], pb[NB][NP];
      int i0[NB], i1[NB], row[NB];
#pragma unroll
      for (int u = 0; u < NB; u++) {
        const int w = base + u * AR_THREADS;
        a[u] = b[u] = 0.f; cv[u] = 1.f; sv[u] = 0.f; i0[u] = i1[u] = 0;
        row[u] = -1;
        if (w < n_tasks) {
          row[u] = w / (HD / 2);                       // 0..gs-1: q heads; gs: k; gs + 1: v
          const int pp = w - row[u] * (HD / 2);
          const bool is_v = row[u] == gs + 1;
          const bool rot = pp < half && !is_v;
          if (is_v || p.pairing == 0) { i0[u] = 2 * pp; i1[u] = 2 * pp + 1; }
          else if (pp < half) { i0[u] = pp; i1[u] = pp + half; }
          else { int jj = 2 * (pp - half) + p.rotary_dim; i0[u] = jj; i1[u] = jj + 1; }
          const int e = (row[u] < gs ? g * gs + row[u] : (row[u] == gs ? H + g : H + G + g)) * HD;
          if (p.bias) { a[u] = p.bias[e + i0[u]]; b[u] = p.bias[e + i1[u]]; }
          if (rot && p.cos_t) { cv[u] = p.cos_t[(size_t)pos * half + pp]; sv[u] = p.sin_t[(size_t)pos * half + pp]; }
          const float* src = acc + e;
#pragma unroll
          for (int q = 0; q < NP; q++) {
            pa[u][q] = q < p.n_parts ? __ldcg(src + q * part_stride + i0[u]) : 0.f;
            pb[u][q] = q < p.n_parts ? __ldcg(src + q * part_stride + i1[u]) : 0.f;
          }
        } else {
#pragma unroll
          for (int q = 0; q < NP; q++) pa[u][q] = pb[u][q] = 0.f;
        }
      }
      // The loads of all shares (up to NP) are out before any is used: a loop over a number of shares known only
      // at run time would wait for each share's loads in turn.  The sums keep the order of the shares; more than
      // NP shares: the rest one after the other.
#pragma unroll
      for (int u = 0; u < NB; u++) {
        if (row[u] < 0) continue;
#pragma unroll
        for (int q = 0; q < NP; q++) { a[u] += pa[u][q]; b[u] += pb[u][q]; }
        if (p.n_parts > NP) {
          const int e = (row[u] < gs ? g * gs + row[u] : (row[u] == gs ? H + g : H + G + g)) * HD;
          for (int q = NP; q < p.n_parts; q++) {
            a[u] += __ldcg(acc + e + q * part_stride + i0[u]);
            b[u] += __ldcg(acc + e + q * part_stride + i1[u]);
          }
        }
      }
#pragma unroll
      for (int u = 0; u < NB; u++) {
        if (row[u] < 0) continue;
        const bf16 ha = __float2bfloat16_rn(a[u] * cv[u] - b[u] * sv[u]);
        const bf16 hb = __float2bfloat16_rn(a[u] * sv[u] + b[u] * cv[u]);
        if (row[u] < gs) {
          qs[row[u] * LD + i0[u]] = ha; qs[row[u] * LD + i1[u]] = hb;
        } else {
          bf16* stage = newkv + (row[u] - gs) * HD;
          bf16* dst = row[u] == gs ? kdst : vdst;
          stage[i0[u]] = ha; stage[i1[u]] = hb;
          dst[i0[u]] = ha; dst[i1[u]] = hb;
        }
      }
    }
    __syncthreads();
    ar_stamp(p, 3);

    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
    float o[HD / 8][4];
#pragma unroll
    for (int i = 0; i < HD / 8; i++) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    // q as MMA fragments, once for all chunks: matrices (rows 0-7 | 8-15) x (k 0-7 | 8-15) in the order a0..a3
    unsigned qa[HD / 16][4];
#pragma unroll
    for (int kk = 0; kk < HD / 16; kk++)
      ar_ldmatrix_x4(qa[kk], qs + ((lane & 7) + 8 * ((lane >> 3) & 1)) * LD + kk * 16 + 8 * (lane >> 4));
    int it = 0;
    for (int c = c_first; c < c1; c += AR_WARPS, it++) {
      const int key0 = c * 16;
      const int stage = it % NS;
      bf16* ks = wbuf + (size_t)stage * STAGE;
      bf16* vs = ks + 16 * LD;
      if (!p.write_kv && c == chunk_hi - 1) asm volatile("cp.async.wait_group 0;\n" ::);   // asked for late: all
      else asm volatile("cp.async.wait_group %0;\n" ::"n"(NS - 1));     // NS groups are out: the oldest is this chunk's
      __syncwarp();
      if (p.write_kv && c == chunk_hi - 1) {
        // the token's own k and v, made above: into this warp's copy of the chunk (no trip through memory)
        const int new_row = pos - key0;
        for (int i = lane; i < HD / 4; i += 32) {
          reinterpret_cast<uint2*>(ks + new_row * LD)[i] = reinterpret_cast<const uint2*>(newkv)[i];
          reinterpret_cast<uint2*>(vs + new_row * LD)[i] = reinterpret_cast<const uint2*>(newkv + HD)[i];
        }
        __syncwarp();
      }
      // the chunk's K fragments are all loaded before the first MMA; four chains of MMAs (keys 0-7 and 8-15,
      // even and odd k-steps) that are added at the end
      float sc[2][4], sd[2][4];
#pragma unroll
      for (int n = 0; n < 2; n++) sc[n][0] = sc[n][1] = sc[n][2] = sc[n][3] = sd[n][0] = sd[n][1] = sd[n][2] = sd[n][3] = 0.f;
      unsigned kb[HD / 16][4];
#pragma unroll
      for (int kk = 0; kk < HD / 16; kk++)
        ar_ldmatrix_x4(kb[kk], ks + ((lane & 7) + 8 * (lane >> 4)) * LD + kk * 16 + 8 * ((lane >> 3) & 1));
#pragma unroll
      for (int kk = 0; kk < HD / 16; kk++) {
        if (kk & 1) {
          ar_mma(sd[0], qa[kk][0], qa[kk][1], qa[kk][2], qa[kk][3], kb[kk][0], kb[kk][1]);
          ar_mma(sd[1], qa[kk][0], qa[kk][1], qa[kk][2], qa[kk][3], kb[kk][2], kb[kk][3]);
        } else {
          ar_mma(sc[0], qa[kk][0], qa[kk][1], qa[kk][2], qa[kk][3], kb[kk][0], kb[kk][1]);
          ar_mma(sc[1], qa[kk][0], qa[kk][1], qa[kk][2], qa[kk][3], kb[kk][2], kb[kk][3]);
        }
      }
#pragma unroll
      for (int n = 0; n < 2; n++)
#pragma unroll
        for (int jx = 0; jx < 4; jx++) sc[n][jx] += sd[n][jx];
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
      float a0 = ar_exp2(m0 - ref0), a1 = ar_exp2(m1 - ref1);
      m0 = mn0; m1 = mn1;
      float pr[2][4];
#pragma unroll
      for (int n = 0; n < 2; n++) {
        pr[n][0] = ar_exp2(sc[n][0] - ref0); pr[n][1] = ar_exp2(sc[n][1] - ref0);
        pr[n][2] = ar_exp2(sc[n][2] - ref1); pr[n][3] = ar_exp2(sc[n][3] - ref1);
      }
      l0 = l0 * a0 + pr[0][0] + pr[0][1] + pr[1][0] + pr[1][1];
      l1 = l1 * a1 + pr[0][2] + pr[0][3] + pr[1][2] + pr[1][3];
      unsigned pa0 = ar_pack(pr[0][0], pr[0][1]), pa1 = ar_pack(pr[0][2], pr[0][3]);
      unsigned pa2 = ar_pack(pr[1][0], pr[1][1]), pa3 = ar_pack(pr[1][2], pr[1][3]);
#pragma unroll
      for (int n = 0; n < HD / 8; n++) { o[n][0] *= a0; o[n][1] *= a0; o[n][2] *= a1; o[n][3] *= a1; }
#pragma unroll
      for (int dn = 0; dn < HD / 16; dn++) {
        unsigned b[4];
        ar_ldmatrix_x4_trans(b, vs + ((lane & 7) + 8 * ((lane >> 3) & 1)) * LD + dn * 16 + 8 * (lane >> 4));
        ar_mma(o[2 * dn], pa0, pa1, pa2, pa3, b[0], b[1]);
        ar_mma(o[2 * dn + 1], pa0, pa1, pa2, pa3, b[2], b[3]);
      }
      __syncwarp();
      if (c + NS * AR_WARPS < c1) request_chunk(c + NS * AR_WARPS, stage);       // the stage is free again
      asm volatile("cp.async.commit_group;\n" ::);
    }
    asm volatile("cp.async.wait_group 0;\n" ::);
    ar_stamp(p, 4);
    pdl_launch_dependents();
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    // ---- merge the 8 warps; a warp's partial output [16][HD + 8] float32 lies over its own K/V chunk buffers
    // (a stage is 2 * 16 * LD bfloat16 = 16 * (HD + 8) floats), which it no longer reads.  Rows HD + 8 floats
    // apart: the eight rows a store instruction touches fall on different banks (two by two)
    constexpr int OLD = HD + 8;
    {
      const int r0 = lane >> 2, r1 = r0 + 8, cq = (lane & 3) * 2;
      __syncwarp();
#pragma unroll
      for (int n = 0; n < HD / 8; n++) {
        *reinterpret_cast<float2*>(reinterpret_cast<float*>(wbuf) + (size_t)r0 * OLD + n * 8 + cq) = make_float2(o[n][0], o[n][1]);
        *reinterpret_cast<float2*>(reinterpret_cast<float*>(wbuf) + (size_t)r1 * OLD + n * 8 + cq) = make_float2(o[n][2], o[n][3]);
      }
      if ((lane & 3) == 0) {
        mm[warp * 16 + r0] = m0; mm[warp * 16 + r1] = m1;
        ml[warp * 16 + r0] = l0; ml[warp * 16 + r1] = l1;
      }
    }
    __syncthreads();
    // a thread takes four columns of a head: the factors of the eight warps once, the sums as float4
    for (int idx = threadIdx.x; idx < gs * (HD / 4); idx += AR_THREADS) {
      const int row = idx / (HD / 4), dim = (idx - row * (HD / 4)) * 4;
      float M = -INFINITY;
#pragma unroll
      for (int w = 0; w < AR_WARPS; w++) M = fmaxf(M, mm[w * 16 + row]);
      float Lsum = 0.f;
      float4 O = make_float4(0.f, 0.f, 0.f, 0.f);
      if (M != -INFINITY) {
#pragma unroll
        for (int w = 0; w < AR_WARPS; w++) {
          const float f = ar_exp2(mm[w * 16 + row] - M);
          Lsum += ml[w * 16 + row] * f;
          const float4 v = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(kvs + (size_t)w * NS * STAGE) +
                                                            (size_t)row * OLD + dim);
          O.x += v.x * f; O.y += v.y * f; O.z += v.z * f; O.w += v.w * f;
        }
      }
      const int hd = g * gs + row;
      if (p.splits == 1) {
        const float inv = 1.f / Lsum;
        uint2 raw;
        raw.x = ar_pack(O.x * inv, O.y * inv);
        raw.y = ar_pack(O.z * inv, O.w * inv);
        *reinterpret_cast<uint2*>(p.out + (size_t)t * H * HD + (size_t)hd * HD + dim) = raw;
      } else {
        const size_t pi = ((size_t)t * H + hd) * p.splits + s;
        *reinterpret_cast<float4*>(p.part_o + pi * HD + dim) = O;
        if (dim == 0) { p.part_ml[pi * 2] = M; p.part_ml[pi * 2 + 1] = Lsum; }
      }
    }
    ar_stamp(p, 5);
    if (p.splits > 1) {
      // The CTA's partial results are written by all its threads; they meet, then one thread takes the ticket
      // with release and acquire at GPU scope: the barrier before it puts the others' writes before the release,
      // the barrier after it puts the others' reads after the acquire.  One fence inside the atomic instead of
      // one per thread before it and another after it.
      __syncthreads();
      if (threadIdx.x == 0) {
        unsigned old;
        asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;" : "=r"(old) : "l"(p.tickets + (size_t)t * G + g) : "memory");
        s_ticket = old;
      }
      __syncthreads();
      ar_stamp(p, 6);
      if (s_ticket == (unsigned)p.splits - 1) {          // the last item of this (t, g) combines
        // A thread takes four output columns of one head (a warp: one head when HD = 128).  It asks for the
        // maxima and sums of all splits of its head and for its columns of the first 16 partial outputs in one
        // go, makes the factors itself (the lanes of a warp read the same maxima and sums: one access) and adds
        // up: one trip through L2, no exchange through shared memory, no barrier.
        constexpr int PB = 16;
        const int n_out = gs * (HD / 4);
        for (int idx = threadIdx.x; idx < n_out; idx += AR_THREADS) {
          const int row = idx / (HD / 4), d4 = idx - row * (HD / 4);
          const size_t base = ((size_t)t * H + (size_t)g * gs + row) * p.splits;
          const float2* ml_g = reinterpret_cast<const float2*>(p.part_ml) + base;
          float2 mlv[PB];
          float4 pv[PB];
#pragma unroll
          for (int u = 0; u < PB; u++) {
            mlv[u] = u < p.splits ? __ldcg(ml_g + u) : make_float2(-INFINITY, 0.f);
            pv[u] = u < p.splits ? __ldcg(reinterpret_cast<const float4*>(p.part_o + (base + u) * HD) + d4)
                                 : make_float4(0.f, 0.f, 0.f, 0.f);
          }
          float M = -INFINITY;
#pragma unroll
          for (int u = 0; u < PB; u++) M = fmaxf(M, mlv[u].x);
          for (int s0 = PB; s0 < p.splits; s0++) M = fmaxf(M, __ldcg(ml_g + s0).x);      // more than 16 splits
          float Lsum = 0.f;
          float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
          for (int u = 0; u < PB; u++) {
            const float f = u < p.splits ? ar_exp2(mlv[u].x - M) : 0.f;
            Lsum += mlv[u].y * f;
            a.x += pv[u].x * f; a.y += pv[u].y * f; a.z += pv[u].z * f; a.w += pv[u].w * f;
          }
          for (int s0 = PB; s0 < p.splits; s0++) {
            const float2 v = __ldcg(ml_g + s0);
            const float4 o4 = __ldcg(reinterpret_cast<const float4*>(p.part_o + (base + s0) * HD) + d4);
            const float f = ar_exp2(v.x - M);
            Lsum += v.y * f;
            a.x += o4.x * f; a.y += o4.y * f; a.z += o4.z * f; a.w += o4.w * f;
          }
          const float inv = 1.f / Lsum;
          bf16* dst = p.out + (size_t)t * H * HD + ((size_t)g * gs + row) * HD + 4 * d4;
          uint2 raw;
          raw.x = ar_pack(a.x * inv, a.y * inv);
          raw.y = ar_pack(a.z * inv, a.w * inv);
          *reinterpret_cast<uint2*>(dst) = raw;
        }
        if (threadIdx.x == 0) p.tickets[(size_t)t * G + g] = 0;
        ar_stamp(p, 7);
      }
    }
    __syncthreads();
  }
}


template <int HD, int NS>
static int ar_launch_ns(const ArParams& p, cudaStream_t stream) {
  size_t smem = (size_t)16 * (HD + AR_PAD) * sizeof(bf16) + (size_t)AR_WARPS * NS * 2 * 16 * (HD + AR_PAD) * sizeof(bf16) +
                (size_t)AR_WARPS * 16 * 2 * sizeof(float) +
                (size_t)2 * HD * sizeof(bf16);
  auto kernel = decode_attention_rope_kernel<HD, NS>;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
    cudaGetLastError();
    return QD_ERR_UNSUPPORTED;
  }
  qd_launch(kernel, dim3((unsigned)(p.T * p.G * p.splits)), dim3(AR_THREADS), smem, stream, p);
  return (int)cudaGetLastError();
}

static int ar_sm_count() {
  static int sms[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 1;
  if (!sms[dev]) cudaDeviceGetAttribute(&sms[dev], cudaDevAttrMultiProcessorCount, dev);
  return sms[dev] > 0 ? sms[dev] : 1;
}

// Three chunks in flight per warp while every CTA has an SM of its own, else one (two CTAs per SM).
template <int HD>
static int ar_launch(const ArParams& p, cudaStream_t stream) {
  int stages = (long long)p.T * p.G * p.splits <= ar_sm_count() ? 3 : 1;
  if (const char* e = getenv("QD_DECODE_ROPE_STAGES")) stages = atoi(e);
  if (stages >= 3) return ar_launch_ns<HD, 3>(p, stream);
  return ar_launch_ns<HD, 1>(p, stream);
}

// One decoded token per request: q, k, v from partial sums, rotation, cache write and attention.
// Refuses head sizes other than 16..128 in steps as listed, more than 16 query heads per kv head, a
// page size that is no multiple of 16, more than 64 splits.
extern "C" int qd_decode_attention_rope(const float* part, int n_parts, const float* bias, bf16* out, bf16* kv,
                                        const int* block_table, int max_blocks, const int* token_req,
                                        const int* positions, const int* slot_map, int T, int H, int G, int d,
                                        int page_size, float scale, int window, int splits, int write_kv,
                                        const float* cos_t, const float* sin_t, int rotary_dim, int pairing,
                                        float* part_o, float* part_ml, unsigned* tickets, long long* timeline,
                                        cudaStream_t stream) {
  if (T < 1 || G < 1 || H % G != 0 || H / G > 16 || page_size % 16 != 0 || splits < 1 || splits > 64 || n_parts < 1)
    return QD_ERR_UNSUPPORTED;
  if ((rotary_dim & 1) || rotary_dim > d || (rotary_dim > 0 && (!cos_t || !sin_t))) return QD_ERR_UNSUPPORTED;
  if (splits > 1 && (!part_o || !part_ml || !tickets)) return QD_ERR_UNSUPPORTED;
  ArParams p;
  p.part = part; p.n_parts = n_parts; p.bias = bias; p.out = out; p.kv = kv;
  p.block_table = block_table; p.max_blocks = max_blocks; p.token_req = token_req; p.positions = positions;
  p.slot_map = slot_map; p.T = T; p.H = H; p.G = G; p.page_size = page_size; p.window = window; p.splits = splits;
  p.write_kv = write_kv; p.cos_t = rotary_dim > 0 ? cos_t : nullptr; p.sin_t = sin_t; p.rotary_dim = rotary_dim;
  p.pairing = pairing; p.scale_log2e = scale * 1.4426950408889634f;
  p.part_o = part_o; p.part_ml = part_ml; p.tickets = tickets; p.timeline = timeline;
  switch (d) {
    case 16: return ar_launch<16>(p, stream);
    case 32: return ar_launch<32>(p, stream);
    case 48: return ar_launch<48>(p, stream);
    case 64: return ar_launch<64>(p, stream);
    case 96: return ar_launch<96>(p, stream);
    case 128: return ar_launch<128>(p, stream);
    default: return QD_ERR_UNSUPPORTED;
  }
}
