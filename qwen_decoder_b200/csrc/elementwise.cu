// Row-wise kernels of the decoder step: embedding gather, residual add + RMSNorm,
// rotary position encoding fused with the write of K and V into cache pages, and
// the SwiGLU gate.  One template per kernel serves the float32 path and the
// bfloat16 path; all arithmetic is float32.
//
// What each replaces in the reference: embedding_kernel (gpu_kernels.cu:18-29),
// residual_kernel + rmsnorm_kernel (gpu_kernels.cu:136-146, 32-67), rope_kernel +
// kvcache_write_kernel (gpu_kernels.cu:82-133), swiglu_kernel (gpu_kernels.cu:149-160).
#include "common.cuh"
#include "entry_points.h"

// ---------------------------------------------------------------- embedding
// x[t, :] = table[tokens[t], :]; the residual stream x is float32 in both paths.
template <typename TW>
__global__ void embedding_kernel(float* __restrict__ x, const TW* __restrict__ table,
                                 const int* __restrict__ tokens, int D) {
  pdl_launch_dependents();
  pdl_wait();
  int t = blockIdx.x;
  const TW* row = table + (size_t)tokens[t] * D;
  float* out = x + (size_t)t * D;
  for (int i = threadIdx.x; i < D; i += blockDim.x) out[i] = to_float(row[i]);
}

extern "C" int qd_embedding(float* x, const void* table, int table_dtype, const int* tokens,
                            int T, int D, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (table_dtype == QD_F32)
    qd_launch(embedding_kernel<float>, dim3(T), dim3(256), 0, stream, x, (const float*)table, tokens, D);
  else if (table_dtype == QD_BF16)
    qd_launch(embedding_kernel<bf16>, dim3(T), dim3(256), 0, stream, x, (const bf16*)table, tokens, D);
  else
    return QD_ERR_UNSUPPORTED;
  return qd_last_error();
}

// ------------------------------------------------- residual add + RMSNorm
// For output row r (source row s = rows ? rows[r] : r):
//   v = x[s] + delta[s]            (float32; delta may be absent, or be n_parts float32 partial
//                                   sums [n_parts, T, D] that are added up here)
//   x[s] = v                       (if write_back)
//   out[r] = v / sqrt(mean(v^2) + eps) * w
// The sum of squares is taken in a fixed order that depends only on D.
template <typename TD, typename TO>
__global__ void add_rmsnorm_kernel(float* __restrict__ x, const TD* __restrict__ delta,
                                   const float* __restrict__ w, TO* __restrict__ out,
                                   const int* __restrict__ rows, int D, float eps, int write_back,
                                   int n_parts, size_t part_stride) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float sm[];  // D values + 33 scratch
  float* v = sm;
  float* scratch = sm + D;
  int r = blockIdx.x;
  size_t s = rows ? (size_t)rows[r] : (size_t)r;
  float* xr = x + s * D;
  float ss = 0.0f;
  for (int i = threadIdx.x; i < D; i += blockDim.x) {
    float a = xr[i];
    if (delta) {
      float dsum = to_float(delta[s * D + i]);
      for (int p = 1; p < n_parts; p++) dsum += to_float(delta[p * part_stride + s * D + i]);
      a += dsum;
    }
    v[i] = a;
    if (write_back && delta) xr[i] = a;
    ss += a * a;
  }
  ss = block_sum(ss, scratch);
  float inv = 1.0f / sqrtf(ss / (float)D + eps);
  TO* o = out + (size_t)r * D;
  for (int i = threadIdx.x; i < D; i += blockDim.x) o[i] = from_float<TO>(v[i] * inv * w[i]);
}

// The same with one or two float4 per thread held in registers (D a multiple of 4, D <= 8192):
// every load of a row is issued at once, so a few-row launch costs one memory round trip
// instead of one per element, which is what decode steps need.
template <typename TD, typename TO, int VPT>
__global__ void __launch_bounds__(1024)
add_rmsnorm_vec_kernel(float* __restrict__ x, const TD* __restrict__ delta, const float* __restrict__ w,
                       TO* __restrict__ out, const int* __restrict__ rows, int D, float eps, int write_back,
                       int n_parts, size_t part_stride) {
  pdl_launch_dependents();
  // the norm's weight does not come from the kernel before: it travels while that kernel is waited for, and is
  // no round trip of its own after the sum of squares
  const int n4 = D >> 2;
  float4 v[VPT], wv[VPT];
#pragma unroll
  for (int q = 0; q < VPT; q++) {
    const int i4 = threadIdx.x + q * blockDim.x;
    wv[q] = i4 < n4 ? reinterpret_cast<const float4*>(w)[i4] : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  pdl_wait();
  __shared__ float scratch[40];
  int r = blockIdx.x;
  size_t s = rows ? (size_t)rows[r] : (size_t)r;
  float ss = 0.f;
#pragma unroll
  for (int q = 0; q < VPT; q++) {
    int i4 = threadIdx.x + q * blockDim.x;
    v[q] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (i4 < n4) {
      float4 a = reinterpret_cast<const float4*>(x + s * D)[i4];
      if (delta) {
        if (sizeof(TD) == 4) {
          const float* dp = reinterpret_cast<const float*>(delta) + s * D;
          // partial sums in batches of 16: all loads of a batch are in flight together, the sum keeps
          // the order of the parts
          float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
          for (int p0 = 0; p0 < n_parts; p0 += 16) {
            float4 d[16];
#pragma unroll
            for (int u = 0; u < 16; u++)
              d[u] = p0 + u < n_parts ? reinterpret_cast<const float4*>(dp + (size_t)(p0 + u) * part_stride)[i4]
                                      : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int u = 0; u < 16; u++) { acc.x += d[u].x; acc.y += d[u].y; acc.z += d[u].z; acc.w += d[u].w; }
          }
          a.x += acc.x; a.y += acc.y; a.z += acc.z; a.w += acc.w;
        } else {
          const bf16* dp = reinterpret_cast<const bf16*>(delta) + s * D + 4 * (size_t)i4;
          uint2 raw = *reinterpret_cast<const uint2*>(dp);
          __nv_bfloat162 d0 = *reinterpret_cast<__nv_bfloat162*>(&raw.x);
          __nv_bfloat162 d1 = *reinterpret_cast<__nv_bfloat162*>(&raw.y);
          a.x += __low2float(d0); a.y += __high2float(d0); a.z += __low2float(d1); a.w += __high2float(d1);
        }
        if (write_back) reinterpret_cast<float4*>(x + s * D)[i4] = a;
      }
      v[q] = a;
      ss += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
    }
  }
  ss = block_sum(ss, scratch);
  float inv = 1.0f / sqrtf(ss / (float)D + eps);
#pragma unroll
  for (int q = 0; q < VPT; q++) {
    int i4 = threadIdx.x + q * blockDim.x;
    if (i4 < n4) {
      const float4 ww = wv[q];
      float o0 = v[q].x * inv * ww.x, o1 = v[q].y * inv * ww.y, o2 = v[q].z * inv * ww.z, o3 = v[q].w * inv * ww.w;
      if (sizeof(TO) == 4) {
        reinterpret_cast<float4*>(reinterpret_cast<float*>(out) + (size_t)r * D)[i4] = make_float4(o0, o1, o2, o3);
      } else {
        __nv_bfloat162 p0 = __floats2bfloat162_rn(o0, o1), p1 = __floats2bfloat162_rn(o2, o3);
        uint2 raw;
        raw.x = *reinterpret_cast<unsigned*>(&p0);
        raw.y = *reinterpret_cast<unsigned*>(&p1);
        *reinterpret_cast<uint2*>(reinterpret_cast<bf16*>(out) + (size_t)r * D + 4 * (size_t)i4) = raw;
      }
    }
  }
}

// The next launch of this library is ordered after all earlier work of its stream (no programmatic dependent launch).
extern "C" void qd_elementwise_plain_next() { qd_plain_next_launch = true; }

extern "C" int qd_add_rmsnorm(float* x, const void* delta, int delta_dtype, const float* w, void* out,
                              int out_dtype, const int* rows, int n_rows, int D, float eps,
                              int write_back, int n_parts, long long part_stride, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  size_t smem = (size_t)(D + 40) * sizeof(float);
  if (smem > 200 * 1024) return QD_ERR_UNSUPPORTED;
#define LAUNCH(TD, TO)                                                                          \
  do {                                                                                          \
    if (smem > 48 * 1024)                                                                       \
      cudaFuncSetAttribute(add_rmsnorm_kernel<TD, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                           (int)smem);                                                          \
    qd_launch(add_rmsnorm_kernel<TD, TO>, dim3(n_rows), dim3(256), smem, stream, x, (const TD*)delta, w, (TO*)out, rows, \
                                                              D, eps, write_back, n_parts,      \
                                                              (size_t)part_stride);             \
  } while (0)
  bool dbf = delta && delta_dtype == QD_BF16;
  if (delta && delta_dtype != QD_BF16 && delta_dtype != QD_F32) return QD_ERR_UNSUPPORTED;
  if (n_parts < 1 || (n_parts > 1 && delta_dtype != QD_F32)) return QD_ERR_UNSUPPORTED;
  if (out_dtype != QD_F32 && out_dtype != QD_BF16) return QD_ERR_UNSUPPORTED;
  bool aligned = !(((uintptr_t)x | (uintptr_t)delta | (uintptr_t)w | (uintptr_t)out) & 15) && part_stride % 4 == 0;
  if (D % 4 == 0 && D <= 8192 && aligned) {
    int n4 = D / 4;
    int vpt = n4 <= 1024 ? 1 : 2;
    int threads = ((n4 + vpt - 1) / vpt + 31) / 32 * 32;
#define VLAUNCH(TD, TO, V)                                                                              \
    qd_launch(add_rmsnorm_vec_kernel<TD, TO, V>, dim3(n_rows), dim3(threads), 0, stream, x, (const TD*)delta, w, (TO*)out, rows, D, \
                                                                      eps, write_back, n_parts, (size_t)part_stride)
#define VPICK(TD, TO) do { if (vpt == 1) VLAUNCH(TD, TO, 1); else VLAUNCH(TD, TO, 2); } while (0)
    if (out_dtype == QD_F32) { if (dbf) VPICK(bf16, float); else VPICK(float, float); }
    else { if (dbf) VPICK(bf16, bf16); else VPICK(float, bf16); }
#undef VPICK
#undef VLAUNCH
    return qd_last_error();
  }
  if (out_dtype == QD_F32) {
    if (dbf) LAUNCH(bf16, float); else LAUNCH(float, float);
  } else if (out_dtype == QD_BF16) {
    if (dbf) LAUNCH(bf16, bf16); else LAUNCH(float, bf16);
  } else {
    return QD_ERR_UNSUPPORTED;
  }
#undef LAUNCH
  return qd_last_error();
}

// x[t] += delta[t] with no norm after it (used when a residual is left pending at
// the end of a schedule that does not finish with a norm).
template <typename TD>
__global__ void residual_add_kernel(float* __restrict__ x, const TD* __restrict__ delta, size_t n, int n_parts) {
  pdl_launch_dependents();
  pdl_wait();
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float d = to_float(delta[i]);
  for (int p = 1; p < n_parts; p++) d += to_float(delta[p * n + i]);
  x[i] += d;
}

extern "C" int qd_residual_add(float* x, const void* delta, int delta_dtype, long long n, int n_parts,
                               cudaStream_t stream) {
  if (n <= 0) return 0;
  if (n_parts < 1) return QD_ERR_UNSUPPORTED;
  unsigned blocks = (unsigned)((n + 255) / 256);
  if (delta_dtype == QD_F32)
    qd_launch(residual_add_kernel<float>, dim3(blocks), dim3(256), 0, stream, x, (const float*)delta, (size_t)n, n_parts);
  else if (delta_dtype == QD_BF16 && n_parts == 1)
    qd_launch(residual_add_kernel<bf16>, dim3(blocks), dim3(256), 0, stream, x, (const bf16*)delta, (size_t)n, 1);
  else
    return QD_ERR_UNSUPPORTED;
  return qd_last_error();
}

// -------------------------------------------- rotary + K/V write into pages
// qkv row t = [ q (H*d) | k (G*d) | v (G*d) ].  q and k are rotated by the angle
// table row of positions[t]; q stays in place, k and v go to the token's slot of the
// layer's cache, laid out [page][K or V][kv head][offset in page][d].
// Pairing 0 rotates elements (2p, 2p+1) (the reference's rope_kernel,
// gpu_kernels.cu:94-100); pairing 1 rotates (p, p + rotary_dim/2).
// cos/sin are float32 tables [positions, rotary_dim/2]; a null table means "no rotation".
template <typename T>
__global__ void rope_kv_write_kernel(T* __restrict__ qkv, int H, int G, int d, int rotary_dim,
                                     int pairing, const float* __restrict__ cos_t,
                                     const float* __restrict__ sin_t,
                                     const int* __restrict__ positions, T* __restrict__ kv,
                                     const int* __restrict__ slot_map, int page_size, int write_kv) {
  pdl_launch_dependents();
  pdl_wait();
  int t = blockIdx.x;
  int row_w = (H + 2 * G) * d;
  T* row = qkv + (size_t)t * row_w;
  int half = rotary_dim >> 1;
  const float* c = cos_t ? cos_t + (size_t)positions[t] * half : nullptr;
  const float* s = cos_t ? sin_t + (size_t)positions[t] * half : nullptr;
  size_t kbase = 0, vbase = 0;
  int off = 0;
  if (write_kv) {
    int slot = slot_map[t];
    int page = slot / page_size;
    off = slot - page * page_size;
    kbase = (size_t)page * 2 * G * page_size * d;
    vbase = kbase + (size_t)G * page_size * d;
  }
  // One work item = one (head, pair) of q or k, or one (head, element pair) of v.
  int pairs_per_head = d >> 1;
  int n_qk = (H + G) * pairs_per_head;
  for (int w = threadIdx.x; w < n_qk; w += blockDim.x) {
    int head = w / pairs_per_head, p = w - head * pairs_per_head;
    T* hp = row + (size_t)head * d;  // q heads then k heads are contiguous in the row
    int i0, i1;
    bool rot = p < half;
    if (pairing == 0) { i0 = 2 * p; i1 = 2 * p + 1; }
    else if (rot)     { i0 = p; i1 = p + half; }
    else              { // elements beyond the rotated width pass through, two at a time
      int j = 2 * (p - half) + rotary_dim; i0 = j; i1 = j + 1; }
    if (pairing == 0) rot = (2 * p + 1) < rotary_dim;
    float a = to_float(hp[i0]), b = to_float(hp[i1]);
    float ra = a, rb = b;
    if (rot && c) {
      float cv = c[p], sv = s[p];
      ra = a * cv - b * sv;
      rb = a * sv + b * cv;
    }
    if (head < H) {
      hp[i0] = from_float<T>(ra);
      hp[i1] = from_float<T>(rb);
    } else if (write_kv) {
      int g = head - H;
      T* dst = kv + kbase + ((size_t)g * page_size + off) * d;
      dst[i0] = from_float<T>(ra);
      dst[i1] = from_float<T>(rb);
    }
  }
  if (write_kv) {
    const T* vrow = row + (size_t)(H + G) * d;
    for (int w = threadIdx.x; w < G * d; w += blockDim.x) {
      int g = w / d, i = w - g * d;
      kv[vbase + ((size_t)g * page_size + off) * d + i] = vrow[w];
    }
  }
}

// bfloat16, head size a multiple of 8: a thread takes 16 bytes (8 elements) of q, k or v of one token.
// pairing 0 (adjacent pairs, rotated width a multiple of 8): the piece holds four pairs, their cosines and
// sines are two float4.  pairing 1 (element i with i + rotary_dim / 2, rotated width a multiple of 16): the
// thread of a piece in the first half takes the partner piece of the second half as well; the partner's own
// thread has nothing to do.  ``bias`` (float32 [(H + 2G) d] or null) is added first and the sum rounded to
// bfloat16, as a product with a bias epilogue would leave it.
__device__ __forceinline__ void rkv_unpack(const uint4& raw, float (&f)[8]) {
  const unsigned* u = reinterpret_cast<const unsigned*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; i++) {
    __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(&u[i]);
    f[2 * i] = __low2float(v);
    f[2 * i + 1] = __high2float(v);
  }
}
__device__ __forceinline__ uint4 rkv_pack(const float (&f)[8]) {
  uint4 raw;
  unsigned* u = reinterpret_cast<unsigned*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; i++) {
    __nv_bfloat162 r = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    u[i] = *reinterpret_cast<unsigned*>(&r);
  }
  return raw;
}
__device__ __forceinline__ uint4 rkv_add_bias(const uint4& raw, const float* __restrict__ b) {
  float f[8];
  rkv_unpack(raw, f);
  const float4 b0 = *reinterpret_cast<const float4*>(b), b1 = *reinterpret_cast<const float4*>(b + 4);
  f[0] += b0.x; f[1] += b0.y; f[2] += b0.z; f[3] += b0.w;
  f[4] += b1.x; f[5] += b1.y; f[6] += b1.z; f[7] += b1.w;
  return rkv_pack(f);
}

__global__ void __launch_bounds__(256)
rope_kv_write_vec_kernel(bf16* __restrict__ qkv, const float* __restrict__ bias, int T, int H, int G, int d,
                         int rotary_dim, int pairing, const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                         const int* __restrict__ positions, bf16* __restrict__ kv,
                         const int* __restrict__ slot_map, int page_size, int write_kv) {
  pdl_launch_dependents();
  pdl_wait();
  const int per_row = (H + 2 * G) * d / 8;                 // 16-byte pieces per token
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)T * per_row) return;
  const int t = (int)(idx / per_row), piece = (int)(idx - (long long)t * per_row);
  const int head = piece / (d / 8), c8 = (piece - head * (d / 8)) * 8;      // element offset inside the head
  if (head >= H && !write_kv) return;
  const int half = rotary_dim >> 1;
  const bool rotated = head < H + G && cos_t && c8 < rotary_dim;
  if (rotated && pairing == 1 && c8 >= half) return;       // the thread of the first-half piece writes this one
  bf16* src = qkv + (size_t)t * (H + 2 * G) * d + (size_t)head * d + c8;
  // where the piece at offset c goes: q in place, k and v to the token's slot of the cache
  bf16* dst = src;
  if (head >= H) {
    const int slot = slot_map[t];
    const int page = slot / page_size, off = slot - page * page_size;
    const int g = head < H + G ? head - H : head - H - G;
    const size_t base = (size_t)page * 2 * G * page_size * d + (head < H + G ? 0 : (size_t)G * page_size * d);
    dst = kv + base + ((size_t)g * page_size + off) * d + c8;
  }
  uint4 raw = *reinterpret_cast<const uint4*>(src);
  if (bias) raw = rkv_add_bias(raw, bias + (size_t)head * d + c8);
  if (!rotated) {
    *reinterpret_cast<uint4*>(dst) = raw;
    return;
  }
  if (pairing == 0) {
    const size_t tab = (size_t)positions[t] * half + (c8 >> 1);
    const float4 cv = *reinterpret_cast<const float4*>(cos_t + tab), sv = *reinterpret_cast<const float4*>(sin_t + tab);
    const float cs[4] = {cv.x, cv.y, cv.z, cv.w}, sn[4] = {sv.x, sv.y, sv.z, sv.w};
    float f[8];
    rkv_unpack(raw, f);
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const float a = f[2 * i], b = f[2 * i + 1];
      f[2 * i] = a * cs[i] - b * sn[i];
      f[2 * i + 1] = a * sn[i] + b * cs[i];
    }
    *reinterpret_cast<uint4*>(dst) = rkv_pack(f);
    return;
  }
  // pairing 1: elements c8 .. c8+7 with c8+half .. c8+half+7, angles c8 .. c8+7
  uint4 raw2 = *reinterpret_cast<const uint4*>(src + half);
  if (bias) raw2 = rkv_add_bias(raw2, bias + (size_t)head * d + c8 + half);
  const size_t tab = (size_t)positions[t] * half + c8;
  const float4 c0 = *reinterpret_cast<const float4*>(cos_t + tab), c1 = *reinterpret_cast<const float4*>(cos_t + tab + 4);
  const float4 s0 = *reinterpret_cast<const float4*>(sin_t + tab), s1 = *reinterpret_cast<const float4*>(sin_t + tab + 4);
  const float cs[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
  const float sn[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
  float fa[8], fb[8];
  rkv_unpack(raw, fa);
  rkv_unpack(raw2, fb);
#pragma unroll
  for (int i = 0; i < 8; i++) {
    const float a = fa[i], b = fb[i];
    fa[i] = a * cs[i] - b * sn[i];
    fb[i] = a * sn[i] + b * cs[i];
  }
  *reinterpret_cast<uint4*>(dst) = rkv_pack(fa);
  *reinterpret_cast<uint4*>(dst + half) = rkv_pack(fb);
}

// what the vectorized kernel takes
static bool rope_vec_ok(const void* qkv, const float* bias, int d, int rotary_dim, int pairing, const float* cos_t,
                        const float* sin_t, const void* kv, int write_kv) {
  if (d % 8 != 0 || rotary_dim > d || rotary_dim < 0) return false;
  if (pairing == 0 ? rotary_dim % 8 != 0 : (pairing != 1 || rotary_dim % 16 != 0)) return false;
  if (((uintptr_t)qkv & 15) || ((uintptr_t)bias & 15) || (write_kv && ((uintptr_t)kv & 15))) return false;
  if (cos_t && (((uintptr_t)cos_t | (uintptr_t)sin_t) & 15)) return false;
  // pairing 1 reads eight table entries from an offset that is a multiple of 8 floats: rows of rotary_dim / 2
  // floats keep that 16-byte aligned only when rotary_dim / 2 is a multiple of 4 (it is a multiple of 8 here)
  return true;
}

extern "C" int qd_rope_kv_write(void* qkv, int dtype, int T, int H, int G, int d, int rotary_dim,
                                int pairing, const float* cos_t, const float* sin_t,
                                const int* positions, void* kv, const int* slot_map, int page_size,
                                int write_kv, cudaStream_t stream) {
  if (T <= 0) return 0;
  if ((d & 1) || (rotary_dim & 1) || rotary_dim > d || rotary_dim < 0) return QD_ERR_UNSUPPORTED;
  if (dtype == QD_F32)
    qd_launch(rope_kv_write_kernel<float>, dim3(T), dim3(256), 0, stream, (float*)qkv, H, G, d, rotary_dim, pairing, cos_t,
                                                       sin_t, positions, (float*)kv, slot_map,
                                                       page_size, write_kv);
  else if (dtype == QD_BF16 && rope_vec_ok(qkv, nullptr, d, rotary_dim, pairing, cos_t, sin_t, kv, write_kv)) {
    const long long pieces = (long long)T * (H + 2 * G) * d / 8;
    qd_launch(rope_kv_write_vec_kernel, dim3((unsigned)((pieces + 255) / 256)), dim3(256), 0, stream, (bf16*)qkv,
              (const float*)nullptr, T, H, G, d, rotary_dim, pairing, cos_t, sin_t, positions, (bf16*)kv, slot_map,
              page_size, write_kv);
  } else if (dtype == QD_BF16)
    qd_launch(rope_kv_write_kernel<bf16>, dim3(T), dim3(256), 0, stream, (bf16*)qkv, H, G, d, rotary_dim, pairing, cos_t,
                                                      sin_t, positions, (bf16*)kv, slot_map,
                                                      page_size, write_kv);
  else
    return QD_ERR_UNSUPPORTED;
  return qd_last_error();
}

// The vectorized kernel alone, with the projection's float32 bias [(H + 2G) d] added first (null: none):
// bfloat16, head size a multiple of 8, rotated width a multiple of 8 (adjacent pairs) or 16 (half-split pairs),
// 16-byte aligned pointers; refuses anything else.
extern "C" int qd_rope_kv_write_biased(void* qkv, const float* bias, int T, int H, int G, int d, int rotary_dim,
                                       int pairing, const float* cos_t, const float* sin_t, const int* positions,
                                       void* kv, const int* slot_map, int page_size, int write_kv,
                                       cudaStream_t stream) {
  if (T <= 0) return 0;
  if (!rope_vec_ok(qkv, bias, d, rotary_dim, pairing, cos_t, sin_t, kv, write_kv)) return QD_ERR_UNSUPPORTED;
  const long long pieces = (long long)T * (H + 2 * G) * d / 8;
  qd_launch(rope_kv_write_vec_kernel, dim3((unsigned)((pieces + 255) / 256)), dim3(256), 0, stream, (bf16*)qkv, bias, T,
            H, G, d, rotary_dim, pairing, cos_t, sin_t, positions, (bf16*)kv, slot_map, page_size, write_kv);
  return qd_last_error();
}

// The same from float32 partial sums: qkv[t] = sum_p part[p, t] + bias, as the few-token
// contraction leaves them.  q goes to a bfloat16 buffer of its own [T, H*d].
__global__ void rope_kv_write_partial_kernel(const float* __restrict__ part, int n_parts,
                                             const float* __restrict__ bias, bf16* __restrict__ q_out, int T,
                                             int H, int G, int d, int rotary_dim, int pairing,
                                             const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                             const int* __restrict__ positions, bf16* __restrict__ kv,
                                             const int* __restrict__ slot_map, int page_size, int write_kv) {
  pdl_launch_dependents();
  pdl_wait();
  // grid (token, block of pairs); one thread owns one pair of elements of q, k or v
  int t = blockIdx.x;
  int pairs_per_head = d >> 1;
  int w = blockIdx.y * blockDim.x + threadIdx.x;
  if (w >= (H + 2 * G) * pairs_per_head) return;
  int head = w / pairs_per_head, p = w - head * pairs_per_head;
  int row_w = (H + 2 * G) * d;
  size_t pstride = (size_t)T * row_w;
  const float* row = part + (size_t)t * row_w;
  int half = rotary_dim >> 1;
  int i0, i1;
  bool rot = p < half && head < H + G;
  if (head >= H + G || pairing == 0) { i0 = 2 * p; i1 = 2 * p + 1; }
  else if (p < half) { i0 = p; i1 = p + half; }
  else { int jj = 2 * (p - half) + rotary_dim; i0 = jj; i1 = jj + 1; }
  int e0 = head * d + i0, e1 = head * d + i1;
  float a = bias ? bias[e0] : 0.f, b = bias ? bias[e1] : 0.f;
#pragma unroll 4
  for (int q = 0; q < n_parts; q++) { a += row[q * pstride + e0]; b += row[q * pstride + e1]; }
  if (rot && cos_t) {
    float cv = cos_t[(size_t)positions[t] * half + p], sv = sin_t[(size_t)positions[t] * half + p];
    float ra = a * cv - b * sv, rb = a * sv + b * cv;
    a = ra; b = rb;
  }
  if (head < H) {
    bf16* dst = q_out + (size_t)t * H * d + (size_t)head * d;
    dst[i0] = __float2bfloat16_rn(a);
    dst[i1] = __float2bfloat16_rn(b);
  } else if (write_kv) {
    int slot = slot_map[t];
    int page = slot / page_size, off = slot - page * page_size;
    bool is_v = head >= H + G;
    int g = head - H - (is_v ? G : 0);
    bf16* dst = kv + (size_t)page * 2 * G * page_size * d + (is_v ? (size_t)G * page_size * d : 0) +
                ((size_t)g * page_size + off) * d;
    dst[i0] = __float2bfloat16_rn(a);
    dst[i1] = __float2bfloat16_rn(b);
  }
}

extern "C" int qd_rope_kv_write_partial(const float* part, int n_parts, const float* bias, void* q_out, int T,
                                        int H, int G, int d, int rotary_dim, int pairing, const float* cos_t,
                                        const float* sin_t, const int* positions, void* kv,
                                        const int* slot_map, int page_size, int write_kv, cudaStream_t stream) {
  if (T <= 0) return 0;
  if ((d & 1) || (rotary_dim & 1) || rotary_dim > d || rotary_dim < 0 || n_parts < 1) return QD_ERR_UNSUPPORTED;
  int work = (H + 2 * G) * (d / 2);
  dim3 grid(T, (work + 255) / 256);
  if (grid.y > 65535) return QD_ERR_UNSUPPORTED;
  qd_launch(rope_kv_write_partial_kernel, dim3(grid), dim3(256), 0, stream, part, n_parts, bias, (bf16*)q_out, T, H, G, d, rotary_dim,
                                                      pairing, cos_t, sin_t, positions, (bf16*)kv, slot_map,
                                                      page_size, write_kv);
  return qd_last_error();
}

// ------------------------------------------------------------------ SwiGLU
// gate_up row = [ gate (F) | up (F) ];  out = gate / (1 + exp(-gate)) * up, in float32
// (the reference's swiglu_kernel, gpu_kernels.cu:157-158).
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int F, size_t n) {
  // no early start for the successor: it is a library product (the down projection), which gains nothing from it
  pdl_wait();
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  size_t t = i / F;
  int f = (int)(i - t * F);
  float g = to_float(gate_up[t * 2 * F + f]);
  float u = to_float(gate_up[t * 2 * F + F + f]);
  out[i] = from_float<T>(g / (1.0f + expf(-g)) * u);
}

// Eight features per thread and step with 16-byte loads and stores (bfloat16, F a multiple of 8); a thread
// takes two steps, a grid apart, with all four loads in flight together.  The sigmoid uses the fast
// exponential and division: their error (2^-21 relative) is far below the rounding of the bfloat16 result.
__device__ __forceinline__ uint4 swiglu8(const uint4& g, const uint4& u) {
  const __nv_bfloat162* gp = reinterpret_cast<const __nv_bfloat162*>(&g);
  const __nv_bfloat162* up = reinterpret_cast<const __nv_bfloat162*>(&u);
  uint4 o;
  __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
  for (int k = 0; k < 4; k++) {
    float2 gf = __bfloat1622float2(gp[k]), uf = __bfloat1622float2(up[k]);
    op[k] = __floats2bfloat162_rn(__fdividef(gf.x, 1.0f + __expf(-gf.x)) * uf.x,
                                  __fdividef(gf.y, 1.0f + __expf(-gf.y)) * uf.y);
  }
  return o;
}

__global__ void swiglu_vec_kernel(const bf16* __restrict__ gate_up, bf16* __restrict__ out, int F8, size_t n8) {
  pdl_wait();        // as above: the successor is a library product
  const size_t half = (n8 + 1) / 2;
  const size_t i0 = (size_t)blockIdx.x * blockDim.x + threadIdx.x, i1 = i0 + half;
  if (i0 >= half) return;
  const uint4* base = reinterpret_cast<const uint4*>(gate_up);
  const size_t t0 = i0 / F8, t1 = i1 / F8;
  const int a0 = (int)(i0 - t0 * F8), a1 = (int)(i1 - t1 * F8);
  const bool two = i1 < n8;
  uint4 g0 = base[t0 * 2 * F8 + a0], u0 = base[t0 * 2 * F8 + F8 + a0];
  uint4 g1 = make_uint4(0, 0, 0, 0), u1 = g1;
  if (two) { g1 = base[t1 * 2 * F8 + a1]; u1 = base[t1 * 2 * F8 + F8 + a1]; }
  reinterpret_cast<uint4*>(out)[i0] = swiglu8(g0, u0);
  if (two) reinterpret_cast<uint4*>(out)[i1] = swiglu8(g1, u1);
}

// The same from the float32 partial sums of a split-K product: part [n_parts, T, 2F]; the shares are added
// first, exactly (float32), and the result is rounded to bfloat16 once.  Four features per thread with 16-byte
// loads, all shares of a thread's gate and up values asked for before any is used (in groups of four shares).
__global__ void swiglu_partial_kernel(const float* __restrict__ part, int n_parts, bf16* __restrict__ out, int F4,
                                      size_t n4, size_t part_stride4) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n4) return;
  const size_t t = i / F4;
  const int a = (int)(i - t * F4);
  const float4* base = reinterpret_cast<const float4*>(part) + t * 2 * F4 + a;
  float4 g = make_float4(0.f, 0.f, 0.f, 0.f), u = g;
  for (int p0 = 0; p0 < n_parts; p0 += 4) {
    float4 gv[4], uv[4];
#pragma unroll
    for (int q = 0; q < 4; q++) {
      const bool in = p0 + q < n_parts;
      gv[q] = in ? __ldcg(base + (size_t)(p0 + q) * part_stride4) : make_float4(0.f, 0.f, 0.f, 0.f);
      uv[q] = in ? __ldcg(base + (size_t)(p0 + q) * part_stride4 + F4) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int q = 0; q < 4; q++) {
      g.x += gv[q].x; g.y += gv[q].y; g.z += gv[q].z; g.w += gv[q].w;
      u.x += uv[q].x; u.y += uv[q].y; u.z += uv[q].z; u.w += uv[q].w;
    }
  }
  __nv_bfloat162 o0 = __floats2bfloat162_rn(g.x / (1.0f + expf(-g.x)) * u.x, g.y / (1.0f + expf(-g.y)) * u.y);
  __nv_bfloat162 o1 = __floats2bfloat162_rn(g.z / (1.0f + expf(-g.z)) * u.z, g.w / (1.0f + expf(-g.w)) * u.w);
  uint2 o;
  o.x = *reinterpret_cast<unsigned*>(&o0);
  o.y = *reinterpret_cast<unsigned*>(&o1);
  reinterpret_cast<uint2*>(out)[i] = o;
}

// out [T, F] bfloat16 = silu(sum_p part[p, t, f]) * (sum_p part[p, t, F + f]); F a multiple of 4, 16-byte aligned.
extern "C" int qd_swiglu_partial(const float* part, int n_parts, void* out, int T, int F, cudaStream_t stream) {
  if (T <= 0 || F <= 0) return 0;
  if (n_parts < 1 || F % 4 != 0 || (((uintptr_t)part) & 15) || (((uintptr_t)out) & 7)) return QD_ERR_UNSUPPORTED;
  const size_t n4 = (size_t)T * F / 4;
  qd_launch(swiglu_partial_kernel, dim3((unsigned)((n4 + 127) / 128)), dim3(128), 0, stream, part, n_parts, (bf16*)out,
            F / 4, n4, (size_t)T * 2 * F / 4);
  return qd_last_error();
}

extern "C" int qd_swiglu(const void* gate_up, void* out, int dtype, int T, int F, cudaStream_t stream) {
  size_t n = (size_t)T * F;
  if (n == 0) return 0;
  if (dtype == QD_BF16 && F % 8 == 0 && !(((uintptr_t)gate_up | (uintptr_t)out) & 15)) {
    size_t n8 = n / 8;
    qd_launch(swiglu_vec_kernel, dim3((unsigned)(((n8 + 1) / 2 + 255) / 256)), dim3(256), 0, stream, (const bf16*)gate_up,
              (bf16*)out, F / 8, n8);
    return qd_last_error();
  }
  unsigned blocks = (unsigned)((n + 255) / 256);
  if (dtype == QD_F32)
    qd_launch(swiglu_kernel<float>, dim3(blocks), dim3(256), 0, stream, (const float*)gate_up, (float*)out, F, n);
  else if (dtype == QD_BF16)
    qd_launch(swiglu_kernel<bf16>, dim3(blocks), dim3(256), 0, stream, (const bf16*)gate_up, (bf16*)out, F, n);
  else
    return QD_ERR_UNSUPPORTED;
  return qd_last_error();
}
