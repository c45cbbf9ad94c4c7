// The allocation-free variant of decode attention: see decode_attention_noalloc.h for who
// needs it, what it costs and its rules.  The kernels are those of attention_flash.cu,
// compiled into this library a second time; only where the scratch comes from differs.
#include "attention_flash.cu"
#include "decode_attention_noalloc.h"

// The scratch itself: part of this library's device image on every GPU that loads it.
// In host code this name is only a handle for the runtime; the device address is looked up
// below.  Layout per call: T*H*splits*d floats of partial outputs, then T*H*splits*2 floats
// of (maximum, denominator) pairs.
static __device__ __align__(256) float qd_noalloc_scratch[QD_NOALLOC_SCRATCH_FLOATS];

#define QD_NOALLOC_MAX_DEVICES 64
static float* g_scratch_address[QD_NOALLOC_MAX_DEVICES];   // device address per device, 0 = not looked up yet

static int scratch_address(float** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= QD_NOALLOC_MAX_DEVICES) return QD_NOALLOC_SETUP_FAILED;
  if (!g_scratch_address[dev]) {
    float* p = nullptr;
    // with device `dev` current this gives the array's address on that device
    if (cudaGetSymbolAddress((void**)&p, qd_noalloc_scratch) != cudaSuccess || !p) {
      cudaGetLastError();
      return QD_NOALLOC_SETUP_FAILED;
    }
    g_scratch_address[dev] = p;
  }
  *out = g_scratch_address[dev];
  return QD_NOALLOC_OK;
}

extern "C" long long qd_decode_attention_noalloc_scratch_floats(int T, int H, int d, int splits) {
  if (T <= 0 || H <= 0 || d <= 0 || splits <= 1) return 0;
  return (long long)T * H * splits * (d + 2);
}

extern "C" int qd_decode_attention_noalloc(const void* q, long long q_stride, void* out, const void* kv,
                                           const int* block_table, int max_blocks, const int* token_req,
                                           const int* positions, int T, int H, int G, int d, int page_size,
                                           float scale, int window, int splits, cudaStream_t stream) {
  if (T <= 0) return QD_NOALLOC_OK;
  if (H <= 0 || d <= 0 || splits < 1) return QD_NOALLOC_BAD_ARGUMENT;
  long long need = qd_decode_attention_noalloc_scratch_floats(T, H, d, splits);
  if (need > (long long)QD_NOALLOC_SCRATCH_FLOATS) return QD_NOALLOC_TOO_LARGE;
  float* scratch = nullptr;
  int rc = scratch_address(&scratch);
  if (rc != QD_NOALLOC_OK) return rc;
  float* part_o = scratch;
  float* part_ml = scratch + (size_t)T * H * splits * d;
  // no ticket counters: the partial results are added up by the small second kernel, so this
  // entry point needs no state that must start at zero
  rc = qd_decode_attention(q, q_stride, out, kv, block_table, max_blocks, token_req, positions, T, H, G, d,
                           page_size, scale, window, splits, part_o, part_ml, nullptr, stream);
  return rc == QD_ERR_UNSUPPORTED ? QD_NOALLOC_BAD_ARGUMENT : rc;
}

extern "C" const char* qd_decode_attention_noalloc_strerror(int code) {
  switch (code) {
    case QD_NOALLOC_OK: return "success";
    case QD_NOALLOC_TOO_LARGE:
      return "the call needs more scratch than the library's fixed array holds "
             "(T * H * splits * (d + 2) floats must not exceed QD_NOALLOC_SCRATCH_FLOATS = 2097152): "
             "use fewer splits or fewer tokens per call";
    case QD_NOALLOC_BAD_ARGUMENT:
      return "sizes the decode attention kernel does not take (head size 16, 32, 48, 64, 96 or 128; up to 16 "
             "query heads per KV head; page size a multiple of 16; splits >= 1)";
    case QD_NOALLOC_SETUP_FAILED:
      return "the device address of the scratch array could not be looked up on the current device";
    default: return "CUDA error from the kernel launch";
  }
}
