// Shared helpers of the sm_100a kernels: element types, conversions, reductions.
//
// Every launcher is `extern "C"`, takes raw device pointers and a stream, launches
// on that stream and returns the `cudaGetLastError()` code (0 = success).  Element
// types are passed as a code: 0 = float32, 1 = bfloat16.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define QD_F32 0
#define QD_BF16 1

// Returned by launchers for arguments a kernel refuses (never a wrong result).
#define QD_ERR_UNSUPPORTED 10001

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(bf16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_float<bf16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over a block of up to 1024 threads; the order of additions depends only on
// the block size, so a row's result does not depend on what else is in the batch.
__device__ __forceinline__ float block_sum(float v, float* scratch /* >= 33 floats */) {
  int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nwarp ? scratch[lane] : 0.0f;
    t = warp_sum(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

static inline int qd_last_error() { return (int)cudaGetLastError(); }

// ---- programmatic dependent launch -------------------------------------------------
// Every kernel here is launched so that it may begin while the kernel before it in the
// stream is still running (cudaLaunchAttributeProgrammaticStreamSerialization).  A kernel
// first lets its own successor be scheduled (pdl_launch_dependents), may prefetch data that
// no kernel of the step writes (weights), and calls pdl_wait() before it reads or writes
// anything else: pdl_wait() returns when the preceding kernel has completed and its writes
// are visible.  This hides launch latency and first-load latency between the many small
// kernels of a decode step.  QD_PDL=0 in the environment turns the attribute off.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::); }

#include <stdlib.h>
static inline bool qd_pdl_enabled() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("QD_PDL");
    v = (e && e[0] == '0') ? 0 : 1;
  }
  return v == 1;
}

// Set by a library's ``plain_next`` entry point: its next launch goes without the attribute, that is with the
// stream's full ordering after everything before it.  For a kernel that reads what a library kernel wrote whose
// inner workings (several kernels? dependencies of their own among them?) this code cannot see.
static bool qd_plain_next_launch = false;

template <typename... KArgs, typename... Args>
static inline void qd_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                             Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = (qd_pdl_enabled() && !qd_plain_next_launch) ? 1 : 0;
  qd_plain_next_launch = false;
  cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// ---- bounded waits -----------------------------------------------------------------
// Every wait on an mbarrier in these kernels has a limit in polls and in time.  When it runs out the
// waiter sets ``*dead`` (no wait of its CTA spins again), the caller records which wait it was in the
// library's status word, and the kernel runs on to its end with void results: the host reads the
// status word (qd_<library>_status) and raises.  A kernel never hangs on a copy that did not arrive.
__device__ __forceinline__ bool qd_mbar_wait_bounded(unsigned bar_smem_addr, unsigned parity, volatile int* dead,
                                                     unsigned poll_limit, unsigned long long time_limit_ns,
                                                     unsigned backoff_ns = 0) {
  unsigned long long start = 0;
  for (unsigned spin = 0; spin < poll_limit; spin++) {
    if (backoff_ns && spin) __nanosleep(backoff_ns);     // long waits of many threads: leave the issue slots alone
    unsigned ok;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(ok) : "r"(bar_smem_addr), "r"(parity) : "memory");
    if (ok) return true;                                 // a phase that is complete costs one instruction
    if (*dead) return false;
    if ((spin & 255) == 255) {
      unsigned long long now;
      asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
      if (start == 0) start = now;
      else if (now - start > time_limit_ns) break;
    }
  }
  *dead = 1;
  return false;
}

// A probe of a library's wait, for tests: one warp waits, with ``poll_limit`` polls, on an mbarrier that
// nobody arrives at, through the library's own wait function; the wait must run out, the kernel must end
// and the library's status word must read ``code`` afterwards.  ``wait_expr`` may use ``bar`` (the
// barrier), ``dead`` and ``poll_limit``; ``status_fn`` returns the library's status word on the device.
#define QD_DEFINE_WAIT_PROBE(entry, wait_expr, status_fn, code)                                          \
  __global__ void entry##_kernel(int* status, unsigned poll_limit) {                                      \
    __shared__ unsigned long long bar_word;                                                               \
    __shared__ int dead_word;                                                                             \
    unsigned long long* bar = &bar_word;                                                                  \
    volatile int* dead = &dead_word;                                                                      \
    if (threadIdx.x == 0) {                                                                               \
      dead_word = 0;                                                                                      \
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"((unsigned)__cvta_generic_to_shared(bar)), "r"(1u)); \
    }                                                                                                     \
    __syncthreads();                                                                                      \
    if (!(wait_expr) && threadIdx.x == 0) atomicExch(status, code);                                       \
  }                                                                                                       \
  extern "C" int entry(unsigned poll_limit, cudaStream_t stream) {                                        \
    int* status = status_fn();                                                                            \
    if (!status) return QD_ERR_UNSUPPORTED;                                                               \
    entry##_kernel<<<1, 32, 0, stream>>>(status, poll_limit);                                             \
    return (int)cudaGetLastError();                                                                       \
  }
