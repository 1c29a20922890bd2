// Shared definitions for every kernel translation unit of the library.
//
// All entry points are plain C symbols that take raw device pointers and a
// CUDA stream handle; they return 0 on success or a UsStatus code.  Nothing in
// here depends on PyTorch, so a translation unit compiles in seconds.
#pragma once
#include <cuda_runtime.h>
#include <cstdlib>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

#define US_API extern "C" __attribute__((visibility("default")))

enum UsStatus : int {
  US_OK = 0,
  US_ERR_ARG = 1,       // argument rejected by the host-side check
  US_ERR_CUDA = 2,      // a CUDA runtime call failed (see us_last_cuda_error)
  US_ERR_TIMEOUT = 3,   // a bounded device wait ran out
  US_ERR_UNSUPPORTED = 4,
  US_ERR_LIMIT = 5,     // size beyond a stated maximum
};

// Device-side error codes written into the status word by kernels.
enum UsDevError : unsigned int {
  US_DEV_OK = 0,
  US_DEV_TIMEOUT_FULL = 0x100,   // consumer gave up waiting for a TMA stage
  US_DEV_TIMEOUT_EMPTY = 0x200,  // producer gave up waiting for a free stage
  US_DEV_TIMEOUT_ACC = 0x300,    // epilogue gave up waiting for the accumulator
  US_DEV_TIMEOUT_PEER = 0x400,   // a wait on another GPU's flag ran out
  US_DEV_BOUNDS = 0x500,         // an index fell outside its table
  US_DEV_TIMEOUT_GRID = 0x600,   // a wait on another CTA of the same grid ran out
};

#define US_CUDA_CHECK(expr)                                  \
  do {                                                       \
    cudaError_t _e = (expr);                                 \
    if (_e != cudaSuccess) {                                 \
      us_set_last_cuda_error((int)_e, __FILE__, __LINE__);   \
      return US_ERR_CUDA;                                    \
    }                                                        \
  } while (0)

#define US_LAUNCH_CHECK() US_CUDA_CHECK(cudaGetLastError())

#define US_REQUIRE(cond)                                     \
  do {                                                       \
    if (!(cond)) {                                           \
      us_set_last_cuda_error(-1, __FILE__, __LINE__);        \
      return US_ERR_ARG;                                     \
    }                                                        \
  } while (0)

extern "C" void us_set_last_cuda_error(int code, const char* file, int line);

// The library-wide device status word lives in memory that runtime.cu allocates
// once per device (us_status_ptr).  Kernels that can time out take the pointer
// as an argument and record the first error code with us_dev_fail(); the host
// reads and clears the word with us_status_read().
extern "C" unsigned int* us_status_ptr();

__device__ __forceinline__ void us_dev_fail(unsigned int* status, unsigned int code) {
  if (status) atomicCAS(status, 0u, code);
}

// Programmatic dependent launch: every kernel lets its dependents be launched as soon
// as it starts (their launch latency and prologue then overlap this kernel) and
// waits, as its first action, until the kernels it depends on have completed and
// their writes are visible.  Semantics are those of ordinary stream order.
#define US_PDL_PROLOGUE()                                           \
  do {                                                              \
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); \
    asm volatile("griddepcontrol.wait;" ::: "memory");              \
  } while (0)

namespace us {

// US_NO_PDL=1 launches every kernel with plain stream serialisation (A/B switch).
inline bool pdl_enabled() {
  static const bool on = [] {
    const char* e = getenv("US_NO_PDL");
    return !(e && e[0] == '1');
  }();
  return on;
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                              cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

template <typename T> struct Vec8;  // 8 x 16-bit values moved as one 16-byte access

__device__ __forceinline__ float bf2f(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ __nv_bfloat16 f2bf(float v) { return __float2bfloat16_rn(v); }

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

// Block-wide sum for blocks of up to 1024 threads; `scratch` holds 33 floats.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_sum(v);
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  const int nw = (blockDim.x + 31) >> 5;
  if (warp == 0) {
    float t = lane < nw ? scratch[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  float r = scratch[32];
  __syncthreads();
  return r;
}
__device__ __forceinline__ float block_max(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_max(v);
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  const int nw = (blockDim.x + 31) >> 5;
  if (warp == 0) {
    float t = lane < nw ? scratch[lane] : -INFINITY;
    t = warp_max(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  float r = scratch[32];
  __syncthreads();
  return r;
}

union Pack16 {
  uint4 u;
  __nv_bfloat16 b[8];
  __nv_bfloat162 b2[4];
};
union Pack8 {
  uint2 u;
  __nv_bfloat16 b[4];
};

__host__ __device__ __forceinline__ int ceil_div(int a, int b) { return (a + b - 1) / b; }

}  // namespace us
