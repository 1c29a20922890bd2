// Library runtime: error reporting, the per-device status word that kernels
// with bounded waits write into, and TMA tensor-map encoding.
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdio.h>
#include <string.h>
#include <mutex>

#include "include/us_common.cuh"
#include "include/us_tmap.h"

namespace {
thread_local char g_err_text[512] = {0};
std::mutex g_mu;
constexpr int kMaxDevices = 64;
unsigned int* g_status[kMaxDevices] = {nullptr};

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;

EncodeTiledFn encode_fn() {
  if (g_encode) return g_encode;
  std::lock_guard<std::mutex> lock(g_mu);
  if (g_encode) return g_encode;
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) !=
          cudaSuccess ||
      q != cudaDriverEntryPointSuccess)
    return nullptr;
  g_encode = (EncodeTiledFn)fn;
  return g_encode;
}
}  // namespace

extern "C" void us_set_last_cuda_error(int code, const char* file, int line) {
  if (code >= 0)
    snprintf(g_err_text, sizeof(g_err_text), "%s:%d: CUDA error %d (%s)", file, line, code,
             cudaGetErrorString((cudaError_t)code));
  else
    snprintf(g_err_text, sizeof(g_err_text), "%s:%d: argument check failed", file, line);
}

extern "C" void us_set_last_error_text(const char* text) {
  snprintf(g_err_text, sizeof(g_err_text), "%s", text);
}

US_API const char* us_last_error() { return g_err_text; }

// Device pointer of the status word of the current device (allocated on first
// use; call once per device before any stream capture).
extern "C" __attribute__((visibility("default"))) unsigned int* us_status_ptr() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  if (g_status[dev]) return g_status[dev];
  std::lock_guard<std::mutex> lock(g_mu);
  if (g_status[dev]) return g_status[dev];
  unsigned int* p = nullptr;
  if (cudaMalloc(&p, 64) != cudaSuccess) return nullptr;
  cudaMemset(p, 0, 64);
  g_status[dev] = p;
  return p;
}

// Reads the status word (synchronises the device) and clears it.  The block's other words
// (the peer-wait budget at byte 8) stay.
US_API int us_status_read(unsigned int* out) {
  unsigned int* p = us_status_ptr();
  US_REQUIRE(p != nullptr && out != nullptr);
  US_CUDA_CHECK(cudaDeviceSynchronize());
  US_CUDA_CHECK(cudaMemcpy(out, p, sizeof(unsigned int), cudaMemcpyDeviceToHost));
  US_CUDA_CHECK(cudaMemset(p, 0, 8));
  return US_OK;
}

// Stream-ordered copy of the status word into (pinned) host memory: the serving loop reads
// it with the step's tokens, without a synchronisation of its own.
US_API int us_status_copy_async(unsigned int* host_out, void* stream) {
  unsigned int* p = us_status_ptr();
  US_REQUIRE(p != nullptr && host_out != nullptr);
  US_CUDA_CHECK(cudaMemcpyAsync(host_out, p, sizeof(unsigned int), cudaMemcpyDeviceToHost,
                                (cudaStream_t)stream));
  return US_OK;
}

// Stream-ordered clear of the status word (after a failed step was reported).
US_API int us_status_clear_async(void* stream) {
  unsigned int* p = us_status_ptr();
  US_REQUIRE(p != nullptr);
  US_CUDA_CHECK(cudaMemsetAsync(p, 0, 8, (cudaStream_t)stream));
  return US_OK;
}

// Budget (SM clocks) of every wait on another GPU's flag on the current device; 0 restores
// the default (about 1.5 s).  Takes effect for kernels launched after the call returns.
US_API int us_set_peer_wait_clocks(long long clocks) {
  unsigned int* p = us_status_ptr();
  US_REQUIRE(p != nullptr && clocks >= 0);
  US_CUDA_CHECK(cudaDeviceSynchronize());
  US_CUDA_CHECK(cudaMemcpy(p + 2, &clocks, sizeof(clocks), cudaMemcpyHostToDevice));
  return US_OK;
}

int us_tmap_encode(CUtensorMap* out, const void* base, int dtype, int rank, const uint64_t* dims,
                   const uint64_t* strides_bytes, const uint32_t* box, int swizzle) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) {
    us_set_last_cuda_error(-1, __FILE__, __LINE__);
    return US_ERR_CUDA;
  }
  CUtensorMapDataType dt;
  switch (dtype) {
    case US_TMAP_BF16: dt = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16; break;
    case US_TMAP_F16: dt = CU_TENSOR_MAP_DATA_TYPE_FLOAT16; break;
    case US_TMAP_U8: dt = CU_TENSOR_MAP_DATA_TYPE_UINT8; break;
    case US_TMAP_F32: dt = CU_TENSOR_MAP_DATA_TYPE_FLOAT32; break;
    default: return US_ERR_ARG;
  }
  CUtensorMapSwizzle sw;
  switch (swizzle) {
    case US_SWZ_NONE: sw = CU_TENSOR_MAP_SWIZZLE_NONE; break;
    case US_SWZ_32: sw = CU_TENSOR_MAP_SWIZZLE_32B; break;
    case US_SWZ_64: sw = CU_TENSOR_MAP_SWIZZLE_64B; break;
    case US_SWZ_128: sw = CU_TENSOR_MAP_SWIZZLE_128B; break;
    default: return US_ERR_ARG;
  }
  cuuint64_t gdims[5];
  cuuint64_t gstrides[4];
  cuuint32_t gbox[5];
  cuuint32_t estr[5];
  for (int i = 0; i < rank; ++i) {
    gdims[i] = dims[i];
    gbox[i] = box[i];
    estr[i] = 1;
    if (i < rank - 1) gstrides[i] = strides_bytes[i];
  }
  CUresult r = fn(out, dt, (cuuint32_t)rank, const_cast<void*>(base), gdims, gstrides, gbox, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    snprintf(g_err_text, sizeof(g_err_text),
             "cuTensorMapEncodeTiled failed (%d): base=%p rank=%d dims=[%llu,%llu,%llu] "
             "stride0=%llu box=[%u,%u,%u]",
             (int)r, base, rank, (unsigned long long)gdims[0],
             (unsigned long long)(rank > 1 ? gdims[1] : 0),
             (unsigned long long)(rank > 2 ? gdims[2] : 0),
             (unsigned long long)(rank > 1 ? gstrides[0] : 0), gbox[0], rank > 1 ? gbox[1] : 0,
             rank > 2 ? gbox[2] : 0);
    return US_ERR_CUDA;
  }
  return US_OK;
}

static int elem_bytes(int dtype) {
  switch (dtype) {
    case US_TMAP_BF16:
    case US_TMAP_F16: return 2;
    case US_TMAP_U8: return 1;
    default: return 4;
  }
}

int us_tmap_2d(CUtensorMap* out, const void* base, int dtype, uint64_t rows, uint64_t cols,
               uint64_t ld, uint32_t box_rows, uint32_t box_cols, int swizzle) {
  uint64_t dims[2] = {cols, rows};
  uint64_t strides[1] = {ld * (uint64_t)elem_bytes(dtype)};
  uint32_t box[2] = {box_cols, box_rows};
  return us_tmap_encode(out, base, dtype, 2, dims, strides, box, swizzle);
}

int us_tmap_3d(CUtensorMap* out, const void* base, int dtype, uint64_t batch, uint64_t rows,
               uint64_t cols, uint64_t ld, uint64_t batch_stride, uint32_t box_rows,
               uint32_t box_cols, int swizzle) {
  uint64_t dims[3] = {cols, rows, batch};
  uint64_t eb = (uint64_t)elem_bytes(dtype);
  uint64_t strides[2] = {ld * eb, batch_stride * eb};
  uint32_t box[3] = {box_cols, box_rows, 1};
  return us_tmap_encode(out, base, dtype, 3, dims, strides, box, swizzle);
}

US_API int us_device_info(int* sm_count, int* cc_major, int* cc_minor, size_t* smem_optin) {
  int dev = 0;
  US_CUDA_CHECK(cudaGetDevice(&dev));
  cudaDeviceProp p;
  US_CUDA_CHECK(cudaGetDeviceProperties(&p, dev));
  if (sm_count) *sm_count = p.multiProcessorCount;
  if (cc_major) *cc_major = p.major;
  if (cc_minor) *cc_minor = p.minor;
  if (smem_optin) *smem_optin = p.sharedMemPerBlockOptin;
  return US_OK;
}

// Plain device-to-device copy of raw addresses on a stream (either side may be a peer's
// memory mapped into this process: the copy engines move it over NVLink).
US_API int us_copy_async(void* dst, const void* src, long long bytes, void* stream) {
  US_REQUIRE(dst && src && bytes >= 0);
  if (bytes == 0) return US_OK;
  US_CUDA_CHECK(cudaMemcpyAsync(dst, src, (size_t)bytes, cudaMemcpyDefault, (cudaStream_t)stream));
  return US_OK;
}
