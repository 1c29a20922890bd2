// Paged KV cache utilities: the scaled FP8 page write and the page gather.
//
//   us_kv_write_scaled   rows of this launch -> E4M3 pages with one FP32 scale per page and
//                        plane; the write derives the scale from the values it stores and
//                        re-encodes the rows a page already holds when its scale grows
//   us_kv_gather         pages of a batch of sequences -> packed contiguous bf16 rows through
//                        the page table (bf16 or E4M3 pages), for prefill chunks that attend
//                        to cached context: no host-side page list, no host sync
//
// An FP8 plane is [pages, page_size, kv_heads, head_dim] bytes and scale[pages] floats; a
// stored byte b of page p means b * scale[p].  A page has ONE owner per launch: the first
// row of the launch's run of rows that fall into it (rows of one sequence are consecutive
// in a launch and a cache is only ever appended to, so the rows of a page are consecutive).
// The owner computes the largest magnitude of the run, grows the page's scale if needed,
// re-encodes rows [0, first offset) at the new scale, stores the run, and only then writes
// the scale.  A row at offset 0 starts the page afresh (its old scale is not read).
//
// Reference behaviour: crates/ops/src/kv.rs:24-29, crates/ops/kernels/kv_write_scaled
// (reference project paths).
#include "include/us_common.cuh"
#include <cuda_fp8.h>

namespace {

constexpr float kE4M3Max = 448.f;
constexpr float kScaleFloor = 1e-12f;

__device__ __forceinline__ unsigned char to_e4m3(float x) {
  return (unsigned char)__nv_cvt_float_to_fp8(fminf(fmaxf(x, -kE4M3Max), kE4M3Max), __NV_SATFINITE,
                                              __NV_E4M3);
}
__device__ __forceinline__ float from_e4m3(unsigned char b) {
  const __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)b, __NV_E4M3);
  return __half2float(*reinterpret_cast<const __half*>(&h));
}

// grid (rows, 2 planes); src row t of plane z at src_z + t * ld (heads * dim contiguous)
__global__ void __launch_bounds__(128)
kv_write_scaled_kernel(const __nv_bfloat16* __restrict__ k_src, const __nv_bfloat16* __restrict__ v_src,
                       long long ldk, long long ldv, const int* __restrict__ slots,
                       unsigned char* __restrict__ k_cache, unsigned char* __restrict__ v_cache,
                       float* __restrict__ k_scale, float* __restrict__ v_scale, int rows,
                       int page_size, int row_elems) {
  US_PDL_PROLOGUE();
  const int t = blockIdx.x;
  const int slot = slots[t];
  if (slot < 0) return;
  const int page = slot / page_size, off0 = slot - page * page_size;
  if (t > 0) {
    const int prev = slots[t - 1];
    if (prev >= 0 && prev / page_size == page) return;      // an earlier row owns the page
  }
  int n = 1;                                                 // rows of the run
  while (t + n < rows && n < page_size) {
    const int s = slots[t + n];
    if (s < 0 || s / page_size != page) break;
    ++n;
  }
  const bool plane_v = blockIdx.y == 1;
  const __nv_bfloat16* src = plane_v ? v_src : k_src;
  const long long ld = plane_v ? ldv : ldk;
  unsigned char* cache = (plane_v ? v_cache : k_cache) + (long long)page * page_size * row_elems;
  float* scale = (plane_v ? v_scale : k_scale) + page;

  __shared__ float red[4];
  __shared__ int offs[128];
  for (int i = threadIdx.x; i < n; i += 128) offs[i] = slots[t + i] - page * page_size;
  float amax = 0.f;
  for (int i = 0; i < n; ++i) {
    const __nv_bfloat16* r = src + (long long)(t + i) * ld;
    for (int e = threadIdx.x; e < row_elems; e += 128) amax = fmaxf(amax, fabsf(us::bf2f(r[e])));
  }
  amax = us::warp_max(amax);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  amax = fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3]));
  const float old = off0 > 0 ? *scale : 0.f;
  const float want = fmaxf(amax, kScaleFloor) / kE4M3Max;
  const float now = fmaxf(old, want);
  if (now > old && off0 > 0) {
    // the rows the page already holds move to the new scale
    const float f = old / now;
    for (int e = threadIdx.x; e < off0 * row_elems; e += 128) cache[e] = to_e4m3(from_e4m3(cache[e]) * f);
  }
  const float inv = 1.f / now;
  for (int i = 0; i < n; ++i) {
    const __nv_bfloat16* r = src + (long long)(t + i) * ld;
    unsigned char* d = cache + (long long)offs[i] * row_elems;
    for (int e = threadIdx.x; e < row_elems; e += 128) d[e] = to_e4m3(us::bf2f(r[e]) * inv);
  }
  __syncthreads();
  if (threadIdx.x == 0) *scale = now;
}

// Packed context rows of a batch: sequence s contributes rows [0, cu[s + 1] - cu[s]) of its
// pages to out rows [out_cu[s], ...) (out_cu = cu unless the caller leaves room behind each
// sequence's cached rows for its new ones).  grid (row tiles of 8, 2 planes); a warp moves
// one row.
__global__ void __launch_bounds__(256)
kv_gather_kernel(const void* __restrict__ k_cache, const void* __restrict__ v_cache,
                 const float* __restrict__ k_scale, const float* __restrict__ v_scale,
                 const int* __restrict__ page_table, int max_pages, const int* __restrict__ cu,
                 const int* __restrict__ out_cu, int B, int page_size, int row_elems, __nv_bfloat16* __restrict__ k_out,
                 __nv_bfloat16* __restrict__ v_out, long long ldo, int fp8) {
  US_PDL_PROLOGUE();
  const int total = cu[B];
  const int r = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (r >= total) return;
  int lo = 0, hi = B - 1;                       // sequence of packed row r
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (cu[mid] <= r) lo = mid; else hi = mid - 1;
  }
  const int pos = r - cu[lo];
  const int pi = pos / page_size;
  if (pi >= max_pages) return;
  const int page = page_table[(long long)lo * max_pages + pi];
  const long long src_row = (long long)page * page_size + (pos - pi * page_size);
  const bool plane_v = blockIdx.y == 1;
  __nv_bfloat16* out = (plane_v ? v_out : k_out) + (long long)(out_cu[lo] + pos) * ldo;
  if (fp8) {
    const unsigned char* src = (const unsigned char*)(plane_v ? v_cache : k_cache) + src_row * row_elems;
    const float sc = (plane_v ? v_scale : k_scale)[page];
    for (int e = lane * 8; e < row_elems; e += 256) {
      const uint2 raw = *reinterpret_cast<const uint2*>(src + e);
      const unsigned char* b = reinterpret_cast<const unsigned char*>(&raw);
      uint32_t o[4];
#pragma unroll
      for (int j = 0; j < 4; ++j)
        o[j] = (uint32_t)__bfloat16_as_ushort(us::f2bf(from_e4m3(b[2 * j]) * sc)) |
               ((uint32_t)__bfloat16_as_ushort(us::f2bf(from_e4m3(b[2 * j + 1]) * sc)) << 16);
      *reinterpret_cast<uint4*>(out + e) = make_uint4(o[0], o[1], o[2], o[3]);
    }
  } else {
    const __nv_bfloat16* src = (const __nv_bfloat16*)(plane_v ? v_cache : k_cache) + src_row * row_elems;
    for (int e = lane * 8; e < row_elems; e += 256)
      *reinterpret_cast<uint4*>(out + e) = *reinterpret_cast<const uint4*>(src + e);
  }
}

}  // namespace

US_API int us_kv_write_scaled(const void* k_src, const void* v_src, long long ldk, long long ldv,
                              const int* slots, void* k_cache, void* v_cache, float* k_scale,
                              float* v_scale, int rows, int page_size, int heads, int head_dim,
                              void* stream_) {
  US_REQUIRE(k_src && v_src && slots && k_cache && v_cache && k_scale && v_scale);
  US_REQUIRE(page_size >= 1 && page_size <= 128 && heads >= 1 && head_dim >= 1);
  if (rows == 0) return US_OK;
  US_CUDA_CHECK(us::launch_pdl(kv_write_scaled_kernel, dim3(rows, 2), dim3(128), 0,
                               (cudaStream_t)stream_, (const __nv_bfloat16*)k_src,
                               (const __nv_bfloat16*)v_src, ldk, ldv, slots, (unsigned char*)k_cache,
                               (unsigned char*)v_cache, k_scale, v_scale, rows, page_size,
                               heads * head_dim));
  return US_OK;
}

// `total_rows` bounds the grid (the sum of the context lengths, known to the host from the
// scheduler's plan; the device reads the exact layout from `cu`).
US_API int us_kv_gather(const void* k_cache, const void* v_cache, const float* k_scale,
                        const float* v_scale, const int* page_table, int max_pages, const int* cu,
                        const int* out_cu, int B, int total_rows, int page_size, int heads, int head_dim, void* k_out,
                        void* v_out, long long ldo, int fp8, void* stream_) {
  US_REQUIRE(k_cache && v_cache && page_table && cu && k_out && v_out && B >= 1);
  US_REQUIRE(((heads * head_dim) % 8) == 0 && (ldo % 8) == 0 && (!fp8 || (k_scale && v_scale)));
  if (total_rows == 0) return US_OK;
  US_CUDA_CHECK(us::launch_pdl(kv_gather_kernel, dim3((total_rows + 7) / 8, 2), dim3(256), 0,
                               (cudaStream_t)stream_, k_cache, v_cache, k_scale, v_scale, page_table,
                               max_pages, cu, out_cu ? out_cu : cu, B, page_size, heads * head_dim,
                               (__nv_bfloat16*)k_out, (__nv_bfloat16*)v_out, ldo, fp8));
  return US_OK;
}
