// Video sparse attention: the kernels that choose the key tiles each query tile
// attends, and the compressed branch that stands for the tiles it does not.
// Rows are [tiles * 128, heads, 128] bf16 with a row stride; tile tables stay on
// the device, so a captured graph replays the selection.
//
//   vsa_pool_tiles       zero each tile's rows past its valid size (q, k, v in place)
//                        and pool each tile's per-head means into FP32
//   vsa_scores           scores[h, i, j] = <mean_q[i, h], mean_k[j, h]> / sqrt(width)
//   vsa_select_tiles     per (head, query tile): keep every live tile outside the
//                        segments and, of each segment, its `keep` best tiles (ties to
//                        the lower tile); kept tiles first, each part ascending
//   vsa_compress_pooled  softmax over the live tiles of the pooled scores, weighting the
//                        pooled values
//   vsa_add_gated_tiles  fine += compressed[:, tile] * gate, product and sum each
//                        rounded to bf16
//
// Reference behaviour: crates/ops/src/vsa.rs:1-21, crates/nn/src/functional/vsa.rs:1-30,
// crates/ops/kernels/vsa_*/triton (reference project paths).
#include "include/us_common.cuh"

namespace {

constexpr int kTile = 128;
constexpr int kW = 128;

__global__ void __launch_bounds__(kW)
vsa_pool_tiles_kernel(__nv_bfloat16* __restrict__ q, __nv_bfloat16* __restrict__ k,
                      __nv_bfloat16* __restrict__ v, long long ldq, long long ldk, long long ldv,
                      const int* __restrict__ sizes, float* __restrict__ pq,
                      float* __restrict__ pk, float* __restrict__ pv, int heads) {
  US_PDL_PROLOGUE();
  const int tile = blockIdx.x, h = blockIdx.y, w = threadIdx.x;
  const int size = min(max(sizes[tile], 0), kTile);
  __nv_bfloat16* ptrs[3] = {q, k, v};
  const long long lds[3] = {ldq, ldk, ldv};
  float* outs[3] = {pq, pk, pv};
#pragma unroll
  for (int t = 0; t < 3; ++t) {
    if (ptrs[t] == nullptr) continue;
    __nv_bfloat16* base = ptrs[t] + (long long)tile * kTile * lds[t] + (long long)h * kW + w;
    float s = 0.f;
    for (int r = 0; r < size; ++r) s += us::bf2f(base[(long long)r * lds[t]]);
    for (int r = size; r < kTile; ++r) base[(long long)r * lds[t]] = us::f2bf(0.f);
    if (outs[t]) outs[t][((long long)tile * heads + h) * kW + w] = size > 0 ? s / (float)size : 0.f;
  }
}

__global__ void __launch_bounds__(256)
vsa_scores_kernel(const float* __restrict__ pq, const float* __restrict__ pk,
                  float* __restrict__ scores, int q_tiles, int tiles, int heads) {
  US_PDL_PROLOGUE();
  __shared__ float4 qrow[kW / 4];
  const int i = blockIdx.x, h = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x < kW / 4)
    qrow[threadIdx.x] =
        reinterpret_cast<const float4*>(pq + ((long long)i * heads + h) * kW)[threadIdx.x];
  __syncthreads();
  const float4 a = qrow[lane];
  const float inv_root = rsqrtf((float)kW);
  for (int j = warp; j < tiles; j += 8) {
    const float4 b = reinterpret_cast<const float4*>(pk + ((long long)j * heads + h) * kW)[lane];
    float d = a.x * b.x + a.y * b.y + a.z * b.z + a.w * b.w;
    d = us::warp_sum(d);
    if (lane == 0) scores[((long long)h * q_tiles + i) * tiles + j] = d * inv_root;
  }
}

__device__ __forceinline__ uint32_t order_key(float f) {
  if (f != f) return 0xffffffffu;
  const uint32_t u = __float_as_uint(f + 0.f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

constexpr int kMaxTiles = 2048;

__global__ void __launch_bounds__(256)
vsa_select_tiles_kernel(const float* __restrict__ scores, const int* __restrict__ sizes,
                        const int* __restrict__ segments, const int* __restrict__ keep,
                        int* __restrict__ indices, int* __restrict__ counts, int q_tiles,
                        int tiles, int query_offset) {
  US_PDL_PROLOGUE();
  __shared__ uint32_t key[kMaxTiles];
  __shared__ short seg[kMaxTiles];
  __shared__ unsigned char kept[kMaxTiles];
  __shared__ int n_kept;
  const int i = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
  const float* row = scores + ((long long)h * q_tiles + i) * tiles;
  for (int j = tid; j < tiles; j += 256) {
    key[j] = order_key(row[j]);
    seg[j] = sizes[j] > 0 ? (short)max(min(segments[j], 32000), -1) : (short)-2;  // -2 = dead
  }
  __syncthreads();
  const int qt = query_offset + i;
  const bool q_live = sizes[qt] > 0;
  const bool q_in_segment = segments[qt] >= 0;
  for (int j = tid; j < tiles; j += 256) {
    const int sj = seg[j];
    bool kp;
    if (!q_live || sj == -2) {
      kp = false;
    } else if (!q_in_segment || sj < 0) {
      kp = true;
    } else {
      const uint32_t kj = key[j];
      const int limit = keep[sj];
      int ahead = 0;
      for (int t = 0; t < tiles && ahead < limit; ++t)
        if (seg[t] == sj && (key[t] > kj || (key[t] == kj && t < j))) ++ahead;
      kp = ahead < limit;
    }
    kept[j] = kp ? 1 : 0;
  }
  __syncthreads();
  // Warp 0 compacts: kept tiles ascending, then the rest ascending.
  if (tid < 32) {
    int total = 0;
    for (int base = 0; base < tiles; base += 32) {
      const int j = base + tid;
      const unsigned m = __ballot_sync(0xffffffffu, j < tiles && kept[j]);
      total += __popc(m);
    }
    int* out = indices + ((long long)h * q_tiles + i) * tiles;
    int pk = 0, pr = total;
    for (int base = 0; base < tiles; base += 32) {
      const int j = base + tid;
      const bool in = j < tiles;
      const bool kp = in && kept[j];
      const unsigned mk = __ballot_sync(0xffffffffu, kp);
      const unsigned mr = __ballot_sync(0xffffffffu, in && !kp);
      const unsigned below = (1u << tid) - 1u;
      if (kp) out[pk + __popc(mk & below)] = j;
      if (in && !kp) out[pr + __popc(mr & below)] = j;
      pk += __popc(mk);
      pr += __popc(mr);
    }
    if (tid == 0) n_kept = total;
    if (tid == 0) counts[h * q_tiles + i] = total;
  }
}

__global__ void __launch_bounds__(kW)
vsa_compress_pooled_kernel(const float* __restrict__ scores, const float* __restrict__ pv,
                           const int* __restrict__ sizes, __nv_bfloat16* __restrict__ out,
                           int q_tiles, int tiles, int heads) {
  US_PDL_PROLOGUE();
  __shared__ float wgt[kMaxTiles];
  __shared__ float scratch[33];
  const int i = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
  const float* row = scores + ((long long)h * q_tiles + i) * tiles;
  float mx = -INFINITY;
  for (int j = tid; j < tiles; j += kW) {
    const float s = sizes[j] > 0 ? row[j] : -INFINITY;
    wgt[j] = s;
    mx = fmaxf(mx, s);
  }
  mx = us::block_max(mx, scratch);
  float sum = 0.f;
  for (int j = tid; j < tiles; j += kW) {
    const float e = wgt[j] == -INFINITY ? 0.f : __expf(wgt[j] - mx);
    wgt[j] = e;
    sum += e;
  }
  sum = us::block_sum(sum, scratch);
  __syncthreads();
  const float inv = sum > 0.f ? 1.f / sum : 0.f;
  float acc = 0.f;
  for (int j = 0; j < tiles; ++j) {
    const float wj = wgt[j];
    if (wj != 0.f) acc += wj * pv[((long long)j * heads + h) * kW + tid];
  }
  out[((long long)h * q_tiles + i) * kW + tid] = us::f2bf(acc * inv);
}

__global__ void __launch_bounds__(256)
vsa_add_gated_tiles_kernel(__nv_bfloat16* __restrict__ fine, long long ldf,
                           const __nv_bfloat16* __restrict__ compressed,
                           const __nv_bfloat16* __restrict__ gate, long long ldg, int rows,
                           int heads, int q_tiles, int tile_offset) {
  US_PDL_PROLOGUE();
  const long long per_row = (long long)heads * kW / 8;
  const long long total = (long long)rows * per_row;
  for (long long u = (long long)blockIdx.x * blockDim.x + threadIdx.x; u < total;
       u += (long long)gridDim.x * blockDim.x) {
    const int r = (int)(u / per_row);
    const int c = (int)(u % per_row) * 8;   // channel within the row
    const int h = c / kW, w = c % kW;
    const int tile = r / kTile + tile_offset;
    us::Pack16 f, g, z, o;
    f.u = *reinterpret_cast<const uint4*>(fine + (long long)r * ldf + c);
    g.u = *reinterpret_cast<const uint4*>(gate + (long long)r * ldg + c);
    z.u = *reinterpret_cast<const uint4*>(compressed + ((long long)h * q_tiles + tile) * kW + w);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float prod = us::bf2f(us::f2bf(us::bf2f(z.b[i]) * us::bf2f(g.b[i])));
      o.b[i] = us::f2bf(us::bf2f(f.b[i]) + prod);
    }
    *reinterpret_cast<uint4*>(fine + (long long)r * ldf + c) = o.u;
  }
}

}  // namespace

US_API int us_vsa_pool_tiles(void* q, void* k, void* v, long long ldq, long long ldk,
                             long long ldv, const int* sizes, float* pq, float* pk, float* pv,
                             int tiles, int heads, int width, void* stream) {
  US_REQUIRE(sizes && tiles >= 0 && heads >= 1 && width == kW);
  if (tiles == 0) return US_OK;
  US_CUDA_CHECK(us::launch_pdl(vsa_pool_tiles_kernel, dim3(tiles, heads), dim3(kW), 0,
                               (cudaStream_t)stream, (__nv_bfloat16*)q, (__nv_bfloat16*)k,
                               (__nv_bfloat16*)v, ldq, ldk, ldv, sizes, pq, pk, pv, heads));
  return US_OK;
}

US_API int us_vsa_scores(const float* pq, const float* pk, float* scores, int q_tiles, int tiles,
                         int heads, int width, void* stream) {
  US_REQUIRE(pq && pk && scores && q_tiles >= 1 && tiles >= 1 && heads >= 1 && width == kW);
  US_CUDA_CHECK(us::launch_pdl(vsa_scores_kernel, dim3(q_tiles, heads), dim3(256), 0,
                               (cudaStream_t)stream, pq, pk, scores, q_tiles, tiles, heads));
  return US_OK;
}

US_API int us_vsa_select_tiles(const float* scores, const int* sizes, const int* segments,
                               const int* keep, int* indices, int* counts, int heads, int q_tiles,
                               int tiles, int query_offset, void* stream) {
  US_REQUIRE(scores && sizes && segments && keep && indices && counts && heads >= 1 &&
             q_tiles >= 1 && tiles >= 1 && tiles <= kMaxTiles && query_offset >= 0 &&
             query_offset + q_tiles <= tiles);
  US_CUDA_CHECK(us::launch_pdl(vsa_select_tiles_kernel, dim3(q_tiles, heads), dim3(256), 0,
                               (cudaStream_t)stream, scores, sizes, segments, keep, indices,
                               counts, q_tiles, tiles, query_offset));
  return US_OK;
}

US_API int us_vsa_compress_pooled(const float* scores, const float* pv, const int* sizes,
                                  void* out, int heads, int q_tiles, int tiles, int width,
                                  void* stream) {
  US_REQUIRE(scores && pv && sizes && out && heads >= 1 && q_tiles >= 1 && tiles >= 1 &&
             tiles <= kMaxTiles && width == kW);
  US_CUDA_CHECK(us::launch_pdl(vsa_compress_pooled_kernel, dim3(q_tiles, heads), dim3(kW), 0,
                               (cudaStream_t)stream, scores, pv, sizes, (__nv_bfloat16*)out,
                               q_tiles, tiles, heads));
  return US_OK;
}

US_API int us_vsa_add_gated_tiles(void* fine, long long ldf, const void* compressed,
                                  const void* gate, long long ldg, int rows, int heads, int width,
                                  int q_tiles, int tile_offset, void* stream) {
  US_REQUIRE(fine && compressed && gate && rows >= 0 && heads >= 1 && width == kW &&
             (ldf % 8) == 0 && (ldg % 8) == 0 && (rows % kTile) == 0);
  if (rows == 0) return US_OK;
  const long long units = (long long)rows * heads * kW / 8;
  int blocks = (int)((units + 255) / 256);
  if (blocks > 148 * 16) blocks = 148 * 16;
  US_CUDA_CHECK(us::launch_pdl(vsa_add_gated_tiles_kernel, dim3(blocks), dim3(256), 0,
                               (cudaStream_t)stream, (__nv_bfloat16*)fine, ldf,
                               (const __nv_bfloat16*)compressed, (const __nv_bfloat16*)gate, ldg,
                               rows, heads, q_tiles, tile_offset));
  return US_OK;
}
