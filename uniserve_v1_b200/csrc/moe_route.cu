// Mixture-of-experts routing kernels.
//
//   topk_softmax   softmax over all experts -> top-k by repeated argmax (ties to
//                  the lower id) -> optional renormalisation (sum clamped at
//                  FLT_EPSILON) -> ids through an optional logical->physical map,
//                  expert-load counters by logical id.  Rows at or past the
//                  device word `live` route nowhere (id -1, weight 0).
//   moe_sort       counting sort of the (token, route) pairs by local expert;
//                  emits the permutation both ways, the expert offsets and the
//                  list of row tiles the grouped GEMM walks.
//   moe_gather     permuted activation rows  xp[p] = x[route(p) / top_k].
//   moe_unpermute  out[t] = sum_j w[t, j] * y[perm(t, j)]  in FP32, one rounding.
//
// Reference behaviour: crates/ops/kernels/topk_softmax/nvcc/src/topk_softmax.cu:1-27,
// crates/nn/src/functional/moe.rs:301-330, crates/ops/kernels/moe_unpermute
// (reference project paths).
#include <float.h>

#include "include/us_common.cuh"

namespace {

constexpr int kMaxExperts = 1024;
constexpr int kMaxPerLane = kMaxExperts / 32;

// Softmax, top-k and renormalisation of one token's router logits by one warp.
template <int PER_LANE>
__device__ __forceinline__ void topk_token(const float* __restrict__ logits,
                                           int* __restrict__ ids, float* __restrict__ weights,
                                           int t, int E, int top_k, int renorm,
                                           const int* __restrict__ live,
                                           const int* __restrict__ expert_map,
                                           int* __restrict__ load) {
  const int lane = threadIdx.x & 31;
  if (live && t >= *live) {
    for (int j = lane; j < top_k; j += 32) {
      ids[(long long)t * top_k + j] = -1;
      weights[(long long)t * top_k + j] = 0.f;
    }
    return;
  }
  const float* row = logits + (long long)t * E;
  float v[PER_LANE];
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < PER_LANE; ++i) {
    const int e = lane + 32 * i;
    v[i] = e < E ? row[e] : -INFINITY;
    mx = fmaxf(mx, v[i]);
  }
  mx = us::warp_max(mx);
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < PER_LANE; ++i) {
    v[i] = (lane + 32 * i) < E ? __expf(v[i] - mx) : -1.f;
    if (v[i] > 0.f) sum += v[i];
  }
  sum = us::warp_sum(sum);
  const float inv = 1.f / sum;
  float picked_sum = 0.f;
  float my_w = 0.f;
  int my_id = -1;
  for (int j = 0; j < top_k; ++j) {
    float best = -1.f;
    int best_e = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < PER_LANE; ++i) {
      const int e = lane + 32 * i;
      if (v[i] > best) {  // ascending e inside a lane keeps the lower id on ties
        best = v[i];
        best_e = e;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
      if (ob > best || (ob == best && oe < best_e)) {
        best = ob;
        best_e = oe;
      }
    }
    const float p = best * inv;
    picked_sum += p;
    if (lane == j) {
      my_w = p;
      my_id = best_e;
    }
    if ((best_e & 31) == lane) {
#pragma unroll
      for (int i = 0; i < PER_LANE; ++i)
        if (i == (best_e >> 5)) v[i] = -1.f;
    }
  }
  if (lane < top_k) {
    if (renorm) my_w = my_w / fmaxf(picked_sum, FLT_EPSILON);
    if (load) atomicAdd(&load[my_id], 1);
    ids[(long long)t * top_k + lane] = expert_map ? expert_map[my_id] : my_id;
    weights[(long long)t * top_k + lane] = my_w;
  }
}

template <int PER_LANE>
__global__ void __launch_bounds__(128)
topk_softmax_kernel(const float* __restrict__ logits, int* __restrict__ ids,
                    float* __restrict__ weights, int T, int E, int top_k, int renorm,
                    const int* __restrict__ live, const int* __restrict__ expert_map,
                    int* __restrict__ load) {
  US_PDL_PROLOGUE();
  const int t = blockIdx.x * 4 + (threadIdx.x >> 5);
  if (t >= T) return;
  topk_token<PER_LANE>(logits, ids, weights, t, E, top_k, renorm, live, expert_map, load);
}

// One CTA sorts all routes.  Local experts are [e_lo, e_lo + E).
__device__ __forceinline__ void
sort_routes(const int* __restrict__ ids, int R, int e_lo, int E, int block_n, int max_tiles,
            int* __restrict__ sorted_route, int* __restrict__ perm_of_route,
            int* __restrict__ expert_offsets, int* __restrict__ tile_group,
            int* __restrict__ tile_row0, int* __restrict__ tile_rows,
            int* __restrict__ num_tiles, unsigned int* status) {
  __shared__ int cnt[kMaxExperts];
  __shared__ int off[kMaxExperts + 1];
  __shared__ int toff[kMaxExperts + 1];
  __shared__ int cursor[kMaxExperts];
  const int tid = threadIdx.x;
  for (int e = tid; e < E; e += blockDim.x) {
    cnt[e] = 0;
    cursor[e] = 0;
  }
  __syncthreads();
  for (int i = tid; i < R; i += blockDim.x) {
    const int e = ids[i] - e_lo;
    if (e >= 0 && e < E) atomicAdd(&cnt[e], 1);
  }
  __syncthreads();
  // Exclusive scans of the counts and of the per-expert tile counts (warp 0,
  // each lane owns a contiguous run of experts).
  if (tid < 32) {
    const int per = (E + 31) / 32;
    const int lo = tid * per, hi = min(E, lo + per);
    int s = 0, ts = 0;
    for (int e = lo; e < hi; ++e) {
      s += cnt[e];
      ts += (cnt[e] + block_n - 1) / block_n;
    }
    int ps = s, pts = ts;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int a = __shfl_up_sync(0xffffffffu, ps, o);
      const int b = __shfl_up_sync(0xffffffffu, pts, o);
      if (tid >= o) {
        ps += a;
        pts += b;
      }
    }
    int run = ps - s, trun = pts - ts;
    for (int e = lo; e < hi; ++e) {
      off[e] = run;
      toff[e] = trun;
      run += cnt[e];
      trun += (cnt[e] + block_n - 1) / block_n;
    }
    if (tid == 31) {
      off[E] = ps;
      toff[E] = pts;
    }
  }
  __syncthreads();
  for (int e = tid; e <= E; e += blockDim.x) expert_offsets[e] = off[e];
  if (tid == 0) {
    int n = toff[E];
    if (n > max_tiles) {
      us_dev_fail(status, US_DEV_BOUNDS);
      n = max_tiles;
    }
    *num_tiles = n;
  }
  for (int e = tid; e < E; e += blockDim.x) {
    const int c = cnt[e];
    const int nt = (c + block_n - 1) / block_n;
    for (int j = 0; j < nt; ++j) {
      const int ti = toff[e] + j;
      if (ti < max_tiles) {
        tile_group[ti] = e;
        tile_row0[ti] = off[e] + j * block_n;
        tile_rows[ti] = min(block_n, c - j * block_n);
      }
    }
  }
  for (int i = tid; i < R; i += blockDim.x) {
    const int e = ids[i] - e_lo;
    if (e >= 0 && e < E) {
      const int pos = off[e] + atomicAdd(&cursor[e], 1);
      sorted_route[pos] = i;
      perm_of_route[i] = pos;
    } else {
      perm_of_route[i] = -1;
    }
  }
}

__global__ void __launch_bounds__(1024)
moe_sort_kernel(const int* __restrict__ ids, int R, int e_lo, int E, int block_n, int max_tiles,
                int* __restrict__ sorted_route, int* __restrict__ perm_of_route,
                int* __restrict__ expert_offsets, int* __restrict__ tile_group,
                int* __restrict__ tile_row0, int* __restrict__ tile_rows,
                int* __restrict__ num_tiles, unsigned int* status) {
  US_PDL_PROLOGUE();
  sort_routes(ids, R, e_lo, E, block_n, max_tiles, sorted_route, perm_of_route, expert_offsets,
              tile_group, tile_row0, tile_rows, num_tiles, status);
}

// Routing and sorting in one launch (decode-size batches): the CTA's 32 warps take the
// tokens in turn, then the whole CTA sorts the routes they wrote.
template <int PER_LANE>
__global__ void __launch_bounds__(1024)
route_sort_kernel(const float* __restrict__ logits, int* __restrict__ ids,
                  float* __restrict__ weights, int T, int E_all, int top_k, int renorm,
                  const int* __restrict__ live, int e_lo, int E, int block_n, int max_tiles,
                  int* __restrict__ sorted_route, int* __restrict__ perm_of_route,
                  int* __restrict__ expert_offsets, int* __restrict__ tile_group,
                  int* __restrict__ tile_row0, int* __restrict__ tile_rows,
                  int* __restrict__ num_tiles, unsigned int* status) {
  US_PDL_PROLOGUE();
  for (int t = threadIdx.x >> 5; t < T; t += 32)
    topk_token<PER_LANE>(logits, ids, weights, t, E_all, top_k, renorm, live, nullptr, nullptr);
  __syncthreads();   // the routes written above are read below by other threads of the CTA
  sort_routes(ids, T * top_k, e_lo, E, block_n, max_tiles, sorted_route, perm_of_route,
              expert_offsets, tile_group, tile_row0, tile_rows, num_tiles, status);
}

__global__ void __launch_bounds__(256)
moe_gather_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ sorted_route,
                  const int* __restrict__ total, int top_k, int H,
                  __nv_bfloat16* __restrict__ xp) {
  US_PDL_PROLOGUE();
  const int p = blockIdx.x;
  if (p >= *total) return;
  const int t = sorted_route[p] / top_k;
  const uint4* src = reinterpret_cast<const uint4*>(x + (long long)t * H);
  uint4* dst = reinterpret_cast<uint4*>(xp + (long long)p * H);
  for (int v = threadIdx.x; v < (H >> 3); v += blockDim.x) dst[v] = src[v];
}

__global__ void __launch_bounds__(256)
moe_unpermute_kernel(const __nv_bfloat16* __restrict__ y, const int* __restrict__ perm_of_route,
                     const float* __restrict__ weights, int top_k, int H,
                     __nv_bfloat16* __restrict__ out) {
  US_PDL_PROLOGUE();
  const int t = blockIdx.x;
  for (int v = threadIdx.x; v < (H >> 3); v += blockDim.x) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int j = 0; j < top_k; ++j) {
      const int p = perm_of_route[(long long)t * top_k + j];
      if (p < 0) continue;
      const float w = weights[(long long)t * top_k + j];
      us::Pack16 q;
      q.u = *reinterpret_cast<const uint4*>(y + (long long)p * H + v * 8);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] += w * us::bf2f(q.b[i]);
    }
    us::Pack16 o;
#pragma unroll
    for (int i = 0; i < 8; ++i) o.b[i] = us::f2bf(acc[i]);
    *reinterpret_cast<uint4*>(out + (long long)t * H + v * 8) = o.u;
  }
}

}  // namespace

US_API int us_topk_softmax(const float* logits, int* ids, float* weights, int T, int E, int top_k,
                           int renorm, const int* live, const int* expert_map, int* load,
                           void* stream_) {
  US_REQUIRE(logits && ids && weights && T >= 0 && E >= 1 && E <= kMaxExperts && top_k >= 1 &&
             top_k <= 32 && top_k <= E);
  if (T == 0) return US_OK;
  cudaStream_t stream = (cudaStream_t)stream_;
  const int blocks = (T + 3) / 4;
  const int per = (E + 31) / 32;
#define US_TOPK(P)                                                                          \
  if (per <= P) {                                                                           \
    us::launch_pdl(topk_softmax_kernel<P>, dim3(blocks), dim3(128), 0, stream, logits, ids, weights, T, E, top_k,   \
                                                       renorm, live, expert_map, load);     \
    US_LAUNCH_CHECK();                                                                      \
    return US_OK;                                                                           \
  }
  US_TOPK(1) US_TOPK(2) US_TOPK(4) US_TOPK(8) US_TOPK(16) US_TOPK(32)
#undef US_TOPK
  return US_ERR_UNSUPPORTED;
}

US_API int us_moe_sort(const int* ids, int R, int e_lo, int E, int block_n, int max_tiles,
                       int* sorted_route, int* perm_of_route, int* expert_offsets, int* tile_group,
                       int* tile_row0, int* tile_rows, int* num_tiles, void* stream_) {
  US_REQUIRE(ids && R >= 0 && E >= 1 && E <= kMaxExperts && block_n >= 1 && max_tiles >= 1);
  US_REQUIRE(sorted_route && perm_of_route && expert_offsets && tile_group && tile_row0 &&
             tile_rows && num_tiles);
  us::launch_pdl(moe_sort_kernel, dim3(1), dim3(1024), 0, (cudaStream_t)stream_, ids, R, e_lo, E, block_n, max_tiles, sorted_route, perm_of_route, expert_offsets, tile_group,
      tile_row0, tile_rows, num_tiles, us_status_ptr());
  US_LAUNCH_CHECK();
  return US_OK;
}

US_API int us_moe_gather(const void* x, const int* sorted_route, const int* total, int R,
                         int top_k, int H, void* xp, void* stream_) {
  US_REQUIRE(x && sorted_route && total && xp && R >= 0 && (H % 8) == 0 && top_k >= 1);
  if (R == 0) return US_OK;
  us::launch_pdl(moe_gather_kernel, dim3(R), dim3(256), 0, (cudaStream_t)stream_, (const __nv_bfloat16*)x, sorted_route, total, top_k, H, (__nv_bfloat16*)xp);
  US_LAUNCH_CHECK();
  return US_OK;
}

US_API int us_moe_unpermute(const void* y, const int* perm_of_route, const float* weights, int T,
                            int top_k, int H, void* out, void* stream_) {
  US_REQUIRE(y && perm_of_route && weights && out && T >= 0 && (H % 8) == 0);
  if (T == 0) return US_OK;
  us::launch_pdl(moe_unpermute_kernel, dim3(T), dim3(256), 0, (cudaStream_t)stream_, (const __nv_bfloat16*)y, perm_of_route, weights, top_k, H, (__nv_bfloat16*)out);
  US_LAUNCH_CHECK();
  return US_OK;
}

// topk_softmax followed by moe_sort in one launch, for batches of at most 512 tokens.
US_API int us_route_sort(const float* logits, int* ids, float* weights, int T, int E_all,
                         int top_k, int renorm, const int* live, int e_lo, int E, int block_n,
                         int max_tiles, int* sorted_route, int* perm_of_route,
                         int* expert_offsets, int* tile_group, int* tile_row0, int* tile_rows,
                         int* num_tiles, void* stream_) {
  US_REQUIRE(logits && ids && weights && T >= 1 && T <= 512 && E_all >= 1 &&
             E_all <= kMaxExperts && top_k >= 1 && top_k <= 32 && top_k <= E_all);
  US_REQUIRE(E >= 1 && E <= kMaxExperts && block_n >= 1 && max_tiles >= 1 && sorted_route &&
             perm_of_route && expert_offsets && tile_group && tile_row0 && tile_rows && num_tiles);
  cudaStream_t stream = (cudaStream_t)stream_;
  const int per = (E_all + 31) / 32;
#define US_RS_CASE(P)                                                                          \
  if (per <= P) {                                                                              \
    US_CUDA_CHECK(us::launch_pdl(route_sort_kernel<P>, dim3(1), dim3(1024), 0, stream, logits, \
                                 ids, weights, T, E_all, top_k, renorm, live, e_lo, E, block_n,\
                                 max_tiles, sorted_route, perm_of_route, expert_offsets,       \
                                 tile_group, tile_row0, tile_rows, num_tiles,                  \
                                 us_status_ptr()));                                            \
    return US_OK;                                                                              \
  }
  US_RS_CASE(1)
  US_RS_CASE(2)
  US_RS_CASE(4)
  US_RS_CASE(8)
  US_RS_CASE(16)
  US_RS_CASE(32)
#undef US_RS_CASE
  return US_ERR_ARG;
}
