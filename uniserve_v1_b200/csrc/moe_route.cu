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
//   unpermute_add_rmsnorm   the same sum, added to the FP32 residual stream and
//                  normalised in the same launch (the next block's input norm).
//   route_sort_gather   topk_softmax + moe_sort + moe_gather of a decode-size batch in
//                  one launch: the CTAs route their tokens, the last one to arrive
//                  sorts, then all of them gather (two bounded grid-wide waits).
//
// Reference behaviour: crates/ops/kernels/topk_softmax/nvcc/src/topk_softmax.cu:1-27,
// crates/nn/src/functional/moe.rs:301-330, crates/ops/kernels/moe_unpermute
// (reference project paths).
#include <float.h>

#include "include/us_common.cuh"
#include "include/us_tc05.cuh"

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

// The same sort by a cluster of kSortCtas CTAs for prefill-sized route lists: CTA c counts
// and scatters the routes [c * chunk, (c + 1) * chunk).  After the local histograms every
// CTA reads its peers' counts through distributed shared memory: their sum gives the expert
// offsets (scanned redundantly in every CTA), the sum over lower ranks gives where this
// CTA's routes of an expert start inside the expert's run.  CTA 0 writes the offsets and the
// tile list.
constexpr int kSortCtas = 8;
constexpr int kSortClusterMinRoutes = 8192;   // below this one CTA is as fast
__global__ void __launch_bounds__(1024)
moe_sort_cluster_kernel(const int* __restrict__ ids, int R, int e_lo, int E, int block_n,
                        int max_tiles, int* __restrict__ sorted_route,
                        int* __restrict__ perm_of_route, int* __restrict__ expert_offsets,
                        int* __restrict__ tile_group, int* __restrict__ tile_row0,
                        int* __restrict__ tile_rows, int* __restrict__ num_tiles,
                        unsigned int* status) {
  US_PDL_PROLOGUE();
  __shared__ int mine[kMaxExperts];      // this CTA's counts (read by the peers)
  __shared__ int cnt[kMaxExperts];       // counts of the whole cluster
  __shared__ int base[kMaxExperts];      // routes of lower-ranked CTAs, per expert
  __shared__ int off[kMaxExperts + 1];
  __shared__ int toff[kMaxExperts + 1];
  __shared__ int cursor[kMaxExperts];
  const int tid = threadIdx.x;
  const int c = (int)tc::cluster_ctarank();
  const int chunk = (R + kSortCtas - 1) / kSortCtas;
  const int r_lo = min(R, c * chunk), r_hi = min(R, r_lo + chunk);
  for (int e = tid; e < E; e += blockDim.x) {
    mine[e] = 0;
    cursor[e] = 0;
  }
  __syncthreads();
  for (int i = r_lo + tid; i < r_hi; i += blockDim.x) {
    const int e = ids[i] - e_lo;
    if (e >= 0 && e < E) atomicAdd(&mine[e], 1);
  }
  tc::cluster_sync();
  for (int e = tid; e < E; e += blockDim.x) {
    const uint32_t local = (uint32_t)__cvta_generic_to_shared(&mine[e]);
    int all = 0, below = 0;
    for (int p = 0; p < kSortCtas; ++p) {
      const int v = __float_as_int(tc::ld_dsmem_f32(tc::map_to_cta(local, (uint32_t)p)));
      all += v;
      if (p < c) below += v;
    }
    cnt[e] = all;
    base[e] = below;
  }
  tc::cluster_sync();     // nobody's counts are read after this point
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
  if (c == 0) {
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
      const int k = cnt[e];
      const int nt = (k + block_n - 1) / block_n;
      for (int j = 0; j < nt; ++j) {
        const int ti = toff[e] + j;
        if (ti < max_tiles) {
          tile_group[ti] = e;
          tile_row0[ti] = off[e] + j * block_n;
          tile_rows[ti] = min(block_n, k - j * block_n);
        }
      }
    }
  }
  for (int i = r_lo + tid; i < r_hi; i += blockDim.x) {
    const int e = ids[i] - e_lo;
    if (e >= 0 && e < E) {
      const int pos = off[e] + base[e] + atomicAdd(&cursor[e], 1);
      sorted_route[pos] = i;
      perm_of_route[i] = pos;
    } else {
      perm_of_route[i] = -1;
    }
  }
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

// Four permuted rows per CTA: a thread issues its four 16-byte loads before the stores.
constexpr int kGatherRows = 4;
__global__ void __launch_bounds__(256)
moe_gather_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ sorted_route,
                  const int* __restrict__ total, int top_k, int H,
                  __nv_bfloat16* __restrict__ xp) {
  US_PDL_PROLOGUE();
  const int p0 = blockIdx.x * kGatherRows;
  const int n = min(kGatherRows, *total - p0);
  if (n <= 0) return;
  const uint4* src[kGatherRows];
#pragma unroll
  for (int j = 0; j < kGatherRows; ++j) {
    const int t = sorted_route[p0 + (j < n ? j : 0)] / top_k;
    src[j] = reinterpret_cast<const uint4*>(x + (long long)t * H);
  }
  uint4* dst = reinterpret_cast<uint4*>(xp + (long long)p0 * H);
  const int nvec = H >> 3;
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    uint4 r[kGatherRows];
#pragma unroll
    for (int j = 0; j < kGatherRows; ++j) r[j] = src[j][v];
#pragma unroll
    for (int j = 0; j < kGatherRows; ++j)
      if (j < n) dst[(long long)j * nvec + v] = r[j];
  }
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

// out[t] = sum of the token's routed rows, then residual += out, y = rmsnorm(residual) * w.
// One CTA per token; the partial sum is rounded to bf16 once before it joins the FP32
// residual, as the separate un-permute kernel's output would be.
constexpr int kNormVec = 4;   // hidden sizes up to 4 x 256 x 8
__global__ void __launch_bounds__(256)
unpermute_add_rmsnorm_kernel(const __nv_bfloat16* __restrict__ y_perm,
                             const int* __restrict__ perm, const float* __restrict__ weights,
                             int top_k, float* __restrict__ residual,
                             const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y,
                             int H, float eps, int first) {
  US_PDL_PROLOGUE();
  __shared__ float scratch[33];
  const int t = blockIdx.x;
  const int nvec = H >> 3;
  float* rr = residual + (size_t)t * H;
  float ss = 0.f;
  float4 keep[kNormVec][2];
#pragma unroll
  for (int i = 0; i < kNormVec; ++i) {
    const int v = threadIdx.x + i * 256;
    if (v >= nvec) break;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int j = 0; j < top_k; ++j) {
      const int p = perm[(size_t)t * top_k + j];
      if (p < 0) continue;
      const float wj = weights[(size_t)t * top_k + j];
      us::Pack16 q;
      q.u = *reinterpret_cast<const uint4*>(y_perm + (size_t)p * H + v * 8);
#pragma unroll
      for (int c = 0; c < 8; ++c) acc[c] += wj * us::bf2f(q.b[c]);
    }
#pragma unroll
    for (int c = 0; c < 8; ++c) acc[c] = us::bf2f(us::f2bf(acc[c]));
    float4 r0 = make_float4(0.f, 0.f, 0.f, 0.f), r1 = r0;
    if (!first) {
      r0 = *reinterpret_cast<const float4*>(rr + v * 8);
      r1 = *reinterpret_cast<const float4*>(rr + v * 8 + 4);
    }
    r0.x += acc[0]; r0.y += acc[1]; r0.z += acc[2]; r0.w += acc[3];
    r1.x += acc[4]; r1.y += acc[5]; r1.z += acc[6]; r1.w += acc[7];
    *reinterpret_cast<float4*>(rr + v * 8) = r0;
    *reinterpret_cast<float4*>(rr + v * 8 + 4) = r1;
    keep[i][0] = r0;
    keep[i][1] = r1;
    ss += r0.x * r0.x + r0.y * r0.y + r0.z * r0.z + r0.w * r0.w;
    ss += r1.x * r1.x + r1.y * r1.y + r1.z * r1.z + r1.w * r1.w;
  }
  ss = us::block_sum(ss, scratch);
  const float inv = rsqrtf(ss / (float)H + eps);
#pragma unroll
  for (int i = 0; i < kNormVec; ++i) {
    const int v = threadIdx.x + i * 256;
    if (v >= nvec) break;
    const float4 r0 = keep[i][0], r1 = keep[i][1];
    us::Pack16 q, o;
    q.u = *reinterpret_cast<const uint4*>(w + v * 8);
    o.b[0] = us::f2bf(r0.x * inv * us::bf2f(q.b[0]));
    o.b[1] = us::f2bf(r0.y * inv * us::bf2f(q.b[1]));
    o.b[2] = us::f2bf(r0.z * inv * us::bf2f(q.b[2]));
    o.b[3] = us::f2bf(r0.w * inv * us::bf2f(q.b[3]));
    o.b[4] = us::f2bf(r1.x * inv * us::bf2f(q.b[4]));
    o.b[5] = us::f2bf(r1.y * inv * us::bf2f(q.b[5]));
    o.b[6] = us::f2bf(r1.z * inv * us::bf2f(q.b[6]));
    o.b[7] = us::f2bf(r1.w * inv * us::bf2f(q.b[7]));
    *reinterpret_cast<uint4*>(y + (size_t)t * H + v * 8) = o.u;
  }
}

// Bounded spin on a device counter that other CTAs of the same grid advance.
__device__ __forceinline__ bool grid_wait(const unsigned int* ctr, unsigned int want,
                                          unsigned int* status) {
  const long long t0 = clock64();
  while (*(volatile const unsigned int*)ctr < want) {
    if (clock64() - t0 > 400000000LL) {          // about 0.2 s
      us_dev_fail(status, US_DEV_TIMEOUT_GRID);
      return false;
    }
  }
  __threadfence();
  return true;
}

// Routing, route sort and row gather of a decode-size batch in one launch.  Every CTA of
// the grid is resident at once (the host launches at most 128 CTAs of 256 threads).
// `sync` holds three zero-initialised counters: [0] CTAs that routed their tokens, [1] set
// by CTA 0 once the sort is written, [2] CTAs that passed the second wait (the last one
// clears all three for the next launch).
template <int PER_LANE>
__global__ void __launch_bounds__(256)
route_sort_gather_kernel(const float* __restrict__ logits, int* __restrict__ ids,
                         float* __restrict__ weights, int T, int E_all, int top_k, int renorm,
                         const int* __restrict__ live, int e_lo, int E, int block_n,
                         int max_tiles, int* __restrict__ sorted_route,
                         int* __restrict__ perm_of_route, int* __restrict__ expert_offsets,
                         int* __restrict__ tile_group, int* __restrict__ tile_row0,
                         int* __restrict__ tile_rows, int* __restrict__ num_tiles,
                         const __nv_bfloat16* __restrict__ x, int H,
                         __nv_bfloat16* __restrict__ xp, unsigned int* sync,
                         unsigned int* status) {
  US_PDL_PROLOGUE();
  const int warps = blockDim.x >> 5;
  for (int t = blockIdx.x * warps + (threadIdx.x >> 5); t < T; t += gridDim.x * warps)
    topk_token<PER_LANE>(logits, ids, weights, t, E_all, top_k, renorm, live, nullptr, nullptr);
  __threadfence();
  __syncthreads();
  __shared__ int ok_s;
  if (threadIdx.x == 0) {
    atomicAdd(&sync[0], 1u);
    ok_s = 1;
  }
  if (blockIdx.x == 0) {
    if (threadIdx.x == 0) ok_s = grid_wait(&sync[0], gridDim.x, status) ? 1 : 0;
    __syncthreads();
    if (ok_s)
      sort_routes(ids, T * top_k, e_lo, E, block_n, max_tiles, sorted_route, perm_of_route,
                  expert_offsets, tile_group, tile_row0, tile_rows, num_tiles, status);
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) atomicExch(&sync[1], 1u);
  } else {
    if (threadIdx.x == 0) ok_s = grid_wait(&sync[1], 1u, status) ? 1 : 0;
    __syncthreads();
  }
  const int total = ok_s ? *(volatile const int*)(expert_offsets + E) : 0;
  for (int p = blockIdx.x; p < total; p += gridDim.x) {
    const int t = sorted_route[p] / top_k;
    const uint4* src = reinterpret_cast<const uint4*>(x + (long long)t * H);
    uint4* dst = reinterpret_cast<uint4*>(xp + (long long)p * H);
    for (int v = threadIdx.x; v < (H >> 3); v += blockDim.x) dst[v] = src[v];
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    if (atomicAdd(&sync[2], 1u) == gridDim.x - 1) {
      sync[0] = 0;
      sync[1] = 0;
      sync[2] = 0;
    }
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
  if (R >= kSortClusterMinRoutes) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(kSortCtas);
    cfg.blockDim = dim3(1024);
    cfg.stream = (cudaStream_t)stream_;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = us::pdl_enabled() ? 1 : 0;
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = kSortCtas;
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    cudaLaunchKernelEx(&cfg, moe_sort_cluster_kernel, ids, R, e_lo, E, block_n, max_tiles,
                       sorted_route, perm_of_route, expert_offsets, tile_group, tile_row0,
                       tile_rows, num_tiles, us_status_ptr());
    US_LAUNCH_CHECK();
    return US_OK;
  }
  us::launch_pdl(moe_sort_kernel, dim3(1), dim3(1024), 0, (cudaStream_t)stream_, ids, R, e_lo, E, block_n, max_tiles, sorted_route, perm_of_route, expert_offsets, tile_group,
      tile_row0, tile_rows, num_tiles, us_status_ptr());
  US_LAUNCH_CHECK();
  return US_OK;
}

US_API int us_moe_gather(const void* x, const int* sorted_route, const int* total, int R,
                         int top_k, int H, void* xp, void* stream_) {
  US_REQUIRE(x && sorted_route && total && xp && R >= 0 && (H % 8) == 0 && top_k >= 1);
  if (R == 0) return US_OK;
  us::launch_pdl(moe_gather_kernel, dim3((R + kGatherRows - 1) / kGatherRows), dim3(256), 0, (cudaStream_t)stream_, (const __nv_bfloat16*)x, sorted_route, total, top_k, H, (__nv_bfloat16*)xp);
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

// out-of-place un-permute fused with the residual add and the RMSNorm that follow it.
US_API int us_unpermute_add_rmsnorm(const void* y_perm, const int* perm, const float* weights,
                                    int T, int top_k, int H, void* residual, const void* w,
                                    void* y, float eps, int first, void* stream_) {
  US_REQUIRE(y_perm && perm && weights && residual && w && y && T >= 0 && top_k >= 1);
  US_REQUIRE((H % 8) == 0 && H <= 8 * 256 * kNormVec);
  if (T == 0) return US_OK;
  US_CUDA_CHECK(us::launch_pdl(unpermute_add_rmsnorm_kernel, dim3(T), dim3(256), 0,
                               (cudaStream_t)stream_, (const __nv_bfloat16*)y_perm, perm, weights,
                               top_k, (float*)residual, (const __nv_bfloat16*)w,
                               (__nv_bfloat16*)y, H, eps, first));
  return US_OK;
}

// topk_softmax + moe_sort + moe_gather in one launch, for batches of at most 512 tokens.
// `sync`: three zero-initialised uint32 counters owned by the caller's workspace.
US_API int us_route_sort_gather(const float* logits, int* ids, float* weights, int T, int E_all,
                                int top_k, int renorm, const int* live, int e_lo, int E,
                                int block_n, int max_tiles, int* sorted_route,
                                int* perm_of_route, int* expert_offsets, int* tile_group,
                                int* tile_row0, int* tile_rows, int* num_tiles, const void* x,
                                int H, void* xp, void* sync, void* stream_) {
  US_REQUIRE(logits && ids && weights && T >= 1 && T <= 512 && E_all >= 1 &&
             E_all <= kMaxExperts && top_k >= 1 && top_k <= 32 && top_k <= E_all);
  US_REQUIRE(E >= 1 && E <= kMaxExperts && block_n >= 1 && max_tiles >= 1 && sorted_route &&
             perm_of_route && expert_offsets && tile_group && tile_row0 && tile_rows && num_tiles);
  US_REQUIRE(x && xp && sync && (H % 8) == 0);
  cudaStream_t stream = (cudaStream_t)stream_;
  int ctas = (T * top_k + 3) / 4;
  if (ctas < 8) ctas = 8;
  if (ctas > 128) ctas = 128;
  const int per = (E_all + 31) / 32;
#define US_RSG_CASE(P)                                                                         \
  if (per <= P) {                                                                              \
    US_CUDA_CHECK(us::launch_pdl(route_sort_gather_kernel<P>, dim3(ctas), dim3(256), 0, stream,\
                                 logits, ids, weights, T, E_all, top_k, renorm, live, e_lo, E, \
                                 block_n, max_tiles, sorted_route, perm_of_route,              \
                                 expert_offsets, tile_group, tile_row0, tile_rows, num_tiles,  \
                                 (const __nv_bfloat16*)x, H, (__nv_bfloat16*)xp,               \
                                 (unsigned int*)sync, us_status_ptr()));                       \
    return US_OK;                                                                              \
  }
  US_RSG_CASE(1)
  US_RSG_CASE(2)
  US_RSG_CASE(4)
  US_RSG_CASE(8)
  US_RSG_CASE(16)
  US_RSG_CASE(32)
#undef US_RSG_CASE
  return US_ERR_ARG;
}
