// Sampling kernels.  One CTA owns one row of FP32 logits.
//
//   argmax              greedy token (ties to the lower id)
//   logits_shape        ban mask -> logit bias -> repetition / frequency /
//                       presence penalties -> temperature (0 divides by 1)
//   sample_from_logits  top-k, top-p and min-p draw without sorting: the kept
//                       set is { key >= threshold } found by 8-bit radix passes
//                       over order-preserving keys; probability masses are
//                       integers (2^-40 units) so sums do not depend on the
//                       order of accumulation; the draw is the inverse CDF over
//                       kept candidates in ascending token id with one Philox
//                       uniform addressed by (seed, position).
//   logprob_stats       per-row max and log-sum-exp, the chosen token's
//                       log-probability and its one-based competition rank
//
// The sampled token is a function of (seed, position, distribution) only; it
// does not depend on the batch a row runs in.
//
// Reference behaviour: crates/ops/src/sampler.rs:1-36,
// crates/ops/kernels/sampling_from_logits/nvcc, crates/engine/src/batch/philox.rs:18-35
// (reference project paths).
#include "include/us_common.cuh"
#include "include/us_philox.h"

namespace {

constexpr int kThreads = 1024;

__device__ __forceinline__ uint32_t order_key(float f) {
  uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__global__ void __launch_bounds__(kThreads)
argmax_kernel(const float* __restrict__ logits, int V, long long ld, int* __restrict__ out) {
  US_PDL_PROLOGUE();
  __shared__ float sv[32];
  __shared__ int si[32];
  const float* row = logits + (long long)blockIdx.x * ld;
  float best = -INFINITY;
  int best_i = 0x7fffffff;
  for (int i = threadIdx.x; i < V; i += kThreads) {
    const float v = row[i];
    if (v > best || (v == best && i < best_i)) {
      best = v;
      best_i = i;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ob = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
    if (ob > best || (ob == best && oi < best_i)) {
      best = ob;
      best_i = oi;
    }
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) {
    sv[warp] = best;
    si[warp] = best_i;
  }
  __syncthreads();
  if (warp == 0) {
    best = sv[lane];
    best_i = si[lane];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
      if (ob > best || (ob == best && oi < best_i)) {
        best = ob;
        best_i = oi;
      }
    }
    if (lane == 0) out[blockIdx.x] = best_i == 0x7fffffff ? 0 : best_i;
  }
}

__global__ void __launch_bounds__(256)
logits_shape_kernel(float* __restrict__ logits, int V, long long ld,
                    const unsigned char* __restrict__ ban_mask,    // [B, V] or null
                    const int* __restrict__ bias_offsets,          // [B + 1] or null
                    const int* __restrict__ bias_ids, const float* __restrict__ bias_vals,
                    const unsigned short* __restrict__ out_counts, // [B, V] or null
                    const unsigned char* __restrict__ prompt_mask, // [B, V] or null
                    const float* __restrict__ rep, const float* __restrict__ freq,
                    const float* __restrict__ pres, const float* __restrict__ temp) {
  US_PDL_PROLOGUE();
  const int b = blockIdx.y;
  float* row = logits + (long long)b * ld;
  const float r = rep ? rep[b] : 1.f;
  const float fq = freq ? freq[b] : 0.f;
  const float pr = pres ? pres[b] : 0.f;
  float t = temp ? temp[b] : 1.f;
  if (t == 0.f) t = 1.f;
  const float inv_t = 1.f / t;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < V; i += gridDim.x * blockDim.x) {
    float v = row[i];
    if (ban_mask && ban_mask[(long long)b * V + i]) v = -INFINITY;
    const int oc = out_counts ? out_counts[(long long)b * V + i] : 0;
    const bool seen = oc > 0 || (prompt_mask && prompt_mask[(long long)b * V + i]);
    if (seen && r != 1.f) v = v > 0.f ? v / r : v * r;
    if (oc > 0) v -= fq * (float)oc + pr;
    row[i] = v * inv_t;
  }
  // Sparse logit bias is applied by one thread per entry before the dense pass
  // of the next launch; see us_logits_bias.
  (void)bias_offsets; (void)bias_ids; (void)bias_vals;
}

__global__ void logits_bias_kernel(float* __restrict__ logits, long long ld,
                                   const int* __restrict__ bias_offsets,
                                   const int* __restrict__ bias_ids,
                                   const float* __restrict__ bias_vals, int V) {
  US_PDL_PROLOGUE();
  const int b = blockIdx.x;
  for (int j = bias_offsets[b] + threadIdx.x; j < bias_offsets[b + 1]; j += blockDim.x) {
    const int id = bias_ids[j];
    if (id >= 0 && id < V) logits[(long long)b * ld + id] += bias_vals[j];
  }
}

struct SampleArgs {
  const float* logits;
  long long ld;
  int V;
  const int* top_k;       // [B] (<= 0: whole row)
  const float* top_p;     // [B] (>= 1: off)
  const float* min_p;     // [B] (<= 0: off)
  const unsigned long long* seeds;  // [B]
  const long long* positions;       // [B] logical position of the sampled token
  int* out;
};

// Finds the largest key threshold T such that count{key >= T} >= k.
// All threads return the same value.
__device__ uint32_t radix_select_count(const float* row, int V, int k, uint32_t lo_limit,
                                       unsigned int* hist) {
  uint32_t prefix = 0, mask = 0;
  int remaining = k;
  for (int shift = 24; shift >= 0; shift -= 8) {
    for (int i = threadIdx.x; i < 256; i += kThreads) hist[i] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < V; i += kThreads) {
      const uint32_t key = order_key(row[i]);
      if (key >= lo_limit && (key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 0xff], 1u);
    }
    __syncthreads();
    // Walk bins from the top; every thread performs the same walk.
    int bin = 255, above = 0;
    for (; bin > 0; --bin) {
      const int c = (int)hist[bin];
      if (above + c >= remaining) break;
      above += c;
    }
    remaining -= above;
    prefix |= (uint32_t)bin << shift;
    mask |= 0xffu << shift;
    __syncthreads();
  }
  return prefix;
}

// Integer probability mass of one candidate (2^-40 units of the row maximum's
// unnormalised weight 1.0).
__device__ __forceinline__ unsigned long long mass_of(float logit, float mx) {
  const float w = __expf(logit - mx);  // in (0, 1]
  return (unsigned long long)((double)w * 1099511627776.0);
}

// Largest key threshold T such that mass{key >= T} >= target among keys >= lo_limit.
__device__ uint32_t radix_select_mass(const float* row, int V, float mx,
                                      unsigned long long target, uint32_t lo_limit,
                                      unsigned long long* hist) {
  uint32_t prefix = 0, mask = 0;
  unsigned long long remaining = target;
  for (int shift = 24; shift >= 0; shift -= 8) {
    for (int i = threadIdx.x; i < 256; i += kThreads) hist[i] = 0ull;
    __syncthreads();
    for (int i = threadIdx.x; i < V; i += kThreads) {
      const float v = row[i];
      const uint32_t key = order_key(v);
      if (key >= lo_limit && (key & mask) == prefix)
        atomicAdd(&hist[(key >> shift) & 0xff], mass_of(v, mx));
    }
    __syncthreads();
    int bin = 255;
    unsigned long long above = 0;
    for (; bin > 0; --bin) {
      const unsigned long long c = hist[bin];
      if (above + c >= remaining) break;
      above += c;
    }
    remaining -= above;
    prefix |= (uint32_t)bin << shift;
    mask |= 0xffu << shift;
    __syncthreads();
  }
  return prefix;
}

__global__ void __launch_bounds__(kThreads) sample_kernel(const SampleArgs a) {
  US_PDL_PROLOGUE();
  __shared__ float fscratch[33];
  __shared__ unsigned int hist32[256];
  __shared__ unsigned long long hist64[256];
  __shared__ unsigned long long chunk_mass[kThreads];
  __shared__ unsigned long long total_mass;
  __shared__ int pick;

  const int b = blockIdx.x;
  const float* row = a.logits + (long long)b * a.ld;
  const int V = a.V;

  float mx = -INFINITY;
  for (int i = threadIdx.x; i < V; i += kThreads) mx = fmaxf(mx, row[i]);
  mx = us::block_max(mx, fscratch);

  uint32_t thr = order_key(-INFINITY) + 1;  // keep everything finite
  const int k = a.top_k ? a.top_k[b] : 0;
  if (k > 0 && k < V) thr = max(thr, radix_select_count(row, V, k, thr, hist32));
  const float mp = a.min_p ? a.min_p[b] : 0.f;
  if (mp > 0.f) thr = max(thr, order_key(mx + __logf(mp)));
  const float tp = a.top_p ? a.top_p[b] : 1.f;
  if (tp < 1.f) {
    // Mass of the survivors so far, then the nucleus threshold inside them.
    unsigned long long m = 0;
    for (int i = threadIdx.x; i < V; i += kThreads) {
      const float v = row[i];
      if (order_key(v) >= thr) m += mass_of(v, mx);
    }
    chunk_mass[threadIdx.x] = m;
    __syncthreads();
    if (threadIdx.x == 0) {
      unsigned long long s = 0;
      for (int i = 0; i < kThreads; ++i) s += chunk_mass[i];
      total_mass = s;
    }
    __syncthreads();
    const unsigned long long target =
        (unsigned long long)((double)total_mass * (double)fmaxf(tp, 0.f));
    thr = max(thr, radix_select_mass(row, V, mx, target > 0 ? target : 1, thr, hist64));
    __syncthreads();
  }

  // Inverse CDF over kept candidates in ascending token id.
  const int per = (V + kThreads - 1) / kThreads;
  const int lo = threadIdx.x * per, hi = min(V, lo + per);
  unsigned long long m = 0;
  for (int i = lo; i < hi; ++i) {
    const float v = row[i];
    if (order_key(v) >= thr) m += mass_of(v, mx);
  }
  chunk_mass[threadIdx.x] = m;
  if (threadIdx.x == 0) pick = -1;
  __syncthreads();
  if (threadIdx.x == 0) {
    unsigned long long s = 0;
    for (int i = 0; i < kThreads; ++i) {
      const unsigned long long c = chunk_mass[i];
      chunk_mass[i] = s;  // exclusive prefix
      s += c;
    }
    total_mass = s;
  }
  __syncthreads();
  const unsigned long long seed = a.seeds ? a.seeds[b] : 0ull;
  const long long pos = a.positions ? a.positions[b] : 0ll;
  const float u = us_philox_uniform(seed, (unsigned long long)pos, 0u, 0u);
  unsigned long long target = (unsigned long long)((double)u * (double)total_mass);
  if (target >= total_mass) target = total_mass ? total_mass - 1 : 0;
  const unsigned long long before = chunk_mass[threadIdx.x];
  if (m > 0 && target >= before && target < before + m) {
    unsigned long long c = before;
    int chosen = -1;
    for (int i = lo; i < hi; ++i) {
      const float v = row[i];
      if (order_key(v) >= thr) {
        c += mass_of(v, mx);
        if (target < c) {
          chosen = i;
          break;
        }
      }
    }
    pick = chosen;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int r = pick;
    if (r < 0) {  // degenerate row (all -inf / NaN): fall back to the first maximum
      r = 0;
      for (int i = 0; i < V; ++i)
        if (row[i] == mx) {
          r = i;
          break;
        }
    }
    a.out[b] = r;
  }
}

__global__ void __launch_bounds__(kThreads)
logprob_stats_kernel(const float* __restrict__ logits, long long ld, int V,
                     const int* __restrict__ chosen, float* __restrict__ lse_out,
                     float* __restrict__ logprob_out, int* __restrict__ rank_out) {
  US_PDL_PROLOGUE();
  __shared__ float fscratch[33];
  const int b = blockIdx.x;
  const float* row = logits + (long long)b * ld;
  float mx = -INFINITY;
  for (int i = threadIdx.x; i < V; i += kThreads) mx = fmaxf(mx, row[i]);
  mx = us::block_max(mx, fscratch);
  float s = 0.f;
  const int c = chosen ? chosen[b] : 0;
  const float cv = row[c];
  float rank = 0.f;
  for (int i = threadIdx.x; i < V; i += kThreads) {
    const float v = row[i];
    s += __expf(v - mx);
    if (v > cv) rank += 1.f;
  }
  s = us::block_sum(s, fscratch);
  rank = us::block_sum(rank, fscratch);
  if (threadIdx.x == 0) {
    const float lse = mx + __logf(s);
    if (lse_out) lse_out[b] = lse;
    if (logprob_out) logprob_out[b] = cv - lse;
    if (rank_out) rank_out[b] = (int)rank + 1;
  }
}

}  // namespace

US_API int us_argmax(const float* logits, int B, int V, long long ld, int* out, void* stream) {
  US_REQUIRE(logits && out && B >= 0 && V >= 1);
  if (B == 0) return US_OK;
  us::launch_pdl(argmax_kernel, dim3(B), dim3(kThreads), 0, (cudaStream_t)stream, logits, V, ld, out);
  US_LAUNCH_CHECK();
  return US_OK;
}

US_API int us_logits_shape(float* logits, int B, int V, long long ld,
                           const unsigned char* ban_mask, const int* bias_offsets,
                           const int* bias_ids, const float* bias_vals,
                           const unsigned short* out_counts, const unsigned char* prompt_mask,
                           const float* rep, const float* freq, const float* pres,
                           const float* temp, void* stream_) {
  US_REQUIRE(logits && B >= 0 && V >= 1);
  if (B == 0) return US_OK;
  cudaStream_t stream = (cudaStream_t)stream_;
  if (bias_offsets) {
    // Bias comes after bans and before penalties; bans stay -inf under an add,
    // so applying the sparse bias first keeps the documented order.
    us::launch_pdl(logits_bias_kernel, dim3(B), dim3(128), 0, stream, logits, ld, bias_offsets, bias_ids, bias_vals, V);
    US_LAUNCH_CHECK();
  }
  dim3 grid((V + 256 * 8 - 1) / (256 * 8), B);
  us::launch_pdl(logits_shape_kernel, dim3(grid), dim3(256), 0, stream, logits, V, ld, ban_mask, bias_offsets, bias_ids,
                                                bias_vals, out_counts, prompt_mask, rep, freq,
                                                pres, temp);
  US_LAUNCH_CHECK();
  return US_OK;
}

US_API int us_sample_from_logits(const float* logits, int B, int V, long long ld, const int* top_k,
                                 const float* top_p, const float* min_p,
                                 const unsigned long long* seeds, const long long* positions,
                                 int* out, void* stream) {
  US_REQUIRE(logits && out && B >= 0 && V >= 1);
  if (B == 0) return US_OK;
  SampleArgs a;
  a.logits = logits; a.ld = ld; a.V = V; a.top_k = top_k; a.top_p = top_p; a.min_p = min_p;
  a.seeds = seeds; a.positions = positions; a.out = out;
  us::launch_pdl(sample_kernel, dim3(B), dim3(kThreads), 0, (cudaStream_t)stream, a);
  US_LAUNCH_CHECK();
  return US_OK;
}

US_API int us_logprob_stats(const float* logits, int B, int V, long long ld, const int* chosen,
                            float* lse, float* logprob, int* rank, void* stream) {
  US_REQUIRE(logits && B >= 0 && V >= 1);
  if (B == 0) return US_OK;
  us::launch_pdl(logprob_stats_kernel, dim3(B), dim3(kThreads), 0, (cudaStream_t)stream, logits, ld, V, chosen, lse,
                                                                 logprob, rank);
  US_LAUNCH_CHECK();
  return US_OK;
}
