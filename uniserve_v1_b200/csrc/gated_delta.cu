// Recurrent token mixers of the hybrid (linear-attention) layers, for packed batches of
// sequences whose state lives in slots of a state pool:
//
//   us_causal_conv1d        y_t[c] = silu(sum_j w[c, j] * x_{t-(K-1)+j}[c]), state = last K-1 inputs
//   us_gated_delta_rule     S <- e^{g_t} S;  d = beta_t (v_t - S^T k_t);  S <- S + k_t d^T;
//                           o_t = S^T q_t,  q and k L2-normalised per head, q scaled by Dk^-1/2
//   us_rmsnorm_gated        per-head RMSNorm of o times silu(z)
//
// The rule is a strict recurrence over tokens but independent over (sequence, value head,
// value column): a CTA owns 32 value columns of one head of one sequence and keeps its
// [Dk, 32] slice of the state in registers for the whole sequence, so the state crosses
// HBM once per call (a decode step of 64 sequences x 32 heads moves 2 x 134 MB) and the
// per-token work is three fused multiply-adds per state element.  Inside the CTA a warp
// owns 8 columns with the Dk rows split over 4 lanes per column; the two Dk-reductions of
// a token are two shuffle steps, and warps never wait on one another inside a chunk of
// 16 tokens (q, k, v, the decay and beta of a chunk are staged in shared memory, already
// normalised).  The gates can be formed in the kernel from the raw projections
// (g = A * softplus(a + dt_bias), beta = sigmoid(b)).
//
// Reference behaviour: crates/ops/kernels/gated_delta_rule, crates/ops/kernels/causal_conv1d,
// crates/nn/src/modules/gated_delta_net.rs (reference project paths).
#include "include/us_common.cuh"

namespace {

__device__ __forceinline__ float ld_any(const void* base, long long idx, int bf16) {
  return bf16 ? us::bf2f(reinterpret_cast<const __nv_bfloat16*>(base)[idx])
              : reinterpret_cast<const float*>(base)[idx];
}
__device__ __forceinline__ void st_any(void* base, long long idx, int bf16, float v) {
  if (bf16) reinterpret_cast<__nv_bfloat16*>(base)[idx] = us::f2bf(v);
  else reinterpret_cast<float*>(base)[idx] = v;
}
__device__ __forceinline__ float silu(float x) { return x / (1.f + __expf(-x)); }

// sequence that holds packed row t (cu is ascending, cu[0] = 0, cu[B] = rows)
__device__ __forceinline__ int seq_of(const int* cu, int B, int t) {
  int lo = 0, hi = B - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (cu[mid] <= t) lo = mid; else hi = mid - 1;
  }
  return lo;
}

constexpr int kConvTokens = 8;     // rows per CTA of the convolution
constexpr int kMaxTaps = 8;

// x [rows, C] (row stride ldx), w [C, K], state [slots, K-1, C], y [rows, C] (row stride ldy).
__global__ void __launch_bounds__(256)
causal_conv1d_kernel(const void* __restrict__ x, long long ldx, const void* __restrict__ w,
                     const void* __restrict__ state, void* __restrict__ y, long long ldy,
                     const int* __restrict__ cu, const int* __restrict__ slots, int B, int rows,
                     int C, int K, int bf16, int w_bf16) {
  US_PDL_PROLOGUE();
  const int c = blockIdx.x * 256 + threadIdx.x;
  if (c >= C) return;
  float wt[kMaxTaps];
#pragma unroll
  for (int j = 0; j < kMaxTaps; ++j) wt[j] = j < K ? ld_any(w, (long long)c * K + j, w_bf16) : 0.f;
  const int t0 = blockIdx.y * kConvTokens;
  for (int t = t0; t < min(rows, t0 + kConvTokens); ++t) {
    const int s = seq_of(cu, B, t);
    const int start = cu[s];
    const long long sbase = (long long)slots[s] * (K - 1) * C;
    float acc = 0.f;
#pragma unroll
    for (int j = 0; j < kMaxTaps; ++j) {
      if (j >= K) break;
      const int pos = t - (K - 1) + j;          // packed row of the tap
      const float v = pos >= start ? ld_any(x, (long long)pos * ldx + c, bf16)
                                   : ld_any(state, sbase + (long long)(pos - start + K - 1) * C + c,
                                            bf16);
      acc += wt[j] * v;
    }
    st_any(y, (long long)t * ldy + c, bf16, silu(acc));
  }
}

// New state of every sequence: the last K-1 rows of [state; x].  A thread owns one channel
// of one sequence and walks the K-1 rows upwards, so a row is read before it is rewritten.
__global__ void __launch_bounds__(256)
causal_conv1d_state_kernel(const void* __restrict__ x, long long ldx, void* __restrict__ state,
                           const int* __restrict__ cu, const int* __restrict__ slots, int C, int K,
                           int bf16) {
  US_PDL_PROLOGUE();
  const int c = blockIdx.x * 256 + threadIdx.x;
  if (c >= C) return;
  const int s = blockIdx.y;
  const int start = cu[s], T = cu[s + 1] - start;
  const long long sbase = (long long)slots[s] * (K - 1) * C;
  for (int j = 0; j < K - 1; ++j) {
    const int src = T + j;                      // row of [state; x]
    const float v = src < K - 1 ? ld_any(state, sbase + (long long)src * C + c, bf16)
                                : ld_any(x, (long long)(start + src - (K - 1)) * ldx + c, bf16);
    st_any(state, sbase + (long long)j * C + c, bf16, v);
  }
}

constexpr int kChunk = 16;     // tokens staged per round
constexpr int kCols = 32;      // value columns per CTA

struct RuleArgs {
  const void *q, *k, *v;       // [rows, heads, dim] views: element (t, h, i) at t*ld + h*hs + i
  long long ldq, ldk, ldv;
  int hsq, hsk, hsv;
  int bf16;                    // q, k, v element type
  const float *g, *beta;       // [rows, Hv] (stride ldg) or, with A set, the raw a / b projections
  const void *a_raw, *b_raw;   // raw gate projections (element type = bf16 flag), stride ldg
  long long ldg;
  const float *A, *dt_bias;    // [Hv] or null
  float* state;                // [slots, Hv, Dk, Dv]
  float* out;                  // [rows, Hv, Dv]
  const int *cu, *slots;
  int Hv, Hk, Dv;
  float eps;
};

template <int DK>
__global__ void __launch_bounds__(128) gated_delta_rule_kernel(const RuleArgs a) {
  US_PDL_PROLOGUE();
  constexpr int kPer = DK / 4;                // state rows per lane
  static_assert(kPer % 4 == 0, "rows are moved as float4");
  __shared__ __align__(16) float ks[kChunk][DK];
  __shared__ __align__(16) float qs[kChunk][DK];
  __shared__ float vs[kChunk][kCols];
  __shared__ float os[kChunk][kCols];
  __shared__ float eg[kChunk], bt[kChunk];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int vl = lane >> 2, kq = lane & 3;
  const int h = blockIdx.y, s = blockIdx.z;
  const int hk = h / (a.Hv / a.Hk);
  const int col = blockIdx.x * kCols + warp * 8 + vl;
  const bool col_ok = col < a.Dv;
  const int start = a.cu[s], T = a.cu[s + 1] - start;
  float* Sg = a.state + (((long long)a.slots[s] * a.Hv + h) * DK) * a.Dv;
  // lane's rows: float4 group j covers rows (j * 4 + kq) * 4 .. + 3, so the four lanes of a
  // column read 64 contiguous bytes of a staged k or q vector (no bank conflicts)
  float S[kPer];
#pragma unroll
  for (int j = 0; j < kPer / 4; ++j)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int row = (j * 4 + kq) * 4 + e;
      S[j * 4 + e] = col_ok ? Sg[(long long)row * a.Dv + col] : 0.f;
    }
  const float qscale = rsqrtf((float)DK);

  for (int c0 = 0; c0 < T; c0 += kChunk) {
    const int n = min(kChunk, T - c0);
    __syncthreads();                           // the previous chunk's staging is consumed
    // stage: warp w normalises tokens w, w + 4, ...
    for (int t = warp; t < n; t += 4) {
      const long long row = start + c0 + t;
      float kv[(DK + 31) / 32], qv[(DK + 31) / 32];
      float k2 = 0.f, q2 = 0.f;
#pragma unroll
      for (int i = 0; i < (DK + 31) / 32; ++i) {
        const int d = i * 32 + lane;
        kv[i] = d < DK ? ld_any(a.k, row * a.ldk + (long long)hk * a.hsk + d, a.bf16) : 0.f;
        qv[i] = d < DK ? ld_any(a.q, row * a.ldq + (long long)hk * a.hsq + d, a.bf16) : 0.f;
        k2 += kv[i] * kv[i];
        q2 += qv[i] * qv[i];
      }
      k2 = rsqrtf(us::warp_sum(k2) + a.eps);
      q2 = rsqrtf(us::warp_sum(q2) + a.eps) * qscale;
#pragma unroll
      for (int i = 0; i < (DK + 31) / 32; ++i) {
        const int d = i * 32 + lane;
        if (d < DK) { ks[t][d] = kv[i] * k2; qs[t][d] = qv[i] * q2; }
      }
      const int c = blockIdx.x * kCols + lane;
      vs[t][lane] = c < a.Dv ? ld_any(a.v, row * a.ldv + (long long)h * a.hsv + c, a.bf16) : 0.f;
      if (lane == 0) {
        float g, b;
        if (a.A) {
          const float x = ld_any(a.a_raw, row * a.ldg + h, a.bf16) + a.dt_bias[h];
          const float sp = x > 20.f ? x : log1pf(__expf(x));
          g = a.A[h] * sp;
          b = 1.f / (1.f + __expf(-ld_any(a.b_raw, row * a.ldg + h, a.bf16)));
        } else {
          g = a.g[row * a.ldg + h];
          b = a.beta[row * a.ldg + h];
        }
        eg[t] = __expf(g);
        bt[t] = b;
      }
    }
    __syncthreads();
    for (int t = 0; t < n; ++t) {
      const float e = eg[t];
      float mem = 0.f;
#pragma unroll
      for (int j = 0; j < kPer / 4; ++j) {
        const float4 k4 = *reinterpret_cast<const float4*>(&ks[t][(j * 4 + kq) * 4]);
        mem += S[j * 4] * k4.x + S[j * 4 + 1] * k4.y + S[j * 4 + 2] * k4.z + S[j * 4 + 3] * k4.w;
      }
      mem += __shfl_xor_sync(0xffffffffu, mem, 1);
      mem += __shfl_xor_sync(0xffffffffu, mem, 2);
      const float d = (vs[t][warp * 8 + vl] - e * mem) * bt[t];
      float o = 0.f;
#pragma unroll
      for (int j = 0; j < kPer / 4; ++j) {
        const float4 k4 = *reinterpret_cast<const float4*>(&ks[t][(j * 4 + kq) * 4]);
        const float4 q4 = *reinterpret_cast<const float4*>(&qs[t][(j * 4 + kq) * 4]);
        S[j * 4] = fmaf(S[j * 4], e, k4.x * d);
        S[j * 4 + 1] = fmaf(S[j * 4 + 1], e, k4.y * d);
        S[j * 4 + 2] = fmaf(S[j * 4 + 2], e, k4.z * d);
        S[j * 4 + 3] = fmaf(S[j * 4 + 3], e, k4.w * d);
        o += S[j * 4] * q4.x + S[j * 4 + 1] * q4.y + S[j * 4 + 2] * q4.z + S[j * 4 + 3] * q4.w;
      }
      o += __shfl_xor_sync(0xffffffffu, o, 1);
      o += __shfl_xor_sync(0xffffffffu, o, 2);
      if (kq == 0) os[t][warp * 8 + vl] = o;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < n * kCols; e += 128) {
      const int t = e / kCols, c = e - t * kCols;
      const int cg = blockIdx.x * kCols + c;
      if (cg < a.Dv) a.out[((long long)(start + c0 + t) * a.Hv + h) * a.Dv + cg] = os[t][c];
    }
  }
  if (col_ok) {
#pragma unroll
    for (int j = 0; j < kPer / 4; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int row = (j * 4 + kq) * 4 + e;
        Sg[(long long)row * a.Dv + col] = S[j * 4 + e];
      }
  }
}

// One warp per (token, head) row: y = round(round(x * rsqrt(mean x^2 + eps)) * w) * silu(z)
// (the roundings are those of a bf16 model; an FP32 model rounds nowhere).
__global__ void __launch_bounds__(256)
rmsnorm_gated_kernel(const float* __restrict__ x, const void* __restrict__ w,
                     const void* __restrict__ z, long long ldz, int hsz, void* __restrict__ y,
                     int rows, int Hv, int Dv, float eps, int bf16) {
  US_PDL_PROLOGUE();
  const int r = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (r >= rows) return;
  const int t = r / Hv, h = r - t * Hv;
  const float* xr = x + (long long)r * Dv;
  // a bf16 model rounds the rule's output to bf16 before this norm; the same values here
  float ss = 0.f;
  for (int d = lane; d < Dv; d += 32) {
    const float xv = bf16 ? us::bf2f(us::f2bf(xr[d])) : xr[d];
    ss += xv * xv;
  }
  const float inv = rsqrtf(us::warp_sum(ss) / (float)Dv + eps);
  for (int d = lane; d < Dv; d += 32) {
    float v = (bf16 ? us::bf2f(us::f2bf(xr[d])) : xr[d]) * inv;
    float wv = ld_any(w, d, bf16);
    if (bf16) v = us::bf2f(us::f2bf(us::bf2f(us::f2bf(v)) * wv));
    else v = v * wv;
    const float g = ld_any(z, (long long)t * ldz + (long long)h * hsz + d, bf16);
    st_any(y, (long long)r * Dv + d, bf16, v * silu(g));
  }
}

}  // namespace

US_API int us_causal_conv1d(const void* x, long long ldx, const void* w, void* state, void* y,
                            long long ldy, const int* cu, const int* slots, int B, int rows, int C,
                            int K, int bf16, int w_bf16, void* stream_) {
  US_REQUIRE(x && w && state && y && cu && slots && B >= 1 && rows >= 1 && C >= 1);
  if (K < 2 || K > kMaxTaps) return US_ERR_UNSUPPORTED;
  cudaStream_t stream = (cudaStream_t)stream_;
  const dim3 grid((C + 255) / 256, (rows + kConvTokens - 1) / kConvTokens);
  US_CUDA_CHECK(us::launch_pdl(causal_conv1d_kernel, grid, dim3(256), 0, stream, x, ldx, w,
                               (const void*)state, y, ldy, cu, slots, B, rows, C, K, bf16, w_bf16));
  US_CUDA_CHECK(us::launch_pdl(causal_conv1d_state_kernel, dim3((C + 255) / 256, B), dim3(256), 0,
                               stream, x, ldx, state, cu, slots, C, K, bf16));
  return US_OK;
}

// q, k: [rows, Hk, Dk] views, v: [rows, Hv, Dv] view (strides in elements); gates either as
// g / beta [rows, Hv] FP32 (A null) or as the raw projections with A and dt_bias [Hv].
US_API int us_gated_delta_rule(const void* q, const void* k, const void* v, long long ldq,
                               long long ldk, long long ldv, int hsq, int hsk, int hsv, int bf16,
                               const float* g, const float* beta, const void* a_raw,
                               const void* b_raw, long long ldg, const float* A,
                               const float* dt_bias, float* state, float* out, const int* cu,
                               const int* slots, int B, int Hk, int Hv, int Dk, int Dv, float eps,
                               void* stream_) {
  US_REQUIRE(q && k && v && state && out && cu && slots && B >= 1);
  US_REQUIRE(Hk >= 1 && Hv % Hk == 0 && Dv >= 1);
  US_REQUIRE(A ? (a_raw && b_raw && dt_bias) : (g && beta));
  RuleArgs a{q, k, v, ldq, ldk, ldv, hsq, hsk, hsv, bf16, g, beta, a_raw, b_raw, ldg, A, dt_bias,
             state, out, cu, slots, Hv, Hk, Dv, eps};
  cudaStream_t stream = (cudaStream_t)stream_;
  const dim3 grid((Dv + kCols - 1) / kCols, Hv, B), block(128);
  switch (Dk) {
    case 16: US_CUDA_CHECK(us::launch_pdl(gated_delta_rule_kernel<16>, grid, block, 0, stream, a)); break;
    case 32: US_CUDA_CHECK(us::launch_pdl(gated_delta_rule_kernel<32>, grid, block, 0, stream, a)); break;
    case 64: US_CUDA_CHECK(us::launch_pdl(gated_delta_rule_kernel<64>, grid, block, 0, stream, a)); break;
    case 128: US_CUDA_CHECK(us::launch_pdl(gated_delta_rule_kernel<128>, grid, block, 0, stream, a)); break;
    default: return US_ERR_UNSUPPORTED;
  }
  return US_OK;
}

US_API int us_rmsnorm_gated(const float* x, const void* w, const void* z, long long ldz, int hsz,
                            void* y, int rows, int Hv, int Dv, float eps, int bf16, void* stream_) {
  US_REQUIRE(x && w && z && y && rows >= 1 && Hv >= 1 && Dv >= 1);
  US_CUDA_CHECK(us::launch_pdl(rmsnorm_gated_kernel, dim3((rows + 7) / 8), dim3(256), 0,
                               (cudaStream_t)stream_, x, w, z, ldz, hsz, y, rows, Hv, Dv, eps, bf16));
  return US_OK;
}
