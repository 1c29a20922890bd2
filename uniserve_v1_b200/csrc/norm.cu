// Normalisation and residual kernels (bandwidth-bound, one CTA per row, 16-byte
// accesses).  Reductions run in FP32 and every output is rounded once.
//
//   rmsnorm            y = x * rsqrt(mean(x^2) + eps) * w
//   add_rmsnorm        r += x (FP32 residual stream);  y = rmsnorm(r) * w
//   modulated_rmsnorm  y = rmsnorm(x) [* w] * (1 + scale[idx]) + shift[idx]   (AdaLN)
//   gated_residual     h = h + gate[idx] * u
//   layer_norm         y = (x - mean) * rsqrt(var + eps) * w + b
//
// Reference behaviour: crates/ops/kernels/{rms_norm,add_rms_norm,modulated_rms_norm,
// gated_residual,layer_norm}/triton (reference project paths).
#include "include/us_common.cuh"

namespace {

constexpr int kThreads = 256;

__global__ void __launch_bounds__(kThreads)
rmsnorm_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
               __nv_bfloat16* __restrict__ y, int H, long long ldx, long long ldy, float eps) {
  US_PDL_PROLOGUE();
  __shared__ float scratch[33];
  const long long row = blockIdx.x;
  const __nv_bfloat16* xr = x + row * ldx;
  __nv_bfloat16* yr = y + row * ldy;
  const int nvec = H >> 3;
  float ss = 0.f;
  for (int v = threadIdx.x; v < nvec; v += kThreads) {
    us::Pack16 p;
    p.u = *reinterpret_cast<const uint4*>(xr + v * 8);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float f = us::bf2f(p.b[i]);
      ss += f * f;
    }
  }
  ss = us::block_sum(ss, scratch);
  const float inv = rsqrtf(ss / (float)H + eps);
  for (int v = threadIdx.x; v < nvec; v += kThreads) {
    us::Pack16 p, q, o;
    p.u = *reinterpret_cast<const uint4*>(xr + v * 8);
    q.u = *reinterpret_cast<const uint4*>(w + v * 8);
#pragma unroll
    for (int i = 0; i < 8; ++i) o.b[i] = us::f2bf(us::bf2f(p.b[i]) * inv * us::bf2f(q.b[i]));
    *reinterpret_cast<uint4*>(yr + v * 8) = o.u;
  }
}

__global__ void __launch_bounds__(kThreads)
add_rmsnorm_kernel(const __nv_bfloat16* __restrict__ x, float* __restrict__ residual,
                   const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y, int H,
                   float eps, int first) {
  US_PDL_PROLOGUE();
  __shared__ float scratch[33];
  const long long row = blockIdx.x;
  const __nv_bfloat16* xr = x + row * H;
  float* rr = residual + row * H;
  __nv_bfloat16* yr = y + row * H;
  const int nvec = H >> 3;
  float ss = 0.f;
  for (int v = threadIdx.x; v < nvec; v += kThreads) {
    us::Pack16 p;
    p.u = *reinterpret_cast<const uint4*>(xr + v * 8);
    float4 r0, r1;
    if (first) {
      r0 = make_float4(0.f, 0.f, 0.f, 0.f);
      r1 = r0;
    } else {
      r0 = *reinterpret_cast<const float4*>(rr + v * 8);
      r1 = *reinterpret_cast<const float4*>(rr + v * 8 + 4);
    }
    r0.x += us::bf2f(p.b[0]); r0.y += us::bf2f(p.b[1]);
    r0.z += us::bf2f(p.b[2]); r0.w += us::bf2f(p.b[3]);
    r1.x += us::bf2f(p.b[4]); r1.y += us::bf2f(p.b[5]);
    r1.z += us::bf2f(p.b[6]); r1.w += us::bf2f(p.b[7]);
    *reinterpret_cast<float4*>(rr + v * 8) = r0;
    *reinterpret_cast<float4*>(rr + v * 8 + 4) = r1;
    ss += r0.x * r0.x + r0.y * r0.y + r0.z * r0.z + r0.w * r0.w;
    ss += r1.x * r1.x + r1.y * r1.y + r1.z * r1.z + r1.w * r1.w;
  }
  ss = us::block_sum(ss, scratch);
  const float inv = rsqrtf(ss / (float)H + eps);
  for (int v = threadIdx.x; v < nvec; v += kThreads) {
    // Each thread re-reads the residual values it wrote itself.
    const float4 r0 = *reinterpret_cast<const float4*>(rr + v * 8);
    const float4 r1 = *reinterpret_cast<const float4*>(rr + v * 8 + 4);
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
    *reinterpret_cast<uint4*>(yr + v * 8) = o.u;
  }
}

// table: [table_rows, H] FP32 vectors; shift row = idx[row] * stride + shift_slot, etc.
__global__ void __launch_bounds__(kThreads)
modulated_rmsnorm_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                         const float* __restrict__ table, const int* __restrict__ idx,
                         int vectors_per_row, int shift_slot, int scale_slot,
                         __nv_bfloat16* __restrict__ y, int H, float eps) {
  US_PDL_PROLOGUE();
  __shared__ float scratch[33];
  const long long row = blockIdx.x;
  const __nv_bfloat16* xr = x + row * H;
  __nv_bfloat16* yr = y + row * H;
  const long long trow = (long long)idx[row] * vectors_per_row;
  const float* shift = table + (trow + shift_slot) * H;
  const float* scale = table + (trow + scale_slot) * H;
  const int nvec = H >> 3;
  float ss = 0.f;
  for (int v = threadIdx.x; v < nvec; v += kThreads) {
    us::Pack16 p;
    p.u = *reinterpret_cast<const uint4*>(xr + v * 8);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float f = us::bf2f(p.b[i]);
      ss += f * f;
    }
  }
  ss = us::block_sum(ss, scratch);
  const float inv = rsqrtf(ss / (float)H + eps);
  for (int v = threadIdx.x; v < nvec; v += kThreads) {
    us::Pack16 p, q, o;
    p.u = *reinterpret_cast<const uint4*>(xr + v * 8);
    if (w) q.u = *reinterpret_cast<const uint4*>(w + v * 8);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float n = us::bf2f(p.b[i]) * inv;
      if (w) n *= us::bf2f(q.b[i]);
      o.b[i] = us::f2bf(n * (1.f + scale[v * 8 + i]) + shift[v * 8 + i]);
    }
    *reinterpret_cast<uint4*>(yr + v * 8) = o.u;
  }
}

__global__ void __launch_bounds__(kThreads)
gated_residual_kernel(__nv_bfloat16* __restrict__ h, const __nv_bfloat16* __restrict__ u,
                      const float* __restrict__ table, const int* __restrict__ idx,
                      int vectors_per_row, int gate_slot, int H) {
  US_PDL_PROLOGUE();
  const long long row = blockIdx.x;
  __nv_bfloat16* hr = h + row * H;
  const __nv_bfloat16* ur = u + row * H;
  const float* gate = table + ((long long)idx[row] * vectors_per_row + gate_slot) * H;
  const int nvec = H >> 3;
  for (int v = threadIdx.x; v < nvec; v += kThreads) {
    us::Pack16 p, q, o;
    p.u = *reinterpret_cast<const uint4*>(hr + v * 8);
    q.u = *reinterpret_cast<const uint4*>(ur + v * 8);
#pragma unroll
    for (int i = 0; i < 8; ++i)
      o.b[i] = us::f2bf(us::bf2f(p.b[i]) + gate[v * 8 + i] * us::bf2f(q.b[i]));
    *reinterpret_cast<uint4*>(hr + v * 8) = o.u;
  }
}

__global__ void __launch_bounds__(kThreads)
layer_norm_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                  const __nv_bfloat16* __restrict__ b, __nv_bfloat16* __restrict__ y, int H,
                  float eps) {
  US_PDL_PROLOGUE();
  __shared__ float scratch[33];
  const long long row = blockIdx.x;
  const __nv_bfloat16* xr = x + row * H;
  __nv_bfloat16* yr = y + row * H;
  float s = 0.f;
  for (int i = threadIdx.x; i < H; i += kThreads) s += us::bf2f(xr[i]);
  const float mean = us::block_sum(s, scratch) / (float)H;
  float vs = 0.f;
  for (int i = threadIdx.x; i < H; i += kThreads) {
    const float d = us::bf2f(xr[i]) - mean;
    vs += d * d;
  }
  const float inv = rsqrtf(us::block_sum(vs, scratch) / (float)H + eps);
  for (int i = threadIdx.x; i < H; i += kThreads) {
    float n = (us::bf2f(xr[i]) - mean) * inv;
    if (w) n *= us::bf2f(w[i]);
    if (b) n += us::bf2f(b[i]);
    yr[i] = us::f2bf(n);
  }
}

// Second half of a fused reduce-scatter and first half of the all-gather that
// follows: `slots` holds one partial product per rank for this rank's own rows
// ([n_slots, T, H] bf16).  r += sum of the slots (FP32, fixed order), y = rmsnorm(r) * w
// for the own rows, and y is stored into every rank's copy of the gathered activations
// (y_peers[p] + row * ldy): the all-gather rides on this kernel's stores, each row
// crosses NVLink once per peer, and the next GEMM reads local memory only.
struct PeerRows {
  __nv_bfloat16* y[8];
  int n;
};

__global__ void __launch_bounds__(kThreads)
reduce_slots_add_rmsnorm_kernel(const __nv_bfloat16* __restrict__ slots, int n_slots,
                                float* __restrict__ residual, const __nv_bfloat16* __restrict__ w,
                                const PeerRows dst, int T, int H, long long ldy, float eps,
                                int first) {
  US_PDL_PROLOGUE();
  __shared__ float scratch[33];
  const long long row = blockIdx.x;
  float* rr = residual + row * H;
  const int nvec = H >> 3;
  float ss = 0.f;
  for (int v = threadIdx.x; v < nvec; v += kThreads) {
    float acc[8];
    if (first) {
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] = 0.f;
    } else {
      const float4 r0 = *reinterpret_cast<const float4*>(rr + v * 8);
      const float4 r1 = *reinterpret_cast<const float4*>(rr + v * 8 + 4);
      acc[0] = r0.x; acc[1] = r0.y; acc[2] = r0.z; acc[3] = r0.w;
      acc[4] = r1.x; acc[5] = r1.y; acc[6] = r1.z; acc[7] = r1.w;
    }
    for (int s = 0; s < n_slots; ++s) {
      us::Pack16 p;
      p.u = *reinterpret_cast<const uint4*>(slots + ((long long)s * T + row) * H + v * 8);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] += us::bf2f(p.b[i]);
    }
    *reinterpret_cast<float4*>(rr + v * 8) = make_float4(acc[0], acc[1], acc[2], acc[3]);
    *reinterpret_cast<float4*>(rr + v * 8 + 4) = make_float4(acc[4], acc[5], acc[6], acc[7]);
#pragma unroll
    for (int i = 0; i < 8; ++i) ss += acc[i] * acc[i];
  }
  ss = us::block_sum(ss, scratch);
  const float inv = rsqrtf(ss / (float)H + eps);
  for (int v = threadIdx.x; v < nvec; v += kThreads) {
    const float4 r0 = *reinterpret_cast<const float4*>(rr + v * 8);
    const float4 r1 = *reinterpret_cast<const float4*>(rr + v * 8 + 4);
    const float r[8] = {r0.x, r0.y, r0.z, r0.w, r1.x, r1.y, r1.z, r1.w};
    us::Pack16 q, o;
    q.u = *reinterpret_cast<const uint4*>(w + v * 8);
#pragma unroll
    for (int i = 0; i < 8; ++i) o.b[i] = us::f2bf(r[i] * inv * us::bf2f(q.b[i]));
    for (int p = 0; p < dst.n; ++p)
      *reinterpret_cast<uint4*>(dst.y[p] + row * ldy + v * 8) = o.u;
  }
}

// Partial rows -> the slot of the rank that owns them (a reduce-scatter by peer stores for a
// partial sum that no GEMM epilogue produced, e.g. the un-permuted expert output): row r goes
// to peers[r / peer_rows] at row slot * peer_rows + r % peer_rows.  One CTA per row, 16-byte
// stores: a row leaves as one contiguous run of whole lines.
__global__ void __launch_bounds__(kThreads)
push_rows_to_slots_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, const PeerRows dst,
                          int rows, int H, int peer_rows, int slot) {
  US_PDL_PROLOGUE();
  const int r = blockIdx.x;
  const int p = r / peer_rows;
  const uint4* src = reinterpret_cast<const uint4*>(x + (long long)r * ldx);
  uint4* out = reinterpret_cast<uint4*>(dst.y[p] +
                                        ((long long)slot * peer_rows + (r - p * peer_rows)) * H);
  for (int v = threadIdx.x; v < (H >> 3); v += kThreads) out[v] = src[v];
}

}  // namespace

US_API int us_push_rows_to_slots(const void* x, long long ldx, void* const* peers, int n_peers,
                                 int rows, int H, int peer_rows, int slot, void* stream) {
  US_REQUIRE(x && peers && n_peers >= 1 && n_peers <= 8 && rows >= 0 && H > 0 && (H % 8) == 0 &&
             (ldx % 8) == 0 && peer_rows > 0 && peer_rows * n_peers >= rows && slot >= 0);
  if (rows == 0) return US_OK;
  PeerRows dst;
  dst.n = n_peers;
  for (int p = 0; p < 8; ++p) dst.y[p] = p < n_peers ? (__nv_bfloat16*)peers[p] : nullptr;
  for (int p = 0; p < n_peers; ++p) US_REQUIRE(dst.y[p] && ((uintptr_t)dst.y[p] % 16) == 0);
  us::launch_pdl(push_rows_to_slots_kernel, dim3(rows), dim3(kThreads), 0, (cudaStream_t)stream,
                 (const __nv_bfloat16*)x, ldx, dst, rows, H, peer_rows, slot);
  US_LAUNCH_CHECK();
  return US_OK;
}

US_API int us_rmsnorm(const void* x, const void* w, void* y, int T, int H, long long ldx,
                      long long ldy, float eps, void* stream) {
  US_REQUIRE(x && w && y && T >= 0 && H > 0 && (H % 8) == 0 && (ldx % 8) == 0 && (ldy % 8) == 0);
  if (T == 0) return US_OK;
  us::launch_pdl(rmsnorm_kernel, dim3(T), dim3(kThreads), 0, (cudaStream_t)stream, (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, (__nv_bfloat16*)y, H, ldx, ldy, eps);
  US_LAUNCH_CHECK();
  return US_OK;
}

US_API int us_add_rmsnorm(const void* x, void* residual, const void* w, void* y, int T, int H,
                          float eps, int first, void* stream) {
  US_REQUIRE(x && residual && w && y && T >= 0 && H > 0 && (H % 8) == 0);
  if (T == 0) return US_OK;
  us::launch_pdl(add_rmsnorm_kernel, dim3(T), dim3(kThreads), 0, (cudaStream_t)stream, (const __nv_bfloat16*)x, (float*)residual, (const __nv_bfloat16*)w, (__nv_bfloat16*)y, H, eps,
      first);
  US_LAUNCH_CHECK();
  return US_OK;
}

US_API int us_modulated_rmsnorm(const void* x, const void* w, const float* table, const int* idx,
                                int vectors_per_row, int shift_slot, int scale_slot, void* y, int T,
                                int H, float eps, void* stream) {
  US_REQUIRE(x && table && idx && y && T >= 0 && H > 0 && (H % 8) == 0);
  if (T == 0) return US_OK;
  us::launch_pdl(modulated_rmsnorm_kernel, dim3(T), dim3(kThreads), 0, (cudaStream_t)stream, (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, table, idx, vectors_per_row, shift_slot,
      scale_slot, (__nv_bfloat16*)y, H, eps);
  US_LAUNCH_CHECK();
  return US_OK;
}

US_API int us_gated_residual(void* h, const void* u, const float* table, const int* idx,
                             int vectors_per_row, int gate_slot, int T, int H, void* stream) {
  US_REQUIRE(h && u && table && idx && T >= 0 && H > 0 && (H % 8) == 0);
  if (T == 0) return US_OK;
  us::launch_pdl(gated_residual_kernel, dim3(T), dim3(kThreads), 0, (cudaStream_t)stream, (__nv_bfloat16*)h, (const __nv_bfloat16*)u, table, idx, vectors_per_row, gate_slot, H);
  US_LAUNCH_CHECK();
  return US_OK;
}

US_API int us_layer_norm(const void* x, const void* w, const void* b, void* y, int T, int H,
                         float eps, void* stream) {
  US_REQUIRE(x && y && T >= 0 && H > 0);
  if (T == 0) return US_OK;
  us::launch_pdl(layer_norm_kernel, dim3(T), dim3(kThreads), 0, (cudaStream_t)stream, (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, (const __nv_bfloat16*)b, (__nv_bfloat16*)y,
      H, eps);
  US_LAUNCH_CHECK();
  return US_OK;
}

// y_peers[p]: address of this rank's first row inside rank p's gathered-activation
// buffer (n_peers entries; a single entry = a plain local output).
US_API int us_reduce_slots_add_rmsnorm(const void* slots, int n_slots, void* residual,
                                       const void* w, void* const* y_peers, int n_peers, int T,
                                       int H, long long ldy, float eps, int first, void* stream) {
  US_REQUIRE(slots && residual && w && y_peers && n_peers >= 1 && n_peers <= 8 && n_slots >= 1 &&
             T >= 0 && H > 0 && (H % 8) == 0 && (ldy % 8) == 0);
  if (T == 0) return US_OK;
  PeerRows dst;
  dst.n = n_peers;
  for (int p = 0; p < 8; ++p) dst.y[p] = p < n_peers ? (__nv_bfloat16*)y_peers[p] : nullptr;
  for (int p = 0; p < n_peers; ++p) US_REQUIRE(dst.y[p] && ((uintptr_t)dst.y[p] % 16) == 0);
  us::launch_pdl(reduce_slots_add_rmsnorm_kernel, dim3(T), dim3(kThreads), 0,
                 (cudaStream_t)stream, (const __nv_bfloat16*)slots, n_slots, (float*)residual,
                 (const __nv_bfloat16*)w, dst, T, H, ldy, eps, first);
  US_LAUNCH_CHECK();
  return US_OK;
}
