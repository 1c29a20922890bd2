// Diffusion-side kernels of the video pipeline.
//
//   philox_normal   addressable standard normals: element i of a tensor drawn under
//                   (seed, stream) is a function of (seed, stream, i) only, so a
//                   restored request redraws exactly the same noise
//   scaled_add      x += v * s  in FP32 (the Euler step of the flow sampler)
//   patchify        latent [C, F, H, W] fp32 -> rows [F*(H/2)*(W/2), C*4] (1x2x2 patches)
//   unpatchify      the inverse, for the predicted velocity
//   value_first_swiglu  y = value * silu(gate) with stepwise bf16 rounding, for the
//                   unfused path (the GEMM epilogue normally does this)
//
// Reference behaviour: crates/ops/kernels/{philox_noise,scaled_add,patch,unpatchify_video}/triton,
// crates/nn/src/diffusion.rs:9-18 (reference project paths).
#include "include/us_common.cuh"
#include "include/us_philox.h"

namespace {

__global__ void __launch_bounds__(256)
philox_normal_kernel(float* __restrict__ out, long long n, unsigned long long seed,
                     unsigned int stream_id, float scale) {
  US_PDL_PROLOGUE();
  // One counter yields two normals: element pair p covers indices 2p, 2p + 1.
  const long long pairs = (n + 1) / 2;
  for (long long p = (long long)blockIdx.x * blockDim.x + threadIdx.x; p < pairs;
       p += (long long)gridDim.x * blockDim.x) {
    float a, b;
    us_philox_normal2(seed, (unsigned long long)p, stream_id, 1u, &a, &b);
    out[2 * p] = a * scale;
    if (2 * p + 1 < n) out[2 * p + 1] = b * scale;
  }
}

__global__ void __launch_bounds__(256)
scaled_add_kernel(float* __restrict__ x, const float* __restrict__ v, float s, long long n) {
  US_PDL_PROLOGUE();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x)
    x[i] += v[i] * s;
}

// rows[(f*Hp + hp)*Wp + wp][c*4 + dy*2 + dx] = latent[c][f][2hp+dy][2wp+dx]
__global__ void __launch_bounds__(256)
patchify_kernel(const float* __restrict__ latent, float* __restrict__ rows, int C, int Fr, int H,
                int W) {
  US_PDL_PROLOGUE();
  const int Hp = H / 2, Wp = W / 2;
  const long long total = (long long)Fr * Hp * Wp * C * 4;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int col = (int)(i % (C * 4));
    const long long row = i / (C * 4);
    const int c = col >> 2, dy = (col >> 1) & 1, dx = col & 1;
    const int wp = (int)(row % Wp);
    const int hp = (int)((row / Wp) % Hp);
    const int f = (int)(row / ((long long)Wp * Hp));
    rows[i] = latent[(((long long)c * Fr + f) * H + 2 * hp + dy) * W + 2 * wp + dx];
  }
}

__global__ void __launch_bounds__(256)
unpatchify_kernel(const float* __restrict__ rows, float* __restrict__ latent, int C, int Fr,
                  int H, int W) {
  US_PDL_PROLOGUE();
  const int Hp = H / 2, Wp = W / 2;
  const long long total = (long long)Fr * Hp * Wp * C * 4;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int col = (int)(i % (C * 4));
    const long long row = i / (C * 4);
    const int c = col >> 2, dy = (col >> 1) & 1, dx = col & 1;
    const int wp = (int)(row % Wp);
    const int hp = (int)((row / Wp) % Hp);
    const int f = (int)(row / ((long long)Wp * Hp));
    latent[(((long long)c * Fr + f) * H + 2 * hp + dy) * W + 2 * wp + dx] = rows[i];
  }
}

__global__ void __launch_bounds__(256)
value_first_swiglu_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y,
                          long long rows, int I) {
  US_PDL_PROLOGUE();
  const long long total = rows * I;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / I;
    const int c = (int)(i % I);
    const float val = us::bf2f(x[r * 2 * I + c]);
    const float gate = us::bf2f(x[r * 2 * I + I + c]);
    const float s = us::bf2f(us::f2bf(gate / (1.f + __expf(-gate))));
    y[i] = us::f2bf(val * s);
  }
}

int blocks_for(long long n) {
  long long b = (n + 255) / 256;
  return (int)(b < 1 ? 1 : (b > 148 * 16 ? 148 * 16 : b));
}

}  // namespace

US_API int us_philox_normal(float* out, long long n, unsigned long long seed,
                            unsigned int stream_id, float scale, void* stream) {
  US_REQUIRE(out && n >= 0);
  if (n == 0) return US_OK;
  us::launch_pdl(philox_normal_kernel, dim3(blocks_for((n + 1) / 2)), dim3(256), 0, (cudaStream_t)stream, out, n, seed,
                                                                                 stream_id, scale);
  US_LAUNCH_CHECK();
  return US_OK;
}

US_API int us_scaled_add(float* x, const float* v, float s, long long n, void* stream) {
  US_REQUIRE(x && v && n >= 0);
  if (n == 0) return US_OK;
  us::launch_pdl(scaled_add_kernel, dim3(blocks_for(n)), dim3(256), 0, (cudaStream_t)stream, x, v, s, n);
  US_LAUNCH_CHECK();
  return US_OK;
}

US_API int us_patchify(const float* latent, float* rows, int C, int Fr, int H, int W, int inverse,
                       void* stream) {
  US_REQUIRE(latent && rows && C >= 1 && Fr >= 1 && H >= 2 && W >= 2 && (H % 2) == 0 &&
             (W % 2) == 0);
  const long long total = (long long)Fr * (H / 2) * (W / 2) * C * 4;
  if (inverse)
    us::launch_pdl(unpatchify_kernel, dim3(blocks_for(total)), dim3(256), 0, (cudaStream_t)stream, rows, const_cast<float*>(latent), C, Fr, H, W);
  else
    us::launch_pdl(patchify_kernel, dim3(blocks_for(total)), dim3(256), 0, (cudaStream_t)stream, latent, rows, C, Fr, H,
                                                                         W);
  US_LAUNCH_CHECK();
  return US_OK;
}

US_API int us_value_first_swiglu(const void* x, void* y, long long rows, int I, void* stream) {
  US_REQUIRE(x && y && rows >= 0 && I >= 1);
  if (rows == 0) return US_OK;
  us::launch_pdl(value_first_swiglu_kernel, dim3(blocks_for(rows * I)), dim3(256), 0, (cudaStream_t)stream, (const __nv_bfloat16*)x, (__nv_bfloat16*)y, rows, I);
  US_LAUNCH_CHECK();
  return US_OK;
}
