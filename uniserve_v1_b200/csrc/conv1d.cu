// FP32 1-D convolutions of the audio VAE (BigVGAN decoder, DAC encoder): conv1d with
// dilation, transposed conv1d (upsampling), the snake activation and the
// anti-aliased activation (2x FIR upsample -> snake -> 2x FIR downsample) in one pass.
// FP32 accumulate, no TF32, as the audio path requires.
//
// conv1d: out[b, co, t] = bias[co] + sum_{ci, k} w[co, ci, k] * x[b, ci, t*stride - pad + k*dil]
// A CTA computes a [32 output channels x 128 time steps] tile; input rows are staged
// through shared memory in chunks of 8 input channels.
//
// Reference behaviour: crates/ops/kernels/conv/cudnn/src/conv.cu (cuDNN backend graph),
// crates/ops/kernels/{snake,activation1d}/triton, crates/models/src/minimax_h3/audio_vae.rs:1-30
// (reference project paths).
#include "include/us_common.cuh"

namespace {

constexpr int kCo = 32, kT = 128, kCi = 8;

__global__ void __launch_bounds__(256)
conv1d_kernel(const float* __restrict__ x, const float* __restrict__ w,
              const float* __restrict__ bias, float* __restrict__ out, int Cin, int Cout, int Lin,
              int Lout, int K, int stride, int pad, int dil) {
  US_PDL_PROLOGUE();
  extern __shared__ float sm[];
  const int span = (kT - 1) * stride + (K - 1) * dil + 1;
  float* xs = sm;                       // [kCi][span]
  float* ws = sm + kCi * span;          // [kCo][kCi][K]
  const int b = blockIdx.z, co0 = blockIdx.y * kCo, t0 = blockIdx.x * kT;
  const int tid = threadIdx.x;
  const int tl = tid % 32;              // 4 time steps each: tl, tl+32, tl+64, tl+96
  const int cl = tid / 32;              // 4 channels each: cl, cl+8, cl+16, cl+24
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  const int in0 = t0 * stride - pad;
  for (int ci0 = 0; ci0 < Cin; ci0 += kCi) {
    for (int i = tid; i < kCi * span; i += 256) {
      const int c = i / span, p = i % span;
      const int ci = ci0 + c, pos = in0 + p;
      xs[i] = (ci < Cin && pos >= 0 && pos < Lin) ? x[((size_t)b * Cin + ci) * Lin + pos] : 0.f;
    }
    for (int i = tid; i < kCo * kCi * K; i += 256) {
      const int k = i % K, c = (i / K) % kCi, o = i / (K * kCi);
      const int co = co0 + o, ci = ci0 + c;
      ws[i] = (co < Cout && ci < Cin) ? w[((size_t)co * Cin + ci) * K + k] : 0.f;
    }
    __syncthreads();
    for (int c = 0; c < kCi; ++c)
      for (int k = 0; k < K; ++k) {
        float xv[4], wv[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) xv[j] = xs[c * span + (tl + 32 * j) * stride + k * dil];
#pragma unroll
        for (int i = 0; i < 4; ++i) wv[i] = ws[((cl + 8 * i) * kCi + c) * K + k];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[i][j] += wv[i] * xv[j];
      }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int co = co0 + cl + 8 * i;
    if (co >= Cout) continue;
    const float bv = bias ? bias[co] : 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int t = t0 + tl + 32 * j;
      if (t < Lout) out[((size_t)b * Cout + co) * Lout + t] = acc[i][j] + bv;
    }
  }
}

// Transposed conv: out[b, co, t] = bias[co] + sum_{ci, k : (t + pad - k) % stride == 0}
//                                   w[ci, co, k] * x[b, ci, (t + pad - k) / stride]
__global__ void __launch_bounds__(256)
conv_transpose1d_kernel(const float* __restrict__ x, const float* __restrict__ w,
                        const float* __restrict__ bias, float* __restrict__ out, int Cin, int Cout,
                        int Lin, int Lout, int K, int stride, int pad) {
  US_PDL_PROLOGUE();
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  const int co = blockIdx.y, b = blockIdx.z;
  if (t >= Lout) return;
  float acc = bias ? bias[co] : 0.f;
  for (int k = (t + pad) % stride; k < K; k += stride) {
    const int s = (t + pad - k) / stride;
    if (s < 0 || s >= Lin) continue;
    for (int ci = 0; ci < Cin; ++ci)
      acc += w[((size_t)ci * Cout + co) * K + k] * x[((size_t)b * Cin + ci) * Lin + s];
  }
  out[((size_t)b * Cout + co) * Lout + t] = acc;
}

// snake: y = x + sin(alpha x)^2 / (beta + eps), alpha/beta given as logs per channel.
__device__ __forceinline__ float snake_f(float x, float alpha, float inv_beta) {
  const float s = sinf(alpha * x);
  return x + s * s * inv_beta;
}

__global__ void __launch_bounds__(256)
snake_kernel(const float* __restrict__ x, const float* __restrict__ log_alpha,
             const float* __restrict__ log_beta, float* __restrict__ out, int C, long long L,
             long long total) {
  US_PDL_PROLOGUE();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int c = (int)((i / L) % C);
    out[i] = snake_f(x[i], __expf(log_alpha[c]), 1.f / (__expf(log_beta[c]) + 1e-9f));
  }
}

// Anti-aliased activation: zero-stuff x2 and low-pass with `taps` (length 12, gain 2),
// snake at the double rate, low-pass again and keep every second sample.
__global__ void __launch_bounds__(256)
activation1d_kernel(const float* __restrict__ x, const float* __restrict__ taps,
                    const float* __restrict__ log_alpha, const float* __restrict__ log_beta,
                    float* __restrict__ out, int C, int L, int ntaps) {
  US_PDL_PROLOGUE();
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  const int c = blockIdx.y % C;
  const size_t row = (size_t)blockIdx.y * L;
  if (t >= L) return;
  const float alpha = __expf(log_alpha[c]), inv_beta = 1.f / (__expf(log_beta[c]) + 1e-9f);
  const int half = ntaps / 2;
  float acc = 0.f;
  // output sample t sits at up-rate position 2t; the down filter covers 2t - half .. 2t + half - 1
  for (int j = 0; j < ntaps; ++j) {
    const int u = 2 * t - half + j;       // up-rate index
    float up = 0.f;
    for (int k = 0; k < ntaps; ++k) {
      const int src2 = u - half + k;      // zero-stuffed index, even = sample src2 / 2
      if ((src2 & 1) == 0) {
        int s = src2 / 2;
        s = s < 0 ? 0 : (s >= L ? L - 1 : s);   // replicate padding
        up += 2.f * taps[k] * x[row + s];
      }
    }
    acc += taps[j] * snake_f(up, alpha, inv_beta);
  }
  out[row + t] = acc;
}

}  // namespace

US_API int us_conv1d(const float* x, const float* w, const float* bias, float* out, int B, int Cin,
                     int Cout, int Lin, int K, int stride, int pad, int dil, void* stream) {
  US_REQUIRE(x && w && out && B >= 1 && Cin >= 1 && Cout >= 1 && K >= 1 && stride >= 1 && dil >= 1);
  const int Lout = (Lin + 2 * pad - dil * (K - 1) - 1) / stride + 1;
  US_REQUIRE(Lout >= 1);
  const int span = (kT - 1) * stride + (K - 1) * dil + 1;
  const size_t smem = (size_t)(kCi * span + kCo * kCi * K) * sizeof(float);
  US_REQUIRE(smem <= 200 * 1024);
  if (smem > 48 * 1024)
    US_CUDA_CHECK(cudaFuncSetAttribute(conv1d_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)smem));
  dim3 grid((Lout + kT - 1) / kT, (Cout + kCo - 1) / kCo, B);
  us::launch_pdl(conv1d_kernel, dim3(grid), dim3(256), smem, (cudaStream_t)stream, x, w, bias, out, Cin, Cout, Lin, Lout,
                                                           K, stride, pad, dil);
  US_LAUNCH_CHECK();
  return US_OK;
}

US_API int us_conv_transpose1d(const float* x, const float* w, const float* bias, float* out,
                               int B, int Cin, int Cout, int Lin, int K, int stride, int pad,
                               void* stream) {
  US_REQUIRE(x && w && out && B >= 1 && Cin >= 1 && Cout >= 1 && K >= 1 && stride >= 1);
  const int Lout = (Lin - 1) * stride - 2 * pad + K;
  US_REQUIRE(Lout >= 1 && Cout <= 65535);
  dim3 grid((Lout + 255) / 256, Cout, B);
  us::launch_pdl(conv_transpose1d_kernel, dim3(grid), dim3(256), 0, (cudaStream_t)stream, x, w, bias, out, Cin, Cout, Lin,
                                                                  Lout, K, stride, pad);
  US_LAUNCH_CHECK();
  return US_OK;
}

US_API int us_snake(const float* x, const float* log_alpha, const float* log_beta, float* out,
                    int B, int C, long long L, void* stream) {
  US_REQUIRE(x && log_alpha && log_beta && out);
  const long long total = (long long)B * C * L;
  long long blocks = (total + 255) / 256;
  if (blocks > 148 * 32) blocks = 148 * 32;
  us::launch_pdl(snake_kernel, dim3((int)blocks), dim3(256), 0, (cudaStream_t)stream, x, log_alpha, log_beta, out, C, L,
                                                              total);
  US_LAUNCH_CHECK();
  return US_OK;
}

US_API int us_activation1d(const float* x, const float* taps, const float* log_alpha,
                           const float* log_beta, float* out, int B, int C, int L, int ntaps,
                           void* stream) {
  US_REQUIRE(x && taps && log_alpha && log_beta && out && ntaps >= 2 && (ntaps % 2) == 0);
  US_REQUIRE((long long)B * C <= 65535);
  dim3 grid((L + 255) / 256, B * C);
  us::launch_pdl(activation1d_kernel, dim3(grid), dim3(256), 0, (cudaStream_t)stream, x, taps, log_alpha, log_beta, out, C,
                                                              L, ntaps);
  US_LAUNCH_CHECK();
  return US_OK;
}
