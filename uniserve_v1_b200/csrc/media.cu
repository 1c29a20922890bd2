// Pixel- and sample-producing kernels of the video pipeline (all CUDA compute; no
// graphics API is involved anywhere).
//
//   rgb_to_yuv420   decoded frames [F, 3, H, W] in [-1, 1] -> 8-bit BT.709 limited-range
//                   Y, U, V planes ready for the host encoder (4:2:0, 2x2 box chroma)
//   rgb_bytes       the same frames as packed 8-bit RGB (HWC)
//   pcm_interleave  audio [channels, samples] fp32 -> clamp -> interleaved int16
//   tile_stitch     accumulates a decoded spatial tile into the frame canvas with
//                   linear cross-fade weights over the overlap; a second pass divides
//   cross_fade      out = a * (1 - i / n) + b * (i / n) over the temporal overlap tail
//   frame_moments   per-(frame, group) mean / rstd (Welford) for the encoder's GroupNorm
//   frame_norm_pad  pad(silu(group_norm(frame))) for the causal video convolutions
//
// Reference behaviour: crates/ops/kernels/{rgb_bytes,pcm_interleave,tile_stitch,cross_fade}/triton,
// crates/ops/kernels/{frame_moments,frame_norm_pad}/nvcc (reference project paths).
#include "include/us_common.cuh"

namespace {

__device__ __forceinline__ float to_unit(float v) { return fminf(fmaxf(v * 0.5f + 0.5f, 0.f), 1.f); }
__device__ __forceinline__ unsigned char to_u8(float v) {
  return (unsigned char)__float2int_rn(fminf(fmaxf(v, 0.f), 255.f));
}

// grid: (ceil(W/2 / 128), H/2, F); each thread owns a 2x2 pixel quad.
__global__ void __launch_bounds__(128)
rgb_to_yuv420_kernel(const float* __restrict__ rgb, unsigned char* __restrict__ y,
                     unsigned char* __restrict__ u, unsigned char* __restrict__ v, int H, int W) {
  US_PDL_PROLOGUE();
  const int qx = blockIdx.x * blockDim.x + threadIdx.x, qy = blockIdx.y, f = blockIdx.z;
  if (qx >= W / 2) return;
  const size_t plane = (size_t)H * W;
  const float* R = rgb + ((size_t)f * 3 + 0) * plane;
  const float* G = rgb + ((size_t)f * 3 + 1) * plane;
  const float* B = rgb + ((size_t)f * 3 + 2) * plane;
  float cb = 0.f, cr = 0.f;
#pragma unroll
  for (int dy = 0; dy < 2; ++dy)
#pragma unroll
    for (int dx = 0; dx < 2; ++dx) {
      const size_t i = (size_t)(2 * qy + dy) * W + 2 * qx + dx;
      const float r = to_unit(R[i]), g = to_unit(G[i]), b = to_unit(B[i]);
      const float yy = 0.2126f * r + 0.7152f * g + 0.0722f * b;
      y[(size_t)f * plane + i] = to_u8(16.f + 219.f * yy);
      cb += (b - yy) / 1.8556f;
      cr += (r - yy) / 1.5748f;
    }
  const size_t ci = (size_t)f * (plane / 4) + (size_t)qy * (W / 2) + qx;
  u[ci] = to_u8(128.f + 224.f * cb * 0.25f);
  v[ci] = to_u8(128.f + 224.f * cr * 0.25f);
}

__global__ void __launch_bounds__(256)
rgb_bytes_kernel(const float* __restrict__ rgb, unsigned char* __restrict__ out, int H, int W,
                 long long total) {
  US_PDL_PROLOGUE();
  const size_t plane = (size_t)H * W;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int c = (int)(i % 3);
    const long long px = i / 3;
    const long long f = px / plane, p = px % plane;
    out[i] = to_u8(255.f * to_unit(rgb[((size_t)f * 3 + c) * plane + p]));
  }
}

__global__ void __launch_bounds__(256)
pcm_interleave_kernel(const float* __restrict__ x, short* __restrict__ out, int channels,
                      long long samples) {
  US_PDL_PROLOGUE();
  const long long total = samples * channels;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int c = (int)(i % channels);
    const long long s = i / channels;
    const float v = fminf(fmaxf(x[(size_t)c * samples + s], -1.f), 1.f);
    out[i] = (short)__float2int_rn(v * 32767.f);
  }
}

__device__ __forceinline__ float ramp(int i, int n, int overlap, bool lo_edge, bool hi_edge) {
  float w = 1.f;
  if (overlap > 0) {
    if (!lo_edge && i < overlap) w = fminf(w, (i + 1) / (float)(overlap + 1));
    if (!hi_edge && i >= n - overlap) w = fminf(w, (n - i) / (float)(overlap + 1));
  }
  return w;
}

// canvas/weight: [F, C, H, W] / [H, W]; tile: [F, C, th, tw] placed at (y0, x0).
__global__ void __launch_bounds__(256)
tile_stitch_kernel(const float* __restrict__ tile, float* __restrict__ canvas,
                   float* __restrict__ weight, int FC, int H, int W, int th, int tw, int y0,
                   int x0, int overlap, int first_plane) {
  US_PDL_PROLOGUE();
  const long long total = (long long)FC * th * tw;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int tx = (int)(i % tw);
    const int ty = (int)((i / tw) % th);
    const int fc = (int)(i / ((long long)tw * th));
    const int gy = y0 + ty, gx = x0 + tx;
    if (gy >= H || gx >= W) continue;
    const float w = ramp(ty, th, overlap, y0 == 0, y0 + th >= H) *
                    ramp(tx, tw, overlap, x0 == 0, x0 + tw >= W);
    atomicAdd(&canvas[((size_t)fc * H + gy) * W + gx], tile[i] * w);
    if (fc == 0 && first_plane) atomicAdd(&weight[(size_t)gy * W + gx], w);
  }
}

__global__ void __launch_bounds__(256)
tile_normalise_kernel(float* __restrict__ canvas, const float* __restrict__ weight, int FC,
                      long long plane) {
  US_PDL_PROLOGUE();
  const long long total = (long long)FC * plane;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const float w = weight[i % plane];
    canvas[i] = w > 0.f ? canvas[i] / w : 0.f;
  }
}

// a, b: [n, inner]; out[i] = a[i] * (1 - i/n) + b[i] * (i/n)
__global__ void __launch_bounds__(256)
cross_fade_kernel(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ out,
                  int n, long long inner) {
  US_PDL_PROLOGUE();
  const long long total = (long long)n * inner;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const float t = (float)(i / inner) / (float)n;
    out[i] = a[i] * (1.f - t) + b[i] * t;
  }
}

// One CTA per (frame, group): Welford moments over (C/groups) x H x W values.
__global__ void __launch_bounds__(256)
frame_moments_kernel(const float* __restrict__ x, float* __restrict__ mean,
                     float* __restrict__ rstd, long long per_group, float eps) {
  US_PDL_PROLOGUE();
  __shared__ float scratch[33];
  const float* p = x + (size_t)blockIdx.x * per_group;
  float s = 0.f;
  for (long long i = threadIdx.x; i < per_group; i += blockDim.x) s += p[i];
  const float m = us::block_sum(s, scratch) / (float)per_group;
  float v = 0.f;
  for (long long i = threadIdx.x; i < per_group; i += blockDim.x) {
    const float d = p[i] - m;
    v += d * d;
  }
  const float var = us::block_sum(v, scratch) / (float)per_group;
  if (threadIdx.x == 0) {
    mean[blockIdx.x] = m;
    rstd[blockIdx.x] = rsqrtf(var + eps);
  }
}

// x: [F, C, H, W] -> out: [F, C, H + 2p, W + 2p] = pad(silu(group_norm(x))), zero padding.
__global__ void __launch_bounds__(256)
frame_norm_pad_kernel(const float* __restrict__ x, const float* __restrict__ mean,
                      const float* __restrict__ rstd, const float* __restrict__ gamma,
                      const float* __restrict__ beta, float* __restrict__ out, int C, int H, int W,
                      int groups, int pad, long long total) {
  US_PDL_PROLOGUE();
  const int Ho = H + 2 * pad, Wo = W + 2 * pad;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int ox = (int)(i % Wo);
    const int oy = (int)((i / Wo) % Ho);
    const int c = (int)((i / ((long long)Wo * Ho)) % C);
    const long long f = i / ((long long)Wo * Ho * C);
    const int ix = ox - pad, iy = oy - pad;
    float v = 0.f;
    if (ix >= 0 && ix < W && iy >= 0 && iy < H) {
      const int g = c / (C / groups);
      const float n = (x[((f * C + c) * H + iy) * W + ix] - mean[f * groups + g]) *
                          rstd[f * groups + g] * gamma[c] + beta[c];
      v = n / (1.f + __expf(-n));
    }
    out[i] = v;
  }
}

int grid_for(long long n) {
  long long b = (n + 255) / 256;
  return (int)(b < 1 ? 1 : (b > 148 * 32 ? 148 * 32 : b));
}

}  // namespace

US_API int us_rgb_to_yuv420(const float* rgb, void* y, void* u, void* v, int F, int H, int W,
                            void* stream) {
  US_REQUIRE(rgb && y && u && v && F >= 1 && H >= 2 && W >= 2 && (H % 2) == 0 && (W % 2) == 0);
  dim3 grid((W / 2 + 127) / 128, H / 2, F);
  us::launch_pdl(rgb_to_yuv420_kernel, dim3(grid), dim3(128), 0, (cudaStream_t)stream, rgb, (unsigned char*)y, (unsigned char*)u, (unsigned char*)v, H, W);
  US_LAUNCH_CHECK();
  return US_OK;
}

US_API int us_rgb_bytes(const float* rgb, void* out, int F, int H, int W, void* stream) {
  US_REQUIRE(rgb && out && F >= 1 && H >= 1 && W >= 1);
  const long long total = (long long)F * H * W * 3;
  us::launch_pdl(rgb_bytes_kernel, dim3(grid_for(total)), dim3(256), 0, (cudaStream_t)stream, rgb, (unsigned char*)out, H,
                                                                      W, total);
  US_LAUNCH_CHECK();
  return US_OK;
}

US_API int us_pcm_interleave(const float* x, void* out, int channels, long long samples,
                             void* stream) {
  US_REQUIRE(x && out && channels >= 1 && samples >= 0);
  if (samples == 0) return US_OK;
  us::launch_pdl(pcm_interleave_kernel, dim3(grid_for(samples * channels)), dim3(256), 0, (cudaStream_t)stream, x, (short*)out, channels, samples);
  US_LAUNCH_CHECK();
  return US_OK;
}

US_API int us_tile_stitch(const float* tile, float* canvas, float* weight, int FC, int H, int W,
                          int th, int tw, int y0, int x0, int overlap, void* stream) {
  US_REQUIRE(tile && canvas && weight && FC >= 1 && th >= 1 && tw >= 1 && overlap >= 0);
  const long long total = (long long)FC * th * tw;
  us::launch_pdl(tile_stitch_kernel, dim3(grid_for(total)), dim3(256), 0, (cudaStream_t)stream, tile, canvas, weight, FC, H, W, th, tw, y0, x0, overlap, 1);
  US_LAUNCH_CHECK();
  return US_OK;
}

US_API int us_tile_normalise(float* canvas, const float* weight, int FC, int H, int W,
                             void* stream) {
  US_REQUIRE(canvas && weight && FC >= 1);
  const long long plane = (long long)H * W;
  us::launch_pdl(tile_normalise_kernel, dim3(grid_for(plane * FC)), dim3(256), 0, (cudaStream_t)stream, canvas, weight, FC,
                                                                               plane);
  US_LAUNCH_CHECK();
  return US_OK;
}

US_API int us_cross_fade(const float* a, const float* b, float* out, int n, long long inner,
                         void* stream) {
  US_REQUIRE(a && b && out && n >= 1 && inner >= 1);
  us::launch_pdl(cross_fade_kernel, dim3(grid_for((long long)n * inner)), dim3(256), 0, (cudaStream_t)stream, a, b, out, n,
                                                                                      inner);
  US_LAUNCH_CHECK();
  return US_OK;
}

US_API int us_frame_moments(const float* x, float* mean, float* rstd, int frames_x_groups,
                            long long per_group, float eps, void* stream) {
  US_REQUIRE(x && mean && rstd && frames_x_groups >= 1 && per_group >= 1);
  us::launch_pdl(frame_moments_kernel, dim3(frames_x_groups), dim3(256), 0, (cudaStream_t)stream, x, mean, rstd, per_group,
                                                                          eps);
  US_LAUNCH_CHECK();
  return US_OK;
}

US_API int us_frame_norm_pad(const float* x, const float* mean, const float* rstd,
                             const float* gamma, const float* beta, float* out, int F, int C,
                             int H, int W, int groups, int pad, void* stream) {
  US_REQUIRE(x && mean && rstd && gamma && beta && out && C % groups == 0 && pad >= 0);
  const long long total = (long long)F * C * (H + 2 * pad) * (W + 2 * pad);
  us::launch_pdl(frame_norm_pad_kernel, dim3(grid_for(total)), dim3(256), 0, (cudaStream_t)stream, x, mean, rstd, gamma, beta, out, C, H, W, groups, pad, total);
  US_LAUNCH_CHECK();
  return US_OK;
}
