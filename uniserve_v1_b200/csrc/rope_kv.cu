// Per-head q/k RMSNorm fused with the rotary embedding and the paged KV write.
//
// One warp owns one (token, head) row of the fused QKV projection output.  The
// row is normalised in FP32, rotated in FP32 and rounded once; K and V rows are
// also scattered into the paged cache at `slot_mapping[token]` (slot =
// page * page_size + offset, a negative slot writes nothing).
//
// Text models: one position per token, NeoX (half-split) or interleaved pairing
// over the first `rot` channels.  Video transformer: three coordinates per row
// (time, height, width), `freqs_per_axis` frequencies each, rotating
// 2 * 3 * freqs_per_axis channels of every head.
//
// Reference behaviour: crates/ops/kernels/qk_norm_rope/triton, crates/ops/src/rope.rs,
// crates/ops/src/kv.rs (reference project paths).
#include "include/us_common.cuh"

namespace {

constexpr int kWarps = 4;
constexpr int kMaxD = 256;

struct RopeArgs {
  __nv_bfloat16* qkv;      // [T, (Hq + 2 Hkv) * D], rotated in place
  const __nv_bfloat16* qw; // [D] or null
  const __nv_bfloat16* kw; // [D] or null
  const int* positions;    // [T]
  const float* inv_freq;   // [rot / 2]
  const int* slots;        // [T] or null
  __nv_bfloat16* kcache;   // [slots_total, Hkv, D] or null
  __nv_bfloat16* vcache;
  int T, Hq, Hkv, D, rot, interleaved;
  float eps;
};

__global__ void __launch_bounds__(kWarps * 32) qk_norm_rope_kv_kernel(const RopeArgs a) {
  US_PDL_PROLOGUE();
  __shared__ float rows[kWarps][kMaxD];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int heads = a.Hq + 2 * a.Hkv;
  const long long unit = (long long)blockIdx.x * kWarps + warp;
  if (unit >= (long long)a.T * heads) return;
  const int t = (int)(unit / heads), h = (int)(unit % heads);
  __nv_bfloat16* row = a.qkv + ((long long)t * heads + h) * a.D;
  float* buf = rows[warp];
  const int D = a.D;

  const bool is_q = h < a.Hq;
  const bool is_k = !is_q && h < a.Hq + a.Hkv;
  const int slot = a.slots ? a.slots[t] : -1;

  if (!is_q && !is_k) {  // V head: copy into the cache
    if (a.vcache && slot >= 0) {
      __nv_bfloat16* dst = a.vcache + ((long long)slot * a.Hkv + (h - a.Hq - a.Hkv)) * D;
      for (int i = lane; i < D; i += 32) dst[i] = row[i];
    }
    return;
  }

  float ss = 0.f;
  for (int i = lane; i < D; i += 32) {
    const float f = us::bf2f(row[i]);
    buf[i] = f;
    ss += f * f;
  }
  const __nv_bfloat16* w = is_q ? a.qw : a.kw;
  if (w) {
    ss = us::warp_sum(ss);
    const float inv = rsqrtf(ss / (float)D + a.eps);
    __syncwarp();
    for (int i = lane; i < D; i += 32) buf[i] = buf[i] * inv * us::bf2f(w[i]);
  }
  __syncwarp();

  const float pos = (float)a.positions[t];
  const int half = a.rot >> 1;
  __nv_bfloat16* kdst = nullptr;
  if (is_k && a.kcache && slot >= 0)
    kdst = a.kcache + ((long long)slot * a.Hkv + (h - a.Hq)) * D;

  for (int i = lane; i < D; i += 32) {
    float out;
    if (i < a.rot) {
      int pair, fidx;
      float sign;
      if (a.interleaved) {
        fidx = i >> 1;
        pair = i ^ 1;
        sign = (i & 1) ? 1.f : -1.f;
      } else {
        fidx = i < half ? i : i - half;
        pair = i < half ? i + half : i - half;
        sign = i < half ? -1.f : 1.f;
      }
      float sn, cs;
      sincosf(pos * a.inv_freq[fidx], &sn, &cs);
      out = buf[i] * cs + sign * buf[pair] * sn;
    } else {
      out = buf[i];
    }
    const __nv_bfloat16 o = us::f2bf(out);
    row[i] = o;
    if (kdst) kdst[i] = o;
  }
}

// Fast path for 128-wide heads rotated over all channels with half-split (NeoX) pairing:
// a CTA owns one token (and a slice of its heads), computes the token's 64 (cos, sin)
// factors once into shared memory, then every warp takes whole heads: a lane owns four
// adjacent channels (one 8-byte access each way), its rotation partner is lane ^ 16.
// The arithmetic and its rounding points are those of the general kernel above.
constexpr int kFastWarps = 8;
__global__ void __launch_bounds__(kFastWarps * 32) qk_norm_rope_kv_fast_kernel(const RopeArgs a,
                                                                             const int heads_per_cta) {
  US_PDL_PROLOGUE();
  __shared__ float2 tab[64];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int heads = a.Hq + 2 * a.Hkv;
  const int t = blockIdx.x;
  if (threadIdx.x < 64) {
    float sn, cs;
    sincosf((float)a.positions[t] * a.inv_freq[threadIdx.x], &sn, &cs);
    tab[threadIdx.x] = make_float2(cs, sn);
  }
  __syncthreads();
  const int slot = a.slots ? a.slots[t] : -1;
  const int h_lo = blockIdx.y * heads_per_cta;
  const int h_hi = min(heads, h_lo + heads_per_cta);
  const float sign = lane < 16 ? -1.f : 1.f;
  float2 f[4];
#pragma unroll
  for (int e = 0; e < 4; ++e) f[e] = tab[((lane & 15) << 2) + e];
  for (int h = h_lo + warp; h < h_hi; h += kFastWarps) {
    __nv_bfloat16* row = a.qkv + ((long long)t * heads + h) * 128 + lane * 4;
    const uint2 raw = *reinterpret_cast<const uint2*>(row);
    const bool is_q = h < a.Hq;
    const bool is_k = !is_q && h < a.Hq + a.Hkv;
    if (!is_q && !is_k) {
      if (a.vcache && slot >= 0)
        *reinterpret_cast<uint2*>(a.vcache + ((long long)slot * a.Hkv + (h - a.Hq - a.Hkv)) * 128 +
                                  lane * 4) = raw;
      continue;
    }
    const __nv_bfloat162 p0 = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
    const __nv_bfloat162 p1 = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
    float x[4] = {__low2float(p0), __high2float(p0), __low2float(p1), __high2float(p1)};
    const __nv_bfloat16* w = is_q ? a.qw : a.kw;
    if (w) {
      float ss = x[0] * x[0] + x[1] * x[1] + x[2] * x[2] + x[3] * x[3];
      ss = us::warp_sum(ss);
      const float inv = rsqrtf(ss / 128.f + a.eps);
      const uint2 wr = *reinterpret_cast<const uint2*>(w + lane * 4);
      const __nv_bfloat162 w0 = *reinterpret_cast<const __nv_bfloat162*>(&wr.x);
      const __nv_bfloat162 w1 = *reinterpret_cast<const __nv_bfloat162*>(&wr.y);
      x[0] = x[0] * inv * __low2float(w0);
      x[1] = x[1] * inv * __high2float(w0);
      x[2] = x[2] * inv * __low2float(w1);
      x[3] = x[3] * inv * __high2float(w1);
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float y = __shfl_xor_sync(0xffffffffu, x[e], 16);
      x[e] = x[e] * f[e].x + sign * y * f[e].y;
    }
    const __nv_bfloat162 o0 = __floats2bfloat162_rn(x[0], x[1]);
    const __nv_bfloat162 o1 = __floats2bfloat162_rn(x[2], x[3]);
    uint2 out;
    out.x = *reinterpret_cast<const uint32_t*>(&o0);
    out.y = *reinterpret_cast<const uint32_t*>(&o1);
    *reinterpret_cast<uint2*>(row) = out;
    if (is_k && a.kcache && slot >= 0)
      *reinterpret_cast<uint2*>(a.kcache + ((long long)slot * a.Hkv + (h - a.Hq)) * 128 + lane * 4) = out;
  }
}

struct Rope3Args {
  __nv_bfloat16* q;        // [T, Hq * D] rows with leading dimension ldq
  __nv_bfloat16* k;        // [T, Hk * D] rows with leading dimension ldk
  const __nv_bfloat16* qw; // [D] or null
  const __nv_bfloat16* kw;
  const float* coords;     // [3, T] (time, height, width)
  const float* inv_freq;   // [freqs_per_axis]
  const float2* table;     // optional [T, 3 * freqs_per_axis] (cos, sin): replaces sincosf
  int T, Hq, Hk, D, freqs_per_axis;
  long long ldq, ldk;
  float eps;
};

// Channel layout of the rotated part: axis a in {0,1,2} owns channels
// [a * 2F, (a + 1) * 2F) as F half-split pairs (i, i + F).
__global__ void __launch_bounds__(kWarps * 32) qk_norm_rope3_kernel(const Rope3Args a) {
  US_PDL_PROLOGUE();
  __shared__ float rows[kWarps][kMaxD];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int heads = a.Hq + a.Hk;
  const long long unit = (long long)blockIdx.x * kWarps + warp;
  if (unit >= (long long)a.T * heads) return;
  const int t = (int)(unit / heads), h = (int)(unit % heads);
  const bool is_q = h < a.Hq;
  __nv_bfloat16* row = is_q ? a.q + (long long)t * a.ldq + (long long)h * a.D
                            : a.k + (long long)t * a.ldk + (long long)(h - a.Hq) * a.D;
  float* buf = rows[warp];
  const int D = a.D;
  float ss = 0.f;
  for (int i = lane; i < D; i += 32) {
    const float f = us::bf2f(row[i]);
    buf[i] = f;
    ss += f * f;
  }
  const __nv_bfloat16* w = is_q ? a.qw : a.kw;
  if (w) {
    ss = us::warp_sum(ss);
    const float inv = rsqrtf(ss / (float)D + a.eps);
    __syncwarp();
    for (int i = lane; i < D; i += 32) buf[i] = buf[i] * inv * us::bf2f(w[i]);
  }
  __syncwarp();
  const int F = a.freqs_per_axis;
  const int rot = 6 * F;
  for (int i = lane; i < D; i += 32) {
    float out = buf[i];
    if (i < rot) {
      const int axis = i / (2 * F);
      const int j = i - axis * 2 * F;
      const int fidx = j < F ? j : j - F;
      const int pair = j < F ? i + F : i - F;
      const float sign = j < F ? -1.f : 1.f;
      float sn, cs;
      if (a.table != nullptr) {
        const float2 e = a.table[(long long)t * 3 * F + axis * F + fidx];
        cs = e.x;
        sn = e.y;
      } else {
        sincosf(a.coords[(long long)axis * a.T + t] * a.inv_freq[fidx], &sn, &cs);
      }
      out = buf[i] * cs + sign * buf[pair] * sn;
    }
    row[i] = us::f2bf(out);
  }
}

// Fast path of the three-axis rotary for 128-wide heads with 16 frequencies per
// axis and a (cos, sin) table: one warp per (row, head), every lane owns four
// adjacent channels (one 8-byte access each way), the rotation partner of a
// channel lives in lane ^ 4, no shared memory.
__global__ void __launch_bounds__(256) qk_norm_rope3_fast_kernel(const Rope3Args a) {
  US_PDL_PROLOGUE();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int heads = a.Hq + a.Hk;
  const long long unit = (long long)blockIdx.x * 8 + warp;
  if (unit >= (long long)a.T * heads) return;
  const int t = (int)(unit / heads), h = (int)(unit % heads);
  const bool is_q = h < a.Hq;
  __nv_bfloat16* row = is_q ? a.q + (long long)t * a.ldq + (long long)h * 128
                            : a.k + (long long)t * a.ldk + (long long)(h - a.Hq) * 128;
  uint2 raw = *reinterpret_cast<const uint2*>(row + lane * 4);
  const __nv_bfloat162 p0 = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
  const __nv_bfloat162 p1 = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
  float x[4] = {__low2float(p0), __high2float(p0), __low2float(p1), __high2float(p1)};
  const __nv_bfloat16* w = is_q ? a.qw : a.kw;
  if (w) {
    float ss = x[0] * x[0] + x[1] * x[1] + x[2] * x[2] + x[3] * x[3];
    ss = us::warp_sum(ss);
    const float inv = rsqrtf(ss / 128.f + a.eps);
    const uint2 wr = *reinterpret_cast<const uint2*>(w + lane * 4);
    const __nv_bfloat162 w0 = *reinterpret_cast<const __nv_bfloat162*>(&wr.x);
    const __nv_bfloat162 w1 = *reinterpret_cast<const __nv_bfloat162*>(&wr.y);
    x[0] *= inv * __low2float(w0);
    x[1] *= inv * __high2float(w0);
    x[2] *= inv * __low2float(w1);
    x[3] *= inv * __high2float(w1);
  }
  // channels [32 axis, 32 axis + 32): lanes 8 axis .. 8 axis + 7; first half pairs with +16
  float y[4];
#pragma unroll
  for (int e = 0; e < 4; ++e) y[e] = __shfl_xor_sync(0xffffffffu, x[e], 4);
  if (lane < 24) {
    const int axis = lane >> 3;
    const float sign = (lane & 4) ? 1.f : -1.f;
    const float2* tab = a.table + (long long)t * 48 + axis * 16 + (lane & 3) * 4;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 cs = tab[e];
      x[e] = x[e] * cs.x + sign * y[e] * cs.y;
    }
  }
  __nv_bfloat162 o0 = __floats2bfloat162_rn(x[0], x[1]);
  __nv_bfloat162 o1 = __floats2bfloat162_rn(x[2], x[3]);
  uint2 out;
  out.x = *reinterpret_cast<uint32_t*>(&o0);
  out.y = *reinterpret_cast<uint32_t*>(&o1);
  *reinterpret_cast<uint2*>(row + lane * 4) = out;
}

}  // namespace

US_API int us_qk_norm_rope_kv(void* qkv, const void* qw, const void* kw, const int* positions,
                              const float* inv_freq, const int* slots, void* kcache, void* vcache,
                              int T, int Hq, int Hkv, int D, int rot, int interleaved, float eps,
                              void* stream) {
  US_REQUIRE(qkv && positions && inv_freq && T >= 0 && D > 0 && D <= kMaxD && rot <= D &&
             (rot % 2) == 0);
  if (T == 0) return US_OK;
  RopeArgs a;
  a.qkv = (__nv_bfloat16*)qkv;
  a.qw = (const __nv_bfloat16*)qw;
  a.kw = (const __nv_bfloat16*)kw;
  a.positions = positions;
  a.inv_freq = inv_freq;
  a.slots = slots;
  a.kcache = (__nv_bfloat16*)kcache;
  a.vcache = (__nv_bfloat16*)vcache;
  a.T = T; a.Hq = Hq; a.Hkv = Hkv; a.D = D; a.rot = rot; a.interleaved = interleaved;
  a.eps = eps;
  const long long units = (long long)T * (Hq + 2 * Hkv);
  const bool aligned = ((uintptr_t)qkv % 8) == 0 && (!qw || (uintptr_t)qw % 8 == 0) &&
                       (!kw || (uintptr_t)kw % 8 == 0) && (!kcache || (uintptr_t)kcache % 8 == 0) &&
                       (!vcache || (uintptr_t)vcache % 8 == 0);
  if (D == 128 && rot == 128 && !interleaved && aligned) {
    // few tokens (decode): split a token's heads over several CTAs so that the grid fills the GPU
    const int heads = Hq + 2 * Hkv;
    int split = (int)((2 * 148 + T - 1) / T);
    split = split < 1 ? 1 : split;
    const int max_split = (heads + kFastWarps - 1) / kFastWarps;
    if (split > max_split) split = max_split;
    const int per = (heads + split - 1) / split;
    split = (heads + per - 1) / per;
    us::launch_pdl(qk_norm_rope_kv_fast_kernel, dim3((unsigned)T, (unsigned)split), dim3(kFastWarps * 32),
                   0, (cudaStream_t)stream, a, per);
    US_LAUNCH_CHECK();
    return US_OK;
  }
  const int blocks = (int)((units + kWarps - 1) / kWarps);
  us::launch_pdl(qk_norm_rope_kv_kernel, dim3(blocks), dim3(kWarps * 32), 0, (cudaStream_t)stream, a);
  US_LAUNCH_CHECK();
  return US_OK;
}

namespace {
int rope3_impl(void* q, void* k, const void* qw, const void* kw, const float* coords,
               const float* inv_freq, const float* table, int T, int Hq, int Hk, int D,
               int freqs_per_axis, long long ldq, long long ldk, float eps, void* stream) {
  US_REQUIRE(q && k && (table || (coords && inv_freq)) && T >= 0 && D > 0 && D <= kMaxD &&
             6 * freqs_per_axis <= D);
  if (T == 0) return US_OK;
  Rope3Args a;
  a.q = (__nv_bfloat16*)q; a.k = (__nv_bfloat16*)k;
  a.qw = (const __nv_bfloat16*)qw; a.kw = (const __nv_bfloat16*)kw;
  a.coords = coords; a.inv_freq = inv_freq;
  a.table = (const float2*)table;
  a.T = T; a.Hq = Hq; a.Hk = Hk; a.D = D; a.freqs_per_axis = freqs_per_axis;
  a.ldq = ldq; a.ldk = ldk; a.eps = eps;
  const long long units = (long long)T * (Hq + Hk);
  if (table && D == 128 && freqs_per_axis == 16 && (ldq % 4) == 0 && (ldk % 4) == 0 &&
      ((uintptr_t)q % 8) == 0 && ((uintptr_t)k % 8) == 0) {
    us::launch_pdl(qk_norm_rope3_fast_kernel, dim3((unsigned)((units + 7) / 8)), dim3(256), 0,
                   (cudaStream_t)stream, a);
    US_LAUNCH_CHECK();
    return US_OK;
  }
  const int blocks = (int)((units + kWarps - 1) / kWarps);
  us::launch_pdl(qk_norm_rope3_kernel, dim3(blocks), dim3(kWarps * 32), 0, (cudaStream_t)stream, a);
  US_LAUNCH_CHECK();
  return US_OK;
}
}  // namespace

US_API int us_qk_norm_rope3(void* q, void* k, const void* qw, const void* kw, const float* coords,
                            const float* inv_freq, int T, int Hq, int Hk, int D,
                            int freqs_per_axis, long long ldq, long long ldk, float eps,
                            void* stream) {
  return rope3_impl(q, k, qw, kw, coords, inv_freq, nullptr, T, Hq, Hk, D, freqs_per_axis, ldq,
                    ldk, eps, stream);
}

// Same with the rotation factors read from a table [T, 3 * freqs_per_axis] of
// (cos, sin) pairs, built once per request (the coordinates do not change between
// blocks or steps).
US_API int us_qk_norm_rope3_table(void* q, void* k, const void* qw, const void* kw,
                                  const float* table, int T, int Hq, int Hk, int D,
                                  int freqs_per_axis, long long ldq, long long ldk, float eps,
                                  void* stream) {
  return rope3_impl(q, k, qw, kw, nullptr, nullptr, table, T, Hq, Hk, D, freqs_per_axis, ldq, ldk,
                    eps, stream);
}
