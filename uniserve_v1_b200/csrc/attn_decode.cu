// Paged-KV decode attention with split-KV (one query token per sequence).
//
// Grid = (sequence, kv head, split).  A CTA streams its share of the sequence's
// pages through shared memory with cp.async (double buffered), serves all G
// query heads of the kv head from the same tile, and keeps a running
// (max, sum, output) per head.  With more than one split the CTAs write
// normalised partial outputs and log-sum-exp values into a scratch buffer and
// a second kernel merges them.
//
// Cache layout: [pages, page_size, kv_heads, head_dim] bf16 for K and for V;
// page_table [batch, max_pages] int32; seq_lens [batch] int32 counts the keys
// to attend (the current token's K/V is already in the cache).
//
// Reference behaviour: crates/ops/src/attention/mod.rs:7-15 and
// crates/ops/kernels/paged_attention (reference project paths).
#include <stdio.h>

#include "include/us_common.cuh"
#include "include/us_noalloc.h"

namespace {

constexpr int kTile = 32;      // keys per tile
constexpr int kThreads = 128;

struct DecodeArgs {
  const __nv_bfloat16* q;  // [B, Hq, D] with row stride ldq
  const __nv_bfloat16* kc;
  const __nv_bfloat16* vc;
  const int* page_table;
  const int* seq_lens;
  __nv_bfloat16* out;      // [B, Hq, D] with row stride ldo
  float* part_o;           // [B, Hq, splits, D]
  float* part_lse;         // [B, Hq, splits]
  long long ldq, ldo;
  int B, Hq, Hkv, max_pages, page_size, splits, window;
  float scale;
};

__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(
                   (uint32_t)__cvta_generic_to_shared(dst)),
               "l"(src)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

template <int D, int G>
__global__ void __launch_bounds__(kThreads) paged_decode_kernel(const DecodeArgs a) {
  US_PDL_PROLOGUE();
  constexpr int kPad = 8;                      // bf16 elements of row padding for K
  constexpr int kPairs = D / 2;                // bf16x2 columns of V
  constexpr int kGroups = kThreads / kPairs;   // head groups in the PV phase
  constexpr int kHpt = (G + kGroups - 1) / kGroups;
  constexpr int kChunks = D / 8;               // 16-byte chunks per row
  static_assert(kThreads % kPairs == 0, "head_dim must divide the block");

  __shared__ __align__(16) __nv_bfloat16 Ks[2][kTile][D + kPad];
  __shared__ __align__(16) __nv_bfloat16 Vs[2][kTile][D];
  __shared__ __align__(16) float Qs[G][D];
  __shared__ float Ps[G][kTile];
  __shared__ float Scale[G];
  __shared__ float Lsum[G];
  __shared__ float Mmax[G];

  const int b = blockIdx.x, hk = blockIdx.y, split = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int seq_len = a.seq_lens[b];
  int begin_all = 0;
  if (a.window > 0 && seq_len > a.window) begin_all = seq_len - a.window;
  const int span = seq_len - begin_all;
  const int tiles_all = (span + kTile - 1) / kTile;
  const int tiles_per = (tiles_all + a.splits - 1) / a.splits;
  const int k_begin = begin_all + split * tiles_per * kTile;
  const int k_end = min(seq_len, k_begin + tiles_per * kTile);
  const int ntiles = k_end > k_begin ? (k_end - k_begin + kTile - 1) / kTile : 0;

  // Query rows of this kv head's group, pre-scaled.
  for (int i = tid; i < G * D; i += kThreads) {
    const int g = i / D, d = i - g * D;
    Qs[g][d] = us::bf2f(a.q[(long long)b * a.ldq + (long long)(hk * G + g) * D + d]) * a.scale;
  }
  if (tid < G) {
    Mmax[tid] = -INFINITY;
    Lsum[tid] = 0.f;
  }
  float acc[kHpt][2];
#pragma unroll
  for (int i = 0; i < kHpt; ++i) acc[i][0] = acc[i][1] = 0.f;

  const int* pt = a.page_table + (long long)b * a.max_pages;
  const long long tok_stride = (long long)a.Hkv * D;

  auto issue_tile = [&](int tile, int buf) {
    const int k0 = k_begin + tile * kTile;
    for (int c = tid; c < kTile * kChunks; c += kThreads) {
      const int r = c / kChunks, ch = c - r * kChunks;
      const int key = k0 + r;
      if (key < k_end) {
        const int page = pt[key / a.page_size];
        const long long off =
            ((long long)page * a.page_size + (key % a.page_size)) * tok_stride + (long long)hk * D +
            ch * 8;
        cp_async16(&Ks[buf][r][ch * 8], a.kc + off);
        cp_async16(&Vs[buf][r][ch * 8], a.vc + off);
      } else {
        *reinterpret_cast<uint4*>(&Ks[buf][r][ch * 8]) = make_uint4(0, 0, 0, 0);
        *reinterpret_cast<uint4*>(&Vs[buf][r][ch * 8]) = make_uint4(0, 0, 0, 0);
      }
    }
    cp_async_commit();
  };

  if (ntiles > 0) issue_tile(0, 0);
  for (int tile = 0; tile < ntiles; ++tile) {
    const int buf = tile & 1;
    if (tile + 1 < ntiles) {
      issue_tile(tile + 1, buf ^ 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();

    // Scores: lane = key of the tile, warps stride over the heads.
    const int key = k_begin + tile * kTile + lane;
    for (int g = warp; g < G; g += kThreads / 32) {
      float s = 0.f;
#pragma unroll
      for (int ch = 0; ch < kChunks; ++ch) {
        us::Pack16 p;
        p.u = *reinterpret_cast<const uint4*>(&Ks[buf][lane][ch * 8]);
        const float4 q0 = *reinterpret_cast<const float4*>(&Qs[g][ch * 8]);
        const float4 q1 = *reinterpret_cast<const float4*>(&Qs[g][ch * 8 + 4]);
        s += us::bf2f(p.b[0]) * q0.x + us::bf2f(p.b[1]) * q0.y + us::bf2f(p.b[2]) * q0.z +
             us::bf2f(p.b[3]) * q0.w + us::bf2f(p.b[4]) * q1.x + us::bf2f(p.b[5]) * q1.y +
             us::bf2f(p.b[6]) * q1.z + us::bf2f(p.b[7]) * q1.w;
      }
      if (key >= k_end) s = -INFINITY;
      const float m_old = Mmax[g];
      const float m_new = fmaxf(m_old, us::warp_max(s));
      const float p = (key < k_end) ? __expf(s - m_new) : 0.f;
      const float psum = us::warp_sum(p);
      Ps[g][lane] = p;
      if (lane == 0) {
        const float sc = (m_old == -INFINITY) ? 0.f : __expf(m_old - m_new);
        Scale[g] = sc;
        Lsum[g] = Lsum[g] * sc + psum;
        Mmax[g] = m_new;
      }
    }
    __syncthreads();

    // Output: thread = (bf16x2 column, head group).
    const int pair = tid % kPairs, grp = tid / kPairs;
#pragma unroll
    for (int i = 0; i < kHpt; ++i) {
      const int g = grp + i * kGroups;
      if (g < G) {
        const float sc = Scale[g];
        float o0 = acc[i][0] * sc, o1 = acc[i][1] * sc;
#pragma unroll 8
        for (int r = 0; r < kTile; ++r) {
          const __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(&Vs[buf][r][pair * 2]);
          const float p = Ps[g][r];
          o0 += p * __low2float(v);
          o1 += p * __high2float(v);
        }
        acc[i][0] = o0;
        acc[i][1] = o1;
      }
    }
    __syncthreads();
  }

  const int pair = tid % kPairs, grp = tid / kPairs;
#pragma unroll
  for (int i = 0; i < kHpt; ++i) {
    const int g = grp + i * kGroups;
    if (g < G) {
      const float l = Lsum[g];
      const float inv = l > 0.f ? 1.f / l : 0.f;
      const int h = hk * G + g;
      if (a.splits == 1) {
        __nv_bfloat162 o = __floats2bfloat162_rn(acc[i][0] * inv, acc[i][1] * inv);
        *reinterpret_cast<__nv_bfloat162*>(a.out + (long long)b * a.ldo + (long long)h * D +
                                           pair * 2) = o;
      } else {
        const long long base = (((long long)b * a.Hq + h) * a.splits + split);
        a.part_o[base * D + pair * 2] = acc[i][0] * inv;
        a.part_o[base * D + pair * 2 + 1] = acc[i][1] * inv;
        if (pair == 0) a.part_lse[base] = l > 0.f ? Mmax[g] + __logf(l) : -INFINITY;
      }
    }
  }
}

template <int D>
__global__ void __launch_bounds__(D) merge_splits_kernel(const float* __restrict__ part_o,
                                                         const float* __restrict__ part_lse,
                                                         __nv_bfloat16* __restrict__ out,
                                                         long long ldo, int Hq, int splits) {
  US_PDL_PROLOGUE();
  const int b = blockIdx.x, h = blockIdx.y, d = threadIdx.x;
  const long long base = ((long long)b * Hq + h) * splits;
  float m = -INFINITY;
  for (int s = 0; s < splits; ++s) m = fmaxf(m, part_lse[base + s]);
  float num = 0.f, den = 0.f;
  if (m > -INFINITY) {
    for (int s = 0; s < splits; ++s) {
      const float w = __expf(part_lse[base + s] - m);
      num += w * part_o[(base + s) * D + d];
      den += w;
    }
  }
  out[(long long)b * ldo + (long long)h * D + d] = us::f2bf(den > 0.f ? num / den : 0.f);
}

template <int D, int G>
int launch_decode(const DecodeArgs& a, cudaStream_t stream) {
  dim3 grid(a.B, a.Hkv, a.splits);
  us::launch_pdl(paged_decode_kernel<D, G>, dim3(grid), dim3(kThreads), 0, stream, a);
  US_LAUNCH_CHECK();
  if (a.splits > 1) {
    dim3 g2(a.B, a.Hq);
    us::launch_pdl(merge_splits_kernel<D>, dim3(g2), dim3(D), 0, stream, a.part_o, a.part_lse, a.out, a.ldo, a.Hq,
                                                 a.splits);
    US_LAUNCH_CHECK();
  }
  return US_OK;
}

}  // namespace

extern "C" int us_merge_decode_splits(const float* part_o, const float* part_lse, void* out,
                                      long long ldo, int B, int Hq, int D, int splits,
                                      void* stream) {
  dim3 g2(B, Hq);
  if (D == 128)
    us::launch_pdl(merge_splits_kernel<128>, dim3(g2), dim3(128), 0, (cudaStream_t)stream, part_o, part_lse, (__nv_bfloat16*)out, ldo, Hq, splits);
  else if (D == 64)
    us::launch_pdl(merge_splits_kernel<64>, dim3(g2), dim3(64), 0, (cudaStream_t)stream, part_o, part_lse, (__nv_bfloat16*)out, ldo, Hq, splits);
  else
    return US_ERR_UNSUPPORTED;
  US_LAUNCH_CHECK();
  return US_OK;
}

// Bytes of scratch the split path needs: partial outputs then log-sum-exps.
US_API long long us_paged_decode_scratch_bytes(int B, int Hq, int D, int splits) {
  return (long long)B * Hq * splits * (D + 1) * (long long)sizeof(float);
}

US_API int us_paged_decode_attention(const void* q, const void* kcache, const void* vcache,
                                     const int* page_table, const int* seq_lens, void* out,
                                     void* scratch, int B, int Hq, int Hkv, int D, int max_pages,
                                     int page_size, int splits, int window, float scale,
                                     long long ldq, long long ldo, void* stream_) {
  US_REQUIRE(q && kcache && vcache && page_table && seq_lens && out);
  US_REQUIRE(B >= 0 && Hkv >= 1 && Hq % Hkv == 0 && splits >= 1 && page_size >= 1);
  US_REQUIRE(splits == 1 || scratch != nullptr);
  if (B == 0) return US_OK;
  DecodeArgs a;
  a.q = (const __nv_bfloat16*)q;
  a.kc = (const __nv_bfloat16*)kcache;
  a.vc = (const __nv_bfloat16*)vcache;
  a.page_table = page_table;
  a.seq_lens = seq_lens;
  a.out = (__nv_bfloat16*)out;
  a.part_o = (float*)scratch;
  a.part_lse = scratch ? (float*)scratch + (long long)B * Hq * splits * D : nullptr;
  a.ldq = ldq; a.ldo = ldo;
  a.B = B; a.Hq = Hq; a.Hkv = Hkv; a.max_pages = max_pages; a.page_size = page_size;
  a.splits = splits; a.window = window; a.scale = scale;
  cudaStream_t stream = (cudaStream_t)stream_;
  const int G = Hq / Hkv;
#define US_DEC(DD, GG) \
  if (D == DD && G == GG) return launch_decode<DD, GG>(a, stream);
  US_DEC(128, 1) US_DEC(128, 2) US_DEC(128, 4) US_DEC(128, 8) US_DEC(128, 16)
  US_DEC(64, 1) US_DEC(64, 2) US_DEC(64, 4) US_DEC(64, 8)
#undef US_DEC
  return US_ERR_UNSUPPORTED;
}

// ---------------------------------------------------------------------------
// Allocation-free variant (see include/us_noalloc.h).  The partial outputs and
// log-sum-exps of the split path live in this array, which is part of the
// library image on every device that loads it.
static __device__ __align__(256) unsigned char g_noalloc_scratch[US_NOALLOC_SCRATCH_BYTES];

namespace {
constexpr int kNoallocMaxDevices = 64;
void* g_noalloc_ptr[kNoallocMaxDevices] = {nullptr};
}  // namespace

extern "C" void us_set_last_error_text(const char* text);

US_API int us_paged_decode_attention_noalloc(const void* q, const void* kcache,
                                             const void* vcache, const int* page_table,
                                             const int* seq_lens, void* out, int B, int Hq,
                                             int Hkv, int D, int max_pages, int page_size,
                                             int splits, int window, float scale, long long ldq,
                                             long long ldo, void* stream_) {
  US_REQUIRE(B >= 0 && Hq >= 1 && D >= 1 && splits >= 1);
  const long long need = splits > 1 ? us_paged_decode_scratch_bytes(B, Hq, D, splits) : 0;
  if (need > (long long)US_NOALLOC_SCRATCH_BYTES) {
    char msg[256];
    snprintf(msg, sizeof(msg),
             "us_paged_decode_attention_noalloc: B*Hq*splits*(D+1)*4 = %lld bytes exceeds the "
             "built-in scratch of %u bytes; lower `splits` or the batch",
             need, (unsigned)US_NOALLOC_SCRATCH_BYTES);
    us_set_last_error_text(msg);
    return US_ERR_LIMIT;
  }
  // In host code the array's name is only a stand-in; the kernel needs the
  // address the array has on the current device.  Looked up once per device.
  int dev = 0;
  US_CUDA_CHECK(cudaGetDevice(&dev));
  US_REQUIRE(dev >= 0 && dev < kNoallocMaxDevices);
  if (g_noalloc_ptr[dev] == nullptr) {
    void* p = nullptr;
    US_CUDA_CHECK(cudaGetSymbolAddress(&p, g_noalloc_scratch));
    g_noalloc_ptr[dev] = p;
  }
  return us_paged_decode_attention(q, kcache, vcache, page_table, seq_lens, out,
                                   splits > 1 ? g_noalloc_ptr[dev] : nullptr, B, Hq, Hkv, D,
                                   max_pages, page_size, splits, window, scale, ldq, ldo, stream_);
}
