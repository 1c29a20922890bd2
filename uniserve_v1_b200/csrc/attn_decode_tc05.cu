// Paged-KV decode attention on tcgen05 with the keys on the MMA M axis.
//
// A decode step has one query token per sequence, so a conventional attention
// tile (queries on M) would be almost empty.  Here a tile is 128 keys:
//
//   S^T[key, head] = K_tile[128 keys x 128 d] . Q^T          (M=128, N=16, K=128)
//   O^T[d,   head] = V_tile^T[128 d x 128 keys] . P[key, head] (M=128, N=16, K=128)
//
// K pages are TMA-loaded as the K-major A operand; the same V pages serve as an
// MN-major A operand (d contiguous), so neither is transposed.  The G query
// heads that share a kv head are the N columns (zero padded to 16).  Thread t
// of the four softmax warps owns TMEM lane t: key t of the tile when it reads
// S^T, channel d = t when it reads O^T; the running output lives in 16
// registers per thread and is rescaled there, tensor memory holds only the
// current tile's products.
//
// Grid = (sequence, kv head, split); with more than one split the CTAs write
// normalised partial outputs and log-sum-exps.  With an arrival counter per
// (sequence, kv head) the CTA that finishes last merges the splits itself (no
// second launch); without one the merge kernel of attn_decode.cu combines them.
// The first tile's K and V loads are issued before the CTA's set-up (query
// operand, tensor-memory allocation) so that set-up overlaps the first fetch.
//
// Roles: warps 0-3 softmax / output, warp 4 TMA producer, warp 5 TMEM owner +
// MMA issuer.  Every wait is bounded.
//
// FP8 pages (template FP8): a page plane holds E4M3 bytes and one FP32 scale per page.  The
// TMA producer fetches the raw 16 KiB tiles; four more warps (6-9, one key row per thread)
// expand them to FP16 into the operand buffers in the layout the bf16 fetch would have
// produced, so the multiplications are the same instructions with FP16 operand formats
// (Q and P are written as FP16 too).  The page scales never touch the tiles: the key
// scale multiplies the key's score, the value scale its probability, in the softmax
// threads.  HBM traffic per key halves; the expansion runs while the next tiles land.
#include <cuda_fp8.h>
#include "include/us_common.cuh"
#include "include/us_tc05.cuh"
#include "include/us_tmap.h"

namespace {

constexpr int kD = 128;
constexpr int kTileKeys = 128;
constexpr int kNPad = 16;                    // padded head count (UMMA N)
constexpr int kHalfBytes = kTileKeys * 128;  // one 64-column half of a K or V tile
constexpr int kTileBytes = 2 * kHalfBytes;   // 32 KiB
constexpr int kSmallHalf = kNPad * 128;      // one half of the Q or P operand (2 KiB)

struct DecTcArgs {
  const __nv_bfloat16* q;
  const int* page_table;
  const int* seq_lens;
  __nv_bfloat16* out;
  float* part_o;
  float* part_lse;
  int* counters;          // [B * Hkv] zero between launches, or NULL (separate merge kernel)
  long long ldq, ldo;
  int B, Hq, Hkv, max_pages, page_size, splits, window;
  float scale_log2;
  unsigned int* status;
  const float* k_scale;   // FP8 pages: one scale per page and plane
  const float* v_scale;
};

constexpr int kRawBytes = kTileKeys * 128;   // one E4M3 tile: 128 keys x 128 bytes

// Thread `row` expands its key row of an E4M3 tile (128-byte rows, 128-byte swizzle) into the
// two 64-column FP16 halves of an operand buffer.
__device__ __forceinline__ void expand_row(const uint8_t* raw, uint8_t* buf, int row) {
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    const uint4 in = *reinterpret_cast<const uint4*>(raw + tc::sw128_offset(row, c));
    const uint32_t w[4] = {in.x, in.y, in.z, in.w};
    uint32_t o[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const __half2_raw lo = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(w[j] & 0xffffu), __NV_E4M3);
      const __half2_raw hi = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(w[j] >> 16), __NV_E4M3);
      o[2 * j] = (uint32_t)lo.x | ((uint32_t)lo.y << 16);
      o[2 * j + 1] = (uint32_t)hi.x | ((uint32_t)hi.y << 16);
    }
    uint8_t* half = buf + (c >> 2) * kHalfBytes;
    *reinterpret_cast<uint4*>(half + tc::sw128_offset(row, (2 * c) & 7)) =
        make_uint4(o[0], o[1], o[2], o[3]);
    *reinterpret_cast<uint4*>(half + tc::sw128_offset(row, (2 * c + 1) & 7)) =
        make_uint4(o[4], o[5], o[6], o[7]);
  }
}

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}


// Arrival counter of (sequence, kv head): the CTA that adds the last of `splits` arrivals
// merges the partial outputs of the G heads (threads 0..127 own one channel each) and puts
// the counter back to zero for the next launch.  Called by every thread of the CTA.
template <int G>
__device__ __forceinline__ void merge_if_last(const DecTcArgs& a, int b, int hk) {
  __shared__ int last_s;
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    int* c = a.counters + (long long)b * a.Hkv + hk;
    const int old = atomicAdd(c, 1);
    last_s = old == a.splits - 1;
    if (last_s) *c = 0;
  }
  __syncthreads();
  if (!last_s) return;
  __threadfence();
  // log-sum-exps of the G heads x splits first (one load per thread), then every channel
  // thread merges its G heads with independent loads
  __shared__ float lse_s[kNPad * 32];
  const int tid = threadIdx.x;
  const long long base0 = ((long long)b * a.Hq + (long long)hk * G) * a.splits;
  const int n_lse = G * a.splits;
  for (int i = tid; i < n_lse && i < kNPad * 32; i += blockDim.x)
    lse_s[i] = __ldcg(a.part_lse + base0 + i);
  __syncthreads();
  if (tid >= kD) return;
  float m[G], acc[G], den[G];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    m[g] = -INFINITY;
    acc[g] = 0.f;
    den[g] = 0.f;
    for (int s = 0; s < a.splits; ++s) m[g] = fmaxf(m[g], lse_s[g * a.splits + s]);
  }
  for (int s = 0; s < a.splits; ++s) {
    float v[G];
#pragma unroll
    for (int g = 0; g < G; ++g) v[g] = __ldcg(a.part_o + (base0 + g * a.splits + s) * kD + tid);
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const float l = lse_s[g * a.splits + s];
      const float wgt = (l == -INFINITY) ? 0.f : __expf(l - m[g]);
      den[g] += wgt;
      acc[g] += wgt * v[g];
    }
  }
#pragma unroll
  for (int g = 0; g < G; ++g)
    a.out[(long long)b * a.ldo + (long long)(hk * G + g) * kD + tid] =
        us::f2bf(den[g] > 0.f ? acc[g] / den[g] : 0.f);
}

template <int G, bool FP8>
__global__ void __launch_bounds__(FP8 ? 320 : 192)
paged_decode_tc_kernel(const __grid_constant__ CUtensorMap tmK,
                       const __grid_constant__ CUtensorMap tmV, const DecTcArgs a) {
  US_PDL_PROLOGUE();
  const int b = blockIdx.x, hk = blockIdx.y, split = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, tid = threadIdx.x;

  const int seq_len = a.seq_lens[b];
  int begin_all = 0;
  if (a.window > 0 && seq_len > a.window) begin_all = seq_len - a.window;
  begin_all &= ~(a.page_size - 1);  // tiles start on a page; the head is masked
  const int first_key = (a.window > 0 && seq_len > a.window) ? seq_len - a.window : 0;
  const int span = seq_len - begin_all;
  const int tiles_all = (span + kTileKeys - 1) / kTileKeys;
  const int tiles_per = (tiles_all + a.splits - 1) / a.splits;
  const int k_begin = begin_all + split * tiles_per * kTileKeys;
  const int k_end = min(seq_len, k_begin + tiles_per * kTileKeys);
  const int ntiles = k_end > k_begin ? (k_end - k_begin + kTileKeys - 1) / kTileKeys : 0;

  if (ntiles == 0) {  // nothing to attend in this split (uniform for the CTA)
    if (tid < kD) {
      for (int g = 0; g < G; ++g) {
        const int h = hk * G + g;
        if (a.splits == 1) {
          a.out[(long long)b * a.ldo + (long long)h * kD + tid] = us::f2bf(0.f);
        } else {
          const long long base = ((long long)b * a.Hq + h) * a.splits + split;
          a.part_o[base * kD + tid] = 0.f;
          if (tid == 0) a.part_lse[base] = -INFINITY;
        }
      }
    }
    if (a.splits > 1 && a.counters) merge_if_last<G>(a, b, hk);
    return;
  }

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* sK = smem;
  uint8_t* sV = smem + kTileBytes;
  uint8_t* sRawK = smem + 2 * kTileBytes;              // FP8 only
  uint8_t* sRawV = sRawK + kRawBytes;
  uint8_t* sQ = smem + 2 * kTileBytes + (FP8 ? 2 * kRawBytes : 0);
  uint8_t* sP = sQ + 2 * kSmallHalf;
  float* red = (float*)(sP + 2 * kSmallHalf);       // [2][4 warps][16] reduction scratch
  uint64_t* bars = (uint64_t*)(red + 2 * 4 * kNPad);
  uint64_t* k_full = bars + 0;
  uint64_t* k_empty = bars + 1;
  uint64_t* v_full = bars + 2;
  uint64_t* v_empty = bars + 3;
  uint64_t* s_full = bars + 4;
  uint64_t* p_full = bars + 5;
  uint64_t* o_full = bars + 6;
  uint64_t* rawk_full = bars + 7;    // FP8: the raw tile has landed / has been expanded
  uint64_t* rawk_empty = bars + 8;
  uint64_t* rawv_full = bars + 9;
  uint64_t* rawv_empty = bars + 10;
  uint32_t* tmem_slot = (uint32_t*)(bars + 11);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  if (tid == 0) {
    tc::mbar_init(k_full, FP8 ? 128 : 1);     // FP8: the expanding threads fill the operand
    tc::mbar_init(k_empty, 1);
    tc::mbar_init(v_full, FP8 ? 128 : 1);
    tc::mbar_init(v_empty, 1);
    tc::mbar_init(rawk_full, 1);
    tc::mbar_init(rawk_empty, 128);
    tc::mbar_init(rawv_full, 1);
    tc::mbar_init(rawv_empty, 128);
    tc::mbar_init(s_full, 1);
    tc::mbar_init(p_full, 128);
    tc::mbar_init(o_full, 1);
    *abort_flag = 0;
    tc::mbar_fence_init();
  }
  __syncthreads();
  const int* pt_row = a.page_table + (long long)b * a.max_pages;
  const int pages_per_tile = kTileKeys / a.page_size;
  const int seq_pages = (seq_len + a.page_size - 1) / a.page_size;
  // Page ids of a tile: independent loads issued together (one memory latency per tile, not
  // one per page), shared by the K and the V fetch.
  constexpr int kMaxPagesPerTile = kTileKeys / 8;
  auto load_pages = [&](int t, int (&pg)[kMaxPagesPerTile]) {
    const int page0 = (k_begin + t * kTileKeys) / a.page_size;
#pragma unroll
    for (int i = 0; i < kMaxPagesPerTile; ++i) {
      const int pi = page0 + i;
      pg[i] = (i < pages_per_tile && pi < seq_pages && pi < a.max_pages) ? __ldg(pt_row + pi) : 0;
    }
  };
  // One tile's K (or V) pages into their buffer; `bar` was armed by the caller.
  auto issue_tile = [&](const CUtensorMap* tm, uint8_t* buf, uint64_t* bar,
                        const int (&pg)[kMaxPagesPerTile]) {
#pragma unroll
    for (int i = 0; i < kMaxPagesPerTile; ++i) {
      if (i < pages_per_tile) {
        const int row = pg[i] * a.page_size;
        uint8_t* dst = buf + i * a.page_size * 128;
        tc::tma_load_2d(dst, tm, bar, hk * kD, row);
        if (!FP8) tc::tma_load_2d(dst + kHalfBytes, tm, bar, hk * kD + 64, row);
      }
    }
  };
  int pg_next[kMaxPagesPerTile];
  if (warp == 4 && lane == 0) {
    // the first tile needs nothing of the set-up below: fetch it now
    tc::tma_prefetch_desc(&tmK);
    tc::tma_prefetch_desc(&tmV);
    int pg[kMaxPagesPerTile];
    load_pages(0, pg);
    if (ntiles > 1) load_pages(1, pg_next);
    if (FP8) {
      tc::mbar_expect_tx(rawk_full, kRawBytes);
      issue_tile(&tmK, sRawK, rawk_full, pg);
      tc::mbar_expect_tx(rawv_full, kRawBytes);
      issue_tile(&tmV, sRawV, rawv_full, pg);
    } else {
      tc::mbar_expect_tx(k_full, kTileBytes);
      issue_tile(&tmK, sK, k_full, pg);
      tc::mbar_expect_tx(v_full, kTileBytes);
      issue_tile(&tmV, sV, v_full, pg);
    }
  }
  if (warp == 5) {
    tc::tmem_alloc(tmem_slot, 32);
    tc::tmem_relinquish();
  }
  // Q operand: rows = heads (zero padded to 16), K-major, 128-byte swizzle.
  if (tid < 128) {
    for (int c = tid; c < kNPad * 16; c += 128) {
      const int g = c >> 4, ch = c & 15;  // 16-byte chunk ch of head row g
      uint4 v = make_uint4(0, 0, 0, 0);
      if (g < G)
        v = *reinterpret_cast<const uint4*>(a.q + (long long)b * a.ldq +
                                            (long long)(hk * G + g) * kD + ch * 8);
      if (FP8) {                              // operands are FP16 in this form
        uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float lo = __uint_as_float(w[j] << 16), hi = __uint_as_float(w[j] & 0xffff0000u);
          w[j] = (uint32_t)__half_as_ushort(__float2half_rn(lo)) |
                 ((uint32_t)__half_as_ushort(__float2half_rn(hi)) << 16);
        }
        v = make_uint4(w[0], w[1], w[2], w[3]);
      }
      const int half = ch >> 3;
      *reinterpret_cast<uint4*>(sQ + half * kSmallHalf + tc::sw128_offset(g, ch & 7)) = v;
    }
    // Rows of P that no head owns stay zero.
    for (int c = tid; c < 2 * kSmallHalf / 16; c += 128)
      reinterpret_cast<uint4*>(sP)[c] = make_uint4(0, 0, 0, 0);
    tc::fence_async_smem();
  }
  tc::tc_fence_before_sync();
  __syncthreads();
  tc::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_S = tmem_base;
  const uint32_t tmem_O = tmem_base + kNPad;

  if (warp == 4) {
    if (lane == 0) {
      for (int t = 1; t < ntiles; ++t) {
        const uint32_t ph = (uint32_t)t & 1u;
        int pg[kMaxPagesPerTile];
#pragma unroll
        for (int i = 0; i < kMaxPagesPerTile; ++i) pg[i] = pg_next[i];
        if (t + 1 < ntiles) load_pages(t + 1, pg_next);     // in flight during the waits below
        if (!tc::mbar_wait(FP8 ? rawk_empty : k_empty, ph ^ 1u, abort_flag)) {
          us_dev_fail(a.status, US_DEV_TIMEOUT_EMPTY);
          *abort_flag = 1;
          break;
        }
        if (FP8) {
          tc::mbar_expect_tx(rawk_full, kRawBytes);
          issue_tile(&tmK, sRawK, rawk_full, pg);
        } else {
          tc::mbar_expect_tx(k_full, kTileBytes);
          issue_tile(&tmK, sK, k_full, pg);
        }
        if (!tc::mbar_wait(FP8 ? rawv_empty : v_empty, ph ^ 1u, abort_flag)) {
          us_dev_fail(a.status, US_DEV_TIMEOUT_EMPTY);
          *abort_flag = 1;
          break;
        }
        if (FP8) {
          tc::mbar_expect_tx(rawv_full, kRawBytes);
          issue_tile(&tmV, sRawV, rawv_full, pg);
        } else {
          tc::mbar_expect_tx(v_full, kTileBytes);
          issue_tile(&tmV, sV, v_full, pg);
        }
      }
    }
  } else if (warp == 5) {
    if (lane == 0) {
      constexpr uint32_t kFmt = FP8 ? tc::kFmtF16 : tc::kFmtBF16;
      constexpr uint32_t kIdescQK = tc::make_idesc(128, kNPad, kFmt, kFmt, 0, 0);
      constexpr uint32_t kIdescPV = tc::make_idesc(128, kNPad, kFmt, kFmt, 1, 0);
      const uint32_t k_addr = tc::smem_u32(sK), v_addr = tc::smem_u32(sV);
      const uint32_t q_addr = tc::smem_u32(sQ), p_addr = tc::smem_u32(sP);
      auto issue_qk = [&]() {
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t half = kk >> 2, sub = kk & 3;
          const uint64_t ad = tc::smem_desc_kmajor_sw128(k_addr + half * kHalfBytes) + 2 * sub;
          const uint64_t bd = tc::smem_desc_kmajor_sw128(q_addr + half * kSmallHalf) + 2 * sub;
          tc::umma_f16(tmem_S, ad, bd, kIdescQK, kk != 0);
        }
      };
      bool ok = tc::mbar_wait(k_full, 0, abort_flag);
      if (ok) {
        tc::tc_fence_after_sync();
        issue_qk();
        tc::umma_commit(s_full);
        tc::umma_commit(k_empty);
      }
      for (int t = 0; ok && t < ntiles; ++t) {
        const uint32_t ph = (uint32_t)t & 1u;
        // P(t) ready: S(t) has been consumed and O(t-1) has been read.
        if (!tc::mbar_wait(p_full, ph, abort_flag)) { ok = false; break; }
        if (t + 1 < ntiles) {
          if (!tc::mbar_wait(k_full, ph ^ 1u, abort_flag)) { ok = false; break; }
          tc::tc_fence_after_sync();
          issue_qk();
          tc::umma_commit(s_full);
          tc::umma_commit(k_empty);
        }
        if (!tc::mbar_wait(v_full, ph, abort_flag)) { ok = false; break; }
        tc::tc_fence_after_sync();
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          // A = V^T: d on M (two 64-wide chunks, 16 KiB apart), 16 keys = two
          // groups of eight rows (1 KiB apart) per instruction.
          const uint64_t ad =
              tc::smem_desc_mnmajor_sw128(v_addr + kk * 2048, kHalfBytes, 1024);
          const uint32_t half = kk >> 2, sub = kk & 3;
          const uint64_t bd = tc::smem_desc_kmajor_sw128(p_addr + half * kSmallHalf) + 2 * sub;
          tc::umma_f16(tmem_O, ad, bd, kIdescPV, kk != 0);
        }
        tc::umma_commit(o_full);
        tc::umma_commit(v_empty);
      }
      if (!ok) {
        us_dev_fail(a.status, US_DEV_TIMEOUT_FULL);
        *abort_flag = 1;
      }
    }
  } else if (FP8 && warp >= 6) {
    // ---- expanding threads: key row = tid - 192 of every tile ----
    const int row = tid - 192;
    bool ok = true;
    for (int t = 0; ok && t < ntiles; ++t) {
      const uint32_t ph = (uint32_t)t & 1u;
      if (!tc::mbar_wait(rawk_full, ph, abort_flag)) { ok = false; break; }
      if (t > 0 && !tc::mbar_wait(k_empty, ph ^ 1u, abort_flag)) { ok = false; break; }
      expand_row(sRawK, sK, row);
      tc::fence_async_smem();
      tc::mbar_arrive(k_full);
      tc::mbar_arrive(rawk_empty);
      if (!tc::mbar_wait(rawv_full, ph, abort_flag)) { ok = false; break; }
      if (t > 0 && !tc::mbar_wait(v_empty, ph ^ 1u, abort_flag)) { ok = false; break; }
      expand_row(sRawV, sV, row);
      tc::fence_async_smem();
      tc::mbar_arrive(v_full);
      tc::mbar_arrive(rawv_empty);
    }
    if (!ok) {
      us_dev_fail(a.status, US_DEV_TIMEOUT_FULL);
      *abort_flag = 1;
    }
  } else {
    // ---- softmax / output threads: TMEM lane = tid ----
    const uint32_t lane_addr = ((uint32_t)(warp * 32) << 16);
    float m_run[G], l_part[G], o_acc[G], alpha_prev[G];
#pragma unroll
    for (int g = 0; g < G; ++g) {
      m_run[g] = -INFINITY;
      l_part[g] = 0.f;
      o_acc[g] = 0.f;
      alpha_prev[g] = 0.f;
    }
    bool ok = true;
    for (int t = 0; t < ntiles; ++t) {
      const uint32_t ph = (uint32_t)t & 1u;
      float ksc = 1.f, vsc = 1.f;           // FP8: scales of this thread's key's page
      if (FP8) {
        const int key = k_begin + t * kTileKeys + tid;
        const int pi = key / a.page_size;
        if (key < k_end && pi < a.max_pages) {
          const int pg = __ldg(pt_row + pi);
          ksc = __ldg(a.k_scale + pg);
          vsc = __ldg(a.v_scale + pg);
        }
      }
      if (!tc::mbar_wait(s_full, ph)) { ok = false; break; }
      tc::tc_fence_after_sync();
      uint32_t sr[16];
      tc::tmem_ld16(tmem_S + lane_addr, sr);
      tc::tmem_ld_wait();
      const int key = k_begin + t * kTileKeys + tid;
      const bool valid = key < k_end && key >= first_key;
      float s[G];
      float* rbuf = red + (t & 1) * 4 * kNPad;
#pragma unroll
      for (int g = 0; g < G; ++g) {
        s[g] = valid ? __uint_as_float(sr[g]) * (a.scale_log2 * ksc) : -INFINITY;
        const float wm = us::warp_max(s[g]);
        if (lane == 0) rbuf[warp * kNPad + g] = wm;
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      float alpha[G], p[G];
#pragma unroll
      for (int g = 0; g < G; ++g) {
        const float tm = fmaxf(fmaxf(rbuf[g], rbuf[kNPad + g]),
                               fmaxf(rbuf[2 * kNPad + g], rbuf[3 * kNPad + g]));
        const float m_new = fmaxf(m_run[g], tm);
        alpha[g] = (m_run[g] == -INFINITY) ? 0.f : ex2(m_run[g] - m_new);
        p[g] = valid ? ex2(s[g] - m_new) : 0.f;
        l_part[g] = l_part[g] * alpha[g] + p[g];
        m_run[g] = m_new;
      }
      if (t > 0) {
        // O(t-1) is complete: fold it in (it was produced under the previous
        // maximum, so the previous tile's factor applies to the running sum).
        if (!tc::mbar_wait(o_full, ph ^ 1u)) { ok = false; break; }
        tc::tc_fence_after_sync();
        uint32_t orr[16];
        tc::tmem_ld16(tmem_O + lane_addr, orr);
        tc::tmem_ld_wait();
#pragma unroll
        for (int g = 0; g < G; ++g)
          o_acc[g] = o_acc[g] * alpha_prev[g] + __uint_as_float(orr[g]);
      }
#pragma unroll
      for (int g = 0; g < G; ++g) alpha_prev[g] = alpha[g];
      // P^T -> smem as the K-major B operand: row = head, column = key of the tile.
      {
        const int half = tid >> 6, col = tid & 63;
#pragma unroll
        for (int g = 0; g < G; ++g) {
          uint8_t* dst = sP + half * kSmallHalf + tc::sw128_offset(g, col >> 3) + (col & 7) * 2;
          if (FP8) *reinterpret_cast<__half*>(dst) = __float2half_rn(p[g] * vsc);
          else *reinterpret_cast<__nv_bfloat16*>(dst) = us::f2bf(p[g]);
        }
      }
      tc::fence_async_smem();
      tc::tc_fence_before_sync();
      tc::mbar_arrive(p_full);
    }
    if (ok) {
      const uint32_t ph = (uint32_t)(ntiles - 1) & 1u;
      if (tc::mbar_wait(o_full, ph)) {
        tc::tc_fence_after_sync();
        uint32_t orr[16];
        tc::tmem_ld16(tmem_O + lane_addr, orr);
        tc::tmem_ld_wait();
#pragma unroll
        for (int g = 0; g < G; ++g)
          o_acc[g] = o_acc[g] * alpha_prev[g] + __uint_as_float(orr[g]);
        // Row sums: every thread holds the share of its keys.
        float* rbuf = red;
        asm volatile("bar.sync 1, 128;" ::: "memory");
#pragma unroll
        for (int g = 0; g < G; ++g) {
          const float ws = us::warp_sum(l_part[g]);
          if (lane == 0) rbuf[warp * kNPad + g] = ws;
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
#pragma unroll
        for (int g = 0; g < G; ++g) {
          const float l = rbuf[g] + rbuf[kNPad + g] + rbuf[2 * kNPad + g] + rbuf[3 * kNPad + g];
          const float inv = l > 0.f ? 1.f / l : 0.f;
          const int h = hk * G + g;
          if (a.splits == 1) {
            a.out[(long long)b * a.ldo + (long long)h * kD + tid] = us::f2bf(o_acc[g] * inv);
          } else {
            const long long base = ((long long)b * a.Hq + h) * a.splits + split;
            a.part_o[base * kD + tid] = o_acc[g] * inv;
            // m_run is in the log2 domain; the merge kernel works in natural logs.
            if (tid == 0)
              a.part_lse[base] = l > 0.f ? (m_run[g] + log2f(l)) * 0.6931471805599453f : -INFINITY;
          }
        }
      } else {
        ok = false;
      }
    }
    if (!ok) us_dev_fail(a.status, US_DEV_TIMEOUT_ACC);
  }
  tc::tc_fence_before_sync();
  __syncthreads();
  if (warp == 5) {
    __syncwarp();
    tc::tmem_dealloc(tmem_base, 32);
  }
  if (a.splits > 1 && a.counters) merge_if_last<G>(a, b, hk);
}

template <int G, bool FP8>
int launch_tc(const CUtensorMap& tmK, const CUtensorMap& tmV, const DecTcArgs& a,
              cudaStream_t stream) {
  const size_t smem = 2 * kTileBytes + (FP8 ? 2 * kRawBytes : 0) + 4 * kSmallHalf +
                      2 * 4 * kNPad * 4 + 12 * 8 + 16 + 1024;
  static bool configured = false;
  if (!configured) {
    US_CUDA_CHECK(cudaFuncSetAttribute(paged_decode_tc_kernel<G, FP8>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured = true;
  }
  dim3 grid(a.B, a.Hkv, a.splits);
  us::launch_pdl(paged_decode_tc_kernel<G, FP8>, dim3(grid), dim3(FP8 ? 320 : 192), smem, stream,
                 tmK, tmV, a);
  US_LAUNCH_CHECK();
  return US_OK;
}

}  // namespace

extern "C" int us_merge_decode_splits(const float* part_o, const float* part_lse, void* out,
                                      long long ldo, int B, int Hq, int D, int splits,
                                      void* stream);

static int decode_tc(const void* q, const void* kcache, const void* vcache,
                     const float* k_scale, const float* v_scale, const int* page_table, const int* seq_lens, void* out, void* scratch,
                     int* counters, int B, int Hq, int Hkv, int D, int num_pages, int max_pages,
                     int page_size, int splits, int window, float scale, long long ldq,
                     long long ldo, void* stream_) {
  US_REQUIRE(q && kcache && vcache && page_table && seq_lens && out);
  US_REQUIRE(D == kD && Hkv >= 1 && Hq % Hkv == 0 && Hq / Hkv <= kNPad && splits >= 1);
  US_REQUIRE(page_size >= 8 && page_size <= 128 && (kTileKeys % page_size) == 0);
  US_REQUIRE(splits == 1 || scratch != nullptr);
  US_REQUIRE((ldq % 8) == 0 && ((uintptr_t)q % 16) == 0);
  if (B == 0) return US_OK;
  cudaStream_t stream = (cudaStream_t)stream_;
  CUtensorMap tmK, tmV;
  const uint64_t rows = (uint64_t)num_pages * page_size, cols = (uint64_t)Hkv * D;
  const bool fp8 = k_scale != nullptr;
  US_REQUIRE(!fp8 || v_scale != nullptr);
  // bf16 pages are fetched as two 64-column halves per page, E4M3 pages as one 128-byte box
  int rc = us_tmap_2d(&tmK, kcache, fp8 ? US_TMAP_U8 : US_TMAP_BF16, rows, cols, cols, page_size,
                      fp8 ? 128 : 64, US_SWZ_128);
  if (rc) return rc;
  rc = us_tmap_2d(&tmV, vcache, fp8 ? US_TMAP_U8 : US_TMAP_BF16, rows, cols, cols, page_size,
                  fp8 ? 128 : 64, US_SWZ_128);
  if (rc) return rc;
  DecTcArgs a;
  a.q = (const __nv_bfloat16*)q;
  a.page_table = page_table;
  a.seq_lens = seq_lens;
  a.out = (__nv_bfloat16*)out;
  a.part_o = (float*)scratch;
  a.part_lse = scratch ? (float*)scratch + (long long)B * Hq * splits * D : nullptr;
  a.counters = splits > 1 ? counters : nullptr;
  a.ldq = ldq; a.ldo = ldo;
  a.B = B; a.Hq = Hq; a.Hkv = Hkv; a.max_pages = max_pages; a.page_size = page_size;
  a.splits = splits; a.window = window;
  a.scale_log2 = scale * 1.4426950408889634f;
  a.status = us_status_ptr();
  a.k_scale = k_scale;
  a.v_scale = v_scale;
  const int G = Hq / Hkv;
  if (fp8) {
    switch (G) {
      case 1: rc = launch_tc<1, true>(tmK, tmV, a, stream); break;
      case 2: rc = launch_tc<2, true>(tmK, tmV, a, stream); break;
      case 4: rc = launch_tc<4, true>(tmK, tmV, a, stream); break;
      case 8: rc = launch_tc<8, true>(tmK, tmV, a, stream); break;
      case 16: rc = launch_tc<16, true>(tmK, tmV, a, stream); break;
      default: return US_ERR_UNSUPPORTED;
    }
  } else {
    switch (G) {
      case 1: rc = launch_tc<1, false>(tmK, tmV, a, stream); break;
      case 2: rc = launch_tc<2, false>(tmK, tmV, a, stream); break;
      case 4: rc = launch_tc<4, false>(tmK, tmV, a, stream); break;
      case 8: rc = launch_tc<8, false>(tmK, tmV, a, stream); break;
      case 16: rc = launch_tc<16, false>(tmK, tmV, a, stream); break;
      default: return US_ERR_UNSUPPORTED;
    }
  }
  if (rc) return rc;
  if (splits > 1 && !counters)
    return us_merge_decode_splits(a.part_o, a.part_lse, out, ldo, B, Hq, D, splits, stream_);
  return US_OK;
}

// Same contract as us_paged_decode_attention (head_dim 128, page_size dividing 128); the
// splits are merged by a second launch.
US_API int us_paged_decode_attention_tc(const void* q, const void* kcache, const void* vcache,
                                        const int* page_table, const int* seq_lens, void* out,
                                        void* scratch, int B, int Hq, int Hkv, int D,
                                        int num_pages, int max_pages, int page_size, int splits,
                                        int window, float scale, long long ldq, long long ldo,
                                        void* stream_) {
  return decode_tc(q, kcache, vcache, nullptr, nullptr, page_table, seq_lens, out, scratch, nullptr,
                   B, Hq, Hkv, D, num_pages, max_pages, page_size, splits, window, scale, ldq, ldo,
                   stream_);
}

// One launch: `counters` [B * Hkv] int32 must be zero before the first call and is left zero
// by every call (the last CTA of a (sequence, kv head) merges its splits and resets it).
// Calls that share `scratch` / `counters` must be ordered on the device.
US_API int us_paged_decode_attention_tc_merged(const void* q, const void* kcache,
                                               const void* vcache, const int* page_table,
                                               const int* seq_lens, void* out, void* scratch,
                                               int* counters, int B, int Hq, int Hkv, int D,
                                               int num_pages, int max_pages, int page_size,
                                               int splits, int window, float scale,
                                               long long ldq, long long ldo, void* stream_) {
  US_REQUIRE((splits == 1 || counters != nullptr) && splits <= 32);
  return decode_tc(q, kcache, vcache, nullptr, nullptr, page_table, seq_lens, out, scratch,
                   counters, B, Hq, Hkv, D, num_pages, max_pages, page_size, splits, window, scale,
                   ldq, ldo, stream_);
}

// E4M3 pages with one FP32 scale per page and plane (k_scale, v_scale [num_pages]); the
// other arguments as above.  `counters` may be null (the splits are then merged by a second
// launch).
US_API int us_paged_decode_attention_fp8(const void* q, const void* kcache, const void* vcache,
                                         const float* k_scale, const float* v_scale,
                                         const int* page_table, const int* seq_lens, void* out,
                                         void* scratch, int* counters, int B, int Hq, int Hkv,
                                         int D, int num_pages, int max_pages, int page_size,
                                         int splits, int window, float scale, long long ldq,
                                         long long ldo, void* stream_) {
  US_REQUIRE(k_scale && v_scale && splits <= 32);
  return decode_tc(q, kcache, vcache, k_scale, v_scale, page_table, seq_lens, out, scratch,
                   counters, B, Hq, Hkv, D, num_pages, max_pages, page_size, splits, window, scale,
                   ldq, ldo, stream_);
}
