// Persistent paged-KV decode attention (bf16 pages, head_dim 128): one CTA per SM walks a
// contiguous range of the launch's key tiles.
//
// The per-(sequence, kv head) kernel of attn_decode_tc05.cu is bound by latency, not by
// bandwidth: a CTA holds one K and one V tile, so the next tile's fetch starts only when the
// current product has read its operand, every CTA pays its own set-up (tensor-memory
// allocation, barriers, Q operand), and 64 sequences x 4 kv heads are 256 CTAs of eight
// tiles each on 148 SMs.  Here all tiles of the launch form one list, ordered by (sequence,
// kv head, tile); CTA c of n takes tiles [c T / n, (c + 1) T / n).  Its TMA producer runs
// through that range with a three-stage ring of (K, V) tile pairs and never drains between
// (sequence, kv head) pairs; the set-up happens once per SM.  The math of a tile is that of
// the other kernel (keys on the MMA M axis, the heads of a kv head as N = 16 columns, the
// running output in registers).  S, P and the per-tile product O are double-buffered: the
// product S(i + 1) is issued before the softmax of tile i has finished, and the softmax of
// tile i + 1 does not wait for O(i) - a tile's product is folded into the running output two
// tiles later, with the rescaling factor that was current when its P was made.  The issuing
// thread keeps its descriptors as words that advance by additions (64-bit descriptor
// arithmetic per product made the issue, not the tensor pipe, the limit of a tile).
//
// A range may start or end inside a pair.  Such a segment leaves a normalised partial
// output and its log-sum-exp in the CTA's slot (0: the CTA's first segment, 1: a later
// one, which then is its last) and adds one arrival to the pair's counter; the CTA that
// brings the count to the number of CTAs the pair spans merges the slots (their indices
// follow from the partition) and puts the counter back to zero; a CTA looks at the counts
// its arrivals returned, and merges, after its last tile.  Pairs inside one range
// are written directly.  The Q operand of the next segment is staged while the current one
// runs (two buffers).  Every wait is bounded.
//
// Reference behaviour: crates/ops/kernels/paged_attention/trtllm (reference project path).
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
constexpr int kStages = 3;                   // (K, V) tile pairs in flight
constexpr int kMaxSeqs = 1024;

struct PersistArgs {
  const __nv_bfloat16* q;
  const int* page_table;
  const int* seq_lens;
  __nv_bfloat16* out;
  float* part_o;     // [n_cta][2][kNPad][kD]
  float* part_lse;   // [n_cta][2][kNPad]
  int* counters;     // [B * Hkv], zero between launches
  long long ldq, ldo;
  int B, Hq, Hkv, max_pages, page_size;
  float scale_log2;
  unsigned int* status;
};

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// tcgen05.mma with both shared-memory descriptors given as (low, high) words.
__device__ __forceinline__ void umma_words(uint32_t tmem_d, uint32_t a_lo, uint32_t a_hi,
                                           uint32_t b_lo, uint32_t b_hi, uint32_t idesc,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      ".reg .b64 da, db;\n"
      "mov.b64 da, {%1, %2};\n"
      "mov.b64 db, {%3, %4};\n"
      "setp.ne.b32 p, %6, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p;\n"
      "}\n" ::"r"(tmem_d),
      "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Position in the tile list: tile t of (sequence b, kv head hk); `tiles` = tiles of b.
struct Walk {
  int b, hk, t, tiles;
};

// pre[b] = tiles of the sequences before b (pre[B] = all), in shared memory.
__device__ __forceinline__ Walk walk_at(const int* pre, int B, int Hkv, int g) {
  int lo = 0, hi = B - 1;
  while (lo < hi) {          // the last b with Hkv * pre[b] <= g (it has tiles: g < total)
    const int mid = (lo + hi + 1) >> 1;
    if (Hkv * pre[mid] <= g) lo = mid; else hi = mid - 1;
  }
  Walk w;
  w.b = lo;
  w.tiles = pre[lo + 1] - pre[lo];
  const int r = g - Hkv * pre[lo];
  w.hk = r / w.tiles;
  w.t = r - w.hk * w.tiles;
  return w;
}
// The pair after (b, hk), skipping sequences without tiles.  The caller knows one exists.
__device__ __forceinline__ void next_pair(const int* pre, int B, int Hkv, int& b, int& hk,
                                          int& tiles) {
  if (++hk < Hkv) return;
  hk = 0;
  do {
    ++b;
  } while (b < B - 1 && pre[b + 1] == pre[b]);
  tiles = pre[b + 1] - pre[b];
}
__device__ __forceinline__ void walk_next(const int* pre, int B, int Hkv, Walk& w) {
  if (++w.t < w.tiles) return;
  w.t = 0;
  next_pair(pre, B, Hkv, w.b, w.hk, w.tiles);
}

// First tile of CTA c's range, and the CTA that owns tile g.
__device__ __forceinline__ int range_start(int c, int total, int n) {
  return (int)(((long long)c * total) / n);
}
__device__ __forceinline__ int cta_of(int g, int total, int n) {
  int c = (int)(((long long)g * n) / total);
  while (c + 1 < n && range_start(c + 1, total, n) <= g) ++c;
  while (c > 0 && range_start(c, total, n) > g) --c;
  return c;
}

template <int G>
__global__ void __launch_bounds__(192)
paged_decode_persist_kernel(const __grid_constant__ CUtensorMap tmK,
                            const __grid_constant__ CUtensorMap tmV, const PersistArgs a) {
  US_PDL_PROLOGUE();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, tid = threadIdx.x;
  const int cta = blockIdx.x;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* ring = smem;                                    // [kStages][K tile | V tile]
  uint8_t* sQ = smem + kStages * 2 * kTileBytes;           // [2][2 halves]
  uint8_t* sP = sQ + 2 * 2 * kSmallHalf;
  float* red = (float*)(sP + 2 * 2 * kSmallHalf);          // [2][4 warps][16]; sP is [2][2 halves]
  int* pre = (int*)(red + 2 * 4 * kNPad);                  // [B + 1]
  int* lens = pre + kMaxSeqs + 2;                          // [B] keys per sequence
  uint64_t* bars = (uint64_t*)(lens + kMaxSeqs);
  uint64_t* full = bars;             // [kStages]
  uint64_t* empty = bars + 3;        // [kStages]
  uint64_t* s_full = bars + 6;       // [2] by tile parity, like the next two
  uint64_t* p_full = bars + 8;       // [2]
  uint64_t* o_full = bars + 10;      // [2]
  uint64_t* q_ready = bars + 12;     // [2] by segment parity
  uint32_t* tmem_slot = (uint32_t*)(bars + 14);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  volatile int* last_s = (volatile int*)(tmem_slot + 2);

  // ---- tiles per sequence and their prefix sums ----
  const int B = a.B, Hkv = a.Hkv;
  for (int b = tid; b < B; b += blockDim.x) {
    const int len = a.seq_lens[b];
    lens[b] = len;
    pre[b + 1] = (len + kTileKeys - 1) / kTileKeys;
  }
  if (tid == 0) pre[0] = 0;
  __syncthreads();
  if (warp == 0) {
    const int per = (B + 31) / 32;
    const int lo = 1 + lane * per, hi = min(B + 1, lo + per);
    int s = 0;
    for (int i = lo; i < hi; ++i) s += pre[i];
    int ps = s;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, ps, o);
      if (lane >= o) ps += v;
    }
    int run = ps - s;
    for (int i = lo; i < hi; ++i) {
      run += pre[i];
      pre[i] = run;
    }
  }
  __syncthreads();
  const int total = Hkv * pre[B];
  // sequences without keys: zeros (this CTA's share of them)
  if (tid < kD) {
    for (int b = cta; b < B; b += (int)gridDim.x)
      if (pre[b + 1] == pre[b])
        for (int h = 0; h < a.Hq; ++h)
          a.out[(long long)b * a.ldo + (long long)h * kD + tid] = us::f2bf(0.f);
  }
  if (total == 0) return;
  // the list is cut into as many ranges as there are CTAs, or tiles if those are fewer: no
  // range is empty, so the CTAs that share a pair are consecutive
  const int n_cta = min((int)gridDim.x, total);
  if (cta >= n_cta) return;
  const int g0 = range_start(cta, total, n_cta), g1 = range_start(cta + 1, total, n_cta);
  const int n_tiles = g1 - g0;
  if (n_tiles <= 0) return;

  if (tid == 0) {
    for (int s = 0; s < kStages; ++s) {
      tc::mbar_init(&full[s], 1);
      tc::mbar_init(&empty[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      tc::mbar_init(&s_full[i], 1);
      tc::mbar_init(&q_ready[i], 128);
      tc::mbar_init(&p_full[i], 128);
      tc::mbar_init(&o_full[i], 1);
    }
    *abort_flag = 0;
    tc::mbar_fence_init();
  }
  if (warp == 5) {
    tc::tmem_alloc(tmem_slot, 64);
    tc::tmem_relinquish();
  }
  if (tid < 128) {   // rows of P that no head owns stay zero
    for (int c = tid; c < 2 * 2 * kSmallHalf / 16; c += 128)
      reinterpret_cast<uint4*>(sP)[c] = make_uint4(0, 0, 0, 0);
    tc::fence_async_smem();
  }
  tc::tc_fence_before_sync();
  __syncthreads();
  tc::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_O = tmem_base + 2 * kNPad;
  const int pages_per_tile = kTileKeys / a.page_size;

  if (warp == 4) {
    // ---------------------------------------------------------------- producer --
    // The whole warp: lane j fetches page j of every tile (its page id, then two 64-column
    // halves of K and of V), so a tile is four instructions of the warp and the page ids
    // of a tile are one load per lane.  (One thread issuing a tile's 32 copies took as long
    // as a tile's whole computation.)
    {
      if (lane == 0) {
        tc::tma_prefetch_desc(&tmK);
        tc::tma_prefetch_desc(&tmV);
      }
      auto page_of = [&](const Walk& w) -> int {
        const int seq_pages = (lens[w.b] + a.page_size - 1) / a.page_size;
        const int pi = w.t * pages_per_tile + lane;
        return (lane < pages_per_tile && pi < seq_pages && pi < a.max_pages)
                   ? __ldg(a.page_table + (long long)w.b * a.max_pages + pi) : 0;
      };
      Walk w = walk_at(pre, B, Hkv, g0);
      int pg_next = page_of(w);
      for (int i = 0; i < n_tiles; ++i) {
        const int s = i % kStages;
        const uint32_t ph = (uint32_t)(i / kStages) & 1u;
        const int pg = pg_next, hk = w.hk;
        if (i + 1 < n_tiles) {          // the next tile's page ids fly during the wait below
          walk_next(pre, B, Hkv, w);
          pg_next = page_of(w);
        }
        if (!__all_sync(0xffffffffu, tc::mbar_wait(&empty[s], ph ^ 1u, abort_flag))) {
          if (lane == 0) {
            us_dev_fail(a.status, US_DEV_TIMEOUT_EMPTY);
            *abort_flag = 1;
          }
          break;
        }
        if (lane == 0) tc::mbar_expect_tx(&full[s], 2 * kTileBytes);
        __syncwarp();
        if (lane < pages_per_tile) {
          uint8_t* kdst = ring + (size_t)s * 2 * kTileBytes + lane * a.page_size * 128;
          uint8_t* vdst = kdst + kTileBytes;
          const int row = pg * a.page_size;
          tc::tma_load_2d(kdst, &tmK, &full[s], hk * kD, row);
          tc::tma_load_2d(kdst + kHalfBytes, &tmK, &full[s], hk * kD + 64, row);
          tc::tma_load_2d(vdst, &tmV, &full[s], hk * kD, row);
          tc::tma_load_2d(vdst + kHalfBytes, &tmV, &full[s], hk * kD + 64, row);
        }
      }
    }
  } else if (warp == 5) {
    // ------------------------------------------------------------------ issuer --
    if (lane == 0) {
      constexpr uint32_t kIdescQK = tc::make_idesc(128, kNPad, tc::kFmtBF16, tc::kFmtBF16, 0, 0);
      constexpr uint32_t kIdescPV = tc::make_idesc(128, kNPad, tc::kFmtBF16, tc::kFmtBF16, 1, 0);
      // descriptor words: K tiles and the Q / P operands K-major, V tiles MN-major (d on M)
      const uint64_t dk = tc::smem_desc_kmajor_sw128(tc::smem_u32(ring));
      const uint64_t dv = tc::smem_desc_mnmajor_sw128(tc::smem_u32(ring) + kTileBytes, kHalfBytes, 1024);
      const uint64_t dq = tc::smem_desc_kmajor_sw128(tc::smem_u32(sQ));
      const uint64_t dp = tc::smem_desc_kmajor_sw128(tc::smem_u32(sP));
      const uint32_t k_lo = (uint32_t)dk, v_lo = (uint32_t)dv, q_lo = (uint32_t)dq, p_lo = (uint32_t)dp;
      const uint32_t km_hi = (uint32_t)(dk >> 32), mn_hi = (uint32_t)(dv >> 32);
      auto issue_qk = [&](int i, int seg) {
        const uint32_t ka = k_lo + (uint32_t)(i % kStages) * (2 * kTileBytes >> 4);
        const uint32_t qb = q_lo + (uint32_t)(seg & 1) * (2 * kSmallHalf >> 4);
        const uint32_t d = tmem_base + (uint32_t)(i & 1) * kNPad;
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t half = kk >> 2, sub = kk & 3;
          umma_words(d, ka + half * (kHalfBytes >> 4) + 2 * sub, km_hi,
                     qb + half * (kSmallHalf >> 4) + 2 * sub, km_hi, kIdescQK, kk != 0);
        }
        tc::umma_commit(&s_full[i & 1]);
      };
      Walk w = walk_at(pre, B, Hkv, g0);   // position of tile i + 1 after the look-ahead below
      int seg = 0;                          // segment of tile i + 1
      bool ok = tc::mbar_wait(&q_ready[0], 0, abort_flag) && tc::mbar_wait(&full[0], 0, abort_flag);
      if (ok) {
        tc::tc_fence_after_sync();
        issue_qk(0, 0);
      }
      for (int i = 0; ok && i < n_tiles; ++i) {
        if (i + 1 < n_tiles) {
          // S of tile i + 1 (other buffer) before the softmax of tile i is waited for
          const int before = w.b * Hkv + w.hk;
          walk_next(pre, B, Hkv, w);
          if (w.b * Hkv + w.hk != before) {
            ++seg;
            if (!tc::mbar_wait(&q_ready[seg & 1], (uint32_t)(seg >> 1) & 1u, abort_flag)) { ok = false; break; }
          }
          const int s1 = (i + 1) % kStages;
          if (!tc::mbar_wait(&full[s1], (uint32_t)((i + 1) / kStages) & 1u, abort_flag)) { ok = false; break; }
          tc::tc_fence_after_sync();
          issue_qk(i + 1, seg);
        }
        // P(i) ready: S(i) has been consumed and O(i - 2) has been folded
        if (!tc::mbar_wait(&p_full[i & 1], (uint32_t)(i >> 1) & 1u, abort_flag)) { ok = false; break; }
        tc::tc_fence_after_sync();
        const uint32_t va = v_lo + (uint32_t)(i % kStages) * (2 * kTileBytes >> 4);
        const uint32_t pb = p_lo + (uint32_t)(i & 1) * (2 * kSmallHalf >> 4);
        const uint32_t d = tmem_O + (uint32_t)(i & 1) * kNPad;
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          // A = V^T: d on M (two 64-wide chunks, 16 KiB apart), 16 keys = two groups of
          // eight rows (1 KiB apart) per instruction, 2 KiB further per instruction
          const uint32_t half = kk >> 2, sub = kk & 3;
          umma_words(d, va + (uint32_t)kk * (2048 >> 4), mn_hi,
                     pb + half * (kSmallHalf >> 4) + 2 * sub, km_hi, kIdescPV, kk != 0);
        }
        tc::umma_commit(&o_full[i & 1]);
        tc::umma_commit(&empty[i % kStages]);
      }
      if (!ok) {
        us_dev_fail(a.status, US_DEV_TIMEOUT_FULL);
        *abort_flag = 1;
      }
    }
  } else {
    // ------------------------------------------- softmax / output: lane = tid --
    const uint32_t lane_addr = ((uint32_t)(warp * 32) << 16);
    // Q operand of a pair: rows = heads (zero padded to 16), K-major, 128-byte swizzle
    auto stage_q = [&](int b, int hk, int buf) {
      uint8_t* dstq = sQ + buf * 2 * kSmallHalf;
      for (int c = tid; c < kNPad * 16; c += 128) {
        const int g = c >> 4, ch = c & 15;  // 16-byte chunk ch of head row g
        uint4 v = make_uint4(0, 0, 0, 0);
        if (g < G)
          v = *reinterpret_cast<const uint4*>(a.q + (long long)b * a.ldq +
                                              (long long)(hk * G + g) * kD + ch * 8);
        const int half = ch >> 3;
        *reinterpret_cast<uint4*>(dstq + half * kSmallHalf + tc::sw128_offset(g, ch & 7)) = v;
      }
      tc::fence_async_smem();
      tc::mbar_arrive(&q_ready[buf]);
    };
    Walk w = walk_at(pre, B, Hkv, g0);
    int b = w.b, hk = w.hk, t0 = w.t, tiles = w.tiles;
    int g = g0, seg = 0, i = 0;
    stage_q(b, hk, 0);
    if (g + (tiles - t0) < g1) {
      int nb = b, nhk = hk, nt = tiles;
      next_pair(pre, B, Hkv, nb, nhk, nt);
      stage_q(nb, nhk, 1);
    }
    bool ok = true;
    // pairs cut by this range (slot 0: its first segment, slot 1: its last) whose merge is due
    int pb0 = -1, ph0 = 0, pt0 = 0, old0 = 0, pb1 = -1, ph1 = 0, pt1 = 0, old1 = 0;
    while (ok && g < g1) {
      const int n_seg = min(tiles - t0, g1 - g);
      if (seg >= 1 && g + n_seg < g1) {   // the segment after this one: its buffer is free now
        int nb = b, nhk = hk, nt = tiles;
        next_pair(pre, B, Hkv, nb, nhk, nt);
        stage_q(nb, nhk, (seg + 1) & 1);
      }
      const int seq_len = lens[b];
      // a1 / a2: rescaling factors of the previous tile and of the one before it
      float m_run[G], l_part[G], o_acc[G], a1[G], a2[G];
#pragma unroll
      for (int gi = 0; gi < G; ++gi) {
        m_run[gi] = -INFINITY;
        l_part[gi] = 0.f;
        o_acc[gi] = 0.f;
        a1[gi] = 0.f;
        a2[gi] = 0.f;
      }
      // o_acc = o_acc * factor + O of the tile with global index j (buffer j & 1)
      auto fold = [&](int j, const float (&factor)[G]) {
        tc::tc_fence_after_sync();
        uint32_t orr[16];
        tc::tmem_ld16(tmem_O + (uint32_t)(j & 1) * kNPad + lane_addr, orr);
        tc::tmem_ld_wait();
#pragma unroll
        for (int gi = 0; gi < G; ++gi) o_acc[gi] = o_acc[gi] * factor[gi] + __uint_as_float(orr[gi]);
      };
      for (int tt = 0; tt < n_seg; ++tt, ++i) {
        if (!tc::mbar_wait(&s_full[i & 1], (uint32_t)(i >> 1) & 1u, abort_flag)) { ok = false; break; }
        tc::tc_fence_after_sync();
        uint32_t sr[16];
        tc::tmem_ld16(tmem_base + (uint32_t)(i & 1) * kNPad + lane_addr, sr);
        tc::tmem_ld_wait();
        const int key = (t0 + tt) * kTileKeys + tid;
        const bool valid = key < seq_len;
        float s[G];
        float* rbuf = red + (i & 1) * 4 * kNPad;
#pragma unroll
        for (int gi = 0; gi < G; ++gi) {
          s[gi] = valid ? __uint_as_float(sr[gi]) * a.scale_log2 : -INFINITY;
          const float wm = us::warp_max(s[gi]);
          if (lane == 0) rbuf[warp * kNPad + gi] = wm;
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        float alpha[G], p[G];
#pragma unroll
        for (int gi = 0; gi < G; ++gi) {
          const float tm = fmaxf(fmaxf(rbuf[gi], rbuf[kNPad + gi]),
                                 fmaxf(rbuf[2 * kNPad + gi], rbuf[3 * kNPad + gi]));
          const float m_new = fmaxf(m_run[gi], tm);
          alpha[gi] = (m_run[gi] == -INFINITY) ? 0.f : ex2(m_run[gi] - m_new);
          p[gi] = valid ? ex2(s[gi] - m_new) : 0.f;
          l_part[gi] = l_part[gi] * alpha[gi] + p[gi];
          m_run[gi] = m_new;
        }
        if (i >= 2) {
          // the product of tile i - 2 is complete: its P buffer (this tile's) is free, and
          // inside a segment its O is folded in under the factor that tile computed
          if (!tc::mbar_wait(&o_full[i & 1], (uint32_t)((i - 2) >> 1) & 1u, abort_flag)) { ok = false; break; }
          if (tt >= 2) fold(i - 2, a2);
        }
#pragma unroll
        for (int gi = 0; gi < G; ++gi) {
          a2[gi] = a1[gi];
          a1[gi] = alpha[gi];
        }
        {   // P^T -> smem as the K-major B operand: row = head, column = key of the tile
          const int half = tid >> 6, col = tid & 63;
          uint8_t* pbuf = sP + (i & 1) * 2 * kSmallHalf;
#pragma unroll
          for (int gi = 0; gi < G; ++gi) {
            uint8_t* dst = pbuf + half * kSmallHalf + tc::sw128_offset(gi, col >> 3) + (col & 7) * 2;
            *reinterpret_cast<__nv_bfloat16*>(dst) = us::f2bf(p[gi]);
          }
        }
        tc::fence_async_smem();
        tc::tc_fence_before_sync();
        tc::mbar_arrive(&p_full[i & 1]);
      }
      if (!ok) break;
      // ---- end of the segment: the last two tiles' products, the row sums, the result ----
      {
        const int e = i - 1;
        if (n_seg >= 2) {
          if (!tc::mbar_wait(&o_full[(e - 1) & 1], (uint32_t)((e - 1) >> 1) & 1u, abort_flag)) { ok = false; break; }
          fold(e - 1, a2);
        }
        if (!tc::mbar_wait(&o_full[e & 1], (uint32_t)(e >> 1) & 1u, abort_flag)) { ok = false; break; }
        fold(e, a1);
      }
      tc::tc_fence_before_sync();      // the next product into O is ordered after these reads
      float* rbuf = red;
      asm volatile("bar.sync 1, 128;" ::: "memory");
#pragma unroll
      for (int gi = 0; gi < G; ++gi) {
        const float ws = us::warp_sum(l_part[gi]);
        if (lane == 0) rbuf[warp * kNPad + gi] = ws;
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      const bool whole = t0 == 0 && n_seg == tiles;
      const int which = seg == 0 ? 0 : 1;
      const long long slot = ((long long)cta * 2 + which) * kNPad;
#pragma unroll
      for (int gi = 0; gi < G; ++gi) {
        const float l = rbuf[gi] + rbuf[kNPad + gi] + rbuf[2 * kNPad + gi] + rbuf[3 * kNPad + gi];
        const float inv = l > 0.f ? 1.f / l : 0.f;
        if (whole) {
          a.out[(long long)b * a.ldo + (long long)(hk * G + gi) * kD + tid] = us::f2bf(o_acc[gi] * inv);
        } else {
          a.part_o[(slot + gi) * kD + tid] = o_acc[gi] * inv;
          if (tid == 0)   // m_run is in the log2 domain; the merge works in natural logs
            a.part_lse[slot + gi] = l > 0.f ? (m_run[gi] + log2f(l)) * 0.6931471805599453f : -INFINITY;
        }
      }
      if (!whole) {
        // arrival at the pair's counter.  The count it returns is looked at only after the
        // CTA's last tile (an atomic does not stall its thread until the value is used), so
        // the softmax threads go on with the next segment at once.
        __threadfence();
        asm volatile("bar.sync 2, 128;" ::: "memory");
        if (which == 0) {       // scalars, not an indexed array: the count stays in a register
          if (tid == 0) old0 = atomicAdd(a.counters + b * Hkv + hk, 1);
          pb0 = b; ph0 = hk; pt0 = tiles;
        } else {
          if (tid == 0) old1 = atomicAdd(a.counters + b * Hkv + hk, 1);
          pb1 = b; ph1 = hk; pt1 = tiles;
        }
      }
      g += n_seg;
      ++seg;
      t0 = 0;
      if (g < g1) next_pair(pre, B, Hkv, b, hk, tiles);
    }
    if (!ok) us_dev_fail(a.status, US_DEV_TIMEOUT_ACC);
    // the CTA that arrived last at a pair's counter merges the slots of the CTAs the pair spans
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const int pb_ = k == 0 ? pb0 : pb1, phk = k == 0 ? ph0 : ph1, ptiles = k == 0 ? pt0 : pt1;
      const int pold = k == 0 ? old0 : old1;
      if (pb_ < 0) continue;
      const int pair_begin = Hkv * pre[pb_] + phk * ptiles, pair_last = pair_begin + ptiles - 1;
      const int c_first = cta_of(pair_begin, total, n_cta), c_last = cta_of(pair_last, total, n_cta);
      if (tid == 0) {
        const int last = pold == c_last - c_first;
        if (last) a.counters[pb_ * Hkv + phk] = 0;
        *last_s = last;
      }
      asm volatile("bar.sync 2, 128;" ::: "memory");
      if (*last_s) {
        __threadfence();
        float mx[G], acc[G], den[G];
#pragma unroll
        for (int gi = 0; gi < G; ++gi) {
          mx[gi] = -INFINITY;
          acc[gi] = 0.f;
          den[gi] = 0.f;
        }
        for (int c = c_first; c <= c_last; ++c) {
          const int wc = range_start(c, total, n_cta) >= pair_begin ? 0 : 1;
          const long long sl = ((long long)c * 2 + wc) * kNPad;
#pragma unroll
          for (int gi = 0; gi < G; ++gi) mx[gi] = fmaxf(mx[gi], __ldcg(a.part_lse + sl + gi));
        }
        for (int c = c_first; c <= c_last; ++c) {
          const int wc = range_start(c, total, n_cta) >= pair_begin ? 0 : 1;
          const long long sl = ((long long)c * 2 + wc) * kNPad;
#pragma unroll
          for (int gi = 0; gi < G; ++gi) {
            const float l = __ldcg(a.part_lse + sl + gi);
            const float wgt = (l == -INFINITY) ? 0.f : __expf(l - mx[gi]);
            den[gi] += wgt;
            acc[gi] += wgt * __ldcg(a.part_o + (sl + gi) * kD + tid);
          }
        }
#pragma unroll
        for (int gi = 0; gi < G; ++gi)
          a.out[(long long)pb_ * a.ldo + (long long)(phk * G + gi) * kD + tid] =
              us::f2bf(den[gi] > 0.f ? acc[gi] / den[gi] : 0.f);
      }
      asm volatile("bar.sync 2, 128;" ::: "memory");   // last_s is rewritten for the next pair
    }
  }
  tc::tc_fence_before_sync();
  __syncthreads();
  if (warp == 5) {
    __syncwarp();
    tc::tmem_dealloc(tmem_base, 64);
  }
}

template <int G>
int launch_persist(const CUtensorMap& tmK, const CUtensorMap& tmV, const PersistArgs& a, int n_cta,
                   cudaStream_t stream) {
  // ring, Q [2], P [2], reduction scratch, prefix sums, barriers and flags, alignment slack
  const size_t smem = (size_t)kStages * 2 * kTileBytes + 4 * kSmallHalf + 4 * kSmallHalf +
                      2 * 4 * kNPad * 4 + (2 * kMaxSeqs + 2) * 4 + 20 * 8 + 1024;
  static bool configured = false;
  if (!configured) {
    US_CUDA_CHECK(cudaFuncSetAttribute(paged_decode_persist_kernel<G>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured = true;
  }
  us::launch_pdl(paged_decode_persist_kernel<G>, dim3(n_cta), dim3(192), smem, stream, tmK, tmV, a);
  US_LAUNCH_CHECK();
  return US_OK;
}

int sm_count() {
  static const int n = [] {
    int dev = 0, v = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev);
    return v > 0 ? v : 148;
  }();
  return n;
}

}  // namespace

// Bytes of the partial-output scratch and CTAs of a launch on this device.
US_API long long us_paged_decode_persist_scratch_bytes() {
  return (long long)sm_count() * 2 * kNPad * (kD + 1) * (long long)sizeof(float);
}

// q [B, Hq * 128] (row pitch ldq), bf16 caches [pages, page_size, Hkv, 128], page_table
// [B, max_pages], seq_lens [B]; out [B, Hq * 128] (row pitch ldo).  `scratch` of
// us_paged_decode_persist_scratch_bytes() bytes; `counters` [B * Hkv] int32, zero before the
// first call and left zero by every call.  Calls that share them must be ordered on the device.
US_API int us_paged_decode_attention_persist(const void* q, const void* kcache, const void* vcache,
                                             const int* page_table, const int* seq_lens, void* out,
                                             void* scratch, int* counters, int B, int Hq, int Hkv,
                                             int D, int num_pages, int max_pages, int page_size,
                                             float scale, long long ldq, long long ldo,
                                             void* stream_) {
  US_REQUIRE(q && kcache && vcache && page_table && seq_lens && out && scratch && counters);
  US_REQUIRE(D == kD && Hkv >= 1 && Hq % Hkv == 0 && Hq / Hkv <= kNPad && B <= kMaxSeqs);
  US_REQUIRE(page_size >= 8 && page_size <= 128 && (kTileKeys % page_size) == 0);
  US_REQUIRE((ldq % 8) == 0 && ((uintptr_t)q % 16) == 0);
  if (B == 0) return US_OK;
  cudaStream_t stream = (cudaStream_t)stream_;
  CUtensorMap tmK, tmV;
  const uint64_t rows = (uint64_t)num_pages * page_size, cols = (uint64_t)Hkv * D;
  int rc = us_tmap_2d(&tmK, kcache, US_TMAP_BF16, rows, cols, cols, page_size, 64, US_SWZ_128);
  if (rc) return rc;
  rc = us_tmap_2d(&tmV, vcache, US_TMAP_BF16, rows, cols, cols, page_size, 64, US_SWZ_128);
  if (rc) return rc;
  const int n_cta = sm_count();
  PersistArgs a;
  a.q = (const __nv_bfloat16*)q;
  a.page_table = page_table;
  a.seq_lens = seq_lens;
  a.out = (__nv_bfloat16*)out;
  a.part_o = (float*)scratch;
  a.part_lse = (float*)scratch + (long long)n_cta * 2 * kNPad * kD;
  a.counters = counters;
  a.ldq = ldq; a.ldo = ldo;
  a.B = B; a.Hq = Hq; a.Hkv = Hkv; a.max_pages = max_pages; a.page_size = page_size;
  a.scale_log2 = scale * 1.4426950408889634f;
  a.status = us_status_ptr();
  switch (Hq / Hkv) {
    case 1: return launch_persist<1>(tmK, tmV, a, n_cta, stream);
    case 2: return launch_persist<2>(tmK, tmV, a, n_cta, stream);
    case 4: return launch_persist<4>(tmK, tmV, a, n_cta, stream);
    case 8: return launch_persist<8>(tmK, tmV, a, n_cta, stream);
    case 16: return launch_persist<16>(tmK, tmV, a, n_cta, stream);
    default: return US_ERR_UNSUPPORTED;
  }
}
