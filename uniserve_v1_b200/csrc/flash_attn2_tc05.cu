// Varlen flash attention forward, two query tiles per CTA (head_dim 128 or 64, bf16, GQA).
//
// One CTA owns 256 query rows of one (sequence, head) as two 128-row tiles A
// and B and walks the keys in blocks of 128.  The tensor pipe alternates between
// the tiles, so one tile's softmax runs under the other tile's products:
//
//   S_X = Q_X K^T      tcgen05.mma, operands from TMA (K-major, 128-byte swizzle),
//                      S_A and S_B in tensor memory (128 columns each)
//   softmax X          one warpgroup per tile, thread r owns row r: row maximum and
//                      sum in the log2 domain; P is written back over the first 64
//                      columns of S_X as packed bf16 (tcgen05.st) - it never
//                      touches shared memory
//   O_X += P_X V       tcgen05.mma with the A operand in tensor memory, V straight
//                      from TMA as the MN-major B operand; O_A, O_B stay in TMEM and
//                      are rescaled only when a row maximum grew by more than 2^8
//
// Tensor memory: S_A [0,128) S_B [128,256) O_A [256,384) O_B [384,512).
// Roles: warps 0-3 softmax/epilogue of tile A, warps 4-7 of tile B, warp 8 TMA
// producer, warp 9 TMEM owner and MMA issuer.  Products issue in program order
// from one thread, which is what makes the S/P aliasing safe: S_X(j+1) is issued
// after O_X += P_X(j) V(j).  Causal masks are aligned to the bottom right.  Every
// wait is bounded.
//
// The reference runs FlashAttention-4 here (crates/ops/kernels/dense_attention/fa4,
// reference project path); the two-tile ping-pong and P in tensor memory follow the
// same idea, the code is independent.
#include "include/us_common.cuh"
#include "include/us_tc05.cuh"
#include "include/us_tmap.h"

namespace {

constexpr int kDMax = 128;  // head widths served: 128 and 64 (template parameter kD)
constexpr int kBM = 128;   // query rows per tile (two tiles per CTA)
constexpr int kBN = 128;   // keys per block
constexpr int kHalf = 128 * 128;         // bytes of one 64-column half tile (128 rows x 128 B)
constexpr float kRescaleThreshold = 8.f; // log2 units

struct Flash2Args {
  const int* cu_q;
  const int* cu_k;
  __nv_bfloat16* out;
  long long ldo;
  int Hq, Hkv, causal;
  float scale_log2;
  unsigned int* status;
  // Sequence-parallel return: output row r (one sequence) belongs to rank
  // r / peer_rows and is stored into that rank's buffer at row r % peer_rows,
  // column peer_col0 + head * 128 (row pitch peer_ld elements), so the "heads ->
  // rows" exchange happens as peer stores from this epilogue.
  void* peer_out[8];
  int peer_rows;
  int peer_col0;
  long long peer_ld;
};

__device__ __forceinline__ float ex2f(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Packed FP32 pairs (two lanes per instruction) and the three-input maximum: the
// softmax warpgroups are bound by instruction issue, not by the special-function unit.
__device__ __forceinline__ unsigned long long pack2(float a, float b) {
  unsigned long long r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ void unpack2(unsigned long long r, float& a, float& b) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(r));
}
__device__ __forceinline__ unsigned long long fma2(unsigned long long a, unsigned long long b,
                                                   unsigned long long c) {
  unsigned long long d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ unsigned long long add2(unsigned long long a, unsigned long long b) {
  unsigned long long d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

template <int kD>
__global__ void __launch_bounds__(320, 1)
flash2_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                  const __grid_constant__ CUtensorMap tmV, const Flash2Args a) {
  US_PDL_PROLOGUE();
  constexpr int kHalves = kD / 64;          // 64-column (128-byte) slabs per tile
  constexpr int kTile = kHalves * kHalf;    // 32 KiB (head 128) or 16 KiB (head 64)
  const int q_pair = blockIdx.x, h = blockIdx.y, seq = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, tid = threadIdx.x;
  const int q_start = a.cu_q[seq], q_len = a.cu_q[seq + 1] - q_start;
  const int k_start = a.cu_k[seq], kv_len = a.cu_k[seq + 1] - k_start;
  const int q0 = q_pair * 2 * kBM;
  if (q0 >= q_len) return;
  const int hk = h / (a.Hq / a.Hkv);
  const int shift = kv_len - q_len;  // causal: key <= query + shift
  // key blocks each tile walks (0 when the tile has no row or sees no key)
  int nb_t[2];
#pragma unroll
  for (int x = 0; x < 2; ++x) {
    const int q0x = q0 + x * kBM;
    int lim = kv_len;
    if (a.causal) lim = min(kv_len, q0x + kBM + shift);
    nb_t[x] = (q0x < q_len && lim > 0) ? (lim + kBN - 1) / kBN : 0;
  }
  const int nb = max(nb_t[0], nb_t[1]);

  if (tid < 2 * kBM) {  // tiles without a visible key: zeros
    const int x = tid >> 7;
    const int qi = q0 + tid;
    if (nb_t[x] == 0 && qi < q_len) {
      __nv_bfloat16* zrow = a.out + (long long)(q_start + qi) * a.ldo + (long long)h * kD;
      if (a.peer_rows > 0) {
        const int row = q_start + qi;
        const int p = row / a.peer_rows;
        zrow = (__nv_bfloat16*)a.peer_out[p] + (long long)(row - p * a.peer_rows) * a.peer_ld +
               a.peer_col0 + (long long)h * kD;
      }
      uint4* dst = reinterpret_cast<uint4*>(zrow);
      for (int i = 0; i < kD / 8; ++i) dst[i] = make_uint4(0, 0, 0, 0);
    }
  }
  if (nb == 0) return;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* sQ = smem;                  // two tiles
  uint8_t* sK = smem + 2 * kTile;      // two stages
  uint8_t* sV = smem + 4 * kTile;      // two stages
  uint64_t* bars = (uint64_t*)(smem + 6 * kTile);
  uint64_t* q_full = bars;
  uint64_t* k_full = bars + 1;   // [2]
  uint64_t* k_empty = bars + 3;  // [2]
  uint64_t* v_full = bars + 5;   // [2]
  uint64_t* v_empty = bars + 7;  // [2]
  uint64_t* s_full = bars + 9;   // [2] per tile
  uint64_t* p_full = bars + 11;  // [2] per tile
  uint64_t* o_full = bars + 13;  // [2] per tile
  uint32_t* tmem_slot = (uint32_t*)(bars + 15);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  if (tid == 0) {
    tc::mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      tc::mbar_init(&k_full[i], 1);
      tc::mbar_init(&k_empty[i], 1);
      tc::mbar_init(&v_full[i], 1);
      tc::mbar_init(&v_empty[i], 1);
      tc::mbar_init(&s_full[i], 1);
      tc::mbar_init(&p_full[i], 128);
      tc::mbar_init(&o_full[i], 1);
    }
    *abort_flag = 0;
    tc::mbar_fence_init();
  }
  if (warp == 9) {
    tc::tmem_alloc(tmem_slot, 512);
    tc::tmem_relinquish();
  }
  tc::tc_fence_before_sync();
  __syncthreads();
  tc::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 8) {
    if (lane == 0) {
      tc::tma_prefetch_desc(&tmQ);
      tc::tma_prefetch_desc(&tmK);
      tc::tma_prefetch_desc(&tmV);
      tc::mbar_expect_tx(q_full, 2 * kTile);
#pragma unroll
      for (int x = 0; x < 2; ++x) {
        const int row = q_start + q0 + x * kBM;   // rows past the tensor read as zeros
#pragma unroll
        for (int hf = 0; hf < kHalves; ++hf)
          tc::tma_load_2d(sQ + x * kTile + hf * kHalf, &tmQ, q_full, h * kD + 64 * hf, row);
      }
      for (int j = 0; j < nb; ++j) {
        const int st = j & 1;
        const uint32_t ph = (uint32_t)(j >> 1) & 1u;
        const int row = k_start + j * kBN;
        if (!tc::mbar_wait(&k_empty[st], ph ^ 1u, abort_flag)) {
          us_dev_fail(a.status, US_DEV_TIMEOUT_EMPTY);
          *abort_flag = 1;
          break;
        }
        tc::mbar_expect_tx(&k_full[st], kTile);
#pragma unroll
        for (int hf = 0; hf < kHalves; ++hf)
          tc::tma_load_2d(sK + st * kTile + hf * kHalf, &tmK, &k_full[st], hk * kD + 64 * hf, row);
        if (!tc::mbar_wait(&v_empty[st], ph ^ 1u, abort_flag)) {
          us_dev_fail(a.status, US_DEV_TIMEOUT_EMPTY);
          *abort_flag = 1;
          break;
        }
        tc::mbar_expect_tx(&v_full[st], kTile);
#pragma unroll
        for (int hf = 0; hf < kHalves; ++hf)
          tc::tma_load_2d(sV + st * kTile + hf * kHalf, &tmV, &v_full[st], hk * kD + 64 * hf, row);
      }
    }
  } else if (warp == 9) {
    if (lane == 0) {
      constexpr uint32_t kIdescQK = tc::make_idesc(kBM, kBN, tc::kFmtBF16, tc::kFmtBF16, 0, 0);
      constexpr uint32_t kIdescPV = tc::make_idesc(kBM, kD, tc::kFmtBF16, tc::kFmtBF16, 0, 1);
      auto issue_qk = [&](int x, int j) {
        const uint32_t q_addr = tc::smem_u32(sQ + x * kTile);
        const uint32_t k_addr = tc::smem_u32(sK + (j & 1) * kTile);
        const uint32_t s_tmem = tmem_base + (uint32_t)x * kBN;
#pragma unroll
        for (int kk = 0; kk < kD / 16; ++kk) {
          const uint32_t half = kk >> 2, sub = kk & 3;
          const uint64_t ad = tc::smem_desc_kmajor_sw128(q_addr + half * kHalf) + 2 * sub;
          const uint64_t bd = tc::smem_desc_kmajor_sw128(k_addr + half * kHalf) + 2 * sub;
          tc::umma_f16(s_tmem, ad, bd, kIdescQK, kk != 0);
        }
        tc::umma_commit(&s_full[x]);
      };
      auto issue_pv = [&](int x, int j) {
        const uint32_t v_addr = tc::smem_u32(sV + (j & 1) * kTile);
        const uint32_t p_tmem = tmem_base + (uint32_t)x * kBN;
        const uint32_t o_tmem = tmem_base + 256 + (uint32_t)x * kD;
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          // A = P: 16 keys = 8 packed columns per instruction.  B = V: d on N (two
          // 64-wide chunks, 16 KiB apart), 16 keys = two groups of eight rows (1 KiB apart).
          const uint64_t bd = tc::smem_desc_mnmajor_sw128(v_addr + kk * 2048, kHalf, 1024);
          tc::umma_f16_ts(o_tmem, p_tmem + kk * 8, bd, kIdescPV, (j | kk) != 0);
        }
        tc::umma_commit(&o_full[x]);
      };
      bool ok = tc::mbar_wait(q_full, 0, abort_flag) && tc::mbar_wait(&k_full[0], 0, abort_flag);
      if (ok) {
        tc::tc_fence_after_sync();
        if (nb_t[0] > 0) issue_qk(0, 0);
        if (nb_t[1] > 0) issue_qk(1, 0);
        tc::umma_commit(&k_empty[0]);
      }
      for (int j = 0; ok && j < nb; ++j) {
        const uint32_t ph = (uint32_t)(j >> 1) & 1u;
        const uint32_t pj = (uint32_t)j & 1u;
        const bool more = j + 1 < nb;
        if (!tc::mbar_wait(&v_full[j & 1], ph, abort_flag)) { ok = false; break; }
        // tile A: O_A += P_A V_j, then S_A of the next block
        if (j < nb_t[0]) {
          if (!tc::mbar_wait(&p_full[0], pj, abort_flag)) { ok = false; break; }
          tc::tc_fence_after_sync();
          issue_pv(0, j);
        }
        if (more) {
          if (!tc::mbar_wait(&k_full[(j + 1) & 1], (uint32_t)((j + 1) >> 1) & 1u, abort_flag)) {
            ok = false;
            break;
          }
          tc::tc_fence_after_sync();
          if (j + 1 < nb_t[0]) issue_qk(0, j + 1);
        }
        // tile B
        if (j < nb_t[1]) {
          if (!tc::mbar_wait(&p_full[1], pj, abort_flag)) { ok = false; break; }
          tc::tc_fence_after_sync();
          issue_pv(1, j);
        }
        tc::umma_commit(&v_empty[j & 1]);
        if (more) {
          if (j + 1 < nb_t[1]) issue_qk(1, j + 1);
          tc::umma_commit(&k_empty[(j + 1) & 1]);
        }
      }
      if (!ok) {
        us_dev_fail(a.status, US_DEV_TIMEOUT_FULL);
        *abort_flag = 1;
      }
    }
  } else {
    // ---- softmax: warpgroup = tile, thread = query row ----
    const int x = warp >> 2;
    const int r = tid & 127;
    const int nbx = nb_t[x];
    const uint32_t lane_addr = ((uint32_t)((warp & 3) * 32) << 16);
    const uint32_t s_tmem = tmem_base + (uint32_t)x * kBN + lane_addr;
    const uint32_t o_tmem = tmem_base + 256 + (uint32_t)x * kD + lane_addr;
    const int q_idx = q0 + x * kBM + r;
    float m_used = -INFINITY, l_sum = 0.f;
    bool ok = true;
    for (int j = 0; j < nbx; ++j) {
      if (!tc::mbar_wait(&s_full[x], (uint32_t)j & 1u, abort_flag)) { ok = false; break; }
      tc::tc_fence_after_sync();
      const int kbase = j * kBN;
      int lim = kv_len - kbase;   // keys of this block this row may see: [0, lim)
      if (a.causal) lim = min(lim, q_idx + shift - kbase + 1);
      const bool need_mask = lim < kBN;
      // The whole row of S goes to registers in one round trip; four independent
      // chains keep the maximum and the sum from serialising on instruction latency.
      uint32_t v0[32], v1[32], v2[32], v3[32];
      tc::tmem_ld32(s_tmem, v0);
      tc::tmem_ld32(s_tmem + 32, v1);
      tc::tmem_ld32(s_tmem + 64, v2);
      tc::tmem_ld32(s_tmem + 96, v3);
      tc::tmem_ld_wait();
      if (need_mask) {   // last key block of the sequence or the causal diagonal
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          if (i >= lim) v0[i] = 0xff800000u;
          if (32 + i >= lim) v1[i] = 0xff800000u;
          if (64 + i >= lim) v2[i] = 0xff800000u;
          if (96 + i >= lim) v3[i] = 0xff800000u;
        }
      }
      float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
      for (int i = 0; i < 32; i += 2) {
        mx0 = max3(mx0, __uint_as_float(v0[i]), __uint_as_float(v0[i + 1]));
        mx1 = max3(mx1, __uint_as_float(v1[i]), __uint_as_float(v1[i + 1]));
        mx2 = max3(mx2, __uint_as_float(v2[i]), __uint_as_float(v2[i + 1]));
        mx3 = max3(mx3, __uint_as_float(v3[i]), __uint_as_float(v3[i + 1]));
      }
      const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
      const float m_new = fmaxf(m_used, mx * a.scale_log2);
      const bool grow = m_new - m_used > kRescaleThreshold;
      const bool any_grow =
          __any_sync(0xffffffffu, grow || (m_used == -INFINITY && m_new > -INFINITY));
      if (any_grow) {
        const float alpha = (m_used == -INFINITY) ? 0.f : ex2f(m_used - m_new);
        if (j > 0) {
          // O_X is stable once the previous block's second product is done.
          if (!tc::mbar_wait(&o_full[x], (uint32_t)(j - 1) & 1u, abort_flag)) { ok = false; break; }
          tc::tc_fence_after_sync();
#pragma unroll 1
          for (int c = 0; c < kD; c += 32) {
            uint32_t v[32];
            tc::tmem_ld32(o_tmem + c, v);
            tc::tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
            tc::tmem_st32(o_tmem + c, v);
          }
        }
        l_sum *= alpha;
        m_used = m_new;
      }
      const float m_eff = (m_used == -INFINITY) ? 0.f : m_used;
      const float neg_m = -m_eff;
      const unsigned long long sc2 = pack2(a.scale_log2, a.scale_log2);
      const unsigned long long nm2 = pack2(neg_m, neg_m);
      unsigned long long l0 = pack2(0.f, 0.f), l1 = l0, l2 = l0, l3 = l0;
      uint32_t pk0[32], pk1[32];
      auto exp_pair = [&](uint32_t x0, uint32_t x1, unsigned long long& l) -> uint32_t {
        float t0, t1;
        unpack2(fma2(pack2(__uint_as_float(x0), __uint_as_float(x1)), sc2, nm2), t0, t1);
        const float p0 = ex2f(t0), p1 = ex2f(t1);
        l = add2(l, pack2(p0, p1));
        __nv_bfloat162 t = __floats2bfloat162_rn(p0, p1);
        return *reinterpret_cast<uint32_t*>(&t);
      };
#pragma unroll
      for (int i = 0; i < 32; i += 2) {
        pk0[i >> 1] = exp_pair(v0[i], v0[i + 1], l0);
        pk0[16 + (i >> 1)] = exp_pair(v1[i], v1[i + 1], l1);
        pk1[i >> 1] = exp_pair(v2[i], v2[i + 1], l2);
        pk1[16 + (i >> 1)] = exp_pair(v3[i], v3[i + 1], l3);
      }
      {
        float s0, s1;
        unpack2(add2(add2(l0, l1), add2(l2, l3)), s0, s1);
        l_sum += s0 + s1;
      }
      // P (64 packed columns) replaces the first half of S, which is in registers now.
      tc::tmem_st32(s_tmem, pk0);
      tc::tmem_st32(s_tmem + 32, pk1);
      tc::tmem_st_wait();
      tc::tc_fence_before_sync();
      tc::mbar_arrive(&p_full[x]);
    }
    if (nbx > 0) {
      if (ok && tc::mbar_wait(&o_full[x], (uint32_t)(nbx - 1) & 1u, abort_flag)) {
        tc::tc_fence_after_sync();
        const float inv = l_sum > 0.f ? 1.f / l_sum : 0.f;
        const bool row_ok = q_idx < q_len;
        __nv_bfloat16* orow = a.out + (long long)(q_start + q_idx) * a.ldo + (long long)h * kD;
        if (a.peer_rows > 0) {
          const int row = q_start + q_idx;
          const int p = row / a.peer_rows;
          orow = (__nv_bfloat16*)a.peer_out[p] + (long long)(row - p * a.peer_rows) * a.peer_ld +
                 a.peer_col0 + (long long)h * kD;
        }
#pragma unroll 1
        for (int c = 0; c < kD; c += 32) {
          uint32_t v[32];
          tc::tmem_ld32(o_tmem + c, v);
          tc::tmem_ld_wait();
          if (row_ok) {
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4) {
              us::Pack16 o;
#pragma unroll
              for (int i = 0; i < 8; ++i) o.b[i] = us::f2bf(__uint_as_float(v[q4 * 8 + i]) * inv);
              *reinterpret_cast<uint4*>(orow + c + q4 * 8) = o.u;
            }
          }
        }
      } else {
        us_dev_fail(a.status, US_DEV_TIMEOUT_ACC);
      }
    }
  }
  tc::tc_fence_before_sync();
  __syncthreads();
  if (warp == 9) {
    __syncwarp();
    tc::tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace

namespace {

int flash2_impl(const void* q, const void* k, const void* v, void* out, const int* cu_q,
                const int* cu_k, int n_seqs, int Tq, int Tk, int Hq, int Hkv, int D, int max_q,
                long long ldq, long long ldk, long long ldv, long long ldo, float scale, int causal,
                void* const* peer_out, int n_peers, int peer_rows, int peer_col0,
                long long peer_ld, cudaStream_t stream) {
  US_REQUIRE(q && k && v && (out || peer_out) && cu_q && cu_k && n_seqs >= 1 && Tq >= 1 &&
             Tk >= 1);
  US_REQUIRE((D == 128 || D == 64) && Hkv >= 1 && Hq % Hkv == 0 && max_q >= 1);
  US_REQUIRE((ldq % 8) == 0 && (ldk % 8) == 0 && (ldv % 8) == 0 && (ldo % 8) == 0);
  US_REQUIRE(((uintptr_t)q % 16) == 0 && ((uintptr_t)k % 16) == 0 && ((uintptr_t)v % 16) == 0 &&
             ((uintptr_t)out % 16) == 0);
  CUtensorMap tmQ, tmK, tmV;
  int rc = us_tmap_2d(&tmQ, q, US_TMAP_BF16, (uint64_t)Tq, (uint64_t)Hq * D, (uint64_t)ldq, kBM,
                      64, US_SWZ_128);
  if (rc) return rc;
  rc = us_tmap_2d(&tmK, k, US_TMAP_BF16, (uint64_t)Tk, (uint64_t)Hkv * D, (uint64_t)ldk, kBN, 64,
                  US_SWZ_128);
  if (rc) return rc;
  rc = us_tmap_2d(&tmV, v, US_TMAP_BF16, (uint64_t)Tk, (uint64_t)Hkv * D, (uint64_t)ldv, kBN, 64,
                  US_SWZ_128);
  if (rc) return rc;
  Flash2Args a;
  a.cu_q = cu_q;
  a.cu_k = cu_k;
  a.out = (__nv_bfloat16*)out;
  a.ldo = ldo;
  a.Hq = Hq;
  a.Hkv = Hkv;
  a.causal = causal;
  a.scale_log2 = scale * 1.4426950408889634f;
  a.status = us_status_ptr();
  for (int p = 0; p < 8; ++p) a.peer_out[p] = nullptr;
  a.peer_rows = 0;
  a.peer_col0 = 0;
  a.peer_ld = 0;
  if (peer_out) {
    US_REQUIRE(n_seqs == 1 && n_peers >= 1 && n_peers <= 8 && peer_rows >= 1 &&
               (long long)peer_rows * n_peers >= Tq && (peer_ld % 8) == 0 && (peer_col0 % 8) == 0);
    for (int p = 0; p < n_peers; ++p) {
      US_REQUIRE(peer_out[p] && ((uintptr_t)peer_out[p] % 16) == 0);
      a.peer_out[p] = peer_out[p];
    }
    a.peer_rows = peer_rows;
    a.peer_col0 = peer_col0;
    a.peer_ld = peer_ld;
  }
  const size_t smem = 6 * (size_t)(D / 64) * kHalf + 16 * 8 + 16 + 1024;
  static bool configured = false;
  if (!configured) {
    US_CUDA_CHECK(cudaFuncSetAttribute(flash2_fwd_kernel<128>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)(12 * (size_t)kHalf + 16 * 8 + 16 + 1024)));
    US_CUDA_CHECK(cudaFuncSetAttribute(flash2_fwd_kernel<64>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)(6 * (size_t)kHalf + 16 * 8 + 16 + 1024)));
    configured = true;
  }
  dim3 grid((max_q + 2 * kBM - 1) / (2 * kBM), Hq, n_seqs);
  if (D == 128)
    US_CUDA_CHECK(us::launch_pdl(flash2_fwd_kernel<128>, grid, dim3(320), smem, stream, tmQ, tmK,
                                 tmV, a));
  else
    US_CUDA_CHECK(us::launch_pdl(flash2_fwd_kernel<64>, grid, dim3(320), smem, stream, tmQ, tmK,
                                 tmV, a));
  return US_OK;
}

}  // namespace

// Same contract as us_flash_attn_varlen (q [Tq, Hq*128], k/v [Tk, Hkv*128], out
// [Tq, Hq*128], bf16, cu_q/cu_k int32 [n_seqs + 1] on the device).
US_API int us_flash_attn_varlen2(const void* q, const void* k, const void* v, void* out,
                                 const int* cu_q, const int* cu_k, int n_seqs, int Tq, int Tk,
                                 int Hq, int Hkv, int D, int max_q, long long ldq, long long ldk,
                                 long long ldv, long long ldo, float scale, int causal,
                                 void* stream_) {
  return flash2_impl(q, k, v, out, cu_q, cu_k, n_seqs, Tq, Tk, Hq, Hkv, D, max_q, ldq, ldk, ldv,
                     ldo, scale, causal, nullptr, 0, 0, 0, 0, (cudaStream_t)stream_);
}

// One sequence whose output rows are pushed to the ranks that own them (Ulysses
// return fused into the attention epilogue): row r goes to peer_out[r / peer_rows] at
// row r % peer_rows, columns [peer_col0 + h * 128, + 128) of a [peer_rows, peer_ld] buffer.
US_API int us_flash_attn_push(const void* q, const void* k, const void* v, const int* cu_q,
                              const int* cu_k, int Tq, int Tk, int Hq, int Hkv, long long ldq,
                              long long ldk, long long ldv, float scale, void* const* peer_out,
                              int n_peers, int peer_rows, int peer_col0, long long peer_ld,
                              void* stream_) {
  return flash2_impl(q, k, v, nullptr, cu_q, cu_k, 1, Tq, Tk, Hq, Hkv, kDMax, Tq, ldq, ldk, ldv, 8,
                     scale, 0, peer_out, n_peers, peer_rows, peer_col0, peer_ld,
                     (cudaStream_t)stream_);
}
