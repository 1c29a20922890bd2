// Varlen flash attention forward on tcgen05 (head_dim 128, bf16, GQA).
//
// One CTA owns 128 query rows of one (sequence, head) and walks the keys in
// blocks of 128:
//
//   S = Q K^T          tcgen05.mma, Q and K tiles K-major from TMA, S in tensor memory
//                      (two S buffers: the next block's product runs under this block's softmax)
//   softmax            thread r owns row r: reads S with tcgen05.ld, keeps a running maximum
//                      and sum in the log2 domain; the output accumulator in tensor memory is
//                      rescaled (tcgen05.ld / st) only when the maximum grew by more than 2^8
//   P -> shared memory bf16, K-major, 128-byte swizzle (A operand of the second product)
//   O += P V           V tile straight from TMA as the MN-major B operand, O stays in TMEM
//
// Roles: warps 0-3 softmax and epilogue, warp 4 TMA producer, warp 5 TMEM owner
// and MMA issuer.  Causal masks are aligned to the bottom right (query i of a
// sequence sees keys <= i + len_k - len_q), which also serves chunked prefill.
// Every wait is bounded.
//
// Serves the token path's prefill (causal) and the video transformer's long
// bidirectional sequences; the reference runs FlashAttention-4 here
// (crates/ops/kernels/dense_attention/fa4, reference project path).
#include "include/us_common.cuh"
#include "include/us_tc05.cuh"
#include "include/us_tmap.h"

namespace {

constexpr int kD = 128;
constexpr int kBM = 128;   // query rows per CTA
constexpr int kBN = 128;   // keys per block
constexpr int kHalf = 128 * 128;         // bytes of one 64-column half tile (128 rows x 128 B)
constexpr int kTile = 2 * kHalf;         // 32 KiB
constexpr float kRescaleThreshold = 8.f; // log2 units

struct FlashArgs {
  const int* cu_q;
  const int* cu_k;
  __nv_bfloat16* out;
  long long ldo;
  int Hq, Hkv, causal;
  float scale_log2;
  unsigned int* status;
  // Block-sparse form (one sequence of whole 128-row tiles): query tile t of head h
  // reads key blocks indices[(h * q_tiles + t) * sel + 0 .. counts[h * q_tiles + t]);
  // rows of key block b at or past valid[b] are not visible.
  const int* indices;
  const int* counts;
  const int* valid;
  int sel, q_tiles;
  float* lse;   // [heads, rows] natural-log normaliser, or null
};

__device__ __forceinline__ float ex2f(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <bool SPARSE>
__global__ void __launch_bounds__(192, 1)
flash_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const FlashArgs a) {
  US_PDL_PROLOGUE();
  const int q_tile = blockIdx.x, h = blockIdx.y, seq = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, tid = threadIdx.x;
  const int q_start = a.cu_q[seq], q_len = a.cu_q[seq + 1] - q_start;
  const int k_start = a.cu_k[seq], kv_len = a.cu_k[seq + 1] - k_start;
  const int q0 = q_tile * kBM;
  if (q0 >= q_len) return;
  const int hk = h / (a.Hq / a.Hkv);
  const int shift = kv_len - q_len;  // causal: key <= query + shift
  int k_limit = kv_len;
  if (a.causal) k_limit = min(kv_len, q0 + kBM + shift);
  int nblocks = k_limit > 0 ? (k_limit + kBN - 1) / kBN : 0;
  const int* my_blocks = nullptr;
  if (SPARSE) {
    nblocks = min(a.counts[h * a.q_tiles + q_tile], a.sel);
    my_blocks = a.indices + ((long long)h * a.q_tiles + q_tile) * a.sel;
  }

  if (nblocks == 0) {  // no visible key: zeros
    if (tid < kBM && q0 + tid < q_len) {
      uint4* dst = reinterpret_cast<uint4*>(a.out + (long long)(q_start + q0 + tid) * a.ldo +
                                            (long long)h * kD);
      for (int i = 0; i < kD / 8; ++i) dst[i] = make_uint4(0, 0, 0, 0);
      if (SPARSE && a.lse) a.lse[(long long)h * q_len + q0 + tid] = -INFINITY;
    }
    return;
  }

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* sQ = smem;
  uint8_t* sK = smem + kTile;          // two stages
  uint8_t* sV = smem + 3 * kTile;      // two stages
  uint8_t* sP = smem + 5 * kTile;
  uint64_t* bars = (uint64_t*)(smem + 6 * kTile);
  uint64_t* q_full = bars;
  uint64_t* k_full = bars + 1;   // [2]
  uint64_t* k_empty = bars + 3;  // [2]
  uint64_t* v_full = bars + 5;   // [2]
  uint64_t* v_empty = bars + 7;  // [2]
  uint64_t* s_full = bars + 9;   // [2]
  uint64_t* s_empty = bars + 11; // [2]
  uint64_t* p_full = bars + 13;
  uint64_t* o_full = bars + 14;
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
      tc::mbar_init(&s_empty[i], 128);
    }
    tc::mbar_init(p_full, 128);
    tc::mbar_init(o_full, 1);
    *abort_flag = 0;
    tc::mbar_fence_init();
  }
  if (warp == 5) {
    tc::tmem_alloc(tmem_slot, 512);
    tc::tmem_relinquish();
  }
  tc::tc_fence_before_sync();
  __syncthreads();
  tc::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_O = tmem_base + 256;

  if (warp == 4) {
    if (lane == 0) {
      tc::tma_prefetch_desc(&tmQ);
      tc::tma_prefetch_desc(&tmK);
      tc::tma_prefetch_desc(&tmV);
      tc::mbar_expect_tx(q_full, kTile);
      tc::tma_load_2d(sQ, &tmQ, q_full, h * kD, q_start + q0);
      tc::tma_load_2d(sQ + kHalf, &tmQ, q_full, h * kD + 64, q_start + q0);
      for (int j = 0; j < nblocks; ++j) {
        const int st = j & 1;
        const uint32_t ph = (uint32_t)(j >> 1) & 1u;
        const int row = k_start + (SPARSE ? my_blocks[j] : j) * kBN;
        if (!tc::mbar_wait(&k_empty[st], ph ^ 1u, abort_flag)) {
          us_dev_fail(a.status, US_DEV_TIMEOUT_EMPTY);
          *abort_flag = 1;
          break;
        }
        tc::mbar_expect_tx(&k_full[st], kTile);
        tc::tma_load_2d(sK + st * kTile, &tmK, &k_full[st], hk * kD, row);
        tc::tma_load_2d(sK + st * kTile + kHalf, &tmK, &k_full[st], hk * kD + 64, row);
        if (!tc::mbar_wait(&v_empty[st], ph ^ 1u, abort_flag)) {
          us_dev_fail(a.status, US_DEV_TIMEOUT_EMPTY);
          *abort_flag = 1;
          break;
        }
        tc::mbar_expect_tx(&v_full[st], kTile);
        tc::tma_load_2d(sV + st * kTile, &tmV, &v_full[st], hk * kD, row);
        tc::tma_load_2d(sV + st * kTile + kHalf, &tmV, &v_full[st], hk * kD + 64, row);
      }
    }
  } else if (warp == 5) {
    if (lane == 0) {
      constexpr uint32_t kIdescQK = tc::make_idesc(kBM, kBN, tc::kFmtBF16, tc::kFmtBF16, 0, 0);
      constexpr uint32_t kIdescPV = tc::make_idesc(kBM, kD, tc::kFmtBF16, tc::kFmtBF16, 0, 1);
      const uint32_t q_addr = tc::smem_u32(sQ), p_addr = tc::smem_u32(sP);
      auto issue_qk = [&](int j) {
        const uint32_t k_addr = tc::smem_u32(sK + (j & 1) * kTile);
        const uint32_t s_tmem = tmem_base + (uint32_t)(j & 1) * kBN;
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t half = kk >> 2, sub = kk & 3;
          const uint64_t ad = tc::smem_desc_kmajor_sw128(q_addr + half * kHalf) + 2 * sub;
          const uint64_t bd = tc::smem_desc_kmajor_sw128(k_addr + half * kHalf) + 2 * sub;
          tc::umma_f16(s_tmem, ad, bd, kIdescQK, kk != 0);
        }
        tc::umma_commit(&s_full[j & 1]);
        tc::umma_commit(&k_empty[j & 1]);
      };
      bool ok = tc::mbar_wait(q_full, 0, abort_flag) && tc::mbar_wait(&k_full[0], 0, abort_flag);
      if (ok) {
        tc::tc_fence_after_sync();
        issue_qk(0);
      }
      for (int j = 0; ok && j < nblocks; ++j) {
        if (j + 1 < nblocks) {
          const int b = (j + 1) & 1;
          const uint32_t ph = (uint32_t)((j + 1) >> 1) & 1u;
          if (!tc::mbar_wait(&k_full[b], ph, abort_flag) ||
              !tc::mbar_wait(&s_empty[b], ph ^ 1u, abort_flag)) {
            ok = false;
            break;
          }
          tc::tc_fence_after_sync();
          issue_qk(j + 1);
        }
        if (!tc::mbar_wait(&v_full[j & 1], (uint32_t)(j >> 1) & 1u, abort_flag) ||
            !tc::mbar_wait(p_full, (uint32_t)j & 1u, abort_flag)) {
          ok = false;
          break;
        }
        tc::tc_fence_after_sync();
        const uint32_t v_addr = tc::smem_u32(sV + (j & 1) * kTile);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t half = kk >> 2, sub = kk & 3;
          const uint64_t ad = tc::smem_desc_kmajor_sw128(p_addr + half * kHalf) + 2 * sub;
          // B = V: d on N (two 64-wide chunks, 16 KiB apart), 16 keys per
          // instruction = two groups of eight rows (1 KiB apart).
          const uint64_t bd = tc::smem_desc_mnmajor_sw128(v_addr + kk * 2048, kHalf, 1024);
          tc::umma_f16(tmem_O, ad, bd, kIdescPV, (j | kk) != 0);
        }
        tc::umma_commit(o_full);
        tc::umma_commit(&v_empty[j & 1]);
      }
      if (!ok) {
        us_dev_fail(a.status, US_DEV_TIMEOUT_FULL);
        *abort_flag = 1;
      }
    }
  } else {
    // ---- softmax: thread = query row ----
    const int r = tid;
    const uint32_t lane_addr = ((uint32_t)(warp * 32) << 16);
    const int q_idx = q0 + r;
    float m_used = -INFINITY, l_sum = 0.f;
    bool ok = true;
    for (int j = 0; j < nblocks; ++j) {
      const int b = j & 1;
      if (!tc::mbar_wait(&s_full[b], (uint32_t)(j >> 1) & 1u)) { ok = false; break; }
      tc::tc_fence_after_sync();
      const uint32_t s_tmem = tmem_base + (uint32_t)b * kBN + lane_addr;
      const int kbase = j * kBN;
      // keys of this block this row may see: [0, lim)
      int lim = kv_len - kbase;
      if (a.causal) lim = min(lim, q_idx + shift - kbase + 1);
      if (SPARSE) lim = a.valid[my_blocks[j]];
      const bool need_mask = lim < kBN;   // per-thread; the loads below stay uniform
      // The whole row of S goes to registers in one round trip; four independent
      // chains keep the maximum and the sum from serialising on instruction latency.
      uint32_t v0[32], v1[32], v2[32], v3[32];
      tc::tmem_ld32(s_tmem, v0);
      tc::tmem_ld32(s_tmem + 32, v1);
      tc::tmem_ld32(s_tmem + 64, v2);
      tc::tmem_ld32(s_tmem + 96, v3);
      tc::tmem_ld_wait();
      if (need_mask) {
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
      for (int i = 0; i < 32; ++i) {
        mx0 = fmaxf(mx0, __uint_as_float(v0[i]));
        mx1 = fmaxf(mx1, __uint_as_float(v1[i]));
        mx2 = fmaxf(mx2, __uint_as_float(v2[i]));
        mx3 = fmaxf(mx3, __uint_as_float(v3[i]));
      }
      const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
      const float m_new = fmaxf(m_used, mx * a.scale_log2);
      const bool grow = m_new - m_used > kRescaleThreshold;   // -inf start counts as growth
      const bool any_grow = __any_sync(0xffffffffu, grow || (m_used == -INFINITY && m_new > -INFINITY));
      if (j > 0) {
        // P and O are free again once the previous block's second product is done.
        if (!tc::mbar_wait(o_full, (uint32_t)(j - 1) & 1u)) { ok = false; break; }
        tc::tc_fence_after_sync();
      }
      if (any_grow) {
        const float alpha = (m_used == -INFINITY) ? 0.f : ex2f(m_used - m_new);
        if (j > 0) {
#pragma unroll 1
          for (int c = 0; c < kD; c += 32) {
            uint32_t v[32];
            tc::tmem_ld32(tmem_O + lane_addr + c, v);
            tc::tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
            tc::tmem_st32(tmem_O + lane_addr + c, v);
          }
          tc::tmem_st_wait();
        }
        l_sum *= alpha;
        m_used = m_new;
      }
      const float m_eff = (m_used == -INFINITY) ? 0.f : m_used;
      const float neg_m = -m_eff;
      float l0 = 0.f, l1 = 0.f, l2 = 0.f, l3 = 0.f;
      auto exp_chunk = [&](const uint32_t (&v)[32], int c, float& l) {
        uint32_t packed[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const float p0 = ex2f(fmaf(__uint_as_float(v[i]), a.scale_log2, neg_m));
          const float p1 = ex2f(fmaf(__uint_as_float(v[i + 1]), a.scale_log2, neg_m));
          l += p0 + p1;
          __nv_bfloat162 pk = __floats2bfloat162_rn(p0, p1);
          packed[i >> 1] = *reinterpret_cast<uint32_t*>(&pk);
        }
        uint8_t* prow = sP + (c >> 6) * kHalf;
        const int chunk0 = (c & 63) >> 3;
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4)
          *reinterpret_cast<uint4*>(prow + tc::sw128_offset(r, chunk0 + q4)) =
              make_uint4(packed[4 * q4], packed[4 * q4 + 1], packed[4 * q4 + 2],
                         packed[4 * q4 + 3]);
      };
      exp_chunk(v0, 0, l0);
      exp_chunk(v1, 32, l1);
      exp_chunk(v2, 64, l2);
      exp_chunk(v3, 96, l3);
      l_sum += (l0 + l1) + (l2 + l3);
      tc::tc_fence_before_sync();
      tc::mbar_arrive(&s_empty[b]);
      tc::fence_async_smem();
      tc::mbar_arrive(p_full);
    }
    if (ok && tc::mbar_wait(o_full, (uint32_t)(nblocks - 1) & 1u)) {
      tc::tc_fence_after_sync();
      const float inv = l_sum > 0.f ? 1.f / l_sum : 0.f;
      const bool row_ok = q_idx < q_len;
      if (SPARSE && a.lse && row_ok)
        a.lse[(long long)h * q_len + q_idx] =
            l_sum > 0.f ? (m_used + log2f(l_sum)) * 0.6931471805599453f : -INFINITY;
      __nv_bfloat16* orow = a.out + (long long)(q_start + q_idx) * a.ldo + (long long)h * kD;
#pragma unroll 1
      for (int c = 0; c < kD; c += 32) {
        uint32_t v[32];
        tc::tmem_ld32(tmem_O + lane_addr + c, v);
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
  tc::tc_fence_before_sync();
  __syncthreads();
  if (warp == 5) {
    __syncwarp();
    tc::tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace

namespace {

int flash_impl(const void* q, const void* k, const void* v, void* out, const int* cu_q,
               const int* cu_k, int n_seqs, int Tq, int Tk, int Hq, int Hkv, int D, int max_q,
               long long ldq, long long ldk, long long ldv, long long ldo, float scale, int causal,
               const int* indices, const int* counts, const int* valid, int sel, float* lse,
               cudaStream_t stream) {
  US_REQUIRE(q && k && v && out && cu_q && cu_k && n_seqs >= 1 && Tq >= 1 && Tk >= 1);
  US_REQUIRE(D == kD && Hkv >= 1 && Hq % Hkv == 0 && max_q >= 1);
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
  FlashArgs a;
  a.cu_q = cu_q;
  a.cu_k = cu_k;
  a.out = (__nv_bfloat16*)out;
  a.ldo = ldo;
  a.Hq = Hq;
  a.Hkv = Hkv;
  a.causal = causal;
  a.scale_log2 = scale * 1.4426950408889634f;
  a.status = us_status_ptr();
  a.indices = indices;
  a.counts = counts;
  a.valid = valid;
  a.sel = sel;
  a.q_tiles = (max_q + kBM - 1) / kBM;
  a.lse = lse;
  const size_t smem = 6 * (size_t)kTile + 16 * 8 + 16 + 1024;
  static bool configured = false;
  if (!configured) {
    US_CUDA_CHECK(cudaFuncSetAttribute(flash_fwd_kernel<false>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    US_CUDA_CHECK(cudaFuncSetAttribute(flash_fwd_kernel<true>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured = true;
  }
  dim3 grid((max_q + kBM - 1) / kBM, Hq, n_seqs);
  if (indices)
    US_CUDA_CHECK(us::launch_pdl(flash_fwd_kernel<true>, grid, dim3(192), smem, stream, tmQ, tmK,
                                 tmV, a));
  else
    US_CUDA_CHECK(us::launch_pdl(flash_fwd_kernel<false>, grid, dim3(192), smem, stream, tmQ, tmK,
                                 tmV, a));
  return US_OK;
}

}  // namespace

// q [Tq, Hq*128] (row stride ldq), k/v [Tk, Hkv*128] (row strides ldk/ldv), out
// [Tq, Hq*128] (row stride ldo), all bf16; cu_q/cu_k int32 [n_seqs + 1] on the device.
US_API int us_flash_attn_varlen(const void* q, const void* k, const void* v, void* out,
                                const int* cu_q, const int* cu_k, int n_seqs, int Tq, int Tk,
                                int Hq, int Hkv, int D, int max_q, long long ldq, long long ldk,
                                long long ldv, long long ldo, float scale, int causal,
                                void* stream_) {
  return flash_impl(q, k, v, out, cu_q, cu_k, n_seqs, Tq, Tk, Hq, Hkv, D, max_q, ldq, ldk, ldv,
                    ldo, scale, causal, nullptr, nullptr, nullptr, 0, nullptr,
                    (cudaStream_t)stream_);
}

// Block-sparse attention over selected 128-row key blocks (video sparse attention):
// q [Tq, H*128] and k/v [Tk, H*128] in whole 128-row tiles (one sequence; `cu`
// is the int32 pair [0, Tq] / [0, Tk] on the device), indices [H, Tq/128, sel] global
// key-block ids, counts [H, Tq/128], valid [Tk/128] visible rows per key block,
// lse [H, Tq] FP32 (natural log) or null.  A query tile that selects no block writes
// zeros and an lse of -inf.
US_API int us_sparse_attn_block128(const void* q, const void* k, const void* v, void* out,
                                   const int* cu_q, const int* cu_k, int Tq, int Tk, int H,
                                   long long ldq, long long ldk, long long ldv, long long ldo,
                                   float scale, const int* indices, const int* counts,
                                   const int* valid, int sel, float* lse, void* stream_) {
  US_REQUIRE(indices && counts && valid && sel >= 1 && (Tq % kBM) == 0 && (Tk % kBN) == 0);
  return flash_impl(q, k, v, out, cu_q, cu_k, 1, Tq, Tk, H, H, kD, Tq, ldq, ldk, ldv, ldo, scale,
                    0, indices, counts, valid, sel, lse, (cudaStream_t)stream_);
}
