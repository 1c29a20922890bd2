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
#include <mutex>
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
  // Linear launches (one sequence, no mask): CTA i of a launch with kv_parts >= 1 takes work
  // item item0 + i / kv_parts = (query pair, head) with the pair running fastest, and key
  // blocks [part * per, (part + 1) * per) of it.  With kv_parts > 1 the CTA leaves its rows
  // unnormalised in part_o with their maxima and sums in part_ml; flash2_merge_kernel folds
  // the parts.  kv_parts == 0: the (pair, head, sequence) grid.
  int kv_parts, item0, items_x, blocks_per_part;
  float* part_o;    // [CTA][256 rows][kD]
  float* part_ml;   // [CTA][256 rows][2]: running maximum (log2 domain), sum
  int no_wait;      // the launch reads only what the launch before it has waited for
  int tail_follows; // the next launch is this one's tail and has no_wait set
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
__device__ __forceinline__ unsigned long long add2_rm(unsigned long long a, unsigned long long b) {
  unsigned long long d;
  asm("add.rm.ftz.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
// 2^t for a pair of arguments in [-126, 128) on the FMA pipe, for the share of the softmax
// that the special-function unit cannot take: with 128-wide heads a key block costs the
// tensor pipe as many cycles as its 2 x 128 x 128 exponentials cost that unit, so the unit
// is the limit unless part of the work leaves it.  t = n + f with n = floor(t) taken from
// the low mantissa bits of t + 1.5 * 2^23 (rounded down), 2^f by a cubic with 2^0 exact
// (relative error 8.6e-5, far under the bf16 rounding of P), and n added into the exponent
// field.  Arguments below -126 are raised to it (2^-126 rounds to nothing in P and in the
// row sum); the caller keeps -inf (masked keys) on the exact path.
__device__ __forceinline__ void ex2_poly2(float t0, float t1, float& p0, float& p1) {
  const float kMagic = 12582912.f;
  const unsigned long long x = pack2(fmaxf(t0, -126.f), fmaxf(t1, -126.f));
  const unsigned long long tt = add2_rm(x, pack2(kMagic, kMagic));
  const unsigned long long fi = add2(tt, pack2(-kMagic, -kMagic));
  const unsigned long long fr = fma2(fi, pack2(-1.f, -1.f), x);
  unsigned long long p = fma2(fr, pack2(0.07706704f, 0.07706704f), pack2(0.22764499f, 0.22764499f));
  p = fma2(p, fr, pack2(0.69511676f, 0.69511676f));
  p = fma2(p, fr, pack2(1.f, 1.f));
  float q0, q1, u0, u1;
  unpack2(p, q0, q1);
  unpack2(tt, u0, u1);
  p0 = __uint_as_float(__float_as_uint(q0) + (__float_as_uint(u0) << 23));
  p1 = __uint_as_float(__float_as_uint(q1) + (__float_as_uint(u1) << 23));
}
// tcgen05.mma with the shared-memory descriptors given as (low, high) words.  The thread that
// issues the products is a single instruction stream: with 64 cycles of tensor work per
// 128 x 128 x 16 product, a dozen dependent instructions of 64-bit descriptor arithmetic per
// product make the issue the limit.  The high words are constants of the layout and the low
// words (start address in 16-byte units) advance by compile-time offsets, so a product costs
// one 32-bit add per operand.
//
// The whole issuing warp runs the loop and one elected lane executes each tcgen05 instruction:
// addresses, descriptors and loop control are then the same in all lanes, which lets the
// compiler keep them in the uniform datapath where the instruction takes its operands from
// (a single lane inside a divergent branch computes them in vector registers and moves every
// operand of every product across).
__device__ __forceinline__ void umma_f16_words(uint32_t tmem_d, uint32_t a_lo, uint32_t a_hi,
                                               uint32_t b_lo, uint32_t b_hi, uint32_t idesc,
                                               uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p, q;\n"
      ".reg .b64 da, db;\n"
      "mov.b64 da, {%1, %2};\n"
      "mov.b64 db, {%3, %4};\n"
      "setp.ne.b32 p, %6, 0;\n"
      "elect.sync _|q, 0xffffffff;\n"
      "@q tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p;\n"
      "}\n" ::"r"(tmem_d),
      "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_f16_ts_words(uint32_t tmem_d, uint32_t tmem_a, uint32_t b_lo,
                                                  uint32_t b_hi, uint32_t idesc,
                                                  uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p, q;\n"
      ".reg .b64 db;\n"
      "mov.b64 db, {%2, %3};\n"
      "setp.ne.b32 p, %5, 0;\n"
      "elect.sync _|q, 0xffffffff;\n"
      "@q tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, p;\n"
      "}\n" ::"r"(tmem_d),
      "r"(tmem_a), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
      : "memory");
}
// tcgen05.commit by one elected lane of a converged warp.
__device__ __forceinline__ void umma_commit_elect(uint64_t* bar) {
  asm volatile(
      "{\n"
      ".reg .pred q;\n"
      "elect.sync _|q, 0xffffffff;\n"
      "@q tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n"
      "}\n" ::"r"(tc::smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

// kEmu: which of every eight exponential pairs go to the polynomial (bit = pair slot).
// kSplit: threads per query row.  1: a warpgroup per tile, a thread owns a whole row of S
// (128 columns).  2: two warpgroups per tile, a thread owns half a row (64 columns); the two
// threads of a row are in warps with the same number modulo 4 (the same tensor-memory lanes),
// exchange their half-row maxima through shared memory under a 64-thread named barrier and
// keep partial row sums that meet in the epilogue.  Four softmax warps per scheduler instead
// of two hide the latency of the dependent chains (exponential, pack, store) that bound the
// one-thread-per-row form.
// kHalfP (with kSplit == 1): P is handed to the issuing thread in two halves of 64 keys, so
// that O += P V starts on the first half while the second half's exponentials run.
template <int kD, uint32_t kEmu, int kSplit, bool kHalfP>
__global__ void __launch_bounds__((8 * kSplit + 2) * 32, 1)
flash2_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                  const __grid_constant__ CUtensorMap tmV, const Flash2Args a) {
  // A launch that is followed by its own tail launch lets that one start only once every
  // CTA here is past its wait: the tail launch does not wait itself.
  if (a.no_wait) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  } else if (a.tail_follows) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  } else {
    US_PDL_PROLOGUE();
  }
  constexpr int kHalves = kD / 64;          // 64-column (128-byte) slabs per tile
  constexpr int kTile = kHalves * kHalf;    // 32 KiB (head 128) or 16 KiB (head 64)
  // causal: the last query pairs walk the most key blocks; they start first
  int q_pair = a.causal ? (int)gridDim.x - 1 - (int)blockIdx.x : (int)blockIdx.x;
  int h = blockIdx.y, part = 0;
  const int seq = blockIdx.z;
  if (a.kv_parts > 0) {
    const int item = a.item0 + (int)blockIdx.x / a.kv_parts;
    part = (int)blockIdx.x % a.kv_parts;
    q_pair = item % a.items_x;
    h = item / a.items_x;
  }
  const bool partial = a.kv_parts > 1;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, tid = threadIdx.x;
  constexpr int kTmaWarp = 8 * kSplit, kMmaWarp = 8 * kSplit + 1;
  constexpr int kCols = kBN / kSplit;       // columns of S a softmax thread owns
  constexpr int kChunks = kCols / 32;
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
  // this CTA's key blocks are jb, jb + 1, ... (all of them unless the launch splits the keys)
  const int jb = partial ? part * a.blocks_per_part : 0;
  if (partial) {
#pragma unroll
    for (int x = 0; x < 2; ++x) nb_t[x] = max(0, min(nb_t[x] - jb, a.blocks_per_part));
  }
  const int nb = max(nb_t[0], nb_t[1]);

  if (!partial && tid < 2 * kBM) {  // tiles without a visible key: zeros
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
  if (nb == 0) {
    if (partial && tid < 2 * kBM) {   // a part without keys: weight zero in the merge
      const long long prow = (long long)blockIdx.x * (2 * kBM) + tid;
      a.part_ml[prow * 2] = -INFINITY;
      a.part_ml[prow * 2 + 1] = 0.f;
    }
    return;
  }

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* sQ = smem;                  // two tiles
  uint8_t* sK = smem + 2 * kTile;      // two stages
  uint8_t* sV = smem + 4 * kTile;      // two stages
  uint64_t* bars = (uint64_t*)(smem + 6 * kTile);
  // One "full" and one "empty" barrier per key block j (slot j & 1) instead of one per
  // operand: kv_full[j & 1] counts the bytes of V(j) and K(j + 1), which the producer loads
  // back to back and the issuing thread needs back to back (O += P V(j), then S = Q K(j+1)^T);
  // kv_empty[j & 1], committed once after the block's four products, frees V stage j & 1
  // and K stage (j + 1) & 1 together.  K(0) arrives with Q.  The issuing thread is a single
  // instruction stream that the tensor pipe waits for: every wait and commit it does not
  // execute is tensor time.
  uint64_t* q_full = bars;
  uint64_t* kv_full = bars + 1;   // [2]
  uint64_t* kv_empty = bars + 3;  // [2]
  uint64_t* s_full = bars + 9;   // [2] per tile
  uint64_t* p_full = bars + 11;  // [2] per tile
  uint64_t* p_second = bars + 5; // [2] per tile: the second half of P (kHalfP)
  uint64_t* o_full = bars + 13;  // [2] per tile
  uint32_t* tmem_slot = (uint32_t*)(bars + 15);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  // kSplit == 2: half-row maxima [slot j & 1][tile][half][row], then partial sums [tile][half][row]
  float* xch_max = (float*)(bars + 18);
  float* xch_sum = xch_max + 2 * 2 * 2 * kBM;

  if (tid == 0) {
    tc::mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      tc::mbar_init(&kv_full[i], 1);
      tc::mbar_init(&kv_empty[i], 1);
      tc::mbar_init(&s_full[i], 1);
      tc::mbar_init(&p_full[i], 128 * kSplit);
      tc::mbar_init(&p_second[i], 128 * kSplit);
      tc::mbar_init(&o_full[i], 1);
    }
    *abort_flag = 0;
    tc::mbar_fence_init();
  }
  if (warp == kMmaWarp) {
    tc::tmem_alloc(tmem_slot, 512);
    tc::tmem_relinquish();
  }
  tc::tc_fence_before_sync();
  __syncthreads();
  tc::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == kTmaWarp) {
    if (lane == 0) {
      tc::tma_prefetch_desc(&tmQ);
      tc::tma_prefetch_desc(&tmK);
      tc::tma_prefetch_desc(&tmV);
      tc::mbar_expect_tx(q_full, 3 * kTile);
#pragma unroll
      for (int x = 0; x < 2; ++x) {
        const int row = q_start + q0 + x * kBM;   // rows past the tensor read as zeros
#pragma unroll
        for (int hf = 0; hf < kHalves; ++hf)
          tc::tma_load_2d(sQ + x * kTile + hf * kHalf, &tmQ, q_full, h * kD + 64 * hf, row);
      }
#pragma unroll
      for (int hf = 0; hf < kHalves; ++hf)
        tc::tma_load_2d(sK + hf * kHalf, &tmK, q_full, hk * kD + 64 * hf, k_start + jb * kBN);
      for (int j = 0; j < nb; ++j) {
        const int st = j & 1;
        const bool more = j + 1 < nb;
        // kv_empty[0] completes after blocks 0, 2, 4 ..., kv_empty[1] after the first S
        // products (which read K stage 0, the stage K(2) goes to) and after blocks 1, 3, ...:
        // block j waits for completion number (j + 1) / 2 of its slot, none for block 0
        if (!tc::mbar_wait(&kv_empty[st], ((uint32_t)((j + 1) >> 1) & 1u) ^ 1u, abort_flag)) {
          us_dev_fail(a.status, US_DEV_TIMEOUT_EMPTY);
          *abort_flag = 1;
          break;
        }
        tc::mbar_expect_tx(&kv_full[st], more ? 2 * kTile : kTile);
#pragma unroll
        for (int hf = 0; hf < kHalves; ++hf)
          tc::tma_load_2d(sV + st * kTile + hf * kHalf, &tmV, &kv_full[st], hk * kD + 64 * hf,
                          k_start + (jb + j) * kBN);
        if (more) {
#pragma unroll
          for (int hf = 0; hf < kHalves; ++hf)
            tc::tma_load_2d(sK + (st ^ 1) * kTile + hf * kHalf, &tmK, &kv_full[st],
                            hk * kD + 64 * hf, k_start + (jb + j + 1) * kBN);
        }
      }
    }
  } else if (warp == kMmaWarp) {
    {   // all 32 lanes, converged; single lanes are elected per instruction
      // every lane waits; the vote makes the outcome (and the control flow) the same in all
      auto warp_wait = [&](uint64_t* bar, uint32_t parity, volatile uint32_t* abort) -> bool {
        return __all_sync(0xffffffffu, tc::mbar_wait(bar, parity, abort));
      };
      constexpr uint32_t kIdescQK = tc::make_idesc(kBM, kBN, tc::kFmtBF16, tc::kFmtBF16, 0, 0);
      constexpr uint32_t kIdescPV = tc::make_idesc(kBM, kD, tc::kFmtBF16, tc::kFmtBF16, 0, 1);
      // descriptor words of the operands: Q tiles and K stages K-major, V stages MN-major
      const uint64_t dq = tc::smem_desc_kmajor_sw128(tc::smem_u32(sQ));
      const uint64_t dk = tc::smem_desc_kmajor_sw128(tc::smem_u32(sK));
      const uint64_t dv = tc::smem_desc_mnmajor_sw128(tc::smem_u32(sV), kHalf, 1024);
      const uint32_t q_lo = (uint32_t)dq, k_lo = (uint32_t)dk, v_lo = (uint32_t)dv;
      const uint32_t km_hi = (uint32_t)(dq >> 32), mn_hi = (uint32_t)(dv >> 32);
      auto issue_qk = [&](int x, int j) {
        const uint32_t qa = q_lo + (uint32_t)x * (kTile >> 4);
        const uint32_t kb = k_lo + (uint32_t)(j & 1) * (kTile >> 4);
        const uint32_t s_tmem = tmem_base + (uint32_t)x * kBN;
#pragma unroll
        for (int kk = 0; kk < kD / 16; ++kk) {
          const uint32_t off = (uint32_t)(kk >> 2) * (kHalf >> 4) + 2u * (uint32_t)(kk & 3);
          umma_f16_words(s_tmem, qa + off, km_hi, kb + off, km_hi, kIdescQK, kk != 0);
        }
        umma_commit_elect(&s_full[x]);
      };
      auto issue_pv = [&](int x, int j) -> bool {
        const uint32_t vb = v_lo + (uint32_t)(j & 1) * (kTile >> 4);
        const uint32_t p_tmem = tmem_base + (uint32_t)x * kBN;
        const uint32_t o_tmem = tmem_base + 256 + (uint32_t)x * kD;
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          if (kHalfP && kk == 4) {   // the second half of P
            if (!warp_wait(&p_second[x], (uint32_t)j & 1u, abort_flag)) return false;
            tc::tc_fence_after_sync();
          }
          // A = P: 16 keys = 8 packed columns per instruction.  B = V: d on N (two
          // 64-wide chunks, 16 KiB apart), 16 keys = two groups of eight rows (1 KiB apart),
          // 2 KiB further per instruction.
          // kSplit == 2 keeps the P of every 32 keys in the first 16 columns of their own S
          const uint32_t p_col = kSplit == 2 ? (kk >> 1) * 32 + (kk & 1) * 8 : kk * 8;
          umma_f16_ts_words(o_tmem, p_tmem + p_col, vb + (uint32_t)kk * (2048 >> 4), mn_hi,
                            kIdescPV, (j | kk) != 0);
        }
        // a tile's accumulator is waited for only after its last block: before that, the next
        // S of the tile (issued after this product, committed to s_full) says the same
        if (j == nb_t[x] - 1) umma_commit_elect(&o_full[x]);
        return true;
      };
      bool ok = warp_wait(q_full, 0, abort_flag);
      if (ok) {
        tc::tc_fence_after_sync();
        if (nb_t[0] > 0) issue_qk(0, 0);
        if (nb_t[1] > 0) issue_qk(1, 0);
        umma_commit_elect(&kv_empty[1]);   // K stage 0 may be refilled (with K(2), by block 1's loads)
      }
      for (int j = 0; ok && j < nb; ++j) {
        const uint32_t pj = (uint32_t)j & 1u;
        // V(j) and K(j + 1) are there
        if (!warp_wait(&kv_full[j & 1], (uint32_t)(j >> 1) & 1u, abort_flag)) { ok = false; break; }
        // tile A: O_A += P_A V_j, then S_A of the next block
        if (j < nb_t[0]) {
          if (!warp_wait(&p_full[0], pj, abort_flag)) { ok = false; break; }
          tc::tc_fence_after_sync();
          if (!issue_pv(0, j)) { ok = false; break; }
          if (j + 1 < nb_t[0]) issue_qk(0, j + 1);
        }
        // tile B
        if (j < nb_t[1]) {
          if (!warp_wait(&p_full[1], pj, abort_flag)) { ok = false; break; }
          tc::tc_fence_after_sync();
          if (!issue_pv(1, j)) { ok = false; break; }
          if (j + 1 < nb_t[1]) issue_qk(1, j + 1);
        }
        umma_commit_elect(&kv_empty[j & 1]);
      }
      if (!ok && lane == 0) {
        us_dev_fail(a.status, US_DEV_TIMEOUT_FULL);
        *abort_flag = 1;
      }
    }
  } else {
    // ---- softmax: tile = warp / (4 kSplit), thread = query row (or half of one) ----
    const int x = warp / (4 * kSplit);
    const int hx = kSplit == 2 ? (warp >> 2) & 1 : 0;   // which half of the row's columns
    const int r = (warp & 3) * 32 + lane;
    const int nbx = nb_t[x];
    const int col0 = hx * kCols;
    const uint32_t lane_addr = ((uint32_t)((warp & 3) * 32) << 16);
    const uint32_t s_tmem = tmem_base + (uint32_t)x * kBN + lane_addr;
    const uint32_t o_tmem = tmem_base + 256 + (uint32_t)x * kD + lane_addr;
    const int q_idx = q0 + x * kBM + r;
    const uint32_t pair_bar = 1u + (uint32_t)x * 4u + (uint32_t)(warp & 3);   // the row's two warps
    auto pair_sync = [&]() { asm volatile("bar.sync %0, 64;" ::"r"(pair_bar) : "memory"); };
    float m_used = -INFINITY, l_sum = 0.f;
    bool ok = true;
    for (int j = 0; j < nbx; ++j) {
      // A warp that gave up keeps meeting its partner at the pair barrier (once per block and
      // once after the loop), so that the other warp of the row is never left waiting there.
      if (ok) ok = __all_sync(0xffffffffu, tc::mbar_wait(&s_full[x], (uint32_t)j & 1u, abort_flag));
      if (!ok) {
        if (kSplit == 2) pair_sync();
        continue;
      }
      tc::tc_fence_after_sync();
      const int kbase = (jb + j) * kBN + col0;
      int lim = kv_len - kbase;   // keys of this thread's columns this row may see: [0, lim)
      if (a.causal) lim = min(lim, q_idx + shift - kbase + 1);
      const bool need_mask = lim < kCols;
      const unsigned long long sc2 = pack2(a.scale_log2, a.scale_log2);
      auto exp_pair = [&](uint32_t x0, uint32_t x1, unsigned long long nm2, unsigned long long& l,
                          bool poly) -> uint32_t {
        float t0, t1, p0, p1;
        unpack2(fma2(pack2(__uint_as_float(x0), __uint_as_float(x1)), sc2, nm2), t0, t1);
        if (poly) {
          ex2_poly2(t0, t1, p0, p1);
        } else {
          p0 = ex2f(t0);
          p1 = ex2f(t1);
        }
        l = add2(l, pack2(p0, p1));
        __nv_bfloat162 t = __floats2bfloat162_rn(p0, p1);
        return *reinterpret_cast<uint32_t*>(&t);
      };
      if constexpr (kSplit == 2) {
        // Half a row in two chunks of 32 columns.  Pass 1 takes the maximum of both chunks and
        // keeps the second in registers; after the exchange with the other half of the row,
        // pass 2 turns the second chunk into P, reads the first again from tensor memory and
        // does the same.  At most one chunk of S and one of P are live: the thread fits the
        // 96 registers that 18 warps leave it.  The P of a chunk goes over the first 16
        // columns of that chunk's own S, so no thread writes where another still reads.
        uint32_t v[32];
        auto chunk_max = [&](int c) -> float {
          if (need_mask) {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (32 * c + i >= lim) v[i] = 0xff800000u;
          }
          float m0 = -INFINITY, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            m0 = max3(m0, __uint_as_float(v[i]), __uint_as_float(v[i + 1]));
            m1 = max3(m1, __uint_as_float(v[i + 2]), __uint_as_float(v[i + 3]));
            m2 = max3(m2, __uint_as_float(v[i + 4]), __uint_as_float(v[i + 5]));
            m3 = max3(m3, __uint_as_float(v[i + 6]), __uint_as_float(v[i + 7]));
          }
          return fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
        };
        tc::tmem_ld32(s_tmem + col0, v);
        tc::tmem_ld_wait();
        float mx = chunk_max(0);
        tc::tmem_ld32(s_tmem + col0 + 32, v);
        tc::tmem_ld_wait();
        mx = fmaxf(mx, chunk_max(1));
        {
          // the other half's maximum; slot j & 1 is rewritten at j + 2, after the barrier of
          // j + 1 that both threads pass once they have read slot j
          float* slot = xch_max + ((j & 1) * 4 + x * 2) * kBM;
          slot[hx * kBM + r] = mx;
          pair_sync();
          mx = fmaxf(mx, slot[(hx ^ 1) * kBM + r]);
        }
        const float m_new = fmaxf(m_used, mx * a.scale_log2);
        const bool grow = m_new - m_used > kRescaleThreshold;
        const bool any_grow =
            __any_sync(0xffffffffu, grow || (m_used == -INFINITY && m_new > -INFINITY));
        if (any_grow) {
          const float alpha = (m_used == -INFINITY) ? 0.f : ex2f(m_used - m_new);
          if (j > 0) {
            // O_X is stable: this block's S was issued after the previous block's second
            // product by the same thread, and the commit that filled s_full covers both.
#pragma unroll 1
            for (int c = hx * (kD / 2); c < (hx + 1) * (kD / 2); c += 16) {
              uint32_t w[16];
              tc::tmem_ld16(o_tmem + c, w);
              tc::tmem_ld_wait();
#pragma unroll
              for (int i = 0; i < 16; ++i) w[i] = __float_as_uint(__uint_as_float(w[i]) * alpha);
              tc::tmem_st16(o_tmem + c, w);
            }
          }
          l_sum *= alpha;
          m_used = m_new;
        }
        const float neg_m = (m_used == -INFINITY) ? 0.f : -m_used;
        const unsigned long long nm2 = pack2(neg_m, neg_m);
        const bool poly_ok = kEmu != 0 && !__any_sync(0xffffffffu, need_mask);
        unsigned long long la = pack2(0.f, 0.f), lb = la;
        auto chunk_exp = [&](int c) {
          uint32_t pk[16];
          if (poly_ok) {
#pragma unroll
            for (int i = 0; i < 32; i += 4) {
              pk[i >> 1] = exp_pair(v[i], v[i + 1], nm2, la, (kEmu >> ((i >> 1) & 7)) & 1u);
              pk[(i >> 1) + 1] = exp_pair(v[i + 2], v[i + 3], nm2, lb, (kEmu >> (((i >> 1) + 1) & 7)) & 1u);
            }
          } else {
#pragma unroll
            for (int i = 0; i < 32; i += 4) {
              pk[i >> 1] = exp_pair(v[i], v[i + 1], nm2, la, false);
              pk[(i >> 1) + 1] = exp_pair(v[i + 2], v[i + 3], nm2, lb, false);
            }
          }
          tc::tmem_st16(s_tmem + col0 + 32 * c, pk);
        };
        chunk_exp(1);
        tc::tmem_ld32(s_tmem + col0, v);
        tc::tmem_ld_wait();
        if (need_mask) {
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (i >= lim) v[i] = 0xff800000u;
        }
        chunk_exp(0);
        {
          float s0, s1;
          unpack2(add2(la, lb), s0, s1);
          l_sum += s0 + s1;
        }
      } else {
        // The thread's columns of S go to registers in one round trip; four independent
        // chains keep the maximum and the sum from serialising on instruction latency.
        uint32_t v[kCols];
  #pragma unroll
        for (int c = 0; c < kChunks; ++c) tc::tmem_ld32(s_tmem + col0 + 32 * c, *reinterpret_cast<uint32_t(*)[32]>(v + 32 * c));
        tc::tmem_ld_wait();
        if (need_mask) {   // last key block of the sequence or the causal diagonal
  #pragma unroll
          for (int i = 0; i < kCols; ++i)
            if (i >= lim) v[i] = 0xff800000u;
        }
        float mxs[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
  #pragma unroll
        for (int i = 0; i < 32; i += 2) {
  #pragma unroll
          for (int c = 0; c < kChunks; ++c) {
            const int ch = kChunks == 4 ? c : c * 2 + ((i >> 1) & 1);
            mxs[ch] = max3(mxs[ch], __uint_as_float(v[32 * c + i]), __uint_as_float(v[32 * c + i + 1]));
          }
        }
        float mx = fmaxf(fmaxf(mxs[0], mxs[1]), fmaxf(mxs[2], mxs[3]));
        const float m_new = fmaxf(m_used, mx * a.scale_log2);
        const bool grow = m_new - m_used > kRescaleThreshold;
        const bool any_grow =
            __any_sync(0xffffffffu, grow || (m_used == -INFINITY && m_new > -INFINITY));
        if (any_grow) {
          const float alpha = (m_used == -INFINITY) ? 0.f : ex2f(m_used - m_new);
          if (j > 0) {
            // O_X is stable: this block's S was issued after the previous block's second
            // product by the same thread, and the commit that filled s_full covers both.
  #pragma unroll 1
            for (int c = hx * (kD / kSplit); c < (hx + 1) * (kD / kSplit); c += 32) {
              uint32_t w[32];
              tc::tmem_ld32(o_tmem + c, w);
              tc::tmem_ld_wait();
  #pragma unroll
              for (int i = 0; i < 32; ++i) w[i] = __float_as_uint(__uint_as_float(w[i]) * alpha);
              tc::tmem_st32(o_tmem + c, w);
            }
          }
          l_sum *= alpha;
          m_used = m_new;
        }
        const float m_eff = (m_used == -INFINITY) ? 0.f : m_used;
        const float neg_m = -m_eff;
        const unsigned long long nm2 = pack2(neg_m, neg_m);
        unsigned long long ls[4];
  #pragma unroll
        for (int c = 0; c < 4; ++c) ls[c] = pack2(0.f, 0.f);
        uint32_t pk[kCols / 2];
        if constexpr (kHalfP && kSplit == 1) {
          // keys 0 - 63 first: their P is stored and announced, then keys 64 - 127
  #pragma unroll
          for (int i = 0; i < 32; i += 2) {
  #pragma unroll
            for (int c = 0; c < 2; ++c)
              pk[16 * c + (i >> 1)] = exp_pair(v[32 * c + i], v[32 * c + i + 1], nm2,
                                               ls[c * 2 + ((i >> 1) & 1)], false);
          }
          tc::tmem_st32(s_tmem, *reinterpret_cast<const uint32_t(*)[32]>(pk));
          tc::tmem_st_wait();
          tc::tc_fence_before_sync();
          tc::mbar_arrive(&p_full[x]);
  #pragma unroll
          for (int i = 0; i < 32; i += 2) {
  #pragma unroll
            for (int c = 2; c < 4; ++c)
              pk[16 * c + (i >> 1)] = exp_pair(v[32 * c + i], v[32 * c + i + 1], nm2,
                                               ls[(c - 2) * 2 + ((i >> 1) & 1)], false);
          }
        } else
        // Blocks with masked keys (-inf scores) stay on the exact path, whole warps at a time.
        if (kEmu != 0 && !__any_sync(0xffffffffu, need_mask)) {
  #pragma unroll
          for (int i = 0; i < 32; i += 2) {
  #pragma unroll
            for (int c = 0; c < kChunks; ++c) {
              const int ch = kChunks == 4 ? c : c * 2 + ((i >> 1) & 1);
              const int slot8 = kChunks == 4 ? ((i >> 1) & 1) * 4 + c : ((i >> 1) & 3) * 2 + c;
              pk[16 * c + (i >> 1)] =
                  exp_pair(v[32 * c + i], v[32 * c + i + 1], nm2, ls[ch], (kEmu >> slot8) & 1u);
            }
          }
        } else {
  #pragma unroll
          for (int i = 0; i < 32; i += 2) {
  #pragma unroll
            for (int c = 0; c < kChunks; ++c) {
              const int ch = kChunks == 4 ? c : c * 2 + ((i >> 1) & 1);
              pk[16 * c + (i >> 1)] = exp_pair(v[32 * c + i], v[32 * c + i + 1], nm2, ls[ch], false);
            }
          }
        }
        {
          float s0, s1;
          unpack2(add2(add2(ls[0], ls[1]), add2(ls[2], ls[3])), s0, s1);
          l_sum += s0 + s1;
        }
        // P (packed pairs) replaces the first half of S, which is in registers by now.
  #pragma unroll
        for (int c = (kHalfP && kSplit == 1) ? 1 : 0; c < kChunks / 2; ++c)
          tc::tmem_st32(s_tmem + col0 / 2 + 32 * c, *reinterpret_cast<const uint32_t(*)[32]>(pk + 32 * c));
      }
      tc::tmem_st_wait();
      tc::tc_fence_before_sync();
      if (kHalfP) {
        if (kSplit != 1) tc::mbar_arrive(&p_full[x]);
        tc::mbar_arrive(&p_second[x]);
      } else {
        tc::mbar_arrive(&p_full[x]);
      }
    }
    if (nbx > 0) {
      if (kSplit == 2) {   // the row's sum: both halves
        float* sums = xch_sum + x * 2 * kBM;
        sums[hx * kBM + r] = l_sum;
        pair_sync();
        l_sum += sums[(hx ^ 1) * kBM + r];
      }
      if (ok && tc::mbar_wait(&o_full[x], 0, abort_flag)) {
        tc::tc_fence_after_sync();
        bool continue_epilogue = true;
        if (partial) {
          // unnormalised rows of this part of the keys, with the row's maximum and sum
          const long long prow = (long long)blockIdx.x * (2 * kBM) + x * kBM + r;
          float* po = a.part_o + prow * kD;
          if (hx == 0) {
            a.part_ml[prow * 2] = m_used;
            a.part_ml[prow * 2 + 1] = l_sum;
          }
#pragma unroll 1
          for (int c = hx * (kD / kSplit); c < (hx + 1) * (kD / kSplit); c += 32) {
            uint32_t w[32];
            tc::tmem_ld32(o_tmem + c, w);
            tc::tmem_ld_wait();
#pragma unroll
            for (int q4 = 0; q4 < 8; ++q4)
              *reinterpret_cast<uint4*>(po + c + q4 * 4) =
                  make_uint4(w[q4 * 4], w[q4 * 4 + 1], w[q4 * 4 + 2], w[q4 * 4 + 3]);
          }
          continue_epilogue = false;
        }
        const float inv = l_sum > 0.f ? 1.f / l_sum : 0.f;
        const bool row_ok = q_idx < q_len && continue_epilogue;
        __nv_bfloat16* orow = a.out + (long long)(q_start + q_idx) * a.ldo + (long long)h * kD;
        if (a.peer_rows > 0) {
          const int row = q_start + q_idx;
          const int p = row / a.peer_rows;
          orow = (__nv_bfloat16*)a.peer_out[p] + (long long)(row - p * a.peer_rows) * a.peer_ld +
                 a.peer_col0 + (long long)h * kD;
        }
#pragma unroll 1
        for (int c = hx * (kD / kSplit); continue_epilogue && c < (hx + 1) * (kD / kSplit); c += 32) {
          uint32_t w[32];
          tc::tmem_ld32(o_tmem + c, w);
          tc::tmem_ld_wait();
          if (row_ok) {
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4) {
              us::Pack16 o;
#pragma unroll
              for (int i = 0; i < 8; ++i) o.b[i] = us::f2bf(__uint_as_float(w[q4 * 8 + i]) * inv);
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
  if (warp == kMmaWarp) {
    __syncwarp();
    tc::tmem_dealloc(tmem_base, 512);
  }
}

// Folds the parts of a key-split tail launch: row r of work item i has `parts` unnormalised
// partial rows (CTA i * parts + p of the tail launch) with maxima m_p and sums l_p;
// out = sum_p 2^(m_p - M) O_p / sum_p 2^(m_p - M) l_p.  A thread owns eight channels of a row.
__global__ void __launch_bounds__(128)
flash2_merge_kernel(const Flash2Args a, int parts, int kD) {
  const int item_local = blockIdx.x;
  const int item = a.item0 + item_local;
  const int q_pair = item % a.items_x, h = item / a.items_x;
  const int chunks = kD / 8;                       // threads per row
  const int rows_per_cta = 128 / chunks;
  const int r = blockIdx.y * rows_per_cta + (int)threadIdx.x / chunks;   // row of the pair
  const int c = ((int)threadIdx.x % chunks) * 8;
  const int q_len = a.cu_q[1] - a.cu_q[0];
  const int q_idx = q_pair * 2 * kBM + r;
  if (r >= 2 * kBM || q_idx >= q_len) return;
  float M = -INFINITY;
  for (int p = 0; p < parts; ++p)
    M = fmaxf(M, a.part_ml[((long long)(item_local * parts + p) * (2 * kBM) + r) * 2]);
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f}, den = 0.f;
  for (int p = 0; p < parts; ++p) {
    const long long prow = (long long)(item_local * parts + p) * (2 * kBM) + r;
    const float m = a.part_ml[prow * 2], l = a.part_ml[prow * 2 + 1];
    const float wgt = (m == -INFINITY) ? 0.f : exp2f(m - M);
    den += wgt * l;
    const float4 v0 = *reinterpret_cast<const float4*>(a.part_o + prow * kD + c);
    const float4 v1 = *reinterpret_cast<const float4*>(a.part_o + prow * kD + c + 4);
    acc[0] += wgt * v0.x; acc[1] += wgt * v0.y; acc[2] += wgt * v0.z; acc[3] += wgt * v0.w;
    acc[4] += wgt * v1.x; acc[5] += wgt * v1.y; acc[6] += wgt * v1.z; acc[7] += wgt * v1.w;
  }
  const float inv = den > 0.f ? 1.f / den : 0.f;
  const int row = a.cu_q[0] + q_idx;
  __nv_bfloat16* orow = a.out + (long long)row * a.ldo + (long long)h * kD;
  if (a.peer_rows > 0) {
    const int p = row / a.peer_rows;
    orow = (__nv_bfloat16*)a.peer_out[p] + (long long)(row - p * a.peer_rows) * a.peer_ld +
           a.peer_col0 + (long long)h * kD;
  }
  us::Pack16 o;
#pragma unroll
  for (int i = 0; i < 8; ++i) o.b[i] = us::f2bf(acc[i] * inv);
  *reinterpret_cast<uint4*>(orow + c) = o.u;
}

}  // namespace

namespace {

// Scratch of the key-split tail launch (at most one wave of CTAs), one per stream that used it.
struct TailScratch {
  cudaStream_t stream;
  float* part_o;
  float* part_ml;
};
constexpr int kTailStreams = 8;
constexpr int kTailCtas = 160;

bool tail_scratch(cudaStream_t stream, float** part_o, float** part_ml) {
  static TailScratch table[kTailStreams] = {};
  static int used = 0;
  static std::mutex lock;                  // launches may come from several host threads
  std::lock_guard<std::mutex> guard(lock);
  for (int i = 0; i < used; ++i)
    if (table[i].stream == stream) {
      *part_o = table[i].part_o;
      *part_ml = table[i].part_ml;
      return true;
    }
  if (used == kTailStreams) return false;
  cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(stream, &cap) != cudaSuccess || cap != cudaStreamCaptureStatusNone)
    return false;                       // no allocation inside a graph capture
  float *po = nullptr, *pm = nullptr;
  if (cudaMalloc(&po, (size_t)kTailCtas * 2 * kBM * kDMax * sizeof(float)) != cudaSuccess) return false;
  if (cudaMalloc(&pm, (size_t)kTailCtas * 2 * kBM * 2 * sizeof(float)) != cudaSuccess) {
    cudaFree(po);
    return false;
  }
  table[used++] = {stream, po, pm};
  *part_o = po;
  *part_ml = pm;
  return true;
}

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
  // barriers and flags (18 words), half-row maxima (2 x 2 x 2 x 128 floats) and sums (2 x 2 x 128)
  constexpr size_t kTail = 18 * 8 + (8 + 4) * kBM * sizeof(float) + 1024;
  const size_t smem = 6 * (size_t)(D / 64) * kHalf + kTail;
  // Share of the exponentials computed by the polynomial (US_FLASH_EMU = 0, 2, 3 or 4 of
  // every 8 pairs) and threads per query row (US_FLASH_SPLIT = 1 or 2).
  static const int emu = [] {
    const char* e = getenv("US_FLASH_EMU");
    const int v = e ? atoi(e) : 0;
    return (v == 0 || v == 2 || v == 3 || v == 4) ? v : 0;
  }();
  static const int emu64 = [] {
    const char* e = getenv("US_FLASH_EMU64");
    const int v = e ? atoi(e) : 2;     // a quarter: 4.78 -> 4.44 ms at 20,164 rows x 32 heads
    return (v == 0 || v == 2 || v == 4) ? v : 2;
  }();
  static const int split = [] {
    const char* e = getenv("US_FLASH_SPLIT");
    return (e && atoi(e) == 2) ? 2 : 1;
  }();
  const int smem128 = (int)(12 * (size_t)kHalf + kTail);
  const int smem64 = (int)(6 * (size_t)kHalf + kTail);
#define US_FLASH2_LAUNCH4(DD, MASK, SP, HP)                                                        \
  do {                                                                                          \
    static bool configured = false;                                                             \
    if (!configured) {                                                                          \
      US_CUDA_CHECK(cudaFuncSetAttribute(flash2_fwd_kernel<DD, MASK, SP, HP>,                   \
                                         cudaFuncAttributeMaxDynamicSharedMemorySize,           \
                                         DD == 128 ? smem128 : smem64));                        \
      configured = true;                                                                        \
    }                                                                                           \
    US_CUDA_CHECK(us::launch_pdl(flash2_fwd_kernel<DD, MASK, SP, HP>, grid,                     \
                                 dim3((8 * SP + 2) * 32), smem, stream, tmQ, tmK, tmV, aa));    \
  } while (0)
#define US_FLASH2_LAUNCH(DD, MASK, SP) US_FLASH2_LAUNCH4(DD, MASK, SP, false)
  static const bool half_p = [] {
    const char* e = getenv("US_FLASH_PHALF");
    return e && e[0] == '1';
  }();
  auto launch = [&](dim3 grid, const Flash2Args& aa) -> int {
    if (D == 128 && split == 1 && emu == 0 && half_p) {
      US_FLASH2_LAUNCH4(128, 0x00u, 1, true);
    } else if (D == 128 && split == 2) {
      if (emu == 0) US_FLASH2_LAUNCH(128, 0x00u, 2);
      else if (emu == 2) US_FLASH2_LAUNCH(128, 0x21u, 2);
      else if (emu == 3) US_FLASH2_LAUNCH(128, 0x29u, 2);
      else US_FLASH2_LAUNCH(128, 0xA5u, 2);
    } else if (D == 128) {
      if (emu == 0) US_FLASH2_LAUNCH(128, 0x00u, 1);
      else US_FLASH2_LAUNCH(128, 0x21u, 1);
    } else if (split == 2) {
      if (emu == 0) US_FLASH2_LAUNCH(64, 0x00u, 2);
      else US_FLASH2_LAUNCH(64, 0xA5u, 2);
    } else {
      // 64-wide heads: half the tensor work per exponential, so the special-function unit is
      // the limit by a factor of two and a polynomial share pays (emu64: US_FLASH_EMU64)
      if (emu64 == 0) US_FLASH2_LAUNCH(64, 0x00u, 1);
      else if (emu64 == 2) US_FLASH2_LAUNCH(64, 0x21u, 1);
      else US_FLASH2_LAUNCH(64, 0xA5u, 1);
    }
    return US_OK;
  };
  a.kv_parts = 0;
  a.item0 = 0;
  a.items_x = 0;
  a.blocks_per_part = 0;
  a.part_o = nullptr;
  a.part_ml = nullptr;
  a.no_wait = 0;
  a.tail_follows = 0;
  const int q_pairs = (max_q + 2 * kBM - 1) / (2 * kBM);
  // One sequence without a mask whose (pair, head) items leave a last wave at most half
  // full: that wave's items are split over the keys so that they fill the GPU, and merged.
  // (A rank of an 8-way Ulysses group has 152 pairs x 7 heads = 7.2 waves of 148 CTAs.)
  static const bool tail_on = [] {
    const char* e = getenv("US_FLASH_TAIL");
    return !(e && e[0] == '0');
  }();
  static const int sms = [] {
    int dev = 0, n = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    return n > 0 ? n : 148;
  }();
  if (tail_on && n_seqs == 1 && !causal && max_q == Tq) {
    const int total = q_pairs * Hq;
    const int full = (total / sms) * sms, tail = total - full;
    const int nb = (Tk + kBN - 1) / kBN;
    if (full > 0 && tail > 0 && 2 * tail <= sms && nb >= 8) {
      int parts = sms / tail;
      if (parts > 8) parts = 8;
      if (parts > nb / 4) parts = nb / 4;
      const int per = (nb + parts - 1) / parts;
      parts = (nb + per - 1) / per;
      float *po = nullptr, *pm = nullptr;
      if (parts >= 2 && tail * parts <= kTailCtas && tail_scratch(stream, &po, &pm)) {
        Flash2Args a1 = a;
        a1.kv_parts = 1;
        a1.items_x = q_pairs;
        a1.tail_follows = 1;
        int rc1 = launch(dim3(full), a1);
        if (rc1) return rc1;
        Flash2Args a2 = a;
        a2.kv_parts = parts;
        a2.item0 = full;
        a2.items_x = q_pairs;
        a2.blocks_per_part = per;
        a2.part_o = po;
        a2.part_ml = pm;
        a2.no_wait = 1;
        rc1 = launch(dim3(tail * parts), a2);
        if (rc1) return rc1;
        // plain stream order: everything before it in the stream is complete and visible
        const int rows_per_cta = 128 / (D / 8);
        flash2_merge_kernel<<<dim3(tail, 2 * kBM / rows_per_cta), 128, 0, stream>>>(a2, parts, D);
        US_LAUNCH_CHECK();
        return US_OK;
      }
    }
  }
  const int rc0 = launch(dim3(q_pairs, Hq, n_seqs), a);
  if (rc0) return rc0;
#undef US_FLASH2_LAUNCH
#undef US_FLASH2_LAUNCH4
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
