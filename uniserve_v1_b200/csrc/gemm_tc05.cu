// Weight-stationary tcgen05 GEMM family:  out[row, m] = sum_k X[row, k] * W[g, m, k].
//
// The weight matrix is the A operand (128 output features per CTA sit in the
// 128 TMEM lanes) and the activation rows are the B operand, so the UMMA N
// extent is the number of rows in the tile: 16 for a decode step, up to 256
// for prefill or the video transformer.  One kernel therefore serves skinny
// memory-bound shapes and large compute-bound ones, dense or grouped (one
// group per expert, tiles listed by the MoE sort).
//
// Warp roles: warp 0 = TMA producer, warp 1 = TMEM owner + MMA issuer,
// warps 2-5 = epilogue (one TMEM lane quarter each).
//
// Epilogues: plain store (bf16 or fp32, optional bias / per-row scale / output
// row map) and the dual-accumulator gated activation out = first * act(second)
// used by the experts' FC1 (first = up rows, second = gate rows of the stacked
// weight) and the video transformer's value-first SwiGLU.
#include <string.h>

#include "include/us_common.cuh"
#include "include/us_tc05.cuh"
#include "include/us_tmap.h"
#include "include/us_gemm_args.cuh"

namespace {

template <int BN, bool DUAL>
__global__ void __launch_bounds__(192)
gemm_wx_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ BMaps tmBs,
               const GemmArgs args) {
  // Programmatic dependent launch, with the wait moved down: what does not depend on the
  // kernels before this one - barrier set-up, the tensor-memory allocation and, for a dense
  // problem, the first stages' WEIGHT tiles (weights are never written by a kernel) - runs
  // while the previous kernel is still finishing.  Everything that reads activations or the
  // tile lists comes after griddepcontrol.wait.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  constexpr int kBTile = BN * kBlockK * 2;
  constexpr int kStageBytes = kATile * (DUAL ? 2 : 1) + kBTile;
  constexpr uint32_t kCols = tmem_cols<BN>(DUAL);
  constexpr uint32_t kIdesc = tc::make_idesc(kBlockM, BN, tc::kFmtBF16, tc::kFmtBF16);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m_tile = blockIdx.x;
  const int n_tile = blockIdx.y;
  const bool grouped = args.num_tiles != nullptr;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const int stages = args.stages;
  uint64_t* full_bar = (uint64_t*)(smem + (size_t)stages * kStageBytes);
  uint64_t* empty_bar = full_bar + stages;
  uint64_t* acc_bar = empty_bar + stages;
  uint32_t* tmem_slot = (uint32_t*)(acc_bar + 1);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  volatile uint32_t* epi_fail = tmem_slot + 2;
  const int num_k_total = (args.K + kBlockK - 1) / kBlockK;
  const int kb0 = blockIdx.z * args.kb_per_split;
  const int num_k = min(num_k_total - kb0, args.kb_per_split);
  // stages whose weight tiles are fetched ahead of the wait (dense problems only)
  const int early = (grouped || !args.early) ? 0 : min(stages, num_k);

  int group = 0, row0 = n_tile * BN, nrows;
  if (grouped || !args.early) asm volatile("griddepcontrol.wait;" ::: "memory");
  if (grouped) {
    // the tile list comes from the kernels before: leave at once when this CTA's tile is
    // past the list (nothing is allocated yet)
    if (n_tile >= *args.num_tiles) return;
    group = args.tile_group[n_tile];
    row0 = args.tile_row0[n_tile];
    nrows = args.tile_rows[n_tile];
  } else {
    nrows = min(BN, args.rows - row0);
  }
  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      tc::mbar_init(&full_bar[s], 1);
      tc::mbar_init(&empty_bar[s], 1);
    }
    tc::mbar_init(acc_bar, 1);
    *abort_flag = 0;
    *epi_fail = 0;
    tc::mbar_fence_init();
    tc::tma_prefetch_desc(&tmA);
    tc::tma_prefetch_desc(&tmBs.m[0]);
    for (int kb = 0; kb < early; ++kb) {
      uint8_t* st = smem + (size_t)kb * kStageBytes;
      tc::mbar_expect_tx(&full_bar[kb], kStageBytes);
      const int kx = (kb0 + kb) * kBlockK;
      tc::tma_load_3d(st, &tmA, &full_bar[kb], kx, m_tile * kBlockM, 0);
      if (DUAL)
        tc::tma_load_3d(st + kATile, &tmA, &full_bar[kb], kx,
                        args.dual_offset + m_tile * kBlockM, 0);
    }
  }
  if (warp == 1) {
    tc::tmem_alloc(tmem_slot, kCols);
    tc::tmem_relinquish();
  }
  if (!grouped && args.early) asm volatile("griddepcontrol.wait;" ::: "memory");
  tc::tc_fence_before_sync();
  __syncthreads();
  tc::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      auto load_b = [&](uint8_t* st, uint64_t* bar, int kx) {
        if (args.rows_per_peer > 0) {
          const int src = row0 / args.rows_per_peer;
          tc::tma_load_2d(st + kATile * (DUAL ? 2 : 1), &tmBs.m[src], bar, kx,
                          row0 - src * args.rows_per_peer);
        } else {
          const int src = args.k_per_peer > 0 ? kx / args.k_per_peer : 0;
          tc::tma_load_2d(st + kATile * (DUAL ? 2 : 1), &tmBs.m[src], bar,
                          kx - src * args.k_per_peer, row0);
        }
      };
      // activation tiles of the stages whose weights are already on their way
      for (int kb = 0; kb < early; ++kb)
        load_b(smem + (size_t)kb * kStageBytes, &full_bar[kb], (kb0 + kb) * kBlockK);
      for (int kb = early; kb < num_k; ++kb) {
        const int s = kb % stages;
        const uint32_t ph = (uint32_t)(kb / stages) & 1u;
        if (!tc::mbar_wait(&empty_bar[s], ph ^ 1u, abort_flag)) {
          us_dev_fail(args.status, US_DEV_TIMEOUT_EMPTY);
          *abort_flag = 1;
          break;
        }
        uint8_t* st = smem + (size_t)s * kStageBytes;
        tc::mbar_expect_tx(&full_bar[s], kStageBytes);
        const int kx = (kb0 + kb) * kBlockK;
        tc::tma_load_3d(st, &tmA, &full_bar[s], kx, m_tile * kBlockM, group);
        if (DUAL)
          tc::tma_load_3d(st + kATile, &tmA, &full_bar[s], kx,
                          args.dual_offset + m_tile * kBlockM, group);
        load_b(st, &full_bar[s], kx);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      bool ok = true;
      for (int kb = 0; kb < num_k; ++kb) {
        const int s = kb % stages;
        const uint32_t ph = (uint32_t)(kb / stages) & 1u;
        if (!tc::mbar_wait(&full_bar[s], ph, abort_flag)) {
          us_dev_fail(args.status, US_DEV_TIMEOUT_FULL);
          *abort_flag = 1;
          ok = false;
          break;
        }
        tc::tc_fence_after_sync();
        const uint32_t a_addr = tc::smem_u32(smem + (size_t)s * kStageBytes);
        const uint32_t b_addr = a_addr + kATile * (DUAL ? 2 : 1);
        const uint64_t adesc = tc::smem_desc_kmajor_sw128(a_addr);
        const uint64_t bdesc = tc::smem_desc_kmajor_sw128(b_addr);
#pragma unroll
        for (int k = 0; k < kBlockK / 16; ++k) {
          const uint32_t acc = (kb | k) != 0;
          // 16 bf16 along K = 32 bytes = 2 descriptor address units
          tc::umma_f16(tmem_base, adesc + 2 * k, bdesc + 2 * k, kIdesc, acc);
          if (DUAL) {
            const uint64_t a2desc = tc::smem_desc_kmajor_sw128(a_addr + kATile);
            tc::umma_f16(tmem_base + BN, a2desc + 2 * k, bdesc + 2 * k, kIdesc, acc);
          }
        }
        tc::umma_commit(&empty_bar[s]);
      }
      if (ok) tc::umma_commit(acc_bar);
    }
  } else {
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    const int ml = q * 32 + lane;
    if (!tc::mbar_wait(acc_bar, 0, abort_flag)) {
      us_dev_fail(args.status, US_DEV_TIMEOUT_ACC);
      *epi_fail = 1;
    }
    // All 128 epilogue threads meet here, so the decision below is uniform and the
    // staged stores' barriers cannot be left waiting.
    asm volatile("bar.sync 1, 128;" ::: "memory");
    if (*epi_fail == 0) {
      tc::tc_fence_after_sync();
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16);
      if (!DUAL && args.splits > 1) {
        // Split-K: park the FP32 partial tile [row][feature] in this CTA's shared
        // memory (the pipeline stages are idle now); the cluster reduces it below.
        float* part = reinterpret_cast<float*>(smem);
#pragma unroll 1
        for (int c = 0; c < BN; c += 16) {
          if (c >= nrows) break;
          uint32_t v[16];
          tc::tmem_ld16(taddr + c, v);
          tc::tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j) part[(c + j) * kBlockM + ml] = __uint_as_float(v[j]);
        }
      } else {
        // The pipeline stages are idle: their first 16 KiB stage the stores.
        Epilogue<DUAL> epi(args, group, m_tile * kBlockM, ml, row0);
        int chunk = 0;
#pragma unroll 1
        for (int c = 0; c < BN; c += 16, ++chunk) {
          if (c >= nrows) break;  // uniform over the CTA
          uint32_t v[16], g[16];
          tc::tmem_ld16(taddr + c, v);
          if (DUAL) tc::tmem_ld16(taddr + BN + c, g);
          tc::tmem_ld_wait();
          epi.store_chunk16(c, chunk, v, g, nrows, smem);
        }
      }
    }
  }
  if (!DUAL && args.splits > 1) {
    // The `splits` CTAs of a tile form one cluster along z.  After the first
    // cluster barrier every partial is visible through distributed shared
    // memory; CTA r sums rows r, r + splits, ... over the CTAs in rank order (a
    // fixed order, so the result does not depend on timing) and stores them.
    tc::cluster_sync();
    if (warp >= 2 && !*abort_flag) {
      const int q = warp & 3;
      const int ml = q * 32 + lane;
      const uint32_t my_rank = tc::cluster_ctarank();
      Epilogue<false> epi(args, group, m_tile * kBlockM, ml, row0);
      const uint32_t local = tc::smem_u32(smem) + (uint32_t)ml * 4u;
      for (int r = (int)my_rank; r < nrows; r += args.splits) {
        float acc = 0.f;
        for (int sp = 0; sp < args.splits; ++sp)
          acc += tc::ld_dsmem_f32(tc::map_to_cta(local + (uint32_t)r * kBlockM * 4u, sp));
        epi.store(r, acc, 0.f);
      }
    }
    tc::cluster_sync();  // peers may still be reading this CTA's partial
  }
  tc::tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc::tmem_dealloc(tmem_base, kCols);
  }
}

// Persistent form for dense problems of more than one wave: one CTA per SM
// walks the output tiles (weight tile fastest, so CTAs running together share an
// activation tile in L2); two TMEM accumulators let the epilogue of tile i run
// under the multiplications of tile i + 1, and the TMA ring never drains
// between tiles.
template <int BN, bool DUAL, bool FP8>
__global__ void __launch_bounds__(192)
gemm_wx_persist_kernel(const __grid_constant__ CUtensorMap tmA,
                       const __grid_constant__ BMaps tmBs, const GemmArgs args) {
  US_PDL_PROLOGUE();
  // A k-block is 128 bytes of K either way: 64 bf16 or 128 e4m3 elements, four
  // tensor-core instructions (K = 16 resp. 32 each).
  constexpr int kBK = FP8 ? 2 * kBlockK : kBlockK;
  constexpr int kBTile = BN * kBlockK * 2;
  constexpr int kStageBytes = kATile * (DUAL ? 2 : 1) + kBTile;
  constexpr uint32_t kAccCols = DUAL ? 2 * BN : BN;
  constexpr uint32_t kCols = tmem_cols<2 * BN>(DUAL);
  static_assert(kCols <= 512, "two accumulators must fit tensor memory");
  constexpr uint32_t kIdesc = FP8 ? tc::make_idesc(kBlockM, BN, tc::kFmtE4M3, tc::kFmtE4M3)
                                  : tc::make_idesc(kBlockM, BN, tc::kFmtBF16, tc::kFmtBF16);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m_tiles = (args.M + kBlockM - 1) / kBlockM;
  const int n_tiles = (args.rows + BN - 1) / BN;
  const int total = m_tiles * n_tiles;
  const int num_k = (args.K + kBK - 1) / kBK;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const int stages = args.stages;
  uint64_t* full_bar = (uint64_t*)(smem + (size_t)stages * kStageBytes);
  uint64_t* empty_bar = full_bar + stages;
  uint64_t* acc_full = empty_bar + stages;   // [2]
  uint64_t* acc_empty = acc_full + 2;        // [2]
  uint32_t* tmem_slot = (uint32_t*)(acc_empty + 2);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  volatile uint32_t* epi_fail = tmem_slot + 2;
  uint8_t* epi_stage = smem + (size_t)stages * kStageBytes + 1024;   // after the barrier words

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      tc::mbar_init(&full_bar[s], 1);
      tc::mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      tc::mbar_init(&acc_full[b], 1);
      tc::mbar_init(&acc_empty[b], 128);
    }
    *abort_flag = 0;
    *epi_fail = 0;
    tc::mbar_fence_init();
  }
  if (warp == 1) {
    tc::tmem_alloc(tmem_slot, kCols);
    tc::tmem_relinquish();
  }
  tc::tc_fence_before_sync();
  __syncthreads();
  tc::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      tc::tma_prefetch_desc(&tmA);
      tc::tma_prefetch_desc(&tmBs.m[0]);
      int s = 0;          // stage and phase of the ring, carried over all tiles
      uint32_t ph = 0;
      bool ok = true;
      for (int t = blockIdx.x; ok && t < total; t += gridDim.x) {
        const int m_tile = t % m_tiles, row0 = (t / m_tiles) * BN;
        for (int kb = 0; kb < num_k; ++kb) {
          if (!tc::mbar_wait(&empty_bar[s], ph ^ 1u, abort_flag)) {
            us_dev_fail(args.status, US_DEV_TIMEOUT_EMPTY);
            *abort_flag = 1;
            ok = false;
            break;
          }
          uint8_t* st = smem + (size_t)s * kStageBytes;
          tc::mbar_expect_tx(&full_bar[s], kStageBytes);
          const int kx = kb * kBK;
          tc::tma_load_3d(st, &tmA, &full_bar[s], kx, m_tile * kBlockM, 0);
          if (DUAL)
            tc::tma_load_3d(st + kATile, &tmA, &full_bar[s], kx,
                            args.dual_offset + m_tile * kBlockM, 0);
          if (args.rows_per_peer > 0) {
            const int src = row0 / args.rows_per_peer;
            tc::tma_load_2d(st + kATile * (DUAL ? 2 : 1), &tmBs.m[src], &full_bar[s], kx,
                            row0 - src * args.rows_per_peer);
          } else {
            const int src = args.k_per_peer > 0 ? kx / args.k_per_peer : 0;
            tc::tma_load_2d(st + kATile * (DUAL ? 2 : 1), &tmBs.m[src], &full_bar[s],
                            kx - src * args.k_per_peer, row0);
          }
          if (++s == stages) {
            s = 0;
            ph ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // This one thread feeds the tensor core; everything it executes per k-block is
      // latency in series with the multiplications, so the loop carries its ring
      // position instead of dividing, builds descriptors by addition, and probes the
      // next stage's barrier while the current stage's instructions are in flight.
      int s = 0;
      uint32_t ph = 0;
      bool ok = true, ready = false;
      int it = 0;
      const uint64_t desc0 = tc::smem_desc_kmajor_sw128(tc::smem_u32(smem));
      for (int t = blockIdx.x; ok && t < total; t += gridDim.x, ++it) {
        const int buf = it & 1;
        if (!tc::mbar_wait(&acc_empty[buf], ((uint32_t)(it >> 1) & 1u) ^ 1u, abort_flag)) {
          us_dev_fail(args.status, US_DEV_TIMEOUT_ACC);
          *abort_flag = 1;
          break;
        }
        tc::tc_fence_after_sync();
        const uint32_t d = tmem_base + (uint32_t)buf * kAccCols;
        for (int kb = 0; kb < num_k; ++kb) {
          if (!ready && !tc::mbar_wait(&full_bar[s], ph, abort_flag)) {
            us_dev_fail(args.status, US_DEV_TIMEOUT_FULL);
            *abort_flag = 1;
            ok = false;
            break;
          }
          tc::tc_fence_after_sync();
          const uint64_t adesc = desc0 + (uint64_t)((uint32_t)s * (uint32_t)(kStageBytes >> 4));
          const uint64_t bdesc = adesc + (uint64_t)((kATile * (DUAL ? 2 : 1)) >> 4);
          int sn = s + 1;
          uint32_t phn = ph;
          if (sn == stages) {
            sn = 0;
            phn ^= 1u;
          }
          ready = tc::mbar_test_wait(&full_bar[sn], phn);
#pragma unroll
          for (int k = 0; k < kBlockK / 16; ++k) {
            const uint32_t acc = (kb | k) != 0;
            if (FP8)
              tc::umma_f8(d, adesc + 2 * k, bdesc + 2 * k, kIdesc, acc);
            else
              tc::umma_f16(d, adesc + 2 * k, bdesc + 2 * k, kIdesc, acc);
            if (DUAL) {
              const uint64_t a2desc = adesc + (uint64_t)(kATile >> 4);
              if (FP8)
                tc::umma_f8(d + BN, a2desc + 2 * k, bdesc + 2 * k, kIdesc, acc);
              else
                tc::umma_f16(d + BN, a2desc + 2 * k, bdesc + 2 * k, kIdesc, acc);
            }
          }
          tc::umma_commit(&empty_bar[s]);
          s = sn;
          ph = phn;
        }
        if (ok) tc::umma_commit(&acc_full[buf]);
      }
    }
  } else {
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    const int ml = q * 32 + lane;
    int it = 0;
    for (int t = blockIdx.x; t < total; t += gridDim.x, ++it) {
      const int buf = it & 1;
      const int m_tile = t % m_tiles, row0 = (t / m_tiles) * BN;
      const int nrows = min(BN, args.rows - row0);
      if (!tc::mbar_wait(&acc_full[buf], (uint32_t)(it >> 1) & 1u, abort_flag)) {
        us_dev_fail(args.status, US_DEV_TIMEOUT_ACC);
        *epi_fail = 1;
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");   // uniform decision, see above
      if (*epi_fail != 0) break;
      tc::tc_fence_after_sync();
      const uint32_t taddr = tmem_base + (uint32_t)buf * kAccCols + ((uint32_t)(q * 32) << 16);
      Epilogue<DUAL> epi(args, 0, m_tile * kBlockM, ml, row0);
      int chunk = 0;
#pragma unroll 1
      for (int c = 0; c < BN; c += 16, ++chunk) {
        if (c >= nrows) break;  // uniform over the CTA
        uint32_t v[16], g[16];
        tc::tmem_ld16(taddr + c, v);
        if (DUAL) tc::tmem_ld16(taddr + BN + c, g);
        tc::tmem_ld_wait();
        epi.store_chunk16(c, chunk, v, g, nrows, epi_stage);
      }
      // the staging halves are reused by the next tile: every read must be done
      asm volatile("bar.sync 1, 128;" ::: "memory");
      tc::tc_fence_before_sync();
      tc::mbar_arrive(&acc_empty[buf]);
    }
  }
  tc::tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc::tmem_dealloc(tmem_base, kCols);
  }
}

constexpr int kPairChunks = 2;   // k-blocks per stage of the CTA-pair kernel

// Order of the swapped form's tiles: bands of kBandRows row pairs, and inside a band the
// row pair runs fastest.  The pairs running together then cover about 8 row pairs x 9
// feature tiles, so a weight tile is shared by 8 and an activation tile by 9 of them in
// L2 (feature-fastest order streamed a 308 MB gated weight once per 256 rows: 9.7 GB of
// DRAM reads for 0.4 GB of operands).
constexpr int kBandRows = 8;
__device__ __forceinline__ void swapped_tile(int t, int m_pairs, int n_tiles, int& mp, int& nt) {
  const int band = t / (kBandRows * n_tiles);
  const int r = t - band * (kBandRows * n_tiles);
  const int in_band = min(kBandRows, m_pairs - band * kBandRows);
  nt = r / in_band;
  mp = band * kBandRows + (r - nt * in_band);
}

// CTA-pair form of the persistent kernel: the two CTAs of a cluster own one
// 256 x BN output tile and multiply it with cta_group::2 instructions, so every
// SM fetches its own 128 weight rows and only half of the activation rows from
// shared memory per instruction (the single-CTA form is bound by that operand
// fetch, not by the multipliers).  Each CTA loads its operands with its own TMA
// ring; the odd CTA forwards its "stage filled" events to the even CTA, whose
// MMA thread issues for both and releases the stages and accumulators of both
// through commits addressed to either CTA's barriers.  A stage holds kPairChunks
// k-blocks, fetched by one TMA instruction per operand through tensor maps that
// view K as [K / chunk, chunk]: the feed of the single-CTA form measured a fixed
// cost per TMA instruction, not per byte.
//
// SWAP: the operands change roles.  The activation rows are the 256-row side (128
// per CTA) and every epilogue thread owns one activation row, whose features it
// stores from registers as 32-byte pieces - no staging tile, and every destination
// (plain, row-mapped, a peer's buffer by feature block or by row interval, the
// token owner's combine buffer) is one pointer per thread.  SWAP = 2 (dense): the
// other side is 256 weight rows, 128 per CTA.  SWAP = 1 (gated): 128 value rows in
// the even CTA and the matching 128 gate rows in the odd CTA, so one N = 256
// instruction produces both halves and a thread finds value j in column j and its
// gate in column 128 + j of its own lane.  The caller passes the activation's map
// as tmA and the weight's as tmBs.m[0].
// Whether the swapped epilogue's rows go to other GPUs' buffers (env US_GEMM_LINES=0 keeps
// the per-thread 32-byte pieces for an A/B measurement; the host sets args.remote_lines).
__device__ __forceinline__ bool remote_lines(const GemmArgs& a) {
  return a.remote_lines != 0 &&
         (a.route_map != nullptr || a.peer_rows > 0 || a.peer_cols > 0);
}

template <int BN, bool DUAL, bool FP8, int SWAP>
__global__ void __launch_bounds__(192)
gemm_wx_pair_kernel(const __grid_constant__ CUtensorMap tmA,
                    const __grid_constant__ BMaps tmBs, const GemmArgs args) {
  US_PDL_PROLOGUE();
  constexpr int kBK = FP8 ? 2 * kBlockK : kBlockK;
  constexpr int kATiles = kATile * (DUAL ? 2 : 1);
  constexpr int kBHalf = (BN / 2) * kBlockK * 2;
  constexpr int kKC = kPairChunks;
  constexpr int kStageBytes = kKC * (kATiles + kBHalf);
  constexpr uint32_t kAccCols = DUAL ? 2 * BN : BN;
  constexpr uint32_t kCols = tmem_cols<2 * BN>(DUAL);
  static_assert(kCols <= 512, "two accumulators must fit tensor memory");
  constexpr uint32_t kIdesc =
      FP8 ? tc::make_idesc(2 * kBlockM, BN, tc::kFmtE4M3, tc::kFmtE4M3)
          : tc::make_idesc(2 * kBlockM, BN, tc::kFmtBF16, tc::kFmtBF16);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = tc::cluster_ctarank();          // 0 issues the multiplications
  const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
  static_assert(!SWAP || (BN == 256 && !DUAL), "the swapped form is one 256-column accumulator");
  // m: tiles of the 256-row (A) side, n: tiles of the other side
  const int m_tiles = SWAP ? (args.rows + kBlockM - 1) / kBlockM : (args.M + kBlockM - 1) / kBlockM;
  // Grouped (swapped forms only): the row tiles come from the sort kernel's list - tile i is
  // up to 256 rows of ONE group starting at tile_row0[i] (the even CTA takes the first 128,
  // the odd CTA the rest), and the group's weights are rows [group * group_rows, ...) of the
  // stacked weight map.  The list's length is on the device (the launch before wrote it).
  const bool grouped = SWAP != 0 && args.num_tiles != nullptr;
  const int m_pairs = grouped ? *args.num_tiles : (m_tiles + 1) / 2;
  auto a_row_of = [&](int mp) -> int {
    return grouped ? args.tile_row0[mp] + (int)rank * kBlockM : (2 * mp + (int)rank) * kBlockM;
  };
  auto b_off_of = [&](int mp) -> int { return grouped ? args.tile_group[mp] * args.group_rows : 0; };
  constexpr int kFeat = SWAP == 2 ? 2 * kBlockM : kBlockM;   // features per swapped tile
  const int n_tiles = SWAP ? (args.M + kFeat - 1) / kFeat : (args.rows + BN - 1) / BN;
  const int total = m_pairs * n_tiles;
  const int num_k = (args.K + kKC * kBK - 1) / (kKC * kBK);   // stages of K

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const int stages = args.stages;
  uint64_t* full_bar = (uint64_t*)(smem + (size_t)stages * kStageBytes);
  uint64_t* empty_bar = full_bar + stages;
  uint64_t* peer_full = empty_bar + stages;  // even CTA: the odd CTA's stage is filled
  uint64_t* acc_full = peer_full + stages;   // [2]
  uint64_t* acc_empty = acc_full + 2;        // [2], used in the even CTA only
  uint32_t* tmem_slot = (uint32_t*)(acc_empty + 2);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  volatile uint32_t* epi_fail = tmem_slot + 2;
  uint8_t* epi_stage = smem + (size_t)stages * kStageBytes + 1024;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      tc::mbar_init(&full_bar[s], 1);
      tc::mbar_init(&empty_bar[s], 1);
      tc::mbar_init(&peer_full[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      tc::mbar_init(&acc_full[b], 1);
      tc::mbar_init(&acc_empty[b], 256);     // the epilogue threads of both CTAs
    }
    *abort_flag = 0;
    *epi_fail = 0;
    tc::mbar_fence_init();
  }
  if (warp == 1) {
    tc::tmem_alloc(tmem_slot, kCols);
    tc::tmem_relinquish();
  }
  tc::tc_fence_before_sync();
  tc::cluster_sync();     // both CTAs' barriers exist before anything arrives remotely
  tc::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  // The pair instruction addresses both CTAs' tensor memory with one address:
  // both must have received the same columns (all 512 of an otherwise empty SM).
  const bool tmem_ok = (tmem_base & 0xffffu) == 0;
  if (!tmem_ok && threadIdx.x == 0) us_dev_fail(args.status, US_DEV_TIMEOUT_ACC);

  if (!tmem_ok) {
    // nothing is issued; the peer's waits run out and report
  } else if (warp == 0) {
    if (lane == 0) {
      tc::tma_prefetch_desc(&tmA);
      tc::tma_prefetch_desc(&tmBs.m[0]);
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int t = pair; ok && t < total; t += pairs) {
        int mp = t % m_pairs, nt = t / m_pairs;
        if (SWAP) swapped_tile(t, m_pairs, n_tiles, mp, nt);
        const int m_tile = 2 * mp + (int)rank;
        const int row0 = SWAP == 1   ? nt * kBlockM + (rank ? args.dual_offset : 0)
                         : SWAP == 2 ? nt * kFeat + (int)rank * kBlockM
                                     : nt * BN + (int)rank * (BN / 2);
        const int a_row = SWAP ? a_row_of(mp) : 0;
        const int b_off = SWAP ? b_off_of(mp) : 0;
        for (int kb = 0; kb < num_k; ++kb) {
          if (!tc::mbar_wait(&empty_bar[s], ph ^ 1u, abort_flag)) {
            us_dev_fail(args.status, US_DEV_TIMEOUT_EMPTY);
            *abort_flag = 1;
            ok = false;
            break;
          }
          uint8_t* st = smem + (size_t)s * kStageBytes;
          tc::mbar_expect_tx(&full_bar[s], kStageBytes);
          // weight rows past the last tile and chunks past K read as zeros
          tc::tma_load_3d(st, &tmA, &full_bar[s], 0, SWAP ? a_row : m_tile * kBlockM, kb * kKC);
          if (DUAL)
            tc::tma_load_3d(st + kKC * kATile, &tmA, &full_bar[s], 0,
                            args.dual_offset + m_tile * kBlockM, kb * kKC);
          tc::tma_load_3d(st + kKC * kATiles, &tmBs.m[0], &full_bar[s], 0, row0 + b_off,
                          kb * kKC);
          if (++s == stages) {
            s = 0;
            ph ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 1) {
      // forward "stage filled" to the issuing CTA
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      const uint32_t peer0 = tc::map_to_cta(tc::smem_u32(&peer_full[0]), 0);
      for (int t = pair; ok && t < total; t += pairs) {
        for (int kb = 0; kb < num_k; ++kb) {
          if (!tc::mbar_wait(&full_bar[s], ph, abort_flag)) {
            us_dev_fail(args.status, US_DEV_TIMEOUT_FULL);
            *abort_flag = 1;
            ok = false;
            break;
          }
          tc::mbar_arrive_cluster(peer0 + 8u * (uint32_t)s);
          if (++s == stages) {
            s = 0;
            ph ^= 1u;
          }
        }
      }
    } else if (lane == 0) {
      // One thread feeds both tensor cores: its loop is latency in series with the
      // multiplications, so it carries the ring position, adds descriptors, and
      // probes the next stage's barriers while the current instructions issue.
      int s = 0;
      uint32_t ph = 0;
      bool ok = true, ready = false;
      int it = 0;
      const uint64_t desc0 = tc::smem_desc_kmajor_sw128(tc::smem_u32(smem));
      const uint32_t empty0 = tc::smem_u32(&empty_bar[0]);
      const uint32_t empty0_peer = tc::map_to_cta(empty0, 1);
      for (int t = pair; ok && t < total; t += pairs, ++it) {
        const int buf = it & 1;
        if (!tc::mbar_wait_cluster(&acc_empty[buf], ((uint32_t)(it >> 1) & 1u) ^ 1u,
                                   abort_flag)) {
          us_dev_fail(args.status, US_DEV_TIMEOUT_ACC);
          *abort_flag = 1;
          break;
        }
        tc::tc_fence_after_sync();
        const uint32_t d = tmem_base + (uint32_t)buf * kAccCols;
        for (int kb = 0; kb < num_k; ++kb) {
          if (!ready && (!tc::mbar_wait(&full_bar[s], ph, abort_flag) ||
                         !tc::mbar_wait_cluster(&peer_full[s], ph, abort_flag))) {
            us_dev_fail(args.status, US_DEV_TIMEOUT_FULL);
            *abort_flag = 1;
            ok = false;
            break;
          }
          tc::tc_fence_after_sync();
          const uint64_t adesc = desc0 + (uint64_t)((uint32_t)s * (uint32_t)(kStageBytes >> 4));
          const uint64_t bdesc = adesc + (uint64_t)((kKC * kATiles) >> 4);
          int sn = s + 1;
          uint32_t phn = ph;
          if (sn == stages) {
            sn = 0;
            phn ^= 1u;
          }
          ready = tc::mbar_test_wait(&full_bar[sn], phn) &&
                  tc::mbar_test_wait(&peer_full[sn], phn);
#pragma unroll
          for (int c = 0; c < kKC; ++c) {
            const uint64_t ad = adesc + (uint64_t)((c * kATile) >> 4);
            const uint64_t bd = bdesc + (uint64_t)((c * kBHalf) >> 4);
#pragma unroll
            for (int k = 0; k < kBlockK / 16; ++k) {
              const uint32_t acc = (kb | c | k) != 0;
                if (FP8)
                tc::umma_f8_pair(d, ad + 2 * k, bd + 2 * k, kIdesc, acc);
              else
                tc::umma_f16_pair(d, ad + 2 * k, bd + 2 * k, kIdesc, acc);
              if (DUAL) {
                const uint64_t a2d = ad + (uint64_t)((kKC * kATile) >> 4);
                if (FP8)
                  tc::umma_f8_pair(d + BN, a2d + 2 * k, bd + 2 * k, kIdesc, acc);
                else
                  tc::umma_f16_pair(d + BN, a2d + 2 * k, bd + 2 * k, kIdesc, acc);
              }
            }
          }
          tc::umma_commit_pair(empty0 + 8u * (uint32_t)s);
          tc::umma_commit_pair(empty0_peer + 8u * (uint32_t)s);
          s = sn;
          ph = phn;
        }
        if (ok) {
          const uint32_t f = tc::smem_u32(&acc_full[buf]);
          tc::umma_commit_pair(f);
          tc::umma_commit_pair(tc::map_to_cta(f, 1));
        }
      }
    }
  } else {
    const int q = warp & 3;
    const int ml = q * 32 + lane;
    int it = 0;
    for (int t = pair; t < total; t += pairs, ++it) {
      const int buf = it & 1;
      int mp = t % m_pairs, nt = t / m_pairs;
      if (SWAP) swapped_tile(t, m_pairs, n_tiles, mp, nt);
      const int m_tile = 2 * mp + (int)rank;
      const int row0 = SWAP ? 0 : nt * BN;
      const int nrows = SWAP ? 0 : (m_tile < m_tiles ? min(BN, args.rows - row0) : 0);
      if (!tc::mbar_wait(&acc_full[buf], (uint32_t)(it >> 1) & 1u, abort_flag)) {
        us_dev_fail(args.status, US_DEV_TIMEOUT_ACC);
        *epi_fail = 1;
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");   // uniform decision over the 128 threads
      if (*epi_fail != 0) break;
      tc::tc_fence_after_sync();
      const uint32_t taddr = tmem_base + (uint32_t)buf * kAccCols + ((uint32_t)(q * 32) << 16);
      if (SWAP) {
        // this thread's activation row; its features leave as 32-byte pieces
        const int xrow = a_row_of(mp) + ml;
        const bool row_ok = grouped ? ((int)rank * kBlockM + ml) < args.tile_rows[mp]
                                    : xrow < args.rows;
        const int f0 = nt * kFeat;
        const int act = args.act;
        const int esz = args.out_dtype == 0 ? 2 : 4;
        const int M = args.M;
        const bool vec = args.vec_store != 0;
        const float* bias_f = args.bias_dtype == 0 ? nullptr : (const float*)args.bias;
        const __nv_bfloat16* bias_h = args.bias_dtype == 0 ? (const __nv_bfloat16*)args.bias : nullptr;
        const int peer_cols = args.peer_cols;
        float pre = 1.f, post = 1.f;          // scale before the activation / of the result
        char* dst = nullptr;                  // element (xrow, feature 0); null: row dropped
        if (row_ok) {
          if (args.row_scale != nullptr) (args.scale_first ? pre : post) = args.row_scale[xrow];
          if (args.route_map != nullptr) {
            const int i = args.route_map[xrow];
            const int src = i / args.route_per;
            post *= args.route_w[i];
            dst = (char*)args.peer_out[src] + (size_t)(i - src * args.route_per) * args.ldo * 2;
          } else if (args.out_row_map != nullptr) {
            const int orow = args.out_row_map[xrow];
            if (orow >= 0) dst = (char*)args.out + (size_t)orow * args.ldo * esz;
          } else if (args.peer_rows > 0) {
            const int p = xrow / args.peer_rows;
            dst = (char*)args.peer_out[p] +
                  ((size_t)args.peer_slot * args.peer_rows + (size_t)(xrow - p * args.peer_rows)) *
                      args.ldo * esz;
          } else if (peer_cols > 0) {
            dst = (char*)(size_t)1;           // resolved per feature block below
          } else {
            dst = (char*)args.out + (size_t)xrow * args.ldo * esz;
          }
        }
        // Rows that leave for another GPU go out as whole 128-byte lines: a thread's 32-byte
        // pieces of 32 different rows would cross NVLink as 32 small packets per store
        // instruction.  The warp collects 64 features of its 32 rows in its 4 KiB of the
        // staging area (16-byte chunks XOR-swizzled by row) and writes them back out with
        // eight lanes per row; the row's destination comes from the lane that owns it.
        const bool lines = remote_lines(args) && esz == 2 && vec && (M % 64) == 0;
        uint8_t* wstage = epi_stage + q * 4096;
#pragma unroll 1
        for (int c = 0; c < kFeat; c += 16) {
          if (f0 + c >= M) break;             // uniform: features past the last one
          uint32_t v[16], g[16];
          tc::tmem_ld16(taddr + c, v);
          if (SWAP == 1) tc::tmem_ld16(taddr + kBlockM + c, g);
          tc::tmem_ld_wait();
          float x[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            float val = __uint_as_float(v[j]) * pre;
            if (SWAP == 1) {
              const float gate = __uint_as_float(g[j]) * pre;
              if (act == 0) {
                val = val * silu_f(gate);
              } else if (act == 1) {
                const float sg = us::bf2f(us::f2bf(silu_f(us::bf2f(us::f2bf(gate)))));
                val = us::bf2f(us::f2bf(val)) * sg;
              } else {
                val = val * gelu_tanh_f(gate);
              }
            }
            x[j] = val;
          }
          if (bias_f != nullptr || bias_h != nullptr) {
#pragma unroll
            for (int j = 0; j < 16; ++j)
              if (f0 + c + j < M)
                x[j] += bias_f ? bias_f[f0 + c + j] : us::bf2f(bias_h[f0 + c + j]);
          }
          if (lines) {
            const int ch = (c & 63) >> 3;     // first of this piece's two 16-byte chunks
            uint32_t o[8];
#pragma unroll
            for (int j = 0; j < 8; ++j)
              o[j] = (uint32_t)__bfloat16_as_ushort(us::f2bf(x[2 * j] * post)) |
                     ((uint32_t)__bfloat16_as_ushort(us::f2bf(x[2 * j + 1] * post)) << 16);
            *reinterpret_cast<uint4*>(wstage + lane * 128 + ((ch ^ (lane & 7)) << 4)) =
                make_uint4(o[0], o[1], o[2], o[3]);
            *reinterpret_cast<uint4*>(wstage + lane * 128 + (((ch + 1) ^ (lane & 7)) << 4)) =
                make_uint4(o[4], o[5], o[6], o[7]);
            if ((c & 63) != 48) continue;
            // this lane's row, features [f0 + c - 48, f0 + c + 16)
            const int fb = f0 + c - 48;
            char* d64 = nullptr;
            if (dst != nullptr) {
              d64 = dst + (size_t)fb * 2;
              if (peer_cols > 0) {
                const int p = fb / peer_cols;
                d64 = (char*)args.peer_out[p] +
                      ((size_t)(args.peer_row_offset + xrow) * args.ldo + (fb - p * peer_cols)) * 2;
              }
            }
            __syncwarp();
            const unsigned long long mine = (unsigned long long)(uintptr_t)d64;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int r = i * 4 + (lane >> 3), cc = lane & 7;
              const unsigned long long dp = __shfl_sync(0xffffffffu, mine, r);
              const uint4 val =
                  *reinterpret_cast<const uint4*>(wstage + r * 128 + ((cc ^ (r & 7)) << 4));
              if (dp != 0ull) *reinterpret_cast<uint4*>((char*)(uintptr_t)dp + cc * 16) = val;
            }
            __syncwarp();
            continue;
          }
          if (dst == nullptr) continue;
          char* d = dst + (size_t)(f0 + c) * esz;
          if (peer_cols > 0) {
            const int p = (f0 + c) / peer_cols;
            d = (char*)args.peer_out[p] +
                ((size_t)(args.peer_row_offset + xrow) * args.ldo + (f0 + c - p * peer_cols)) * esz;
          }
          const bool whole = vec && f0 + c + 16 <= M;
          if (esz == 2) {
            uint32_t o[8];
#pragma unroll
            for (int j = 0; j < 8; ++j)
              o[j] = (uint32_t)__bfloat16_as_ushort(us::f2bf(x[2 * j] * post)) |
                     ((uint32_t)__bfloat16_as_ushort(us::f2bf(x[2 * j + 1] * post)) << 16);
            if (whole) {
              *reinterpret_cast<uint4*>(d) = make_uint4(o[0], o[1], o[2], o[3]);
              *reinterpret_cast<uint4*>(d + 16) = make_uint4(o[4], o[5], o[6], o[7]);
            } else {
#pragma unroll
              for (int j = 0; j < 16; ++j)
                if (f0 + c + j < M)
                  ((unsigned short*)d)[j] = (unsigned short)(o[j >> 1] >> ((j & 1) * 16));
            }
          } else {
            if (whole) {
#pragma unroll
              for (int j = 0; j < 16; j += 4)
                *reinterpret_cast<float4*>(d + j * 4) =
                    make_float4(x[j] * post, x[j + 1] * post, x[j + 2] * post, x[j + 3] * post);
            } else {
#pragma unroll
              for (int j = 0; j < 16; ++j)
                if (f0 + c + j < M) ((float*)d)[j] = x[j] * post;
            }
          }
        }
      } else {
        Epilogue<DUAL> epi(args, 0, m_tile * kBlockM, ml, row0);
        int chunk = 0;
#pragma unroll 1
        for (int c = 0; c < BN; c += 16, ++chunk) {
          if (c >= nrows) break;  // uniform over the CTA
          uint32_t v[16], g[16];
          tc::tmem_ld16(taddr + c, v);
          if (DUAL) tc::tmem_ld16(taddr + BN + c, g);
          tc::tmem_ld_wait();
          epi.store_chunk16(c, chunk, v, g, nrows, epi_stage);
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
      }
      tc::tc_fence_before_sync();
      if (rank == 0)
        tc::mbar_arrive(&acc_empty[buf]);
      else
        tc::mbar_arrive_cluster(tc::map_to_cta(tc::smem_u32(&acc_empty[buf]), 0));
    }
  }
  tc::tc_fence_before_sync();
  tc::cluster_sync();     // no CTA leaves while the other may still signal it
  if (warp == 1) {
    __syncwarp();
    tc::tmem_dealloc(tmem_base, kCols);
  }
}

template <int BN, bool DUAL, bool FP8 = false, int SWAP = 0>
int launch_pair(const CUtensorMap& tmA, const BMaps& tmB, GemmArgs a, int pair_tiles,
                cudaStream_t stream) {
  constexpr int kStageBytes = kPairChunks * (kATile * (DUAL ? 2 : 1) + (BN / 2) * kBlockK * 2);
  int stages = (192 * 1024) / kStageBytes;
  if (stages > 8) stages = 8;
  a.stages = stages;
  a.splits = 1;
  const size_t smem = (size_t)stages * kStageBytes + 1024 + kEpiStageBytes + 1024;
  static bool configured = false;
  static int sms = 0;
  if (!configured) {
    US_CUDA_CHECK(cudaFuncSetAttribute(gemm_wx_pair_kernel<BN, DUAL, FP8, SWAP>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    int dev = 0;
    US_CUDA_CHECK(cudaGetDevice(&dev));
    US_CUDA_CHECK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    configured = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(sms & ~1);
  cfg.blockDim = dim3(192);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  // Tiles are dealt to the pairs round-robin, so every pair must be resident at
  // once: not every SM need have a partner free for a cluster of two.
  static int max_pairs = 0;
  if (max_pairs == 0) {
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    US_CUDA_CHECK(cudaOccupancyMaxActiveClusters(&n, gemm_wx_pair_kernel<BN, DUAL, FP8, SWAP>, &cfg));
    max_pairs = n < 1 ? 1 : n;
  }
  const int pairs = pair_tiles < max_pairs ? pair_tiles : max_pairs;
  cfg.gridDim = dim3(2 * pairs);
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = us::pdl_enabled() ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  US_CUDA_CHECK(cudaLaunchKernelEx(&cfg, gemm_wx_pair_kernel<BN, DUAL, FP8, SWAP>, tmA, tmB, a));
  return US_OK;
}

template <int BN, bool DUAL, bool FP8 = false>
int launch_persist(const CUtensorMap& tmA, const BMaps& tmB, GemmArgs a, int tiles,
                   cudaStream_t stream) {
  constexpr int kBTile = BN * kBlockK * 2;
  constexpr int kStageBytes = kATile * (DUAL ? 2 : 1) + kBTile;
  int stages = (192 * 1024) / kStageBytes;
  if (stages > 8) stages = 8;
  a.stages = stages;
  a.splits = 1;
  const size_t smem = (size_t)stages * kStageBytes + 1024 + kEpiStageBytes + 1024;
  static bool configured = false;
  static int sms = 0;
  if (!configured) {
    US_CUDA_CHECK(cudaFuncSetAttribute(gemm_wx_persist_kernel<BN, DUAL, FP8>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    int dev = 0;
    US_CUDA_CHECK(cudaGetDevice(&dev));
    US_CUDA_CHECK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    configured = true;
  }
  const int grid = tiles < sms ? tiles : sms;
  US_CUDA_CHECK(us::launch_pdl(gemm_wx_persist_kernel<BN, DUAL, FP8>, dim3(grid), dim3(192), smem,
                               stream, tmA, tmB, a));
  return US_OK;
}

// Live CTAs expected of the next grouped launch of this thread (us_gemm_wx_hint); 0 = none.
thread_local int g_cta_hint = 0;

template <int BN, bool DUAL>
int launch(const CUtensorMap& tmA, const BMaps& tmB, GemmArgs a, int m_tiles, int n_tiles,
           cudaStream_t stream) {
  constexpr int kBTile = BN * kBlockK * 2;
  constexpr int kStageBytes = kATile * (DUAL ? 2 : 1) + kBTile;
  const int num_k = (a.K + kBlockK - 1) / kBlockK;
  // Split K over a cluster when a dense launch would leave most SMs idle
  // (skinny weights): up to 8 CTAs per tile, at least two k-blocks each.
  int splits = 1;
  const int tiles = m_tiles * n_tiles;
  if (!DUAL && BN <= 64 && a.num_tiles == nullptr && tiles < 96 && num_k >= 4) {
    splits = (200 + tiles - 1) / tiles;
    if (splits > num_k / 2) splits = num_k / 2;
    static const int max_splits = [] {
      const char* e = getenv("US_GEMM_SPLITS");
      const int v = e ? atoi(e) : 8;
      return v >= 1 && v <= 8 ? v : 8;
    }();
    if (splits > max_splits) splits = max_splits;
  }
  int kb_per = (num_k + splits - 1) / splits;
  splits = (num_k + kb_per - 1) / kb_per;
  a.splits = splits;
  a.kb_per_split = kb_per;
  // Small row tiles are memory-bound: keep two CTAs per SM resident.
  // Small single-accumulator tiles (decode, grouped FC2) are latency-bound streams:
  // three stages per CTA and three to four CTAs per SM measured 5 % faster on the MoE
  // layer than five stages and two CTAs.  US_GEMM_SMALL_KB overrides the budget.
  static const int small_kb = [] {
    const char* e = getenv("US_GEMM_SMALL_KB");
    return e ? atoi(e) : 56;
  }();
  int budget = (BN <= 64 && !DUAL) ? small_kb * 1024 : (BN <= 32 ? 104 * 1024 : 200 * 1024);
  // A launch that cannot fill the SMs (a rank's share under tensor / expert parallelism)
  // is bound by the bytes each CTA keeps in flight, not by occupancy: give every CTA the
  // shared memory the missing neighbours would have used.  Grouped launches list more
  // tiles than are live (the list is sized for the worst case): the caller's hint, else
  // half the list, stands for the live count.
  // Measured on a 64-row decode step: deeper pipelines for the grouped expert GEMMs are
  // 7 % faster at 16 experts per rank and neutral at 128; deepening the dense skinny
  // GEMMs too cost 2.7 % on one GPU, so they keep their depth (US_GEMM_DEEP=2 deepens both,
  // 0 neither).
  static const int deep_mode = [] {
    const char* e = getenv("US_GEMM_DEEP");
    return (e && e[0] >= '0' && e[0] <= '2') ? e[0] - '0' : 1;
  }();
  const int hint = g_cta_hint;
  g_cta_hint = 0;
  if ((deep_mode == 1 && a.num_tiles && hint > 0) || deep_mode == 2) {
    const int est = hint > 0 ? hint
                             : (a.num_tiles ? m_tiles * ((n_tiles + 1) / 2) : tiles * splits);
    const int per_sm = (est + 147) / 148;
    const int room = per_sm <= 1 ? 200 * 1024 : per_sm == 2 ? 110 * 1024 : per_sm == 3 ? 72 * 1024 : 0;
    if (room > budget) budget = room;
  }
  int stages = budget / kStageBytes;
  if (stages > 8) stages = 8;
  if (stages > kb_per) stages = kb_per;
  if (stages < 1) stages = 1;
  a.stages = stages;
  static const bool early_ok = [] {
    const char* e = getenv("US_GEMM_EARLY");
    return !(e && e[0] == '0');
  }();
  a.early = early_ok ? 1 : 0;
  const size_t smem = (size_t)stages * kStageBytes + (2 * stages + 1) * 8 + 16 + 1024;
  static bool configured = false;
  if (!configured) {
    US_CUDA_CHECK(cudaFuncSetAttribute(gemm_wx_kernel<BN, DUAL>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    configured = true;
  }
  // The split-K partial tile (BN x 128 fp32, BN <= 64) reuses the stage memory:
  // at least two stages of >= 18 KiB each are always there for it.
  const size_t smem_needed = smem;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(m_tiles, n_tiles, splits);
  cfg.blockDim = dim3(192);
  cfg.dynamicSmemBytes = smem_needed;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = splits;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = us::pdl_enabled() ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  US_CUDA_CHECK(cudaLaunchKernelEx(&cfg, gemm_wx_kernel<BN, DUAL>, tmA, tmB, a));
  return US_OK;
}

// Operand view of the CTA-pair kernel: [rows, K] row-major seen as
// (chunk, rows, K / chunk) with chunk = 128 bytes of K, box (chunk, box_rows, kPairChunks).
static int pair_tmap(CUtensorMap* out, const void* base, int dtype, int rows, int K, long long ld,
                     uint32_t box_rows) {
  const uint64_t eb = dtype == US_TMAP_U8 ? 1 : 2;
  const uint64_t chunk = 128 / eb;
  uint64_t dims[3] = {chunk, (uint64_t)rows, (uint64_t)K / chunk};
  uint64_t strides[2] = {(uint64_t)ld * eb, 128};
  uint32_t box[3] = {(uint32_t)chunk, box_rows, (uint32_t)kPairChunks};
  return us_tmap_encode(out, base, dtype, 3, dims, strides, box, US_SWZ_128);
}

// US_GEMM_PAIR: 0 = single-CTA persistent kernel, 2 = CTA pairs with the weight on the
// 256-row side (staged epilogue), default 1 = CTA pairs with the operands swapped.
static int pair_mode() {
  static const int mode = [] {
    const char* e = getenv("US_GEMM_PAIR");
    return (e != nullptr && e[0] >= '0' && e[0] <= '2') ? e[0] - '0' : 1;
  }();
  return mode;
}
static bool pair_enabled() { return pair_mode() != 0; }

struct PeerSpec {
  const void* const* x_peers = nullptr;  // pull: activation base per rank
  int n_peers = 0;
  int k_per_peer = 0;
  void* const* out_peers = nullptr;      // scatter: output base per rank
  int peer_cols = 0;
  int peer_row_offset = 0;
  const int* route_map = nullptr;        // route push: see GemmArgs
  const float* route_w = nullptr;
  int route_per = 0;
  int n_out_peers = 0;
  int rows_per_peer = 0;                 // gather: rows of the activation per rank
  int peer_rows = 0;                     // reduce-scatter: rows owned per rank
  int peer_slot = 0;
};

int gemm_impl(const void* W, const void* X, void* out, int G, int w_rows, int M, int K, int x_rows,
              long long ldw, long long ldx, long long ldo, int dual, int dual_offset, int act,
              int out_dtype, const void* bias, int bias_dtype, const float* row_scale,
              const int* out_row_map, const int* tile_group, const int* tile_row0,
              const int* tile_rows, const int* num_tiles, int max_tiles, int block_n,
              const PeerSpec& ps, cudaStream_t stream) {
  US_REQUIRE(W && (X || ps.x_peers) && (out || ps.out_peers) && G >= 1 && M >= 1 && K >= 8 &&
             (K % 8) == 0);
  US_REQUIRE((ldw % 8) == 0 && (ldx % 8) == 0);
  US_REQUIRE(((uintptr_t)W % 16) == 0 && ((uintptr_t)X % 16) == 0);
  US_REQUIRE(x_rows >= 1);
  if (num_tiles) US_REQUIRE(tile_group && tile_row0 && tile_rows && max_tiles >= 1);

  // Dense problems of more than one wave run on CTA pairs (US_GEMM_PAIR=0: single CTAs).
  const bool pair = pair_enabled() && num_tiles == nullptr && G == 1 && !ps.x_peers &&
                    (K % kBlockK) == 0 &&
                    (dual ? block_n == 128 : block_n == 256) &&
                    (long long)((M + kBlockM - 1) / kBlockM) * ((x_rows + block_n - 1) / block_n) >
                        148;
  // Grouped problems with 256-row tiles (prefill-size expert batches) run the swapped CTA-pair
  // kernel over the sort kernel's tile list.
  const bool gpair = pair_enabled() && pair_mode() == 1 && num_tiles != nullptr && block_n == 256 &&
                     !ps.x_peers && !ps.out_peers && (K % kBlockK) == 0 && bias == nullptr &&
                     ldw == K;
  const uint32_t box_n = (uint32_t)(pair ? block_n / 2 : block_n);
  // operands swapped: one activation row per epilogue thread
  const bool swap = (pair && pair_mode() == 1) || gpair;

  CUtensorMap tmA;
  BMaps tmB;
  int rc;
  if (swap) {
    rc = pair_tmap(&tmA, X, US_TMAP_BF16, x_rows, K, ldx, kBlockM);
    if (rc) return rc;
    // grouped: the groups' weight rows are one stacked [G * w_rows, K] matrix
    rc = pair_tmap(&tmB.m[0], W, US_TMAP_BF16, gpair ? G * w_rows : w_rows, K, ldw, kBlockM);
    if (rc) return rc;
    for (int p = 1; p < 8; ++p) tmB.m[p] = tmB.m[0];
  } else if (pair) {
    rc = pair_tmap(&tmA, W, US_TMAP_BF16, w_rows, K, ldw, kBlockM);
    if (rc) return rc;
    rc = pair_tmap(&tmB.m[0], X, US_TMAP_BF16, x_rows, K, ldx, box_n);
    if (rc) return rc;
    for (int p = 1; p < 8; ++p) tmB.m[p] = tmB.m[0];
  } else {
    rc = us_tmap_3d(&tmA, W, US_TMAP_BF16, (uint64_t)G, (uint64_t)w_rows, (uint64_t)K,
                    (uint64_t)ldw, (uint64_t)w_rows * (uint64_t)ldw, kBlockM, kBlockK,
                    US_SWZ_128);
    if (rc) return rc;
  }
  if (pair || gpair) {
    // maps built above
  } else if (ps.x_peers && ps.rows_per_peer > 0) {
    US_REQUIRE(ps.n_peers >= 1 && ps.n_peers <= 8 && (ps.rows_per_peer % block_n) == 0 &&
               ps.rows_per_peer * ps.n_peers >= x_rows && num_tiles == nullptr);
    for (int p = 0; p < ps.n_peers; ++p) {
      US_REQUIRE(ps.x_peers[p] && ((uintptr_t)ps.x_peers[p] % 16) == 0);
      rc = us_tmap_2d(&tmB.m[p], ps.x_peers[p], US_TMAP_BF16, (uint64_t)ps.rows_per_peer,
                      (uint64_t)K, (uint64_t)ldx, (uint32_t)block_n, kBlockK, US_SWZ_128);
      if (rc) return rc;
    }
    for (int p = ps.n_peers; p < 8; ++p) tmB.m[p] = tmB.m[0];
  } else if (ps.x_peers) {
    US_REQUIRE(ps.n_peers >= 1 && ps.n_peers <= 8 && ps.k_per_peer > 0 &&
               (ps.k_per_peer % kBlockK) == 0 && ps.k_per_peer * ps.n_peers == K);
    for (int p = 0; p < ps.n_peers; ++p) {
      US_REQUIRE(ps.x_peers[p] && ((uintptr_t)ps.x_peers[p] % 16) == 0);
      rc = us_tmap_2d(&tmB.m[p], ps.x_peers[p], US_TMAP_BF16, (uint64_t)x_rows,
                      (uint64_t)ps.k_per_peer, (uint64_t)ldx, box_n, kBlockK, US_SWZ_128);
      if (rc) return rc;
    }
    for (int p = ps.n_peers; p < 8; ++p) tmB.m[p] = tmB.m[0];
  } else {
    rc = us_tmap_2d(&tmB.m[0], X, US_TMAP_BF16, (uint64_t)x_rows, (uint64_t)K, (uint64_t)ldx,
                    box_n, kBlockK, US_SWZ_128);
    if (rc) return rc;
    for (int p = 1; p < 8; ++p) tmB.m[p] = tmB.m[0];
  }

  GemmArgs a;
  a.M = M;
  a.K = K;
  a.rows = x_rows;
  a.dual_offset = dual_offset;
  a.stages = 0;
  a.early = 0;
  a.act = act;
  a.out_dtype = out_dtype;
  a.bias_dtype = bias_dtype;
  a.ldo = ldo;
  a.out = out;
  a.bias = bias;
  a.row_scale = row_scale;
  a.out_row_map = out_row_map;
  a.tile_group = tile_group;
  a.tile_row0 = tile_row0;
  a.tile_rows = tile_rows;
  a.num_tiles = num_tiles;
  a.group_rows = w_rows;
  a.status = us_status_ptr();
  a.splits = 1;
  a.kb_per_split = 0;
  a.k_per_peer = (ps.x_peers && ps.rows_per_peer == 0) ? ps.k_per_peer : 0;
  a.rows_per_peer = ps.x_peers ? ps.rows_per_peer : 0;
  a.peer_rows = 0;
  a.peer_slot = 0;
  a.peer_cols = 0;
  a.peer_row_offset = 0;
  for (int p = 0; p < 8; ++p) a.peer_out[p] = nullptr;
  a.route_map = nullptr;
  a.route_w = nullptr;
  a.route_per = 0;
  a.scale_first = 0;
  if (ps.route_map) {
    US_REQUIRE(ps.out_peers && ps.route_w && ps.route_per > 0 && ps.n_out_peers >= 1 &&
               ps.n_out_peers <= 8 && out_dtype == 0);
    a.route_map = ps.route_map;
    a.route_w = ps.route_w;
    a.route_per = ps.route_per;
    for (int p = 0; p < ps.n_out_peers; ++p) {
      US_REQUIRE(ps.out_peers[p] != nullptr);
      a.peer_out[p] = ps.out_peers[p];
    }
  } else if (ps.out_peers && ps.peer_rows > 0) {
    US_REQUIRE(ps.n_out_peers >= 1 && ps.n_out_peers <= 8 && ps.peer_slot >= 0 &&
               ps.peer_slot < ps.n_out_peers && ps.peer_rows * ps.n_out_peers >= x_rows &&
               (ps.peer_rows % block_n) == 0 && num_tiles == nullptr);
    a.peer_rows = ps.peer_rows;
    a.peer_slot = ps.peer_slot;
    for (int p = 0; p < ps.n_out_peers; ++p) {
      US_REQUIRE(ps.out_peers[p] != nullptr);
      a.peer_out[p] = ps.out_peers[p];
    }
  } else if (ps.out_peers) {
    US_REQUIRE(ps.peer_cols > 0 && (ps.peer_cols % kBlockM) == 0 && M % ps.peer_cols == 0 &&
               M / ps.peer_cols <= 8 && out_dtype == 0);
    a.peer_cols = ps.peer_cols;
    a.peer_row_offset = ps.peer_row_offset;
    for (int p = 0; p < M / ps.peer_cols; ++p) {
      US_REQUIRE(ps.out_peers[p] != nullptr);
      a.peer_out[p] = ps.out_peers[p];
    }
  }

  {
    const long long esz = out_dtype == 0 ? 2 : 4;
    bool ok = ((ldo * esz) % 16) == 0 && ((uintptr_t)out % 16) == 0;
    for (int p = 0; p < 8; ++p) ok = ok && ((uintptr_t)a.peer_out[p] % 16) == 0;
    a.vec_store = ok ? 1 : 0;
    static const int lines = [] {
      const char* e = getenv("US_GEMM_LINES");
      return (e && e[0] == '0') ? 0 : 1;
    }();
    a.remote_lines = lines;
  }
  const int m_tiles = (M + kBlockM - 1) / kBlockM;
  const int n_tiles = num_tiles ? max_tiles : (x_rows + block_n - 1) / block_n;
  US_REQUIRE(n_tiles <= 65535);

  // Dense problems of more than one wave run the persistent kernel (two
  // accumulators in tensor memory: row tiles up to 256, gated up to 128).
  static const bool no_persist = [] {
    const char* e = getenv("US_NO_PERSIST");
    return e && e[0] == '1';
  }();
  if (swap) {
    if (gpair) g_cta_hint = 0;      // the hint sizes the single-CTA kernel's pipeline only
    const int x_pairs = gpair ? max_tiles : ((x_rows + kBlockM - 1) / kBlockM + 1) / 2;
    if (dual)
      return launch_pair<256, false, false, 1>(tmA, tmB, a, x_pairs * ((M + 127) / 128), stream);
    return launch_pair<256, false, false, 2>(tmA, tmB, a, x_pairs * ((M + 255) / 256), stream);
  }
  if (pair) {
    const int pair_tiles = ((m_tiles + 1) / 2) * n_tiles;
    if (dual) return launch_pair<128, true>(tmA, tmB, a, pair_tiles, stream);
    return launch_pair<256, false>(tmA, tmB, a, pair_tiles, stream);
  }
  if (!no_persist && num_tiles == nullptr && G == 1 && m_tiles * n_tiles > 148 &&
      (dual ? block_n == 128 : (block_n == 128 || block_n == 256))) {
    const int tiles = m_tiles * n_tiles;
    if (dual) return launch_persist<128, true>(tmA, tmB, a, tiles, stream);
    if (block_n == 128) return launch_persist<128, false>(tmA, tmB, a, tiles, stream);
    return launch_persist<256, false>(tmA, tmB, a, tiles, stream);
  }
#define US_GEMM_CASE(BN)                                                              \
  case BN:                                                                            \
    return dual ? launch<BN, true>(tmA, tmB, a, m_tiles, n_tiles, stream)             \
                : launch<BN, false>(tmA, tmB, a, m_tiles, n_tiles, stream);
  switch (block_n) {
    US_GEMM_CASE(16)
    US_GEMM_CASE(32)
    US_GEMM_CASE(64)
    US_GEMM_CASE(128)
    US_GEMM_CASE(256)
    default:
      return US_ERR_ARG;
  }
#undef US_GEMM_CASE
}

}  // namespace

// W: [G, w_rows, K] bf16 (ld = ldw elements between rows, groups contiguous),
// X: [x_rows, K] bf16 with ldx.  Dense when num_tiles == nullptr (then
// n_tiles = ceil(rows / block_n)); grouped otherwise with `max_tiles` CTAs
// along the row-tile axis.
// Expected number of live CTAs of this thread's next grouped us_gemm_wx launch (the tile
// list of a grouped launch is sized for the worst case; the pipeline depth is chosen from
// how many CTAs will really run).  Consumed by that launch.
US_API int us_gemm_wx_hint(int live_ctas) {
  g_cta_hint = live_ctas > 0 ? live_ctas : 0;
  return US_OK;
}

US_API int us_gemm_wx(const void* W, const void* X, void* out, int G, int w_rows, int M, int K,
                      int x_rows, long long ldw, long long ldx, long long ldo, int dual,
                      int dual_offset, int act, int out_dtype, const void* bias, int bias_dtype,
                      const float* row_scale, const int* out_row_map, const int* tile_group,
                      const int* tile_row0, const int* tile_rows, const int* num_tiles,
                      int max_tiles, int block_n, void* stream_) {
  PeerSpec ps;
  return gemm_impl(W, X, out, G, w_rows, M, K, x_rows, ldw, ldx, ldo, dual, dual_offset, act,
                   out_dtype, bias, bias_dtype, row_scale, out_row_map, tile_group, tile_row0,
                   tile_rows, num_tiles, max_tiles, block_n, ps, (cudaStream_t)stream_);
}

// Dense GEMM whose output tiles are scattered into the peers' buffers from the
// epilogue (Ulysses projection: feature m goes to rank m / peer_cols, at row
// peer_row_offset + row and column m % peer_cols of a [*, ldo] buffer).
US_API int us_gemm_wx_scatter(const void* W, const void* X, int M, int K, int x_rows,
                              long long ldw, long long ldx, long long ldo, void* const* out_peers,
                              int peer_cols, int peer_row_offset, int block_n, void* stream_) {
  PeerSpec ps;
  ps.out_peers = out_peers;
  ps.peer_cols = peer_cols;
  ps.peer_row_offset = peer_row_offset;
  return gemm_impl(W, X, nullptr, 1, M, M, K, x_rows, ldw, ldx, ldo, 0, 0, 0, 0, nullptr, 0,
                   nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, 0, block_n, ps,
                   (cudaStream_t)stream_);
}

// Dense GEMM whose activation tiles are pulled from the peers' memory by TMA
// (no cluster multicast): columns [p * k_per_peer, (p + 1) * k_per_peer) of the
// K extent are rank p's [x_rows, k_per_peer] buffer (Ulysses return + to_out).
US_API int us_gemm_wx_pull(const void* W, const void* const* x_peers, int n_peers, int k_per_peer,
                           void* out, int M, int K, int x_rows, long long ldw, long long ldx,
                           long long ldo, int out_dtype, int block_n, void* stream_) {
  PeerSpec ps;
  ps.x_peers = x_peers;
  ps.n_peers = n_peers;
  ps.k_per_peer = k_per_peer;
  return gemm_impl(W, nullptr, out, 1, M, M, K, x_rows, ldw, ldx, ldo, 0, 0, 0, out_dtype,
                   nullptr, 0, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, 0, block_n,
                   ps, (cudaStream_t)stream_);
}

// Grouped FC2 of an expert-parallel layer: the epilogue applies the gate weight and
// stores every output row into the combine buffer of the rank that owns the token
// (see GemmArgs::route_map).  `recv_peers[p]` is rank p's combine buffer [*, ldo].
US_API int us_gemm_wx_route_push(const void* W, const void* X, int G, int M, int K, int x_rows,
                                 long long ldw, long long ldx, long long ldo,
                                 void* const* recv_peers, int n_peers, const int* route_map,
                                 const float* route_w, int route_per, const int* tile_group,
                                 const int* tile_row0, const int* tile_rows, const int* num_tiles,
                                 int max_tiles, int block_n, void* stream_) {
  PeerSpec ps;
  ps.out_peers = recv_peers;
  ps.n_out_peers = n_peers;
  ps.route_map = route_map;
  ps.route_w = route_w;
  ps.route_per = route_per;
  return gemm_impl(W, X, nullptr, G, M, M, K, x_rows, ldw, ldx, ldo, 0, 0, 0, 0, nullptr, 0,
                   nullptr, nullptr, tile_group, tile_row0, tile_rows, num_tiles, max_tiles,
                   block_n, ps, (cudaStream_t)stream_);
}

// Column-parallel linear with the all-gather fused into its operand loads: the
// activation's rows [p * rows_per_peer, ...) are read by TMA (no cluster multicast)
// from rank p's [rows_per_peer, K] buffer; W is this rank's [w_rows, K] weight shard.
// `dual` selects the gated form (value rows [0, M), gate rows [dual_offset, dual_offset + M)).
US_API int us_gemm_wx_gather(const void* W, const void* const* x_peers, int n_peers,
                             int rows_per_peer, void* out, int w_rows, int M, int K, int x_rows,
                             long long ldw, long long ldx, long long ldo, int dual,
                             int dual_offset, int act, int out_dtype, int block_n,
                             void* stream_) {
  PeerSpec ps;
  ps.x_peers = x_peers;
  ps.n_peers = n_peers;
  ps.rows_per_peer = rows_per_peer;
  return gemm_impl(W, nullptr, out, 1, w_rows, M, K, x_rows, ldw, ldx, ldo, dual, dual_offset,
                   act, out_dtype, nullptr, 0, nullptr, nullptr, nullptr, nullptr, nullptr,
                   nullptr, 0, block_n, ps, (cudaStream_t)stream_);
}

// Row-parallel linear with the reduce-scatter fused into its epilogue: row r of
// this rank's partial product is stored into slot `slot` of the buffer of the
// rank that owns the row (`out_peers[r / peer_rows]`, laid out
// [n_peers, peer_rows, ldo], bf16 or fp32 by out_dtype).
US_API int us_gemm_wx_reduce_scatter(const void* W, const void* X, int M, int K, int x_rows,
                                     long long ldw, long long ldx, long long ldo,
                                     void* const* out_peers, int n_peers, int peer_rows, int slot,
                                     int out_dtype, int block_n, void* stream_) {
  PeerSpec ps;
  ps.out_peers = out_peers;
  ps.n_out_peers = n_peers;
  ps.peer_rows = peer_rows;
  ps.peer_slot = slot;
  return gemm_impl(W, X, nullptr, 1, M, M, K, x_rows, ldw, ldx, ldo, 0, 0, 0, out_dtype, nullptr,
                   0, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, 0, block_n, ps,
                   (cudaStream_t)stream_);
}

// Per-tensor (or per-row) scaled FP8 GEMM: Wq [w_rows, K] and Xq [x_rows, K] are E4M3
// bytes; the product accumulates over the whole K in tensor memory and the epilogue
// multiplies row r by row_scale[r] (activation scale x weight scale).  With `dual`
// the scale is applied to both halves before the gated activation.  Persistent kernel.
US_API int us_gemm_fp8_rowscale(const void* Wq, const void* Xq, void* out, int w_rows, int M,
                                int K, int x_rows, long long ldw, long long ldx, long long ldo,
                                int dual, int dual_offset, int act, int out_dtype,
                                const float* row_scale, int block_n, void* stream_) {
  US_REQUIRE(Wq && Xq && out && row_scale && M >= 1 && K >= 128 && (K % 16) == 0 && x_rows >= 1);
  US_REQUIRE((ldw % 16) == 0 && (ldx % 16) == 0 && ((uintptr_t)Wq % 16) == 0 &&
             ((uintptr_t)Xq % 16) == 0);
  US_REQUIRE(dual ? block_n == 128 : (block_n == 128 || block_n == 256));
  CUtensorMap tmA;
  BMaps tmB;
  const int m_tiles = (M + kBlockM - 1) / kBlockM;
  const int n_tiles = (x_rows + block_n - 1) / block_n;
  const int tiles = m_tiles * n_tiles;
  const bool pair = pair_enabled() && tiles > 148 && (K % 128) == 0 &&
                    (dual ? block_n == 128 : block_n == 256);
  int rc;
  const bool swap = pair && pair_mode() == 1;
  if (swap) {
    rc = pair_tmap(&tmA, Xq, US_TMAP_U8, x_rows, K, ldx, kBlockM);
    if (rc) return rc;
    rc = pair_tmap(&tmB.m[0], Wq, US_TMAP_U8, w_rows, K, ldw, kBlockM);
  } else if (pair) {
    rc = pair_tmap(&tmA, Wq, US_TMAP_U8, w_rows, K, ldw, kBlockM);
    if (rc) return rc;
    rc = pair_tmap(&tmB.m[0], Xq, US_TMAP_U8, x_rows, K, ldx, (uint32_t)block_n / 2);
  } else {
    rc = us_tmap_3d(&tmA, Wq, US_TMAP_U8, 1, (uint64_t)w_rows, (uint64_t)K, (uint64_t)ldw,
                    (uint64_t)w_rows * (uint64_t)ldw, kBlockM, 2 * kBlockK, US_SWZ_128);
    if (rc) return rc;
    rc = us_tmap_2d(&tmB.m[0], Xq, US_TMAP_U8, (uint64_t)x_rows, (uint64_t)K, (uint64_t)ldx,
                    (uint32_t)block_n, 2 * kBlockK, US_SWZ_128);
  }
  if (rc) return rc;
  for (int p = 1; p < 8; ++p) tmB.m[p] = tmB.m[0];
  GemmArgs a;
  memset(&a, 0, sizeof(a));
  a.M = M; a.K = K; a.rows = x_rows; a.dual_offset = dual_offset; a.act = act;
  a.out_dtype = out_dtype; a.ldo = ldo; a.out = out; a.row_scale = row_scale;
  a.scale_first = 1;
  a.status = us_status_ptr(); a.splits = 1;
  const long long esz = out_dtype == 0 ? 2 : 4;
  a.vec_store = (((ldo * esz) % 16) == 0 && ((uintptr_t)out % 16) == 0) ? 1 : 0;
  cudaStream_t stream = (cudaStream_t)stream_;
  if (swap) {
    const int x_pairs = ((x_rows + kBlockM - 1) / kBlockM + 1) / 2;
    if (dual)
      return launch_pair<256, false, true, 1>(tmA, tmB, a, x_pairs * ((M + 127) / 128), stream);
    return launch_pair<256, false, true, 2>(tmA, tmB, a, x_pairs * ((M + 255) / 256), stream);
  }
  if (pair) {
    const int pair_tiles = ((m_tiles + 1) / 2) * n_tiles;
    if (dual) return launch_pair<128, true, true>(tmA, tmB, a, pair_tiles, stream);
    return launch_pair<256, false, true>(tmA, tmB, a, pair_tiles, stream);
  }
  if (dual) return launch_persist<128, true, true>(tmA, tmB, a, tiles, stream);
  if (block_n == 128) return launch_persist<128, false, true>(tmA, tmB, a, tiles, stream);
  return launch_persist<256, false, true>(tmA, tmB, a, tiles, stream);
}
