// Block-scaled FP8 (E4M3) weight-stationary GEMM on tcgen05, dense or grouped:
//
//   out[row, m] = sum_kb  ws[g, m / 128, kb] * xs[kb, row] *
//                 sum_{k in block kb} Wq[g, m, k] * Xq[row, k]
//
// Weights carry one FP32 scale per 128 x 128 block (the `weight_scale_inv` tensor of
// block-quantised checkpoints), activations one FP32 scale per row and 128-wide K
// block.  The tensor core cannot apply such scales, so every 128-deep K block is
// multiplied into a fresh TMEM accumulator (kind::f8f6f4, four K=32 instructions)
// and the epilogue warps promote it: they read the block's partial with
// tcgen05.ld, multiply by ws * xs and add it to FP32 accumulators held in
// registers.  Two TMEM buffers let block kb+1 multiply while block kb is promoted.
//
// Warp roles: warp 0 = TMA producer, warp 1 = TMEM owner + MMA issuer,
// warps 2-5 = promotion + epilogue (thread = output feature).  The dual form
// keeps two accumulator sets (value rows and gate rows of the stacked expert
// weight) and applies the gated activation in the final store.
//
// The reference serves per-tensor FP8 and refuses block-scaled checkpoints
// (crates/nn/src/quantization.rs:26-31, reference project path); this kernel has no
// counterpart there.
#include "include/us_common.cuh"
#include "include/us_tc05.cuh"
#include "include/us_tmap.h"
#include "include/us_gemm_args.cuh"

#include <cuda_fp8.h>

namespace {

constexpr int kBK8 = 128;                       // K elements (= bytes) per block
constexpr int kATile8 = kBlockM * kBK8;         // 16 KiB

struct Fp8Args {
  GemmArgs g;
  const float* w_scale;   // [G, w_scale_rows, k_blocks]
  const float* x_scale;   // [k_blocks, xs_ld]  (transposed: rows contiguous)
  long long xs_ld;
  int w_scale_rows;       // weight rows / 128 per group
  int k_blocks;
};

template <int BN, bool DUAL>
__global__ void __launch_bounds__(192)
gemm_fp8_block_kernel(const __grid_constant__ CUtensorMap tmA,
                      const __grid_constant__ CUtensorMap tmB, const Fp8Args fa) {
  US_PDL_PROLOGUE();
  const GemmArgs& args = fa.g;
  constexpr int kBTile = BN * kBK8;
  constexpr int kStageBytes = kATile8 * (DUAL ? 2 : 1) + kBTile;
  constexpr uint32_t kBufCols = DUAL ? 2 * BN : BN;   // columns of one TMEM buffer
  constexpr uint32_t kCols = tmem_cols<2 * BN>(DUAL);  // two buffers
  constexpr uint32_t kIdesc = tc::make_idesc(kBlockM, BN, tc::kFmtE4M3, tc::kFmtE4M3);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m_tile = blockIdx.x;
  const int n_tile = blockIdx.y;

  int group = 0, row0 = n_tile * BN, nrows;
  if (args.num_tiles != nullptr) {
    if (n_tile >= *args.num_tiles) return;
    group = args.tile_group[n_tile];
    row0 = args.tile_row0[n_tile];
    nrows = args.tile_rows[n_tile];
  } else {
    nrows = min(BN, args.rows - row0);
  }

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const int stages = args.stages;
  uint64_t* full_bar = (uint64_t*)(smem + (size_t)stages * kStageBytes);
  uint64_t* empty_bar = full_bar + stages;
  uint64_t* tfull_bar = empty_bar + stages;   // [2]
  uint64_t* tempty_bar = tfull_bar + 2;       // [2]
  uint32_t* tmem_slot = (uint32_t*)(tempty_bar + 2);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  volatile uint32_t* epi_fail = tmem_slot + 2;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      tc::mbar_init(&full_bar[s], 1);
      tc::mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      tc::mbar_init(&tfull_bar[b], 1);
      tc::mbar_init(&tempty_bar[b], 128);
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
  const int num_k = fa.k_blocks;

  if (warp == 0) {
    if (lane == 0) {
      tc::tma_prefetch_desc(&tmA);
      tc::tma_prefetch_desc(&tmB);
      for (int kb = 0; kb < num_k; ++kb) {
        const int s = kb % stages;
        const uint32_t ph = (uint32_t)(kb / stages) & 1u;
        if (!tc::mbar_wait(&empty_bar[s], ph ^ 1u, abort_flag)) {
          us_dev_fail(args.status, US_DEV_TIMEOUT_EMPTY);
          *abort_flag = 1;
          break;
        }
        uint8_t* st = smem + (size_t)s * kStageBytes;
        tc::mbar_expect_tx(&full_bar[s], kStageBytes);
        const int kx = kb * kBK8;
        tc::tma_load_3d(st, &tmA, &full_bar[s], kx, m_tile * kBlockM, group);
        if (DUAL)
          tc::tma_load_3d(st + kATile8, &tmA, &full_bar[s], kx,
                          args.dual_offset + m_tile * kBlockM, group);
        tc::tma_load_2d(st + kATile8 * (DUAL ? 2 : 1), &tmB, &full_bar[s], kx, row0);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      for (int kb = 0; kb < num_k; ++kb) {
        const int s = kb % stages;
        const uint32_t ph = (uint32_t)(kb / stages) & 1u;
        const int buf = kb & 1;
        if (!tc::mbar_wait(&full_bar[s], ph, abort_flag) ||
            !tc::mbar_wait(&tempty_bar[buf], ((uint32_t)(kb >> 1) & 1u) ^ 1u, abort_flag)) {
          us_dev_fail(args.status, US_DEV_TIMEOUT_FULL);
          *abort_flag = 1;
          break;
        }
        tc::tc_fence_after_sync();
        const uint32_t a_addr = tc::smem_u32(smem + (size_t)s * kStageBytes);
        const uint32_t b_addr = a_addr + kATile8 * (DUAL ? 2 : 1);
        const uint64_t adesc = tc::smem_desc_kmajor_sw128(a_addr);
        const uint64_t bdesc = tc::smem_desc_kmajor_sw128(b_addr);
        const uint32_t d = tmem_base + (uint32_t)buf * kBufCols;
#pragma unroll
        for (int k = 0; k < kBK8 / 32; ++k) {
          // 32 one-byte elements along K = 32 bytes = 2 descriptor address units
          tc::umma_f8(d, adesc + 2 * k, bdesc + 2 * k, kIdesc, k != 0);
          if (DUAL) {
            const uint64_t a2desc = tc::smem_desc_kmajor_sw128(a_addr + kATile8);
            tc::umma_f8(d + BN, a2desc + 2 * k, bdesc + 2 * k, kIdesc, k != 0);
          }
        }
        tc::umma_commit(&empty_bar[s]);
        tc::umma_commit(&tfull_bar[buf]);
      }
    }
  } else {
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    const int ml = q * 32 + lane;
    const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16);
    float acc[BN];
    float acc2[DUAL ? BN : 1];
#pragma unroll
    for (int i = 0; i < BN; ++i) acc[i] = 0.f;
    if (DUAL) {
#pragma unroll
      for (int i = 0; i < BN; ++i) acc2[DUAL ? i : 0] = 0.f;
    }
    const float* ws_row =
        fa.w_scale + ((size_t)group * fa.w_scale_rows + m_tile) * (size_t)fa.k_blocks;
    const float* ws2_row = ws_row + (size_t)(args.dual_offset / kBlockM) * (size_t)fa.k_blocks;
    bool ok = true;
    for (int kb = 0; kb < num_k; ++kb) {
      const int buf = kb & 1;
      if (!tc::mbar_wait(&tfull_bar[buf], (uint32_t)(kb >> 1) & 1u, abort_flag)) {
        us_dev_fail(args.status, US_DEV_TIMEOUT_ACC);
        ok = false;
        break;
      }
      tc::tc_fence_after_sync();
      const float ws = ws_row[kb];
      const float ws2 = DUAL ? ws2_row[kb] : 0.f;
      // Row starts of grouped tiles are arbitrary: scalar (warp-broadcast) loads.
      const float* xs = fa.x_scale + (size_t)kb * fa.xs_ld + row0;
      const uint32_t t = taddr + (uint32_t)buf * kBufCols;
#pragma unroll
      for (int c = 0; c < BN; c += 16) {
        if (c < nrows) {  // warp-uniform
          uint32_t v[16], g[16];
          tc::tmem_ld16(t + c, v);
          if (DUAL) tc::tmem_ld16(t + BN + c, g);
          float sc[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) sc[j] = __ldg(xs + c + j);
          tc::tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            acc[c + j] = fmaf(__uint_as_float(v[j]), ws * sc[j], acc[c + j]);
            if (DUAL)
              acc2[DUAL ? c + j : 0] =
                  fmaf(__uint_as_float(g[j]), ws2 * sc[j], acc2[DUAL ? c + j : 0]);
          }
        }
      }
      tc::tc_fence_before_sync();
      tc::mbar_arrive(&tempty_bar[buf]);
    }
    if (!ok) *epi_fail = 1;
    // All 128 epilogue threads meet here: the decision is uniform, and every
    // multiplication has completed, so the pipeline stages can stage the stores.
    asm volatile("bar.sync 1, 128;" ::: "memory");
    if (*epi_fail == 0) {
      Epilogue<DUAL> epi(args, group, m_tile * kBlockM, ml, row0);
#pragma unroll
      for (int c = 0; c < BN; c += 16) {
        if (c < nrows) {  // uniform over the CTA
          uint32_t v[16], g[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            v[j] = __float_as_uint(acc[c + j]);
            g[j] = DUAL ? __float_as_uint(acc2[DUAL ? c + j : 0]) : 0u;
          }
          epi.store_chunk16(c, c >> 4, v, g, nrows, smem);
        }
      }
    }
  }
  tc::tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc::tmem_dealloc(tmem_base, kCols);
  }
}

template <int BN, bool DUAL>
int launch8(const CUtensorMap& tmA, const CUtensorMap& tmB, Fp8Args fa, int m_tiles, int n_tiles,
            cudaStream_t stream) {
  constexpr int kStageBytes = kATile8 * (DUAL ? 2 : 1) + BN * kBK8;
  const int budget = BN <= 32 ? 104 * 1024 : 200 * 1024;
  int stages = budget / kStageBytes;
  if (stages > 8) stages = 8;
  if (stages > fa.k_blocks) stages = fa.k_blocks;
  if (stages < 1) stages = 1;
  fa.g.stages = stages;
  const size_t smem = (size_t)stages * kStageBytes + (2 * stages + 4) * 8 + 16 + 1024;
  static bool configured = false;
  if (!configured) {
    US_CUDA_CHECK(cudaFuncSetAttribute(gemm_fp8_block_kernel<BN, DUAL>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    configured = true;
  }
  US_CUDA_CHECK(us::launch_pdl(gemm_fp8_block_kernel<BN, DUAL>, dim3(m_tiles, n_tiles, 1),
                               dim3(192), smem, stream, tmA, tmB, fa));
  return US_OK;
}

// ----------------------------------------------------------------- quantise --
__device__ __forceinline__ uint8_t to_e4m3(float v) {
  return (uint8_t)__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3);
}

// One warp per (row, 128-wide K block): amax -> scale = amax / 448 (1 when the
// block is zero), q = x / scale.  Scales are stored transposed [k_blocks, xs_ld].
__global__ void __launch_bounds__(256)
quantize_rows_block128_kernel(const __nv_bfloat16* __restrict__ x, long long ldx,
                              uint8_t* __restrict__ q, long long ldq, float* __restrict__ scales,
                              long long xs_ld, int rows, int K, const int* __restrict__ live_rows) {
  US_PDL_PROLOGUE();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kblocks = K / 128;
  const long long unit = (long long)blockIdx.x * 8 + warp;
  const int limit = live_rows ? min(rows, *live_rows) : rows;
  if (unit >= (long long)limit * kblocks) return;
  const int row = (int)(unit / kblocks), kb = (int)(unit % kblocks);
  const __nv_bfloat16* src = x + (long long)row * ldx + kb * 128 + lane * 4;
  const uint2 raw = *reinterpret_cast<const uint2*>(src);
  const __nv_bfloat162 p0 = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
  const __nv_bfloat162 p1 = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
  const float f0 = __low2float(p0), f1 = __high2float(p0);
  const float f2 = __low2float(p1), f3 = __high2float(p1);
  float amax = fmaxf(fmaxf(fabsf(f0), fabsf(f1)), fmaxf(fabsf(f2), fabsf(f3)));
  amax = us::warp_max(amax);
  const float scale = amax > 0.f ? amax / 448.f : 1.f;
  const float inv = 1.f / scale;
  uchar4 o;
  o.x = to_e4m3(f0 * inv);
  o.y = to_e4m3(f1 * inv);
  o.z = to_e4m3(f2 * inv);
  o.w = to_e4m3(f3 * inv);
  *reinterpret_cast<uchar4*>(q + (long long)row * ldq + kb * 128 + lane * 4) = o;
  if (lane == 0) scales[(long long)kb * xs_ld + row] = scale;
}

// One CTA per row: amax over the whole row -> scale = amax / 448 (1 for a zero row),
// q = x / scale; out_scale[row] = scale * weight_scale (what the GEMM epilogue applies).
__global__ void __launch_bounds__(256)
quantize_rows_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, uint8_t* __restrict__ q,
                     long long ldq, float* __restrict__ out_scale, int K, float weight_scale) {
  US_PDL_PROLOGUE();
  __shared__ float scratch[33];
  const long long row = blockIdx.x;
  const __nv_bfloat16* xr = x + row * ldx;
  uint8_t* qr = q + row * ldq;
  float amax = 0.f;
  for (int v = threadIdx.x; v < (K >> 3); v += 256) {
    us::Pack16 p;
    p.u = *reinterpret_cast<const uint4*>(xr + v * 8);
#pragma unroll
    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(us::bf2f(p.b[i])));
  }
  amax = us::block_max(amax, scratch);
  const float scale = amax > 0.f ? amax / 448.f : 1.f;
  const float inv = 1.f / scale;
  for (int v = threadIdx.x; v < (K >> 3); v += 256) {
    us::Pack16 p;
    p.u = *reinterpret_cast<const uint4*>(xr + v * 8);
    uint8_t o[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i] = to_e4m3(us::bf2f(p.b[i]) * inv);
    *reinterpret_cast<uint2*>(qr + v * 8) = *reinterpret_cast<const uint2*>(o);
  }
  if (threadIdx.x == 0) out_scale[row] = scale * weight_scale;
}

// Per-tensor quantisation with a given scale (q = x / scale), or, when
// `amax_in` is set, with scale = *amax_in / 448 computed on the device.
__global__ void __launch_bounds__(256)
quantize_tensor_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ q, long long n,
                       float scale, const float* __restrict__ amax_in,
                       float* __restrict__ scale_out) {
  US_PDL_PROLOGUE();
  if (amax_in) scale = *amax_in > 0.f ? *amax_in / 448.f : 1.f;
  if (scale_out && blockIdx.x == 0 && threadIdx.x == 0) *scale_out = scale;
  const float inv = 1.f / scale;
  for (long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 8; i < n;
       i += (long long)gridDim.x * blockDim.x * 8) {
    if (i + 8 <= n) {
      us::Pack16 p;
      p.u = *reinterpret_cast<const uint4*>(x + i);
      uint8_t o[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = to_e4m3(us::bf2f(p.b[j]) * inv);
      *reinterpret_cast<uint2*>(q + i) = *reinterpret_cast<const uint2*>(o);
    } else {
      for (long long j = i; j < n; ++j) q[j] = to_e4m3(us::bf2f(x[j]) * inv);
    }
  }
}

// Absolute maximum of a bf16 tensor into *out (FP32 bits compare as integers for
// non-negative values); *out must be zeroed by the caller.
__global__ void __launch_bounds__(256)
absmax_kernel(const __nv_bfloat16* __restrict__ x, long long n, float* __restrict__ out) {
  US_PDL_PROLOGUE();
  __shared__ float scratch[33];
  float m = 0.f;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x)
    m = fmaxf(m, fabsf(us::bf2f(x[i])));
  m = us::block_max(m, scratch);
  if (threadIdx.x == 0) atomicMax(reinterpret_cast<int*>(out), __float_as_int(m));
}

}  // namespace

namespace {

struct RouteSpec {
  void* const* recv_peers = nullptr;
  int n_peers = 0;
  const int* route_map = nullptr;
  const float* route_w = nullptr;
  int route_per = 0;
};

int fp8_impl(const void* Wq, const float* w_scale, const void* Xq, const float* x_scale,
             long long xs_ld, void* out, int G, int w_rows, int M, int K, int x_rows,
             long long ldw, long long ldx, long long ldo, int dual, int dual_offset, int act,
             int out_dtype, const float* row_scale, const int* out_row_map, const int* tile_group,
             const int* tile_row0, const int* tile_rows, const int* num_tiles, int max_tiles,
             int block_n, const RouteSpec& rs, void* stream_) {
  US_REQUIRE(Wq && w_scale && Xq && x_scale && (out || rs.route_map) && G >= 1 && M >= 1 &&
             K >= 128 &&
             (K % 128) == 0 && (w_rows % 128) == 0);
  US_REQUIRE((ldw % 16) == 0 && (ldx % 16) == 0 && ((uintptr_t)Wq % 16) == 0 &&
             ((uintptr_t)Xq % 16) == 0 );
  US_REQUIRE(x_rows >= 1 && (dual_offset % 128) == 0);
  if (num_tiles) US_REQUIRE(tile_group && tile_row0 && tile_rows && max_tiles >= 1);
  US_REQUIRE(dual ? (block_n == 16 || block_n == 32 || block_n == 64)
                  : (block_n == 16 || block_n == 32 || block_n == 64 || block_n == 128));
  const int n_tiles = num_tiles ? max_tiles : (x_rows + block_n - 1) / block_n;
  // The scale rows of a tile's padding are read (and ignored): xs_ld covers them.
  US_REQUIRE(n_tiles <= 65535 && xs_ld >= (long long)x_rows + block_n);

  CUtensorMap tmA, tmB;
  int rc = us_tmap_3d(&tmA, Wq, US_TMAP_U8, (uint64_t)G, (uint64_t)w_rows, (uint64_t)K,
                      (uint64_t)ldw, (uint64_t)w_rows * (uint64_t)ldw, kBlockM, kBK8, US_SWZ_128);
  if (rc) return rc;
  rc = us_tmap_2d(&tmB, Xq, US_TMAP_U8, (uint64_t)x_rows, (uint64_t)K, (uint64_t)ldx,
                  (uint32_t)block_n, kBK8, US_SWZ_128);
  if (rc) return rc;

  Fp8Args fa;
  GemmArgs& a = fa.g;
  a.M = M; a.K = K; a.rows = x_rows; a.dual_offset = dual_offset; a.stages = 0; a.act = act;
  a.out_dtype = out_dtype; a.bias_dtype = 0; a.ldo = ldo; a.out = out; a.bias = nullptr;
  a.row_scale = row_scale; a.out_row_map = out_row_map; a.tile_group = tile_group;
  a.tile_row0 = tile_row0; a.tile_rows = tile_rows; a.num_tiles = num_tiles;
  a.status = us_status_ptr(); a.splits = 1; a.kb_per_split = 0; a.k_per_peer = 0;
  a.peer_cols = 0; a.peer_row_offset = 0; a.rows_per_peer = 0; a.peer_rows = 0; a.peer_slot = 0;
  for (int p = 0; p < 8; ++p) a.peer_out[p] = nullptr;
  a.route_map = nullptr; a.route_w = nullptr; a.route_per = 0;
  a.vec_store = 0;
  a.scale_first = 0;
  if (rs.route_map) {
    US_REQUIRE(rs.recv_peers && rs.route_w && rs.route_per > 0 && rs.n_peers >= 1 &&
               rs.n_peers <= 8 && out_dtype == 0 && !dual);
    a.route_map = rs.route_map;
    a.route_w = rs.route_w;
    a.route_per = rs.route_per;
    for (int p = 0; p < rs.n_peers; ++p) {
      US_REQUIRE(rs.recv_peers[p] != nullptr);
      a.peer_out[p] = rs.recv_peers[p];
    }
  }
  {
    const long long esz = out_dtype == 0 ? 2 : 4;
    bool okv = ((ldo * esz) % 16) == 0 && ((uintptr_t)out % 16) == 0;
    for (int p = 0; p < 8; ++p) okv = okv && ((uintptr_t)a.peer_out[p] % 16) == 0;
    a.vec_store = okv ? 1 : 0;
  }
  fa.w_scale = w_scale;
  fa.x_scale = x_scale;
  fa.xs_ld = xs_ld;
  fa.w_scale_rows = w_rows / 128;
  fa.k_blocks = K / 128;
  const int m_tiles = (M + kBlockM - 1) / kBlockM;
  cudaStream_t stream = (cudaStream_t)stream_;
#define US_FP8_CASE(BN)                                                      \
  case BN:                                                                   \
    return dual ? launch8<(BN > 64 ? 64 : BN), true>(tmA, tmB, fa, m_tiles, n_tiles, stream) \
                : launch8<BN, false>(tmA, tmB, fa, m_tiles, n_tiles, stream);
  switch (block_n) {
    US_FP8_CASE(16)
    US_FP8_CASE(32)
    US_FP8_CASE(64)
    US_FP8_CASE(128)
    default:
      return US_ERR_ARG;
  }
#undef US_FP8_CASE
}

}  // namespace

// Wq: [G, w_rows, K] e4m3 bytes (ldw bytes between rows), w_scale [G, w_rows / 128, K / 128];
// Xq: [x_rows, K] e4m3 with ldx, x_scale [K / 128, xs_ld] (transposed).  Remaining
// arguments as us_gemm_wx (bf16 or fp32 output, dense when num_tiles is null).
US_API int us_gemm_fp8_block(const void* Wq, const float* w_scale, const void* Xq,
                             const float* x_scale, long long xs_ld, void* out, int G, int w_rows,
                             int M, int K, int x_rows, long long ldw, long long ldx, long long ldo,
                             int dual, int dual_offset, int act, int out_dtype,
                             const float* row_scale, const int* out_row_map, const int* tile_group,
                             const int* tile_row0, const int* tile_rows, const int* num_tiles,
                             int max_tiles, int block_n, void* stream_) {
  RouteSpec rs;
  return fp8_impl(Wq, w_scale, Xq, x_scale, xs_ld, out, G, w_rows, M, K, x_rows, ldw, ldx, ldo,
                  dual, dual_offset, act, out_dtype, row_scale, out_row_map, tile_group, tile_row0,
                  tile_rows, num_tiles, max_tiles, block_n, rs, stream_);
}

// Grouped FC2 of an expert-parallel layer with block-scaled FP8 weights: the epilogue
// applies the gate weight and stores every output row into the combine buffer of the
// rank that owns the token (same routing arguments as us_gemm_wx_route_push).
US_API int us_gemm_fp8_block_route_push(const void* Wq, const float* w_scale, const void* Xq,
                                        const float* x_scale, long long xs_ld, int G, int M, int K,
                                        int x_rows, long long ldw, long long ldx, long long ldo,
                                        void* const* recv_peers, int n_peers, const int* route_map,
                                        const float* route_w, int route_per, const int* tile_group,
                                        const int* tile_row0, const int* tile_rows,
                                        const int* num_tiles, int max_tiles, int block_n,
                                        void* stream_) {
  RouteSpec rs;
  rs.recv_peers = recv_peers;
  rs.n_peers = n_peers;
  rs.route_map = route_map;
  rs.route_w = route_w;
  rs.route_per = route_per;
  return fp8_impl(Wq, w_scale, Xq, x_scale, xs_ld, nullptr, G, M, M, K, x_rows, ldw, ldx, ldo, 0,
                  0, 0, 0, nullptr, nullptr, tile_group, tile_row0, tile_rows, num_tiles,
                  max_tiles, block_n, rs, stream_);
}

// x [rows, K] bf16 -> q [rows, K] e4m3 + scales [K / 128, xs_ld].  `live_rows`
// (device word, optional) bounds the rows that are quantised.
US_API int us_fp8_quantize_rows_block128(const void* x, long long ldx, void* q, long long ldq,
                                         float* scales, long long xs_ld, int rows, int K,
                                         const int* live_rows, void* stream) {
  US_REQUIRE(x && q && scales && rows >= 0 && K >= 128 && (K % 128) == 0 && (ldx % 4) == 0 &&
             (ldq % 4) == 0 && xs_ld >= rows);
  if (rows == 0) return US_OK;
  const long long units = (long long)rows * (K / 128);
  US_CUDA_CHECK(us::launch_pdl(quantize_rows_block128_kernel, dim3((unsigned)((units + 7) / 8)),
                               dim3(256), 0, (cudaStream_t)stream, (const __nv_bfloat16*)x, ldx,
                               (uint8_t*)q, ldq, scales, xs_ld, rows, K, live_rows));
  return US_OK;
}

// Per-tensor: q = x / scale.  With `amax_scratch` (one FP32 word) the scale is
// measured on the device (two launches: absmax, then encode) and written to
// *scale_out; otherwise `scale` is used as given.
US_API int us_fp8_quantize_tensor(const void* x, void* q, long long n, float scale,
                                  float* amax_scratch, float* scale_out, void* stream_) {
  US_REQUIRE(x && q && n >= 0 && ((uintptr_t)x % 16) == 0 && ((uintptr_t)q % 8) == 0);
  if (n == 0) return US_OK;
  cudaStream_t stream = (cudaStream_t)stream_;
  int blocks = (int)((n / 8 + 255) / 256);
  if (blocks > 148 * 8) blocks = 148 * 8;
  if (blocks < 1) blocks = 1;
  if (amax_scratch) {
    US_CUDA_CHECK(cudaMemsetAsync(amax_scratch, 0, sizeof(float), stream));
    US_CUDA_CHECK(us::launch_pdl(absmax_kernel, dim3(blocks), dim3(256), 0, stream,
                                 (const __nv_bfloat16*)x, n, amax_scratch));
  } else {
    US_REQUIRE(scale > 0.f);
  }
  US_CUDA_CHECK(us::launch_pdl(quantize_tensor_kernel, dim3(blocks), dim3(256), 0, stream,
                               (const __nv_bfloat16*)x, (uint8_t*)q, n, scale,
                               (const float*)amax_scratch, scale_out));
  return US_OK;
}

// x [rows, K] bf16 -> q [rows, K] e4m3 with one dynamic scale per row; out_scale[row] =
// row scale * weight_scale.
US_API int us_fp8_quantize_rows(const void* x, long long ldx, void* q, long long ldq,
                                float* out_scale, int rows, int K, float weight_scale,
                                void* stream) {
  US_REQUIRE(x && q && out_scale && rows >= 0 && K >= 8 && (K % 8) == 0 && (ldx % 8) == 0 &&
             (ldq % 8) == 0 && ((uintptr_t)x % 16) == 0 && ((uintptr_t)q % 8) == 0);
  if (rows == 0) return US_OK;
  US_CUDA_CHECK(us::launch_pdl(quantize_rows_kernel, dim3(rows), dim3(256), 0,
                               (cudaStream_t)stream, (const __nv_bfloat16*)x, ldx, (uint8_t*)q,
                               ldq, out_scale, K, weight_scale));
  return US_OK;
}
