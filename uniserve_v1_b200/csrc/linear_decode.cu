// Decode-size dense linear:  out[row, m] = sum_k X[row, k] * W[m, k] (+ bias[m])  for at
// most 64 activation rows.
//
// A 64-row projection of a decode step (QKV, attention output, router, LM head of one
// rank) moves a few megabytes of weights once and does almost no arithmetic: it is bound
// by launch-to-first-byte latency, not by tensor throughput.  The tcgen05 kernel of
// gemm_tc05.cu spends about 12 us on such a shape (tensor-memory allocation, tensor-map
// fetch, a two-stage TMA ring, a cluster reduction for its split K).  This kernel has no
// set-up at all: every lane streams its share of the weight rows straight from global
// memory with 16-byte loads kept several deep in registers, the activation rows sit in
// shared memory, and the products run on the warp-level tensor instruction
// (mma.sync m16n8k16, bf16 in, fp32 out), whose operands need no staging.  The large
// and the grouped GEMMs stay on tcgen05.
//
// CTA = 8 warps = 2 groups of 8 output features x 4 slices of K; grid = M / 16.
// K order inside an instruction is free (both operands use the same order), so a lane's
// one 16-byte weight load (8 consecutive k of its feature) feeds two instructions.
//
// Few output features (a router's 128, one rank's share of a QKV projection) would leave
// most SMs idle with one CTA per 16 features: such launches split K over the S CTAs of a
// thread-block cluster (grid = M / 16 x S).  CTA s takes the K iterations s, s + S, ...;
// the partial sums meet in the first CTA through distributed shared memory, in a fixed
// order (the result does not depend on timing).
#include "include/us_common.cuh"
#include "include/us_tc05.cuh"

namespace {

constexpr int kFeat = 16;        // output features per CTA
constexpr int kSlices = 4;       // K slices per CTA (one warp each per feature group)
constexpr int kChunk = 64;       // k per slice per iteration
constexpr int kIterK = kSlices * kChunk;   // 256 k per CTA iteration
constexpr int kRowPieces = kIterK / 8;     // 16-byte pieces per activation row of an iteration
constexpr int kStages = 4;                 // activation tiles in the shared-memory ring
// Piece c of row r is stored at c ^ ((r & 1) << 2): the eight lanes of a quarter warp (two
// rows x four pieces) then read eight different 16-byte columns.
__device__ __forceinline__ int swz(int piece, int row) { return piece ^ ((row & 1) << 2); }

__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                         uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
      "{%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
  const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
  const int n = valid ? 16 : 0;      // zero-fill rows past the batch
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(s), "l"(gmem), "r"(n)
               : "memory");
}

// MT = 16-row tiles of the activation (rows <= 16 * MT).
template <int MT>
__global__ void __launch_bounds__(256)
linear_decode_kernel(const __nv_bfloat16* __restrict__ W, const __nv_bfloat16* __restrict__ X,
                     void* __restrict__ out, const void* __restrict__ bias, int rows, int M, int K,
                     long long ldw, long long ldx, long long ldo, int out_f32, int bias_f32,
                     int ksplit) {
  // Weights are never written by a kernel: the first loads go out before the wait on the
  // kernels that produce the activation.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  // activation tiles [kStages][rows][pieces] (a cp.async ring, kStages - 1 tiles in flight:
  // the tiles come from L2, a tile's arithmetic is far shorter than its latency); the
  // K-slice partial sums [slice][group][row][8 + 1] reuse the memory after the loop
  extern __shared__ uint4 smem_dyn[];
  uint4 (*xs)[16 * MT][kRowPieces] = reinterpret_cast<uint4 (*)[16 * MT][kRowPieces]>(smem_dyn);
  float (*red)[2][16 * MT][9] = reinterpret_cast<float (*)[2][16 * MT][9]>(smem_dyn);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int ng = warp & 1, ks = warp >> 1;              // feature group, K slice
  const int n = lane >> 2, kq = lane & 3;
  const int feat = blockIdx.x * kFeat + ng * 8 + n;
  const bool feat_ok = feat < M;
  const __nv_bfloat16* wrow = W + (long long)(feat_ok ? feat : 0) * ldw;
  // this CTA's K iterations: every ksplit-th one starting at its cluster rank
  const int kr = ksplit > 1 ? (int)tc::cluster_ctarank() : 0;
  const int all_iters = K / kIterK;
  const int iters = all_iters > kr ? (all_iters - kr + ksplit - 1) / ksplit : 0;
  auto k_of = [&](int it) { return (it * ksplit + kr) * kIterK; };
  constexpr int kAhead = 4;                             // iterations of weights in registers
  uint4 wreg[kAhead][2];
  // lane's weights of iteration it: k = it*256 + ks*64 + b*32 + kq*8 .. +7, b = 0, 1
  auto load_w = [&](int it, uint4 (&dst)[2]) {
#pragma unroll
    for (int b = 0; b < 2; ++b) {
      const int k = k_of(it) + ks * kChunk + b * 32 + kq * 8;
      dst[b] = (feat_ok && it < iters)
                   ? __ldg(reinterpret_cast<const uint4*>(wrow + k))
                   : make_uint4(0, 0, 0, 0);
    }
  };
#pragma unroll
  for (int a = 0; a < kAhead; ++a) load_w(a, wreg[a]);
  asm volatile("griddepcontrol.wait;" ::: "memory");

  // activation tile of iteration it: rows x 256 k, 16-byte pieces by all threads
  auto load_x = [&](int it, int buf) {
    constexpr int kPieces = 16 * MT * (kIterK / 8);
    for (int p = threadIdx.x; p < kPieces; p += 256) {
      const int r = p / (kIterK / 8), c = p - r * (kIterK / 8);
      cp_async16(&xs[buf][r][swz(c, r)],
                 X + (long long)(r < rows ? r : 0) * ldx + k_of(it) + c * 8, r < rows);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  float acc[MT][4];
#pragma unroll
  for (int m = 0; m < MT; ++m)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[m][j] = 0.f;

  // every iteration commits exactly one group (an empty one past the end), so "all but the
  // newest kStages - 1 groups are complete" always means "this iteration's tile has landed"
#pragma unroll
  for (int a = 0; a < kStages - 1; ++a) {
    if (a < iters) load_x(a, a);
    else asm volatile("cp.async.commit_group;" ::: "memory");
  }
  // The weight registers are indexed statically (the loop is unrolled by kAhead): moving a
  // register whose load is still in flight would wait for that load.
  for (int it0 = 0; it0 < iters; it0 += kAhead) {
#pragma unroll
    for (int a = 0; a < kAhead; ++a) {
      const int it = it0 + a;
      if (it >= iters) break;
      const int buf = it % kStages;
      asm volatile("cp.async.wait_group %0;" ::"n"(kStages - 2) : "memory");
      __syncthreads();    // the tile is visible to every warp; the buffer refilled below was
                          // read by every warp one iteration ago
      if (it + kStages - 1 < iters) load_x(it + kStages - 1, (it + kStages - 1) % kStages);
      else asm volatile("cp.async.commit_group;" ::: "memory");
      const uint4 w0 = wreg[a][0], w1 = wreg[a][1];
      load_w(it + kAhead, wreg[a]);
#pragma unroll
      for (int b = 0; b < 2; ++b) {
        const uint4 wv = b == 0 ? w0 : w1;
        // the lane's 8 k as words {k0k1, k2k3, k4k5, k6k7}: instruction 0 takes (x, y),
        // instruction 1 takes (z, w); the activation piece holds the same 8 k
        const int piece = (ks * kChunk + b * 32) / 8 + kq;
#pragma unroll
        for (int m = 0; m < MT; ++m) {
          const uint4 lo = xs[buf][m * 16 + n][swz(piece, n)];
          const uint4 hi = xs[buf][m * 16 + n + 8][swz(piece, n)];       // same row parity
          mma16816(acc[m], lo.x, hi.x, lo.y, hi.y, wv.x, wv.y);
          mma16816(acc[m], lo.z, hi.z, lo.w, hi.w, wv.z, wv.w);
        }
      }
    }
  }
  __syncthreads();        // every warp is done with the tiles: the partial sums reuse them
  // sum the K slices: C fragment (row = n (+8), col = 2 kq + {0, 1}) -> red[ks][ng][row][col]
#pragma unroll
  for (int m = 0; m < MT; ++m) {
    red[ks][ng][m * 16 + n][2 * kq] = acc[m][0];
    red[ks][ng][m * 16 + n][2 * kq + 1] = acc[m][1];
    red[ks][ng][m * 16 + n + 8][2 * kq] = acc[m][2];
    red[ks][ng][m * 16 + n + 8][2 * kq + 1] = acc[m][3];
  }
  __syncthreads();
  if (ksplit > 1) {
    // every CTA folds its K slices into slice 0, then the first CTA of the cluster adds the
    // others' sums in rank order
    for (int e = threadIdx.x; e < 16 * MT * kFeat; e += 256) {
      const int r = e / kFeat, f = e - r * kFeat;
      float v = 0.f;
#pragma unroll
      for (int s = 0; s < kSlices; ++s) v += red[s][f >> 3][r][f & 7];
      red[0][f >> 3][r][f & 7] = v;
    }
    tc::cluster_sync();
    if (kr == 0) {
      for (int e = threadIdx.x; e < 16 * MT * kFeat; e += 256) {
        const int r = e / kFeat, f = e - r * kFeat;
        const int col = blockIdx.x * kFeat + f;
        if (r >= rows || col >= M) continue;
        const uint32_t local = (uint32_t)__cvta_generic_to_shared(&red[0][f >> 3][r][f & 7]);
        float v = red[0][f >> 3][r][f & 7];
        for (int p = 1; p < ksplit; ++p) v += tc::ld_dsmem_f32(tc::map_to_cta(local, (uint32_t)p));
        if (bias)
          v += bias_f32 ? reinterpret_cast<const float*>(bias)[col]
                        : us::bf2f(reinterpret_cast<const __nv_bfloat16*>(bias)[col]);
        if (out_f32)
          reinterpret_cast<float*>(out)[(long long)r * ldo + col] = v;
        else
          reinterpret_cast<__nv_bfloat16*>(out)[(long long)r * ldo + col] = us::f2bf(v);
      }
    }
    tc::cluster_sync();           // nobody leaves while its sums may still be read
    return;
  }
  for (int e = threadIdx.x; e < 16 * MT * kFeat; e += 256) {
    const int r = e / kFeat, f = e - r * kFeat;
    const int col = blockIdx.x * kFeat + f;
    if (r >= rows || col >= M) continue;
    float v = 0.f;
#pragma unroll
    for (int s = 0; s < kSlices; ++s) v += red[s][f >> 3][r][f & 7];
    if (bias)
      v += bias_f32 ? reinterpret_cast<const float*>(bias)[col]
                    : us::bf2f(reinterpret_cast<const __nv_bfloat16*>(bias)[col]);
    if (out_f32)
      reinterpret_cast<float*>(out)[(long long)r * ldo + col] = v;
    else
      reinterpret_cast<__nv_bfloat16*>(out)[(long long)r * ldo + col] = us::f2bf(v);
  }
}

}  // namespace

// rows <= 64, K a multiple of 256, 16-byte aligned rows of W and X.  Returns
// US_ERR_UNSUPPORTED for other shapes (the caller then takes the tcgen05 kernel).
US_API int us_linear_decode(const void* W, const void* X, void* out, const void* bias, int rows,
                            int M, int K, long long ldw, long long ldx, long long ldo,
                            int out_f32, int bias_f32, void* stream_) {
  US_REQUIRE(W && X && out && rows >= 1 && M >= 1 && K >= 1);
  if (rows > 64 || (K % kIterK) != 0 || (ldw % 8) != 0 || (ldx % 8) != 0 ||
      ((uintptr_t)W % 16) != 0 || ((uintptr_t)X % 16) != 0)
    return US_ERR_UNSUPPORTED;
  cudaStream_t stream = (cudaStream_t)stream_;
  const dim3 grid((M + kFeat - 1) / kFeat), block(256);
  const __nv_bfloat16* w = (const __nv_bfloat16*)W;
  const __nv_bfloat16* x = (const __nv_bfloat16*)X;
  static bool configured = false;
  if (!configured) {
    US_CUDA_CHECK(cudaFuncSetAttribute(linear_decode_kernel<4>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       4 * kStages * 8192));
    US_CUDA_CHECK(cudaFuncSetAttribute(linear_decode_kernel<2>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       2 * kStages * 8192));
    configured = true;
  }
  // K split over a cluster when one CTA per 16 features would leave most SMs idle
  static int sms = 0;
  static int max_split = -1;
  if (sms == 0) {
    int dev = 0;
    US_CUDA_CHECK(cudaGetDevice(&dev));
    US_CUDA_CHECK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    const char* e = getenv("US_LINEAR_KSPLIT");      // 1 switches the split off
    max_split = e ? atoi(e) : 8;
    if (max_split < 1) max_split = 1;
    if (max_split > 8) max_split = 8;
  }
  int ksplit = 1;
  const int iters = K / kIterK;
  // double while the CTAs still fit one wave and every CTA keeps at least one K iteration
  while (ksplit * 2 <= max_split && (int)grid.x * ksplit * 2 <= sms && iters >= ksplit * 2)
    ksplit *= 2;
  auto launch = [&](auto kernel, size_t smem) -> cudaError_t {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid.x, ksplit);
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = us::pdl_enabled() ? 1 : 0;
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = 1;
    attr[1].val.clusterDim.y = ksplit;
    attr[1].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ksplit > 1 ? 2 : 1;
    return cudaLaunchKernelEx(&cfg, kernel, w, x, out, bias, rows, M, K, ldw, ldx, ldo, out_f32,
                              bias_f32, ksplit);
  };
  // kStages buffers x (16 MT) rows x 512 bytes
  if (rows <= 16)
    US_CUDA_CHECK(launch(linear_decode_kernel<1>, kStages * 8192));
  else if (rows <= 32)
    US_CUDA_CHECK(launch(linear_decode_kernel<2>, 2 * kStages * 8192));
  else
    US_CUDA_CHECK(launch(linear_decode_kernel<4>, 4 * kStages * 8192));
  return US_OK;
}
