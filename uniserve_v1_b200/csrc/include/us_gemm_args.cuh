// Argument block and per-thread epilogue shared by the weight-stationary GEMM
// kernels (bf16 and block-scaled fp8).
#pragma once
#include "us_common.cuh"
#include "us_tc05.cuh"
#include "us_tmap.h"

namespace {

struct GemmArgs {
  int M;            // output features per group
  int K;
  int rows;         // activation rows (dense)
  int dual_offset;  // row offset of the second weight tile (dual epilogue)
  int stages;
  int early;        // dense: weight tiles of the first stages are fetched before the PDL wait
  int act;          // dual: 0 = silu fused rounding, 1 = silu stepwise rounding, 2 = gelu-tanh
  int out_dtype;    // 0 = bf16, 1 = fp32
  int bias_dtype;   // 0 = bf16, 1 = fp32
  long long ldo;
  void* out;
  const void* bias;        // [G, M] or null
  const float* row_scale;  // [rows] or null
  const int* out_row_map;  // [rows] destination row, <0 skips; null = identity
  const int* tile_group;   // grouped: group of each row tile
  const int* tile_row0;    // grouped: first activation row of each tile
  const int* tile_rows;    // grouped: valid rows of each tile
  const int* num_tiles;    // grouped: device word, number of row tiles
  unsigned int* status;
  // split-K (dense, single accumulator): the `splits` CTAs along z form one
  // thread-block cluster; CTA z owns k-blocks [z * kb_per_split, ...).
  int splits;
  int kb_per_split;
  // Peer modes (sequence parallelism).  Pull: the activation's K extent is the
  // concatenation of `k_per_peer`-wide slices that live in different ranks'
  // memory, one tensor map per rank.  Scatter: output feature m belongs to rank
  // m / peer_cols and is stored into that rank's buffer at row
  // peer_row_offset + row, column m % peer_cols.
  int k_per_peer;
  int peer_cols;
  int peer_row_offset;
  void* peer_out[8];
  // Tensor parallelism.  Gather: the activation's rows are the concatenation of
  // `rows_per_peer`-row intervals that live in different ranks' memory (all-gather
  // fused into the operand loads, one tensor map per rank).  Reduce-scatter: the
  // partial product's row r belongs to rank r / peer_rows and is stored into slot
  // `peer_slot` of that rank's [slots, peer_rows, ldo] buffer, where the owner sums
  // the slots.
  int rows_per_peer;
  int peer_rows;
  int peer_slot;
  // 1 when every destination row starts on a 16-byte boundary (base pointers and
  // row pitch): the epilogue then stores 16-byte pieces through a staging tile.
  int vec_store;
  // 1: the row scale multiplies both accumulators before the gated activation
  // (scaled low-precision operands); 0: it multiplies the finished value.
  int scale_first;
  // Route push (expert-parallel combine): permuted row r carries route
  // i = route_map[r] = (source rank * route_per + token * top_k + slot); the epilogue
  // multiplies by the gate weight route_w[i] and stores the row into the source
  // rank's combine buffer at row i % route_per.
  const int* route_map;
  const float* route_w;
  int route_per;
  // Grouped launches of the CTA-pair kernel: weight rows per group (the weight map stacks the
  // groups' rows; a tile's group comes from tile_group).
  int group_rows;
  // 1: the swapped epilogue writes rows bound for another GPU as whole 128-byte lines
  // (collected per warp in the staging area) instead of 32-byte pieces per thread.
  int remote_lines;
};

struct BMaps {
  CUtensorMap m[8];
};

constexpr int kBlockM = 128;
constexpr int kBlockK = 64;
constexpr int kATile = kBlockM * kBlockK * 2;  // 16 KiB

__device__ __forceinline__ float silu_f(float x) { return x / (1.f + __expf(-x)); }
__device__ __forceinline__ float gelu_tanh_f(float x) {
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  return 0.5f * x * (1.f + tanhf(k0 * (x + k1 * x * x * x)));
}

template <int BN>
constexpr int tmem_cols(bool dual) {
  int need = dual ? 2 * BN : BN;
  int c = 32;
  while (c < need) c <<= 1;
  return c;
}

constexpr int kEpiStageBytes = 16 * 1024;   // two staging tiles of 16 rows x 128 features x 4 B

// Epilogue of one 128-feature tile, run by the four epilogue warps (thread `ml`
// owns feature m0 + ml, i.e. TMEM lane ml).  Values get their activation, bias and
// scales in registers; stores go through a shared staging tile, 16 rows at a time,
// so that every row leaves as contiguous 16-byte pieces (256 B per row for bf16)
// whatever the destination: the plain output, a row-mapped output, a peer's buffer
// (scatter by feature, reduce-scatter by row) or the token owner's combine buffer.
template <bool DUAL>
struct Epilogue {
  // Everything the per-element code needs is copied out of the argument block
  // once: the block lives in parameter memory, and reading it per element (after
  // every barrier the compiler must re-read it) cost several dependent loads and
  // branches per value - 3,300 clocks per 16-row chunk, more than the mainloop.
  const int m0, ml, m, row0;
  const bool m_ok;
  float bias;
  char* tile_base;     // element (row0, m0) of the destination; null = per-row lookup
  long long row_bytes;
  int esz;
  int M, act, route_per, vec_store;
  long long ldo;
  const float* scale_rows;   // row_scale + row0, or null
  bool scale_first;
  const int* route_rows;     // route_map + row0, or null
  const float* route_w;
  const int* out_rows;       // out_row_map + row0, or null
  char* out;
  const GemmArgs& a;         // rare paths only (the peer table of the route push)
  __device__ __forceinline__ Epilogue(const GemmArgs& args, int group, int m0_, int ml_, int row0_)
      : m0(m0_), ml(ml_), m(m0_ + ml_), row0(row0_), m_ok(m0_ + ml_ < args.M), bias(0.f),
        tile_base(nullptr), row_bytes(0), esz(args.out_dtype == 0 ? 2 : 4), M(args.M),
        act(args.act), route_per(args.route_per), vec_store(args.vec_store), ldo(args.ldo),
        scale_rows(args.row_scale ? args.row_scale + row0_ : nullptr),
        scale_first(args.scale_first != 0),
        route_rows(args.route_map ? args.route_map + row0_ : nullptr), route_w(args.route_w),
        out_rows(args.out_row_map ? args.out_row_map + row0_ : nullptr), out((char*)args.out),
        a(args) {
    if (args.bias != nullptr && m_ok) {
      const size_t bi = (size_t)group * args.M + m;
      bias = args.bias_dtype == 0 ? us::bf2f(((const __nv_bfloat16*)args.bias)[bi])
                                  : ((const float*)args.bias)[bi];
    }
    row_bytes = ldo * esz;
    if (route_rows != nullptr || out_rows != nullptr) return;
    if (args.peer_rows > 0) {   // a tile lies inside one owner's interval
      const int p = row0 / args.peer_rows;
      tile_base = (char*)args.peer_out[p] +
                  (((size_t)args.peer_slot * args.peer_rows +
                    (size_t)(row0 - p * args.peer_rows)) * ldo + m0) * esz;
    } else if (args.peer_cols > 0) {
      const int p = m0 / args.peer_cols;
      tile_base = (char*)args.peer_out[p] +
                  ((size_t)(args.peer_row_offset + row0) * ldo + (m0 - p * args.peer_cols)) * esz;
    } else {
      tile_base = out + ((size_t)row0 * ldo + m0) * esz;
    }
  }
  // Value of tile row r for this thread's feature (everything but the store).
  __device__ __forceinline__ float value(int r, float val, float gate) const {
    if (scale_first && scale_rows != nullptr) {
      const float sc = scale_rows[r];
      val *= sc;
      gate *= sc;
    }
    if (DUAL) {
      if (act == 0) {
        val = val * silu_f(gate);
      } else if (act == 1) {
        const float sg = us::bf2f(us::f2bf(silu_f(us::bf2f(us::f2bf(gate)))));
        val = us::bf2f(us::f2bf(val)) * sg;
      } else {
        val = val * gelu_tanh_f(gate);
      }
    }
    val += bias;
    if (route_rows != nullptr) return val * route_w[route_rows[r]];
    if (scale_rows != nullptr && !scale_first) val *= scale_rows[r];
    return val;
  }
  // Destination of tile row r, feature m0 (null = the row is dropped).
  __device__ __forceinline__ char* row_ptr(int r) const {
    if (tile_base != nullptr) return tile_base + (long long)r * row_bytes;
    if (route_rows != nullptr) {
      const int i = route_rows[r];
      const int src = i / route_per;
      const int dst = i - src * route_per;
      return (char*)a.peer_out[src] + ((size_t)dst * ldo + m0) * 2;
    }
    const int orow = out_rows[r];
    if (orow < 0) return nullptr;
    return out + ((size_t)orow * ldo + m0) * esz;
  }
  // Scalar store of one element (split-K reduction, unaligned destinations).
  __device__ __forceinline__ void store(int r, float val, float gate) const {
    if (!m_ok) return;
    char* dst = row_ptr(r);
    if (dst == nullptr) return;
    const float x = value(r, val, gate);
    if (esz == 2)
      ((__nv_bfloat16*)dst)[ml] = us::f2bf(x);
    else
      ((float*)dst)[ml] = x;
  }
  // Rows [c, c + 16) of the tile, called by all 128 epilogue threads together.
  // `stage` is kEpiStageBytes of shared memory; chunks alternate its halves, so
  // one named barrier per chunk orders writers and readers.
  __device__ __forceinline__ void store_chunk16(int c, int chunk, const uint32_t (&v)[16],
                                                const uint32_t (&g)[16], int nrows,
                                                uint8_t* stage) const {
    if (!vec_store) {
#pragma unroll
      for (int j = 0; j < 16; ++j)
        if (c + j < nrows) store(c + j, __uint_as_float(v[j]), DUAL ? __uint_as_float(g[j]) : 0.f);
      return;
    }
    const uint32_t buf = tc::smem_u32(stage) + (uint32_t)(chunk & 1) * (kEpiStageBytes / 2);
    // fast path: nothing per row but the gated activation and the bias
    const bool plain = scale_rows == nullptr && route_rows == nullptr;
    if (esz == 2) {
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        float x = 0.f;
        if (c + j < nrows) {
          if (plain && !DUAL)
            x = __uint_as_float(v[j]) + bias;
          else
            x = value(c + j, __uint_as_float(v[j]), DUAL ? __uint_as_float(g[j]) : 0.f);
        }
        const unsigned short h = __bfloat16_as_ushort(us::f2bf(x));
        asm volatile("st.shared.u16 [%0], %1;" ::"r"(buf + (uint32_t)(j * 256 + ml * 2)), "h"(h)
                     : "memory");
      }
    } else {
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        float x = 0.f;
        if (c + j < nrows)
          x = value(c + j, __uint_as_float(v[j]), DUAL ? __uint_as_float(g[j]) : 0.f);
        asm volatile("st.shared.f32 [%0], %1;" ::"r"(buf + (uint32_t)(j * 512 + ml * 4)), "f"(x)
                     : "memory");
      }
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");
    // 16-byte pieces: 16 per row (bf16, 8 features each) or 32 per row (fp32, 4 each)
    const int shift = esz == 2 ? 4 : 5;
    const int feats = esz == 2 ? 8 : 4;
    const int pieces = 16 << shift;
    for (int id = ml; id < pieces; id += 128) {
      const int r = id >> shift, seg = id & ((1 << shift) - 1);
      if (c + r >= nrows) continue;
      char* dst = row_ptr(c + r);
      if (dst == nullptr) continue;
      const int f0 = m0 + seg * feats;
      uint4 piece;
      asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                   : "=r"(piece.x), "=r"(piece.y), "=r"(piece.z), "=r"(piece.w)
                   : "r"(buf + (uint32_t)(id * 16))
                   : "memory");
      if (f0 + feats <= M) {
        *reinterpret_cast<uint4*>(dst + seg * 16) = piece;
      } else {
        const uint32_t w[4] = {piece.x, piece.y, piece.z, piece.w};
        for (int f = 0; f0 + f < M && f < feats; ++f) {
          if (esz == 2)
            ((unsigned short*)dst)[seg * feats + f] =
                (unsigned short)(w[f >> 1] >> ((f & 1) * 16));
          else
            ((uint32_t*)dst)[seg * feats + f] = w[f];
        }
      }
    }
  }
};

}  // namespace
