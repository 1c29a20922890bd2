// Argument block and per-thread epilogue shared by the weight-stationary GEMM
// kernels (bf16 and block-scaled fp8).
#pragma once
#include "us_common.cuh"
#include "us_tmap.h"

namespace {

struct GemmArgs {
  int M;            // output features per group
  int K;
  int rows;         // activation rows (dense)
  int dual_offset;  // row offset of the second weight tile (dual epilogue)
  int stages;
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
  // Route push (expert-parallel combine): permuted row r carries route
  // i = route_map[r] = (source rank * route_per + token * top_k + slot); the epilogue
  // multiplies by the gate weight route_w[i] and stores the row into the source
  // rank's combine buffer at row i % route_per.
  const int* route_map;
  const float* route_w;
  int route_per;
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

// Per-thread epilogue of one output feature `m`: activation, bias, row scale,
// row map, rounding.  The destination of row 0 of the tile is resolved once
// (which buffer, which rank); rows then advance by a fixed stride unless a row
// map or a route map redirects them one by one.
template <bool DUAL>
struct Epilogue {
  const GemmArgs& a;
  const int m, row0;
  const bool m_ok;
  float bias;
  char* base;          // element (row0, m) of the destination; null = per-row lookup
  long long row_bytes;
  __device__ __forceinline__ Epilogue(const GemmArgs& args, int group, int m_, int row0_)
      : a(args), m(m_), row0(row0_), m_ok(m_ < args.M), bias(0.f), base(nullptr), row_bytes(0) {
    if (!m_ok) return;
    if (a.bias != nullptr) {
      const size_t bi = (size_t)group * a.M + m;
      bias = a.bias_dtype == 0 ? us::bf2f(((const __nv_bfloat16*)a.bias)[bi])
                               : ((const float*)a.bias)[bi];
    }
    const int esz = a.out_dtype == 0 ? 2 : 4;
    row_bytes = a.ldo * esz;
    if (a.route_map != nullptr || a.out_row_map != nullptr) return;
    if (a.peer_rows > 0) {   // a tile lies inside one owner's interval
      const int p = row0 / a.peer_rows;
      base = (char*)a.peer_out[p] +
             (((size_t)a.peer_slot * a.peer_rows + (size_t)(row0 - p * a.peer_rows)) * a.ldo + m) *
                 esz;
    } else if (a.peer_cols > 0) {
      const int p = m / a.peer_cols;
      base = (char*)a.peer_out[p] +
             ((size_t)(a.peer_row_offset + row0) * a.ldo + (m - p * a.peer_cols)) * esz;
    } else {
      base = (char*)a.out + ((size_t)row0 * a.ldo + m) * esz;
    }
  }
  __device__ __forceinline__ void store(int r, float val, float gate) const {
    if (!m_ok) return;
    if (DUAL) {
      if (a.act == 0) {
        val = val * silu_f(gate);
      } else if (a.act == 1) {
        const float sg = us::bf2f(us::f2bf(silu_f(us::bf2f(us::f2bf(gate)))));
        val = us::bf2f(us::f2bf(val)) * sg;
      } else {
        val = val * gelu_tanh_f(gate);
      }
    }
    val += bias;
    int orow = row0 + r;
    if (a.route_map != nullptr) {
      const int i = a.route_map[orow];
      const int src = i / a.route_per;
      const int dst = i - src * a.route_per;
      ((__nv_bfloat16*)a.peer_out[src])[(size_t)dst * a.ldo + m] = us::f2bf(val * a.route_w[i]);
      return;
    }
    if (a.row_scale != nullptr) val *= a.row_scale[orow];
    if (base != nullptr) {
      char* dst = base + (long long)r * row_bytes;
      if (a.out_dtype == 0)
        *(__nv_bfloat16*)dst = us::f2bf(val);
      else
        *(float*)dst = val;
      return;
    }
    orow = a.out_row_map[orow];
    if (orow < 0) return;
    const size_t o = (size_t)orow * a.ldo + m;
    if (a.out_dtype == 0)
      ((__nv_bfloat16*)a.out)[o] = us::f2bf(val);
    else
      ((float*)a.out)[o] = val;
  }
};

}  // namespace
