// Symmetric peer-memory heaps and the collectives fused into their consumers.
//
// Every rank (one process per GPU) allocates a heap with cudaMalloc, exports it as
// a CUDA IPC handle and maps every peer's heap, so a kernel can load and store any
// rank's heap directly over NVLink.  A process may hold several heaps (one per
// parallel axis: tensor, Ulysses, ...); every entry point takes the heap it works
// on.  Layout of a heap:
//
//   [flags: sites x kMaxCtas x kMaxRanks uint32] [data: sites x site_bytes]
//
// A *site* is a named buffer with its own flags.  Flags carry a monotonically
// growing epoch that each CTA keeps in local memory; nothing in a launch depends
// on a host-side counter, so captured graphs replay correctly.  The flag protocol
// is per CTA index: every rank must launch the same grid for the same use of a
// site (the grids are functions of the row count, which is equal on all ranks).
//
// Decode-size all-reduce, push form (us_symm_allreduce_add_rmsnorm): the CTA of a
// row stores this rank's partial row into slot [rank] of the site on EVERY peer,
// raises one flag per peer, waits (bounded) for the peers' flags in its OWN memory,
// then sums the P slots from its OWN memory in rank order, adds the FP32 residual
// stream and normalises.  A row crosses NVLink once, as fire-and-forget stores; no
// load ever waits on a remote read.  The partial row is either read from a local
// tensor (the output of a row-parallel GEMM) or formed on the fly as the weighted
// sum of the token's local expert rows (the MoE un-permute), so expert output
// -> all-reduce -> residual add -> RMSNorm is one launch.  Slots are double-buffered
// by the parity of the CTA's epoch: the stores of use e + 2 can only start after
// this rank saw every peer's flag of use e + 1, which a peer raises after it has
// read use e; so a site may be reused back to back, by any number of uses.
//
// The pull-form kernels (allreduce, allgather) read the peers' site buffers after
// an arrival barrier.  They have no release barrier: their buffer may be rewritten
// only after another barrier was crossed in between (the host wrapper inserts one
// when a site is reused back to back).
//
// The reference sums these tensors with NCCL all_reduce
// (crates/nn/src/modules/linear.rs:684, moe.rs:740, reference project paths).
#include <string.h>

#include <mutex>
#include <vector>

#include "../include/us_common.cuh"
#include "../include/us_peer.cuh"

namespace {

constexpr int kMaxRanks = peer::kMaxRanks;
constexpr int kMaxCtas = 256;

struct Symm {
  int world = 0, rank = 0;
  int sites = 0;
  size_t site_bytes = 0, heap_bytes = 0, flag_bytes = 0;
  uint8_t* local = nullptr;
  uint8_t* peers[kMaxRanks] = {nullptr};
  unsigned int* epochs = nullptr;  // [sites][kMaxCtas], local only
  bool opened[kMaxRanks] = {false};
  bool loopback = false;           // peers are further local allocations (tests)
};

std::mutex g_mu;
std::vector<Symm*> g_heaps;

bool known(const Symm* s) {
  std::lock_guard<std::mutex> lock(g_mu);
  for (const Symm* h : g_heaps)
    if (h == s) return true;
  return false;
}

using PeerTable = peer::Table;
using peer::ld_acquire_sys;
using peer::st_release_sys;

__device__ __forceinline__ uint4 ld_peer16(const void* p) { return peer::ld16_sys(p); }

// Next epoch of (site, cta), published to the CTA through shared memory.
__device__ __forceinline__ unsigned int next_epoch(unsigned int* epochs, int site, int cta,
                                                   unsigned int* smem_flag) {
  if (threadIdx.x == 0) {
    unsigned int* e = epochs + (size_t)site * kMaxCtas + cta;
    *smem_flag = *e + 1;
    *e = *e + 1;
  }
  __syncthreads();
  return *smem_flag;
}

// Tells every peer "this CTA's part of this site is ready at epoch ep" and waits until every
// peer has announced the same epoch.  Returns false when a peer did not arrive in time.
__device__ __forceinline__ bool announce_and_wait(const PeerTable& pt, int world, int rank,
                                                  int site, int cta, unsigned int ep,
                                                  unsigned int* status) {
  const size_t slot = ((size_t)site * kMaxCtas + cta) * kMaxRanks;
  bool ok = true;
  if ((int)threadIdx.x < world) {
    const int r = threadIdx.x;
    __threadfence_system();
    st_release_sys(reinterpret_cast<unsigned int*>(pt.base[r]) + slot + rank, ep);
    const unsigned int* mine = reinterpret_cast<const unsigned int*>(pt.base[rank]) + slot + r;
    ok = peer::wait_flag(mine, ep, status);
  }
  __syncthreads();
  return ok;
}

__device__ __forceinline__ bool site_barrier(const PeerTable& pt, int world, int rank, int site,
                                             int cta, unsigned int* epochs, unsigned int* status,
                                             unsigned int* smem_flag) {
  const unsigned int ep = next_epoch(epochs, site, cta, smem_flag);
  return announce_and_wait(pt, world, rank, site, cta, ep, status);
}

constexpr int kVecPerThread = 4;   // hidden sizes up to 4 x 256 x 8 = 8192

// Push-form all-reduce + residual add + RMSNorm of one row per CTA (see the file header).
// Partial row: `partial` [T, H] bf16, or (when `perm` is given) the weighted sum over the
// token's top_k routes of the rows y_perm[perm[t, j]] (perm < 0: the route is not local).
__global__ void __launch_bounds__(256)
allreduce_push_add_rmsnorm_kernel(PeerTable pt, int world, int rank, int site, size_t data_off,
                                  size_t slot_bytes, unsigned int* epochs,
                                  const __nv_bfloat16* __restrict__ partial,
                                  const __nv_bfloat16* __restrict__ y_perm,
                                  const int* __restrict__ perm,
                                  const float* __restrict__ weights, int top_k,
                                  float* __restrict__ residual,
                                  const __nv_bfloat16* __restrict__ w,
                                  __nv_bfloat16* __restrict__ y, int H, float eps, int first,
                                  unsigned int* status) {
  US_PDL_PROLOGUE();
  __shared__ float scratch[33];
  __shared__ unsigned int flag;
  const int row = blockIdx.x;
  const int nvec = H >> 3;
  const unsigned int ep = next_epoch(epochs, site, row, &flag);
  const size_t parity = ep & 1u;
  us::Pack16 mine[kVecPerThread];
#pragma unroll
  for (int i = 0; i < kVecPerThread; ++i) {
    const int v = threadIdx.x + i * 256;
    if (v >= nvec) break;
    if (perm) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int j = 0; j < top_k; ++j) {
        const int p = perm[(size_t)row * top_k + j];
        if (p < 0) continue;
        const float wj = weights[(size_t)row * top_k + j];
        us::Pack16 q;
        q.u = *reinterpret_cast<const uint4*>(y_perm + (size_t)p * H + v * 8);
#pragma unroll
        for (int c = 0; c < 8; ++c) acc[c] += wj * us::bf2f(q.b[c]);
      }
#pragma unroll
      for (int c = 0; c < 8; ++c) mine[i].b[c] = us::f2bf(acc[c]);
    } else {
      mine[i].u = *reinterpret_cast<const uint4*>(partial + (size_t)row * H + v * 8);
    }
    // this rank's slot on every peer: [parity][rank][row][H]
    const size_t off = data_off + (parity * world + rank) * slot_bytes +
                       ((size_t)row * H + (size_t)v * 8) * sizeof(__nv_bfloat16);
    for (int r = 0; r < world; ++r)
      if (r != rank) peer::st16_sys(pt.base[r] + off, mine[i].u);
  }
  // one system-scope fence per flag (by the thread that raises it, after this barrier) orders
  // the whole CTA's stores before the flag; a fence per storing thread costs microseconds
  __syncthreads();
  announce_and_wait(pt, world, rank, site, row, ep, status);
  float* rr = residual + (size_t)row * H;
  __nv_bfloat16* yr = y + (size_t)row * H;
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < kVecPerThread; ++i) {
    const int v = threadIdx.x + i * 256;
    if (v >= nvec) break;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int r = 0; r < world; ++r) {      // rank order: every rank forms the same sum
      us::Pack16 p;
      if (r == rank) {
        p.u = mine[i].u;
      } else {
        const size_t off = data_off + (parity * world + r) * slot_bytes +
                           ((size_t)row * H + (size_t)v * 8) * sizeof(__nv_bfloat16);
        p.u = ld_peer16(pt.base[rank] + off);
      }
#pragma unroll
      for (int c = 0; c < 8; ++c) acc[c] += us::bf2f(p.b[c]);
    }
    float4 r0 = make_float4(0.f, 0.f, 0.f, 0.f), r1 = r0;
    if (!first) {
      r0 = *reinterpret_cast<const float4*>(rr + v * 8);
      r1 = *reinterpret_cast<const float4*>(rr + v * 8 + 4);
    }
    r0.x += acc[0]; r0.y += acc[1]; r0.z += acc[2]; r0.w += acc[3];
    r1.x += acc[4]; r1.y += acc[5]; r1.z += acc[6]; r1.w += acc[7];
    *reinterpret_cast<float4*>(rr + v * 8) = r0;
    *reinterpret_cast<float4*>(rr + v * 8 + 4) = r1;
    ss += r0.x * r0.x + r0.y * r0.y + r0.z * r0.z + r0.w * r0.w;
    ss += r1.x * r1.x + r1.y * r1.y + r1.z * r1.z + r1.w * r1.w;
  }
  ss = us::block_sum(ss, scratch);
  const float inv = rsqrtf(ss / (float)H + eps);
#pragma unroll
  for (int i = 0; i < kVecPerThread; ++i) {
    const int v = threadIdx.x + i * 256;
    if (v >= nvec) break;
    const float4 r0 = *reinterpret_cast<const float4*>(rr + v * 8);
    const float4 r1 = *reinterpret_cast<const float4*>(rr + v * 8 + 4);
    us::Pack16 q, o;
    q.u = *reinterpret_cast<const uint4*>(w + v * 8);
    o.b[0] = us::f2bf(r0.x * inv * us::bf2f(q.b[0]));
    o.b[1] = us::f2bf(r0.y * inv * us::bf2f(q.b[1]));
    o.b[2] = us::f2bf(r0.z * inv * us::bf2f(q.b[2]));
    o.b[3] = us::f2bf(r0.w * inv * us::bf2f(q.b[3]));
    o.b[4] = us::f2bf(r1.x * inv * us::bf2f(q.b[4]));
    o.b[5] = us::f2bf(r1.y * inv * us::bf2f(q.b[5]));
    o.b[6] = us::f2bf(r1.z * inv * us::bf2f(q.b[6]));
    o.b[7] = us::f2bf(r1.w * inv * us::bf2f(q.b[7]));
    *reinterpret_cast<uint4*>(yr + v * 8) = o.u;
  }
}

// Greedy token of a vocabulary-sharded head: every rank finds the maximum of its own logits
// columns, pushes (value, global column) to every peer, and all ranks pick the same winner
// (largest value, lowest column on ties).  One CTA per row; slots are double-buffered by epoch
// parity like the all-reduce's.
__global__ void __launch_bounds__(512)
argmax_exchange_kernel(PeerTable pt, int world, int rank, int site, size_t data_off,
                       unsigned int* epochs, const float* __restrict__ logits, long long ld,
                       int cols, int col0, int rows_cap, int* __restrict__ out,
                       unsigned int* status) {
  US_PDL_PROLOGUE();
  __shared__ float sv[16];
  __shared__ int si[16];
  __shared__ unsigned int flag;
  const int row = blockIdx.x;
  const unsigned int ep = next_epoch(epochs, site, row, &flag);
  const size_t parity = ep & 1u;
  const float* lr = logits + (size_t)row * ld;
  float best = -INFINITY;
  int best_i = 0x7fffffff;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) {
    const float v = lr[c];
    if (v > best) {           // ascending c per thread keeps the lowest column on ties
      best = v;
      best_i = c;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ob = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
    if (ob > best || (ob == best && oi < best_i)) {
      best = ob;
      best_i = oi;
    }
  }
  if ((threadIdx.x & 31) == 0) {
    sv[threadIdx.x >> 5] = best;
    si[threadIdx.x >> 5] = best_i;
  }
  __syncthreads();
  if (threadIdx.x < 32) {
    const int nw = blockDim.x >> 5;
    best = threadIdx.x < nw ? sv[threadIdx.x] : -INFINITY;
    best_i = threadIdx.x < nw ? si[threadIdx.x] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
      if (ob > best || (ob == best && oi < best_i)) {
        best = ob;
        best_i = oi;
      }
    }
  }
  // slot of (parity, source rank, row): one (value, column) pair of 8 bytes
  const size_t slot0 = data_off + parity * (size_t)world * rows_cap * 8;
  if ((int)threadIdx.x < world && (int)threadIdx.x != rank) {
    const float v = __shfl_sync(0xffffffffu, best, 0);
    const int gi = __shfl_sync(0xffffffffu, best_i, 0);
    uint2 pr = make_uint2(__float_as_uint(v), (unsigned int)(gi == 0x7fffffff ? gi : gi + col0));
    asm volatile("st.relaxed.sys.global.v2.u32 [%0], {%1,%2};" ::"l"(
                     pt.base[threadIdx.x] + slot0 + ((size_t)rank * rows_cap + row) * 8),
                 "r"(pr.x), "r"(pr.y)
                 : "memory");
  } else if (threadIdx.x < 32) {
    (void)__shfl_sync(0xffffffffu, best, 0);
    (void)__shfl_sync(0xffffffffu, best_i, 0);
  }
  if (threadIdx.x == 0) {
    sv[0] = best;
    si[0] = best_i == 0x7fffffff ? best_i : best_i + col0;
  }
  __syncthreads();
  announce_and_wait(pt, world, rank, site, row, ep, status);
  if (threadIdx.x == 0) {
    float bv = sv[0];
    int bi = si[0];
    for (int r = 0; r < world; ++r) {
      if (r == rank) continue;
      uint2 pr;
      asm volatile("ld.relaxed.sys.global.v2.u32 {%0,%1}, [%2];"
                   : "=r"(pr.x), "=r"(pr.y)
                   : "l"(pt.base[rank] + slot0 + ((size_t)r * rows_cap + row) * 8)
                   : "memory");
      const float v = __uint_as_float(pr.x);
      const int gi = (int)pr.y;
      if (v > bv || (v == bv && gi < bi)) {
        bv = v;
        bi = gi;
      }
    }
    out[row] = bi;
  }
}

// Plain sum of the P partial buffers of a site into a local tensor (bf16 or fp32
// elements; `elem` = bytes per element).  One CTA per `chunk` of 16-byte units.
__global__ void __launch_bounds__(256)
allreduce_kernel(PeerTable pt, int world, int rank, int site, size_t data_off,
                 unsigned int* epochs, void* __restrict__ out, long long units16, int is_f32,
                 unsigned int* status) {
  US_PDL_PROLOGUE();
  __shared__ unsigned int flag;
  site_barrier(pt, world, rank, site, blockIdx.x, epochs, status, &flag);
  const long long per = (units16 + gridDim.x - 1) / gridDim.x;
  const long long lo = (long long)blockIdx.x * per;
  const long long hi = lo + per < units16 ? lo + per : units16;
  for (long long u = lo + threadIdx.x; u < hi; u += blockDim.x) {
    if (is_f32) {
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int r = 0; r < world; ++r) {
        const uint4 v = ld_peer16(pt.base[r] + data_off + (size_t)u * 16);
        acc.x += __uint_as_float(v.x); acc.y += __uint_as_float(v.y);
        acc.z += __uint_as_float(v.z); acc.w += __uint_as_float(v.w);
      }
      reinterpret_cast<float4*>(out)[u] = acc;
    } else {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int r = 0; r < world; ++r) {
        us::Pack16 p;
        p.u = ld_peer16(pt.base[r] + data_off + (size_t)u * 16);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] += us::bf2f(p.b[i]);
      }
      us::Pack16 o;
#pragma unroll
      for (int i = 0; i < 8; ++i) o.b[i] = us::f2bf(acc[i]);
      reinterpret_cast<uint4*>(out)[u] = o.u;
    }
  }
}

// All-gather of equal blocks: rank r's block (already in its site buffer) is
// copied from every peer into out[r * units16 ...].
__global__ void __launch_bounds__(256)
allgather_kernel(PeerTable pt, int world, int rank, int site, size_t data_off,
                 unsigned int* epochs, void* __restrict__ out, long long units16,
                 unsigned int* status) {
  US_PDL_PROLOGUE();
  __shared__ unsigned int flag;
  site_barrier(pt, world, rank, site, blockIdx.x, epochs, status, &flag);
  const long long per = (units16 + gridDim.x - 1) / gridDim.x;
  const long long lo = (long long)blockIdx.x * per;
  const long long hi = lo + per < units16 ? lo + per : units16;
  for (int r = 0; r < world; ++r)
    for (long long u = lo + threadIdx.x; u < hi; u += blockDim.x)
      reinterpret_cast<uint4*>(out)[(long long)r * units16 + u] =
          ld_peer16(pt.base[r] + data_off + (size_t)u * 16);
}


PeerTable table(const Symm& s) {
  PeerTable t;
  for (int i = 0; i < kMaxRanks; ++i) t.base[i] = s.peers[i];
  return t;
}

size_t site_off(const Symm& s, int site) { return s.flag_bytes + (size_t)site * s.site_bytes; }

int create(Symm** out, int world, int rank, int sites, long long site_bytes) {
  Symm* s = new Symm();
  s->world = world; s->rank = rank; s->sites = sites; s->site_bytes = (size_t)site_bytes;
  s->flag_bytes = (((size_t)sites * kMaxCtas * kMaxRanks * 4) + 255) & ~(size_t)255;
  s->heap_bytes = s->flag_bytes + (size_t)sites * s->site_bytes;
  if (cudaMalloc(&s->local, s->heap_bytes) != cudaSuccess ||
      cudaMemset(s->local, 0, s->heap_bytes) != cudaSuccess ||
      cudaMalloc(&s->epochs, (size_t)sites * kMaxCtas * 4) != cudaSuccess ||
      cudaMemset(s->epochs, 0, (size_t)sites * kMaxCtas * 4) != cudaSuccess ||
      cudaDeviceSynchronize() != cudaSuccess) {
    us_set_last_cuda_error((int)cudaGetLastError(), __FILE__, __LINE__);
    if (s->local) cudaFree(s->local);
    if (s->epochs) cudaFree(s->epochs);
    delete s;
    return US_ERR_CUDA;
  }
  s->peers[rank] = s->local;
  {
    std::lock_guard<std::mutex> lock(g_mu);
    g_heaps.push_back(s);
  }
  *out = s;
  return US_OK;
}

}  // namespace

#define US_HEAP(h)                               \
  Symm* sp_ = (Symm*)(h);                        \
  US_REQUIRE(sp_ != nullptr && known(sp_));      \
  Symm& s = *sp_

// Allocates a heap on the current device; writes its 64-byte IPC handle and the heap handle
// every other entry point takes.
US_API int us_symm_create(int world, int rank, int sites, long long site_bytes,
                          unsigned char* handle_out, void** heap_out) {
  US_REQUIRE(world >= 1 && world <= kMaxRanks && rank >= 0 && rank < world && sites >= 1);
  US_REQUIRE(site_bytes > 0 && (site_bytes % 256) == 0 && handle_out && heap_out);
  Symm* s = nullptr;
  const int rc = create(&s, world, rank, sites, site_bytes);
  if (rc != US_OK) return rc;
  cudaIpcMemHandle_t h;
  US_CUDA_CHECK(cudaIpcGetMemHandle(&h, s->local));
  memcpy(handle_out, &h, sizeof(h));
  *heap_out = s;
  return US_OK;
}

// A heap whose "peers" are further allocations of this process on the same device: nothing
// ever writes them unless the caller does.  For single-GPU tests of the failure path (a flag
// that never arrives) and of the data paths of one rank.
US_API int us_symm_create_loopback(int world, int rank, int sites, long long site_bytes,
                                   void** heap_out) {
  US_REQUIRE(world >= 1 && world <= kMaxRanks && rank >= 0 && rank < world && sites >= 1);
  US_REQUIRE(site_bytes > 0 && (site_bytes % 256) == 0 && heap_out);
  Symm* s = nullptr;
  const int rc = create(&s, world, rank, sites, site_bytes);
  if (rc != US_OK) return rc;
  s->loopback = true;
  for (int r = 0; r < world; ++r) {
    if (r == rank) continue;
    US_CUDA_CHECK(cudaMalloc(&s->peers[r], s->heap_bytes));
    US_CUDA_CHECK(cudaMemset(s->peers[r], 0, s->heap_bytes));
    s->opened[r] = true;
  }
  US_CUDA_CHECK(cudaDeviceSynchronize());
  *heap_out = s;
  return US_OK;
}

// Maps the peers' heaps; `handles` holds world x 64 bytes in rank order.
US_API int us_symm_attach(void* heap, const unsigned char* handles) {
  US_HEAP(heap);
  US_REQUIRE(handles != nullptr && !s.loopback);
  for (int r = 0; r < s.world; ++r) {
    if (r == s.rank || s.opened[r]) continue;
    cudaIpcMemHandle_t h;
    memcpy(&h, handles + (size_t)r * sizeof(h), sizeof(h));
    void* p = nullptr;
    US_CUDA_CHECK(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
    s.peers[r] = (uint8_t*)p;
    s.opened[r] = true;
  }
  return US_OK;
}

US_API int us_symm_destroy(void* heap) {
  US_HEAP(heap);
  for (int r = 0; r < kMaxRanks; ++r)
    if (s.opened[r]) {
      if (s.loopback) cudaFree(s.peers[r]);
      else cudaIpcCloseMemHandle(s.peers[r]);
      s.opened[r] = false;
    }
  if (s.local) cudaFree(s.local);
  if (s.epochs) cudaFree(s.epochs);
  {
    std::lock_guard<std::mutex> lock(g_mu);
    for (size_t i = 0; i < g_heaps.size(); ++i)
      if (g_heaps[i] == sp_) {
        g_heaps.erase(g_heaps.begin() + i);
        break;
      }
  }
  delete sp_;
  return US_OK;
}

// Zeroes this rank's flags and epochs (stream-ordered).  After a failed wait the ranks'
// epochs may disagree: every rank calls this between two host-side barriers, with none of its
// kernels in flight, before the heap is used again.
US_API int us_symm_reset(void* heap, void* stream) {
  US_HEAP(heap);
  US_CUDA_CHECK(cudaMemsetAsync(s.local, 0, s.flag_bytes, (cudaStream_t)stream));
  US_CUDA_CHECK(cudaMemsetAsync(s.epochs, 0, (size_t)s.sites * kMaxCtas * 4,
                                (cudaStream_t)stream));
  return US_OK;
}

// Device address of this rank's buffer of a site (producers write there).
US_API void* us_symm_site_ptr(void* heap, int site) {
  Symm* s = (Symm*)heap;
  if (!s || !known(s) || site < 0 || site >= s->sites) return nullptr;
  return s->local + site_off(*s, site);
}

US_API long long us_symm_site_bytes(void* heap) {
  Symm* s = (Symm*)heap;
  return (s && known(s)) ? (long long)s->site_bytes : 0;
}

// Address, in this process, of rank `rank`'s buffer of a site (for kernels that
// store to or TMA-load from a peer).
US_API void* us_symm_peer_site_ptr(void* heap, int rank, int site) {
  Symm* s = (Symm*)heap;
  if (!s || !known(s) || site < 0 || site >= s->sites || rank < 0 || rank >= s->world)
    return nullptr;
  return s->peers[rank] + site_off(*s, site);
}

// Push-form all-reduce of T <= 256 partial rows + residual add + RMSNorm.  The partial rows
// come from `partial` [T, H] bf16, or (perm != NULL) are formed as the weighted sum of the
// token's local expert rows: y_perm [R, H], perm [T, top_k] (row of y_perm or -1), weights
// [T, top_k] f32.  The site must hold 2 x world x T x H bf16.
US_API int us_symm_allreduce_add_rmsnorm(void* heap, int site, const void* partial,
                                         const void* y_perm, const int* perm,
                                         const float* weights, int top_k, void* residual,
                                         const void* w, void* y, int T, int H, float eps,
                                         int first, void* stream) {
  US_HEAP(heap);
  US_REQUIRE(site >= 0 && site < s.sites && T >= 1 && T <= kMaxCtas && (H % 8) == 0);
  US_REQUIRE(H <= 8 * 256 * kVecPerThread && residual && w && y);
  US_REQUIRE((partial != nullptr) != (perm != nullptr));
  US_REQUIRE(!perm || (y_perm && weights && top_k >= 1));
  const size_t slot_bytes = (size_t)T * H * 2;
  US_REQUIRE(2 * (size_t)s.world * slot_bytes <= s.site_bytes);
  US_CUDA_CHECK(us::launch_pdl(allreduce_push_add_rmsnorm_kernel, dim3(T), dim3(256), 0,
                               (cudaStream_t)stream, table(s), s.world, s.rank, site,
                               site_off(s, site), slot_bytes, s.epochs,
                               (const __nv_bfloat16*)partial, (const __nv_bfloat16*)y_perm, perm,
                               weights, top_k, (float*)residual, (const __nv_bfloat16*)w,
                               (__nv_bfloat16*)y, H, eps, first, us_status_ptr()));
  return US_OK;
}

// Greedy tokens of a vocabulary-sharded head: logits [B, >= cols] f32 with row stride `ld`
// hold this rank's columns [col0, col0 + cols) of the vocabulary; out [B] int32 is the same on
// every rank.  B <= 256; the site must hold 2 x world x B x 8 bytes.
US_API int us_symm_argmax(void* heap, int site, const void* logits, long long ld, int B,
                          int cols, int col0, void* out, void* stream) {
  US_HEAP(heap);
  US_REQUIRE(site >= 0 && site < s.sites && B >= 1 && B <= kMaxCtas && cols >= 0 && logits &&
             out && ld >= cols);
  US_REQUIRE(2 * (size_t)s.world * B * 8 <= s.site_bytes);
  US_CUDA_CHECK(us::launch_pdl(argmax_exchange_kernel, dim3(B), dim3(512), 0,
                               (cudaStream_t)stream, table(s), s.world, s.rank, site,
                               site_off(s, site), s.epochs, (const float*)logits, ld, cols, col0,
                               B, (int*)out, us_status_ptr()));
  return US_OK;
}

US_API int us_symm_allreduce(void* heap, int site, void* out, long long nbytes, int is_f32,
                             void* stream) {
  US_HEAP(heap);
  US_REQUIRE(site >= 0 && site < s.sites && out && nbytes > 0 && (nbytes % 16) == 0);
  US_REQUIRE((size_t)nbytes <= s.site_bytes);
  const long long units = nbytes / 16;
  int ctas = (int)((units + 1023) / 1024);
  if (ctas > kMaxCtas) ctas = kMaxCtas;
  if (ctas < 1) ctas = 1;
  US_CUDA_CHECK(us::launch_pdl(allreduce_kernel, dim3(ctas), dim3(256), 0, (cudaStream_t)stream,
                               table(s), s.world, s.rank, site, site_off(s, site), s.epochs, out,
                               units, is_f32, us_status_ptr()));
  return US_OK;
}

US_API int us_symm_allgather(void* heap, int site, void* out, long long nbytes_per_rank,
                             void* stream) {
  US_HEAP(heap);
  US_REQUIRE(site >= 0 && site < s.sites && out && nbytes_per_rank > 0);
  US_REQUIRE((nbytes_per_rank % 16) == 0 && (size_t)nbytes_per_rank <= s.site_bytes);
  const long long units = nbytes_per_rank / 16;
  int ctas = (int)((units + 1023) / 1024);
  if (ctas > kMaxCtas) ctas = kMaxCtas;
  if (ctas < 1) ctas = 1;
  US_CUDA_CHECK(us::launch_pdl(allgather_kernel, dim3(ctas), dim3(256), 0, (cudaStream_t)stream,
                               table(s), s.world, s.rank, site, site_off(s, site), s.epochs, out,
                               units, us_status_ptr()));
  return US_OK;
}

namespace {
__global__ void barrier_kernel(PeerTable pt, int world, int rank, int site, unsigned int* epochs,
                               unsigned int* status) {
  US_PDL_PROLOGUE();
  __shared__ unsigned int flag;
  site_barrier(pt, world, rank, site, 0, epochs, status, &flag);
}
}  // namespace

// Stream-ordered barrier over the group: everything this rank launched before
// it (including stores into peers' heaps) is visible to every rank's work
// launched after it.  Bounded like every other wait.
US_API int us_symm_barrier(void* heap, int site, void* stream) {
  US_HEAP(heap);
  US_REQUIRE(site >= 0 && site < s.sites);
  US_CUDA_CHECK(us::launch_pdl(barrier_kernel, dim3(1), dim3(32), 0, (cudaStream_t)stream,
                               table(s), s.world, s.rank, site, s.epochs, us_status_ptr()));
  return US_OK;
}
