// Symmetric peer-memory heap and the collectives fused into their consumers.
//
// Every rank (one process per GPU) allocates one heap with cudaMalloc, exports
// it as a CUDA IPC handle and maps every peer's heap, so a kernel can load and
// store any rank's heap directly over NVLink.  Layout of a heap:
//
//   [flags: sites x kMaxCtas x kMaxRanks uint32] [data: sites x site_bytes]
//
// A *site* is one collective call position inside a forward pass (layer i's
// attention output, layer i's expert output, ...).  Each site owns its buffer
// and its flags, so a buffer is rewritten only a whole forward pass later, after
// every peer has long finished reading it.  Flags carry a monotonically growing
// epoch that each CTA keeps in local memory; nothing in a launch depends on a
// host-side counter, so captured graphs replay correctly.
//
// all_reduce + residual add + RMSNorm in one kernel: the producer (a GEMM or the
// expert un-permute) writes this rank's partial rows straight into the site
// buffer; the consumer CTA of a row tells every peer "my partial is ready",
// waits (bounded) for theirs, sums the P partial rows in rank order through
// peer loads, adds the FP32 residual stream and normalises.  There is no
// separate collective launch.
//
// The reference sums these tensors with NCCL all_reduce
// (crates/nn/src/modules/linear.rs:684, moe.rs:740, reference project paths).
#include <string.h>

#include "../include/us_common.cuh"

namespace {

constexpr int kMaxRanks = 8;
constexpr int kMaxCtas = 256;
constexpr long long kPeerWaitClocks = 3000000000LL;  // about 1.5 s

struct Symm {
  int world = 0, rank = 0;
  int sites = 0;
  size_t site_bytes = 0, heap_bytes = 0, flag_bytes = 0;
  uint8_t* local = nullptr;
  uint8_t* peers[kMaxRanks] = {nullptr};
  unsigned int* epochs = nullptr;  // [sites][kMaxCtas], local only
  bool opened[kMaxRanks] = {false};
};
Symm g_symm;

struct PeerTable {
  uint8_t* base[kMaxRanks];
};

__device__ __forceinline__ void st_release_sys(unsigned int* p, unsigned int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint4 ld_peer16(const void* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}

// Announces "my partial of this CTA's rows at this site is ready" to every
// peer and waits until every peer has announced the same epoch.  Returns false
// when a peer did not arrive within the budget.
__device__ __forceinline__ bool site_barrier(const PeerTable& pt, int world, int rank, int site,
                                             int cta, unsigned int* epochs, unsigned int* status,
                                             unsigned int* smem_flag) {
  const size_t slot = ((size_t)site * kMaxCtas + cta) * kMaxRanks;
  if (threadIdx.x == 0) {
    unsigned int* e = epochs + (size_t)site * kMaxCtas + cta;
    *smem_flag = *e + 1;
    *e = *e + 1;
  }
  __syncthreads();
  const unsigned int ep = *smem_flag;
  bool ok = true;
  if ((int)threadIdx.x < world) {
    const int r = threadIdx.x;
    __threadfence_system();
    st_release_sys(reinterpret_cast<unsigned int*>(pt.base[r]) + slot + rank, ep);
    const unsigned int* mine = reinterpret_cast<const unsigned int*>(pt.base[rank]) + slot + r;
    const long long t0 = clock64();
    // Once any wait of this process has failed the status word is set; later
    // waits give up at once so a lost peer costs one budget, not one per launch.
    const long long budget = (status && *(volatile unsigned int*)status) ? 0 : kPeerWaitClocks;
    while ((int)(ld_acquire_sys(mine) - ep) < 0) {
      if (clock64() - t0 > budget) {
        ok = false;
        us_dev_fail(status, US_DEV_TIMEOUT_PEER);
        break;
      }
    }
  }
  __syncthreads();
  return ok;
}

__global__ void __launch_bounds__(256)
allreduce_add_rmsnorm_kernel(PeerTable pt, int world, int rank, int site, size_t data_off,
                             unsigned int* epochs, float* __restrict__ residual,
                             const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y,
                             int H, float eps, int first, unsigned int* status) {
  US_PDL_PROLOGUE();
  __shared__ float scratch[33];
  __shared__ unsigned int flag;
  const int row = blockIdx.x;
  site_barrier(pt, world, rank, site, row, epochs, status, &flag);
  float* rr = residual + (size_t)row * H;
  __nv_bfloat16* yr = y + (size_t)row * H;
  const size_t off = data_off + (size_t)row * H * sizeof(__nv_bfloat16);
  const int nvec = H >> 3;
  float ss = 0.f;
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int r = 0; r < world; ++r) {
      us::Pack16 p;
      p.u = ld_peer16(pt.base[r] + off + (size_t)v * 16);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] += us::bf2f(p.b[i]);
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
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
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

PeerTable table() {
  PeerTable t;
  for (int i = 0; i < kMaxRanks; ++i) t.base[i] = g_symm.peers[i];
  return t;
}

}  // namespace

// Allocates this rank's heap and writes its 64-byte IPC handle.
US_API int us_symm_create(int world, int rank, int sites, long long site_bytes,
                          unsigned char* handle_out) {
  US_REQUIRE(world >= 1 && world <= kMaxRanks && rank >= 0 && rank < world && sites >= 1);
  US_REQUIRE(site_bytes > 0 && (site_bytes % 256) == 0 && g_symm.local == nullptr);
  Symm& s = g_symm;
  s.world = world; s.rank = rank; s.sites = sites; s.site_bytes = (size_t)site_bytes;
  s.flag_bytes = (((size_t)sites * kMaxCtas * kMaxRanks * 4) + 255) & ~(size_t)255;
  s.heap_bytes = s.flag_bytes + (size_t)sites * s.site_bytes;
  US_CUDA_CHECK(cudaMalloc(&s.local, s.heap_bytes));
  US_CUDA_CHECK(cudaMemset(s.local, 0, s.heap_bytes));
  US_CUDA_CHECK(cudaMalloc(&s.epochs, (size_t)sites * kMaxCtas * 4));
  US_CUDA_CHECK(cudaMemset(s.epochs, 0, (size_t)sites * kMaxCtas * 4));
  US_CUDA_CHECK(cudaDeviceSynchronize());
  cudaIpcMemHandle_t h;
  US_CUDA_CHECK(cudaIpcGetMemHandle(&h, s.local));
  memcpy(handle_out, &h, sizeof(h));
  s.peers[rank] = s.local;
  return US_OK;
}

// Maps the peers' heaps; `handles` holds world x 64 bytes in rank order.
US_API int us_symm_attach(const unsigned char* handles) {
  Symm& s = g_symm;
  US_REQUIRE(s.local != nullptr && handles != nullptr);
  for (int r = 0; r < s.world; ++r) {
    if (r == s.rank) continue;
    cudaIpcMemHandle_t h;
    memcpy(&h, handles + (size_t)r * sizeof(h), sizeof(h));
    void* p = nullptr;
    US_CUDA_CHECK(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
    s.peers[r] = (uint8_t*)p;
    s.opened[r] = true;
  }
  return US_OK;
}

US_API int us_symm_destroy() {
  Symm& s = g_symm;
  for (int r = 0; r < kMaxRanks; ++r)
    if (s.opened[r]) {
      cudaIpcCloseMemHandle(s.peers[r]);
      s.opened[r] = false;
    }
  if (s.local) cudaFree(s.local);
  if (s.epochs) cudaFree(s.epochs);
  s = Symm();
  return US_OK;
}

// Device address of this rank's buffer of a site (producers write there).
US_API void* us_symm_site_ptr(int site) {
  Symm& s = g_symm;
  if (!s.local || site < 0 || site >= s.sites) return nullptr;
  return s.local + s.flag_bytes + (size_t)site * s.site_bytes;
}

US_API long long us_symm_site_bytes() { return (long long)g_symm.site_bytes; }

US_API int us_allreduce_add_rmsnorm(int site, void* residual, const void* w, void* y, int T, int H,
                                    float eps, int first, void* stream) {
  Symm& s = g_symm;
  US_REQUIRE(s.local && site >= 0 && site < s.sites && T >= 1 && T <= kMaxCtas && (H % 8) == 0);
  US_REQUIRE((size_t)T * H * 2 <= s.site_bytes && residual && w && y);
  us::launch_pdl(allreduce_add_rmsnorm_kernel, dim3(T), dim3(256), 0, (cudaStream_t)stream, table(), s.world, s.rank, site, s.flag_bytes + (size_t)site * s.site_bytes, s.epochs,
      (float*)residual, (const __nv_bfloat16*)w, (__nv_bfloat16*)y, H, eps, first,
      us_status_ptr());
  US_LAUNCH_CHECK();
  return US_OK;
}

US_API int us_symm_allreduce(int site, void* out, long long nbytes, int is_f32, void* stream) {
  Symm& s = g_symm;
  US_REQUIRE(s.local && site >= 0 && site < s.sites && out && nbytes > 0 && (nbytes % 16) == 0);
  US_REQUIRE((size_t)nbytes <= s.site_bytes);
  const long long units = nbytes / 16;
  int ctas = (int)((units + 1023) / 1024);
  if (ctas > kMaxCtas) ctas = kMaxCtas;
  if (ctas < 1) ctas = 1;
  us::launch_pdl(allreduce_kernel, dim3(ctas), dim3(256), 0, (cudaStream_t)stream, table(), s.world, s.rank, site, s.flag_bytes + (size_t)site * s.site_bytes, s.epochs, out,
      units, is_f32, us_status_ptr());
  US_LAUNCH_CHECK();
  return US_OK;
}

US_API int us_symm_allgather(int site, void* out, long long nbytes_per_rank, void* stream) {
  Symm& s = g_symm;
  US_REQUIRE(s.local && site >= 0 && site < s.sites && out && nbytes_per_rank > 0);
  US_REQUIRE((nbytes_per_rank % 16) == 0 && (size_t)nbytes_per_rank <= s.site_bytes);
  const long long units = nbytes_per_rank / 16;
  int ctas = (int)((units + 1023) / 1024);
  if (ctas > kMaxCtas) ctas = kMaxCtas;
  if (ctas < 1) ctas = 1;
  us::launch_pdl(allgather_kernel, dim3(ctas), dim3(256), 0, (cudaStream_t)stream, table(), s.world, s.rank, site, s.flag_bytes + (size_t)site * s.site_bytes, s.epochs, out,
      units, us_status_ptr());
  US_LAUNCH_CHECK();
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

// Address, in this process, of rank `rank`'s buffer of a site (for kernels that
// store to or TMA-load from a peer).
US_API void* us_symm_peer_site_ptr(int rank, int site) {
  Symm& s = g_symm;
  if (!s.local || site < 0 || site >= s.sites || rank < 0 || rank >= s.world) return nullptr;
  return s.peers[rank] + s.flag_bytes + (size_t)site * s.site_bytes;
}

// Stream-ordered barrier over the group: everything this rank launched before
// it (including stores into peers' heaps) is visible to every rank's work
// launched after it.  Bounded like every other wait.
US_API int us_symm_barrier(int site, void* stream) {
  Symm& s = g_symm;
  US_REQUIRE(s.local && site >= 0 && site < s.sites);
  us::launch_pdl(barrier_kernel, dim3(1), dim3(32), 0, (cudaStream_t)stream, table(), s.world, s.rank, site, s.epochs,
                                                     us_status_ptr());
  US_LAUNCH_CHECK();
  return US_OK;
}
