// Expert-parallel token exchange over peer memory, fused into its neighbours.
//
// Layout: every rank owns T local tokens per step (data-parallel attention) and
// E / P whole experts.  Per MoE layer:
//
// The windows are laid out with the step's row count T as the per-source stride
// (every rank runs the same T in a step), so a decode step of 64 rows sorts
// P x 64 x k routes, not the prefill capacity.
//
//   source rank   route_dispatch   one CTA per token: stores the token's row once into
//                                  the window of every rank that owns one of its top-k
//                                  experts, and its ids / gate weights into every rank's
//                                  window; the CTA that finishes last raises this rank's
//                                  "dispatched" flag at every peer.
//   expert rank   moe_sort (waits for every source's flag in its prologue) -> gather ->
//                 grouped FC1 -> grouped FC2 whose epilogue multiplies by the gate weight
//                 and stores each output row straight into the token owner's combine
//                 buffer (peer stores from the GEMM epilogue) -> ep_signal.
//   source rank   combine_add_rmsnorm: waits for every expert rank's "combined" flag,
//                 sums the token's k weighted rows in FP32 (local reads), adds the
//                 residual stream and normalises - the next layer's input norm.
//
// Attention-FFN disaggregation is the same exchange with disjoint roles: attention
// ranks only dispatch and combine, expert ranks only sort / compute / push.
//
// Windows are single-buffered: a source can dispatch layer L+1 only after its
// combine of layer L, which every expert rank's FC2 of layer L precedes, and an
// expert rank pushes layer L+1 only after every source dispatched L+1, which each
// source's combine of layer L precedes.  Flags carry per-rank epochs kept on the
// device, so captured graphs replay.
//
// Reference behaviour: crates/ops/kernels/expert_exchange/alltoall/src/exchange.cu:357-469
// (dispatch), :537-614 (combine), crates/nn/src/functional/moe.rs:1344-1402 (reference
// project paths).  Unlike there, every wait here is bounded.
#include <string.h>

#include "../include/us_common.cuh"
#include "../include/us_peer.cuh"

namespace {

struct Ep {
  int world = 0, rank = 0;
  int T = 0, k = 0, H = 0;
  size_t off_x = 0, off_ids = 0, off_w = 0, off_recv = 0, off_flags = 0, bytes = 0;
  uint8_t* local = nullptr;
  uint8_t* peers[peer::kMaxRanks] = {nullptr};
  bool opened[peer::kMaxRanks] = {false};
  unsigned int* state = nullptr;   // [0] dispatch epoch, [1] combine epoch, [2] done counter,
                                   // [3] dispatch epochs seen by sort, [4] combine epochs seen
};
// One exchange per handle: a process may hold several (one per expert union it belongs to,
// or one per micro-batch window).
peer::Table table(const Ep& e) {
  peer::Table t;
  for (int i = 0; i < peer::kMaxRanks; ++i) t.base[i] = e.peers[i];
  return t;
}

// flags: [2][kMaxRanks] uint32 at off_flags: [0][src] = src dispatched epoch, [1][src] = src
// (expert rank) combined epoch.

__global__ void __launch_bounds__(256)
route_dispatch_kernel(peer::Table pt, int world, int rank, const __nv_bfloat16* __restrict__ x,
                      const int* __restrict__ ids, const float* __restrict__ weights,
                      const int* __restrict__ live, int T, int k, int H, int experts_per_rank,
                      int first_expert_rank, size_t off_x, size_t off_ids, size_t off_w,
                      size_t off_flags, unsigned int* state) {
  US_PDL_PROLOGUE();
  const int t = blockIdx.x;
  const bool on = !live || t < *live;
  __shared__ unsigned int targets;
  if (threadIdx.x == 0) targets = 0;
  __syncthreads();
  if ((int)threadIdx.x < k) {
    const int e = on ? ids[(size_t)t * k + threadIdx.x] : -1;
    if (e >= 0) atomicOr(&targets, 1u << (first_expert_rank + e / experts_per_rank));
  }
  __syncthreads();
  const unsigned int tg = targets;
  // ids / weights go to every rank (a rank must see -1 for rows that skip it)
  for (int i = threadIdx.x; i < world * k; i += blockDim.x) {
    const int p = i / k, j = i - p * k;
    const int e = on ? ids[(size_t)t * k + j] : -1;
    const bool mine = e >= 0 && (first_expert_rank + e / experts_per_rank) == p;
    int* dst_i = reinterpret_cast<int*>(pt.base[p] + off_ids) + ((size_t)rank * T + t) * k + j;
    float* dst_w = reinterpret_cast<float*>(pt.base[p] + off_w) + ((size_t)rank * T + t) * k + j;
    *dst_i = mine ? e : -1;
    *dst_w = mine ? weights[(size_t)t * k + j] : 0.f;
  }
  const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)t * H);
  for (int p = 0; p < world; ++p) {
    if (!(tg >> p & 1u)) continue;
    uint4* dst = reinterpret_cast<uint4*>(pt.base[p] + off_x) + ((size_t)rank * T + t) * (H >> 3);
    for (int v = threadIdx.x; v < (H >> 3); v += blockDim.x) peer::st16_sys(dst + v, src[v]);
  }
  // One fence per CTA, by the thread that counts the CTA in: the barrier orders every thread's
  // stores before it, and a fence per thread cost more than the stores themselves (membar
  // stalls were two thirds of this kernel's issue slots).
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    const unsigned int done = atomicAdd(&state[2], 1u);
    if (done == gridDim.x - 1) {
      state[2] = 0;
      const unsigned int ep = ++state[0];
      __threadfence_system();
      for (int p = 0; p < world; ++p)
        peer::st_release_sys(reinterpret_cast<unsigned int*>(pt.base[p] + off_flags) + rank, ep);
    }
  }
}

// Waits until every rank in [lo, hi) has raised flag row `which` to the next epoch.
__global__ void ep_wait_kernel(peer::Table pt, int rank, int lo, int hi, int which,
                               size_t off_flags, unsigned int* state, unsigned int* status) {
  US_PDL_PROLOGUE();
  __shared__ unsigned int ep;
  if (threadIdx.x == 0) ep = ++state[3 + which];
  __syncthreads();
  const int p = lo + threadIdx.x;
  if (p < hi)
    peer::wait_flag(reinterpret_cast<const unsigned int*>(pt.base[rank] + off_flags) +
                        which * peer::kMaxRanks + p, ep, status);
}

// Raises this rank's flag of row `which` at the ranks in [lo, hi).
__global__ void ep_signal_kernel(peer::Table pt, int rank, int lo, int hi, int which,
                                 size_t off_flags, unsigned int* state) {
  US_PDL_PROLOGUE();
  __shared__ unsigned int ep;
  if (threadIdx.x == 0) ep = ++state[which];
  __syncthreads();
  __threadfence_system();
  const int p = lo + threadIdx.x;
  if (p < hi)
    peer::st_release_sys(reinterpret_cast<unsigned int*>(pt.base[p] + off_flags) +
                             which * peer::kMaxRanks + rank, ep);
}

// One CTA per token: wait for the expert ranks, sum the k weighted rows, add the
// residual, normalise.  Rows at or past `live` produce zeros.
__global__ void __launch_bounds__(256)
combine_add_rmsnorm_kernel(peer::Table pt, int rank, int lo, int hi, size_t off_recv,
                           size_t off_flags, const int* __restrict__ ids,
                           const int* __restrict__ live, float* __restrict__ residual,
                           const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y,
                           int k, int H, float eps, unsigned int* state, unsigned int* status) {
  US_PDL_PROLOGUE();
  __shared__ float scratch[33];
  __shared__ unsigned int ep;
  const int t = blockIdx.x;
  if (threadIdx.x == 0) ep = state[4] + 1;     // bumped once per launch by the last CTA below
  __syncthreads();
  const int p = lo + threadIdx.x;
  if (p < hi)
    peer::wait_flag(reinterpret_cast<const unsigned int*>(pt.base[rank] + off_flags) +
                        peer::kMaxRanks + p, ep, status);
  __syncthreads();
  const bool on = !live || t < *live;
  float* rr = residual + (size_t)t * H;
  __nv_bfloat16* yr = y + (size_t)t * H;
  const __nv_bfloat16* rows =
      reinterpret_cast<const __nv_bfloat16*>(pt.base[rank] + off_recv) + (size_t)t * k * H;
  const int nvec = H >> 3;
  float ss = 0.f;
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (on) {
      for (int j = 0; j < k; ++j) {
        if (ids[(size_t)t * k + j] < 0) continue;
        us::Pack16 q;
        q.u = peer::ld16_sys(rows + (size_t)j * H + v * 8);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] += us::bf2f(q.b[i]);
      }
    }
    float4 r0 = *reinterpret_cast<const float4*>(rr + v * 8);
    float4 r1 = *reinterpret_cast<const float4*>(rr + v * 8 + 4);
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
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int done = atomicAdd(&state[5], 1u);
    if (done == gridDim.x - 1) {
      state[5] = 0;
      state[4] = ep;
    }
  }
}

}  // namespace

// Allocates this rank's exchange heap (windows for T tokens per source rank, top-k k,
// hidden H) and writes its IPC handle.
US_API int us_ep_create(int world, int rank, int T, int k, int H, unsigned char* handle_out,
                        void** ep_out) {
  US_REQUIRE(world >= 1 && world <= peer::kMaxRanks && rank >= 0 && rank < world);
  US_REQUIRE(T >= 1 && k >= 1 && k <= 32 && (H % 8) == 0 && handle_out && ep_out);
  Ep* ep = new Ep();
  *ep_out = ep;
  Ep& e = *ep;
  e.world = world; e.rank = rank; e.T = T; e.k = k; e.H = H;
  auto align = [](size_t v) { return (v + 255) & ~(size_t)255; };
  e.off_flags = 0;
  e.off_x = align(2 * peer::kMaxRanks * 4);
  e.off_ids = e.off_x + align((size_t)world * T * H * 2);
  e.off_w = e.off_ids + align((size_t)world * T * k * 4);
  e.off_recv = e.off_w + align((size_t)world * T * k * 4);
  e.bytes = e.off_recv + align((size_t)T * k * H * 2);
  US_CUDA_CHECK(cudaMalloc(&e.local, e.bytes));
  US_CUDA_CHECK(cudaMemset(e.local, 0, e.bytes));
  US_CUDA_CHECK(cudaMemset(e.local + e.off_ids, 0xff, (size_t)world * T * k * 4));
  US_CUDA_CHECK(cudaMalloc(&e.state, 64));
  US_CUDA_CHECK(cudaMemset(e.state, 0, 64));
  US_CUDA_CHECK(cudaDeviceSynchronize());
  cudaIpcMemHandle_t h;
  US_CUDA_CHECK(cudaIpcGetMemHandle(&h, e.local));
  memcpy(handle_out, &h, sizeof(h));
  e.peers[rank] = e.local;
  return US_OK;
}

US_API int us_ep_attach(void* ep, const unsigned char* handles) {
  US_REQUIRE(ep && handles);
  Ep& e = *(Ep*)ep;
  US_REQUIRE(e.local);
  for (int r = 0; r < e.world; ++r) {
    if (r == e.rank) continue;
    cudaIpcMemHandle_t h;
    memcpy(&h, handles + (size_t)r * sizeof(h), sizeof(h));
    void* p = nullptr;
    US_CUDA_CHECK(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
    e.peers[r] = (uint8_t*)p;
    e.opened[r] = true;
  }
  return US_OK;
}

US_API int us_ep_destroy(void* ep) {
  if (!ep) return US_OK;
  Ep& e = *(Ep*)ep;
  for (int r = 0; r < peer::kMaxRanks; ++r)
    if (e.opened[r]) cudaIpcCloseMemHandle(e.peers[r]);
  if (e.local) cudaFree(e.local);
  if (e.state) cudaFree(e.state);
  delete (Ep*)ep;
  return US_OK;
}

// Pointers the expert side of the layer needs: this rank's windows and, for the FC2
// epilogue, every source rank's combine buffer.
US_API void* us_ep_window(void* ep, int which) {   // 0 rows, 1 ids, 2 weights, 3 recv
  if (!ep) return nullptr;
  Ep& e = *(Ep*)ep;
  if (!e.local) return nullptr;
  const size_t off[4] = {e.off_x, e.off_ids, e.off_w, e.off_recv};
  return which >= 0 && which < 4 ? e.local + off[which] : nullptr;
}
US_API void* us_ep_peer_recv(void* ep, int rank) {
  if (!ep) return nullptr;
  Ep& e = *(Ep*)ep;
  return (e.local && rank >= 0 && rank < e.world) ? e.peers[rank] + e.off_recv : nullptr;
}

US_API int us_ep_route_dispatch(void* ep, const void* x, const int* ids, const float* weights,
                                const int* live, int T, int experts_per_rank,
                                int first_expert_rank, void* stream) {
  US_REQUIRE(ep);
  Ep& e = *(Ep*)ep;
  US_REQUIRE(e.local && x && ids && weights && T >= 1 && T <= e.T && experts_per_rank >= 1);
  us::launch_pdl(route_dispatch_kernel, dim3(T), dim3(256), 0, (cudaStream_t)stream, table(e), e.world, e.rank, (const __nv_bfloat16*)x, ids, weights, live, T, e.k, e.H,
      experts_per_rank, first_expert_rank, e.off_x, e.off_ids, e.off_w, e.off_flags, e.state);
  US_LAUNCH_CHECK();
  return US_OK;
}

// which: 0 = wait for the source ranks' dispatch, 1 = wait for the expert ranks' combine.
US_API int us_ep_wait(void* ep, int which, int lo, int hi, void* stream) {
  US_REQUIRE(ep);
  Ep& e = *(Ep*)ep;
  US_REQUIRE(e.local && (which == 0 || which == 1) && lo >= 0 && hi <= e.world && lo < hi);
  us::launch_pdl(ep_wait_kernel, dim3(1), dim3(32), 0, (cudaStream_t)stream, table(e), e.rank, lo, hi, which, e.off_flags,
                                                     e.state, us_status_ptr());
  US_LAUNCH_CHECK();
  return US_OK;
}

// Expert rank: "my pushes of this layer are complete" to the source ranks [lo, hi).
US_API int us_ep_signal_combined(void* ep, int lo, int hi, void* stream) {
  US_REQUIRE(ep);
  Ep& e = *(Ep*)ep;
  US_REQUIRE(e.local && lo >= 0 && hi <= e.world && lo < hi);
  us::launch_pdl(ep_signal_kernel, dim3(1), dim3(32), 0, (cudaStream_t)stream, table(e), e.rank, lo, hi, 1, e.off_flags,
                                                       e.state);
  US_LAUNCH_CHECK();
  return US_OK;
}

US_API int us_ep_combine_add_rmsnorm(void* ep, const int* ids, const int* live, void* residual,
                                     const void* w, void* y, int T, float eps, int expert_lo,
                                     int expert_hi, void* stream) {
  US_REQUIRE(ep);
  Ep& e = *(Ep*)ep;
  US_REQUIRE(e.local && ids && residual && w && y && T >= 1 && T <= e.T);
  us::launch_pdl(combine_add_rmsnorm_kernel, dim3(T), dim3(256), 0, (cudaStream_t)stream, table(e), e.rank, expert_lo, expert_hi, e.off_recv, e.off_flags, ids, live, (float*)residual,
      (const __nv_bfloat16*)w, (__nv_bfloat16*)y, e.k, e.H, eps, e.state, us_status_ptr());
  US_LAUNCH_CHECK();
  return US_OK;
}
