// Fence probe: one warp stamps the GPU's global nanosecond timer (and the SM
// clock) into a slot of a pinned host buffer when the stream reaches it.  The
// store has system scope and release semantics, so a host thread that sees the
// stamp also sees everything the stream wrote before the probe.  Probes cost one
// tiny launch each; a step normally carries two (begin, end).
//
// Reference behaviour: crates/ops/kernels/range_marker/nvcc/src/range_marker.cu,
// crates/engine/src/profiling/markers.rs (reference project paths).
#include "include/us_common.cuh"

namespace {

__global__ void __launch_bounds__(32)
range_marker_kernel(unsigned long long* __restrict__ slots, int index, unsigned long long tag) {
  US_PDL_PROLOGUE();
  if (threadIdx.x != 0) return;
  unsigned long long t, c;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  asm volatile("mov.u64 %0, %%clock64;" : "=l"(c));
  unsigned long long* s = slots + (size_t)index * 4;
  s[1] = c;
  s[2] = tag;
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(s), "l"(t) : "memory");
}

}  // namespace

// slots: pinned host memory (device-accessible), 4 x u64 per probe:
// [timer ns, SM clock, tag, unused].
US_API int us_range_marker(void* slots, int index, unsigned long long tag, void* stream) {
  US_REQUIRE(slots && index >= 0);
  US_CUDA_CHECK(us::launch_pdl(range_marker_kernel, dim3(1), dim3(32), 0, (cudaStream_t)stream,
                               (unsigned long long*)slots, index, tag));
  return US_OK;
}
