// Small data-movement kernels of the token path: embedding lookup (vocab-shard
// aware), row gather, device-side slot advance between decode steps, dtype
// casts and fills.
//
// Reference behaviour: crates/ops/kernels/{embedding,logits_gather,slot_commit,cast}/triton
// (reference project paths).
#include "include/us_common.cuh"

namespace {

__global__ void __launch_bounds__(256)
embedding_kernel(const int* __restrict__ ids, const __nv_bfloat16* __restrict__ table, int H,
                 int vocab_lo, int vocab_hi, __nv_bfloat16* __restrict__ out) {
  US_PDL_PROLOGUE();
  const int t = blockIdx.x;
  const int id = ids[t];
  uint4* dst = reinterpret_cast<uint4*>(out + (long long)t * H);
  if (id < vocab_lo || id >= vocab_hi) {
    for (int v = threadIdx.x; v < (H >> 3); v += blockDim.x) dst[v] = make_uint4(0, 0, 0, 0);
    return;
  }
  const uint4* src = reinterpret_cast<const uint4*>(table + (long long)(id - vocab_lo) * H);
  for (int v = threadIdx.x; v < (H >> 3); v += blockDim.x) dst[v] = src[v];
}

__global__ void __launch_bounds__(256)
gather_rows_kernel(const __nv_bfloat16* __restrict__ src, const int* __restrict__ idx, int H,
                   long long lds, __nv_bfloat16* __restrict__ dst) {
  US_PDL_PROLOGUE();
  const int r = blockIdx.x;
  const int s = idx[r];
  uint4* d = reinterpret_cast<uint4*>(dst + (long long)r * H);
  if (s < 0) {
    for (int v = threadIdx.x; v < (H >> 3); v += blockDim.x) d[v] = make_uint4(0, 0, 0, 0);
    return;
  }
  const uint4* p = reinterpret_cast<const uint4*>(src + (long long)s * lds);
  for (int v = threadIdx.x; v < (H >> 3); v += blockDim.x) d[v] = p[v];
}

// After a decode step: the sampled token becomes the next input, the position
// and the sequence length advance and the next cache slot is looked up in the
// page table, all on the device, so the next step can be enqueued (or a whole
// run of steps replayed from one graph) before the host has read anything.
__global__ void decode_advance_kernel(const int* __restrict__ sampled, int* __restrict__ input_ids,
                                      int* __restrict__ positions, int* __restrict__ seq_lens,
                                      int* __restrict__ slots, const int* __restrict__ page_table,
                                      int max_pages, int page_size, int B,
                                      const int* __restrict__ live, int* __restrict__ history,
                                      int history_stride, int history_rows,
                                      const int* __restrict__ step) {
  US_PDL_PROLOGUE();
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= B) return;
  const bool on = !live || b < *live;
  const int tok = sampled[b];
  if (history && step && *step >= 0 && *step < history_rows)
    history[(long long)(*step) * history_stride + b] = on ? tok : -1;
  if (!on) {
    slots[b] = -1;
    return;
  }
  input_ids[b] = tok;
  const int pos = positions[b] + 1;
  positions[b] = pos;
  seq_lens[b] = pos + 1;
  const int page_idx = pos / page_size;
  slots[b] = page_idx < max_pages
                 ? page_table[(long long)b * max_pages + page_idx] * page_size + pos % page_size
                 : -1;
}

__global__ void bump_kernel(int* p) {
  US_PDL_PROLOGUE(); *p += 1; }

__global__ void __launch_bounds__(256)
cast_f32_bf16_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, long long n) {
  US_PDL_PROLOGUE();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x)
    dst[i] = us::f2bf(src[i]);
}
__global__ void __launch_bounds__(256)
cast_bf16_f32_kernel(const __nv_bfloat16* __restrict__ src, float* __restrict__ dst, long long n) {
  US_PDL_PROLOGUE();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x)
    dst[i] = us::bf2f(src[i]);
}

}  // namespace

US_API int us_embedding(const int* ids, const void* table, int T, int H, int vocab_lo,
                        int vocab_hi, void* out, void* stream) {
  US_REQUIRE(ids && table && out && T >= 0 && (H % 8) == 0);
  if (T == 0) return US_OK;
  us::launch_pdl(embedding_kernel, dim3(T), dim3(256), 0, (cudaStream_t)stream, ids, (const __nv_bfloat16*)table, H,
                                                        vocab_lo, vocab_hi, (__nv_bfloat16*)out);
  US_LAUNCH_CHECK();
  return US_OK;
}

US_API int us_gather_rows(const void* src, const int* idx, int M, int H, long long lds, void* dst,
                          void* stream) {
  US_REQUIRE(src && idx && dst && M >= 0 && (H % 8) == 0 && (lds % 8) == 0);
  if (M == 0) return US_OK;
  us::launch_pdl(gather_rows_kernel, dim3(M), dim3(256), 0, (cudaStream_t)stream, (const __nv_bfloat16*)src, idx, H, lds,
                                                          (__nv_bfloat16*)dst);
  US_LAUNCH_CHECK();
  return US_OK;
}

US_API int us_decode_advance(const int* sampled, int* input_ids, int* positions, int* seq_lens,
                             int* slots, const int* page_table, int max_pages, int page_size,
                             int B, const int* live, int* history, int history_stride,
                             int history_rows, int* step, void* stream_) {
  US_REQUIRE(sampled && input_ids && positions && seq_lens && slots && page_table && B >= 0);
  if (B == 0) return US_OK;
  cudaStream_t stream = (cudaStream_t)stream_;
  us::launch_pdl(decode_advance_kernel, dim3((B + 127) / 128), dim3(128), 0, stream, sampled, input_ids, positions,
                                                             seq_lens, slots, page_table, max_pages,
                                                             page_size, B, live, history,
                                                             history_stride, history_rows, step);
  US_LAUNCH_CHECK();
  if (step) {
    us::launch_pdl(bump_kernel, dim3(1), dim3(1), 0, stream, step);
    US_LAUNCH_CHECK();
  }
  return US_OK;
}

US_API int us_cast(const void* src, void* dst, long long n, int to_bf16, void* stream) {
  US_REQUIRE(src && dst && n >= 0);
  if (n == 0) return US_OK;
  const int blocks = (int)((n + 256 * 8 - 1) / (256 * 8) < 65535 ? (n + 256 * 8 - 1) / (256 * 8)
                                                                  : 65535);
  if (to_bf16)
    us::launch_pdl(cast_f32_bf16_kernel, dim3(blocks), dim3(256), 0, (cudaStream_t)stream, (const float*)src,
                                                                   (__nv_bfloat16*)dst, n);
  else
    us::launch_pdl(cast_bf16_f32_kernel, dim3(blocks), dim3(256), 0, (cudaStream_t)stream, (const __nv_bfloat16*)src,
                                                                   (float*)dst, n);
  US_LAUNCH_CHECK();
  return US_OK;
}
