// Decode attention without any allocation.  This entry point has no counterpart in the reference
// (zhangjianbang-nb/qwen25vl-lite); it exists for callers of this library that cannot allocate.
//
// Who cannot allocate.  The split-KV decode attention (q25_attention_decode_bf16) needs scratch
// memory for the partial results of its key ranges, and leaves it to the caller to bring that
// buffer.  Some callers have nowhere to get one from at the moment of the call:
//   * a serving process that sized its KV-cache pool to the last free byte of the device, so a
//     later cudaMalloc fails;
//   * a host runtime that owns all device memory through its own pool and forbids its plug-ins
//     to call the CUDA allocator (the allocation would bypass its accounting);
//   * a step loop with work in flight on other streams: cudaMalloc and cudaFree synchronise the
//     whole device, which stalls those streams for the length of the call.
// For them this variant keeps the scratch in a file-scope `static __device__` array inside the
// library.  The caller still passes every input and the output.
//
// What it costs and what to know.
//   * The array is Q25_NOALLOC_SCRATCH_FLOATS floats (16 MiB).  Every GPU on which the library is
//     loaded holds it until the process exits, whether or not this entry point is ever called.
//   * A call needs n_items * nq * n_splits * (head_dim + 2) floats when n_splits > 1 (none for one
//     split).  A call that needs more than the array holds is refused: the function returns
//     Q25_NOALLOC_TOO_LARGE and launches nothing; q25_attention_decode_noalloc_error() then gives
//     a message with both numbers.  Use fewer splits, or the allocating entry point.  The number
//     of splits itself has no limit of its own (the combine step walks any number of partials);
//     the array's size is the only bound.
//   * The first call on a device looks up the array's device address (cudaGetSymbolAddress, with
//     that device current) and keeps it; later calls on that device reuse it.  Make that first
//     call before any stream capture begins.
//   * All calls share the one array, and it keeps what the last call left.  Nothing in it has to
//     start at zero: every launch writes each partial it later reads.  Two calls whose kernels
//     overlap on the GPU (different streams, no ordering between them) race on the array and
//     corrupt each other's results; order them, or give at most one of them more than one split.
//   * No cudaMalloc, cudaFree or allocating library routine is called, on any path.
//
// Arguments are those of q25_attention_decode_bf16 without the scratch pointer; the return value
// is 0, a cudaError_t of the set-up or the launch, or Q25_NOALLOC_TOO_LARGE.
#pragma once

#define Q25_NOALLOC_SCRATCH_FLOATS (4 * 1024 * 1024)
#define Q25_NOALLOC_TOO_LARGE (-2)

#ifdef __cplusplus
extern "C" {
#endif

int q25_attention_decode_bf16_noalloc(const void* qkv, int qkv_stride, void* out, const void* k_pages,
                                      const void* v_pages, const int* block_table, int table_width, const int* cu_q,
                                      const int* q_start_pos, const int* items, int n_items, int nq, int nkv,
                                      int head_dim, int page_size, int window, float scale, int n_splits, void* stream);

// Message of the last refusal or set-up failure of this thread's calls ("" if none).
const char* q25_attention_decode_noalloc_error(void);

#ifdef __cplusplus
}
#endif
