// Allocation-free C entry point for split-KV paged decode attention.
//
// This entry point has no counterpart in the reference project. It exists for callers that cannot allocate device memory
// at the moment of the call: code running inside a stream capture or a latency-critical serving loop where cudaMalloc (an
// implicit device synchronisation) is off limits, plugins that are handed raw device pointers by a host framework and own no
// allocator, and bindings from languages without a torch runtime. The torch-facing op allocates its split-KV partial buffers
// per call; here they live in a file-scope `static __device__` array inside the library, so the call performs no cudaMalloc,
// no cudaFree and no allocating library routine. The caller still owns inputs and outputs.
//
// Limits and rules:
//   * scratch capacity is DLV_NOALLOC_SCRATCH_FLOATS floats (4 MiB) per GPU that loads the library, held until the process
//     exits; a call needs num_seqs * num_heads * splits * (head_dim + 2) floats and is rejected with
//     DLV_NOALLOC_TOO_LARGE when that exceeds the capacity (nothing is launched);
//   * the first call on each device resolves the scratch address (cudaGetSymbolAddress) with that device current; make this
//     first call before any stream capture begins;
//   * every call on a device shares the same scratch and finds the previous call's contents in it (each launch overwrites
//     all the partials it later reads, so nothing needs clearing), therefore two calls whose kernels may overlap on the GPU
//     (different streams, no dependency) race: serialise them on one stream or with events.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

#define DLV_NOALLOC_SCRATCH_FLOATS (1u << 20)

enum {
  DLV_NOALLOC_OK = 0,
  DLV_NOALLOC_BAD_ARGUMENT = 1,   // null pointer, unsupported head_dim / group size, q / k_cache / v_cache not 16-byte aligned,
                                  // q_stride not a multiple of 8 elements, out not 4-byte aligned, page size not a multiple of 32
  DLV_NOALLOC_TOO_LARGE = 2,      // the partial buffers would not fit in the built-in scratch
  DLV_NOALLOC_CUDA_ERROR = 3      // a CUDA runtime call failed; see dlv_noalloc_last_cuda_error()
};

// q: bf16 rows, row t at q + t * q_stride elements, heads contiguous [num_heads, head_dim]; q must be 16-byte aligned and
// q_stride a multiple of 8 elements (rows are read with 16-byte loads); k_cache / v_cache 16-byte aligned as well.
// k_cache / v_cache: bf16 [pages, kv_heads, page_size, head_dim]. block_tables: int32 [num_seqs, bt_stride]. ctx_lens: int32.
// out: bf16 [num_seqs, num_heads * head_dim]. splits >= 1 (1 uses no scratch at all).
int dlv_decode_attention_noalloc(const void* q, long long q_stride, const void* k_cache, const void* v_cache, const int* block_tables,
                                 int bt_stride, const int* ctx_lens, void* out, int num_seqs, int num_heads, int kv_heads, int head_dim,
                                 int page_size, float scale, float softcap, int window, int splits, cudaStream_t stream);

// floats of scratch a call with these sizes needs (0 when splits <= 1)
unsigned long long dlv_decode_attention_noalloc_scratch_floats(int num_seqs, int num_heads, int head_dim, int splits);

// the cudaError_t recorded by the last call that returned DLV_NOALLOC_CUDA_ERROR (as an int)
int dlv_noalloc_last_cuda_error(void);

#ifdef __cplusplus
}
#endif
