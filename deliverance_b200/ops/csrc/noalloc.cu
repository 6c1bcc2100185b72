// Allocation-free split-KV decode attention: see noalloc.h for who needs it and the rules that come with it.
#include "noalloc.h"

#include "gemm_api.h"

namespace {

// Split-KV partials for every call on this device. In host code this name is only a handle for the runtime: kernels must
// be given the device address obtained with cudaGetSymbolAddress, never `g_scratch` itself.
static __device__ __align__(256) float g_scratch[DLV_NOALLOC_SCRATCH_FLOATS];

constexpr int kMaxDevices = 64;
float* g_scratch_addr[kMaxDevices] = {nullptr};
int g_last_cuda_error = 0;

// Resolves (once per device, with that device current) the device address of the scratch array.
int scratch_for_current_device(float** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    g_last_cuda_error = static_cast<int>(e);
    return DLV_NOALLOC_CUDA_ERROR;
  }
  if (g_scratch_addr[dev] == nullptr) {
    float* p = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_scratch);
    if (e != cudaSuccess || p == nullptr) {
      g_last_cuda_error = static_cast<int>(e);
      return DLV_NOALLOC_CUDA_ERROR;
    }
    g_scratch_addr[dev] = p;
  }
  *out = g_scratch_addr[dev];
  return DLV_NOALLOC_OK;
}

}  // namespace

extern "C" unsigned long long dlv_decode_attention_noalloc_scratch_floats(int num_seqs, int num_heads, int head_dim, int splits) {
  if (splits <= 1 || num_seqs <= 0 || num_heads <= 0 || head_dim <= 0) return 0ull;
  return static_cast<unsigned long long>(num_seqs) * num_heads * splits * (static_cast<unsigned long long>(head_dim) + 2ull);
}

extern "C" int dlv_noalloc_last_cuda_error(void) { return g_last_cuda_error; }

extern "C" int dlv_decode_attention_noalloc(const void* q, long long q_stride, const void* k_cache, const void* v_cache,
                                            const int* block_tables, int bt_stride, const int* ctx_lens, void* out, int num_seqs,
                                            int num_heads, int kv_heads, int head_dim, int page_size, float scale, float softcap,
                                            int window, int splits, cudaStream_t stream) {
  if (q == nullptr || k_cache == nullptr || v_cache == nullptr || block_tables == nullptr || ctx_lens == nullptr || out == nullptr)
    return DLV_NOALLOC_BAD_ARGUMENT;
  if (num_seqs < 0 || num_heads <= 0 || kv_heads <= 0 || num_heads % kv_heads != 0 || num_heads / kv_heads > 8) return DLV_NOALLOC_BAD_ARGUMENT;
  if (head_dim != 64 && head_dim != 128 && head_dim != 256) return DLV_NOALLOC_BAD_ARGUMENT;
  if (page_size <= 0 || page_size % 32 != 0 || bt_stride <= 0 || q_stride < static_cast<long long>(num_heads) * head_dim) return DLV_NOALLOC_BAD_ARGUMENT;
  // the kernels read q and the caches with 16-byte vector loads (row t of q starts at q + t * q_stride elements) and write out
  // with 4-byte stores: anything less aligned would fault on the device instead of being refused here
  const unsigned long long align16 = reinterpret_cast<unsigned long long>(q) | reinterpret_cast<unsigned long long>(k_cache) |
                                     reinterpret_cast<unsigned long long>(v_cache);
  if ((align16 & 15ull) != 0 || q_stride % 8 != 0 || (reinterpret_cast<unsigned long long>(out) & 3ull) != 0) return DLV_NOALLOC_BAD_ARGUMENT;
  if (splits < 1 || splits > 64) return DLV_NOALLOC_BAD_ARGUMENT;
  if (num_seqs == 0) return DLV_NOALLOC_OK;
  float* part_o = nullptr;
  float* part_ml = nullptr;
  if (splits > 1) {
    const unsigned long long need = dlv_decode_attention_noalloc_scratch_floats(num_seqs, num_heads, head_dim, splits);
    if (need > DLV_NOALLOC_SCRATCH_FLOATS) return DLV_NOALLOC_TOO_LARGE;
    float* base = nullptr;
    const int rc = scratch_for_current_device(&base);
    if (rc != DLV_NOALLOC_OK) return rc;
    part_o = base;                                                                        // [seqs, heads, splits, head_dim]
    part_ml = base + static_cast<size_t>(num_seqs) * num_heads * splits * head_dim;       // [seqs, heads, splits, 2]
  }
  const int rc = dlv::launch_decode_attention(q, q_stride, k_cache, v_cache, block_tables, bt_stride, ctx_lens, out, part_o, part_ml, num_seqs,
                                              num_heads, kv_heads, head_dim, page_size, scale, softcap, window, splits, stream);
  if (rc != 0) return DLV_NOALLOC_BAD_ARGUMENT;
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    g_last_cuda_error = static_cast<int>(e);
    return DLV_NOALLOC_CUDA_ERROR;
  }
  return DLV_NOALLOC_OK;
}
