// Sampler-side kernels over fp32 logits [B, V] (V up to 256k): greedy argmax with "first maximum wins", logit
// post-processing (Granite logits scaling, final-logit softcap cap*tanh(v/cap), guided-decoding allow-bitmask -> -inf).
// Reference order of operations: core/.../model/AbstractGeneratorSampler.java:117-155, GuideLogitsProcessor.java:23-41.
#include "common.cuh"

namespace dlv {

__device__ __forceinline__ float post_logit(float v, float softcap, float inv_scale) {
  v *= inv_scale;
  if (softcap > 0.f) v = softcap * tanhf(v / softcap);
  return v;
}
__device__ __forceinline__ bool mask_allows(const uint32_t* mask_row, int i) {
  return mask_row == nullptr || ((mask_row[i >> 5] >> (i & 31)) & 1u);
}

// one CTA per row
__global__ void __launch_bounds__(1024) argmax_kernel(const float* __restrict__ logits, int ld, int V,
                                                      const uint32_t* __restrict__ mask, int mask_ld, float softcap,
                                                      float inv_scale, long long* __restrict__ out_idx, float* __restrict__ out_val) {
  pdl_wait();     // no-op unless launched with programmatic stream serialization: the kernel in front has completed
  pdl_trigger();  // the next kernel may start its prologue (and a GEMM its weight prefetch) under this kernel's tail
  __shared__ float sv[32];
  __shared__ int si[32];
  const int b = blockIdx.x;
  const float* row = logits + static_cast<size_t>(b) * ld;
  const uint32_t* mrow = mask ? mask + static_cast<size_t>(b) * mask_ld : nullptr;
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    if (!mask_allows(mrow, i)) continue;
    const float v = row[i];
    if (v > best || (v == best && i < bi)) {
      best = v;
      bi = i;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) {
      best = ov;
      bi = oi;
    }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) {
    sv[warp] = best;
    si[warp] = bi;
  }
  __syncthreads();
  if (warp == 0) {
    const int nw = blockDim.x >> 5;
    best = lane < nw ? sv[lane] : -INFINITY;
    bi = lane < nw ? si[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) {
        best = ov;
        bi = oi;
      }
    }
    if (lane == 0) {
      if (bi == 0x7fffffff) bi = 0;  // every token masked or all logits -inf / NaN
      out_idx[b] = bi;
      if (out_val) out_val[b] = post_logit(row[bi], softcap, inv_scale);
    }
  }
}

__global__ void __launch_bounds__(256) logits_post_kernel(float* __restrict__ logits, int ld, int V, const uint32_t* __restrict__ mask,
                                                          int mask_ld, float softcap, float inv_scale) {
  pdl_wait();     // no-op unless launched with programmatic stream serialization: the kernel in front has completed
  pdl_trigger();  // the next kernel may start its prologue (and a GEMM its weight prefetch) under this kernel's tail
  const int b = blockIdx.y;
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= V) return;
  float* row = logits + static_cast<size_t>(b) * ld;
  const uint32_t* mrow = mask ? mask + static_cast<size_t>(b) * mask_ld : nullptr;
  row[i] = mask_allows(mrow, i) ? post_logit(row[i], softcap, inv_scale) : -INFINITY;
}

void launch_argmax(const float* logits, int ld, int B, int V, const uint32_t* mask, int mask_ld, float softcap, float inv_scale,
                   long long* out_idx, float* out_val, cudaStream_t st) {
  if (B == 0) return;
  launch_pdl(argmax_kernel, dim3(B), dim3(1024), 0, st, logits, ld, V, mask, mask_ld, softcap, inv_scale, out_idx, out_val);
}
void launch_logits_post(float* logits, int ld, int B, int V, const uint32_t* mask, int mask_ld, float softcap, float inv_scale,
                        cudaStream_t st) {
  if (B == 0) return;
  dim3 grid((V + 255) / 256, B);
  logits_post_kernel<<<grid, 256, 0, st>>>(logits, ld, V, mask, mask_ld, softcap, inv_scale);
}

}  // namespace dlv
