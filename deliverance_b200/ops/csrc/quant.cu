// JQ4 quantise / dequantise on the device, bit-exact with the host definition: block of 32, scale = v_max / -8 where
// v_max is the signed value of the first element of largest magnitude, q = min(15, trunc(v * inv + 8.5)), byte j of a
// block = q[j] | q[j + 16] << 4 (reference: safetensors/.../ModelQuantizer.java:491-531,
// tensor/.../impl/Q4ByteBufferTensor.java:55-109). Multiplication and addition are kept as two rounded operations.
#include "common.cuh"

namespace dlv {

template <typename T>
__device__ __forceinline__ float load_as_float(const T* p, long long i);
template <>
__device__ __forceinline__ float load_as_float<float>(const float* p, long long i) { return p[i]; }
template <>
__device__ __forceinline__ float load_as_float<__nv_bfloat16>(const __nv_bfloat16* p, long long i) { return bf2f(p[i]); }
template <>
__device__ __forceinline__ float load_as_float<__half>(const __half* p, long long i) { return __half2float(p[i]); }

template <typename T>
__global__ void __launch_bounds__(256) q4_quantize_kernel(const T* __restrict__ w, long long n_blocks, uint8_t* __restrict__ packed,
                                                          float* __restrict__ scales) {
  pdl_wait();     // no-op unless launched with programmatic stream serialization: the kernel in front has completed
  pdl_trigger();  // the next kernel may start its prologue (and a GEMM its weight prefetch) under this kernel's tail
  const long long blk = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (blk >= n_blocks) return;
  float v[32];
  float vmax = 0.f, amax = 0.f;
  bool any = false;
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    v[i] = load_as_float<T>(w, blk * 32 + i);
    const float a = v[i] < 0.f ? -v[i] : v[i];
    if (a > amax) {
      amax = a;
      vmax = v[i];
      any = true;
    }
  }
  const float scale = any ? __fdiv_rn(vmax, -8.0f) : -0.0f;
  const float inv = scale != 0.0f ? __fdiv_rn(1.0f, scale) : 0.0f;
  uint4 out;
  uint32_t* ow = reinterpret_cast<uint32_t*>(&out);
#pragma unroll
  for (int wd = 0; wd < 4; ++wd) {
    uint32_t word = 0;
#pragma unroll
    for (int b = 0; b < 4; ++b) {
      const int j = wd * 4 + b;
      const float f0 = __fadd_rn(__fmul_rn(v[j], inv), 8.5f);
      const float f1 = __fadd_rn(__fmul_rn(v[j + 16], inv), 8.5f);
      int q0 = (f0 != f0) ? 0 : static_cast<int>(f0);
      int q1 = (f1 != f1) ? 0 : static_cast<int>(f1);
      q0 = q0 > 15 ? 15 : (q0 < 0 ? 0 : q0);
      q1 = q1 > 15 ? 15 : (q1 < 0 ? 0 : q1);
      word |= static_cast<uint32_t>(q0 | (q1 << 4)) << (8 * b);
    }
    ow[wd] = word;
  }
  reinterpret_cast<uint4*>(packed)[blk] = out;
  scales[blk] = scale;
}

template <typename T>
__device__ __forceinline__ T from_float(float v);
template <>
__device__ __forceinline__ float from_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return f2bf(v); }

template <typename T>
__global__ void __launch_bounds__(256) q4_dequantize_kernel(const uint8_t* __restrict__ packed, const float* __restrict__ scales,
                                                            long long n_blocks, T* __restrict__ out) {
  pdl_wait();     // no-op unless launched with programmatic stream serialization: the kernel in front has completed
  pdl_trigger();  // the next kernel may start its prologue (and a GEMM its weight prefetch) under this kernel's tail
  const long long blk = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (blk >= n_blocks) return;
  const uint4 w = reinterpret_cast<const uint4*>(packed)[blk];
  const uint32_t words[4] = {w.x, w.y, w.z, w.w};
  const float s = scales[blk];
#pragma unroll
  for (int wd = 0; wd < 4; ++wd) {
#pragma unroll
    for (int b = 0; b < 4; ++b) {
      const uint32_t byte = (words[wd] >> (8 * b)) & 0xFFu;
      const int j = wd * 4 + b;
      out[blk * 32 + j] = from_float<T>(static_cast<float>(static_cast<int>(byte & 0xFu) - 8) * s);
      out[blk * 32 + j + 16] = from_float<T>(static_cast<float>(static_cast<int>(byte >> 4) - 8) * s);
    }
  }
}

void launch_q4_quantize(const void* w, int src_dtype, long long n_blocks, uint8_t* packed, float* scales, cudaStream_t st) {
  if (n_blocks == 0) return;
  const unsigned grid = static_cast<unsigned>((n_blocks + 255) / 256);
  if (src_dtype == 0) q4_quantize_kernel<float><<<grid, 256, 0, st>>>(static_cast<const float*>(w), n_blocks, packed, scales);
  else if (src_dtype == 1) q4_quantize_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(w), n_blocks, packed, scales);
  else q4_quantize_kernel<__half><<<grid, 256, 0, st>>>(static_cast<const __half*>(w), n_blocks, packed, scales);
}
void launch_q4_dequantize(const uint8_t* packed, const float* scales, long long n_blocks, void* out, int dst_dtype, cudaStream_t st) {
  if (n_blocks == 0) return;
  const unsigned grid = static_cast<unsigned>((n_blocks + 255) / 256);
  if (dst_dtype == 0) q4_dequantize_kernel<float><<<grid, 256, 0, st>>>(packed, scales, n_blocks, static_cast<float*>(out));
  else q4_dequantize_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(packed, scales, n_blocks, static_cast<__nv_bfloat16*>(out));
}

}  // namespace dlv
