// Small device kernels off the generation hot path: run-time LoRA delta, sentence pooling (+ L2 normalisation), row softmax for the
// classifier head, and the MSE "TurboQuant" codec for KV snapshots.
// Reference math: core/.../generator/LoraDeltaApplier.java:43-63, core/.../embedding/SentenceTransformersPooling.java:4-150,
// core/.../model/AbstractModel.java:905-998, core/.../tensor/MseTurboQuantCodec.java:84-160.
#include "common.cuh"
#include "gemm_api.h"

namespace dlv {

// ------------------------------------------------------------------------------------------------ LoRA delta
// y[m, :] += (x[m, :] @ A^T) @ Bs^T with A [r, K] and Bs = scale * B [N, r], r <= 64 (bf16 in, fp32 math). One CTA per token row:
// the r inner products first (one warp per adapter row, strided over K), then every thread adds its columns of the delta.
__global__ void __launch_bounds__(256) lora_delta_kernel(const __nv_bfloat16* __restrict__ x, int ldx, const __nv_bfloat16* __restrict__ A,
                                                         const __nv_bfloat16* __restrict__ Bs, __nv_bfloat16* __restrict__ y, int ldy, int K,
                                                         int N, int r) {
  pdl_wait();
  pdl_trigger();
  __shared__ float t[64];
  const int m = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const __nv_bfloat16* xr = x + static_cast<size_t>(m) * ldx;
  for (int j = warp; j < r; j += 8) {
    const __nv_bfloat16* ar = A + static_cast<size_t>(j) * K;
    float acc = 0.f;
    for (int k = lane * 2; k + 1 < K; k += 64) {
      const float2 xv = unpack_bf162(*reinterpret_cast<const uint32_t*>(xr + k));
      const float2 av = unpack_bf162(*reinterpret_cast<const uint32_t*>(ar + k));
      acc += xv.x * av.x + xv.y * av.y;
    }
    if ((K & 1) && lane == 0) acc += bf2f(xr[K - 1]) * bf2f(ar[K - 1]);
    acc = warp_sum(acc);
    if (lane == 0) t[j] = acc;
  }
  __syncthreads();
  __nv_bfloat16* yr = y + static_cast<size_t>(m) * ldy;
  for (int n = threadIdx.x; n < N; n += blockDim.x) {
    const __nv_bfloat16* br = Bs + static_cast<size_t>(n) * r;
    float acc = 0.f;
    for (int j = 0; j < r; ++j) acc += t[j] * bf2f(br[j]);
    yr[n] = f2bf(bf2f(yr[n]) + acc);
  }
}

void launch_lora_delta(const void* x, int ldx, const void* A, const void* Bs, void* y, int ldy, int M, int K, int N, int r, cudaStream_t st) {
  if (M == 0) return;
  launch_pdl(lora_delta_kernel, dim3(M), dim3(256), 0, st, static_cast<const __nv_bfloat16*>(x), ldx, static_cast<const __nv_bfloat16*>(A),
             static_cast<const __nv_bfloat16*>(Bs), static_cast<__nv_bfloat16*>(y), ldy, K, N, r);
}

// ------------------------------------------------------------------------------------------------ pooling
// One CTA per sequence: rows [start, start + len) of the hidden states [T, H] (bf16) -> one fp32 vector [H].
// mode: 0 mean, 1 max, 2 sum, 3 first row (CLS), 4 last row, 5 mean * sqrt(len) (sum / sqrt(len)), 6 position-weighted mean
// (weights 1..len). normalize: divide by the L2 norm.
__global__ void __launch_bounds__(256) pool_kernel(const __nv_bfloat16* __restrict__ h, int H, const int* __restrict__ start, const int* __restrict__ len,
                                                   int mode, int normalize, float* __restrict__ out) {
  __shared__ float red[32];
  const int s = blockIdx.x;
  const int r0 = start[s], n = len[s];
  float ss = 0.f;
  for (int c = threadIdx.x; c < H; c += blockDim.x) {
    float acc = mode == 1 ? -INFINITY : 0.f;
    if (mode == 3) acc = n > 0 ? bf2f(h[static_cast<size_t>(r0) * H + c]) : 0.f;
    else if (mode == 4) acc = n > 0 ? bf2f(h[static_cast<size_t>(r0 + n - 1) * H + c]) : 0.f;
    else {
      for (int i = 0; i < n; ++i) {
        const float v = bf2f(h[static_cast<size_t>(r0 + i) * H + c]);
        if (mode == 1) acc = fmaxf(acc, v);
        else if (mode == 6) acc += v * static_cast<float>(i + 1);
        else acc += v;
      }
      if (mode == 0) acc /= static_cast<float>(n > 0 ? n : 1);
      else if (mode == 5) acc /= sqrtf(static_cast<float>(n > 0 ? n : 1));
      else if (mode == 6) acc /= 0.5f * static_cast<float>(n) * static_cast<float>(n + 1) + (n > 0 ? 0.f : 1.f);
      else if (mode == 1 && n == 0) acc = 0.f;
    }
    out[static_cast<size_t>(s) * H + c] = acc;
    ss += acc * acc;
  }
  if (normalize) {
    ss = block_sum(ss, red);
    const float inv = 1.f / fmaxf(sqrtf(ss), 1e-12f);
    for (int c = threadIdx.x; c < H; c += blockDim.x) out[static_cast<size_t>(s) * H + c] *= inv;
  }
}

void launch_pool(const void* h, int H, const int* start, const int* len, int S, int mode, int normalize, float* out, cudaStream_t st) {
  if (S == 0) return;
  pool_kernel<<<S, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(h), H, start, len, mode, normalize, out);
}

// ------------------------------------------------------------------------------------------------ row softmax (classifier head)
__global__ void __launch_bounds__(256) softmax_rows_kernel(const float* __restrict__ x, float* __restrict__ y, int C) {
  __shared__ float red[32];
  const float* xr = x + static_cast<size_t>(blockIdx.x) * C;
  float mx = -INFINITY;
  for (int c = threadIdx.x; c < C; c += blockDim.x) mx = fmaxf(mx, xr[c]);
  mx = block_max(mx, red);
  float sum = 0.f;
  for (int c = threadIdx.x; c < C; c += blockDim.x) sum += __expf(xr[c] - mx);
  sum = block_sum(sum, red);
  for (int c = threadIdx.x; c < C; c += blockDim.x) y[static_cast<size_t>(blockIdx.x) * C + c] = __expf(xr[c] - mx) / sum;
}

void launch_softmax_rows(const float* x, float* y, int rows, int C, cudaStream_t st) {
  if (rows == 0) return;
  softmax_rows_kernel<<<rows, 256, 0, st>>>(x, y, C);
}

// ------------------------------------------------------------------------------------------------ TurboQuant codec
__device__ __forceinline__ float tq_load(const float* p) { return *p; }
__device__ __forceinline__ float tq_load(const __nv_bfloat16* p) { return bf2f(*p); }
__device__ __forceinline__ void tq_store(float* p, float v) { *p = v; }
__device__ __forceinline__ void tq_store(__nv_bfloat16* p, float v) { *p = f2bf(v); }
// One CTA of pdim threads per row (pdim = dim rounded up to a power of two, <= 1024). Encode: row norm, normalise, random signs,
// Walsh-Hadamard transform in shared memory (result ~ N(0, 1) per coordinate after scaling), Lloyd-Max code per coordinate by binary
// search over the 2^bits - 1 edges, codes packed bit by bit (LSB first, pdim * bits / 8 bytes per row). Decode is the inverse.
__device__ __forceinline__ void fwht_smem(float* v, int pdim, int tid) {
  for (int hlen = 1; hlen < pdim; hlen <<= 1) {
    __syncthreads();
    const int i = tid;
    float a = 0.f, b = 0.f;
    const bool lo = (i & hlen) == 0;
    a = v[lo ? i : i - hlen];
    b = v[lo ? i + hlen : i];
    __syncthreads();
    v[i] = lo ? a + b : a - b;
  }
  __syncthreads();
}

template <typename T>
__global__ void __launch_bounds__(1024) tq_encode_kernel(const T* __restrict__ x, int dim, int pdim, int bits, const float* __restrict__ signs,
                                                         const float* __restrict__ edges, uint8_t* __restrict__ codes, float* __restrict__ norms) {
  extern __shared__ float tq_smem[];  // pdim floats, then pdim code bytes
  __shared__ float red[32];
  float* v = tq_smem;
  uint8_t* cd = reinterpret_cast<uint8_t*>(tq_smem + pdim);
  const int row = blockIdx.x, tid = threadIdx.x;
  const float xv = tid < dim ? tq_load(x + static_cast<size_t>(row) * dim + tid) : 0.f;
  const float ss = block_sum(xv * xv, red);
  const float nrm = sqrtf(ss);
  if (tid == 0) norms[row] = nrm;
  v[tid] = xv / fmaxf(nrm, 1e-20f) * signs[tid];
  fwht_smem(v, pdim, tid);
  const float z = v[tid];  // the unnormalised transform of a unit vector: variance 1 per coordinate
  int lo = 0, hi = (1 << bits) - 1;  // number of edges below z
  while (lo < hi) {
    const int mid = (lo + hi) >> 1;
    if (edges[mid] < z) lo = mid + 1; else hi = mid;
  }
  cd[tid] = static_cast<uint8_t>(lo);
  __syncthreads();
  const int row_bytes = pdim * bits / 8;
  for (int j = tid; j < row_bytes; j += blockDim.x) {
    unsigned int byte = 0;
    for (int tb = 0; tb < 8; ++tb) {
      const int pos = j * 8 + tb;
      const int ci = pos / bits, cb = pos - ci * bits;
      byte |= ((cd[ci] >> cb) & 1u) << tb;
    }
    codes[static_cast<size_t>(row) * row_bytes + j] = static_cast<uint8_t>(byte);
  }
}

template <typename T>
__global__ void __launch_bounds__(1024) tq_decode_kernel(const uint8_t* __restrict__ codes, const float* __restrict__ norms, int dim, int pdim, int bits,
                                                         const float* __restrict__ signs, const float* __restrict__ centroids, T* __restrict__ out) {
  extern __shared__ float tq_smem[];
  float* v = tq_smem;
  const int row = blockIdx.x, tid = threadIdx.x;
  const int row_bytes = pdim * bits / 8;
  const uint8_t* cr = codes + static_cast<size_t>(row) * row_bytes;
  unsigned int code = 0;
  for (int cb = 0; cb < bits; ++cb) {
    const int pos = tid * bits + cb;
    code |= ((cr[pos >> 3] >> (pos & 7)) & 1u) << cb;
  }
  v[tid] = centroids[code];
  fwht_smem(v, pdim, tid);
  if (tid < dim) tq_store(out + static_cast<size_t>(row) * dim + tid, v[tid] / static_cast<float>(pdim) * signs[tid] * norms[row]);
}

void launch_tq_encode(const void* x, int src_dtype, long long rows, int dim, int pdim, int bits, const float* signs, const float* edges, uint8_t* codes,
                      float* norms, cudaStream_t st) {
  if (rows == 0) return;
  const size_t smem = static_cast<size_t>(pdim) * 5;
  if (src_dtype == 0) tq_encode_kernel<float><<<static_cast<unsigned>(rows), pdim, smem, st>>>(static_cast<const float*>(x), dim, pdim, bits, signs, edges, codes, norms);
  else tq_encode_kernel<__nv_bfloat16><<<static_cast<unsigned>(rows), pdim, smem, st>>>(static_cast<const __nv_bfloat16*>(x), dim, pdim, bits, signs, edges, codes, norms);
}

void launch_tq_decode(const uint8_t* codes, const float* norms, long long rows, int dim, int pdim, int bits, const float* signs, const float* centroids,
                      void* out, int dst_dtype, cudaStream_t st) {
  if (rows == 0) return;
  const size_t smem = static_cast<size_t>(pdim) * 4;
  if (dst_dtype == 0) tq_decode_kernel<float><<<static_cast<unsigned>(rows), pdim, smem, st>>>(codes, norms, dim, pdim, bits, signs, centroids, static_cast<float*>(out));
  else tq_decode_kernel<__nv_bfloat16><<<static_cast<unsigned>(rows), pdim, smem, st>>>(codes, norms, dim, pdim, bits, signs, centroids, static_cast<__nv_bfloat16*>(out));
}

}  // namespace dlv
