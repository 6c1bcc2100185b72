// Memory-bound fused elementwise / normalisation kernels (bf16 activations, fp32 math).
//   rmsnorm, residual-add + rmsnorm (Gemma "1 + w" offset, Granite residual multiplier), LayerNorm,
//   act(gate) * up on a concatenated projection, embedding gather (+ scale, + positional / token-type tables),
//   per-head q/k RMSNorm + HF half-rotation RoPE + paged KV-cache write in one pass.
// Reference math: core/.../generator/RmsNorm.java:107-121, TransformerBlock.java:265-276, LayerNorm.java:20-151,
// CausalSelfAttention.java:315-372,429-446, Qwen3CausalSelfAttention.java:74-92, EmbedInput.java:26-44,
// native/src/main/c/simd/vector_simd.c:185-213 (the fused activation; here the product stays bf16, no int8 requant).
#include "common.cuh"

namespace dlv {

// ------------------------------------------------------------------------------------------------ RMSNorm
// One CTA per row. x, residual, y: bf16 [T, H]; H % 8 == 0. When residual != nullptr: residual += x * res_mult first
// (written back) and the norm runs on the updated residual.
__global__ void __launch_bounds__(256) rmsnorm_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* residual,
                                                      const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y,
                                                      int H, float eps, float offset, float res_mult) {
  pdl_wait();     // no-op unless launched with programmatic stream serialization: the kernel in front has completed
  pdl_trigger();  // the next kernel may start its prologue (and a GEMM its weight prefetch) under this kernel's tail
  extern __shared__ float row[];  // H floats
  __shared__ float red[32];
  const size_t base = static_cast<size_t>(blockIdx.x) * H;
  float ss = 0.f;
  for (int i = threadIdx.x * 8; i < H; i += blockDim.x * 8) {
    uint4 xv = *reinterpret_cast<const uint4*>(x + base + i);
    const uint32_t* xu = reinterpret_cast<const uint32_t*>(&xv);
    float v[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 f = unpack_bf162(xu[j]);
      v[2 * j] = f.x;
      v[2 * j + 1] = f.y;
    }
    if (residual != nullptr) {
      uint4 rv = *reinterpret_cast<const uint4*>(residual + base + i);
      const uint32_t* ru = reinterpret_cast<const uint32_t*>(&rv);
      uint4 ov;
      uint32_t* ou = reinterpret_cast<uint32_t*>(&ov);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 f = unpack_bf162(ru[j]);
        float a = f.x + v[2 * j] * res_mult, b = f.y + v[2 * j + 1] * res_mult;
        ou[j] = pack_bf162(a, b);
        float2 back = unpack_bf162(ou[j]);  // the norm sees the stored (rounded) residual
        v[2 * j] = back.x;
        v[2 * j + 1] = back.y;
      }
      *reinterpret_cast<uint4*>(residual + base + i) = ov;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      row[i + j] = v[j];
      ss += v[j] * v[j];
    }
  }
  ss = block_sum(ss, red);
  const float inv = rsqrtf(ss / H + eps);
  for (int i = threadIdx.x * 8; i < H; i += blockDim.x * 8) {
    uint4 wv = *reinterpret_cast<const uint4*>(w + i);
    const uint32_t* wu = reinterpret_cast<const uint32_t*>(&wv);
    uint4 ov;
    uint32_t* ou = reinterpret_cast<uint32_t*>(&ov);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 f = unpack_bf162(wu[j]);
      ou[j] = pack_bf162(row[i + 2 * j] * inv * (f.x + offset), row[i + 2 * j + 1] * inv * (f.y + offset));
    }
    *reinterpret_cast<uint4*>(y + base + i) = ov;
  }
}

// ------------------------------------------------------------------------------------------------ LayerNorm
__global__ void __launch_bounds__(256) layernorm_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                                                        const __nv_bfloat16* __restrict__ b, __nv_bfloat16* __restrict__ y, int H,
                                                        float eps) {
  pdl_wait();     // no-op unless launched with programmatic stream serialization: the kernel in front has completed
  pdl_trigger();  // the next kernel may start its prologue (and a GEMM its weight prefetch) under this kernel's tail
  extern __shared__ float row[];
  __shared__ float red[32];
  const size_t base = static_cast<size_t>(blockIdx.x) * H;
  float s = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float v = bf2f(x[base + i]);
    row[i] = v;
    s += v;
  }
  const float mean = block_sum(s, red) / H;
  float ss = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float d = row[i] - mean;
    ss += d * d;
  }
  const float inv = rsqrtf(block_sum(ss, red) / H + eps);
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float v = (row[i] - mean) * inv * bf2f(w[i]) + (b ? bf2f(b[i]) : 0.f);
    y[base + i] = f2bf(v);
  }
}

// ------------------------------------------------------------------------------------------------ act(gate) * up
__device__ __forceinline__ float act_apply(float g, int act) {
  switch (act) {
    case 0: return g / (1.f + __expf(-g));                                                     // silu
    case 1: return 0.5f * g * (1.f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g)));  // gelu tanh
    case 2: return 0.5f * g * (1.f + erff(g * 0.7071067811865475f));                            // gelu erf
    case 3: return fmaxf(g, 0.f);
    default: return tanhf(g);
  }
}

// in: [T, 2*I] (gate | up), out: [T, I]; I % 8 == 0
__global__ void __launch_bounds__(256) act_mul_kernel(const __nv_bfloat16* __restrict__ in, __nv_bfloat16* __restrict__ out, int I,
                                                      int act, long long total_vec) {
  pdl_wait();     // no-op unless launched with programmatic stream serialization: the kernel in front has completed
  pdl_trigger();  // the next kernel may start its prologue (and a GEMM its weight prefetch) under this kernel's tail
  const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= total_vec) return;
  const int per_row = I / 8;
  const long long t = idx / per_row;
  const int c = static_cast<int>(idx % per_row) * 8;
  const __nv_bfloat16* g = in + t * 2 * I + c;
  uint4 gv = *reinterpret_cast<const uint4*>(g);
  uint4 uv = *reinterpret_cast<const uint4*>(g + I);
  const uint32_t* gu = reinterpret_cast<const uint32_t*>(&gv);
  const uint32_t* uu = reinterpret_cast<const uint32_t*>(&uv);
  uint4 ov;
  uint32_t* ou = reinterpret_cast<uint32_t*>(&ov);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    float2 a = unpack_bf162(gu[j]), b = unpack_bf162(uu[j]);
    ou[j] = pack_bf162(act_apply(a.x, act) * b.x, act_apply(a.y, act) * b.y);
  }
  *reinterpret_cast<uint4*>(out + t * I + c) = ov;
}

// unary activation in place-capable form (gpt2 / bert MLP without an up projection)
__global__ void __launch_bounds__(256) act_kernel(const __nv_bfloat16* __restrict__ in, __nv_bfloat16* __restrict__ out, int act,
                                                  long long n) {
  pdl_wait();     // no-op unless launched with programmatic stream serialization: the kernel in front has completed
  pdl_trigger();  // the next kernel may start its prologue (and a GEMM its weight prefetch) under this kernel's tail
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < n) out[i] = f2bf(act_apply(bf2f(in[i]), act));
}

// ------------------------------------------------------------------------------------------------ embedding
// out[t] = table[ids[t]] * scale (+ pos_table[pos[t]]) (+ type_table[types[t]]); H % 8 == 0
__global__ void __launch_bounds__(128) embedding_kernel(const __nv_bfloat16* __restrict__ table, const int* __restrict__ ids,
                                                        const __nv_bfloat16* __restrict__ pos_table, const int* __restrict__ pos,
                                                        const __nv_bfloat16* __restrict__ type_table, const int* __restrict__ types,
                                                        __nv_bfloat16* __restrict__ out, int H, int vocab, float scale) {
  pdl_wait();     // no-op unless launched with programmatic stream serialization: the kernel in front has completed
  pdl_trigger();  // the next kernel may start its prologue (and a GEMM its weight prefetch) under this kernel's tail
  const int t = blockIdx.x;
  int id = ids[t];
  if (id < 0 || id >= vocab) id = 0;  // host validates ids; never read out of the table
  const __nv_bfloat16* src = table + static_cast<size_t>(id) * H;
  const __nv_bfloat16* ps = pos_table ? pos_table + static_cast<size_t>(pos[t]) * H : nullptr;
  const __nv_bfloat16* ts = type_table ? type_table + static_cast<size_t>(types ? types[t] : 0) * H : nullptr;
  for (int i = threadIdx.x * 8; i < H; i += blockDim.x * 8) {
    uint4 v = *reinterpret_cast<const uint4*>(src + i);
    const uint32_t* vu = reinterpret_cast<const uint32_t*>(&v);
    float f[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 a = unpack_bf162(vu[j]);
      f[2 * j] = a.x * scale;
      f[2 * j + 1] = a.y * scale;
    }
    if (ps) {
      uint4 pv = *reinterpret_cast<const uint4*>(ps + i);
      const uint32_t* pu = reinterpret_cast<const uint32_t*>(&pv);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 a = unpack_bf162(pu[j]);
        f[2 * j] += a.x;
        f[2 * j + 1] += a.y;
      }
    }
    if (ts) {
      uint4 pv = *reinterpret_cast<const uint4*>(ts + i);
      const uint32_t* pu = reinterpret_cast<const uint32_t*>(&pv);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 a = unpack_bf162(pu[j]);
        f[2 * j] += a.x;
        f[2 * j + 1] += a.y;
      }
    }
    uint4 o;
    uint32_t* ou = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
    for (int j = 0; j < 4; ++j) ou[j] = pack_bf162(f[2 * j], f[2 * j + 1]);
    *reinterpret_cast<uint4*>(out + static_cast<size_t>(t) * H + i) = o;
  }
}

// ------------------------------------------------------------------------------------------------ q/k norm + RoPE + KV write
// qkv: [T, (H + 2 KV) * D] bf16. One warp per (token, head). q heads are normalised/rotated in place; k heads are
// normalised/rotated and written to the paged cache; v heads are copied to the cache.
// cache layout: [num_blocks, KV, block_size, D]; slot = block * block_size + offset; slot < 0 skips the cache write.
template <int D>
__global__ void __launch_bounds__(256) rope_kv_kernel(__nv_bfloat16* __restrict__ qkv, const int* __restrict__ positions,
                                                      const long long* __restrict__ slots, const __nv_bfloat16* __restrict__ q_norm_w,
                                                      const __nv_bfloat16* __restrict__ k_norm_w, const float* __restrict__ cos_t,
                                                      const float* __restrict__ sin_t, __nv_bfloat16* __restrict__ k_cache,
                                                      __nv_bfloat16* __restrict__ v_cache, int T, int H, int KV, int block_size,
                                                      int rot_half, float eps, float norm_offset, int max_pos) {
  pdl_wait();     // no-op unless launched with programmatic stream serialization: the kernel in front has completed
  pdl_trigger();  // the next kernel may start its prologue (and a GEMM its weight prefetch) under this kernel's tail
  const int warp_global = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  const int heads = H + 2 * KV;
  if (warp_global >= T * heads) return;
  const int t = warp_global / heads, h = warp_global % heads;
  __nv_bfloat16* src = qkv + static_cast<size_t>(t) * heads * D + static_cast<size_t>(h) * D;
  constexpr int HALF = D / 2;
  constexpr int PER = HALF / 32 > 0 ? HALF / 32 : 1;  // pairs per lane (D >= 64)
  const bool is_q = h < H, is_k = !is_q && h < H + KV;
  const long long slot = slots ? slots[t] : -1;
  const int kvh = is_q ? 0 : (is_k ? h - H : h - H - KV);
  __nv_bfloat16* dst = nullptr;
  if (!is_q && slot >= 0) {
    const long long blk = slot / block_size, off = slot % block_size;
    __nv_bfloat16* cache = is_k ? k_cache : v_cache;
    dst = cache + ((blk * KV + kvh) * block_size + off) * D;
  }
  float a[PER], b[PER];
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int d = lane + 32 * i;
    a[i] = d < HALF ? bf2f(src[d]) : 0.f;
    b[i] = d < HALF ? bf2f(src[d + HALF]) : 0.f;
  }
  if (!is_q && !is_k) {  // v: plain copy
    if (dst) {
#pragma unroll
      for (int i = 0; i < PER; ++i) {
        const int d = lane + 32 * i;
        if (d < HALF) {
          dst[d] = f2bf(a[i]);
          dst[d + HALF] = f2bf(b[i]);
        }
      }
    }
    return;
  }
  const __nv_bfloat16* nw = is_q ? q_norm_w : k_norm_w;
  if (nw != nullptr) {
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < PER; ++i) ss += a[i] * a[i] + b[i] * b[i];
    ss = warp_sum(ss);
    const float inv = rsqrtf(ss / D + eps);
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const int d = lane + 32 * i;
      if (d < HALF) {
        // round through bf16 like a separate norm kernel would
        a[i] = bf2f(f2bf(a[i] * inv * (bf2f(nw[d]) + norm_offset)));
        b[i] = bf2f(f2bf(b[i] * inv * (bf2f(nw[d + HALF]) + norm_offset)));
      }
    }
  }
  if (cos_t != nullptr) {
    int pos = positions[t];
    pos = pos < 0 ? 0 : (pos >= max_pos ? max_pos - 1 : pos);
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const int d = lane + 32 * i;
      if (d < rot_half) {
        const float c = cos_t[static_cast<size_t>(pos) * rot_half + d], s = sin_t[static_cast<size_t>(pos) * rot_half + d];
        const float x0 = a[i], x1 = b[i];
        a[i] = x0 * c - x1 * s;
        b[i] = x1 * c + x0 * s;
      }
    }
  }
  __nv_bfloat16* out = is_q ? src : dst;
  if (out) {
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const int d = lane + 32 * i;
      if (d < HALF) {
        out[d] = f2bf(a[i]);
        out[d + HALF] = f2bf(b[i]);
      }
    }
  }
}

// ------------------------------------------------------------------------------------------------ launchers
void launch_rmsnorm(const void* x, void* residual, const void* w, void* y, int T, int H, float eps, float offset,
                    float res_mult, cudaStream_t st) {
  if (T == 0) return;
  launch_pdl(rmsnorm_kernel, dim3(T), dim3(256), H * sizeof(float), st, static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(residual),
                                                    static_cast<const __nv_bfloat16*>(w), static_cast<__nv_bfloat16*>(y), H, eps,
                                                    offset, res_mult);
}
void launch_layernorm(const void* x, const void* w, const void* b, void* y, int T, int H, float eps, cudaStream_t st) {
  if (T == 0) return;
  layernorm_kernel<<<T, 256, H * sizeof(float), st>>>(static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(w),
                                                      static_cast<const __nv_bfloat16*>(b), static_cast<__nv_bfloat16*>(y), H, eps);
}
void launch_act_mul(const void* in, void* out, long long T, int I, int act, cudaStream_t st) {
  const long long total = T * (I / 8);
  if (total == 0) return;
  launch_pdl(act_mul_kernel, dim3(static_cast<unsigned>((total + 255) / 256)), dim3(256), 0, st, static_cast<const __nv_bfloat16*>(in),
                                                                             static_cast<__nv_bfloat16*>(out), I, act, total);
}
void launch_act(const void* in, void* out, long long n, int act, cudaStream_t st) {
  if (n == 0) return;
  act_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, st>>>(static_cast<const __nv_bfloat16*>(in),
                                                                     static_cast<__nv_bfloat16*>(out), act, n);
}
void launch_embedding(const void* table, const int* ids, const void* pos_table, const int* pos, const void* type_table,
                      const int* types, void* out, int T, int H, int vocab, float scale, cudaStream_t st) {
  if (T == 0) return;
  launch_pdl(embedding_kernel, dim3(T), dim3(128), 0, st, static_cast<const __nv_bfloat16*>(table), ids, static_cast<const __nv_bfloat16*>(pos_table), pos,
                                      static_cast<const __nv_bfloat16*>(type_table), types, static_cast<__nv_bfloat16*>(out), H, vocab,
                                      scale);
}
int launch_rope_kv(void* qkv, const int* positions, const long long* slots, const void* qn, const void* kn, const float* cos_t,
                   const float* sin_t, void* k_cache, void* v_cache, int T, int H, int KV, int D, int block_size, int rot_half,
                   float eps, float norm_offset, int max_pos, cudaStream_t st) {
  if (T == 0) return 0;
  const long long warps = static_cast<long long>(T) * (H + 2 * KV);
  const unsigned grid = static_cast<unsigned>((warps + 7) / 8);
#define DLV_ROPE(DD)                                                                                                         \
  launch_pdl(rope_kv_kernel<DD>, dim3(grid), dim3(256), 0, st, static_cast<__nv_bfloat16*>(qkv), positions, slots,                                \
                                           static_cast<const __nv_bfloat16*>(qn), static_cast<const __nv_bfloat16*>(kn), cos_t, \
                                           sin_t, static_cast<__nv_bfloat16*>(k_cache), static_cast<__nv_bfloat16*>(v_cache), T, \
                                           H, KV, block_size, rot_half, eps, norm_offset, max_pos)
  switch (D) {
    case 64: DLV_ROPE(64); break;
    case 128: DLV_ROPE(128); break;
    case 256: DLV_ROPE(256); break;
    default: return 1;
  }
#undef DLV_ROPE
  return 0;
}

}  // namespace dlv
