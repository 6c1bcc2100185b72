// Paged-KV attention.
//   * decode: one query token per sequence, split-KV, all query heads of a GQA group share one pass over K/V
//     (the kernel is KV-bandwidth bound; CUDA-core math keeps up with HBM for group sizes <= 8), merge kernel.
//   * prefill: flash-style tiles of 64 query rows x 64 keys, online softmax in registers, causal + sliding window +
//     logit softcap, K/V fetched from the paged cache with cp.async into swizzled shared memory.
// KV cache layout: [num_pages, KV, page_size, D] bf16, page_size % 32 == 0. Queries are read in place from the fused
// qkv activation (row stride given). Scores: softmax(softcap(scale * q.k)), key j visible to position p iff j <= p
// and (window == 0 or j > p - window)  (reference: core/.../generator/CausalSelfAttention.java:458-532,
// tensor/.../operations/TensorOperations.java:225-271, tensor/.../VectorTensorMathUtils.java:34-78).
#include "common.cuh"

namespace dlv {

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
  const int sz = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(sz) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ float softcap_apply(float s, float cap) { return cap > 0.f ? cap * tanhf(s / cap) : s; }

// =====================================================================================================================
// Decode
// =====================================================================================================================
// grid (num_seqs, KV, splits), 128 threads. GP = padded group size (power of two >= H / KV).
// Shared-memory traffic is the limiter of this kernel, so the queries live in registers for the whole CTA (thread
// (key slot, part) keeps the D / PARTS query elements of all GP heads that it multiplies), K rows are read once per key with
// 16-byte loads, and the P.V pass reads V with 8-byte loads and the probabilities four keys at a time.
template <int D, int GP>
__global__ void __launch_bounds__(128) decode_attn_kernel(
    const __nv_bfloat16* __restrict__ q, long long q_stride,  // q row t at q + t * q_stride, heads contiguous [H, D]
    const __nv_bfloat16* __restrict__ k_cache, const __nv_bfloat16* __restrict__ v_cache,
    const int* __restrict__ block_tables, int bt_stride, const int* __restrict__ ctx_lens,
    __nv_bfloat16* __restrict__ out,          // [num_seqs, H, D] (used when splits == 1)
    float* __restrict__ part_o,               // [num_seqs, H, splits, D]
    float* __restrict__ part_ml,              // [num_seqs, H, splits, 2]
    int H, int KV, int page_size, float scale, float softcap, int window, int splits) {
  pdl_wait();     // no-op unless launched with programmatic stream serialization: the kernel in front has completed
  pdl_trigger();  // the next kernel may start its prologue (and a GEMM its weight prefetch) under this kernel's tail
  constexpr int PARTS0 = D * GP / 64;
  constexpr int PARTS = PARTS0 < 8 ? 8 : (PARTS0 > 32 ? 32 : PARTS0);  // threads that share one key
  constexpr int EPT = D / PARTS;                                       // query elements per thread and head
  constexpr int CPT = EPT / 8;                                         // 16-byte K chunks per thread and key
  constexpr int KPP = 128 / PARTS;                                     // keys per pass
  constexpr int DQ = D / 4;                                            // threads that cover D in the P.V pass (4 columns each)
  constexpr int KG = 128 / DQ;                                         // key groups in the P.V pass
  static_assert(EPT % 8 == 0 && CPT >= 1 && 32 % KPP == 0 && 32 % KG == 0, "decode attention tiling");
  extern __shared__ __align__(16) uint8_t dsm[];
  __nv_bfloat16* sK = reinterpret_cast<__nv_bfloat16*>(dsm);        // [2][32][D]
  __nv_bfloat16* sV = sK + 2 * 32 * D;                               // [2][32][D]
  float* sS = reinterpret_cast<float*>(sV + 2 * 32 * D);             // [GP][32] scores, then probabilities
  float* sM = sS + GP * 32;                                          // [GP] running max
  float* sL = sM + GP;                                               // [GP] running sum
  float* sA = sL + GP;                                               // [GP] rescale factor of this tile
  constexpr int HDR = (GP * 32 + 3 * GP + 3) & ~3;                   // keep the float4 stores below 16-byte aligned
  float* sRed = sS + HDR;                                            // [KG][GP][D] cross-group reduction

  const int b = blockIdx.x, kvh = blockIdx.y, sp = blockIdx.z;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int G = H / KV;
  const int ctx = ctx_lens[b];
  const int first_key = (window > 0 && ctx > window) ? ctx - window : 0;
  const int tile_lo = first_key / 32, tile_hi = (ctx + 31) / 32;
  const int ntiles = tile_hi - tile_lo;
  const int per = (ntiles + splits - 1) / splits;
  const int t0 = tile_lo + sp * per, t1 = min(tile_hi, t0 + per);

  // queries -> registers (pre-scaled); thread (slot = tid / PARTS, part = tid % PARTS) owns elements chunk c * PARTS + part
  const int part = tid % PARTS, slot = tid / PARTS;
  float qreg[GP][EPT];
#pragma unroll
  for (int g = 0; g < GP; ++g) {
#pragma unroll
    for (int c = 0; c < CPT; ++c) {
      const int d0 = (c * PARTS + part) * 8;
      if (g < G) {
        const uint4 qv = *reinterpret_cast<const uint4*>(q + b * q_stride + static_cast<long long>(kvh * G + g) * D + d0);
        const uint32_t* qu = reinterpret_cast<const uint32_t*>(&qv);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = unpack_bf162(qu[e]);
          qreg[g][c * 8 + 2 * e] = f.x * scale;
          qreg[g][c * 8 + 2 * e + 1] = f.y * scale;
        }
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) qreg[g][c * 8 + e] = 0.f;
      }
    }
  }
  if (tid < GP) {
    sM[tid] = -INFINITY;
    sL[tid] = 0.f;
  }
  float acc[GP][4];
#pragma unroll
  for (int g = 0; g < GP; ++g) acc[g][0] = acc[g][1] = acc[g][2] = acc[g][3] = 0.f;

  auto load_tile = [&](int tile, int buf) {
    const int key0 = tile * 32;
    const int page = block_tables[static_cast<long long>(b) * bt_stride + key0 / page_size];
    const long long base = ((static_cast<long long>(page) * KV + kvh) * page_size + key0 % page_size) * D;
    constexpr int CPR = D / 8;  // 16 B chunks per row
    for (int c = tid; c < 32 * CPR; c += 128) {
      const int r = c / CPR, cc = c % CPR;
      const bool valid = key0 + r < ctx;
      cp_async16(smem_u32(sK + (buf * 32 + r) * D + cc * 8), k_cache + base + r * D + cc * 8, valid);
      cp_async16(smem_u32(sV + (buf * 32 + r) * D + cc * 8), v_cache + base + r * D + cc * 8, valid);
    }
    cp_async_commit();
  };

  if (t0 < t1) load_tile(t0, 0);
  for (int tile = t0; tile < t1; ++tile) {
    const int buf = (tile - t0) & 1;
    if (tile + 1 < t1) {
      load_tile(tile + 1, buf ^ 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    // ---- scores: KPP keys per pass, PARTS threads per key (a key's threads read 16-byte chunks that are contiguous)
#pragma unroll
    for (int pass = 0; pass < 32 / KPP; ++pass) {
      const int j = pass * KPP + slot;
      const __nv_bfloat16* krow = sK + (buf * 32 + j) * D;
      float s[GP];
#pragma unroll
      for (int g = 0; g < GP; ++g) s[g] = 0.f;
#pragma unroll
      for (int c = 0; c < CPT; ++c) {
        const uint4 kv = *reinterpret_cast<const uint4*>(krow + (c * PARTS + part) * 8);
        const uint32_t* ku = reinterpret_cast<const uint32_t*>(&kv);
        float kf[8];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = unpack_bf162(ku[e]);
          kf[2 * e] = f.x;
          kf[2 * e + 1] = f.y;
        }
#pragma unroll
        for (int g = 0; g < GP; ++g) {
#pragma unroll
          for (int e = 0; e < 8; ++e) s[g] += qreg[g][c * 8 + e] * kf[e];
        }
      }
#pragma unroll
      for (int g = 0; g < GP; ++g) {
#pragma unroll
        for (int o = 1; o < PARTS; o <<= 1) s[g] += __shfl_xor_sync(0xffffffffu, s[g], o);
      }
      if (part == 0) {
        const int key = tile * 32 + j;
        const bool vis = key < ctx && key >= first_key;
#pragma unroll
        for (int g = 0; g < GP; ++g) sS[g * 32 + j] = vis ? softcap_apply(s[g], softcap) : -INFINITY;
      }
    }
    __syncthreads();
    // ---- online softmax: warp w owns heads w, w + 4, ...
    for (int g = warp; g < GP; g += 4) {
      const float sv = sS[g * 32 + lane];
      const float m_old = sM[g];
      const float m_new = fmaxf(m_old, warp_max(sv));
      const float pexp = (sv == -INFINITY) ? 0.f : __expf(sv - m_new);
      const float psum = warp_sum(pexp);
      sS[g * 32 + lane] = pexp;
      if (lane == 0) {
        const float alpha = (m_old == -INFINITY) ? 0.f : __expf(m_old - m_new);
        sA[g] = alpha;
        sM[g] = m_new;
        sL[g] = sL[g] * alpha + psum;
      }
    }
    __syncthreads();
    // ---- P.V: thread (4 columns dq, key group kg) walks the keys kg * (32 / KG) .. in blocks of four
    {
      const int dq = tid % DQ, kg = tid / DQ;
      constexpr int KPG = 32 / KG;  // keys per group (multiple of 4 for every supported D)
#pragma unroll
      for (int g = 0; g < GP; ++g) {
        const float a = sA[g];
        acc[g][0] *= a; acc[g][1] *= a; acc[g][2] *= a; acc[g][3] *= a;
      }
#pragma unroll
      for (int jb = 0; jb < KPG; jb += 4) {
        const int j0 = kg * KPG + jb;
        float vf[4][4];
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) {
          const uint2 v = *reinterpret_cast<const uint2*>(sV + (buf * 32 + j0 + jj) * D + 4 * dq);
          const float2 lo = unpack_bf162(v.x), hi = unpack_bf162(v.y);
          vf[jj][0] = lo.x; vf[jj][1] = lo.y; vf[jj][2] = hi.x; vf[jj][3] = hi.y;
        }
#pragma unroll
        for (int g = 0; g < GP; ++g) {
          const float4 p4 = *reinterpret_cast<const float4*>(sS + g * 32 + j0);
          const float pj[4] = {p4.x, p4.y, p4.z, p4.w};
#pragma unroll
          for (int jj = 0; jj < 4; ++jj) {
            acc[g][0] += pj[jj] * vf[jj][0];
            acc[g][1] += pj[jj] * vf[jj][1];
            acc[g][2] += pj[jj] * vf[jj][2];
            acc[g][3] += pj[jj] * vf[jj][3];
          }
        }
      }
    }
    __syncthreads();
  }
  // ---- reduce key groups, write (partial) output
  {
    const int dq = tid % DQ, kg = tid / DQ;
#pragma unroll
    for (int g = 0; g < GP; ++g)
      *reinterpret_cast<float4*>(sRed + (kg * GP + g) * D + 4 * dq) = make_float4(acc[g][0], acc[g][1], acc[g][2], acc[g][3]);
  }
  __syncthreads();
  for (int i = tid; i < G * D; i += 128) {
    const int g = i / D, d = i % D;
    float o = 0.f;
#pragma unroll
    for (int kg = 0; kg < KG; ++kg) o += sRed[(kg * GP + g) * D + d];
    const int h = kvh * G + g;
    if (splits == 1) {
      const float l = sL[g];
      out[(static_cast<long long>(b) * H + h) * D + d] = f2bf(l > 0.f ? o / l : 0.f);
    } else {
      part_o[((static_cast<long long>(b) * H + h) * splits + sp) * D + d] = o;
    }
  }
  if (splits > 1 && tid < G) {
    const int h = kvh * G + tid;
    float* ml = part_ml + ((static_cast<long long>(b) * H + h) * splits + sp) * 2;
    ml[0] = sM[tid];
    ml[1] = sL[tid];
  }
}

// grid (num_seqs, H), D threads (D = 64 / 128 / 256). The split weights are computed once per CTA (thread s takes split s) and kept
// in shared memory; the weighted sum over the splits then runs with independent loads. (The first version had every thread walk
// all splits twice with dependent loads: 12 us at 64 splits, more than the attention kernel it follows.)
__global__ void decode_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                    __nv_bfloat16* __restrict__ out, int H, int D, int splits) {
  __shared__ float w_s[256];
  __shared__ float red[2][8];
  pdl_wait();     // no-op unless launched with programmatic stream serialization: the kernel in front has completed
  pdl_trigger();  // the next kernel may start its prologue (and a GEMM its weight prefetch) under this kernel's tail
  const int b = blockIdx.x, h = blockIdx.y, d = threadIdx.x, lane = d & 31, wp = d >> 5, nw = (blockDim.x + 31) >> 5;
  const long long base = (static_cast<long long>(b) * H + h) * splits;
  // maximum over the splits
  float m = -INFINITY;
  for (int s = d; s < splits; s += blockDim.x) m = fmaxf(m, part_ml[(base + s) * 2]);
  m = warp_max(m);
  if (lane == 0) red[0][wp] = m;
  __syncthreads();
  m = -INFINITY;
  for (int i = 0; i < nw; ++i) m = fmaxf(m, red[0][i]);
  // weights and the denominator
  float den = 0.f;
  for (int s = d; s < splits; s += blockDim.x) {
    const float ms = part_ml[(base + s) * 2];
    const float w = (ms == -INFINITY) ? 0.f : __expf(ms - m);
    if (s < 256) w_s[s] = w;
    den += w * part_ml[(base + s) * 2 + 1];
  }
  den = warp_sum(den);
  if (lane == 0) red[1][wp] = den;
  __syncthreads();
  den = 0.f;
  for (int i = 0; i < nw; ++i) den += red[1][i];
  float num = 0.f;
  const int n_fast = splits < 256 ? splits : 256;
#pragma unroll 8
  for (int s = 0; s < n_fast; ++s) num += w_s[s] * part_o[(base + s) * D + d];
  for (int s = n_fast; s < splits; ++s) {  // (more than 256 splits: weights recomputed)
    const float ms = part_ml[(base + s) * 2];
    num += ((ms == -INFINITY) ? 0.f : __expf(ms - m)) * part_o[(base + s) * D + d];
  }
  out[(static_cast<long long>(b) * H + h) * D + d] = f2bf(den > 0.f ? num / den : 0.f);
}

template <int D, int GP>
static size_t decode_smem_bytes() {
  constexpr int KG = 128 / (D / 4);
  const size_t kv = static_cast<size_t>(4) * 32 * D * 2;
  const size_t fl = (static_cast<size_t>((GP * 32 + 3 * GP + 3) & ~3) + static_cast<size_t>(KG) * GP * D) * 4;
  return kv + fl;
}

template <int D, int GP>
static int launch_decode_t(const void* q, long long q_stride, const void* kc, const void* vc, const int* bt, int bt_stride,
                           const int* ctx, void* out, float* po, float* pml, int B, int H, int KV, int page, float scale,
                           float cap, int window, int splits, cudaStream_t st) {
  const size_t smem = decode_smem_bytes<D, GP>();
  static PerDeviceOnce attr_once;
  if (attr_once.first()) {
    cudaFuncSetAttribute(decode_attn_kernel<D, GP>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  }
  dim3 grid(B, KV, splits);
  decode_attn_kernel<D, GP><<<grid, 128, smem, st>>>(static_cast<const __nv_bfloat16*>(q), q_stride,
                                                      static_cast<const __nv_bfloat16*>(kc), static_cast<const __nv_bfloat16*>(vc),
                                                      bt, bt_stride, ctx, static_cast<__nv_bfloat16*>(out), po, pml, H, KV, page,
                                                      scale, cap, window, splits);
  if (splits > 1) {
    dim3 g2(B, H);
    launch_pdl(decode_merge_kernel, dim3(g2), dim3(D), 0, st, po, pml, static_cast<__nv_bfloat16*>(out), H, D, splits);
  }
  return 0;
}

int launch_decode_attention(const void* q, long long q_stride, const void* kc, const void* vc, const int* bt, int bt_stride,
                            const int* ctx, void* out, float* po, float* pml, int B, int H, int KV, int D, int page, float scale,
                            float cap, int window, int splits, cudaStream_t st) {
  if (B == 0) return 0;
  const int G = H / KV;
  int gp = 1;
  while (gp < G) gp <<= 1;
#define DLV_DEC(DD, GG) \
  return launch_decode_t<DD, GG>(q, q_stride, kc, vc, bt, bt_stride, ctx, out, po, pml, B, H, KV, page, scale, cap, window, splits, st)
#define DLV_DEC_D(DD)                \
  switch (gp) {                      \
    case 1: DLV_DEC(DD, 1);          \
    case 2: DLV_DEC(DD, 2);          \
    case 4: DLV_DEC(DD, 4);          \
    case 8: DLV_DEC(DD, 8);          \
    default: return 2;               \
  }
  switch (D) {
    case 64: DLV_DEC_D(64)
    case 128: DLV_DEC_D(128)
    case 256: DLV_DEC_D(256)
    default: return 1;
  }
#undef DLV_DEC_D
#undef DLV_DEC
}

// =====================================================================================================================
// Prefill (flash, mma.sync m16n8k16 bf16 -> fp32)
// =====================================================================================================================
__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void mma_bf16_16816(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// tile (row-major [rows][D] bf16, 16 B chunks XOR-swizzled with row % 8): byte offset of (row, chunk)
template <int D>
__device__ __forceinline__ uint32_t swz(int row, int chunk) {
  return static_cast<uint32_t>(row * D * 2 + ((chunk ^ (row & 7)) << 4));
}

// =====================================================================================================================
// Decode on the tensor cores (GQA groups of up to 16 query heads)
// =====================================================================================================================
// The CUDA-core decode kernel above needs one FMA per (key, dim, head) and is issue bound long before the KV stream reaches
// the HBM rate. Here the G query heads that share a KV head are the rows of a 16 x D MMA A-operand (rows >= G are zero), so a
// 16-key slice of K / V costs 2 * D / 8 mma.sync instead of 16 * D * G FMAs.
//   grid (num_seqs, KV, splits), 4 warps. The warps work independently: warp w takes the 16-key slices w, w + 4, ... of the
//   CTA's key range through its own three-stage cp.async ring (no CTA-wide barrier in the loop) and keeps its own online-
//   softmax state; the four states are merged through shared memory at the end. A slice never straddles a page
//   (page_size % 16 == 0), so it needs one block-table lookup.
template <int D>
struct DecodeMma {
  static constexpr int kStages = 3;
  static constexpr int kSliceBytes = 16 * D * 2;                 // K or V of one slice
  static constexpr int kWarpBytes = kStages * 2 * kSliceBytes;   // ring of one warp
  static constexpr int kQBytes = 16 * D * 2;                     // D > 128: the query tile stays in shared memory
  static constexpr int kRing = 4 * kWarpBytes;
  static constexpr int kMerge = 4 * 16 * (D + 2) * 4;            // per warp: 16 rows x (D + m + l) fp32 (aliases the rings)
  static constexpr int kBytes = (kRing > kMerge ? kRing : kMerge) + (D > 128 ? kQBytes : 0);
};

template <int D>
__global__ void __launch_bounds__(128, (D <= 128 ? 2 : 1)) decode_attn_mma_kernel(
    const __nv_bfloat16* __restrict__ q, long long q_stride, const __nv_bfloat16* __restrict__ k_cache,
    const __nv_bfloat16* __restrict__ v_cache, const int* __restrict__ block_tables, int bt_stride,
    const int* __restrict__ ctx_lens, __nv_bfloat16* __restrict__ out, float* part_o, float* part_ml, int* __restrict__ arrivals,
    int H, int KV, int page_size, float scale, float softcap, int window, int splits) {
  pdl_wait();     // no-op unless launched with programmatic stream serialization: the kernel in front has completed
  pdl_trigger();  // the next kernel may start its prologue (and a GEMM its weight prefetch) under this kernel's tail
  using L = DecodeMma<D>;
  constexpr int CPR = D / 8;  // 16-byte chunks per row
  extern __shared__ __align__(128) uint8_t msm[];
  const int b = blockIdx.x, kvh = blockIdx.y, sp = blockIdx.z;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t4 = lane & 3;
  const int G = H / KV;
  const int ctx = ctx_lens[b];
  const int first_key = (window > 0 && ctx > window) ? ctx - window : 0;
  // slices of 16 keys; the CTA's share of [first_key, ctx)
  const int sl_lo = first_key / 16, sl_hi = (ctx + 15) / 16;
  const int per = (sl_hi - sl_lo + splits - 1) / splits;
  const int s0 = sl_lo + sp * per, s1 = min(sl_hi, s0 + per);
  uint8_t* ring = msm + warp * L::kWarpBytes;
  const uint32_t ring_u = smem_u32(ring);
  const __nv_bfloat16* qrow = q + static_cast<long long>(b) * q_stride + static_cast<long long>(kvh) * G * D;

  // ---- query A-fragments: registers (D <= 128) or a swizzled shared tile read with ldmatrix (D = 256)
  uint32_t qa[D <= 128 ? D / 16 : 1][4];
  uint8_t* sQ = msm + (L::kRing > L::kMerge ? L::kRing : L::kMerge);
  if constexpr (D <= 128) {
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
      const int d0 = ks * 16 + 2 * t4;
      qa[ks][0] = g < G ? *reinterpret_cast<const uint32_t*>(qrow + g * D + d0) : 0u;
      qa[ks][1] = g + 8 < G ? *reinterpret_cast<const uint32_t*>(qrow + (g + 8) * D + d0) : 0u;
      qa[ks][2] = g < G ? *reinterpret_cast<const uint32_t*>(qrow + g * D + d0 + 8) : 0u;
      qa[ks][3] = g + 8 < G ? *reinterpret_cast<const uint32_t*>(qrow + (g + 8) * D + d0 + 8) : 0u;
    }
  } else {
    for (int c = tid; c < 16 * CPR; c += 128) {
      const int r = c / CPR, cc = c % CPR;
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      if (r < G) v = *reinterpret_cast<const uint4*>(qrow + r * D + cc * 8);
      *reinterpret_cast<uint4*>(sQ + swz<D>(r, cc)) = v;
    }
    __syncthreads();
  }

  auto load_slice = [&](int sl, int stage) {
    // 16 keys x D of K and V: 2 * 16 * CPR chunks over 32 lanes
    const int key0 = sl * 16;
    const int page = block_tables[static_cast<long long>(b) * bt_stride + key0 / page_size];
    const long long base = ((static_cast<long long>(page) * KV + kvh) * page_size + key0 % page_size) * D;
    const uint32_t kdst = ring_u + stage * 2 * L::kSliceBytes, vdst = kdst + L::kSliceBytes;
#pragma unroll
    for (int i = 0; i < 16 * CPR / 32; ++i) {
      const int c = i * 32 + lane;
      const int r = c / CPR, cc = c % CPR;
      const bool valid = key0 + r < ctx;
      const long long off = base + static_cast<long long>(valid ? r : 0) * D + cc * 8;
      cp_async16(kdst + swz<D>(r, cc), k_cache + off, valid);
      cp_async16(vdst + swz<D>(r, cc), v_cache + off, valid);
    }
  };
  // ---- per-warp pipeline over its slices
  float o[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  const int first = s0 + warp;
  const int n_mine = first < s1 ? (s1 - first + 3) / 4 : 0;
#pragma unroll
  for (int j = 0; j < L::kStages - 1; ++j) {
    if (j < n_mine) load_slice(first + 4 * j, j);
    cp_async_commit();
  }
  for (int j = 0; j < n_mine; ++j) {
    const int stage = j % L::kStages;
    if (j + L::kStages - 1 < n_mine) load_slice(first + 4 * (j + L::kStages - 1), (j + L::kStages - 1) % L::kStages);
    cp_async_commit();
    cp_async_wait<L::kStages - 1>();
    __syncwarp();
    const int key0 = (first + 4 * j) * 16;
    const uint32_t kbase = ring_u + stage * 2 * L::kSliceBytes, vbase = kbase + L::kSliceBytes;
    // S (16 heads x 16 keys) = Q K^T
    float sc[2][4];
#pragma unroll
    for (int i = 0; i < 2; ++i) sc[i][0] = sc[i][1] = sc[i][2] = sc[i][3] = 0.f;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
      uint32_t b0, b1, b2, b3;
      ldmatrix_x4(kbase + swz<D>((lane & 7) + (lane >> 4) * 8, ks * 2 + ((lane >> 3) & 1)), b0, b1, b2, b3);
      if constexpr (D <= 128) {
        mma_bf16_16816(sc[0], qa[ks], b0, b1);
        mma_bf16_16816(sc[1], qa[ks], b2, b3);
      } else {
        uint32_t a[4];
        ldmatrix_x4(smem_u32(sQ) + swz<D>((lane & 7) + ((lane >> 3) & 1) * 8, ks * 2 + (lane >> 4)), a[0], a[1], a[2], a[3]);
        mma_bf16_16816(sc[0], a, b0, b1);
        mma_bf16_16816(sc[1], a, b2, b3);
      }
    }
    // scale, softcap, mask (keys outside [first_key, ctx)), online softmax per head row
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int key = key0 + nt * 8 + 2 * t4 + (e & 1);
        float v = softcap_apply(sc[nt][e] * scale, softcap);
        v = (key < ctx && key >= first_key) ? v : -INFINITY;
        sc[nt][e] = v;
        mx[e >> 1] = fmaxf(mx[e >> 1], v);
      }
    }
    float alpha[2], m_new[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
      m_new[r] = fmaxf(m_run[r], mx[r]);
      alpha[r] = (m_run[r] == -INFINITY) ? 0.f : __expf(m_run[r] - m_new[r]);
      m_run[r] = m_new[r];
    }
    float rs[2] = {0.f, 0.f};
    uint32_t pa[4];
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
      float pr[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float mm = m_new[e >> 1];
        pr[e] = (sc[nt][e] == -INFINITY || mm == -INFINITY) ? 0.f : __expf(sc[nt][e] - mm);
        rs[e >> 1] += pr[e];
      }
      pa[nt * 2 + 0] = pack_bf162(pr[0], pr[1]);
      pa[nt * 2 + 1] = pack_bf162(pr[2], pr[3]);
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      rs[r] += __shfl_xor_sync(0xffffffffu, rs[r], 1);
      rs[r] += __shfl_xor_sync(0xffffffffu, rs[r], 2);
      l_run[r] = l_run[r] * alpha[r] + rs[r];
    }
    const bool rescale = alpha[0] != 1.f || alpha[1] != 1.f;
    if (__any_sync(0xffffffffu, rescale)) {
#pragma unroll
      for (int i = 0; i < D / 8; ++i) {
        o[i][0] *= alpha[0];
        o[i][1] *= alpha[0];
        o[i][2] *= alpha[1];
        o[i][3] *= alpha[1];
      }
    }
    // O (16 heads x D) += P V
#pragma unroll
    for (int dt = 0; dt < D / 8; dt += 2) {
      uint32_t b0, b1, b2, b3;
      ldmatrix_x4_trans(vbase + swz<D>((lane & 7) + ((lane >> 3) & 1) * 8, dt + (lane >> 4)), b0, b1, b2, b3);
      mma_bf16_16816(o[dt], pa, b0, b1);
      mma_bf16_16816(o[dt + 1], pa, b2, b3);
    }
    __syncwarp();  // the stage is refilled by this warp's next load_slice
  }
  cp_async_wait<0>();
  __syncthreads();  // every warp is done with its ring: the merge area aliases the rings

  // ---- merge the four warps: each stores its rows < G as [row][D + 2] = O (unnormalised), m, l
  float* mg = reinterpret_cast<float*>(msm);
  {
    float* mine = mg + static_cast<size_t>(warp) * 16 * (D + 2);
#pragma unroll
    for (int dt = 0; dt < D / 8; ++dt) {
      const int d = dt * 8 + 2 * t4;
      if (g < G) *reinterpret_cast<float2*>(mine + g * (D + 2) + d) = make_float2(o[dt][0], o[dt][1]);
      if (g + 8 < G) *reinterpret_cast<float2*>(mine + (g + 8) * (D + 2) + d) = make_float2(o[dt][2], o[dt][3]);
    }
    if (t4 == 0) {
      if (g < G) {
        mine[g * (D + 2) + D] = m_run[0];
        mine[g * (D + 2) + D + 1] = l_run[0];
      }
      if (g + 8 < G) {
        mine[(g + 8) * (D + 2) + D] = m_run[1];
        mine[(g + 8) * (D + 2) + D + 1] = l_run[1];
      }
    }
  }
  __syncthreads();
  for (int idx = tid; idx < G * (D / 2); idx += 128) {
    const int r = idx / (D / 2), d = (idx % (D / 2)) * 2;
    float m = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) m = fmaxf(m, mg[(w * 16 + r) * (D + 2) + D]);
    float n0 = 0.f, n1 = 0.f, den = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float* row = mg + (w * 16 + r) * (D + 2);
      const float wt = (row[D] == -INFINITY) ? 0.f : __expf(row[D] - m);
      n0 += wt * row[d];
      n1 += wt * row[d + 1];
      den += wt * row[D + 1];
    }
    const int h = kvh * G + r;
    if (splits == 1) {
      const float inv = den > 0.f ? 1.f / den : 0.f;
      *reinterpret_cast<uint32_t*>(out + (static_cast<long long>(b) * H + h) * D + d) = pack_bf162(n0 * inv, n1 * inv);
    } else {
      const long long base = (static_cast<long long>(b) * H + h) * splits + sp;
      *reinterpret_cast<float2*>(part_o + base * D + d) = make_float2(n0, n1);
      if (d == 0) {
        part_ml[base * 2] = m;
        part_ml[base * 2 + 1] = den;
      }
    }
  }
  if (splits == 1 || arrivals == nullptr) return;  // (no arrival counters: decode_merge_kernel follows)

  // ---- (opt-in; measured slower than decode_merge_kernel) merge of the splits by the CTA that finishes last for this
  // (sequence, KV head): no second launch.
  // Every CTA publishes its partials (fence), then counts itself in; the one that sees splits - 1 earlier arrivals puts the
  // counter back to zero for the next launch and combines all partials in split order, so the result does not depend on
  // which CTA came last. Nothing waits.
  __shared__ int s_last;
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const int prev = atomicAdd(arrivals + b * KV + kvh, 1);
    s_last = prev == splits - 1;
    if (s_last) arrivals[b * KV + kvh] = 0;
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  float* w_s = mg;  // [G][splits] weights, then [G] denominators (the warp-merge area is free again)
  float* den_s = mg + G * splits;
  if (G * (splits + 1) <= L::kMerge / 4) {
    for (int r = warp; r < G; r += 4) {
      const long long base = (static_cast<long long>(b) * H + kvh * G + r) * splits;
      float m = -INFINITY;
      for (int s2 = lane; s2 < splits; s2 += 32) m = fmaxf(m, __ldcg(part_ml + (base + s2) * 2));
      m = warp_max(m);
      float den = 0.f;
      for (int s2 = lane; s2 < splits; s2 += 32) {
        const float ms = __ldcg(part_ml + (base + s2) * 2);
        const float w = (ms == -INFINITY) ? 0.f : __expf(ms - m);
        w_s[r * splits + s2] = w;
        den += w * __ldcg(part_ml + (base + s2) * 2 + 1);
      }
      den = warp_sum(den);
      if (lane == 0) den_s[r] = den;
    }
    __syncthreads();
    for (int idx = tid; idx < G * (D / 2); idx += 128) {
      const int r = idx / (D / 2), d = (idx % (D / 2)) * 2;
      const int h = kvh * G + r;
      const long long base = (static_cast<long long>(b) * H + h) * splits;
      float n0 = 0.f, n1 = 0.f;
#pragma unroll 4
      for (int s2 = 0; s2 < splits; ++s2) {
        const float2 v = __ldcg(reinterpret_cast<const float2*>(part_o + (base + s2) * D + d));
        const float w = w_s[r * splits + s2];
        n0 += w * v.x;
        n1 += w * v.y;
      }
      const float den = den_s[r];
      const float inv = den > 0.f ? 1.f / den : 0.f;
      *reinterpret_cast<uint32_t*>(out + (static_cast<long long>(b) * H + h) * D + d) = pack_bf162(n0 * inv, n1 * inv);
    }
  }
}

template <int D>
static int launch_decode_mma_t(const void* q, long long q_stride, const void* kc, const void* vc, const int* bt, int bt_stride,
                               const int* ctx, void* out, float* po, float* pml, int* arrivals, int B, int H, int KV, int page,
                               float scale, float cap, int window, int splits, cudaStream_t st) {
  using L = DecodeMma<D>;
  // the in-kernel merge keeps its weights in the warp-merge area of shared memory
  if (splits > 1 && (H / KV) * (splits + 1) > L::kMerge / 4) arrivals = nullptr;
  static PerDeviceOnce attr_once;
  if (attr_once.first()) {
    cudaFuncSetAttribute(decode_attn_mma_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kBytes);
  }
  dim3 grid(B, KV, splits);
  launch_pdl(decode_attn_mma_kernel<D>, dim3(grid), dim3(128), L::kBytes, st, static_cast<const __nv_bfloat16*>(q), q_stride,
                                                          static_cast<const __nv_bfloat16*>(kc), static_cast<const __nv_bfloat16*>(vc), bt,
                                                          bt_stride, ctx, static_cast<__nv_bfloat16*>(out), po, pml, arrivals, H, KV, page, scale,
                                                          cap, window, splits);
  if (splits > 1 && arrivals == nullptr) {
    dim3 g2(B, H);
    launch_pdl(decode_merge_kernel, dim3(g2), dim3(D), 0, st, po, pml, static_cast<__nv_bfloat16*>(out), H, D, splits);
  }
  return 0;
}

// impl: 0 = tensor-core kernel when it applies (group <= 16, page_size % 16 == 0), 1 = CUDA-core kernel
int launch_decode_attention_impl(const void* q, long long q_stride, const void* kc, const void* vc, const int* bt, int bt_stride,
                                 const int* ctx, void* out, float* po, float* pml, int* arrivals, int B, int H, int KV, int D, int page,
                                 float scale, float cap, int window, int splits, int impl, cudaStream_t st) {
  if (B == 0) return 0;
  const int G = H / KV;
  if (impl == 0 && G <= 16 && page % 16 == 0 && (q_stride % 2) == 0) {
    switch (D) {
      case 64: return launch_decode_mma_t<64>(q, q_stride, kc, vc, bt, bt_stride, ctx, out, po, pml, arrivals, B, H, KV, page, scale, cap, window, splits,
                                                st);
      case 128: return launch_decode_mma_t<128>(q, q_stride, kc, vc, bt, bt_stride, ctx, out, po, pml, arrivals, B, H, KV, page, scale, cap, window, splits,
                                                st);
      case 256: return launch_decode_mma_t<256>(q, q_stride, kc, vc, bt, bt_stride, ctx, out, po, pml, arrivals, B, H, KV, page, scale, cap, window, splits,
                                                st);
      default: return 1;
    }
  }
  return launch_decode_attention(q, q_stride, kc, vc, bt, bt_stride, ctx, out, po, pml, B, H, KV, D, page, scale, cap, window, splits, st);
}

// grid (num_q_tiles, H), 128 threads; tile i covers query rows [tile_q0[i], tile_q0[i] + 64) of sequence tile_seq[i]
template <int D>
__global__ void __launch_bounds__(128) prefill_attn_kernel(
    const __nv_bfloat16* __restrict__ q, long long q_stride, const __nv_bfloat16* __restrict__ k_cache,
    const __nv_bfloat16* __restrict__ v_cache, const int* __restrict__ block_tables, int bt_stride,
    const int* __restrict__ q_start, const int* __restrict__ q_len, const int* __restrict__ ctx_lens,
    const int* __restrict__ tile_seq, const int* __restrict__ tile_q0, __nv_bfloat16* __restrict__ out,  // [T, H, D]
    int H, int KV, int page_size, float scale, float softcap, int window, int causal) {
  pdl_wait();     // no-op unless launched with programmatic stream serialization: the kernel in front has completed
  pdl_trigger();  // the next kernel may start its prologue (and a GEMM its weight prefetch) under this kernel's tail
  constexpr int BM = 64, BN = 64, CPR = D / 8;
  extern __shared__ __align__(128) uint8_t psm[];
  uint8_t* sQ = psm;                       // BM * D * 2
  uint8_t* sK = sQ + BM * D * 2;           // 2 buffers
  uint8_t* sV = sK + 2 * BN * D * 2;       // 2 buffers
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int seq = tile_seq[blockIdx.x], q0 = tile_q0[blockIdx.x], h = blockIdx.y;
  const int kvh = h / (H / KV);
  const int qs = q_start[seq], ql = q_len[seq], ctx = ctx_lens[seq];
  const int pos0 = ctx - ql;  // position of query row 0 of this sequence
  const int rows = min(BM, ql - q0);
  // key range needed by this tile
  const int last_pos = causal ? pos0 + q0 + rows - 1 : ctx - 1;
  const int first_pos = pos0 + q0;
  const int key_hi = min(ctx, last_pos + 1);
  const int key_lo = (window > 0) ? max(0, first_pos - window + 1) : 0;
  const int kt0 = key_lo / BN, kt1 = (key_hi + BN - 1) / BN;

  // ---- Q tile
  for (int c = tid; c < BM * CPR; c += 128) {
    const int r = c / CPR, cc = c % CPR;
    const bool valid = r < rows;
    const __nv_bfloat16* src = q + static_cast<long long>(qs + q0 + (valid ? r : 0)) * q_stride + static_cast<long long>(h) * D + cc * 8;
    cp_async16(smem_u32(sQ) + swz<D>(r, cc), src, valid);
  }
  auto load_kv = [&](int kt, int buf) {
    for (int c = tid; c < BN * CPR; c += 128) {
      const int r = c / CPR, cc = c % CPR;
      const int key = kt * BN + r;
      const bool valid = key < ctx;
      const int kk = valid ? key : 0;
      const int page = block_tables[static_cast<long long>(seq) * bt_stride + kk / page_size];
      const long long off = ((static_cast<long long>(page) * KV + kvh) * page_size + kk % page_size) * D + cc * 8;
      cp_async16(smem_u32(sK) + buf * BN * D * 2 + swz<D>(r, cc), k_cache + off, valid);
      cp_async16(smem_u32(sV) + buf * BN * D * 2 + swz<D>(r, cc), v_cache + off, valid);
    }
    cp_async_commit();
  };
  if (kt0 < kt1) load_kv(kt0, 0); else cp_async_commit();

  float o[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  const int g = lane >> 2, t4 = lane & 3;
  const int row_a = warp * 16 + g, row_b = row_a + 8;           // rows inside the tile
  const int pos_a = first_pos + row_a, pos_b = first_pos + row_b;  // absolute positions (first_pos = pos0 + q0)

  for (int kt = kt0; kt < kt1; ++kt) {
    const int buf = (kt - kt0) & 1;
    if (kt + 1 < kt1) {
      load_kv(kt + 1, buf ^ 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const uint32_t kbase = smem_u32(sK) + buf * BN * D * 2, vbase = smem_u32(sV) + buf * BN * D * 2;
    // ---- S = Q K^T (16 rows x 64 keys per warp)
    float s[BN / 8][4];
#pragma unroll
    for (int i = 0; i < BN / 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
      uint32_t a[4];
      ldmatrix_x4(smem_u32(sQ) + swz<D>(warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, ks * 2 + (lane >> 4)), a[0], a[1], a[2], a[3]);
#pragma unroll
      for (int nt = 0; nt < BN / 8; nt += 2) {
        // two key tiles (nt, nt + 1) x this k-step: matrices (keys nt, d lo), (keys nt, d hi), (keys nt+1, d lo), (keys nt+1, d hi)
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4(kbase + swz<D>(nt * 8 + (lane & 7) + (lane >> 4) * 8, ks * 2 + ((lane >> 3) & 1)), b0, b1, b2, b3);
        mma_bf16_16816(s[nt], a, b0, b1);
        mma_bf16_16816(s[nt + 1], a, b2, b3);
      }
    }
    // ---- scale, softcap, mask, online softmax
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nt = 0; nt < BN / 8; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int key = kt * BN + nt * 8 + 2 * t4 + (e & 1);
        const int pos = (e < 2) ? pos_a : pos_b;
        float v = softcap_apply(s[nt][e] * scale, softcap);
        bool vis = key < ctx;
        if (causal) vis = vis && key <= pos;
        if (window > 0) vis = vis && key > pos - window;
        v = vis ? v : -INFINITY;
        s[nt][e] = v;
        mx[e >> 1] = fmaxf(mx[e >> 1], v);
      }
    }
    float alpha[2], m_new[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
      m_new[r] = fmaxf(m_run[r], mx[r]);
      alpha[r] = (m_run[r] == -INFINITY) ? 0.f : __expf(m_run[r] - m_new[r]);
      m_run[r] = m_new[r];
    }
    float rs[2] = {0.f, 0.f};
    uint32_t pa[BN / 16][4];
#pragma unroll
    for (int nt = 0; nt < BN / 8; ++nt) {
      float p[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float mm = m_new[e >> 1];
        p[e] = (s[nt][e] == -INFINITY || mm == -INFINITY) ? 0.f : __expf(s[nt][e] - mm);
        rs[e >> 1] += p[e];
      }
      pa[nt >> 1][(nt & 1) * 2 + 0] = pack_bf162(p[0], p[1]);
      pa[nt >> 1][(nt & 1) * 2 + 1] = pack_bf162(p[2], p[3]);
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      rs[r] += __shfl_xor_sync(0xffffffffu, rs[r], 1);
      rs[r] += __shfl_xor_sync(0xffffffffu, rs[r], 2);
      l_run[r] = l_run[r] * alpha[r] + rs[r];
    }
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
      o[i][0] *= alpha[0];
      o[i][1] *= alpha[0];
      o[i][2] *= alpha[1];
      o[i][3] *= alpha[1];
    }
    // ---- O += P V
#pragma unroll
    for (int kk = 0; kk < BN / 16; ++kk) {
#pragma unroll
      for (int dt = 0; dt < D / 8; dt += 2) {
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4_trans(vbase + swz<D>(kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, dt + (lane >> 4)), b0, b1, b2, b3);
        mma_bf16_16816(o[dt], pa[kk], b0, b1);
        mma_bf16_16816(o[dt + 1], pa[kk], b2, b3);
      }
    }
    __syncthreads();
  }
  cp_async_wait<0>();
  // ---- write
  const float inv_a = l_run[0] > 0.f ? 1.f / l_run[0] : 0.f, inv_b = l_run[1] > 0.f ? 1.f / l_run[1] : 0.f;
#pragma unroll
  for (int dt = 0; dt < D / 8; ++dt) {
    const int d = dt * 8 + 2 * t4;
    if (row_a < rows)
      *reinterpret_cast<uint32_t*>(out + (static_cast<long long>(qs + q0 + row_a) * H + h) * D + d) = pack_bf162(o[dt][0] * inv_a, o[dt][1] * inv_a);
    if (row_b < rows)
      *reinterpret_cast<uint32_t*>(out + (static_cast<long long>(qs + q0 + row_b) * H + h) * D + d) = pack_bf162(o[dt][2] * inv_b, o[dt][3] * inv_b);
  }
}

template <int D>
static int launch_prefill_t(const void* q, long long q_stride, const void* kc, const void* vc, const int* bt, int bt_stride,
                            const int* q_start, const int* q_len, const int* ctx, const int* tile_seq, const int* tile_q0,
                            int num_tiles, void* out, int H, int KV, int page, float scale, float cap, int window, int causal,
                            cudaStream_t st) {
  const size_t smem = static_cast<size_t>(64 * D * 2) * 5;
  static PerDeviceOnce attr_once;
  if (attr_once.first()) {
    cudaFuncSetAttribute(prefill_attn_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  }
  dim3 grid(num_tiles, H);
  prefill_attn_kernel<D><<<grid, 128, smem, st>>>(static_cast<const __nv_bfloat16*>(q), q_stride, static_cast<const __nv_bfloat16*>(kc),
                                                   static_cast<const __nv_bfloat16*>(vc), bt, bt_stride, q_start, q_len, ctx, tile_seq,
                                                   tile_q0, static_cast<__nv_bfloat16*>(out), H, KV, page, scale, cap, window, causal);
  return 0;
}

int launch_prefill_attention(const void* q, long long q_stride, const void* kc, const void* vc, const int* bt, int bt_stride,
                             const int* q_start, const int* q_len, const int* ctx, const int* tile_seq, const int* tile_q0,
                             int num_tiles, void* out, int H, int KV, int D, int page, float scale, float cap, int window,
                             int causal, cudaStream_t st) {
  if (num_tiles == 0) return 0;
  switch (D) {
    case 64:
      return launch_prefill_t<64>(q, q_stride, kc, vc, bt, bt_stride, q_start, q_len, ctx, tile_seq, tile_q0, num_tiles, out, H, KV,
                                  page, scale, cap, window, causal, st);
    case 128:
      return launch_prefill_t<128>(q, q_stride, kc, vc, bt, bt_stride, q_start, q_len, ctx, tile_seq, tile_q0, num_tiles, out, H, KV,
                                   page, scale, cap, window, causal, st);
    case 256:
      return launch_prefill_t<256>(q, q_stride, kc, vc, bt, bt_stride, q_start, q_len, ctx, tile_seq, tile_q0, num_tiles, out, H, KV,
                                   page, scale, cap, window, causal, st);
    default:
      return 1;
  }
}

}  // namespace dlv
