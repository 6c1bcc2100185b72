// Paged flash attention for prefill on the 5th-generation tensor cores (tcgen05 / TMEM / TMA).
//
// One CTA per (128 query rows of one sequence, query head). Six warps:
//   warp 4, one lane  = TMA producer: the Q tile once (D / 64 boxes of 128 rows x 64 columns), then per 128-key tile the K and V rows
//                       of four cache pages (a page slice of one KV head is 32 rows x D contiguous bf16 = D / 64 boxes of 32 x 64),
//                       all into 128-byte-swizzled shared memory, completion on mbarriers; two K/V stages when they fit;
//   warp 5, one lane  = MMA issuer: S = Q K^T (both operands from shared memory, K-major, accumulator = 128 TMEM columns), then
//                       O += P V (P from tensor memory as the A operand, V from shared memory as an MN-major B operand);
//   warps 0-3         = softmax: thread r owns query row r (TMEM lane r): tcgen05.ld of the score row in 32-column chunks, mask
//                       (causal / sliding window / context end), optional logit soft-cap, running maximum and sum kept in
//                       registers, rescale of the O accumulator in tensor memory when the maximum moves, P written back to tensor
//                       memory as packed bf16 (tcgen05.st), final O / l to global memory.
// Tensor memory: S at columns [0, 128), P at [128, 192), O at [256, 256 + D) (at [192, 256) for D = 64, where 256 columns are allocated).
// The MMAs of one thread execute in issue order, so "S of tile j + 1 complete" also means "P V of tile j complete": the softmax
// warps may rescale O as soon as the next scores have arrived, and no separate barrier guards the accumulator.
// Every wait is bounded (common.cuh); on expiry the CTA records a status word, skips its stores, frees tensor memory and returns.
//
// Replaces the reference's packed prefill attention (core/.../generator/CausalSelfAttention.java:458-502: per head QK^T GEMM over
// the visible pages, causal scaled softmax with optional soft-cap, saxpy with V).
#include <stdexcept>
#include <string>

#include "common.cuh"
#include "gemm_api.h"

namespace dlv {

void encode_map_2d(CUtensorMap* map, int dtype_code, const void* base, uint64_t rows, uint64_t cols, uint64_t pitch_bytes, uint32_t box_rows,
                   uint32_t box_cols, int swizzle_code);

struct AttnTcParams {
  const int* block_tables;
  int bt_stride;
  const int* q_start;
  const int* q_len;
  const int* ctx_lens;
  const int* tile_seq;
  const int* tile_q0;
  __nv_bfloat16* out;  // [T, H * D]
  int H, KV, page_size;
  float scale, softcap;
  int window, causal;
  int* status;
};

// MN-major shared-memory descriptor (128-byte swizzle): the operand tile is stored as rows of the K dimension, each row 64 elements of
// the MN dimension (128 bytes); 8 rows form a 1 KB swizzle atom. lbo: bytes between atoms along MN (the next 64 columns), sbo: bytes
// between atoms along K (the next 8 rows).
__device__ __forceinline__ uint64_t umma_desc_mn_sw128(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}
// kind::f16, bf16 x bf16 -> fp32, A K-major, B MN-major
__host__ __device__ constexpr uint32_t umma_idesc_bf16_bmn(int m, int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (0u << 15) | (1u << 16) | (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}
__device__ __forceinline__ void tmem_ld_x32(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]),
        "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
}
__device__ __forceinline__ void tmem_st_x32(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]),
      "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]),
      "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}

constexpr int kAtBM = 128, kAtBN = 128;  // query rows / keys per tile
constexpr int kAtThreads = 192;

template <int D>
struct AttnTcSmem {
  static constexpr int kSub = D / 64;                 // 64-column sub-tiles per operand tile
  static constexpr int kTile = kAtBM * 128 * kSub;    // bytes of a [128 rows][D] bf16 tile (Q, K or V)
  static constexpr int kStages = D <= 128 ? 2 : 1;
  static constexpr int kOffK = kTile;
  static constexpr int kOffV = kOffK + kStages * kTile;
  static constexpr int kOffCtrl = kOffV + kStages * kTile;
  static constexpr int kBytes = kOffCtrl + 256 + 1024;  // barriers + alignment slack
};

template <int D>
__global__ void __launch_bounds__(kAtThreads, 1) prefill_attn_tc_kernel(const __grid_constant__ CUtensorMap map_q,  // [T, H * D], box 128 x 64
                                                                        const __grid_constant__ CUtensorMap map_k,  // [pages * KV * page, D], box 32 x 64
                                                                        const __grid_constant__ CUtensorMap map_v, const AttnTcParams p) {
  using L = AttnTcSmem<D>;
  constexpr int NS = L::kStages, SUB = L::kSub;
  extern __shared__ uint8_t at_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(at_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bar_q = reinterpret_cast<uint64_t*>(smem + L::kOffCtrl);
  uint64_t* bar_k_full = bar_q + 1;        // [2]
  uint64_t* bar_v_full = bar_k_full + 2;   // [2]
  uint64_t* bar_kv_empty = bar_v_full + 2; // [2]
  uint64_t* bar_s_full = bar_kv_empty + 2;
  uint64_t* bar_p_full = bar_s_full + 1;
  uint64_t* bar_o_final = bar_p_full + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_o_final + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // a CTA that starts after another one of this or an earlier launch has recorded a failed wait leaves at once: one stuck tile
  // must not make every later tile sit out its own time limit
  if (__syncthreads_or(threadIdx.x == 0 && *reinterpret_cast<volatile int*>(p.status) != 0)) return;
  const int seq = p.tile_seq[blockIdx.x], q0 = p.tile_q0[blockIdx.x], h = blockIdx.y;
  const int kvh = h / (p.H / p.KV);
  const int qs = p.q_start[seq], ql = p.q_len[seq], ctx = p.ctx_lens[seq];
  const int pos0 = ctx - ql;                       // position of the sequence's first query row
  const int rows = min(kAtBM, ql - q0);
  const int first_pos = pos0 + q0;
  const int last_pos = p.causal ? first_pos + rows - 1 : ctx - 1;
  const int key_hi = min(ctx, last_pos + 1);
  const int key_lo = p.window > 0 ? max(0, first_pos - p.window + 1) : 0;
  const int kt0 = key_lo / kAtBN, kt1 = (key_hi + kAtBN - 1) / kAtBN;
  const int n_tiles = kt1 - kt0;

  if (threadIdx.x == 0) {
    mbar_init(smem_u32(bar_q), 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(smem_u32(&bar_k_full[s]), 1);
      mbar_init(smem_u32(&bar_v_full[s]), 1);
      mbar_init(smem_u32(&bar_kv_empty[s]), 1);
    }
    mbar_init(smem_u32(bar_s_full), 1);
    mbar_init(smem_u32(bar_p_full), 4);
    mbar_init(smem_u32(bar_o_final), 1);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&map_q);
    tma_prefetch_desc(&map_k);
    tma_prefetch_desc(&map_v);
  }
  constexpr uint32_t kTmemCols = D <= 64 ? 256 : 512;  // D = 64: two CTAs fit one SM's shared memory, and so do their 2 x 256 columns
  if (warp == 5) tmem_alloc(smem_u32(tmem_slot), kTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  constexpr uint32_t kColS = 0, kColP = 128, kColO = D <= 64 ? 192 : 256;
  pdl_wait();
  pdl_trigger();

  if (warp == 4) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      mbar_expect_tx(smem_u32(bar_q), L::kTile);
      for (int c = 0; c < SUB; ++c) tma_load_2d(smem_u32(smem + c * (kAtBM * 128)), &map_q, smem_u32(bar_q), h * D + c * 64, qs + q0);
      const int pages_per_tile = kAtBN / p.page_size;  // page_size is 32, 64 or 128
      const int box_rows = p.page_size < kAtBN ? p.page_size : kAtBN;
      int issued = 0;
      for (int j = 0; j < n_tiles; ++j, ++issued) {
        const int s = j % NS;
        if (j >= NS && !mbar_wait(smem_u32(&bar_kv_empty[s]), ((j / NS) - 1) & 1, abort_flag, p.status)) break;
        const int kt = kt0 + j;
        mbar_expect_tx(smem_u32(&bar_k_full[s]), L::kTile);
        mbar_expect_tx(smem_u32(&bar_v_full[s]), L::kTile);
        for (int pg = 0; pg < (pages_per_tile > 0 ? pages_per_tile : 1); ++pg) {
          const int key0 = kt * kAtBN + pg * box_rows;
          // pages past the context are never read by an unmasked score; the scratch page 0 keeps the copy inside the cache
          const int page = key0 < ctx ? p.block_tables[static_cast<long long>(seq) * p.bt_stride + key0 / p.page_size] : 0;
          const int row = (page * p.KV + kvh) * p.page_size + (key0 % p.page_size);
          for (int c = 0; c < SUB; ++c) {
            const uint32_t off = c * (kAtBN * 128) + pg * box_rows * 128;
            tma_load_2d(smem_u32(smem + L::kOffK + s * L::kTile + off), &map_k, smem_u32(&bar_k_full[s]), c * 64, row);
            tma_load_2d(smem_u32(smem + L::kOffV + s * L::kTile + off), &map_v, smem_u32(&bar_v_full[s]), c * 64, row);
          }
        }
      }
      if (*abort_flag) {
        // a wait ran out somewhere in the CTA: before shared memory goes away let the copies already issued land (bounded)
        for (int j = issued > NS ? issued - NS : 0; j < issued; ++j) {
          const unsigned long long t0 = globaltimer_ns();
          while (!(mbar_try_wait(smem_u32(&bar_k_full[j % NS]), (j / NS) & 1) && mbar_try_wait(smem_u32(&bar_v_full[j % NS]), (j / NS) & 1)) &&
                 globaltimer_ns() - t0 < 20000000ull) {
          }
        }
      }
    }
  } else if (warp == 5) {
    // ---------------- MMA issuer ----------------
    bool ok = mbar_wait(smem_u32(bar_q), 0, abort_flag, p.status);
    constexpr uint32_t idesc_s = umma_idesc_bf16(kAtBM, kAtBN);
    constexpr uint32_t idesc_o = umma_idesc_bf16_bmn(kAtBM, D);
    const uint64_t desc_q = umma_desc_k_sw128(smem_u32(smem));
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int s = j % NS;
      ok = mbar_wait(smem_u32(&bar_k_full[s]), (j / NS) & 1, abort_flag, p.status);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      if (lane == 0) {
        const uint64_t desc_k = umma_desc_k_sw128(smem_u32(smem + L::kOffK + s * L::kTile));
#pragma unroll
        for (int k16 = 0; k16 < D / 16; ++k16) {
          const uint64_t adv = static_cast<uint64_t>(((k16 >> 2) * (kAtBM * 128) + (k16 & 3) * 32) >> 4);
          umma_bf16(tmem_base + kColS, desc_q + adv, desc_k + adv, idesc_s, k16 > 0 ? 1u : 0u);
        }
        umma_commit(smem_u32(bar_s_full));
      }
      __syncwarp();
      ok = mbar_wait(smem_u32(bar_p_full), j & 1, abort_flag, p.status);
      ok = ok && mbar_wait(smem_u32(&bar_v_full[s]), (j / NS) & 1, abort_flag, p.status);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      if (lane == 0) {
        const uint32_t vbase = smem_u32(smem + L::kOffV + s * L::kTile);
#pragma unroll
        for (int k16 = 0; k16 < kAtBN / 16; ++k16) {
          // 16 keys = two 8-row swizzle atoms further down the V tile; the 64-column blocks of D are kAtBN * 128 bytes apart
          const uint64_t desc_v = umma_desc_mn_sw128(vbase + k16 * 2048, kAtBN * 128, 1024);
          umma_bf16_ts(tmem_base + kColO, tmem_base + kColP + k16 * 8, desc_v, idesc_o, (j > 0 || k16 > 0) ? 1u : 0u);
        }
        umma_commit(smem_u32(&bar_kv_empty[s]));
        if (j == n_tiles - 1) umma_commit(smem_u32(bar_o_final));
      }
      __syncwarp();
    }
    if (lane == 0 && (!ok || n_tiles == 0)) {
      umma_commit(smem_u32(bar_o_final));  // also lets outstanding MMAs retire before tensor memory is released
      const unsigned long long t0 = globaltimer_ns();
      while (!mbar_try_wait(smem_u32(bar_o_final), 0) && globaltimer_ns() - t0 < 20000000ull) {
      }
    }
    __syncwarp();
  } else {
    // ---------------- softmax warps: thread = query row ----------------
    const int r = warp * 32 + lane;
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(warp * 32) << 16);
    const int my_pos = first_pos + r;
    const float c_log2 = 1.4426950408889634f;
    float m_run = -INFINITY, l_run = 0.f;
    bool ok = true;
    for (int j = 0; j < n_tiles && ok; ++j) {
      ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(bar_s_full), j & 1, abort_flag, p.status));  // warp-uniform: the loop holds warp-collective TMEM accesses
      if (!ok) break;
      tc_fence_after();
      const int key_base = (kt0 + j) * kAtBN;
      // visible keys of this row inside the tile: [lo, hi)
      int hi = min(ctx, p.causal ? my_pos + 1 : ctx) - key_base;
      int lo = (p.window > 0 ? max(0, my_pos - p.window + 1) : 0) - key_base;
      if (r >= rows) hi = lo = 0;
      hi = hi > kAtBN ? kAtBN : hi;
      lo = lo < 0 ? 0 : lo;
      // pass 1: row maximum of the (scaled, soft-capped) scores
      float mx = -INFINITY;
#pragma unroll 1
      for (int c0 = 0; c0 < kAtBN; c0 += 32) {
        uint32_t v[32];
        tmem_ld_x32(lane_addr + kColS + c0, v);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float sc = __uint_as_float(v[i]) * p.scale;
          if (p.softcap > 0.f) sc = p.softcap * tanhf(sc / p.softcap);
          const int col = c0 + i;
          if (col >= lo && col < hi) mx = fmaxf(mx, sc);
        }
      }
      const float m_new = fmaxf(m_run, mx);
      const float alpha = (m_run == -INFINITY) ? 0.f : exp2f((m_run - m_new) * c_log2);
      // the O accumulator follows the maximum (P V of the previous tile has retired: the MMAs run in issue order and S of this tile is complete)
      // (tcgen05.ld / st are warp-collective: the decision must be the same for the 32 rows of a warp)
      if (j > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
#pragma unroll 1
        for (int c0 = 0; c0 < D; c0 += 32) {
          uint32_t v[32];
          tmem_ld_x32(lane_addr + kColO + c0, v);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
          tmem_st_x32(lane_addr + kColO + c0, v);
        }
      }
      // pass 2: probabilities -> packed bf16 in tensor memory, row sum
      float lsum = 0.f;
#pragma unroll 1
      for (int c0 = 0; c0 < kAtBN; c0 += 32) {
        uint32_t v[32];
        tmem_ld_x32(lane_addr + kColS + c0, v);
        tmem_ld_wait();
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float pv[2];
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            float sc = __uint_as_float(v[i + e]) * p.scale;
            if (p.softcap > 0.f) sc = p.softcap * tanhf(sc / p.softcap);
            const int col = c0 + i + e;
            pv[e] = (col >= lo && col < hi) ? exp2f((sc - m_new) * c_log2) : 0.f;
          }
          const __nv_bfloat162 b2 = __floats2bfloat162_rn(pv[0], pv[1]);
          const float2 back = __bfloat1622float2(b2);  // the sum matches what the tensor core multiplies
          lsum += back.x + back.y;
          pk[i >> 1] = *reinterpret_cast<const uint32_t*>(&b2);
        }
        tmem_st_x16(lane_addr + kColP + (c0 >> 1), pk);
      }
      l_run = l_run * alpha + lsum;
      m_run = m_new;
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(bar_p_full));
    }
    // ---------------- epilogue ----------------
    if (ok) ok = mbar_wait(smem_u32(bar_o_final), 0, abort_flag, p.status);
    ok = __all_sync(0xffffffffu, ok && *abort_flag == 0);
    if (ok) {
      tc_fence_after();
      const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
      __nv_bfloat16* orow = p.out + static_cast<size_t>(qs + q0 + r) * (static_cast<size_t>(p.H) * D) + static_cast<size_t>(h) * D;
#pragma unroll 1
      for (int c0 = 0; c0 < D; c0 += 32) {
        uint32_t v[32];
        if (n_tiles > 0) {
          tmem_ld_x32(lane_addr + kColO + c0, v);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = 0u;
        }
        if (r < rows) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint4 o;
            o.x = pack_bf162(__uint_as_float(v[i]) * inv, __uint_as_float(v[i + 1]) * inv);
            o.y = pack_bf162(__uint_as_float(v[i + 2]) * inv, __uint_as_float(v[i + 3]) * inv);
            o.z = pack_bf162(__uint_as_float(v[i + 4]) * inv, __uint_as_float(v[i + 5]) * inv);
            o.w = pack_bf162(__uint_as_float(v[i + 6]) * inv, __uint_as_float(v[i + 7]) * inv);
            *reinterpret_cast<uint4*>(orow + c0 + i) = o;
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 5) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

template <int D>
static int launch_prefill_tc_t(const void* q, long long q_stride, long long T, const void* kc, const void* vc, long long cache_rows, const AttnTcParams& p,
                               int num_tiles, cudaStream_t st) {
  using L = AttnTcSmem<D>;
  static PerDeviceOnce attr_once;
  if (attr_once.first()) {
    cudaError_t e = cudaFuncSetAttribute(prefill_attn_tc_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kBytes);
    if (e != cudaSuccess) throw std::runtime_error(std::string("prefill attention (tcgen05): cudaFuncSetAttribute: ") + cudaGetErrorString(e));
  }
  CUtensorMap mq, mk, mv;
  encode_map_2d(&mq, 0, q, static_cast<uint64_t>(T), static_cast<uint64_t>(p.H) * D, static_cast<uint64_t>(q_stride) * 2, kAtBM, 64, 128);
  const uint32_t box_rows = p.page_size < kAtBN ? p.page_size : kAtBN;
  encode_map_2d(&mk, 0, kc, static_cast<uint64_t>(cache_rows), D, static_cast<uint64_t>(D) * 2, box_rows, 64, 128);
  encode_map_2d(&mv, 0, vc, static_cast<uint64_t>(cache_rows), D, static_cast<uint64_t>(D) * 2, box_rows, 64, 128);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(num_tiles, p.H);
  cfg.blockDim = dim3(kAtThreads);
  cfg.dynamicSmemBytes = L::kBytes;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = g_pdl_enabled ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, prefill_attn_tc_kernel<D>, mq, mk, mv, p);
  if (e != cudaSuccess) throw std::runtime_error(std::string("prefill attention (tcgen05) launch: ") + cudaGetErrorString(e));
  return 0;
}

// tile arrays: 128 query rows per tile. page_size must be 32, 64 or 128. Returns 1 for an unsupported head_dim / page size.
int launch_prefill_attention_tc(const void* q, long long q_stride, long long T, const void* kc, const void* vc, long long num_pages, const int* bt,
                                int bt_stride, const int* q_start, const int* q_len, const int* ctx, const int* tile_seq, const int* tile_q0,
                                int num_tiles, void* out, int H, int KV, int D, int page, float scale, float cap, int window, int causal, int* status,
                                cudaStream_t st) {
  if (num_tiles == 0) return 0;
  if (page != 32 && page != 64 && page != 128) return 1;
  AttnTcParams p = {};
  p.block_tables = bt;
  p.bt_stride = bt_stride;
  p.q_start = q_start;
  p.q_len = q_len;
  p.ctx_lens = ctx;
  p.tile_seq = tile_seq;
  p.tile_q0 = tile_q0;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.H = H;
  p.KV = KV;
  p.page_size = page;
  p.scale = scale;
  p.softcap = cap;
  p.window = window;
  p.causal = causal;
  p.status = status;
  const long long cache_rows = num_pages * KV * page;
  switch (D) {
    case 64: return launch_prefill_tc_t<64>(q, q_stride, T, kc, vc, cache_rows, p, num_tiles, st);
    case 128: return launch_prefill_tc_t<128>(q, q_stride, T, kc, vc, cache_rows, p, num_tiles, st);
    case 256: return launch_prefill_tc_t<256>(q, q_stride, T, kc, vc, cache_rows, p, num_tiles, st);
    default: return 1;
  }
}

}  // namespace dlv
