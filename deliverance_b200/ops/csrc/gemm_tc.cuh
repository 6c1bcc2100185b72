// tcgen05 / TMEM GEMM for  out[m, n] = sum_k X[m, k] * W[n, k]  (+ bias[n]).
//
// The weight matrix is the MMA "A" operand (128 weight rows per CTA = UMMA M), the activations are the "B" operand
// (BN tokens = UMMA N, 16..256), so that decode batches of 1..64 tokens still fill a full-height tensor-core tile and
// the kernel is weight-bandwidth bound. W is either dense bf16 (TMA straight into 128B-swizzled tiles) or JQ4:
// packed nibbles + per-32 fp32 scales arrive by TMA in a staging buffer, eight warps expand them into the swizzled
// bf16 tile in shared memory ((nibble - 8) * scale), and a single elected thread issues tcgen05.mma with the
// accumulator in TMEM. Split-K partials are reduced by the last CTA to arrive at a tile (fixed order, deterministic).
//
// Roles per CTA (320 threads): warp 0 = TMA producer, warp 1 = TMEM owner + MMA issuer, warps 2..9 = JQ4 dequant and
// epilogue (tcgen05.ld -> convert -> global).
//
// This replaces the reference's CPU kernels gemm_q8_q4 / gemm_bf16_q4 / gemm_bf16
// (native/src/main/c/simd/vector_simd.c:339-633,1186-1411,1414-1668) and the WGSL gemm_q4 / gemm_i8q4_v5 shaders.
#pragma once
#include "common.cuh"

namespace dlv {

constexpr int kGemmBM = 128;       // weight rows per CTA
constexpr int kGemmBK = 128;       // reduction elements per pipeline stage (two 64-wide swizzle atoms)
constexpr int kGemmThreads = 320;  // 10 warps
constexpr int kGemmEpiThreads = 256;

struct GemmParams {
  int M, N, K;
  int kb_total;      // ceil(K / 128)
  int splits;        // split-K factor (>= 1)
  int kb_per_split;  // k-blocks handled by one split
  int n_tiles, m_tiles;
  void* out;         // [M, ldo] bf16 or fp32
  int ldo;
  int out_f32;
  const float* bias;  // [N] fp32 or nullptr
  float* ws;          // split-K partials: [tile][split][BN][128] fp32
  int* counters;      // one per tile, zero between launches (the reducing CTA resets its counter)
  int* status;        // kernel status word (0 = ok)
};

template <bool Q4, int BN>
struct GemmSmem {
  static constexpr int kWTile = kGemmBM * 128;        // one 64-wide bf16 sub-tile of W: 16 KB
  static constexpr int kXTile = BN * 128;             // one 64-wide bf16 sub-tile of X
  static constexpr int kRaw = Q4 ? kGemmBM * 64 : 0;  // packed nibbles for 128 k
  static constexpr int kScales = Q4 ? kGemmBM * 16 : 0;
  static constexpr int kStage = 2 * kWTile + 2 * kXTile + kRaw + kScales;
  static constexpr int kMaxSmem = 232448 - 2048;
  static constexpr int kStages = (kMaxSmem / kStage) > 8 ? 8 : (kMaxSmem / kStage);
  static constexpr int kBytes = kStages * kStage + 2048;  // + barriers and 1024 B alignment slack
  static constexpr uint32_t kTxBytes = Q4 ? (kRaw + kScales + 2 * kXTile) : (2 * kWTile + 2 * kXTile);
};

__device__ __forceinline__ uint32_t q4_pair_to_bf162(uint32_t nib4, uint32_t sel, __nv_bfloat162 s2) {
  // bytes of nib4 are nibbles (0..15); build two bf16 values 128 + q, subtract 136 exactly, scale.
  uint32_t u = __byte_perm(nib4, 0x43434343u, sel);
  __nv_bfloat162 v = *reinterpret_cast<__nv_bfloat162*>(&u);
  const __nv_bfloat162 off = __floats2bfloat162_rn(136.f, 136.f);
  v = __hmul2(__hsub2(v, off), s2);
  return *reinterpret_cast<uint32_t*>(&v);
}

template <bool Q4, int BN>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_w,   // Q4: packed bytes [N, K/2]; dense: bf16 [N, K]
               const __grid_constant__ CUtensorMap map_s,   // Q4: scales f32 [N, K/32]; dense: unused
               const __grid_constant__ CUtensorMap map_x,   // bf16 [M, K]
               const GemmParams p) {
  using L = GemmSmem<Q4, BN>;
  constexpr int STAGES = L::kStages;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* ctrl = smem + STAGES * L::kStage;
  uint64_t* bar_full = reinterpret_cast<uint64_t*>(ctrl);
  uint64_t* bar_empty = bar_full + STAGES;
  uint64_t* bar_deq = bar_empty + STAGES;
  uint64_t* bar_acc = bar_deq + STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_acc + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* s_last = const_cast<int*>(abort_flag) + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_tile = blockIdx.x, m_tile = blockIdx.y, split = blockIdx.z;
  const int n0 = n_tile * kGemmBM, m0 = m_tile * BN;
  const int kb_begin = split * p.kb_per_split;
  const int kb_end = min(p.kb_total, kb_begin + p.kb_per_split);
  const int nkb = max(0, kb_end - kb_begin);
  constexpr uint32_t TMEM_COLS = BN < 32 ? 32 : BN;

  auto stage_w = [&](int s, int sub) { return smem + s * L::kStage + sub * L::kWTile; };
  auto stage_x = [&](int s, int sub) { return smem + s * L::kStage + 2 * L::kWTile + sub * L::kXTile; };
  auto stage_raw = [&](int s) { return smem + s * L::kStage + 2 * L::kWTile + 2 * L::kXTile; };
  auto stage_sc = [&](int s) { return smem + s * L::kStage + 2 * L::kWTile + 2 * L::kXTile + L::kRaw; };

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&bar_full[s]), 1);
      mbar_init(smem_u32(&bar_empty[s]), 1);
      mbar_init(smem_u32(&bar_deq[s]), kGemmEpiThreads);
    }
    mbar_init(smem_u32(bar_acc), 1);
    *abort_flag = 0;
    *s_last = 0;
    mbar_fence_init();
    tma_prefetch_desc(&map_w);
    tma_prefetch_desc(&map_x);
    if (Q4) tma_prefetch_desc(&map_s);
  }
  if (warp == 1) tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      int issued = 0;
      for (int i = 0; i < nkb; ++i) {
        const int s = i % STAGES;
        const uint32_t ph = (i / STAGES) & 1;
        if (!mbar_wait(smem_u32(&bar_empty[s]), ph ^ 1, abort_flag, p.status)) break;
        const uint32_t full = smem_u32(&bar_full[s]);
        mbar_expect_tx(full, L::kTxBytes);
        const int kb = kb_begin + i;
        if (Q4) {
          tma_load_2d(smem_u32(stage_raw(s)), &map_w, full, kb * 64, n0);
          tma_load_2d(smem_u32(stage_sc(s)), &map_s, full, kb * 4, n0);
        } else {
          tma_load_2d(smem_u32(stage_w(s, 0)), &map_w, full, kb * kGemmBK, n0);
          tma_load_2d(smem_u32(stage_w(s, 1)), &map_w, full, kb * kGemmBK + 64, n0);
        }
        tma_load_2d(smem_u32(stage_x(s, 0)), &map_x, full, kb * kGemmBK, m0);
        tma_load_2d(smem_u32(stage_x(s, 1)), &map_x, full, kb * kGemmBK + 64, m0);
        ++issued;
      }
      if (*abort_flag) {
        // let copies that are still in flight land before the CTA goes away (bounded: ~50 ms per stage)
        const int first = issued > STAGES ? issued - STAGES : 0;
        for (int i = first; i < issued; ++i) {
          const uint32_t bar = smem_u32(&bar_full[i % STAGES]);
          const uint32_t ph = (i / STAGES) & 1;
          const unsigned long long t0 = globaltimer_ns();
          while (!mbar_try_wait(bar, ph) && globaltimer_ns() - t0 < 50000000ull) {
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_bf16(kGemmBM, BN);
      bool ok = true;
      for (int i = 0; i < nkb && ok; ++i) {
        const int s = i % STAGES;
        const uint32_t ph = (i / STAGES) & 1;
        if (Q4) ok = mbar_wait(smem_u32(&bar_deq[s]), ph, abort_flag, p.status);
        ok = ok && mbar_wait(smem_u32(&bar_full[s]), ph, abort_flag, p.status);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int k4 = 0; k4 < 8; ++k4) {
          const int sub = k4 >> 2, kk = k4 & 3;
          const uint64_t da = umma_desc_k_sw128(smem_u32(stage_w(s, sub)) + kk * 32);
          const uint64_t db = umma_desc_k_sw128(smem_u32(stage_x(s, sub)) + kk * 32);
          umma_bf16(tmem_base, da, db, idesc, (i > 0 || k4 > 0) ? 1u : 0u);
        }
        umma_commit(smem_u32(&bar_empty[s]));
      }
      umma_commit(smem_u32(bar_acc));
      if (!ok) {
        // outstanding MMAs must retire before TMEM is released
        const unsigned long long t0 = globaltimer_ns();
        while (!mbar_try_wait(smem_u32(bar_acc), 0) && globaltimer_ns() - t0 < 50000000ull) {
        }
      }
    }
  } else {
    // ---------------- dequant + epilogue warps (256 threads) ----------------
    const int t = threadIdx.x - 64;
    bool ok = true;
    if (Q4) {
      const int r = t & 127, h = t >> 7;
      for (int i = 0; i < nkb; ++i) {
        const int s = i % STAGES;
        const uint32_t ph = (i / STAGES) & 1;
        if (!mbar_wait(smem_u32(&bar_full[s]), ph, abort_flag, p.status)) { ok = false; break; }
        const uint8_t* raw = stage_raw(s) + r * 64;
        const float4 sc4 = *reinterpret_cast<const float4*>(stage_sc(s) + r * 16);
        const float sc[4] = {sc4.x, sc4.y, sc4.z, sc4.w};
        uint8_t* wrow = stage_w(s, h) + r * 128;
#pragma unroll
        for (int b = 0; b < 2; ++b) {
          const int blk = 2 * h + b;
          const uint4 w = *reinterpret_cast<const uint4*>(raw + ((blk ^ ((r >> 1) & 3)) << 4));
          const __nv_bfloat162 s2 = __float2bfloat162_rn(sc[blk]);
          const uint32_t words[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
          for (int hl = 0; hl < 2; ++hl) {
#pragma unroll
            for (int wp = 0; wp < 2; ++wp) {
              const uint32_t a = (words[2 * wp] >> (4 * hl)) & 0x0F0F0F0Fu;
              const uint32_t c = (words[2 * wp + 1] >> (4 * hl)) & 0x0F0F0F0Fu;
              uint4 o;
              o.x = q4_pair_to_bf162(a, 0x4140u, s2);
              o.y = q4_pair_to_bf162(a, 0x4342u, s2);
              o.z = q4_pair_to_bf162(c, 0x4140u, s2);
              o.w = q4_pair_to_bf162(c, 0x4342u, s2);
              const int chunk = 4 * b + 2 * hl + wp;
              *reinterpret_cast<uint4*>(wrow + ((chunk ^ (r & 7)) << 4)) = o;
            }
          }
        }
        fence_proxy_async_smem();
        mbar_arrive(smem_u32(&bar_deq[s]));
      }
    }
    // ---- epilogue ----
    if (ok) ok = mbar_wait(smem_u32(bar_acc), 0, abort_flag, p.status);
    // All 256 threads reach this barrier; afterwards the abort flag gives a CTA-uniform decision (it is only ever
    // raised before the accumulator barrier can complete), so the named barriers below never miss a thread.
    asm volatile("bar.sync 1, 256;" ::: "memory");
    ok = (*abort_flag == 0);
    if (ok) {
      tc_fence_after();
      const int we = warp - 2;
      const int q = warp & 3;            // TMEM lane quarter this warp may read
      const int half = we >> 2;          // column half
      const int row = q * 32 + lane;
      const int n = n0 + row;
      constexpr int COLS = BN / 2;
      constexpr int CH = COLS >= 16 ? 16 : 8;
      const uint32_t taddr0 = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + half * COLS;
      const int tile_id = m_tile * p.n_tiles + n_tile;
      if (p.splits == 1) {
        const float bias = (p.bias != nullptr && n < p.N) ? p.bias[n] : 0.f;
#pragma unroll 1
        for (int c0 = 0; c0 < COLS; c0 += CH) {
          uint32_t v[CH];
          if constexpr (CH == 16) tmem_ld_x16(taddr0 + c0, v); else tmem_ld_x8(taddr0 + c0, v);
          tmem_ld_wait();
          if (n < p.N) {
#pragma unroll
            for (int j = 0; j < CH; ++j) {
              const int m = m0 + half * COLS + c0 + j;
              if (m < p.M) {
                const float acc = (nkb > 0 ? __uint_as_float(v[j]) : 0.f) + bias;
                if (p.out_f32) reinterpret_cast<float*>(p.out)[static_cast<size_t>(m) * p.ldo + n] = acc;
                else reinterpret_cast<__nv_bfloat16*>(p.out)[static_cast<size_t>(m) * p.ldo + n] = f2bf(acc);
              }
            }
          }
        }
      } else {
        float* part = p.ws + (static_cast<size_t>(tile_id) * p.splits + split) * (BN * kGemmBM);
#pragma unroll 1
        for (int c0 = 0; c0 < COLS; c0 += CH) {
          uint32_t v[CH];
          if constexpr (CH == 16) tmem_ld_x16(taddr0 + c0, v); else tmem_ld_x8(taddr0 + c0, v);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < CH; ++j)
            part[(half * COLS + c0 + j) * kGemmBM + row] = nkb > 0 ? __uint_as_float(v[j]) : 0.f;
        }
        __threadfence();
        asm volatile("bar.sync 1, 256;" ::: "memory");
        if (t == 0) {
          const int old = atomicAdd(&p.counters[tile_id], 1);
          *s_last = (old == p.splits - 1) ? 1 : 0;
        }
        asm volatile("bar.sync 1, 256;" ::: "memory");
        if (*s_last) {
          __threadfence();
          const float bias = (p.bias != nullptr && n < p.N) ? p.bias[n] : 0.f;
          const float* base = p.ws + static_cast<size_t>(tile_id) * p.splits * (BN * kGemmBM);
          for (int c = 0; c < COLS; ++c) {
            const int col = half * COLS + c;
            const int m = m0 + col;
            if (m >= p.M) break;
            float acc = 0.f;
            for (int sp = 0; sp < p.splits; ++sp)
              acc += __ldcg(base + (static_cast<size_t>(sp) * BN + col) * kGemmBM + row);
            acc += bias;
            if (n < p.N) {
              if (p.out_f32) reinterpret_cast<float*>(p.out)[static_cast<size_t>(m) * p.ldo + n] = acc;
              else reinterpret_cast<__nv_bfloat16*>(p.out)[static_cast<size_t>(m) * p.ldo + n] = f2bf(acc);
            }
          }
          if (t == 0) p.counters[tile_id] = 0;
        }
      }
    }
  }
  // ---------------- teardown ----------------
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

}  // namespace dlv
