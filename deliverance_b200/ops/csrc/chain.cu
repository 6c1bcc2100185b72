// Persistent decode chain: several JQ4 projections of a decoder layer and the tile-wise work between them in ONE launch.
//
// At decode sizes (1..64 tokens) a projection streams a few MB of weights, which takes a few microseconds, while a stand-alone
// GEMM launch pays about as much again for its prologue (barrier set-up, tensor-memory allocation), its epilogue (split-K
// reduction, store) and the gap to the next kernel, and a grid of whole tiles rarely matches 148 SMs. This kernel runs one CTA
// per SM for a whole chain
//     o_proj -> (+residual, norm) -> gate|up -> act(gate) * up -> down -> (+residual, norm) -> q|k|v -> (q/k norm, rotary, KV write)
// as a dataflow over weight tiles, without any grid-wide barrier:
//   * stream-K: the (weight tile, k-block) units of a projection are dealt out evenly, CTA c takes units [c U / P, (c + 1) U / P)
//     in tile-major order, which is ONE contiguous byte range of the tile-packed weight, whatever the shape. A CTA accumulates each
//     run of units that belong to one tile (a segment) in tensor memory, writes it as an fp32 partial tile to a workspace slot and
//     counts it in (release-add on the tile's counter, nobody waits for the result);
//   * when a CTA has delivered all its segments of a projection it helps to finish the tiles it contributed to: the holders of a
//     tile's segments share the tile's token rows, wait (bounded) until every segment of the tile is counted in, sum the partial tiles
//     of their rows in slot order (deterministic) and apply what follows the projection to the tile's 128 columns: bias, residual
//     add, activation, per-head norm / rotary embedding / KV-cache write. Then they count themselves in on the projection's "finished"
//     counter; nobody waits inside a tile for anything but that tile's own segments;
//   * the activation producers of the NEXT projection wait for that one counter (a single flag, one round trip), the weight producers
//     never wait for anything but ring space, so up to 160 KB of weights per SM are already on chip when the rows arrive;
//   * RMSNorm needs a whole row, which would be a barrier. It is split instead: the tile stage writes residual * norm_weight and the
//     tile's share of the row's sum of squares; the per-row factor rsqrt(mean(r^2) + eps) commutes with the next projection and is
//     applied by that projection's tile stage, by which time every share exists.
// The GEMM engine is the one of gemm_tc.cuh: packed JQ4 stages by bulk copy into a deep ring, 16 warps expand them to bf16 straight
// into tensor memory (the MMA A operand), activations by TMA into 128B-swizzled tiles (B operand), four MMA-issuing warps with one
// accumulator each. Every wait is bounded; when one runs out the CTA sets the status word, lets its copies land, frees tensor memory
// and returns.
//
// Status: numerically equal to the separate kernels (tests/test_gpu_kernels.py::test_decode_chain_matches_separate_kernels) but not
// faster yet, so the models do not use it. Measured on one B200, Qwen3-4B layer shapes, weights past L2
// (python -m deliverance_b200.bench.chain_bench): 64 / 69 / 84 us per layer at 1 / 8 / 64 tokens against 47 / 49 / 62 us for the
// separate launches. Every hand-over between stages is a chain of dependent L2 round trips (partial tiles -> counter -> finishing
// loads -> counter -> activation loads, about 5 us on this part, four times per layer) and a segment boundary drains the MMA pipe;
// together they cost more than the launches they save, whose prologues programmatic dependent launch already hides.
//
// Replaces, for decode batches, the sequence of separate launches behind the reference's per-projection calls
// (core/.../generator/CausalSelfAttention.java:226-420, MLPBlock.java:197-329, TransformerBlock.java:161-200).
#include <stdexcept>
#include <string>

#include "gemm_tc.cuh"
#include "chain_api.h"
#include "gemm_api.h"

namespace dlv {

struct ChainOpDev {
  const uint8_t* wq;   // tile-packed JQ4 weight
  float* ws;           // partial tiles [n_tiles][smax][BN][128] fp32
  float* ssq;          // kChainRowAddNorm: the tiles' shares of the rows' sums of squares [n_tiles][64]
  int N, K, n_tiles, kbt, smax, kind;
  int dep;             // 1: the input rows are the output of the projection in front (wait for its tile flags), 0: external input
  int scale_src;       // index of the add + norm stage whose per-row factor scales this projection's output, or -1
  int off_cnt, off_done, fin_total;  // word offsets into `sync`: segment counters [n_tiles], finishers counted in [1]; its final value
  const float* bias;
  __nv_bfloat16* residual;
  const __nv_bfloat16* norm_w;
  __nv_bfloat16* out;
  float eps, offset, res_mult;
  int act;
};

struct ChainParams {
  CUtensorMap maps[kChainMaxOps];  // activations of every projection, [rows][K] bf16 seen as k-chunks (one box = one stage)
  ChainOpDev op[kChainMaxOps];
  ChainQkvArgs qkv;
  int n_ops, M, sync_words;
  unsigned* sync;  // [0] CTAs that left, then per projection the counters described in ChainOpDev; all zero between launches
  int* status;
};
static_assert(sizeof(ChainParams) <= 4000, "kernel parameter space");

// The CTA that owns unit x of a projection with U units on P CTAs (CTA c starts at floor(c U / P)): the largest c with start(c) <= x.
__host__ __device__ __forceinline__ int chain_cta_of_unit(long long x, long long U, int P) {
  return static_cast<int>(((x + 1) * P + U - 1) / U) - 1;
}
// Partial tiles (segments) of weight tile t. With more units than CTAs every CTA has work and the CTAs of a tile are consecutive:
// one segment per CTA from the owner of the tile's first unit to the owner of its last. With at most one unit per CTA (U <= P, some
// CTAs idle) every k-block is a segment of its own.
__host__ __device__ __forceinline__ int chain_nseg(int t, int kbt, long long U, int P) {
  if (U <= P) return kbt;
  return chain_cta_of_unit(static_cast<long long>(t + 1) * kbt - 1, U, P) - chain_cta_of_unit(static_cast<long long>(t) * kbt, U, P) + 1;
}
// Workspace slot of the segment of tile t that CTA c computes and that starts at k-block kb0.
__device__ __forceinline__ int chain_slot(int c, int t, int kb0, int kbt, long long U, int P) {
  if (U <= P) return kb0;
  return c - chain_cta_of_unit(static_cast<long long>(t) * kbt, U, P);
}

__device__ __forceinline__ float chain_act(float g, int act) {
  switch (act) {
    case 0: return g / (1.f + __expf(-g));
    case 1: return 0.5f * g * (1.f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g)));
    case 2: return 0.5f * g * (1.f + erff(g * 0.7071067811865475f));
    case 3: return fmaxf(g, 0.f);
    default: return tanhf(g);
  }
}
__device__ __forceinline__ float bf16_round(float v) { return bf2f(f2bf(v)); }
__device__ __forceinline__ void st_release_gpu(uint32_t* p, uint32_t v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Sum over the segments of (tile, row m, columns 4 lane .. 4 lane + 3) in slot order.
__device__ __forceinline__ float4 chain_tile_sum4(const ChainOpDev& o, int BN, int tile, int ns, int m, int lane) {
  const float* b = o.ws + ((static_cast<size_t>(tile) * o.smax) * BN + m) * 128 + lane * 4;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
  for (int j = 0; j < ns; ++j) {
    const float4 v = __ldcg(reinterpret_cast<const float4*>(b + static_cast<size_t>(j) * BN * 128));
    acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
  }
  return acc;
}

template <int BN>
__global__ void __launch_bounds__(kGemmThreads, 1) decode_chain_kernel(const __grid_constant__ ChainParams p) {
  using L = GemmSmem<true, BN>;
  constexpr int NX = L::kNX, NR = L::kNR, NA = L::kNA, NI = L::kNI;
  static_assert(NI == 4 && NA == 4, "the chain kernel is written for token tiles of at most 64 rows (four issuers, four A stages)");
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* ctrl = smem + L::kOffCtrl;
  uint64_t* bar_a_full = reinterpret_cast<uint64_t*>(ctrl);
  uint64_t* bar_a_empty = bar_a_full + 8;
  uint64_t* bar_x_full = bar_a_empty + 8;
  uint64_t* bar_x_empty = bar_x_full + NX;
  uint64_t* bar_r_full = bar_x_empty + NX;
  uint64_t* bar_r_empty = bar_r_full + NR;
  uint64_t* bar_acc_full = bar_r_empty + NR;
  uint64_t* bar_acc_empty = bar_acc_full + 1;
  uint64_t* bar_drain = bar_acc_empty + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_drain + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* s_flag = const_cast<int*>(abort_flag) + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int P = gridDim.x, c = blockIdx.x;
  auto x_tile = [&](int s) { return smem + L::kOffX + s * L::kXStage; };
  auto raw_tile = [&](int s) { return smem + L::kOffRaw + s * L::kRawStage; };
  auto sc_tile = [&](int s) { return smem + L::kOffRaw + s * L::kRawStage + kGemmBM * 64; };
  auto unit_range = [&](const ChainOpDev& o, long long& u0, long long& u1) {
    const long long U = static_cast<long long>(o.n_tiles) * o.kbt;
    u0 = (static_cast<long long>(c) * U) / P;
    u1 = (static_cast<long long>(c + 1) * U) / P;
  };

  if (threadIdx.x == 0) {
    for (int s = 0; s < 2 * NA; ++s) {  // every A stage is handed over in two halves of 64 k (see the dequant loop)
      mbar_init(smem_u32(&bar_a_full[s]), 4);
      mbar_init(smem_u32(&bar_a_empty[s]), 1);
    }
    for (int s = 0; s < NX; ++s) {
      mbar_init(smem_u32(&bar_x_full[s]), 1);
      mbar_init(smem_u32(&bar_x_empty[s]), 1);
    }
    for (int s = 0; s < NR; ++s) {
      mbar_init(smem_u32(&bar_r_full[s]), 1);
      mbar_init(smem_u32(&bar_r_empty[s]), 4);
    }
    mbar_init(smem_u32(bar_acc_full), NI);
    mbar_init(smem_u32(bar_acc_empty), 1);
    mbar_init(smem_u32(bar_drain), 1);
    *abort_flag = 0;
    *s_flag = 0;
    mbar_fence_init();
    for (int g = 0; g < p.n_ops; ++g) tma_prefetch_desc(&p.maps[g]);
  }
  pdl_trigger();
  if (warp == 1) tmem_alloc(smem_u32(tmem_slot), kGemmTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0 || warp == 19) {
    // ---------------- weight producers: one 10 KB bulk copy per unit, never waiting for anything but ring space ----------------
    if (lane == 0) {
      const int mine = warp == 0 ? 0 : 1;
      int i = 0, last_issued = -1, n_issued = 0;
      bool ok = true;
      for (int g = 0; g < p.n_ops && ok; ++g) {
        const ChainOpDev& o = p.op[g];
        long long u0, u1;
        unit_range(o, u0, u1);
        for (long long u = u0; u < u1; ++u, ++i) {
          if ((i & 1) != mine) continue;
          const int s = i % NR;
          if (!mbar_wait(smem_u32(&bar_r_empty[s]), ((i / NR) & 1) ^ 1, abort_flag, p.status)) { ok = false; break; }
          const uint32_t full = smem_u32(&bar_r_full[s]);
          mbar_expect_tx(full, L::kRawStage);
          bulk_load_1d(smem_u32(raw_tile(s)), o.wq + static_cast<size_t>(u) * kQ4StageBytes, L::kRawStage, full);
          last_issued = i;
          ++n_issued;
        }
      }
      if (*abort_flag) {
        const int keep = n_issued < NR / 2 ? n_issued : NR / 2;
        for (int j = 0; j < keep; ++j) {
          const int ii = last_issued - 2 * j;
          const unsigned long long t0 = globaltimer_ns();
          while (!mbar_try_wait(smem_u32(&bar_r_full[ii % NR]), (ii / NR) & 1) && globaltimer_ns() - t0 < 20000000ull) {
          }
        }
      }
    }
  } else if (warp == 2 || warp == 20) {
    // ---------------- activation producers: wait until the stage in front is finished, then one TMA box per unit ----------------
    if (lane == 0) {
      const int mine = warp == 2 ? 0 : 1;
      int i = 0, last_issued = -1, n_issued = 0;
      bool ok = true;
      pdl_wait();  // the first projection reads what the kernel in front of this one wrote
      for (int g = 0; g < p.n_ops && ok; ++g) {
        const ChainOpDev& o = p.op[g];
        long long u0, u1;
        unit_range(o, u0, u1);
        if (o.dep && u1 > u0) {
          // every tile of the stage in front has been finished (rows written by other SMs with ordinary stores are read by TMA below)
          if (!flag_wait_ge(p.sync + p.op[g - 1].off_done, static_cast<uint32_t>(p.op[g - 1].fin_total), p.status)) {
            *abort_flag = 1;
            break;
          }
          fence_proxy_async_all();
        }
        for (long long u = u0; u < u1; ++u, ++i) {
          if ((i & 1) != mine) continue;
          const int kb = static_cast<int>(u % o.kbt);
          const int s = i % NX;
          if (!mbar_wait(smem_u32(&bar_x_empty[s]), ((i / NX) & 1) ^ 1, abort_flag, p.status)) { ok = false; break; }
          const uint32_t full = smem_u32(&bar_x_full[s]);
          mbar_expect_tx(full, L::kXStage);
          tma_load_3d(smem_u32(x_tile(s)), &p.maps[g], full, 0, 0, kb * 2);
          last_issued = i;
          ++n_issued;
        }
      }
      if (*abort_flag) {
        const int keep = n_issued < NX / 2 ? n_issued : NX / 2;
        for (int j = 0; j < keep; ++j) {
          const int ii = last_issued - 2 * j;
          const unsigned long long t0 = globaltimer_ns();
          while (!mbar_try_wait(smem_u32(&bar_x_full[ii % NX]), (ii / NX) & 1) && globaltimer_ns() - t0 < 20000000ull) {
          }
        }
      }
    }
  } else if (warp == 1 || warp >= 21) {
    // ---------------- MMA issuers: unit i goes to issuer i % 4 and accumulator i % 4 ----------------
    const int issuer = warp == 1 ? 0 : warp - 20;
    constexpr uint32_t idesc = umma_idesc_bf16(kGemmBM, BN);
    const uint64_t desc_x0 = umma_desc_k_sw128(smem_u32(smem + L::kOffX));
    const uint32_t tmem_acc = tmem_base + issuer * BN;
    int i = 0, segn = 0;
    bool ok = true, started = false;
    for (int g = 0; g < p.n_ops && ok; ++g) {
      const ChainOpDev& o = p.op[g];
      long long u0, u1;
      unit_range(o, u0, u1);
      int kb = static_cast<int>(u0 % o.kbt);
      for (long long u = u0; u < u1 && ok; ++u, ++i) {
        if (u == u0 || kb == 0) {
          // a new segment: the epilogue must have drained the accumulators of the one before
          started = false;
          if (segn > 0) {
            ok = mbar_wait(smem_u32(bar_acc_empty), (segn - 1) & 1, abort_flag, p.status);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
          }
        }
        if ((i & 3) == issuer) {
          const int sa = i & 3, sx = i % NX;
          ok = mbar_wait(smem_u32(&bar_x_full[sx]), (i / NX) & 1, abort_flag, p.status);
          const uint64_t dx = desc_x0 + static_cast<uint64_t>((sx * L::kXStage) >> 4);
#pragma unroll
          for (int hf = 0; hf < 2 && ok; ++hf) {
            // the two 64-k halves of the stage arrive separately: the MMAs of the first half run while the second is being expanded
            ok = mbar_wait(smem_u32(&bar_a_full[2 * sa + hf]), (i / NA) & 1, abort_flag, p.status);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            if (lane == 0) {
#pragma unroll
              for (int kk = 0; kk < 4; ++kk) {
                const int k4 = hf * 4 + kk;
                const uint64_t db = dx + static_cast<uint64_t>((hf * (BN * 128) + kk * 32) >> 4);
                umma_bf16_ts(tmem_acc, tmem_base + L::kTmemA + sa * kGemmTmemAStage + k4 * 8, db, idesc, (started || k4 > 0) ? 1u : 0u);
              }
              umma_commit(smem_u32(&bar_a_empty[2 * sa + hf]));
              if (hf == 1) umma_commit(smem_u32(&bar_x_empty[sx]));
            }
            __syncwarp();
          }
          if (!ok) break;
          started = true;
        }
        if (u == u1 - 1 || kb == o.kbt - 1) {
          if (lane == 0) {
            if (started) umma_commit(smem_u32(bar_acc_full));  // arrives when this issuer's MMAs of the segment have retired
            else mbar_arrive(smem_u32(bar_acc_full));
          }
          ++segn;
          __syncwarp();
        }
        kb = kb + 1 == o.kbt ? 0 : kb + 1;
      }
    }
    if (!ok && lane == 0) {
      // outstanding MMAs must retire before tensor memory is released
      umma_commit(smem_u32(bar_drain));
      const unsigned long long t0 = globaltimer_ns();
      while (!mbar_try_wait(smem_u32(bar_drain), 0) && globaltimer_ns() - t0 < 20000000ull) {
      }
    }
    __syncwarp();
  } else if (warp >= kGemmEpiWarp0 && warp < kGemmEpiWarp0 + 16) {
    // ---------------- dequant + segment epilogue + tile stage (512 threads) ----------------
    const int t = threadIdx.x - kGemmEpiWarp0 * 32;
    const int we = warp - kGemmEpiWarp0;
    const int q = warp & 3;     // tensor-memory lane quarter of this warp
    const int grp4 = we >> 2;   // dequant group = A stage = unit index mod 4; also the column group of the epilogue
    const int r = q * 32 + lane;
    int i = 0, segn = 0;
    bool ok = true;
    pdl_wait();
    for (int g = 0; g < p.n_ops && ok; ++g) {
      const ChainOpDev& o = p.op[g];
      long long u0, u1;
      unit_range(o, u0, u1);
      const long long U = static_cast<long long>(o.n_tiles) * o.kbt;
      int seg_i0 = i;
      int kb = static_cast<int>(u0 % o.kbt), tile = static_cast<int>(u0 / o.kbt);
      for (long long u = u0; u < u1 && ok; ++u, ++i) {
        if (u == u0 || kb == 0) seg_i0 = i;
        if ((i & 3) == grp4) {
          const int sr = i % NR, sa = i & 3;
          if (!mbar_wait(smem_u32(&bar_r_full[sr]), (i / NR) & 1, abort_flag, p.status)) { ok = false; break; }
          uint4 wq[4];
#pragma unroll
          for (int b = 0; b < 4; ++b) wq[b] = *reinterpret_cast<const uint4*>(raw_tile(sr) + r * 64 + ((b ^ ((r >> 1) & 3)) << 4));
          const float4 sc4 = *reinterpret_cast<const float4*>(sc_tile(sr) + r * 16);
          const float sc[4] = {sc4.x, sc4.y, sc4.z, sc4.w};
          const uint32_t tdst = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + L::kTmemA + sa * kGemmTmemAStage;
#pragma unroll
          for (int b = 0; b < 4; ++b) {
            if ((b & 1) == 0) {  // a half stage (64 k) is free once the MMAs that read it for unit i - 4 have retired
              if (!mbar_wait(smem_u32(&bar_a_empty[2 * sa + (b >> 1)]), ((i / NA) & 1) ^ 1, abort_flag, p.status)) { ok = false; break; }
              tc_fence_after();
            }
            const __nv_bfloat162 s2 = __float2bfloat162_rn(sc[b]);
            const uint32_t words[4] = {wq[b].x, wq[b].y, wq[b].z, wq[b].w};
            uint32_t ov[16];
#pragma unroll
            for (int hl = 0; hl < 2; ++hl) {
#pragma unroll
              for (int wd = 0; wd < 4; ++wd) {
                const uint32_t a = (words[wd] >> (4 * hl)) & 0x0F0F0F0Fu;
                ov[hl * 8 + wd * 2 + 0] = q4_pair_to_bf162(a, 0x4140u, s2);
                ov[hl * 8 + wd * 2 + 1] = q4_pair_to_bf162(a, 0x4342u, s2);
              }
            }
            tmem_st_x16(tdst + b * 16, ov);
            if (b & 1) {
              tmem_st_wait();
              tc_fence_before();
              __syncwarp();
              if (lane == 0) {
                if (b == 3) mbar_arrive(smem_u32(&bar_r_empty[sr]));
                mbar_arrive(smem_u32(&bar_a_full[2 * sa + (b >> 1)]));
              }
            }
          }
          if (!ok) break;
        }
        if (u == u1 - 1 || kb == o.kbt - 1) {
          // ---- segment epilogue: accumulators -> fp32 partial tile in the workspace slot of (tile, this segment) ----
          const int len = i + 1 - seg_i0;
          if (!mbar_wait(smem_u32(bar_acc_full), segn & 1, abort_flag, p.status)) { ok = false; break; }
          tc_fence_after();
          constexpr int GROUPS = BN >= 32 ? 4 : BN / 8;
          constexpr int COLS = BN / GROUPS;
          if (grp4 < GROUPS) {
            const int slot = chain_slot(c, tile, kb + 1 - len, o.kbt, U, P);
            float* dst = o.ws + ((static_cast<size_t>(tile) * o.smax + slot) * BN) * 128 + r;
            const uint32_t taddr0 = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + grp4 * COLS;
            float sum[COLS];
#pragma unroll
            for (int j = 0; j < COLS; ++j) sum[j] = 0.f;
            const int nacc = len < NI ? len : NI;
            for (int a = 0; a < nacc; ++a) {
              const int acc = (seg_i0 + a) & 3;
              uint32_t v[COLS];
              if constexpr (COLS == 16) tmem_ld_x16(taddr0 + acc * BN, v); else tmem_ld_x8(taddr0 + acc * BN, v);
              tmem_ld_wait();
#pragma unroll
              for (int j = 0; j < COLS; ++j) sum[j] += __uint_as_float(v[j]);
            }
#pragma unroll
            for (int j = 0; j < COLS; ++j) {
              const int m = grp4 * COLS + j;
              if (m < p.M) dst[static_cast<size_t>(m) * 128] = sum[j];
            }
          }
          tc_fence_before();
          asm volatile("bar.sync 1, 512;" ::: "memory");
          if (t == 0) {
            mbar_arrive(smem_u32(bar_acc_empty));
            red_release_gpu_add(p.sync + o.off_cnt + tile, 1u);  // cumulative over the stores of all 512 threads (ordered by the barrier)
          }
          ++segn;
        }
        if (kb + 1 == o.kbt) { kb = 0; ++tile; } else ++kb;
      }
      // ---- tile stages. This comes after ALL segments of the projection that this CTA owes have been delivered (a CTA that waited
      // for a tile's other segments before delivering its own next segment would make the tiles finish one after the other). The
      // holders of a tile's segments share its rows: slot s of ns finishes rows [s M / ns, (s + 1) M / ns). gate|up: the holders of
      // the up tile finish the pair. ----
      if (!ok || u1 <= u0) continue;
      const int half = o.n_tiles >> 1;
      const bool pair = o.kind == kChainRowActMul;
      for (int tile = static_cast<int>(u0 / o.kbt); tile <= static_cast<int>((u1 - 1) / o.kbt) && ok; ++tile) {
        if (!pair || tile >= half) {
          const int out_tile = pair ? tile - half : tile;
          const int ns = chain_nseg(tile, o.kbt, U, P);
          const int ns_g = pair ? chain_nseg(out_tile, o.kbt, U, P) : 0;
          const long long first_unit = static_cast<long long>(tile) * o.kbt;
          const int my_slot = chain_slot(c, tile, static_cast<int>((u0 > first_unit ? u0 : first_unit) - first_unit), o.kbt, U, P);
          const int m_lo = (my_slot * p.M) / ns, m_hi = ((my_slot + 1) * p.M) / ns;
          if (t < 32) {
            // three waits side by side: the tile's segments, the gate tile's segments, the norm stage whose row factor applies
            bool got = true;
            if (t == 0) got = flag_wait_ge(p.sync + o.off_cnt + tile, static_cast<uint32_t>(ns), p.status);
            if (t == 1 && pair) got = flag_wait_ge(p.sync + o.off_cnt + out_tile, static_cast<uint32_t>(ns_g), p.status);
            if (t == 2 && o.scale_src >= 0)
              got = flag_wait_ge(p.sync + p.op[o.scale_src].off_done, static_cast<uint32_t>(p.op[o.scale_src].fin_total), p.status);
            got = __all_sync(0xffffffffu, got);
            if (t == 0) *s_flag = got ? 1 : 0;
          }
          asm volatile("bar.sync 1, 512;" ::: "memory");
          if (*s_flag == 0) {
            *abort_flag = 1;
            ok = false;
            break;
          }
          for (int m = m_lo + we; m < m_hi; m += 16) {
            float inv = 1.f;
            if (o.scale_src >= 0) {
              const ChainOpDev& sop = p.op[o.scale_src];
              float a = 0.f;
              for (int tt = lane; tt < sop.n_tiles; tt += 32) a += __ldcg(sop.ssq + tt * 64 + m);
              a = warp_sum(a);
              inv = rsqrtf(a / sop.N + sop.eps);
            }
            const int n = tile * 128 + lane * 4;  // first of this lane's four columns of the projection's output
            float4 y = chain_tile_sum4(o, BN, tile, ns, m, lane);
            y.x *= inv; y.y *= inv; y.z *= inv; y.w *= inv;
            if (o.bias != nullptr && n < o.N) {
              const float4 b = *reinterpret_cast<const float4*>(o.bias + n);
              y.x += b.x; y.y += b.y; y.z += b.z; y.w += b.w;
            }
            // rounded to bf16 like the output of a stand-alone projection would be
            y = make_float4(bf16_round(y.x), bf16_round(y.y), bf16_round(y.z), bf16_round(y.w));
            if (o.kind == kChainRowStore) {
              if (n < o.N) {
                uint2 pk;
                pk.x = pack_bf162(y.x, y.y);
                pk.y = pack_bf162(y.z, y.w);
                *reinterpret_cast<uint2*>(o.out + static_cast<size_t>(m) * o.N + n) = pk;
              }
            } else if (o.kind == kChainRowAddNorm || o.kind == kChainRowAdd) {
              float ss = 0.f;
              if (n < o.N) {
                __nv_bfloat16* rp = o.residual + static_cast<size_t>(m) * o.N + n;
                const uint2 rv = *reinterpret_cast<const uint2*>(rp);
                const float2 r0 = unpack_bf162(rv.x), r1 = unpack_bf162(rv.y);
                uint2 pk;
                pk.x = pack_bf162(r0.x + y.x * o.res_mult, r0.y + y.y * o.res_mult);
                pk.y = pack_bf162(r1.x + y.z * o.res_mult, r1.y + y.w * o.res_mult);
                *reinterpret_cast<uint2*>(rp) = pk;
                if (o.kind == kChainRowAddNorm) {
                  const float2 b0 = unpack_bf162(pk.x), b1 = unpack_bf162(pk.y);  // the norm sees the stored (rounded) residual
                  ss = b0.x * b0.x + b0.y * b0.y + b1.x * b1.x + b1.y * b1.y;
                  const uint2 wv = *reinterpret_cast<const uint2*>(o.norm_w + n);
                  const float2 w0 = unpack_bf162(wv.x), w1 = unpack_bf162(wv.y);
                  uint2 xk;  // residual * norm weight; the row's 1 / rms is applied behind the next projection
                  xk.x = pack_bf162(b0.x * (w0.x + o.offset), b0.y * (w0.y + o.offset));
                  xk.y = pack_bf162(b1.x * (w1.x + o.offset), b1.y * (w1.y + o.offset));
                  *reinterpret_cast<uint2*>(o.out + static_cast<size_t>(m) * o.N + n) = xk;
                }
              }
              if (o.kind == kChainRowAddNorm) {
                ss = warp_sum(ss);
                if (lane == 0) o.ssq[tile * 64 + m] = ss;
              }
            } else if (o.kind == kChainRowActMul) {
              float4 gt = chain_tile_sum4(o, BN, out_tile, ns_g, m, lane);
              gt = make_float4(bf16_round(gt.x * inv), bf16_round(gt.y * inv), bf16_round(gt.z * inv), bf16_round(gt.w * inv));
              const int I = o.N >> 1, nh = out_tile * 128 + lane * 4;
              if (nh < I) {
                uint2 pk;
                pk.x = pack_bf162(chain_act(gt.x, o.act) * y.x, chain_act(gt.y, o.act) * y.y);
                pk.y = pack_bf162(chain_act(gt.z, o.act) * y.z, chain_act(gt.w, o.act) * y.w);
                *reinterpret_cast<uint2*>(o.out + static_cast<size_t>(m) * I + nh) = pk;
              }
            } else {  // kChainRowQkvRope: the tile holds 128 / head_dim whole heads (head_dim 64 or 128)
              const ChainQkvArgs& a = p.qkv;
              const int D = a.head_dim, lph = D >> 2;          // lanes per head
              const int h = (tile * 128 + lane * 4) / D;       // this lane's head
              const int d0 = (lane & (lph - 1)) * 4;           // its first dim inside the head
              const bool is_q = h < a.heads, is_k = !is_q && h < a.heads + a.kv_heads;
              const int kvh = is_q ? 0 : (is_k ? h - a.heads : h - a.heads - a.kv_heads);
              float v[4] = {y.x, y.y, y.z, y.w};
              const __nv_bfloat16* nw = is_q ? a.q_norm_w : (is_k ? a.k_norm_w : nullptr);
              if (a.q_norm_w != nullptr) {  // the reduction runs on all lanes (warp-uniform shuffles); value heads ignore it
                float ss = v[0] * v[0] + v[1] * v[1] + v[2] * v[2] + v[3] * v[3];
                for (int ofs = lph >> 1; ofs > 0; ofs >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, ofs);
                if (nw != nullptr) {
                  const float rinv = rsqrtf(ss / D + a.eps);
#pragma unroll
                  for (int e2 = 0; e2 < 4; ++e2) v[e2] = bf16_round(v[e2] * rinv * (bf2f(nw[d0 + e2]) + a.norm_offset));
                }
              }
              if (a.cos_t != nullptr) {
                int pos = a.positions[m];
                pos = pos < 0 ? 0 : (pos >= a.max_pos ? a.max_pos - 1 : pos);
                const bool low = (lane & (lph - 1)) < (lph >> 1);
                const int dr = low ? d0 : d0 - (D >> 1);
#pragma unroll
                for (int e2 = 0; e2 < 4; ++e2) {
                  const float other = __shfl_xor_sync(0xffffffffu, v[e2], lph >> 1);  // dim d +- head_dim / 2
                  if (is_q || is_k) {
                    const float cs = a.cos_t[static_cast<size_t>(pos) * a.rot_half + dr + e2], sn = a.sin_t[static_cast<size_t>(pos) * a.rot_half + dr + e2];
                    v[e2] = low ? v[e2] * cs - other * sn : v[e2] * cs + other * sn;
                  }
                }
              }
              uint2 pk;
              pk.x = pack_bf162(v[0], v[1]);
              pk.y = pack_bf162(v[2], v[3]);
              if (h < a.heads + 2 * a.kv_heads) {
                if (is_q) {
                  *reinterpret_cast<uint2*>(o.out + static_cast<size_t>(m) * a.heads * D + static_cast<size_t>(h) * D + d0) = pk;
                } else {
                  const long long slot = a.slots != nullptr ? a.slots[m] : -1;
                  if (slot >= 0) {
                    const long long blk = slot / a.block_size, off = slot % a.block_size;
                    __nv_bfloat16* cache = is_k ? a.k_cache : a.v_cache;
                    *reinterpret_cast<uint2*>(cache + ((blk * a.kv_heads + kvh) * a.block_size + off) * D + d0) = pk;
                  }
                }
              }
            }
          }
          asm volatile("bar.sync 1, 512;" ::: "memory");
          if (t == 0) red_release_gpu_add(p.sync + o.off_done, 1u);
        }
      }
    }
  }
  // ---------------- teardown ----------------
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kGemmTmemCols);
  }
  if (*abort_flag == 0) {
    // the last CTA to leave clears the counters for the next launch (every CTA has passed all its waits by then)
    if (threadIdx.x == 0) {
      __threadfence();
      *s_flag = atomicAdd(p.sync, 1u) == static_cast<unsigned>(P) - 1u ? 1 : 0;
    }
    __syncthreads();
    if (*s_flag) {
      for (int j = threadIdx.x; j < p.sync_words; j += blockDim.x) p.sync[j] = 0u;
    }
  }
}

// ------------------------------------------------------------------------------------------------ host side
void encode_map_kchunks(CUtensorMap* map, const void* base, uint64_t rows, uint64_t K, uint64_t pitch_bytes, uint32_t box_rows);
int gemm_num_sms();

int chain_smax(int n_tiles, int kbt, int P) {
  const long long U = static_cast<long long>(n_tiles) * kbt;
  int smax = 1;
  for (int t = 0; t < n_tiles; ++t) {
    const int ns = chain_nseg(t, kbt, U, P);
    if (ns > smax) smax = ns;
  }
  return smax;
}

size_t chain_ws_floats(int N, int K, int P) {
  const int n_tiles = (N + 127) / 128, kbt = (K + 127) / 128;
  return static_cast<size_t>(n_tiles) * chain_smax(n_tiles, kbt, P) * kChainMaxRows * 128;
}

int chain_ctas() { return gemm_num_sms(); }

int chain_sync_words(const ChainOp* ops, int n_ops) {
  int words = 1;
  for (int g = 0; g < n_ops; ++g) words += (ops[g].N + 127) / 128 + 1;
  return words;
}

template <int BN>
static void chain_launch_t(const ChainParams& p, int P, cudaStream_t st) {
  using L = GemmSmem<true, BN>;
  static PerDeviceOnce attr_once;
  if (attr_once.first()) {
    cudaError_t e = cudaFuncSetAttribute(decode_chain_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kBytes);
    if (e != cudaSuccess) throw std::runtime_error(std::string("decode chain: cudaFuncSetAttribute: ") + cudaGetErrorString(e));
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(P);
  cfg.blockDim = dim3(kGemmThreads);
  cfg.dynamicSmemBytes = L::kBytes;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = g_pdl_enabled ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, decode_chain_kernel<BN>, p);
  if (e != cudaSuccess) throw std::runtime_error(std::string("decode chain launch: ") + cudaGetErrorString(e));
}

void chain_run(const ChainOp* ops, int n_ops, const ChainQkvArgs* qkv, int M, unsigned* sync, int sync_words, int* status, cudaStream_t st) {
  if (M <= 0) return;
  if (n_ops < 1 || n_ops > kChainMaxOps) throw std::runtime_error("decode chain: 1..4 projections per launch");
  if (M > kChainMaxRows) throw std::runtime_error("decode chain: at most 64 token rows");
  if (sync_words < chain_sync_words(ops, n_ops)) throw std::runtime_error("decode chain: counter array too small");
  const int P = chain_ctas();
  const int BN = M <= 16 ? 16 : (M <= 32 ? 32 : 64);
  ChainParams p = {};
  p.n_ops = n_ops;
  p.M = M;
  p.sync = sync;
  p.sync_words = chain_sync_words(ops, n_ops);
  p.status = status;
  if (qkv != nullptr) p.qkv = *qkv;
  int off = 1;
  for (int g = 0; g < n_ops; ++g) {
    const ChainOp& s = ops[g];
    if (s.K % 64 != 0 || s.N % 8 != 0) throw std::runtime_error("decode chain: K must be a multiple of 64 and N of 8");
    if (s.K > 32768) throw std::runtime_error("decode chain: K of at most 32768");
    const int n_tiles = (s.N + 127) / 128;
    if (s.kind == kChainRowActMul && (n_tiles % 2 != 0 || (s.N / 2) % 128 != 0)) throw std::runtime_error("decode chain: gate|up halves must be whole tiles");
    if (s.kind == kChainRowQkvRope && (qkv == nullptr || (qkv->head_dim != 64 && qkv->head_dim != 128) || s.N != (qkv->heads + 2 * qkv->kv_heads) * qkv->head_dim ||
                                       (qkv->cos_t != nullptr && qkv->rot_half != qkv->head_dim / 2)))
      throw std::runtime_error("decode chain: the q|k|v stage takes head_dim 64 or 128 with full rotary embedding");
    if (g > 0 && s.dep && (ops[g - 1].kind == kChainRowQkvRope || ops[g - 1].kind == kChainRowAdd)) throw std::runtime_error("decode chain: stage without row output feeds a projection");
    if (s.dep && (g == 0 || s.K != (ops[g - 1].kind == kChainRowActMul ? ops[g - 1].N / 2 : ops[g - 1].N))) throw std::runtime_error("decode chain: input width does not match the stage in front");
    if (s.scale_src >= g || (s.scale_src >= 0 && ops[s.scale_src].kind != kChainRowAddNorm)) throw std::runtime_error("decode chain: bad scale source");
    ChainOpDev& d = p.op[g];
    d.wq = static_cast<const uint8_t*>(s.wq);
    d.ws = s.ws;
    d.ssq = s.ssq;
    d.N = s.N;
    d.K = s.K;
    d.n_tiles = n_tiles;
    d.kbt = (s.K + 127) / 128;
    d.smax = chain_smax(d.n_tiles, d.kbt, P);
    d.kind = s.kind;
    d.dep = s.dep ? 1 : 0;
    d.scale_src = s.scale_src;
    d.off_cnt = off;
    d.off_done = off + n_tiles;
    off = d.off_done + 1;
    d.fin_total = 0;  // finishers of the projection: every segment holder of every tile (gate|up: of the up tiles)
    for (int tt = (s.kind == kChainRowActMul ? n_tiles / 2 : 0); tt < n_tiles; ++tt)
      d.fin_total += chain_nseg(tt, d.kbt, static_cast<long long>(n_tiles) * d.kbt, P);
    d.bias = s.bias;
    d.residual = static_cast<__nv_bfloat16*>(s.residual);
    d.norm_w = static_cast<const __nv_bfloat16*>(s.norm_w);
    d.out = static_cast<__nv_bfloat16*>(s.out);
    d.eps = s.eps;
    d.offset = s.offset;
    d.res_mult = s.res_mult;
    d.act = s.act;
    encode_map_kchunks(&p.maps[g], s.x, static_cast<uint64_t>(s.x_rows), static_cast<uint64_t>(s.K), static_cast<uint64_t>(s.K) * 2, BN);
  }
  switch (BN) {
    case 16: chain_launch_t<16>(p, P, st); break;
    case 32: chain_launch_t<32>(p, P, st); break;
    default: chain_launch_t<64>(p, P, st); break;
  }
}

}  // namespace dlv
