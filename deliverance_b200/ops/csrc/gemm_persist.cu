// Persistent JQ4 GEMM for prefill-size batches: one CTA per SM walks many 128 x 128 output tiles and the epilogue of tile i runs
// under the main loop of tile i + 1.
//
// Why: the one-tile-per-CTA kernel (gemm_tc.cuh) spends about half of a CTA's life at these sizes outside the main loop: barrier
// set-up, tensor-memory allocation and the first copies in flight before it, the drain of the accumulator through a staging tile
// after it, with the tensor pipe idle both times (tensor pipe 48 % active; switching the activation copies and the weight expansion
// off inside that kernel gained 11 % together, so its main loop is not supply-bound).
// Here the rings (packed weights 8 x 10 KB, activations 4 x 32 KB in shared memory; expanded weights 4 x 64 columns of tensor memory)
// run across tile boundaries, two accumulators of 128 columns alternate, and four epilogue warps store a finished accumulator straight
// from tensor memory to global memory while the issuers are already in the next tile.
//   warp 0      producers: lanes 0 / 1 copy the packed-weight stage of the even / odd k-blocks, lanes 2 / 3 the activation stage
//               (a thread can start a copy only every few hundred nanoseconds, lanes of one warp do so side by side)
//   warps 1-3, 24  four MMA issuers, k-blocks g, g + 4, ..., all into the tile's accumulator: the owner of a tile's first k-block
//               (always issuer 0: the number of k-blocks is a multiple of 4) overwrites, and the others do not issue into the
//               tile before that first k-block has retired (barrier `first`)
//   warps 4-19  four groups of four warps expand nibbles to bf16 pairs and store them into the tensor-memory A ring (group g takes
//               the k-blocks g, g + 4, ...; a warp owns the TMEM lane quarter warp % 4), exactly as in gemm_tc.cuh
//   warps 20-23 epilogue: warp % 4 = TMEM lane quarter; a thread holds one weight row (= output column) of the tile, reads its 128
//               token values with tcgen05.ld, adds the bias and stores bf16 or fp32 (a warp writes 32 consecutive outputs per token)
// Parity-only mbarrier waits must see every phase of a barrier, so every stage belongs to one producer lane, one dequant group and
// one issuer for the whole kernel (ring depths are multiples of 2 and 4, k-blocks are numbered across tiles).
// Every wait is bounded (common.cuh); on expiry the CTA raises its abort flag, every role leaves its loop, copies and MMAs in flight
// are given a bounded time to land, tensor memory is freed and a status word tells the host.
//
// Status (B200, JQ4, M = 2048 / 8192 tokens, us; one-tile kernel in brackets), issuers racing: 6144 x 2560 61 / 224 (70 / 245),
// 2560 x 4096 48 / 161 (57 / 160), 19456 x 2560 180 / 720 (202 / 734), 2560 x 9728 112 / 419 (127 / 368). With two issuers it only
// matched the one-tile kernel: in-kernel clocks showed each issuer 1,070 cycles per k-block issuing (its 8 MMAs queue behind the
// other's: the pipe is busy), 340 waiting for operands and 310 between turns, i.e. the pipe 59 % busy; four issuers cover each
// other's turn-around. Letting an issuer take two k-blocks per turn instead moved the time into the operand waits (the four-stage
// ring of expanded weights).
// Racing issuers reach the one accumulator in an order that varies from launch to launch, and fp32 accumulation depends on the
// order: repeated launches differed in the last bits. With the issuers taking turns in k-block order (a counter in shared memory;
// the default of this kernel) the results are bit-reproducible and the gain is gone: 75 / 246, 60 / 156, 199 / 770, 129 / 344 us,
// because the gain came from several threads having MMAs queued at the same time. The engine promises the same logits for the same
// prompt (prefix-cache hits, replicas, tensor-parallel ranks), and the whole prefill moved by 0.6 % (99.7K against 99.1K tokens/s,
// its chunks are 8192 tokens), so the kernel is off by default: DLV_GEMM_PERSIST=1 turns it on ordered, =race turns it on racing.
//
// The reference has no counterpart (its prefill multiplies token by token on the CPU: core/.../generator/MLPBlock.java and
// native/src/main/c/simd/vector_simd.c:595).
#include <stdexcept>
#include <string>

#include "gemm_api.h"
#include "gemm_tc.cuh"

namespace dlv {

void encode_map_kchunks(CUtensorMap* map, const void* base, uint64_t rows, uint64_t K, uint64_t pitch_bytes, uint32_t box_rows);
int gemm_num_sms();

namespace {

constexpr int kPT = 128;                       // tokens per tile
constexpr int kPNR = 8, kPNX = 4, kPNA = 4;    // ring depths
constexpr int kPRaw = kGemmBM * 64 + kGemmBM * 16;  // packed nibbles (8 KB) + scales (2 KB)
constexpr int kPXStage = kPT * 256;            // two 64-wide bf16 sub-tiles of 128 tokens
constexpr int kPOffRaw = kPNX * kPXStage;
constexpr int kPOffCtrl = kPOffRaw + kPNR * kPRaw;
constexpr int kPBytes = kPOffCtrl + 1024 + 1024;  // barriers + alignment slack
constexpr int kPTmemA = 256;                   // accumulators at columns [0, 256), A ring behind them
constexpr int kPNI = 4;                        // MMA-issuing threads (k-blocks g, g + 4, ... each)
constexpr int kPThreads = 800;                 // 25 warps: 72 registers per thread

struct PersistParams {
  const uint8_t* wq;
  void* out;
  const float* bias;
  int* status;
  int M, N, K, ldo, out_f32;
  int n_tiles, m_tiles, nkb, total_tiles;
  int ordered;  // issuers take turns in k-block order (bit-reproducible results)
};

__global__ void __launch_bounds__(kPThreads, 1) gemm_persist_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                                                                    const PersistParams p) {
  extern __shared__ uint8_t ps_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(ps_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bar_r_full = reinterpret_cast<uint64_t*>(smem + kPOffCtrl);
  uint64_t* bar_r_empty = bar_r_full + kPNR;
  uint64_t* bar_x_full = bar_r_empty + kPNR;
  uint64_t* bar_x_empty = bar_x_full + kPNX;
  uint64_t* bar_a_full = bar_x_empty + kPNX;
  uint64_t* bar_a_empty = bar_a_full + kPNA;
  uint64_t* bar_acc_full = bar_a_empty + kPNA;   // [2]
  uint64_t* bar_acc_empty = bar_acc_full + 2;    // [2]
  uint64_t* bar_first = bar_acc_empty + 2;       // [2]
  uint64_t* bar_drain = bar_first + 2;           // [kPNI] issuers' outstanding MMAs (abort path)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_drain + kPNI);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* issue_seq = abort_flag + 1;  // number of k-blocks whose MMAs have been issued (the issuers take turns in k-block order)

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // tiles of this CTA: blockIdx.x, blockIdx.x + gridDim.x, ...; consecutive tiles share a weight tile (m is the fast index)
  const int my_tiles = (p.total_tiles - static_cast<int>(blockIdx.x) + static_cast<int>(gridDim.x) - 1) / static_cast<int>(gridDim.x);
  const int nkb = p.nkb;
  const int total_kb = my_tiles * nkb;  // k-blocks of this CTA, numbered across its tiles (32-bit on purpose: a 64-bit division per
                                        // k-block on an issuer's path cost as much as the k-block's MMAs)

  if (threadIdx.x == 0) {
    for (int s = 0; s < kPNR; ++s) {
      mbar_init(smem_u32(&bar_r_full[s]), 1);
      mbar_init(smem_u32(&bar_r_empty[s]), 4);
    }
    for (int s = 0; s < kPNX; ++s) {
      mbar_init(smem_u32(&bar_x_full[s]), 1);
      mbar_init(smem_u32(&bar_x_empty[s]), 1);
    }
    for (int s = 0; s < kPNA; ++s) {
      mbar_init(smem_u32(&bar_a_full[s]), 4);
      mbar_init(smem_u32(&bar_a_empty[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&bar_acc_full[b]), kPNI);
      mbar_init(smem_u32(&bar_acc_empty[b]), 4);
      mbar_init(smem_u32(&bar_first[b]), 1);
    }
    for (int j = 0; j < kPNI; ++j) mbar_init(smem_u32(&bar_drain[j]), 1);
    *abort_flag = 0;
    *issue_seq = 0;
    mbar_fence_init();
    tma_prefetch_desc(&map_w);
    tma_prefetch_desc(&map_x);
  }
  pdl_trigger();
  if (warp == 1) tmem_alloc(smem_u32(tmem_slot), kGemmTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  auto raw_tile = [&](int s) { return smem + kPOffRaw + s * kPRaw; };
  auto x_tile = [&](int s, int sub) { return smem + s * kPXStage + sub * (kPT * 128); };
  auto tile_of = [&](int it, int& n_tile, int& m_tile) {
    const int t = static_cast<int>(blockIdx.x) + it * static_cast<int>(gridDim.x);
    n_tile = t / p.m_tiles;
    m_tile = t - n_tile * p.m_tiles;
  };

  if (warp == 0) {
    // ---------------- producers ----------------
    if (lane < 4) {
      const bool is_x = lane >= 2;
      const int par = lane & 1;
      if (is_x) pdl_wait();  // the activations come from the kernel in front; weights may stream before it has finished
      int last = -1;
      int n_issued = 0;
      int it = 0, i = par;  // tile and k-block inside the tile of g (the number of k-blocks per tile is even)
      for (int g = par; g < total_kb; g += 2, i += 2) {
        if (i >= nkb) { i -= nkb; ++it; }
        int n_tile, m_tile;
        tile_of(it, n_tile, m_tile);
        if (!is_x) {
          const int s = g % kPNR;
          if (!mbar_wait(smem_u32(&bar_r_empty[s]), (static_cast<uint32_t>(g / kPNR) & 1) ^ 1, abort_flag, p.status)) break;
          const uint32_t full = smem_u32(&bar_r_full[s]);
          mbar_expect_tx(full, kPRaw);
          tma_load_2d(smem_u32(raw_tile(s)), &map_w, full, 0, (n_tile * nkb + i) * 10);
        } else {
          const int s = g % kPNX;
          if (!mbar_wait(smem_u32(&bar_x_empty[s]), (static_cast<uint32_t>(g / kPNX) & 1) ^ 1, abort_flag, p.status)) break;
          const uint32_t full = smem_u32(&bar_x_full[s]);
          mbar_expect_tx(full, kPXStage);
          tma_load_3d(smem_u32(x_tile(s, 0)), &map_x, full, 0, m_tile * kPT, i * 2);
        }
        last = g;
        ++n_issued;
      }
      if (*abort_flag && last >= 0) {
        // let the copies that are still in flight land before the CTA goes away (bounded)
        const int ring = is_x ? kPNX : kPNR;
        for (int j = 0; j < ring / 2 && j < n_issued; ++j) {
          const int g = last - 2 * j;
          const uint32_t bar = smem_u32(is_x ? &bar_x_full[g % kPNX] : &bar_r_full[g % kPNR]);
          const uint32_t ph = static_cast<uint32_t>(g / ring) & 1;
          const unsigned long long t0 = globaltimer_ns();
          while (!mbar_try_wait(bar, ph) && globaltimer_ns() - t0 < 20000000ull) {
          }
        }
      }
    }
  } else if (warp == 1 || warp == 2 || warp == 3 || warp == 24) {
    // ---------------- MMA issuers (one lane each) ----------------
    if (lane == 0) {
      const int par = warp == 24 ? 3 : warp - 1;
      constexpr uint32_t idesc = umma_idesc_bf16(kGemmBM, kPT);
      const uint64_t desc_x0 = umma_desc_k_sw128(smem_u32(smem));
      bool ok = true;
      int it = 0, i = par;
      for (int g = par; g < total_kb && ok; g += kPNI, i += kPNI) {
        if (i >= nkb) { i -= nkb; ++it; }
        const int b = it & 1;
        if (i == par) {
          // first k-block of this issuer in the tile
          if (par == 0) ok = mbar_wait(smem_u32(&bar_acc_empty[b]), ((static_cast<uint32_t>(it) >> 1) & 1) ^ 1, abort_flag, p.status);
          else ok = mbar_wait(smem_u32(&bar_first[b]), (static_cast<uint32_t>(it) >> 1) & 1, abort_flag, p.status);
          if (!ok) break;
        }
        const int sa = g % kPNA, sx = g % kPNX;
        ok = mbar_wait(smem_u32(&bar_a_full[sa]), static_cast<uint32_t>(g / kPNA) & 1, abort_flag, p.status) &&
             mbar_wait(smem_u32(&bar_x_full[sx]), static_cast<uint32_t>(g / kPNX) & 1, abort_flag, p.status);
        if (!ok) break;
        // Turn-taking: the MMAs of k-block g are issued after those of k-block g - 1 (by another thread). The tensor pipe executes
        // in the order of issue, so the accumulation order is the k order and results are bit-reproducible; the issuer whose turn
        // comes next has its operands checked already and starts the moment its predecessor has issued.
        if (p.ordered && *issue_seq < g) {
            const long long t0 = clock64();
            while (*issue_seq < g) {
                if (clock64() - t0 > kWaitLimitCycles || *abort_flag) {
                    *abort_flag = 1;
                    if (p.status) atomicCAS(p.status, kStatusOk, kStatusBarrierTimeout);
                    ok = false;
                    break;
                }
            }
            if (!ok) break;
        }
        tc_fence_after();
        const uint32_t tmem_acc = tmem_base + b * kPT;
        const uint64_t dx = desc_x0 + static_cast<uint64_t>((sx * kPXStage) >> 4);
#pragma unroll
        for (int k4 = 0; k4 < 8; ++k4) {
          const uint64_t db = dx + static_cast<uint64_t>(((k4 >> 2) * (kPT * 128) + (k4 & 3) * 32) >> 4);
          umma_bf16_ts(tmem_acc, tmem_base + kPTmemA + sa * kGemmTmemAStage + k4 * 8, db, idesc, (i > 0 || k4 > 0) ? 1u : 0u);
        }
        __threadfence_block();
        *issue_seq = g + 1;
        umma_commit(smem_u32(&bar_a_empty[sa]));
        umma_commit(smem_u32(&bar_x_empty[sx]));
        if (i == 0) umma_commit(smem_u32(&bar_first[b]));
        if (i + kPNI >= nkb) umma_commit(smem_u32(&bar_acc_full[b]));  // this issuer's last k-block of the tile
      }
      if (!ok) {
        umma_commit(smem_u32(&bar_drain[par]));
        const unsigned long long t0 = globaltimer_ns();
        while (!mbar_try_wait(smem_u32(&bar_drain[par]), 0) && globaltimer_ns() - t0 < 20000000ull) {
        }
      }
    }
  } else if (warp >= 4 && warp < 20) {
    // ---------------- weight expansion: packed nibbles -> bf16 pairs in the tensor-memory A ring ----------------
    const int we = warp - 4, grp = we >> 2, q = warp & 3;
    const int r = q * 32 + lane;
    for (int g = grp; g < total_kb; g += 4) {
      const int sr = g % kPNR, sa = g % kPNA;
      if (!mbar_wait(smem_u32(&bar_r_full[sr]), static_cast<uint32_t>(g / kPNR) & 1, abort_flag, p.status)) break;
      uint4 wq[4];
#pragma unroll
      for (int blk = 0; blk < 4; ++blk) wq[blk] = *reinterpret_cast<const uint4*>(raw_tile(sr) + r * 64 + ((blk ^ ((r >> 1) & 3)) << 4));
      const float4 sc4 = *reinterpret_cast<const float4*>(raw_tile(sr) + kGemmBM * 64 + r * 16);
      const float sc[4] = {sc4.x, sc4.y, sc4.z, sc4.w};
      // the tensor-memory stage is free once the MMAs of k-block g - 4 have retired
      if (!mbar_wait(smem_u32(&bar_a_empty[sa]), (static_cast<uint32_t>(g / kPNA) & 1) ^ 1, abort_flag, p.status)) break;
      tc_fence_after();
      const uint32_t tdst = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + kPTmemA + sa * kGemmTmemAStage;
#pragma unroll
      for (int blk = 0; blk < 4; ++blk) {
        const __nv_bfloat162 s2 = __float2bfloat162_rn(sc[blk]);
        const uint32_t words[4] = {wq[blk].x, wq[blk].y, wq[blk].z, wq[blk].w};
        uint32_t o[16];  // 32 bf16: elements 0..15 from the low nibbles of bytes 0..15, 16..31 from the high nibbles
#pragma unroll
        for (int hl = 0; hl < 2; ++hl) {
#pragma unroll
          for (int wd = 0; wd < 4; ++wd) {
            const uint32_t a = (words[wd] >> (4 * hl)) & 0x0F0F0F0Fu;
            o[hl * 8 + wd * 2 + 0] = q4_pair_to_bf162(a, 0x4140u, s2);
            o[hl * 8 + wd * 2 + 1] = q4_pair_to_bf162(a, 0x4342u, s2);
          }
        }
        tmem_st_x16(tdst + blk * 16, o);
      }
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(smem_u32(&bar_r_empty[sr]));
        mbar_arrive(smem_u32(&bar_a_full[sa]));
      }
    }
  } else if (warp >= 20) {
    // ---------------- epilogue: accumulator b of tile `it` -> global memory, while the issuers work on the other accumulator ----------------
    const int q = warp & 3;
    pdl_wait();  // global memory is written only after the kernel in front has completed
    for (int it = 0; it < my_tiles; ++it) {
      const int b = it & 1;
      int n_tile, m_tile;
      tile_of(it, n_tile, m_tile);
      // warp-uniform: the loop holds warp-collective tensor-memory loads
      const bool ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&bar_acc_full[b]), (static_cast<uint32_t>(it) >> 1) & 1, abort_flag, p.status));
      if (!ok) break;
      tc_fence_after();
      const int n = n_tile * kGemmBM + q * 32 + lane;  // output column of this thread
      const float bv = (p.bias != nullptr && n < p.N) ? p.bias[n] : 0.f;
      const int m0 = m_tile * kPT;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + b * kPT;
#pragma unroll 1
      for (int c0 = 0; c0 < kPT; c0 += 16) {
        uint32_t v[16];
        tmem_ld_x16(taddr + c0, v);
        tmem_ld_wait();
        if (n < p.N) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int m = m0 + c0 + j;
            if (m < p.M) {
              const float val = __uint_as_float(v[j]) + bv;
              if (p.out_f32) static_cast<float*>(p.out)[static_cast<size_t>(m) * p.ldo + n] = val;
              else static_cast<__nv_bfloat16*>(p.out)[static_cast<size_t>(m) * p.ldo + n] = f2bf(val);
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bar_acc_empty[b]));
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kGemmTmemCols);
  }
}

}  // namespace

bool g_gemm_persist = false;         // prefill-size JQ4 projections on the persistent kernel (binding gemm_persist; off by default, see Status above)
bool g_gemm_persist_ordered = true;  // its issuers take turns in k-block order; false: they race (faster, results vary in the last bits)

bool gemm_persist_supported(const GemmWeightDesc* w, int M, int ldx) {
  // every issuer must have the same k-blocks in every tile
  return w->is_q4 && w->K % (kGemmBK * kPNI) == 0 && w->N % 4 == 0 && ldx % 8 == 0 && M >= 256;
}
// Where the racing form measured faster than the one-tile kernel (B200, four issuers): every shape at 2048 tokens by 11-16 %, wide
// projections (6144 and 19456 rows) also at 8192 tokens by 2-9 %; narrow deep ones (2560 x 9728) lose 14 % at 8192 tokens.
bool gemm_persist_preferred(const GemmWeightDesc* w, int M) { return M <= 4096 || w->N >= 4096; }

void gemm_persist_run(const GemmWeightDesc* w, const void* x, int M, int ldx, void* out, int ldo, bool out_f32, const float* bias, int* status,
                      cudaStream_t st) {
  static PerDeviceOnce attr_once;
  if (attr_once.first()) {
    cudaError_t e = cudaFuncSetAttribute(gemm_persist_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kPBytes);
    if (e != cudaSuccess) throw std::runtime_error(std::string("persistent gemm: cudaFuncSetAttribute: ") + cudaGetErrorString(e));
  }
  PersistParams p = {};
  p.wq = static_cast<const uint8_t*>(w->data);
  p.out = out;
  p.bias = bias;
  p.status = status;
  p.M = M;
  p.N = w->N;
  p.K = w->K;
  p.ldo = ldo;
  p.out_f32 = out_f32 ? 1 : 0;
  p.n_tiles = (w->N + kGemmBM - 1) / kGemmBM;
  p.m_tiles = (M + kPT - 1) / kPT;
  p.nkb = w->K / kGemmBK;
  p.total_tiles = p.n_tiles * p.m_tiles;
  p.ordered = g_gemm_persist_ordered ? 1 : 0;
  CUtensorMap map_x;
  encode_map_kchunks(&map_x, x, static_cast<uint64_t>(M), static_cast<uint64_t>(w->K), static_cast<uint64_t>(ldx) * 2, kPT);
  const int grid = p.total_tiles < gemm_num_sms() ? p.total_tiles : gemm_num_sms();
  cudaError_t e = launch_pdl(gemm_persist_kernel, dim3(grid), dim3(kPThreads), static_cast<size_t>(kPBytes), st, w->map_w, map_x, p);
  if (e != cudaSuccess) throw std::runtime_error(std::string("persistent gemm launch: ") + cudaGetErrorString(e));
}

}  // namespace dlv
