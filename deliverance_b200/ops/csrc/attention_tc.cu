// Paged flash attention for prefill on the 5th-generation tensor cores (tcgen05 / TMEM / TMA).
//
// One CTA per (256 query rows of one sequence, query head): two 128-row query tiles that share every K / V tile (one tile when fewer
// than 129 rows are left, or for head_dim 256, whose accumulator leaves no room for a second one). Keys go by in tiles of 64.
//   warp 1            = TMA producer: the Q tiles once (D / 64 boxes of 128 rows x 64 columns each), then per key tile the K and V rows
//                       of its cache pages (a page slice of one KV head is `page` rows x D contiguous bf16 = D / 64 boxes of up to 64
//                       rows x 64 columns), all into 128-byte-swizzled shared memory, completion on mbarriers, 4 stages (2 for D = 256);
//                       the copies of a tile are spread over the warp's lanes;
//   warp 0, one lane  = issues S = Q K^T for every (key tile, query tile): both operands from shared memory, K-major, the
//                       accumulator is one of the query tile's two 64-column score slots in tensor memory;
//   warp 2, one lane  = issues O += P V: P from tensor memory as the A operand, V from shared memory as an MN-major B operand;
//   warps 4-7 (8-11)  = softmax of query tile 0 (1): thread r owns query row r (TMEM lane r): tcgen05.ld of the 64 scores, mask
//                       (causal / sliding window / context end), optional logit soft-cap, running maximum and sum in registers, rescale
//                       of the O accumulator in tensor memory when the maximum has moved by more than 2^8, P written back over the
//                       scores as packed bf16 (tcgen05.st), finally O / l to global memory.
// Tensor memory (512 columns): score slots at [0, 256) = (query tile, slot) x 64, accumulators at 256 + query tile x D.
// Why two issuing threads: a tcgen05.mma holds its thread until the pipe accepts it and the pipe queues almost nothing, so the tensor
// cores idle whenever their issuer waits on a barrier (even a complete one costs a few hundred cycles) or walks its loop; with the
// Q K^T and the P V streams on threads of their own, one feeds the pipe while the other waits. Measured on the way here (B200, 32 query
// / 8 KV heads of 128, 2 x 8192 tokens causal): one issuing warp whose 32 lanes all wait and vote 442 TFLOP/s, the same loop on one
// lane 443, two issuing threads 729; a single thread issuing all copies of a tile 265, the lanes of the warp 733.
// Every wait is bounded (common.cuh); on expiry the CTA records a status word, skips its stores, lets its copies and MMAs drain
// (bounded), frees tensor memory and returns; CTAs that start after a recorded failure leave at once.
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

constexpr int kAtBM = 128, kAtBN = 64;  // query rows per score tile / keys per tile

template <int D, int QT>
struct AttnTcSmem {
  static constexpr int kSub = D / 64;                  // 64-column sub-tiles per operand tile
  static constexpr int kTileQ = kAtBM * 128 * kSub;    // bytes of a [128 rows][D] bf16 query tile
  static constexpr int kTileKV = kAtBN * 128 * kSub;   // bytes of a [64 keys][D] bf16 K or V tile
  static constexpr int kStages = D <= 128 ? 4 : 2;
  static constexpr int kOffK = QT * kTileQ;
  static constexpr int kOffV = kOffK + kStages * kTileKV;
  static constexpr int kOffCtrl = kOffV + kStages * kTileKV;
  static constexpr int kNeed = kOffCtrl + 512 + 1024;  // barriers + alignment slack
  // every CTA allocates all 512 tensor-memory columns, so two CTAs must never share an SM: ask for more than half of its shared memory
  static constexpr int kBytes = kNeed > 118 * 1024 ? kNeed : 118 * 1024;
  static constexpr int kThreads = 128 + 128 * QT;  // warp 0 issues Q K^T, warp 1 the copies, warp 2 issues P V, warp 3 idles, warps 4.. softmax
};

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float y;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(y) : "f"(a), "f"(b), "f"(c));
  return y;
}

template <int D, int QT>
__global__ void __launch_bounds__(AttnTcSmem<D, QT>::kThreads, 1)
    prefill_attn_tc_kernel(const __grid_constant__ CUtensorMap map_q,  // [T, H * D], box 128 x 64
                           const __grid_constant__ CUtensorMap map_k,  // [pages * KV * page, D], box min(page, 64) x 64
                           const __grid_constant__ CUtensorMap map_v, const AttnTcParams p) {
  using L = AttnTcSmem<D, QT>;
  constexpr int NS = L::kStages, SUB = L::kSub;
  constexpr int kProducer = 1, kIssuer = 0, kIssuerPV = 2;
  extern __shared__ uint8_t at_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(at_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bar_q = reinterpret_cast<uint64_t*>(smem + L::kOffCtrl);
  uint64_t* bar_k_full = bar_q + 1;        // [4] K tile landed
  uint64_t* bar_v_full = bar_k_full + 4;   // [4] V tile landed
  uint64_t* bar_k_empty = bar_v_full + 4;  // [4] every Q K^T of the tile has retired
  uint64_t* bar_v_empty = bar_k_empty + 4; // [4] every P V of the tile has retired
  uint64_t* bar_s_full = bar_v_empty + 4;  // [2 query tiles][2 slots] scores complete
  uint64_t* bar_p_full = bar_s_full + 4;   // [2][2] probabilities written over the scores
  uint64_t* bar_pv_done = bar_p_full + 4;  // [2][2] the P V that read the slot's probabilities has retired
  uint64_t* bar_o_final = bar_pv_done + 4;
  uint64_t* bar_drain = bar_o_final + 1;    // [2] an issuing thread's MMAs have retired (only used when a wait ran out)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_drain + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // a CTA that starts after another one of this or an earlier launch has recorded a failed wait leaves at once: one stuck tile
  // must not make every later tile sit out its own time limit
  if (__syncthreads_or(threadIdx.x == 0 && *reinterpret_cast<volatile int*>(p.status) != 0)) return;
  // heavy tiles first: inside a sequence the late query tiles see the most keys, and the host lists tiles in ascending order
  const int tile = static_cast<int>(gridDim.x) - 1 - static_cast<int>(blockIdx.x);
  const int seq = p.tile_seq[tile], q0 = p.tile_q0[tile], h = blockIdx.y;
  const int kvh = h / (p.H / p.KV);
  const int qs = p.q_start[seq], ql = p.q_len[seq], ctx = p.ctx_lens[seq];
  const int pos0 = ctx - ql;  // position of the sequence's first query row
  const int rows_all = min(QT * kAtBM, ql - q0);
  const bool two = QT == 2 && rows_all > kAtBM;  // two query tiles share every K / V tile
  // key tiles [a, b) each query tile sees
  int rows_q[2], first_q[2], a_q[2], b_q[2];
#pragma unroll
  for (int q = 0; q < 2; ++q) {
    rows_q[q] = max(0, min(kAtBM, rows_all - q * kAtBM));
    first_q[q] = pos0 + q0 + q * kAtBM;
    const int last_pos = p.causal ? first_q[q] + rows_q[q] - 1 : ctx - 1;
    const int key_hi = min(ctx, last_pos + 1);
    const int key_lo = p.window > 0 ? max(0, first_q[q] - p.window + 1) : 0;
    a_q[q] = key_lo / kAtBN;
    b_q[q] = rows_q[q] > 0 ? (key_hi + kAtBN - 1) / kAtBN : a_q[q];
  }
  const int a0 = a_q[0], b0 = b_q[0], a1 = a_q[1], b1 = two ? b_q[1] : a_q[1];
  const int lo = a0, hi = two ? max(b0, b1) : b0;  // key tiles this CTA loads
  const int n_tiles = hi - lo;

  if (threadIdx.x == 0) {
    mbar_init(smem_u32(bar_q), 1);
    for (int s = 0; s < 4; ++s) {
      mbar_init(smem_u32(&bar_k_full[s]), 1);
      mbar_init(smem_u32(&bar_v_full[s]), 1);
      mbar_init(smem_u32(&bar_k_empty[s]), 1);
      mbar_init(smem_u32(&bar_v_empty[s]), 1);
      mbar_init(smem_u32(&bar_s_full[s]), 1);
      mbar_init(smem_u32(&bar_p_full[s]), 4);
      mbar_init(smem_u32(&bar_pv_done[s]), 1);
    }
    mbar_init(smem_u32(&bar_drain[0]), 1);
    mbar_init(smem_u32(&bar_drain[1]), 1);
    mbar_init(smem_u32(bar_o_final), 1);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&map_q);
    tma_prefetch_desc(&map_k);
    tma_prefetch_desc(&map_v);
  }
  constexpr uint32_t kTmemCols = 512;
  if (warp == kIssuer) tmem_alloc(smem_u32(tmem_slot), kTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  constexpr uint32_t kColS = 0, kColO = 256;  // score slot b of query tile q at kColS + (2 q + b) 64, accumulator of query tile q at kColO + q D
  pdl_wait();
  pdl_trigger();

  if (warp == kProducer) {
    // ---------------- TMA producer ----------------
    // One thread can start a tensor copy only every few hundred nanoseconds, whatever its size, and a key tile is several copies
    // (pages x D / 64 column blocks, for K and for V): the copies of a tile are spread over the lanes of the warp.
    if (lane == 0) {
      mbar_expect_tx(smem_u32(bar_q), (two ? 2 : 1) * L::kTileQ);
      for (int q = 0; q < (two ? 2 : 1); ++q)
        for (int c = 0; c < SUB; ++c)
          tma_load_2d(smem_u32(smem + q * L::kTileQ + c * (kAtBM * 128)), &map_q, smem_u32(bar_q), h * D + c * 64, qs + q0 + q * kAtBM);
    }
    const int box_rows = p.page_size < kAtBN ? p.page_size : kAtBN;  // page_size is 32, 64 or 128
    const int n_copy = (kAtBN / box_rows) * SUB;
    int issued = 0;
    bool ok = true;
    for (int t = 0; t < n_tiles; ++t, ++issued) {
      const int s = t % NS;
      const int kt = lo + t;
      for (int kv = 0; kv < 2; ++kv) {
        uint64_t* full = kv == 0 ? &bar_k_full[s] : &bar_v_full[s];
        uint64_t* empty = kv == 0 ? &bar_k_empty[s] : &bar_v_empty[s];
        if (t >= NS) ok = mbar_wait(smem_u32(empty), ((t / NS) - 1) & 1, abort_flag, p.status);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        if (lane == 0) mbar_expect_tx(smem_u32(full), L::kTileKV);
        __syncwarp();
        for (int i = lane; i < n_copy; i += 32) {
          const int pg = i / SUB, c = i - pg * SUB;
          const int key0 = kt * kAtBN + pg * box_rows;
          // pages past the context are never read by an unmasked score; the scratch page 0 keeps the copy inside the cache
          const int page = key0 < ctx ? p.block_tables[static_cast<long long>(seq) * p.bt_stride + key0 / p.page_size] : 0;
          const int row = (page * p.KV + kvh) * p.page_size + (key0 % p.page_size);
          const uint32_t off = c * (kAtBN * 128) + pg * box_rows * 128;
          tma_load_2d(smem_u32(smem + (kv == 0 ? L::kOffK : L::kOffV) + s * L::kTileKV + off), kv == 0 ? &map_k : &map_v, smem_u32(full), c * 64, row);
        }
      }
      if (!ok) break;
    }
    if (lane == 0 && *abort_flag) {
      // a wait ran out somewhere in the CTA: before shared memory goes away let the copies already issued land (bounded)
      for (int t = issued > NS ? issued - NS : 0; t < issued; ++t) {
        const unsigned long long t0 = globaltimer_ns();
        while (!(mbar_try_wait(smem_u32(&bar_k_full[t % NS]), (t / NS) & 1) && mbar_try_wait(smem_u32(&bar_v_full[t % NS]), (t / NS) & 1)) &&
               globaltimer_ns() - t0 < 20000000ull) {
        }
      }
    }
    __syncwarp();
  } else if (warp == kIssuer || warp == kIssuerPV) {
    // ---------------- MMA issuers ----------------
    // Work items (key tile j, query tile q) in order: (j, 0), (j, 1) for every j the query tile sees. Each query tile has two score
    // slots, used by its key tiles in turn.
    // A tcgen05.mma holds the issuing thread until the tensor pipe accepts it and the pipe queues next to nothing, so the pipe idles
    // whenever its issuer does anything else, and even a wait on a barrier that is already complete costs a few hundred cycles.
    // Hence two issuing threads with loops of their own: one thread of warp 0 issues the Q K^T of every item as soon as its slot is
    // free again (the P V that read the probabilities kept there has retired) and its K tile has landed; one thread of warp 2
    // issues the P V of every item once its probabilities are written and its V tile has landed. While one of them waits, the other
    // feeds the pipe. Everything the two depend on travels through mbarriers; tcgen05.commit covers the MMAs of its own thread.
    constexpr uint32_t idesc_s = umma_idesc_bf16(kAtBM, kAtBN);
    constexpr uint32_t idesc_o = umma_idesc_bf16_bmn(kAtBM, D);
    auto valid = [&](int j, int q) { return q == 0 ? (j >= a0 && j < b0) : (j >= a1 && j < b1); };
    auto advance = [&](int& j, int& q) {  // next valid item; j == hi when there is none
      do {
        if (two && q == 0) q = 1;
        else { q = 0; ++j; }
      } while (j < hi && !valid(j, q));
    };
    auto last_of_tile = [&](int j, int q) { return !two || q == 1 || !(j >= a1 && j < b1); };
    if (lane == 0) {
      bool ok = true;
      int j = lo, q = 0;
      if (n_tiles > 0 && !valid(j, q)) advance(j, q);
      if (warp == kIssuer) {
        ok = mbar_wait(smem_u32(bar_q), 0, abort_flag, p.status);
        const uint64_t desc_q0 = umma_desc_k_sw128(smem_u32(smem)), desc_k0 = umma_desc_k_sw128(smem_u32(smem + L::kOffK));
        int k_seen = lo - 1;  // key tiles whose K has been waited for
        while (ok && j < hi) {
          const int t = j - (q == 0 ? a0 : a1);
          const int s = (j - lo) % NS;
          const uint32_t slot = q * 2 + (t & 1);
          if (t >= 2) ok = mbar_wait(smem_u32(&bar_pv_done[slot]), ((t >> 1) - 1) & 1, abort_flag, p.status);
          if (ok && j > k_seen) {
            ok = mbar_wait(smem_u32(&bar_k_full[s]), ((j - lo) / NS) & 1, abort_flag, p.status);
            k_seen = j;
          }
          if (!ok) break;
          tc_fence_after();
          const uint64_t desc_q = desc_q0 + static_cast<uint64_t>((q * L::kTileQ) >> 4);
          const uint64_t desc_k = desc_k0 + static_cast<uint64_t>((s * L::kTileKV) >> 4);
          const uint32_t d_s = tmem_base + kColS + slot * kAtBN;
#pragma unroll
          for (int k16 = 0; k16 < D / 16; ++k16) {
            const uint64_t adv_q = static_cast<uint64_t>(((k16 >> 2) * (kAtBM * 128) + (k16 & 3) * 32) >> 4);
            const uint64_t adv_k = static_cast<uint64_t>(((k16 >> 2) * (kAtBN * 128) + (k16 & 3) * 32) >> 4);
            umma_bf16(d_s, desc_q + adv_q, desc_k + adv_k, idesc_s, k16 > 0 ? 1u : 0u);
          }
          if (last_of_tile(j, q)) umma_commit(smem_u32(&bar_k_empty[s]));
          umma_commit(smem_u32(&bar_s_full[slot]));
          advance(j, q);
        }
      } else {
        const uint32_t v_base = smem_u32(smem + L::kOffV);
        while (ok && j < hi) {
          const int t = j - (q == 0 ? a0 : a1);
          const int s = (j - lo) % NS;
          const uint32_t slot = q * 2 + (t & 1);
          ok = mbar_wait(smem_u32(&bar_p_full[slot]), (t >> 1) & 1, abort_flag, p.status) &&
               mbar_wait(smem_u32(&bar_v_full[s]), ((j - lo) / NS) & 1, abort_flag, p.status);
          if (!ok) break;
          tc_fence_after();
          const uint32_t tmem_p = tmem_base + kColS + slot * kAtBN, d_o = tmem_base + kColO + q * D;
          const uint64_t desc_v0 = umma_desc_mn_sw128(v_base + s * L::kTileKV, kAtBN * 128, 1024);
#pragma unroll
          for (int k16 = 0; k16 < kAtBN / 16; ++k16) {
            // 16 keys = two 8-row swizzle atoms (2048 bytes) further down the V tile; the 64-column blocks of D are kAtBN * 128 bytes apart
            umma_bf16_ts(d_o, tmem_p + k16 * 8, desc_v0 + static_cast<uint64_t>((k16 * 2048) >> 4), idesc_o, (t == 0 && k16 == 0) ? 0u : 1u);
          }
          if (last_of_tile(j, q)) umma_commit(smem_u32(&bar_v_empty[s]));
          umma_commit(smem_u32(&bar_pv_done[slot]));
          advance(j, q);
          if (j >= hi) umma_commit(smem_u32(bar_o_final));
        }
        if (n_tiles == 0) umma_commit(smem_u32(bar_o_final));
      }
      if (!ok) {
        // a wait ran out: let this thread's outstanding MMAs retire (bounded) before tensor memory is released
        uint64_t* drain = &bar_drain[warp == kIssuer ? 0 : 1];
        umma_commit(smem_u32(drain));
        const unsigned long long t0 = globaltimer_ns();
        while (!mbar_try_wait(smem_u32(drain), 0) && globaltimer_ns() - t0 < 20000000ull) {
        }
      }
    }
    __syncwarp();
  } else if (warp >= 4 && (warp < 8 || two)) {
    // ---------------- softmax warps: thread = query row ----------------
    const int q = (warp >> 2) - 1;  // query tile of this warpgroup
    const int r = (warp & 3) * 32 + lane;
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>((warp & 3) * 32) << 16);
    const int my_rows = q == 0 ? rows_q[0] : rows_q[1], my_first = q == 0 ? first_q[0] : first_q[1];
    const int ja = q == 0 ? a0 : a1, jb = q == 0 ? b0 : b1;
    const int my_pos = my_first + r;
    const float c_log2 = 1.4426950408889634f;
    // scores stay in the units the tensor core delivers; kf turns a difference of scores into a base-2 exponent
    const float kf = p.softcap > 0.f ? c_log2 : p.scale * c_log2;
    float m_run = -INFINITY, l_run = 0.f;
    bool ok = true;
    for (int j = ja; j < jb && ok; ++j) {
      const int t = j - ja;  // key tiles of this query tile so far
      const uint32_t slot = q * 2 + (t & 1);
      const uint32_t sb = lane_addr + kColS + slot * kAtBN;
      // warp-uniform: the loop holds warp-collective TMEM accesses
      ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&bar_s_full[slot]), (t >> 1) & 1, abort_flag, p.status));
      if (!ok) break;
      tc_fence_after();
      const int key_base = j * kAtBN;
      float f[kAtBN];
      {
        uint32_t* u = reinterpret_cast<uint32_t*>(f);
#pragma unroll
        for (int c = 0; c < kAtBN / 32; ++c) tmem_ld_x32(sb + c * 32, u + c * 32);
        tmem_ld_wait();
      }
      if (p.softcap > 0.f) {
        const float a = p.scale / p.softcap;
#pragma unroll
        for (int i = 0; i < kAtBN; ++i) f[i] = p.softcap * tanhf(f[i] * a);
      }
      // is the whole tile visible to all 128 rows? (row 0 sees the fewest late keys, row 127 the fewest early ones)
      const bool full = key_base + kAtBN <= min(ctx, p.causal ? my_first + 1 : ctx) && (p.window <= 0 || key_base >= my_first + kAtBM - p.window) &&
                        my_rows == kAtBM;
      if (!full) {
        // visible keys of this row inside the tile: [vlo, vhi)
        int vhi = min(ctx, p.causal ? my_pos + 1 : ctx) - key_base;
        int vlo = (p.window > 0 ? max(0, my_pos - p.window + 1) : 0) - key_base;
        if (r >= my_rows) vhi = vlo = 0;
#pragma unroll
        for (int i = 0; i < kAtBN; ++i) f[i] = (i >= vlo && i < vhi) ? f[i] : -INFINITY;
      }
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int i = 0; i < kAtBN; i += 8) {
        mx4[0] = fmax3(mx4[0], f[i], f[i + 1]);
        mx4[1] = fmax3(mx4[1], f[i + 2], f[i + 3]);
        mx4[2] = fmax3(mx4[2], f[i + 4], f[i + 5]);
        mx4[3] = fmax3(mx4[3], f[i + 6], f[i + 7]);
      }
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      // The running maximum only follows the scores when one of the warp's rows has outgrown it by more than 2^8: a stale
      // maximum costs nothing but head-room (probabilities up to 256), a new one costs a pass over the O accumulator.
      float m_new = m_run;
      if (t == 0) {
        m_new = mx;
      } else if (__any_sync(0xffffffffu, (mx - m_run) * kf > 8.f)) {
        m_new = fmaxf(m_run, mx);
        const float alpha = m_new == -INFINITY ? 1.f : ex2_approx((m_run - m_new) * kf);
        // P V of the previous key tile must have retired before the accumulator is touched (these scores were issued ahead of it)
        ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&bar_pv_done[q * 2 + ((t - 1) & 1)]), ((t - 1) >> 1) & 1, abort_flag, p.status));
        if (!ok) break;
        tc_fence_after();
#pragma unroll 1
        for (int c0 = 0; c0 < D; c0 += 32) {
          uint32_t v[32];
          tmem_ld_x32(lane_addr + kColO + q * D + c0, v);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
          tmem_st_x32(lane_addr + kColO + q * D + c0, v);
        }
        l_run *= alpha;
      }
      m_run = m_new;
      const float neg_mk = m_new == -INFINITY ? 0.f : -m_new * kf;
      // probabilities -> packed bf16 over the first half of the score slot's columns (every score is in registers by now)
      float ls4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int c = 0; c < kAtBN / 32; ++c) {
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
          const float p0 = ex2_approx(fmaf(f[c * 32 + i], kf, neg_mk)), p1 = ex2_approx(fmaf(f[c * 32 + i + 1], kf, neg_mk));
          const float p2 = ex2_approx(fmaf(f[c * 32 + i + 2], kf, neg_mk)), p3 = ex2_approx(fmaf(f[c * 32 + i + 3], kf, neg_mk));
          ls4[0] += p0;
          ls4[1] += p1;
          ls4[2] += p2;
          ls4[3] += p3;
          pk[i >> 1] = pack_bf162(p0, p1);
          pk[(i >> 1) + 1] = pack_bf162(p2, p3);
        }
        tmem_st_x16(sb + c * 16, pk);
      }
      l_run += (ls4[0] + ls4[1]) + (ls4[2] + ls4[3]);
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bar_p_full[slot]));
    }
    // ---------------- epilogue ----------------
    if (ok) ok = mbar_wait(smem_u32(bar_o_final), 0, abort_flag, p.status);
    ok = __all_sync(0xffffffffu, ok && *abort_flag == 0);
    if (ok) {
      tc_fence_after();
      const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
      __nv_bfloat16* orow = p.out + static_cast<size_t>(qs + q0 + q * kAtBM + r) * (static_cast<size_t>(p.H) * D) + static_cast<size_t>(h) * D;
#pragma unroll 1
      for (int c0 = 0; c0 < D; c0 += 32) {
        uint32_t v[32];
        if (jb > ja) {
          tmem_ld_x32(lane_addr + kColO + q * D + c0, v);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = 0u;
        }
        if (r < my_rows) {
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
  if (warp == kIssuer) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

template <int D, int QT>
static int launch_prefill_tc_t(const void* q, long long q_stride, long long T, const void* kc, const void* vc, long long cache_rows, const AttnTcParams& p,
                               int num_tiles, cudaStream_t st) {
  using L = AttnTcSmem<D, QT>;
  static PerDeviceOnce attr_once;
  if (attr_once.first()) {
    cudaError_t e = cudaFuncSetAttribute(prefill_attn_tc_kernel<D, QT>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kBytes);
    if (e != cudaSuccess) throw std::runtime_error(std::string("prefill attention (tcgen05): cudaFuncSetAttribute: ") + cudaGetErrorString(e));
  }
  CUtensorMap mq, mk, mv;
  encode_map_2d(&mq, 0, q, static_cast<uint64_t>(T), static_cast<uint64_t>(p.H) * D, static_cast<uint64_t>(q_stride) * 2, kAtBM, 64, 128);
  const uint32_t box_rows = p.page_size < kAtBN ? p.page_size : kAtBN;
  encode_map_2d(&mk, 0, kc, static_cast<uint64_t>(cache_rows), D, static_cast<uint64_t>(D) * 2, box_rows, 64, 128);
  encode_map_2d(&mv, 0, vc, static_cast<uint64_t>(cache_rows), D, static_cast<uint64_t>(D) * 2, box_rows, 64, 128);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(num_tiles, p.H);
  cfg.blockDim = dim3(L::kThreads);
  cfg.dynamicSmemBytes = L::kBytes;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = g_pdl_enabled ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, prefill_attn_tc_kernel<D, QT>, mq, mk, mv, p);
  if (e != cudaSuccess) throw std::runtime_error(std::string("prefill attention (tcgen05) launch: ") + cudaGetErrorString(e));
  return 0;
}

// Query rows one CTA of the tcgen05 prefill kernel covers: two 128-row tiles share the K / V tiles where their two accumulators fit
// tensor memory beside the two score slots.
int prefill_attention_tc_tile_rows(int D) { return D <= 128 ? 256 : 128; }

// tile arrays: prefill_attention_tc_tile_rows(D) query rows per tile. page_size must be 32, 64 or 128. Returns 1 for an unsupported head_dim / page size.
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
    case 64: return launch_prefill_tc_t<64, 2>(q, q_stride, T, kc, vc, cache_rows, p, num_tiles, st);
    case 128: return launch_prefill_tc_t<128, 2>(q, q_stride, T, kc, vc, cache_rows, p, num_tiles, st);
    case 256: return launch_prefill_tc_t<256, 1>(q, q_stride, T, kc, vc, cache_rows, p, num_tiles, st);
    default: return 1;
  }
}

}  // namespace dlv
