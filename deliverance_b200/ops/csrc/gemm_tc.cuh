// tcgen05 / TMEM GEMM for  out[m, n] = sum_k X[m, k] * W[n, k]  (+ bias[n]).
//
// The weight matrix is the MMA "A" operand (128 weight rows per CTA = UMMA M), the activations are the "B" operand
// (BN tokens = UMMA N, 16..256), so that decode batches of 1..64 tokens still fill a full-height tensor-core tile and
// the kernel is weight-bandwidth bound.
//
// JQ4 weights: packed nibbles + per-32 fp32 scales are pre-arranged at load time as one contiguous 10 KB chunk per
// 128x128 tile, so a pipeline stage is a single bulk copy of consecutive DRAM bytes into a deep staging ring (up to 16
// stages per SM). Sixteen warps expand a stage to bf16 ((nibble - 8) * scale) in registers and write it with tcgen05.st
// straight into TENSOR MEMORY, from where tcgen05.mma reads its A operand: the dequantised weights never touch shared
// memory, whose bandwidth (128 B/clk) would otherwise cap the kernel at about half of the HBM rate (a bf16 tile in shared
// memory costs a 32 KB write plus a 32 KB tensor-core read per 10 KB of HBM traffic). Activations stream through their
// own TMA ring. Dense bf16 weights take the classic path (TMA into 128B-swizzled tiles, both operands from shared memory).
//
// Split-K: the CTAs that share an output tile form a thread-block cluster (<= 8). Each writes its fp32 partial tile to
// its own shared memory, and after a cluster barrier every CTA reduces a slice of the tile's columns by reading all
// peers' partials through distributed shared memory in a fixed order (deterministic), then writes the final output.
// A global-memory workspace + last-arriver reduction remains as the fallback when clusters cannot be scheduled.
//
// Tensor-parallel fusion (row-parallel o_proj / down_proj, decode batches): instead of writing its tile to the output, a
// CTA stores its partial sums as bf16 straight into the receive area of EVERY rank (plain peer stores over NVLink, own rank
// included), publishes them with one release-add per rank on that rank's flag matrix, waits (bounded) until all ranks have
// published the same tile to it, and only then sums the tp_size partials in rank order and writes the final output: GEMM
// and one-shot all-reduce are one kernel, and the transfer of finished tiles overlaps the math of the others. Receive
// areas are double-buffered on the parity of a per-rank launch counter; flags are cumulative, so CUDA-graph replays need
// no host-side reset.
//
// Roles per CTA (768 threads): warps 0 + 19 = weight producers (TMA, alternate k-blocks), warp 1 = TMEM owner, warps 1 + 21..23 =
// MMA issuers (alternate k-blocks, one accumulator each),
// warps 2 + 20 = activation TMA producers, warps 3..18 = JQ4 dequant (one 32-element block per thread and stage) and epilogue
// (tcgen05.ld -> fp32 tile in shared memory -> reduce over the cluster -> 8/16-byte global stores).
//
// Epilogue variants (template EPI): 0 = store (+ bias, + the tensor-parallel sum above); 1 = gated activation for gate|up weights whose
// rows are interleaved per 64 outputs (act(gate) * up, half as many output columns); 2 = q|k|v heads of dimension 128: per-head
// RMSNorm, rotary embedding and the paged KV-cache write happen on the staged tile, only the query heads are written to `out`;
// 3 = reduce-scatter over the tensor-parallel ranks: the partial tile is stored into the receive area of the rank that owns its
// token rows and published with one release-add; no CTA waits, the reduction is a separate kernel (comm.cu); 4 = store as in 0, but
// the activation producers first wait until the ranks that own the tile's token rows have pushed them into the local gather area
// (all-gather -> GEMM: the weight stream and the other tiles run under the transfer).
//
// This replaces the reference's CPU kernels gemm_q8_q4 / gemm_bf16_q4 / gemm_bf16
// (native/src/main/c/simd/vector_simd.c:339-633,1186-1411,1414-1668) and the WGSL gemm_q4 / gemm_i8q4_v5 shaders.
#pragma once
#include "common.cuh"

namespace dlv {

constexpr int kGemmBM = 128;       // weight rows per CTA
constexpr int kGemmBK = 128;       // reduction elements per pipeline stage
constexpr int kGemmThreads = 768;  // 24 warps
constexpr int kGemmEpiThreads = 512;
constexpr int kGemmEpiWarp0 = 3;
constexpr int kGemmTmemCols = 512;   // whole tensor memory of the SM (one CTA per SM)
constexpr int kGemmTmemAStage = 64;  // 128 k as bf16 pairs

struct GemmParams {
  int M, N, K;
  int kb_total;      // ceil(K / 128)
  int splits;        // split-K factor (>= 1)
  int kb_per_split;  // k-blocks handled by one split
  int n_tiles, m_tiles;
  int cluster_reduce;  // 1: the splits of a tile are one cluster and reduce through distributed shared memory
  void* out;           // [M, ldo] bf16 or fp32
  int ldo;
  int out_f32;
  const float* bias;  // [N] fp32 or nullptr
  const uint8_t* wq;  // JQ4: tile-packed weights [n_tiles][kb_total][10240 B] (see gemm_api.h), else nullptr
  float* ws;          // fallback split-K partials: [tile][split][BN][128] fp32
  int* counters;      // fallback: one per tile, zero between launches (the reducing CTA resets its counter)
  int* status;        // kernel status word (0 = ok)
  // ---- fused tensor-parallel all-reduce (tp_size > 1): see the epilogue ----
  int tp_size, tp_rank;
  int tp_ncta_max;                 // row length of the flag matrix
  long long tp_slab;               // elements per (parity, source) slab of the receive area
  unsigned long long tp_recv[8];   // every rank's receive area (bf16 [2][tp_size][slab]), peer-mapped
  unsigned long long tp_flags[8];  // every rank's flag matrix (u32 [tp_size][tp_ncta_max], cumulative counters)
  unsigned int* tp_rounds;         // local: how many fused calls each CTA index has completed
  unsigned int* tp_call;           // local: [0] = number of fused launches completed, [1] = CTAs done in this launch
  int tp_mode;                     // 0: publish, wait and reduce here; 1: publish to every rank and leave; 2: publish to the own slab and leave
  // ---- grouped (mixture-of-experts) mode: blockIdx.y indexes a work list instead of a token tile ----
  // item = {expert, first row, end row, 0}; expert < 0 marks an unused slot (the CTA returns at once). The weights of all
  // local experts are stacked (JQ4: n_tiles tile rows per expert, dense: N rows per expert); N / n_tiles are per expert.
  const int4* grp_items;
  // ---- tail split: CTAs with blockIdx.x >= tail_tile0 share the last tiles `tail_splits` ways (workspace reduction), so that a
  // grid a few tiles larger than the SM count ends with a short second wave instead of a full one (host: splits == 1) ----
  int tail_tile0, tail_splits, tail_kb_per_split;
  int x3d, w3d;  // the activation / dense weight map is the 3-D chunked form: one copy per stage instead of two
  // ---- gated activation in the epilogue (kernel template ACT): the weight rows of a tile are 64 gate rows followed by the 64 up
  // rows of the same outputs (interleaved at load time); out[m, 64 * tile + r] = act(gate) * up, ldo counts N / 2 columns ----
  int act_kind;  // 1: SiLU, 2: tanh-approximated GELU
  // ---- q | k | v projection with per-head RMSNorm, rotary embedding and the paged KV write in the epilogue (kernel template
  // EPI = 2; head_dim must be 128 so that one weight tile is one head): tiles 0 .. H-1 are query heads (written to out [M, H * 128]),
  // the next KV tiles key heads (normalised, rotated, written to k_cache), the last KV tiles value heads (copied to v_cache) ----
  const int* qk_positions;         // [M]
  const long long* qk_slots;       // [M] flat cache row (block * block_size + offset), < 0: no cache write
  const __nv_bfloat16* q_norm_w;   // [128] or nullptr
  const __nv_bfloat16* k_norm_w;   // [128] or nullptr
  const float* qk_cos;             // [max_pos, rot_half] or nullptr (no rotation)
  const float* qk_sin;
  __nv_bfloat16* k_cache;          // [blocks, KV, block_size, 128]
  __nv_bfloat16* v_cache;
  int qk_heads, qk_kv_heads, qk_block_size, qk_rot_half, qk_max_pos;
  float qk_eps, qk_norm_offset;
  // ---- GEMM -> reduce-scatter (kernel template EPI = 3, prefill-size batches): token rows [r * tp_rows, (r + 1) * tp_rows) belong to
  // rank r. The partial tile goes row by row as bf16 to the owner's receive area tp_recv[owner] = [tp_size sources][tp_rows][N]
  // (plain peer stores) and one release-add per CTA and owner on tp_flags[owner][tp_rank] publishes it. Nothing waits in this kernel, so the grid may be any number of waves; comm.cu reduces and gathers. ----
  int tp_rows;
  // ---- all-gather -> GEMM (kernel template EPI = 4): the activation map covers this rank's gather area [M][K], into which every
  // rank pushes the rows it owns (rows [r * ag_rows, (r + 1) * ag_rows) come from rank r) and then adds to ag_flags[r] (local,
  // cumulative). The activation producers wait (bounded) until the owners of their token tile have reached ag_targets[] ----
  const uint32_t* ag_flags;
  unsigned int ag_targets[8];
  int ag_rows;
};

static_assert(sizeof(GemmParams) + 2 * 128 <= 4096, "kernel parameters (two tensor maps + GemmParams) must fit the 4 KB parameter space");

template <bool Q4, int BN>
struct GemmSmem {
  static constexpr int kWTile = kGemmBM * 128;  // dense: one 64-wide bf16 sub-tile of W: 16 KB
  static constexpr int kWStage = 2 * kWTile;    // dense: 32 KB
  static constexpr int kXStage = BN * 256;      // two 64-wide bf16 sub-tiles of X
  static constexpr int kRawStage = kGemmBM * 64 + kGemmBM * 16;  // packed nibbles (8 KB) + scales (2 KB)
  static constexpr int kBudget = 232448 - 2048;                  // dynamic smem minus barriers / alignment slack
  static constexpr int kStageOut = BN * kGemmBM * 4;             // fp32 output staging tile (aliases the rings)
  // Ring depths. Every ring is shared by several producers and several consumers that take alternate k-blocks (two copy
  // warps, four dequant groups, kNI MMA issuers). mbarrier waits only know the PARITY of a phase, so a thread must see every
  // phase of the barriers it waits on: each ring depth is a multiple of the number of its producers and of its consumers,
  // which ties every stage to one producer and one consumer for the whole kernel.
  static constexpr int kNI = BN <= 64 ? 4 : (BN == 128 ? 2 : 1);  // MMA-issuing warps (see the issuer loop)
  // Issuers that add into ONE accumulator (the only way to have several at BN = 256, where tensor memory has no room for a second
  // accumulator) are written out below but not used: they changed nothing measurable there, and the order in which two racing
  // issuers' k-blocks reach the accumulator varies from launch to launch, so results were not bit-reproducible.
  static constexpr bool kSharedAcc = false;
  static constexpr int kNW = Q4 ? 0 : (BN <= 64 ? 4 : 2);         // dense: W and X rings of equal depth
  static constexpr int kAccCols = kSharedAcc ? BN : kNI * BN;
  static constexpr int kTmemA = kAccCols < 64 ? 64 : kAccCols;  // JQ4: the A-operand ring in tensor memory follows the accumulators
  static constexpr int kNA = 4;                                  // one stage per dequant group
  static constexpr int kNX = Q4 ? (BN <= 32 ? 8 : (BN <= 128 ? 4 : 2)) : kNW;
  static constexpr int kRawRoom = Q4 ? (kBudget - kNX * kXStage) / kRawStage : 0;
  static constexpr int kNR = Q4 ? (kRawRoom >= 16 ? 16 : (kRawRoom >= 12 ? 12 : (kRawRoom >= 8 ? 8 : 4))) : 0;
  static constexpr int kOffX = kNW * kWStage;
  static constexpr int kOffRaw = kOffX + kNX * kXStage;
  static constexpr int kOffCtrl = kOffRaw + kNR * kRawStage;
  static constexpr int kBytes = kOffCtrl + 2048;
  static_assert(!Q4 || kNR >= 4, "packed-weight ring too small");
  static_assert(kNX >= 2, "activation ring too small");
  static_assert(kStageOut <= kOffCtrl, "the fp32 output staging tile must fit in the rings");
  static_assert(kNX % kNI == 0 && kNX % 2 == 0 && (Q4 || kNW % kNI == 0) && (!Q4 || (kNR % 4 == 0 && kNA % kNI == 0)), "ring ownership");
  static_assert(Q4 || (kNW * (kWStage + kXStage) <= kBudget), "dense rings do not fit");
  static_assert(!Q4 || kRawRoom >= kNR, "packed ring does not fit");
  static_assert(kTmemA + kNA * kGemmTmemAStage <= kGemmTmemCols && kAccCols <= kTmemA, "tensor memory plan");
};

__device__ __forceinline__ uint32_t q4_pair_to_bf162(uint32_t nib4, uint32_t sel, __nv_bfloat162 s2) {
  // bytes of nib4 are nibbles (0..15); build two bf16 values 128 + q, subtract 136 exactly, scale.
  uint32_t u = __byte_perm(nib4, 0x43434343u, sel);
  __nv_bfloat162 v = *reinterpret_cast<__nv_bfloat162*>(&u);
  const __nv_bfloat162 off = __floats2bfloat162_rn(136.f, 136.f);
  v = __hmul2(__hsub2(v, off), s2);
  return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ float4 ld_dsmem_f32x4(uint32_t local_addr, uint32_t cta_rank) {
  uint32_t remote;
  float4 v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(cta_rank));
  asm volatile("ld.shared::cluster.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(remote) : "memory");
  return v;
}

// EPI selects the epilogue: 0 = plain store (+ bias, + fused tensor-parallel sum), 1 = gated activation, 2 = q/k norm + rotary + KV write
template <bool Q4, int BN, int EPI = 0>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_w,   // dense: bf16 [N, K] (unused for JQ4, which streams p.wq)
               const __grid_constant__ CUtensorMap map_x,   // bf16 [M, K]
               const GemmParams p) {
  using L = GemmSmem<Q4, BN>;
  constexpr bool ACT = EPI == 1, QKV = EPI == 2, SCAT = EPI == 3;
  constexpr int NW = L::kNW > 0 ? L::kNW : 1, NX = L::kNX, NR = L::kNR > 0 ? L::kNR : 1, NA = L::kNA, NI = L::kNI;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* ctrl = smem + L::kOffCtrl;
  // "a" barriers: the MMA A operand stage (dense: bf16 tile in shared memory, JQ4: bf16 columns in tensor memory)
  uint64_t* bar_a_full = reinterpret_cast<uint64_t*>(ctrl);
  uint64_t* bar_a_empty = bar_a_full + 8;
  uint64_t* bar_x_full = bar_a_empty + 8;
  uint64_t* bar_x_empty = bar_x_full + NX;
  uint64_t* bar_r_full = bar_x_empty + NX;
  uint64_t* bar_r_empty = bar_r_full + NR;
  uint64_t* bar_acc = bar_r_empty + NR;
  uint64_t* bar_first = bar_acc + 1;  // shared accumulator: its first k-block (the one that overwrites) has retired
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_first + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* s_last = const_cast<int*>(abort_flag) + 1;
  constexpr int NAS = Q4 ? NA : NW;  // depth of the A-operand ring

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int n_tile = blockIdx.x, split = blockIdx.z;
  const int m_tile = blockIdx.y;
  int splits = p.splits, kb_per_split = p.kb_per_split, ws_tile = m_tile * p.n_tiles + blockIdx.x;
  if (p.tail_splits > 1 && static_cast<int>(blockIdx.x) >= p.tail_tile0) {
    const int j = static_cast<int>(blockIdx.x) - p.tail_tile0;
    n_tile = p.tail_tile0 + j / p.tail_splits;
    split = j % p.tail_splits;
    splits = p.tail_splits;
    kb_per_split = p.tail_kb_per_split;
    ws_tile = j / p.tail_splits;
  }
  const int n0 = n_tile * kGemmBM;
  int m0 = m_tile * BN, m_lim = p.M, w_tile = n_tile, w_row0 = n0;
  if (p.grp_items != nullptr) {
    pdl_wait();  // the work list is written by the kernels in front of this one
    const int4 it = p.grp_items[blockIdx.y];
    if (it.x < 0) return;  // uniform over the cluster (its CTAs differ in blockIdx.z only); nothing is set up yet
    m0 = it.y;
    m_lim = it.z;
    w_tile = it.x * p.n_tiles + n_tile;
    w_row0 = it.x * p.N + n0;
  }
  const int kb_begin = split * kb_per_split;
  const int kb_end = min(p.kb_total, kb_begin + kb_per_split);
  const int nkb = max(0, kb_end - kb_begin);
  constexpr uint32_t TMEM_COLS = Q4 ? kGemmTmemCols : (L::kAccCols < 32 ? 32 : L::kAccCols);
  // Every CTA walks its k-blocks from a different starting point: CTAs that run at the same time would otherwise all ask
  // the L2 for the same activation lines at the same moment (the activation tile of a k-block is shared by every weight
  // tile), and requests to one line are served one after the other.
  const int rot = nkb > 0 ? static_cast<int>((static_cast<unsigned>(n_tile) * 7u + static_cast<unsigned>(m_tile) * 3u) % static_cast<unsigned>(nkb)) : 0;

  auto w_tile_ptr = [&](int s, int sub) { return smem + s * L::kWStage + sub * L::kWTile; };
  auto x_tile = [&](int s, int sub) { return smem + L::kOffX + s * L::kXStage + sub * (BN * 128); };
  auto raw_tile = [&](int s) { return smem + L::kOffRaw + s * L::kRawStage; };
  auto sc_tile = [&](int s) { return smem + L::kOffRaw + s * L::kRawStage + kGemmBM * 64; };

  if (threadIdx.x == 0) {
    for (int s = 0; s < NAS; ++s) {
      mbar_init(smem_u32(&bar_a_full[s]), Q4 ? 4 : 1);  // JQ4: one arrival per warp of the group that owns the stage
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
    mbar_init(smem_u32(bar_acc), NI);
    mbar_init(smem_u32(bar_first), 1);
    *abort_flag = 0;
    *s_last = 0;
    mbar_fence_init();
    tma_prefetch_desc(&map_w);
    tma_prefetch_desc(&map_x);
  }
  pdl_trigger();  // kernels behind this one may be scheduled as soon as every CTA of this grid has started
  if (warp == 1) tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // A single thread can only issue one bulk / tensor copy about every 0.3 us, whatever the size of the copy. So every stage
  // is ONE copy, and two warps per operand take alternate k-blocks (warps 0 + 19: weights, warps 2 + 20: activations).
  if (warp == 0 || warp == 19) {
    // ---------------- weight producers: packed JQ4 stages (deep ring) or dense bf16 tiles ----------------
    if (lane == 0) {
      constexpr int RING = Q4 ? NR : NW;
      const int first_i = warp == 0 ? 0 : 1;
      int last_issued = -1, n_issued = 0;
      for (int i = first_i; i < nkb; i += 2) {
        const int s = i % RING;
        const uint32_t ph = (i / RING) & 1;
        uint64_t* empty = Q4 ? &bar_r_empty[s] : &bar_a_empty[s];
        uint64_t* fullb = Q4 ? &bar_r_full[s] : &bar_a_full[s];
        if (!mbar_wait(smem_u32(empty), ph ^ 1, abort_flag, p.status)) break;
        const uint32_t full = smem_u32(fullb);
        const int kb = kb_begin + (i + rot >= nkb ? i + rot - nkb : i + rot);
        if (Q4) {
          // one contiguous 10 KB stage: 8 KB of packed nibbles (already in the swizzled shared-memory order) + 2 KB of scales
          mbar_expect_tx(full, L::kRawStage);
          tma_load_2d(smem_u32(raw_tile(s)), &map_w, full, 0, (w_tile * p.kb_total + kb) * 10);
        } else {
          mbar_expect_tx(full, L::kWStage);
          if (p.w3d) {
            tma_load_3d(smem_u32(w_tile_ptr(s, 0)), &map_w, full, 0, w_row0, kb * 2);
          } else {
            tma_load_2d(smem_u32(w_tile_ptr(s, 0)), &map_w, full, kb * kGemmBK, w_row0);
            tma_load_2d(smem_u32(w_tile_ptr(s, 1)), &map_w, full, kb * kGemmBK + 64, w_row0);
          }
        }
        last_issued = i;
        ++n_issued;
      }
      if (*abort_flag) {
        // let copies that are still in flight land before the CTA goes away (bounded: ~20 ms per stage)
        const int keep = n_issued < (RING + 1) / 2 ? n_issued : (RING + 1) / 2;
        for (int j = 0; j < keep; ++j) {
          const int i = last_issued - 2 * j;
          const uint32_t bar = smem_u32(Q4 ? &bar_r_full[i % RING] : &bar_a_full[i % RING]);
          const uint32_t ph = (i / RING) & 1;
          const unsigned long long t0 = globaltimer_ns();
          while (!mbar_try_wait(bar, ph) && globaltimer_ns() - t0 < 20000000ull) {
          }
        }
      }
    }
  } else if (warp == 2 || warp == 20) {
    // ---------------- activation producers ----------------
    if (lane == 0) {
      // Launched with programmatic stream serialization, this kernel may run its prologue and stream weights while the kernel
      // that produces the activations is still finishing; nothing that kernel wrote is read before this point.
      pdl_wait();
      bool ag_ok = true;
      if constexpr (EPI == 4) {
        // all-gather prologue: the rows of this token tile arrive from their owners by peer stores; weights stream meanwhile
        const int o_lo = m0 / p.ag_rows, o_hi = (min(m0 + BN, m_lim) - 1) / p.ag_rows;
        for (int o = o_lo; o <= o_hi; ++o) {
          if (!flag_wait_ge(p.ag_flags + o, p.ag_targets[o], p.status)) {
            *abort_flag = 1;  // nothing is copied; the other roles leave through their own bounded waits
            ag_ok = false;
            break;
          }
        }
        fence_proxy_async_all();
      }
      const int first_i = warp == 2 ? 0 : 1;
      int last_issued = -1, n_issued = 0;
      for (int i = first_i; i < nkb && ag_ok; i += 2) {
        const int s = i % NX;
        const uint32_t ph = (i / NX) & 1;
        if (!mbar_wait(smem_u32(&bar_x_empty[s]), ph ^ 1, abort_flag, p.status)) break;
        const uint32_t full = smem_u32(&bar_x_full[s]);
        const int kb = kb_begin + (i + rot >= nkb ? i + rot - nkb : i + rot);
        mbar_expect_tx(full, L::kXStage);
        if (p.x3d) {
          tma_load_3d(smem_u32(x_tile(s, 0)), &map_x, full, 0, m0, kb * 2);
        } else {
          tma_load_2d(smem_u32(x_tile(s, 0)), &map_x, full, kb * kGemmBK, m0);
          tma_load_2d(smem_u32(x_tile(s, 1)), &map_x, full, kb * kGemmBK + 64, m0);
        }
        last_issued = i;
        ++n_issued;
      }
      if (*abort_flag) {
        const int keep = n_issued < (NX + 1) / 2 ? n_issued : (NX + 1) / 2;
        for (int j = 0; j < keep; ++j) {
          const int i = last_issued - 2 * j;
          const uint32_t bar = smem_u32(&bar_x_full[i % NX]);
          const uint32_t ph = (i / NX) & 1;
          const unsigned long long t0 = globaltimer_ns();
          while (!mbar_try_wait(bar, ph) && globaltimer_ns() - t0 < 20000000ull) {
          }
        }
      }
    }
  } else if (warp == 1 || warp >= 21) {
    // ---------------- MMA issuers ----------------
    // A tcgen05.mma holds its thread until the tensor pipe accepts it, the pipe queues next to nothing, and a wait on an mbarrier,
    // even a complete one, costs the thread a few hundred cycles: a single issuer leaves the pipe idle between k-blocks (measured:
    // groups of 8 MMAs of 128 x 128 x 16 back to back 517 cycles per group, with one satisfied wait between groups 783). NI warps
    // therefore take alternate k-blocks, so that one feeds the pipe while another waits: each into its own accumulator (columns
    // j*BN .., added up by the epilogue), or, where tensor memory has no room for that (BN = 256), all into one. (For the JQ4 prefill
    // shapes the second issuer of BN = 256 changed nothing measurable: there the prologue and epilogue of the one-tile-per-CTA design, not the issuer, leave the tensor pipe idle.) The
    // whole warp follows the barriers, one lane issues.
    const int issuer = warp == 1 ? 0 : warp - 20;
    if (issuer < NI) {
      constexpr uint32_t idesc = umma_idesc_bf16(kGemmBM, BN);
      const uint64_t desc_w0 = umma_desc_k_sw128(smem_u32(smem));
      const uint64_t desc_x0 = umma_desc_k_sw128(smem_u32(smem + L::kOffX));
      const uint32_t tmem_acc = tmem_base + (L::kSharedAcc ? 0 : issuer * BN);
      bool ok = true;
      for (int i = issuer; i < nkb; i += NI) {
        const int sa = i % NAS, sx = i % NX;
        ok = mbar_wait(smem_u32(&bar_a_full[sa]), (i / NAS) & 1, abort_flag, p.status);
        ok = ok && mbar_wait(smem_u32(&bar_x_full[sx]), (i / NX) & 1, abort_flag, p.status);
        // one accumulator for all issuers: the others only add, and not before the k-block that overwrites it has retired
        if (L::kSharedAcc && issuer > 0 && i == issuer) ok = ok && mbar_wait(smem_u32(bar_first), 0, abort_flag, p.status);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        if (lane == 0) {
          // descriptor start-address field counts 16-byte units: stage strides and the 32-byte k-step are added there
          const uint64_t dx = desc_x0 + static_cast<uint64_t>((sx * L::kXStage) >> 4);
#pragma unroll
          for (int k4 = 0; k4 < 8; ++k4) {
            const int sub = k4 >> 2, kk = k4 & 3;
            const uint64_t db = dx + static_cast<uint64_t>((sub * (BN * 128) + kk * 32) >> 4);
            const uint32_t acc = ((L::kSharedAcc ? i > 0 : i >= NI) || k4 > 0) ? 1u : 0u;
            if (Q4) {
              umma_bf16_ts(tmem_acc, tmem_base + L::kTmemA + sa * kGemmTmemAStage + k4 * 8, db, idesc, acc);
            } else {
              const uint64_t da = desc_w0 + static_cast<uint64_t>((sa * L::kWStage + sub * L::kWTile + kk * 32) >> 4);
              umma_bf16(tmem_acc, da, db, idesc, acc);
            }
          }
          umma_commit(smem_u32(&bar_a_empty[sa]));
          umma_commit(smem_u32(&bar_x_empty[sx]));
          if (L::kSharedAcc && i == 0) umma_commit(smem_u32(bar_first));
        }
        __syncwarp();
      }
      if (lane == 0) {
        umma_commit(smem_u32(bar_acc));  // one arrival per issuer
        if (!ok) {
          // outstanding MMAs must retire before TMEM is released
          const unsigned long long t0 = globaltimer_ns();
          while (!mbar_try_wait(smem_u32(bar_acc), 0) && globaltimer_ns() - t0 < 20000000ull) {
          }
        }
      }
      __syncwarp();
    }
  } else if (warp >= kGemmEpiWarp0 && warp < kGemmEpiWarp0 + 16) {
    // ---------------- dequant + epilogue warps (512 threads) ----------------
    const int t = threadIdx.x - kGemmEpiWarp0 * 32;
    const int we = warp - kGemmEpiWarp0;
    const int q = warp & 3;  // tensor-memory lane quarter this warp may access
    bool ok = true;
    if (Q4) {
      // The 16 warps form 4 groups; group g expands the k-blocks i = g, g + 4, ... so that four stages are in flight at
      // once (one warp iteration is a chain of long-latency steps: shared-memory loads, conversion, tcgen05.st and its
      // wait). Inside a group warp `q` owns rows 32q .. 32q+31 (its tensor-memory lane quarter) and all four 32-element
      // blocks of the stage.
      const int grp4 = we >> 2;
      const int r = q * 32 + lane;
      for (int i = grp4; i < nkb; i += 4) {
        const int sr = i % NR, sa = i % NA;
        if (!mbar_wait(smem_u32(&bar_r_full[sr]), (i / NR) & 1, abort_flag, p.status)) { ok = false; break; }
        uint4 wq[4];
#pragma unroll
        for (int b = 0; b < 4; ++b) wq[b] = *reinterpret_cast<const uint4*>(raw_tile(sr) + r * 64 + ((b ^ ((r >> 1) & 3)) << 4));
        const float4 sc4 = *reinterpret_cast<const float4*>(sc_tile(sr) + r * 16);
        const float sc[4] = {sc4.x, sc4.y, sc4.z, sc4.w};
        // the tensor-memory stage is free once the MMAs of k-block i - NA have retired
        if (!mbar_wait(smem_u32(&bar_a_empty[sa]), ((i / NA) & 1) ^ 1, abort_flag, p.status)) { ok = false; break; }
        tc_fence_after();
        const uint32_t tdst = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + L::kTmemA + sa * kGemmTmemAStage;
#pragma unroll
        for (int b = 0; b < 4; ++b) {
          const __nv_bfloat162 s2 = __float2bfloat162_rn(sc[b]);
          const uint32_t words[4] = {wq[b].x, wq[b].y, wq[b].z, wq[b].w};
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
          tmem_st_x16(tdst + b * 16, o);
        }
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(smem_u32(&bar_r_empty[sr]));
          mbar_arrive(smem_u32(&bar_a_full[sa]));
        }
      }
    }
    pdl_wait();  // global memory is written (and the peer-memory bookkeeping read) only after the predecessor grid is complete
    // ---- accumulator -> fp32 tile [col][row] in shared memory (the rings are idle once the MMAs retired) ----
    if (ok) ok = mbar_wait(smem_u32(bar_acc), 0, abort_flag, p.status);
    // All 512 threads reach this barrier; afterwards the abort flag gives a CTA-uniform decision (it is only ever
    // raised before the accumulator barrier can complete), so the named barriers below never miss a thread.
    asm volatile("bar.sync 1, 512;" ::: "memory");
    ok = (*abort_flag == 0);
    if (ok) {
      tc_fence_after();
      constexpr int GROUPS = BN >= 32 ? 4 : BN / 8;  // warps that share a quarter split the columns
      constexpr int COLS = BN / GROUPS;
      constexpr int CH = COLS >= 16 ? 16 : 8;
      const int grp = we >> 2;
      if (grp < GROUPS) {
        const int row = q * 32 + lane;
        const uint32_t taddr0 = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + grp * COLS;
        float* stage = reinterpret_cast<float*>(smem);
#pragma unroll 1
        const int nacc = L::kSharedAcc ? 1 : (nkb < NI ? nkb : NI);  // issuers without a k-block never wrote their accumulator
        for (int c0 = 0; c0 < COLS; c0 += CH) {
          float sum[CH];
#pragma unroll
          for (int j = 0; j < CH; ++j) sum[j] = 0.f;
          for (int a = 0; a < nacc; ++a) {
            uint32_t v[CH];
            if constexpr (CH == 16) tmem_ld_x16(taddr0 + a * BN + c0, v); else tmem_ld_x8(taddr0 + a * BN + c0, v);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < CH; ++j) sum[j] += __uint_as_float(v[j]);
          }
#pragma unroll
          for (int j = 0; j < CH; ++j) stage[(grp * COLS + c0 + j) * kGemmBM + row] = sum[j];
        }
      }
    }
    if (splits == 1 || !p.cluster_reduce) asm volatile("bar.sync 1, 512;" ::: "memory");
  }
  // ---------------- reduce over the split-K cluster (distributed shared memory) and store ----------------
  const bool clustered = splits > 1 && p.cluster_reduce;
  if (clustered) cluster_sync_all();  // every CTA of the cluster has its partial tile in shared memory (or is aborting)
  if (warp >= kGemmEpiWarp0 && warp < kGemmEpiWarp0 + 16 && *abort_flag == 0) {
    const int t = threadIdx.x - kGemmEpiWarp0 * 32;
    const int row4 = (t & 31) * 4, csel = t >> 5;  // 4 consecutive weight rows, column slot 0..15
    const int n = n0 + row4;
    const float* stage = reinterpret_cast<const float*>(smem);
    const uint32_t stage_addr = smem_u32(smem);
    if (splits > 1 && !p.cluster_reduce) {
      // fallback: partial tiles through the global workspace, the last CTA to arrive reduces in split order
      const int tile_id = ws_tile;
      float* part = p.ws + (static_cast<size_t>(tile_id) * splits + split) * (BN * kGemmBM);
      for (int col = csel; col < BN; col += 16)
        *reinterpret_cast<float4*>(part + col * kGemmBM + row4) = *reinterpret_cast<const float4*>(stage + col * kGemmBM + row4);
      __threadfence();
      asm volatile("bar.sync 1, 512;" ::: "memory");
      if (t == 0) {
        const int old = atomicAdd(&p.counters[tile_id], 1);
        *s_last = (old == splits - 1) ? 1 : 0;
      }
      asm volatile("bar.sync 1, 512;" ::: "memory");
      if (*s_last) __threadfence();
    }
    const bool do_store = splits == 1 || p.cluster_reduce || *s_last;
    const bool fused_tp = p.tp_size > 1;
    const uint32_t me = clustered ? cluster_ctarank() : 0u;
    const int stride = clustered ? splits : 1;
    const bool vec_ok = (n + 3 < p.N) && ((p.ldo & 3) == 0);
    // reduced (over split-K) accumulator of column `col`, rows row4 .. row4+3
    auto column_acc = [&](int col) -> float4 {
      float4 acc;
      if (clustered) {
        acc = make_float4(0.f, 0.f, 0.f, 0.f);
        const uint32_t a = stage_addr + static_cast<uint32_t>((col * kGemmBM + row4) * 4);
        for (int sp = 0; sp < splits; ++sp) {
          const float4 v = ld_dsmem_f32x4(a, static_cast<uint32_t>(sp));
          acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
      } else if (splits > 1) {
        acc = make_float4(0.f, 0.f, 0.f, 0.f);
        const float* base = p.ws + static_cast<size_t>(ws_tile) * splits * (BN * kGemmBM);
        for (int sp = 0; sp < splits; ++sp) {
          const float4 v = __ldcg(reinterpret_cast<const float4*>(base + (static_cast<size_t>(sp) * BN + col) * kGemmBM + row4));
          acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
      } else {
        acc = *reinterpret_cast<const float4*>(stage + col * kGemmBM + row4);
      }
      return acc;
    };
    auto store_out = [&](int m, float4 acc) {
      const size_t o = static_cast<size_t>(m) * p.ldo + n;
      if (vec_ok) {
        if (p.out_f32) *reinterpret_cast<float4*>(reinterpret_cast<float*>(p.out) + o) = acc;
        else {
          uint2 pk;
          pk.x = pack_bf162(acc.x, acc.y);
          pk.y = pack_bf162(acc.z, acc.w);
          *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(p.out) + o) = pk;
        }
      } else {
        const float vals[4] = {acc.x, acc.y, acc.z, acc.w};
        for (int e = 0; e < 4; ++e) {
          if (n + e < p.N) {
            if (p.out_f32) reinterpret_cast<float*>(p.out)[o + e] = vals[e];
            else reinterpret_cast<__nv_bfloat16*>(p.out)[o + e] = f2bf(vals[e]);
          }
        }
      }
    };
    float4 bias = make_float4(0.f, 0.f, 0.f, 0.f);
    if (p.bias != nullptr) {
      bias.x = n + 0 < p.N ? p.bias[n + 0] : 0.f;
      bias.y = n + 1 < p.N ? p.bias[n + 1] : 0.f;
      bias.z = n + 2 < p.N ? p.bias[n + 2] : 0.f;
      bias.w = n + 3 < p.N ? p.bias[n + 3] : 0.f;
    }
    if constexpr (QKV) {
      // ---- q | k | v heads: this tile is one head of 128 dims; a warp (32 lanes x 4 dims) holds a whole head of one token ----
      // (host guarantees: head_dim 128, no tensor-parallel fusion; the column loop is warp-uniform, so the shuffles below are safe)
      if (do_store) {
        const int lane_e = t & 31;
        const int head = n_tile;
        const bool is_q = head < p.qk_heads, is_k = !is_q && head < p.qk_heads + p.qk_kv_heads;
        const int kvh = is_q ? 0 : (is_k ? head - p.qk_heads : head - p.qk_heads - p.qk_kv_heads);
        const __nv_bfloat16* nw = is_q ? p.q_norm_w : (is_k ? p.k_norm_w : nullptr);
        float nwv[4] = {0.f, 0.f, 0.f, 0.f};
        if (nw != nullptr) {
#pragma unroll
          for (int e = 0; e < 4; ++e) nwv[e] = bf2f(nw[row4 + e]) + p.qk_norm_offset;
        }
        const bool rotate = (is_q || is_k) && p.qk_cos != nullptr;
        const int dpair = row4 & 63;  // index of this thread's first dim inside its half
        for (int col = static_cast<int>(me) + stride * csel; col < BN; col += stride * 16) {
          const int m = m0 + col;
          if (m >= m_lim) break;
          const float4 a4 = column_acc(col);
          float v[4] = {a4.x + bias.x, a4.y + bias.y, a4.z + bias.z, a4.w + bias.w};
          if (nw != nullptr) {
            float ss = v[0] * v[0] + v[1] * v[1] + v[2] * v[2] + v[3] * v[3];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            const float inv = rsqrtf(ss * (1.f / 128.f) + p.qk_eps);
#pragma unroll
            for (int e = 0; e < 4; ++e) v[e] = bf2f(f2bf(v[e] * inv * nwv[e]));  // rounded like a separate norm kernel would
          }
          if (rotate) {
            int pos = p.qk_positions[m];
            pos = pos < 0 ? 0 : (pos >= p.qk_max_pos ? p.qk_max_pos - 1 : pos);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float other = __shfl_xor_sync(0xffffffffu, v[e], 16);  // dim d +- 64 lives 16 lanes away
              const int d = dpair + e;
              if (d < p.qk_rot_half) {
                const float c = p.qk_cos[static_cast<size_t>(pos) * p.qk_rot_half + d], sn = p.qk_sin[static_cast<size_t>(pos) * p.qk_rot_half + d];
                v[e] = lane_e < 16 ? v[e] * c - other * sn : v[e] * c + other * sn;
              }
            }
          }
          uint2 pk;
          pk.x = pack_bf162(v[0], v[1]);
          pk.y = pack_bf162(v[2], v[3]);
          if (is_q) {
            *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(p.out) + static_cast<size_t>(m) * p.ldo + (head << 7) + row4) = pk;
          } else {
            const long long slot = p.qk_slots != nullptr ? p.qk_slots[m] : -1;
            if (slot >= 0) {
              const long long blk = slot / p.qk_block_size, off = slot % p.qk_block_size;
              __nv_bfloat16* cache = is_k ? p.k_cache : p.v_cache;
              *reinterpret_cast<uint2*>(cache + ((blk * p.qk_kv_heads + kvh) * p.qk_block_size + off) * 128 + row4) = pk;
            }
          }
        }
        if (splits > 1 && !p.cluster_reduce && t == 0) p.counters[ws_tile] = 0;
      }
    } else if constexpr (ACT) {
      // ---- gated activation: rows 0..63 of the tile are gate rows, rows 64..127 the up rows of the same 64 outputs ----
      // (host guarantees: no bias, no tensor-parallel fusion, N a multiple of 128, p.ldo = pitch of the [M, N / 2] output)
      if (do_store) {
        auto acc_at = [&](int col, int r4) -> float4 {
          float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
          if (clustered) {
            const uint32_t a = stage_addr + static_cast<uint32_t>((col * kGemmBM + r4) * 4);
            for (int sp = 0; sp < splits; ++sp) {
              const float4 v = ld_dsmem_f32x4(a, static_cast<uint32_t>(sp));
              acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
            }
          } else if (splits > 1) {
            const float* base = p.ws + static_cast<size_t>(ws_tile) * splits * (BN * kGemmBM);
            for (int sp = 0; sp < splits; ++sp) {
              const float4 v = __ldcg(reinterpret_cast<const float4*>(base + (static_cast<size_t>(sp) * BN + col) * kGemmBM + r4));
              acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
            }
          } else {
            acc = *reinterpret_cast<const float4*>(stage + col * kGemmBM + r4);
          }
          return acc;
        };
        auto act1 = [&](float g) -> float {
          if (p.act_kind == 2) {
            const float u = 0.7978845608028654f * (g + 0.044715f * g * g * g);
            return 0.5f * g * (1.f + tanhf(u));
          }
          return g / (1.f + __expf(-g));
        };
        if (row4 < 64) {
          const int half_n = p.N >> 1;
          const int no = (n_tile << 6) + row4;  // output column of weight row row4 of this tile (per expert in grouped mode)
          for (int col = static_cast<int>(me) + stride * csel; col < BN; col += stride * 16) {
            const int m = m0 + col;
            if (m >= m_lim) break;
            const float4 g = acc_at(col, row4), u = acc_at(col, row4 + 64);
            const float vals[4] = {act1(g.x) * u.x, act1(g.y) * u.y, act1(g.z) * u.z, act1(g.w) * u.w};
            const size_t o = static_cast<size_t>(m) * p.ldo + no;
            if (no + 3 < half_n && (p.ldo & 3) == 0 && !p.out_f32) {
              uint2 pk;
              pk.x = pack_bf162(vals[0], vals[1]);
              pk.y = pack_bf162(vals[2], vals[3]);
              *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(p.out) + o) = pk;
            } else {
              for (int e = 0; e < 4; ++e) {
                if (no + e < half_n) {
                  if (p.out_f32) reinterpret_cast<float*>(p.out)[o + e] = vals[e];
                  else reinterpret_cast<__nv_bfloat16*>(p.out)[o + e] = f2bf(vals[e]);
                }
              }
            }
          }
        }
        if (splits > 1 && !p.cluster_reduce && t == 0) p.counters[ws_tile] = 0;
      }
    } else if constexpr (SCAT) {
      // ---- GEMM -> reduce-scatter (host guarantees: N % 4 == 0, one split or a cluster, tp_size > 1) ----
      // row m belongs to rank m / tp_rows and is row (m - owner * tp_rows) of source slab tp_rank in the owner's receive area
      if (n + 3 < p.N) {
        for (int col = static_cast<int>(me) + stride * csel; col < BN; col += stride * 16) {
          const int m = m0 + col;
          if (m >= m_lim) break;
          const float4 acc = column_acc(col);
          uint2 pk;
          pk.x = pack_bf162(acc.x, acc.y);
          pk.y = pack_bf162(acc.z, acc.w);
          const int owner = m / p.tp_rows;
          __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.tp_recv[owner]) +
                               (static_cast<long long>(p.tp_rank) * p.tp_rows + (m - owner * p.tp_rows)) * static_cast<long long>(p.N);
          *reinterpret_cast<uint2*>(dst + n) = pk;
        }
      }
      __threadfence_system();
      asm volatile("bar.sync 1, 512;" ::: "memory");
      // every CTA of the tile (all splits of a cluster) counts once at every rank that owns some of the tile's rows: an owner
      // expects n_tiles * (m-tiles that overlap its rows) * splits publications per source and launch
      const int o_lo = m0 / p.tp_rows, o_hi = (min(m0 + BN, m_lim) - 1) / p.tp_rows;
      if (t <= o_hi - o_lo) red_release_sys_add(reinterpret_cast<uint32_t*>(p.tp_flags[o_lo + t]) + p.tp_rank, 1u);
    } else if (do_store && !fused_tp) {
      // column c of the tile is finished by cluster rank c % splits; the 16 column slots of this CTA take turns
      for (int col = static_cast<int>(me) + stride * csel; col < BN; col += stride * 16) {
        const int m = m0 + col;
        if (m >= m_lim) break;
        float4 acc = column_acc(col);
        acc.x += bias.x; acc.y += bias.y; acc.z += bias.z; acc.w += bias.w;
        store_out(m, acc);
      }
      if (splits > 1 && !p.cluster_reduce && t == 0) p.counters[ws_tile] = 0;
    }
    if (EPI == 0 && fused_tp) {
      // ---- GEMM + one-shot all-reduce over peer memory (host guarantees: N % 4 == 0, cluster or single split) ----
      const unsigned cta_id = (blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x;
      const unsigned call = *reinterpret_cast<volatile unsigned*>(p.tp_call);
      const long long par_off = static_cast<long long>(call & 1u) * p.tp_size * p.tp_slab;
      // phase A: partial sums -> every rank's receive slab [parity][my rank]
      if (n + 3 < p.N) {
        for (int col = static_cast<int>(me) + stride * csel; col < BN; col += stride * 16) {
          const int m = m0 + col;
          if (m >= m_lim) break;
          const float4 acc = column_acc(col);
          uint2 pk;
          pk.x = pack_bf162(acc.x, acc.y);
          pk.y = pack_bf162(acc.z, acc.w);
          if (p.tp_mode == 2) {  // own slab, slot 0: the reduce kernel sums the ranks' slot 0 through the multicast address
            *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(p.tp_recv[p.tp_rank]) + par_off + static_cast<long long>(m) * p.N + n) = pk;
            continue;
          }
          const long long off = par_off + static_cast<long long>(p.tp_rank) * p.tp_slab + static_cast<long long>(m) * p.N + n;
          for (int r = 0; r < p.tp_size; ++r)
            *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(p.tp_recv[(p.tp_rank + r) % p.tp_size]) + off) = pk;
        }
      }
      __threadfence_system();
      asm volatile("bar.sync 1, 512;" ::: "memory");
      if (t < 32) {
        // One lane per peer: the release-adds (each carries a system-scope fence) and the flag waits of the tp_size peers run
        // side by side; issued by a single thread they cost tp_size serial fence round trips (measured: 8 ranks, +20 us).
        const unsigned round = p.tp_rounds[cta_id];
        bool ok_lane = true;
        if (t < p.tp_size) {
          const int dst = (p.tp_rank + t) % p.tp_size;
          red_release_sys_add(reinterpret_cast<uint32_t*>(p.tp_flags[dst]) + static_cast<size_t>(p.tp_rank) * p.tp_ncta_max + cta_id, 1u);
          // phase B gate: rank `t` has published this CTA's region for this call (modes 1 / 2: the reduce kernel waits instead)
          const uint32_t* mine = reinterpret_cast<const uint32_t*>(p.tp_flags[p.tp_rank]);
          if (p.tp_mode == 0) ok_lane = flag_wait_ge(mine + static_cast<size_t>(t) * p.tp_ncta_max + cta_id, round + 1u, p.status);
        }
        const bool all = __all_sync(0xffffffffu, ok_lane);
        if (t == 0) {
          p.tp_rounds[cta_id] = round + 1u;
          *s_last = (all && p.tp_mode == 0) ? 1 : 0;
        }
      }
      asm volatile("bar.sync 1, 512;" ::: "memory");
      if (*s_last && n + 3 < p.N) {
        const __nv_bfloat16* rbase = reinterpret_cast<const __nv_bfloat16*>(p.tp_recv[p.tp_rank]) + par_off;
        for (int col = static_cast<int>(me) + stride * csel; col < BN; col += stride * 16) {
          const int m = m0 + col;
          if (m >= m_lim) break;
          float4 acc = bias;
          for (int src = 0; src < p.tp_size; ++src) {
            const uint2 pk = __ldcg(reinterpret_cast<const uint2*>(rbase + static_cast<long long>(src) * p.tp_slab + static_cast<long long>(m) * p.N + n));
            const float2 a = unpack_bf162(pk.x), b = unpack_bf162(pk.y);
            acc.x += a.x; acc.y += a.y; acc.z += b.x; acc.w += b.y;
          }
          store_out(m, acc);
        }
      }
      // launch bookkeeping: the last CTA of the grid to get here advances the launch counter (flips the parity)
      asm volatile("bar.sync 1, 512;" ::: "memory");
      if (t == 0) {
        const unsigned total = gridDim.x * gridDim.y * gridDim.z;
        if (atomicAdd(p.tp_call + 1, 1u) == total - 1u) {
          p.tp_call[1] = 0u;
          __threadfence();
          p.tp_call[0] = call + 1u;
        }
      }
    }
  }
  if (clustered) cluster_sync_all();  // no CTA leaves while a peer may still read its shared memory
  // ---------------- teardown ----------------
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

}  // namespace dlv
