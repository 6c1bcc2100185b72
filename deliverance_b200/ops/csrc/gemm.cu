// Host side of the tcgen05 GEMM (tensor-map encoding, tile / split-K selection, launch) plus a CUDA-core GEMV used for
// one to four tokens and as an independent implementation in the numerics tests.
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <stdexcept>
#include <string>

#include "gemm_tc.cuh"
#include "gemm_api.h"

namespace dlv {

// ------------------------------------------------------------------------------------------------ tensor maps
using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                              const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeFn get_encode() {
  static EncodeFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres);
    if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || p == nullptr)
      throw std::runtime_error("cuTensorMapEncodeTiled entry point not available");
    fn = reinterpret_cast<EncodeFn>(p);
  });
  return fn;
}

// 2-D row-major tensor [rows, cols] of `elem_bytes`-sized elements with row pitch `pitch_bytes`; box = [box_rows, box_cols].
void encode_map_2d(CUtensorMap* map, int dtype_code, const void* base, uint64_t rows, uint64_t cols, uint64_t pitch_bytes,
                   uint32_t box_rows, uint32_t box_cols, int swizzle_code) {
  CUtensorMapDataType dt = dtype_code == 0 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                           : dtype_code == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                           : dtype_code == 3 ? CU_TENSOR_MAP_DATA_TYPE_UINT32
                                             : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  CUtensorMapSwizzle sw = swizzle_code == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
                          : swizzle_code == 64 ? CU_TENSOR_MAP_SWIZZLE_64B
                                               : CU_TENSOR_MAP_SWIZZLE_NONE;
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0) throw std::runtime_error("TMA base address must be 16-byte aligned");
  if (pitch_bytes % 16 != 0) throw std::runtime_error("TMA row pitch must be a multiple of 16 bytes");
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {pitch_bytes};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = get_encode()(map, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) throw std::runtime_error("cuTensorMapEncodeTiled failed with code " + std::to_string(static_cast<int>(r)));
}

// bf16 matrix [rows, K] (K % 64 == 0) seen as [K / 64 chunks][rows][64]: one box = `box_rows` rows x 2 chunks lands in shared
// memory as two consecutive 128B-swizzled 64-wide sub-tiles, i.e. a whole 128-k pipeline stage with ONE copy instruction
// (a single thread can only issue a copy every ~0.3 us, whatever its size).
void encode_map_kchunks(CUtensorMap* map, const void* base, uint64_t rows, uint64_t K, uint64_t pitch_bytes, uint32_t box_rows) {
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0) throw std::runtime_error("TMA base address must be 16-byte aligned");
  if (pitch_bytes % 16 != 0 || K % 64 != 0) throw std::runtime_error("chunked TMA map needs K % 64 == 0 and a 16-byte row pitch");
  cuuint64_t dims[3] = {64, rows, K / 64};
  cuuint64_t strides[2] = {pitch_bytes, 128};
  cuuint32_t box[3] = {64, box_rows, 2};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = get_encode()(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) throw std::runtime_error("cuTensorMapEncodeTiled (3-D) failed with code " + std::to_string(static_cast<int>(r)));
}

// ------------------------------------------------------------------------------------------------ weight handle
void gemm_weight_init(GemmWeightDesc* w) {
  if (w->is_q4) {
    if (w->K % 32 != 0) throw std::runtime_error("JQ4 weight needs K % 32 == 0");
    if ((reinterpret_cast<uintptr_t>(w->data) & 15) != 0) throw std::runtime_error("tile-packed JQ4 weights must be 16-byte aligned");
    // the tile-packed bytes seen as rows of 1 KB: one stage = 10 consecutive rows = one 2-D TMA box
    const uint64_t stages = static_cast<uint64_t>((w->N + 127) / 128) * ((w->K + 127) / 128);
    encode_map_2d(&w->map_w, 3, w->data, stages * 10, 256, 1024, 10, 256, 0);
  } else {
    if (w->K % 8 != 0) throw std::runtime_error("dense weight needs K % 8 == 0");
    w->w3d = w->K % 64 == 0;
    if (w->w3d) encode_map_kchunks(&w->map_w, w->data, w->N, w->K, static_cast<uint64_t>(w->K) * 2, kGemmBM);
    else encode_map_2d(&w->map_w, 0, w->data, w->N, w->K, static_cast<uint64_t>(w->K) * 2, kGemmBM, 64, 128);
  }
}

bool g_pdl_enabled = true;
bool& g_gemm_pdl = g_pdl_enabled;  // programmatic dependent launch of the GEMM kernels (ops.set_gemm_pdl / DLV_GEMM_PDL=0 turn it off)
void gemm_set_pdl(bool on) { g_gemm_pdl = on; }


int gemm_num_sms() {
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (sms <= 0) sms = 148;
  }
  return sms;
}

// Number of clusters of `size` CTAs of this kernel that can be resident at once (0 when such a cluster cannot be scheduled).
template <bool Q4, int BN, int EPI = 0>
static int cluster_capacity(int size) {
  using L = GemmSmem<Q4, BN>;
  static int cap[9] = {-1, -1, -1, -1, -1, -1, -1, -1, -1};
  static PerDeviceOnce attr_once;  // the capacities below are shared: the GPUs of one process are the same model
  if (attr_once.first()) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<Q4, BN, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kBytes);
    if (e != cudaSuccess) throw std::runtime_error(std::string("cudaFuncSetAttribute: ") + cudaGetErrorString(e));
  }
  if (size < 1 || size > 8) return 0;
  if (cap[size] < 0) {
    if (size == 1) {
      cap[size] = gemm_num_sms();
    } else {
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3(1, 1, size);
      cfg.blockDim = dim3(kGemmThreads);
      cfg.dynamicSmemBytes = L::kBytes;
      cudaLaunchAttribute attr[1];
      attr[0].id = cudaLaunchAttributeClusterDimension;
      attr[0].val.clusterDim.x = 1;
      attr[0].val.clusterDim.y = 1;
      attr[0].val.clusterDim.z = size;
      cfg.attrs = attr;
      cfg.numAttrs = 1;
      int n = 0;
      cudaError_t e = cudaOccupancyMaxActiveClusters(&n, gemm_tc_kernel<Q4, BN, EPI>, &cfg);
      (void)cudaGetLastError();
      cap[size] = (e == cudaSuccess && n > 0) ? n : 0;
    }
  }
  return cap[size];
}

template <bool Q4, int BN, int EPI = 0>
static void run_tc(const GemmWeightDesc* w, const void* x, int M, int ldx, GemmParams p, float* ws, size_t ws_floats, int* counters,
                   int n_counters, int force_splits, cudaStream_t st, const GemmTpArgs* tp) {
  using L = GemmSmem<Q4, BN>;
  p.n_tiles = (w->N + kGemmBM - 1) / kGemmBM;
  p.m_tiles = (M + BN - 1) / BN;
  const int tiles = p.n_tiles * p.m_tiles;
  // Split-K plan. The CTAs of one output tile form a cluster; cost model (microseconds): every wave of resident clusters
  // pays a fixed prologue/epilogue and its share of the k-blocks, split tiles also pay the cluster reduction.
  const bool no_cluster = force_splits < 0;  // negative: that many splits, reduced through the global workspace
  int splits = 1;
  if (force_splits != 0) {
    splits = force_splits < 0 ? -force_splits : force_splits;
  } else {
    double best = 1e30;
    for (int s = 1; s <= 8; ++s) {
      if (s > 1 && p.kb_total / s < 2) break;
      const int cap = cluster_capacity<Q4, BN, EPI>(s);
      if (cap <= 0) continue;
      if (tp != nullptr && tp->size > 1 && (tiles > cap || tiles * s > tp->ncta_max)) continue;  // fused all-reduce: one wave
      const int waves = (tiles + cap - 1) / cap;
      const int kb = (p.kb_total + s - 1) / s;
      const double per_kb = 0.22 * (BN > 64 ? BN / 64.0 : 1.0);
      const double cost = waves * (3.0 + kb * per_kb + (s > 1 ? 1.0 : 0.0));
      if (cost < best - 1e-9) {
        best = cost;
        splits = s;
      }
    }
  }
  if (splits > p.kb_total) splits = p.kb_total;
  if (splits < 1) splits = 1;
  p.kb_per_split = (p.kb_total + splits - 1) / splits;
  splits = (p.kb_total + p.kb_per_split - 1) / p.kb_per_split;  // no empty split
  bool cluster = splits > 1 && !no_cluster && splits <= 8 && cluster_capacity<Q4, BN, EPI>(splits) > 0;
  if (splits > 1 && !cluster) {
    const size_t need = static_cast<size_t>(tiles) * splits * BN * kGemmBM;
    if (ws == nullptr || counters == nullptr || need > ws_floats || tiles > n_counters) {
      splits = 1;
      p.kb_per_split = p.kb_total;
    }
  }
  (void)cluster_capacity<Q4, BN, EPI>(1);  // sets the shared-memory attribute
  if (tp != nullptr && tp->size > 1) {
    // fused all-reduce: partial tiles must come from a single split or a cluster, and the grid must be resident at once
    if (splits > 1 && !cluster) {
      splits = 1;
      p.kb_per_split = p.kb_total;
    }
    const int cap = cluster_capacity<Q4, BN, EPI>(splits > 1 ? splits : 1);
    if (tiles > cap || tiles * splits > tp->ncta_max) throw std::runtime_error("fused tensor-parallel GEMM: grid does not fit in one wave");
    p.tp_size = tp->size;
    p.tp_rank = tp->rank;
    p.tp_ncta_max = tp->ncta_max;
    p.tp_slab = tp->slab;
    for (int r = 0; r < 8; ++r) {
      p.tp_recv[r] = tp->recv[r];
      p.tp_flags[r] = tp->flags[r];
    }
    p.tp_rounds = tp->rounds;
    p.tp_call = tp->call;
    p.tp_mode = tp->mode;
    tp->last_ctas = tiles * splits;
  }
  p.splits = splits;
  p.cluster_reduce = cluster ? 1 : 0;
  p.ws = ws;
  p.counters = counters;
  p.wq = w->is_q4 ? static_cast<const uint8_t*>(w->data) : nullptr;
  CUtensorMap map_x;
  p.w3d = w->w3d ? 1 : 0;
  p.x3d = w->K % 64 == 0 ? 1 : 0;
  if (p.x3d) encode_map_kchunks(&map_x, x, static_cast<uint64_t>(M), static_cast<uint64_t>(w->K), static_cast<uint64_t>(ldx) * 2, BN);
  else encode_map_2d(&map_x, 0, x, static_cast<uint64_t>(M), static_cast<uint64_t>(w->K), static_cast<uint64_t>(ldx) * 2, BN, 64, 128);
  // Tail split: a single-split grid that is a few tiles larger than the SM count would run a full second wave for those few
  // tiles. They are cut into up to 8 k-ranges each (reduced through the workspace), so the second wave is a short one.
  int grid_x = p.n_tiles;
  if ((tp == nullptr || tp->size <= 1) && splits == 1 && p.m_tiles == 1 && force_splits == 0 && ws != nullptr && counters != nullptr &&
      p.kb_total >= 8) {
    const int cap = gemm_num_sms();
    const int rem = p.n_tiles % cap;
    if (p.n_tiles > cap && rem > 0 && rem * 8 <= cap) {
      const int kb_per = (p.kb_total + 7) / 8;
      const int s_eff = (p.kb_total + kb_per - 1) / kb_per;
      if (s_eff > 1 && static_cast<size_t>(rem) * s_eff * BN * kGemmBM <= ws_floats && rem <= n_counters) {
        p.tail_tile0 = p.n_tiles - rem;
        p.tail_splits = s_eff;
        p.tail_kb_per_split = kb_per;
        grid_x = p.tail_tile0 + rem * s_eff;
      }
    }
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid_x, p.m_tiles, p.splits);
  cfg.blockDim = dim3(kGemmThreads);
  cfg.dynamicSmemBytes = L::kBytes;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  int na = 0;
  if (cluster) {
    attr[na].id = cudaLaunchAttributeClusterDimension;
    attr[na].val.clusterDim.x = 1;
    attr[na].val.clusterDim.y = 1;
    attr[na].val.clusterDim.z = p.splits;
    ++na;
  }
  if (g_gemm_pdl) {
    // programmatic dependent launch: prologue + weight streaming overlap the tail of the kernel in front (see pdl_wait)
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  cfg.attrs = attr;
  cfg.numAttrs = na;
  cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_tc_kernel<Q4, BN, EPI>, w->map_w, map_x, p);
  if (e != cudaSuccess) throw std::runtime_error(std::string("gemm launch: ") + cudaGetErrorString(e));
}

// Choose the token tile. Small batches take the smallest UMMA N that covers them.
struct GemmWeightDesc;
bool gemv_dense_supported(const GemmWeightDesc* w, int M, int ldx);
void gemv_dense_run(const GemmWeightDesc* w, const void* x, int M, int ldx, void* out, int ldo, bool out_f32, const float* bias, int act,
                    cudaStream_t st);
static int pick_bn(int M) {
  if (M <= 16) return 16;
  if (M <= 32) return 32;
  if (M <= 64) return 64;
  if (M <= 128) return 128;
  return 256;
}

// Prefill sizes: 256-token tiles halve the weight traffic per FLOP, but a grid that is a little more than a whole number of waves
// wastes most of its last wave (N = 2560, M = 2048: 160 tiles on 148 SMs). 128-token tiles cost a little more than half as much
// each (kBn128Cost, measured) and come in twice the number, so they win where they fill the waves better.
bool g_gemm_persist_all = false;  // tests: the persistent kernel for every shape it supports
int g_gemm_force_bn = 0;  // 128 / 256: token tile for every batch of more than 128 rows (0: chosen by wave count)
static int pick_bn_waves(int M, int N) {
  const int bn = pick_bn(M);
  if (bn != 256) return bn;
  static const double kCost128 = [] { const char* v = getenv("DLV_GEMM_BN128_COST"); return v ? atof(v) : 0.58; }();
  if (g_gemm_force_bn == 128 || g_gemm_force_bn == 256) return g_gemm_force_bn;  // tests and comparisons
  const int sms = gemm_num_sms();
  const long long n_tiles = (N + kGemmBM - 1) / kGemmBM;
  const long long t256 = n_tiles * ((M + 255) / 256), t128 = n_tiles * ((M + 127) / 128);
  if (t256 <= sms) return 256;  // a single partial wave: measured no gain from smaller tiles (the split-K planner fills the SMs)
  const double c256 = static_cast<double>((t256 + sms - 1) / sms), c128 = static_cast<double>((t128 + sms - 1) / sms) * kCost128;
  return c128 < 0.97 * c256 ? 128 : 256;
}

bool gemm_tp_supported(const GemmWeightDesc* w, int M, const GemmTpArgs* tp) {
  if (tp == nullptr || tp->size <= 1 || tp->size > 8) return false;
  if (w->N % 4 != 0 || M <= 0 || M > 128) return false;
  if (static_cast<long long>(M) * w->N > tp->slab) return false;
  const int BN = pick_bn(M);
  const int tiles = ((w->N + kGemmBM - 1) / kGemmBM) * ((M + BN - 1) / BN);
  return tiles <= gemm_num_sms() && tiles <= tp->ncta_max;
}

void gemm_tc_run(const GemmWeightDesc* w, const void* x, int M, int ldx, void* out, int ldo, bool out_f32, const float* bias,
                 float* ws, size_t ws_floats, int* counters, int n_counters, int* status, int force_splits, cudaStream_t st,
                 const GemmTpArgs* tp) {
  if (M <= 0) return;
  if (ldx % 8 != 0) throw std::runtime_error("activation row pitch must be a multiple of 8 elements");
  if ((tp == nullptr || tp->size <= 1) && force_splits == 0 && gemv_dense_supported(w, M, ldx)) {
    gemv_dense_run(w, x, M, ldx, out, ldo, out_f32, bias, 0, st);
    return;
  }
  if (g_gemm_persist && (tp == nullptr || tp->size <= 1) && force_splits == 0 && g_gemm_force_bn == 0 && gemm_persist_supported(w, M, ldx) &&
      (g_gemm_persist_all || gemm_persist_preferred(w, M))) {
    gemm_persist_run(w, x, M, ldx, out, ldo, out_f32, bias, status, st);
    return;
  }
  const int BN = (tp == nullptr || tp->size <= 1) ? pick_bn_waves(M, w->N) : pick_bn(M);
  GemmParams p = {};
  p.M = M;
  p.N = w->N;
  p.K = w->K;
  p.kb_total = (w->K + kGemmBK - 1) / kGemmBK;
  p.out = out;
  p.ldo = ldo;
  p.out_f32 = out_f32 ? 1 : 0;
  p.bias = bias;
  p.status = status;
#define DLV_LAUNCH(BNV)                                                                              \
  if (w->is_q4) run_tc<true, BNV>(w, x, M, ldx, p, ws, ws_floats, counters, n_counters, force_splits, st, tp); \
  else run_tc<false, BNV>(w, x, M, ldx, p, ws, ws_floats, counters, n_counters, force_splits, st, tp)
  switch (BN) {
    case 16: DLV_LAUNCH(16); break;
    case 32: DLV_LAUNCH(32); break;
    case 64: DLV_LAUNCH(64); break;
    case 128: DLV_LAUNCH(128); break;
    default: DLV_LAUNCH(256); break;
  }
#undef DLV_LAUNCH
}

// Gate | up projection with the gated activation in the epilogue: `w` holds the gate and up rows interleaved per 128-row tile
// (64 gate rows, then the 64 up rows of the same outputs), out is [M, N / 2]. act: 1 = SiLU, 2 = tanh-approximated GELU.
void gemm_tc_run_act(const GemmWeightDesc* w, const void* x, int M, int ldx, void* out, int ldo, int act, float* ws, size_t ws_floats,
                     int* counters, int n_counters, int* status, cudaStream_t st) {
  if (M <= 0) return;
  if (ldx % 8 != 0) throw std::runtime_error("activation row pitch must be a multiple of 8 elements");
  if (w->N % kGemmBM != 0) throw std::runtime_error("fused activation: gate|up rows must be a multiple of 128");
  if (act != 1 && act != 2) throw std::runtime_error("fused activation: unknown activation");
  const int BN = pick_bn(M);
  GemmParams p = {};
  p.M = M;
  p.N = w->N;
  p.K = w->K;
  p.kb_total = (w->K + kGemmBK - 1) / kGemmBK;
  p.out = out;
  p.ldo = ldo;
  p.out_f32 = 0;
  p.status = status;
  p.act_kind = act;
#define DLV_LAUNCH(BNV)                                                                                           \
  if (w->is_q4) run_tc<true, BNV, 1>(w, x, M, ldx, p, ws, ws_floats, counters, n_counters, 0, st, nullptr);     \
  else run_tc<false, BNV, 1>(w, x, M, ldx, p, ws, ws_floats, counters, n_counters, 0, st, nullptr)
  switch (BN) {
    case 16: DLV_LAUNCH(16); break;
    case 32: DLV_LAUNCH(32); break;
    case 64: DLV_LAUNCH(64); break;
    case 128: DLV_LAUNCH(128); break;
    default: DLV_LAUNCH(256); break;
  }
#undef DLV_LAUNCH
}

// ------------------------------------------------------------------------------------------------ GEMM -> reduce-scatter
// Prefill-size row-parallel projections under tensor parallelism. Token rows are cut into one contiguous range per rank (a
// multiple of 8 rows). The GEMM (EPI = 3) stores each partial tile into the receive area of the rank that owns its
// rows while the other tiles are still being computed, and never waits, so the grid may be many waves. comm.cu then sums the
// partial slabs of the owned rows and hands the reduced rows to every rank.
GemmScatterPlan gemm_scatter_plan(int M, int N, int size) {
  GemmScatterPlan plan = {};
  const int per = (M + size - 1) / size;
  plan.rows_per_rank = ((per + kScatterGroupRows - 1) / kScatterGroupRows) * kScatterGroupRows;
  const int n_tiles = (N + kGemmBM - 1) / kGemmBM;
  for (int r = 0; r < 8; ++r) {
    int rows = r < size ? M - r * plan.rows_per_rank : 0;
    rows = rows < 0 ? 0 : (rows > plan.rows_per_rank ? plan.rows_per_rank : rows);
    plan.rows[r] = rows;
    // 256-token tiles of the GEMM that contain at least one of this rank's rows
    const int lo = r * plan.rows_per_rank;
    plan.tiles[r] = rows > 0 ? n_tiles * ((lo + rows - 1) / 256 - lo / 256 + 1) : 0;
    plan.groups[r] = (rows + kScatterGroupRows - 1) / kScatterGroupRows;
  }
  return plan;
}

bool gemm_scatter_supported(const GemmWeightDesc* w, int M, const GemmScatterArgs* a) {
  if (a == nullptr || a->size <= 1 || a->size > 8) return false;
  if (w->N % 8 != 0 || M < 256 * a->size) return false;  // smaller batches: the one-shot epilogue or the library all-reduce
  const GemmScatterPlan plan = gemm_scatter_plan(M, w->N, a->size);
  return static_cast<long long>(a->size) * plan.rows_per_rank * w->N <= a->recv_elems &&
         static_cast<long long>(M) * w->N <= a->gather_elems;
}

void gemm_tc_run_scatter(const GemmWeightDesc* w, const void* x, int M, int ldx, const GemmScatterArgs* a, int* status, cudaStream_t st) {
  if (!gemm_scatter_supported(w, M, a)) throw std::runtime_error("GEMM -> reduce-scatter: shape outside the fused path");
  if (ldx % 8 != 0) throw std::runtime_error("activation row pitch must be a multiple of 8 elements");
  GemmParams p = {};
  p.M = M;
  p.N = w->N;
  p.K = w->K;
  p.kb_total = (w->K + kGemmBK - 1) / kGemmBK;
  p.out = nullptr;
  p.ldo = w->N;
  p.status = status;
  p.tp_size = a->size;
  p.tp_rank = a->rank;
  p.tp_rows = gemm_scatter_plan(M, w->N, a->size).rows_per_rank;
  for (int r = 0; r < 8; ++r) {
    p.tp_recv[r] = a->recv[r];
    p.tp_flags[r] = a->flags[r];
  }
  // one split per tile (force_splits = 1): the owner counts exactly n_tiles * its m-tiles publications per source and launch
  if (w->is_q4) run_tc<true, 256, 3>(w, x, M, ldx, p, nullptr, 0, nullptr, 0, 1, st, nullptr);
  else run_tc<false, 256, 3>(w, x, M, ldx, p, nullptr, 0, nullptr, 0, 1, st, nullptr);
}

// ------------------------------------------------------------------------------------------------ all-gather -> GEMM
// Column-parallel projections whose input rows live sharded over the ranks (sequence parallel). The rows are staged once in
// this GPU's gather area (pushed by their owners over NVLink) and read from there by TMA: a remote tile crosses the link once,
// however many weight tiles use it. The wait for a token tile's owners sits in the activation producers (EPI = 4), so weights
// stream and tiles whose rows have arrived run while other rows are still in flight.
bool gemm_gathered_supported(const GemmWeightDesc* w, int M, const GemmScatterArgs* a) {
  if (a == nullptr || a->size <= 1 || a->size > 8) return false;
  if (w->K % 8 != 0 || M < 256 * a->size) return false;
  return static_cast<long long>(M) * w->K <= a->gather_elems;
}

void gemm_tc_run_gathered(const GemmWeightDesc* w, int M, const GemmScatterArgs* a, const unsigned* group_targets, void* out, int ldo,
                          const float* bias, float* ws, size_t ws_floats, int* counters, int n_counters, int* status, cudaStream_t st) {
  if (!gemm_gathered_supported(w, M, a)) throw std::runtime_error("all-gather -> GEMM: shape outside the fused path");
  GemmParams p = {};
  p.M = M;
  p.N = w->N;
  p.K = w->K;
  p.kb_total = (w->K + kGemmBK - 1) / kGemmBK;
  p.out = out;
  p.ldo = ldo;
  p.out_f32 = 0;
  p.bias = bias;
  p.status = status;
  p.ag_rows = gemm_scatter_plan(M, w->N, a->size).rows_per_rank;
  p.ag_flags = reinterpret_cast<const uint32_t*>(a->flags[a->rank]) + 16;
  for (int r = 0; r < 8; ++r) p.ag_targets[r] = group_targets[r];
  const void* x = reinterpret_cast<const void*>(a->gather[a->rank]);  // [M][K] bf16, this GPU's own memory
  if (w->is_q4) run_tc<true, 256, 4>(w, x, M, w->K, p, ws, ws_floats, counters, n_counters, 0, st, nullptr);
  else run_tc<false, 256, 4>(w, x, M, w->K, p, ws, ws_floats, counters, n_counters, 0, st, nullptr);
}

// ------------------------------------------------------------------------------------------------ grouped (MoE) GEMM
// out[r, :] = xs[r, :] @ W[expert(r)]^T for rows grouped by expert. `items` is the device work list built by
// launch_moe_items with the same token tile `bn`; `max_items` bounds it (unused slots return at once).
template <bool Q4, int BN, int EPI = 0>
static void run_grouped(const GemmWeightDesc* w, const void* x, int rows, int ldx, GemmParams p, int max_items, int splits, cudaStream_t st) {
  using L = GemmSmem<Q4, BN>;
  if (splits > p.kb_total / 2) splits = p.kb_total / 2;
  if (splits < 1) splits = 1;
  while (splits > 1 && cluster_capacity<Q4, BN, EPI>(splits) <= 0) --splits;
  p.kb_per_split = (p.kb_total + splits - 1) / splits;
  splits = (p.kb_total + p.kb_per_split - 1) / p.kb_per_split;
  (void)cluster_capacity<Q4, BN, EPI>(1);  // sets the shared-memory attribute
  p.splits = splits;
  p.cluster_reduce = splits > 1 ? 1 : 0;
  p.wq = w->is_q4 ? static_cast<const uint8_t*>(w->data) : nullptr;
  CUtensorMap map_x;
  p.w3d = w->w3d ? 1 : 0;
  p.x3d = w->K % 64 == 0 ? 1 : 0;
  if (p.x3d) encode_map_kchunks(&map_x, x, static_cast<uint64_t>(rows), static_cast<uint64_t>(w->K), static_cast<uint64_t>(ldx) * 2, BN);
  else encode_map_2d(&map_x, 0, x, static_cast<uint64_t>(rows), static_cast<uint64_t>(w->K), static_cast<uint64_t>(ldx) * 2, BN, 64, 128);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(p.n_tiles, max_items, splits);
  cfg.blockDim = dim3(kGemmThreads);
  cfg.dynamicSmemBytes = L::kBytes;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  int na = 0;
  if (splits > 1) {
    attr[na].id = cudaLaunchAttributeClusterDimension;
    attr[na].val.clusterDim.x = 1;
    attr[na].val.clusterDim.y = 1;
    attr[na].val.clusterDim.z = splits;
    ++na;
  }
  if (g_gemm_pdl) {
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  cfg.attrs = attr;
  cfg.numAttrs = na;
  cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_tc_kernel<Q4, BN, EPI>, w->map_w, map_x, p);
  if (e != cudaSuccess) throw std::runtime_error(std::string("grouped gemm launch: ") + cudaGetErrorString(e));
}

void gemm_tc_run_grouped(const GemmWeightDesc* w, int n_per_expert, const void* x, int rows, int ldx, void* out, int ldo,
                         const int* items, int max_items, int bn, int splits, int* status, cudaStream_t st) {
  if (rows <= 0 || max_items <= 0) return;
  if (ldx % 8 != 0) throw std::runtime_error("activation row pitch must be a multiple of 8 elements");
  if (max_items > 65535) throw std::runtime_error("grouped gemm: work list too long");
  GemmParams p = {};
  p.M = rows;
  p.N = n_per_expert;
  p.K = w->K;
  p.kb_total = (w->K + kGemmBK - 1) / kGemmBK;
  p.n_tiles = (n_per_expert + kGemmBM - 1) / kGemmBM;
  p.m_tiles = max_items;
  p.out = out;
  p.ldo = ldo;
  p.out_f32 = 0;
  p.status = status;
  p.grp_items = reinterpret_cast<const int4*>(items);
#define DLV_LAUNCH(BNV)                                                              \
  if (w->is_q4) run_grouped<true, BNV>(w, x, rows, ldx, p, max_items, splits, st);   \
  else run_grouped<false, BNV>(w, x, rows, ldx, p, max_items, splits, st)
  switch (bn) {
    case 16: DLV_LAUNCH(16); break;
    case 32: DLV_LAUNCH(32); break;
    case 64: DLV_LAUNCH(64); break;
    case 128: DLV_LAUNCH(128); break;
    case 256: DLV_LAUNCH(256); break;
    default: throw std::runtime_error("grouped gemm: token tile must be 16, 32, 64, 128 or 256");
  }
#undef DLV_LAUNCH
}

// q | k | v projection whose epilogue applies the per-head RMSNorm (optional), the rotary embedding (optional) and writes K / V
// straight into the paged cache; only the query heads go to `q_out` [M, H * 128]. head_dim must be 128 (one weight tile = one head).
void gemm_tc_run_qkv(const GemmWeightDesc* w, const void* x, int M, int ldx, void* q_out, int ldo, const float* bias, const GemmQkvArgs* a,
                     float* ws, size_t ws_floats, int* counters, int n_counters, int* status, cudaStream_t st) {
  if (M <= 0) return;
  if (ldx % 8 != 0) throw std::runtime_error("activation row pitch must be a multiple of 8 elements");
  if (w->N != (a->heads + 2 * a->kv_heads) * kGemmBM) throw std::runtime_error("fused q/k/v epilogue: weight rows must be (H + 2 KV) * 128");
  if (ldo % 4 != 0) throw std::runtime_error("fused q/k/v epilogue: query row pitch must be a multiple of 4");
  const int BN = pick_bn(M);
  GemmParams p = {};
  p.M = M;
  p.N = w->N;
  p.K = w->K;
  p.kb_total = (w->K + kGemmBK - 1) / kGemmBK;
  p.out = q_out;
  p.ldo = ldo;
  p.out_f32 = 0;
  p.bias = bias;
  p.status = status;
  p.qk_positions = a->positions;
  p.qk_slots = a->slots;
  p.q_norm_w = static_cast<const __nv_bfloat16*>(a->q_norm_w);
  p.k_norm_w = static_cast<const __nv_bfloat16*>(a->k_norm_w);
  p.qk_cos = a->cos_t;
  p.qk_sin = a->sin_t;
  p.k_cache = static_cast<__nv_bfloat16*>(a->k_cache);
  p.v_cache = static_cast<__nv_bfloat16*>(a->v_cache);
  p.qk_heads = a->heads;
  p.qk_kv_heads = a->kv_heads;
  p.qk_block_size = a->block_size;
  p.qk_rot_half = a->rot_half;
  p.qk_max_pos = a->max_pos;
  p.qk_eps = a->eps;
  p.qk_norm_offset = a->norm_offset;
#define DLV_LAUNCH(BNV)                                                                                        \
  if (w->is_q4) run_tc<true, BNV, 2>(w, x, M, ldx, p, ws, ws_floats, counters, n_counters, 0, st, nullptr);     \
  else run_tc<false, BNV, 2>(w, x, M, ldx, p, ws, ws_floats, counters, n_counters, 0, st, nullptr)
  switch (BN) {
    case 16: DLV_LAUNCH(16); break;
    case 32: DLV_LAUNCH(32); break;
    case 64: DLV_LAUNCH(64); break;
    case 128: DLV_LAUNCH(128); break;
    default: DLV_LAUNCH(256); break;
  }
#undef DLV_LAUNCH
}

// Grouped gate | up projection with the gated activation in the epilogue: every expert's rows are interleaved per 128-row tile
// (64 gate rows, then the 64 up rows of the same outputs); out is [rows, n_per_expert / 2].
void gemm_tc_run_grouped_act(const GemmWeightDesc* w, int n_per_expert, const void* x, int rows, int ldx, void* out, int ldo,
                             const int* items, int max_items, int bn, int splits, int act, int* status, cudaStream_t st) {
  if (rows <= 0 || max_items <= 0) return;
  if (ldx % 8 != 0) throw std::runtime_error("activation row pitch must be a multiple of 8 elements");
  if (max_items > 65535) throw std::runtime_error("grouped gemm: work list too long");
  if (n_per_expert % kGemmBM != 0) throw std::runtime_error("fused activation: gate|up rows per expert must be a multiple of 128");
  if (act != 1 && act != 2) throw std::runtime_error("fused activation: unknown activation");
  GemmParams p = {};
  p.M = rows;
  p.N = n_per_expert;
  p.K = w->K;
  p.kb_total = (w->K + kGemmBK - 1) / kGemmBK;
  p.n_tiles = n_per_expert / kGemmBM;
  p.m_tiles = max_items;
  p.out = out;
  p.ldo = ldo;
  p.out_f32 = 0;
  p.status = status;
  p.grp_items = reinterpret_cast<const int4*>(items);
  p.act_kind = act;
#define DLV_LAUNCH(BNV)                                                                    \
  if (w->is_q4) run_grouped<true, BNV, 1>(w, x, rows, ldx, p, max_items, splits, st);   \
  else run_grouped<false, BNV, 1>(w, x, rows, ldx, p, max_items, splits, st)
  switch (bn) {
    case 16: DLV_LAUNCH(16); break;
    case 32: DLV_LAUNCH(32); break;
    case 64: DLV_LAUNCH(64); break;
    case 128: DLV_LAUNCH(128); break;
    case 256: DLV_LAUNCH(256); break;
    default: throw std::runtime_error("grouped gemm: token tile must be 16, 32, 64, 128 or 256");
  }
#undef DLV_LAUNCH
}

// ------------------------------------------------------------------------------------------------ CUDA-core GEMV
// One warp per weight row, MT tokens. fp32 accumulation; JQ4 blocks are expanded in registers.
template <int MT, bool Q4>
__global__ void __launch_bounds__(128) gemv_simt_kernel(const void* __restrict__ wdata, const __nv_bfloat16* __restrict__ x, int ldx,
                                                        void* __restrict__ out, int ldo, int out_f32, const float* __restrict__ bias,
                                                        int N, int K) {
  const int n = blockIdx.x * 4 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (n >= N) return;
  float acc[MT];
#pragma unroll
  for (int m = 0; m < MT; ++m) acc[m] = 0.f;
  if (Q4) {
    const int kb_total = (K + 127) / 128;
    const int r = n & 127;
    const uint8_t* tile_row = static_cast<const uint8_t*>(wdata) + static_cast<size_t>(n >> 7) * kb_total * kQ4StageBytes;
    for (int blk = lane; blk < K / 32; blk += 32) {
      const uint8_t* stage = tile_row + static_cast<size_t>(blk >> 2) * kQ4StageBytes;
      const uint4 w = __ldg(reinterpret_cast<const uint4*>(stage + r * 64 + (((blk & 3) ^ ((r >> 1) & 3)) << 4)));
      const float sc = __ldg(reinterpret_cast<const float*>(stage + 8192 + r * 16 + (blk & 3) * 4));
      const uint32_t words[4] = {w.x, w.y, w.z, w.w};
      float wf[32];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
#pragma unroll
        for (int b = 0; b < 4; ++b) {
          const uint32_t byte = (words[i] >> (8 * b)) & 0xFFu;
          wf[4 * i + b] = static_cast<float>(static_cast<int>(byte & 0xFu) - 8) * sc;
          wf[16 + 4 * i + b] = static_cast<float>(static_cast<int>(byte >> 4) - 8) * sc;
        }
      }
#pragma unroll
      for (int m = 0; m < MT; ++m) {
        const __nv_bfloat16* xr = x + static_cast<size_t>(m) * ldx + blk * 32;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const uint4 xv = *reinterpret_cast<const uint4*>(xr + c * 8);
          const uint32_t* xu = reinterpret_cast<const uint32_t*>(&xv);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 f = unpack_bf162(xu[e]);
            acc[m] += f.x * wf[c * 8 + 2 * e] + f.y * wf[c * 8 + 2 * e + 1];
          }
        }
      }
    }
  } else {
    const __nv_bfloat16* wrow = static_cast<const __nv_bfloat16*>(wdata) + static_cast<size_t>(n) * K;
    for (int k0 = lane * 8; k0 < K; k0 += 256) {
      const uint4 wv = __ldg(reinterpret_cast<const uint4*>(wrow + k0));
      const uint32_t* wu = reinterpret_cast<const uint32_t*>(&wv);
      float wf[8];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = unpack_bf162(wu[e]);
        wf[2 * e] = f.x;
        wf[2 * e + 1] = f.y;
      }
#pragma unroll
      for (int m = 0; m < MT; ++m) {
        const uint4 xv = *reinterpret_cast<const uint4*>(x + static_cast<size_t>(m) * ldx + k0);
        const uint32_t* xu = reinterpret_cast<const uint32_t*>(&xv);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = unpack_bf162(xu[e]);
          acc[m] += f.x * wf[2 * e] + f.y * wf[2 * e + 1];
        }
      }
    }
  }
#pragma unroll
  for (int m = 0; m < MT; ++m) acc[m] = warp_sum(acc[m]);
  if (lane == 0) {
    const float b = bias ? bias[n] : 0.f;
#pragma unroll
    for (int m = 0; m < MT; ++m) {
      if (out_f32) static_cast<float*>(out)[static_cast<size_t>(m) * ldo + n] = acc[m] + b;
      else static_cast<__nv_bfloat16*>(out)[static_cast<size_t>(m) * ldo + n] = f2bf(acc[m] + b);
    }
  }
}

// ------------------------------------------------------------------------------------------------ grouped CUDA-core GEMV
// Fine-grained mixture-of-experts decode: dozens of experts with one to eight rows each. The tensor-core kernel pays ~5 us
// of fixed cost per CTA on every (expert, tile) pair; here one warp owns one weight row of one work item and multiplies it
// with the item's (up to MT) token rows, so a work item costs a few hundred instructions and the kernel is bound by the
// weight stream. grid (ceil(N / 32), max_items), 4 warps x 8 weight rows each (a CTA per weight row would spend more time
// being launched than working); items as built by launch_moe_items with bn == MT.
constexpr int kGemvRowsPerWarp = 8;
bool g_gemv_simt_only = false;  // comparison switch: keep grouped JQ4 work items on the CUDA-core kernel
template <int MT, bool Q4>
__global__ void __launch_bounds__(128) gemv_grouped_kernel(const void* __restrict__ wdata, const __nv_bfloat16* __restrict__ x, int ldx,
                                                           __nv_bfloat16* __restrict__ out, int ldo, int N, int K,
                                                           const int4* __restrict__ items) {
  pdl_wait();
  pdl_trigger();
  const int4 it = items[blockIdx.y];
  if (it.x < 0) return;
  const int lane = threadIdx.x & 31;
  const int r0 = it.y;
  const int cnt = min(MT, it.z - it.y);
  for (int rw = 0; rw < kGemvRowsPerWarp; ++rw) {
  const int n = (blockIdx.x * 4 + (threadIdx.x >> 5)) * kGemvRowsPerWarp + rw;
  if (n >= N) return;
  float acc[MT];
#pragma unroll
  for (int m = 0; m < MT; ++m) acc[m] = 0.f;
  if (Q4) {
    const int kb_total = (K + 127) / 128;
    const int n_tiles = (N + 127) / 128;
    const int r = n & 127;
    const uint8_t* tile_row = static_cast<const uint8_t*>(wdata) + (static_cast<size_t>(it.x) * n_tiles + (n >> 7)) * kb_total * kQ4StageBytes;
    for (int blk = lane; blk < K / 32; blk += 32) {
      const uint8_t* stage = tile_row + static_cast<size_t>(blk >> 2) * kQ4StageBytes;
      const uint4 w = __ldg(reinterpret_cast<const uint4*>(stage + r * 64 + (((blk & 3) ^ ((r >> 1) & 3)) << 4)));
      const float sc = __ldg(reinterpret_cast<const float*>(stage + 8192 + r * 16 + (blk & 3) * 4));
      const uint32_t words[4] = {w.x, w.y, w.z, w.w};
      float wf[32];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
#pragma unroll
        for (int b = 0; b < 4; ++b) {
          const uint32_t byte = (words[i] >> (8 * b)) & 0xFFu;
          wf[4 * i + b] = static_cast<float>(static_cast<int>(byte & 0xFu) - 8) * sc;
          wf[16 + 4 * i + b] = static_cast<float>(static_cast<int>(byte >> 4) - 8) * sc;
        }
      }
#pragma unroll
      for (int m = 0; m < MT; ++m) {
        if (m < cnt) {
          const __nv_bfloat16* xr = x + static_cast<size_t>(r0 + m) * ldx + blk * 32;
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const uint4 xv = *reinterpret_cast<const uint4*>(xr + c * 8);
            const uint32_t* xu = reinterpret_cast<const uint32_t*>(&xv);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float2 f = unpack_bf162(xu[e]);
              acc[m] += f.x * wf[c * 8 + 2 * e] + f.y * wf[c * 8 + 2 * e + 1];
            }
          }
        }
      }
    }
  } else {
    const __nv_bfloat16* wrow = static_cast<const __nv_bfloat16*>(wdata) + (static_cast<size_t>(it.x) * N + n) * K;
    for (int k0 = lane * 8; k0 < K; k0 += 256) {
      const uint4 wv = __ldg(reinterpret_cast<const uint4*>(wrow + k0));
      const uint32_t* wu = reinterpret_cast<const uint32_t*>(&wv);
      float wf[8];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = unpack_bf162(wu[e]);
        wf[2 * e] = f.x;
        wf[2 * e + 1] = f.y;
      }
#pragma unroll
      for (int m = 0; m < MT; ++m) {
        if (m < cnt) {
          const uint4 xv = *reinterpret_cast<const uint4*>(x + static_cast<size_t>(r0 + m) * ldx + k0);
          const uint32_t* xu = reinterpret_cast<const uint32_t*>(&xv);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 f = unpack_bf162(xu[e]);
            acc[m] += f.x * wf[2 * e] + f.y * wf[2 * e + 1];
          }
        }
      }
    }
  }
#pragma unroll
  for (int m = 0; m < MT; ++m) acc[m] = warp_sum(acc[m]);
  if (lane == 0) {
#pragma unroll
    for (int m = 0; m < MT; ++m)
      if (m < cnt) out[static_cast<size_t>(r0 + m) * ldo + n] = f2bf(acc[m]);
  }
  }
}

// ------------------------------------------------------------------------------------------------ grouped JQ4 GEMV on mma.sync
// The CUDA-core kernel above spends ~200 instructions per 16 bytes of packed weights (nibble -> float conversion, one FMA per
// token and element) and stays far below the HBM rate. Here a warp owns 16 weight rows of one work item and multiplies them with
// the item's up to 8 token rows on the tensor cores (mma.sync m16n8k16, bf16 x bf16 -> fp32): the weights are the 16 x 16 A
// operand, the tokens the 16 x 8 B operand. (tcgen05 needs 128-row tiles and several microseconds of set-up per CTA, which is what
// rules it out for work items of one to eight rows.)
// Operand mapping: inside a 128-wide k-block lane (g, c) = (lane / 4, lane % 4) loads the whole 32-element block c of weight rows
// g and g + 8 (one 16-byte load each: no lane fetches less than a sector's half) and the same 32 elements of token g. Each of the
// 8 MMAs per k-block takes 4 of those elements per lane; since A and B use the same assignment of elements to the instruction's k
// positions, the order in which the 128 products are summed is all that differs from the plain layout.
template <int ACT>
__device__ __forceinline__ float gated_act(float g) {
  if (ACT == 2) return 0.5f * g * (1.f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g)));
  return g / (1.f + __expf(-g));
}
__device__ __forceinline__ void mma_bf16_m16n8k16(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// ACT > 0 (gate | up projection of a gated MLP, N = 2 I rows: gate rows first): the warp's 16 rows are 8 gate rows and the 8 up rows
// of the same outputs, and the epilogue stores act(gate) * up as [rows, I]: the [rows, 2 I] intermediate and the activation
// kernel disappear. ACT: 1 = SiLU, 2 = tanh-approximated GELU, 3 = exact GELU.
// (Two warps per row group on alternate k-blocks, i.e. twice as many CTAs of half the length, to trim the partly filled last wave of
// the 2048-deep gate | up projection of 128 experts: measured no faster, 7.63 against 7.58 ms per decode step, and not kept.)
constexpr int kGemvMmaWarps = 4;
template <int ACT>
__global__ void __launch_bounds__(kGemvMmaWarps * 32) gemv_grouped_mma_kernel(const uint8_t* __restrict__ wdata, const __nv_bfloat16* __restrict__ x, int ldx,
                                                                               __nv_bfloat16* __restrict__ out, int ldo, int N, int K,
                                                                               const int4* __restrict__ items, const int* __restrict__ row_map,
                                                                               int row_div) {
  // row_map (optional): grouped row r reads the token row row_map[r] / row_div of x instead of row r, i.e. x is the ungathered
  // [tokens, K] activation and row_map the grouping permutation (the copy into expert order never happens)
  pdl_wait();
  pdl_trigger();
  const int4 it = items[blockIdx.y];
  if (it.x < 0) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, c = lane & 3;
  constexpr int RW = ACT > 0 ? 8 : 16;  // output rows per warp
  const int n_out = ACT > 0 ? N / 2 : N;
  const int n0 = (blockIdx.x * kGemvMmaWarps + warp) * RW;
  if (n0 >= n_out) return;
  const int r0 = it.y, cnt = min(8, it.z - it.y);
  const int kb_total = K / 128, n_tiles = (N + 127) / 128;
  const int nA = n0 + g, nB = ACT > 0 ? n_out + n0 + g : n0 + g + 8;  // weight rows behind accumulator rows g and g + 8
  const int rA = nA & 127, rB = nB & 127;
  const uint8_t* base = wdata + (static_cast<size_t>(it.x) * n_tiles + (nA >> 7)) * kb_total * kQ4StageBytes;
  const size_t tileB = static_cast<size_t>((nB >> 7) - (nA >> 7)) * kb_total * kQ4StageBytes;
  const uint32_t offA = rA * 64 + ((c ^ ((rA >> 1) & 3)) << 4);
  const size_t offB = tileB + rB * 64 + ((c ^ ((rB >> 1) & 3)) << 4);
  const uint32_t scA = 8192 + rA * 16 + c * 4;
  const size_t scB = tileB + 8192 + rB * 16 + c * 4;
  const bool tok = g < cnt;
  const int xr = r0 + (tok ? g : 0);
  const __nv_bfloat16* xrow = x + static_cast<size_t>(row_map != nullptr ? row_map[xr] / row_div : xr) * ldx + c * 32;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  // (Measured: keeping the weight loads of four k-blocks ahead in registers made the kernel slower, 86 instead of 59 us for the
  // gate | up projection of 128 experts: the 106 registers halve the resident warps, and what limits the kernel is the issue
  // rate of the nibble expansion, not the bytes in flight.)
#pragma unroll 2
  for (int kb = 0; kb < kb_total; ++kb) {
    const uint8_t* stage = base + static_cast<size_t>(kb) * kQ4StageBytes;
    const uint4 wa = __ldg(reinterpret_cast<const uint4*>(stage + offA));
    const uint4 wb = __ldg(reinterpret_cast<const uint4*>(stage + offB));
    const float sa = __ldg(reinterpret_cast<const float*>(stage + scA));
    const float sb = __ldg(reinterpret_cast<const float*>(stage + scB));
    uint4 xv[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) xv[j] = tok ? *reinterpret_cast<const uint4*>(xrow + kb * 128 + j * 8) : make_uint4(0u, 0u, 0u, 0u);
    const __nv_bfloat162 s2a = __float2bfloat162_rn(sa), s2b = __float2bfloat162_rn(sb);
    const uint32_t wwa[4] = {wa.x, wa.y, wa.z, wa.w}, wwb[4] = {wb.x, wb.y, wb.z, wb.w};
    const uint32_t* xu = reinterpret_cast<const uint32_t*>(xv);  // word j = elements 2 j, 2 j + 1 of the block
#pragma unroll
    for (int hl = 0; hl < 2; ++hl) {
#pragma unroll
      for (int wd = 0; wd < 4; ++wd) {
        // elements e0 .. e0 + 3 of the block, e0 = 16 hl + 4 wd: low (hl = 0) or high nibbles of the bytes of word wd
        const uint32_t na = (wwa[wd] >> (4 * hl)) & 0x0F0F0F0Fu, nb = (wwb[wd] >> (4 * hl)) & 0x0F0F0F0Fu;
        uint32_t a[4];
        a[0] = q4_pair_to_bf162(na, 0x4140u, s2a);
        a[1] = q4_pair_to_bf162(nb, 0x4140u, s2b);
        a[2] = q4_pair_to_bf162(na, 0x4342u, s2a);
        a[3] = q4_pair_to_bf162(nb, 0x4342u, s2b);
        mma_bf16_m16n8k16(acc, a, xu[hl * 8 + 2 * wd], xu[hl * 8 + 2 * wd + 1]);
      }
    }
  }
  // accumulator: rows g and g + 8, token columns 2 c and 2 c + 1
  const int t0 = 2 * c;
  if (ACT > 0) {
    // the intermediate is rounded to bf16 as the separate activation kernel sees it
    if (t0 < cnt) out[static_cast<size_t>(r0 + t0) * ldo + n0 + g] = f2bf(gated_act<ACT>(bf2f(f2bf(acc[0]))) * bf2f(f2bf(acc[2])));
    if (t0 + 1 < cnt) out[static_cast<size_t>(r0 + t0 + 1) * ldo + n0 + g] = f2bf(gated_act<ACT>(bf2f(f2bf(acc[1]))) * bf2f(f2bf(acc[3])));
    return;
  }
  if (t0 < cnt) {
    out[static_cast<size_t>(r0 + t0) * ldo + n0 + g] = f2bf(acc[0]);
    out[static_cast<size_t>(r0 + t0) * ldo + n0 + g + 8] = f2bf(acc[2]);
  }
  if (t0 + 1 < cnt) {
    out[static_cast<size_t>(r0 + t0 + 1) * ldo + n0 + g] = f2bf(acc[1]);
    out[static_cast<size_t>(r0 + t0 + 1) * ldo + n0 + g + 8] = f2bf(acc[3]);
  }
}

// ------------------------------------------------------------------------------------------------ dense JQ4 GEMV for 1..8 tokens
// The same operand mapping for an ordinary projection with at most 8 token rows (single requests and small decode batches). These
// GEMMs move a few megabytes, so what counts is how many warps stream at once and how little is set up per launch: the tcgen05 kernel
// pays its prologue and epilogue per CTA (10-12 us per projection at one token). One CTA per 16 weight rows (8 with the gated
// activation), its S warps take interleaved k-blocks and add their partial tiles through shared memory.
// S (4, 8 or 16) is chosen per shape by gemv_pick_split: the time of these kernels is (waves of CTAs) x (k-blocks per warp), and
// both are whole numbers. The gate | up projection of Qwen3-4B (1216 CTAs, 20 k-blocks) with S = 8 ran 2.05 waves of 592 resident
// CTAs (64 registers: four CTAs of 256 threads per SM) with 3 k-blocks on the slowest warp, 9 k-block times in all; with S = 4 and
// at most 56 registers nine CTAs of 128 threads fit per SM, all 1216 are resident at once and every warp has 5 k-blocks. Narrow
// deep projections (160 CTAs, 32 or 76 k-blocks) take S = 16 instead: half the k-blocks per warp, still one wave.
// ACT as above; OUTF: fp32 output (the output head's logits).
// TG: groups of 8 token rows (1: up to 8 rows, 2: 9..16 rows; the expanded weight fragment feeds one MMA per group). Two groups
// are tested but not used by default (g_gemv_max_rows).
template <int S, int TG>
constexpr int gemv_resident() {  // CTAs per SM the register budget is set for
  return TG == 1 ? (S == 4 ? 9 : (S == 8 ? 4 : 2)) : (S == 4 ? 6 : (S == 8 ? 3 : 1));
}
template <int ACT, bool OUTF, int S, int TG>
__global__ void __launch_bounds__(S * 32, gemv_resident<S, TG>()) gemv_dense_mma_kernel(const uint8_t* __restrict__ wdata, const __nv_bfloat16* __restrict__ x,
                                                                                         int ldx, void* __restrict__ out, int ldo,
                                                                                         const float* __restrict__ bias, int M, int N, int K) {
  constexpr int kGemvSplit = S;
  __shared__ float part[kGemvSplit][TG][32][4];
  pdl_wait();
  pdl_trigger();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, c = lane & 3;
  constexpr int RW = ACT > 0 ? 8 : 16;
  const int n_out = ACT > 0 ? N / 2 : N;
  const int n0 = blockIdx.x * RW;
  const int kb_total = K / 128;
  const int nA = min(n0 + g, N - 1), nB = min(ACT > 0 ? n_out + n0 + g : n0 + g + 8, N - 1);  // (rows past the end are computed and dropped)
  const int rA = nA & 127, rB = nB & 127;
  const uint8_t* baseA = wdata + static_cast<size_t>(nA >> 7) * kb_total * kQ4StageBytes;
  const uint8_t* baseB = wdata + static_cast<size_t>(nB >> 7) * kb_total * kQ4StageBytes;
  const uint32_t offA = rA * 64 + ((c ^ ((rA >> 1) & 3)) << 4), offB = rB * 64 + ((c ^ ((rB >> 1) & 3)) << 4);
  const uint32_t scA = 8192 + rA * 16 + c * 4, scB = 8192 + rB * 16 + c * 4;
  bool tok[TG];
  const __nv_bfloat16* xrow[TG];
  float acc[TG][4];
#pragma unroll
  for (int t = 0; t < TG; ++t) {
    tok[t] = g + 8 * t < M;
    xrow[t] = x + static_cast<size_t>(tok[t] ? g + 8 * t : 0) * ldx + c * 32;
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[t][i] = 0.f;
  }
#pragma unroll 2
  for (int kb = warp; kb < kb_total; kb += kGemvSplit) {
    const size_t so = static_cast<size_t>(kb) * kQ4StageBytes;
    const uint4 wa = __ldg(reinterpret_cast<const uint4*>(baseA + so + offA));
    const uint4 wb = __ldg(reinterpret_cast<const uint4*>(baseB + so + offB));
    const float sa = __ldg(reinterpret_cast<const float*>(baseA + so + scA));
    const float sb = __ldg(reinterpret_cast<const float*>(baseB + so + scB));
    uint4 xv[TG][4];
#pragma unroll
    for (int t = 0; t < TG; ++t)
#pragma unroll
      for (int j = 0; j < 4; ++j) xv[t][j] = tok[t] ? *reinterpret_cast<const uint4*>(xrow[t] + kb * 128 + j * 8) : make_uint4(0u, 0u, 0u, 0u);
    const __nv_bfloat162 s2a = __float2bfloat162_rn(sa), s2b = __float2bfloat162_rn(sb);
    const uint32_t wwa[4] = {wa.x, wa.y, wa.z, wa.w}, wwb[4] = {wb.x, wb.y, wb.z, wb.w};
#pragma unroll
    for (int hl = 0; hl < 2; ++hl) {
#pragma unroll
      for (int wd = 0; wd < 4; ++wd) {
        const uint32_t na = (wwa[wd] >> (4 * hl)) & 0x0F0F0F0Fu, nb = (wwb[wd] >> (4 * hl)) & 0x0F0F0F0Fu;
        uint32_t a[4];
        a[0] = q4_pair_to_bf162(na, 0x4140u, s2a);
        a[1] = q4_pair_to_bf162(nb, 0x4140u, s2b);
        a[2] = q4_pair_to_bf162(na, 0x4342u, s2a);
        a[3] = q4_pair_to_bf162(nb, 0x4342u, s2b);
#pragma unroll
        for (int t = 0; t < TG; ++t) {
          const uint32_t* xu = reinterpret_cast<const uint32_t*>(xv[t]);
          mma_bf16_m16n8k16(acc[t], a, xu[hl * 8 + 2 * wd], xu[hl * 8 + 2 * wd + 1]);
        }
      }
    }
  }
#pragma unroll
  for (int t = 0; t < TG; ++t)
#pragma unroll
    for (int i = 0; i < 4; ++i) part[warp][t][lane][i] = acc[t][i];
  __syncthreads();
  if (warp != 0) return;
#pragma unroll
  for (int w2 = 1; w2 < kGemvSplit; ++w2)
#pragma unroll
    for (int t = 0; t < TG; ++t)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[t][i] += part[w2][t][lane][i];
  // accumulator of group t: rows g and g + 8, token columns 8 t + 2 c and 8 t + 2 c + 1
  auto store = [&](int t, int n, float v) {
    if (t >= M || n >= n_out) return;
    if (OUTF) static_cast<float*>(out)[static_cast<size_t>(t) * ldo + n] = v;
    else static_cast<__nv_bfloat16*>(out)[static_cast<size_t>(t) * ldo + n] = f2bf(v);
  };
  const float b0 = ACT == 0 && bias != nullptr && n0 + g < N ? bias[n0 + g] : 0.f;
  const float b1 = ACT == 0 && bias != nullptr && n0 + g + 8 < N ? bias[n0 + g + 8] : 0.f;
#pragma unroll
  for (int t = 0; t < TG; ++t) {
    const int t0 = 8 * t + 2 * c;
    if (ACT > 0) {
      store(t0, n0 + g, gated_act<ACT>(bf2f(f2bf(acc[t][0]))) * bf2f(f2bf(acc[t][2])));
      store(t0 + 1, n0 + g, gated_act<ACT>(bf2f(f2bf(acc[t][1]))) * bf2f(f2bf(acc[t][3])));
    } else {
      store(t0, n0 + g, acc[t][0] + b0);
      store(t0 + 1, n0 + g, acc[t][1] + b0);
      store(t0, n0 + g + 8, acc[t][2] + b1);
      store(t0 + 1, n0 + g + 8, acc[t][3] + b1);
    }
  }
}

bool g_gemv_dense = true;  // small batches of JQ4 projections on the mma.sync GEMV instead of the tcgen05 kernel
// Most token rows it takes. The kernel handles up to 16 (two groups of 8), but measured on the Qwen3-4B shape at 16 sequences the
// tcgen05 kernel is the faster one (3.12 against 3.54 ms per decode step), so the default stays at one group.
int g_gemv_max_rows = 8;
bool gemv_dense_supported(const GemmWeightDesc* w, int M, int ldx) {
  return g_gemv_dense && !g_gemv_simt_only && w->is_q4 && M >= 1 && M <= g_gemv_max_rows && M <= 16 && w->K % 128 == 0 && w->K >= 128 && ldx % 8 == 0;
}
// Warps per CTA that split K: the candidate with the fewest (waves x k-blocks per warp); ties go to the wider split (more loads in flight).
int g_gemv_force_split = 0;  // tests: 4, 8 or 16
static int gemv_pick_split(int ctas, int kb_total, int tg) {
  if (g_gemv_force_split == 4 || g_gemv_force_split == 8 || g_gemv_force_split == 16) return g_gemv_force_split;
  const int sms = gemm_num_sms();
  const int cand[3] = {4, 8, 16};
  const int resident[3] = {tg == 1 ? gemv_resident<4, 1>() : gemv_resident<4, 2>(), tg == 1 ? gemv_resident<8, 1>() : gemv_resident<8, 2>(),
                           tg == 1 ? gemv_resident<16, 1>() : gemv_resident<16, 2>()};
  int best = 8;
  long long best_cost = -1;
  for (int i = 0; i < 3; ++i) {
    const long long slots = static_cast<long long>(sms) * resident[i];
    const long long cost = ((ctas + slots - 1) / slots) * ((kb_total + cand[i] - 1) / cand[i]);
    if (best_cost < 0 || cost <= best_cost) {
      best_cost = cost;
      best = cand[i];
    }
  }
  return best;
}
template <int ACT, bool OUTF, int TG>
static void gemv_dense_launch_tg(int split, dim3 grid, cudaStream_t st, const uint8_t* wd, const __nv_bfloat16* xp, int ldx, void* out, int ldo,
                                 const float* bias, int M, int N, int K) {
  cudaError_t e;
  if (split == 4) e = launch_pdl(gemv_dense_mma_kernel<ACT, OUTF, 4, TG>, grid, dim3(128), 0, st, wd, xp, ldx, out, ldo, bias, M, N, K);
  else if (split == 16) e = launch_pdl(gemv_dense_mma_kernel<ACT, OUTF, 16, TG>, grid, dim3(512), 0, st, wd, xp, ldx, out, ldo, bias, M, N, K);
  else e = launch_pdl(gemv_dense_mma_kernel<ACT, OUTF, 8, TG>, grid, dim3(256), 0, st, wd, xp, ldx, out, ldo, bias, M, N, K);
  if (e != cudaSuccess) throw std::runtime_error(std::string("small-batch gemv launch: ") + cudaGetErrorString(e));
}
template <int ACT, bool OUTF>
static void gemv_dense_launch(dim3 grid, cudaStream_t st, const uint8_t* wd, const __nv_bfloat16* xp, int ldx, void* out, int ldo, const float* bias,
                              int M, int N, int K) {
  const int tg = M > 8 ? 2 : 1;
  const int split = gemv_pick_split(static_cast<int>(grid.x), K / 128, tg);
  if (tg == 2) gemv_dense_launch_tg<ACT, OUTF, 2>(split, grid, st, wd, xp, ldx, out, ldo, bias, M, N, K);
  else gemv_dense_launch_tg<ACT, OUTF, 1>(split, grid, st, wd, xp, ldx, out, ldo, bias, M, N, K);
}
// act: 0 plain (bias, bf16 or fp32 output), 1 / 2: w holds gate | up rows (N = 2 I), out is [M, I] bf16
void gemv_dense_run(const GemmWeightDesc* w, const void* x, int M, int ldx, void* out, int ldo, bool out_f32, const float* bias, int act,
                    cudaStream_t st) {
  const uint8_t* wd = static_cast<const uint8_t*>(w->data);
  const __nv_bfloat16* xp = static_cast<const __nv_bfloat16*>(x);
  if (act == 1 || act == 2) {
    const dim3 grid((w->N / 2 + 7) / 8);
    if (act == 1) gemv_dense_launch<1, false>(grid, st, wd, xp, ldx, out, ldo, bias, M, w->N, w->K);
    else gemv_dense_launch<2, false>(grid, st, wd, xp, ldx, out, ldo, bias, M, w->N, w->K);
    return;
  }
  const dim3 grid((w->N + 15) / 16);
  if (out_f32) gemv_dense_launch<0, true>(grid, st, wd, xp, ldx, out, ldo, bias, M, w->N, w->K);
  else gemv_dense_launch<0, false>(grid, st, wd, xp, ldx, out, ldo, bias, M, w->N, w->K);
}

void gemv_grouped_run(const GemmWeightDesc* w, int n_per_expert, const void* x, int ldx, void* out, int ldo, const int* items,
                      int max_items, int mt, cudaStream_t st) {
  if (max_items <= 0) return;
  if (ldx % 8 != 0 || w->K % 8 != 0) throw std::runtime_error("grouped gemv needs 16-byte aligned rows");
  if (max_items > 65535) throw std::runtime_error("grouped gemv: work list too long");
  const dim3 grid((n_per_expert + 4 * kGemvRowsPerWarp - 1) / (4 * kGemvRowsPerWarp), max_items);
  const int4* it = reinterpret_cast<const int4*>(items);
  const __nv_bfloat16* xp = static_cast<const __nv_bfloat16*>(x);
  __nv_bfloat16* op = static_cast<__nv_bfloat16*>(out);
  if (w->is_q4 && w->K % 128 == 0 && n_per_expert % 16 == 0 && mt <= 8 && !g_gemv_simt_only) {
    const dim3 grid_mma((n_per_expert / 16 + kGemvMmaWarps - 1) / kGemvMmaWarps, max_items);
    launch_pdl(gemv_grouped_mma_kernel<0>, grid_mma, dim3(kGemvMmaWarps * 32), 0, st, static_cast<const uint8_t*>(w->data), xp, ldx, op, ldo, n_per_expert,
               w->K, it, static_cast<const int*>(nullptr), 1);
    return;
  }
#define DLV_GG(MTV)                                                                                                                 \
  if (w->is_q4) launch_pdl(gemv_grouped_kernel<MTV, true>, grid, dim3(128), 0, st, w->data, xp, ldx, op, ldo, n_per_expert, w->K, it); \
  else launch_pdl(gemv_grouped_kernel<MTV, false>, grid, dim3(128), 0, st, w->data, xp, ldx, op, ldo, n_per_expert, w->K, it)
  switch (mt) {
    case 4: DLV_GG(4); break;
    case 8: DLV_GG(8); break;
    default: throw std::runtime_error("grouped gemv: rows per item must be 4 or 8");
  }
#undef DLV_GG
}

// Gate | up projection of the work items (n_per_expert = 2 I weight rows per expert, gate rows first) with act(gate) * up in the
// epilogue; out is [rows, I]. Returns false when the shape is outside the mma.sync kernel (the caller then runs the two steps).
bool gemv_grouped_act_run(const GemmWeightDesc* w, int n_per_expert, const void* x, int ldx, void* out, int ldo, const int* items, int max_items,
                          int act, const int* row_map, int row_div, cudaStream_t st) {
  if (!w->is_q4 || w->K % 128 != 0 || n_per_expert % 16 != 0 || ldx % 8 != 0 || (act != 1 && act != 2) || g_gemv_simt_only) return false;
  if (max_items <= 0) return true;
  if (max_items > 65535) throw std::runtime_error("grouped gemv: work list too long");
  const int inter = n_per_expert / 2;
  const dim3 grid((inter / 8 + kGemvMmaWarps - 1) / kGemvMmaWarps, max_items);
  const int4* it = reinterpret_cast<const int4*>(items);
  const __nv_bfloat16* xp = static_cast<const __nv_bfloat16*>(x);
  __nv_bfloat16* op = static_cast<__nv_bfloat16*>(out);
  if (act == 1) launch_pdl(gemv_grouped_mma_kernel<1>, grid, dim3(kGemvMmaWarps * 32), 0, st, static_cast<const uint8_t*>(w->data), xp, ldx, op, ldo, n_per_expert, w->K, it, row_map, row_div);
  else launch_pdl(gemv_grouped_mma_kernel<2>, grid, dim3(kGemvMmaWarps * 32), 0, st, static_cast<const uint8_t*>(w->data), xp, ldx, op, ldo, n_per_expert, w->K, it, row_map, row_div);
  return true;
}

// (A CUDA-core kernel for dense bf16 projections with few output rows and a decode-size batch, one warp per weight row and group of
// 8 tokens, was tried for the mixture-of-experts router (128 x 2048, 32 tokens) in place of the tcgen05 tile and measured slower:
// 8.35 against 7.59 ms per decode step of the Qwen3-30B-A3B shape. Such projections stay on the tcgen05 kernel.)
void gemv_simt_run(const GemmWeightDesc* w, const void* x, int M, int ldx, void* out, int ldo, bool out_f32, const float* bias,
                   cudaStream_t st) {
  const unsigned grid = (w->N + 3) / 4;
  for (int m0 = 0; m0 < M; m0 += 4) {
    const int mt = M - m0 < 4 ? M - m0 : 4;
    const __nv_bfloat16* xp = static_cast<const __nv_bfloat16*>(x) + static_cast<size_t>(m0) * ldx;
    void* op = out_f32 ? static_cast<void*>(static_cast<float*>(out) + static_cast<size_t>(m0) * ldo)
                       : static_cast<void*>(static_cast<__nv_bfloat16*>(out) + static_cast<size_t>(m0) * ldo);
#define DLV_GEMV(MT)                                                                                                          \
  if (w->is_q4) gemv_simt_kernel<MT, true><<<grid, 128, 0, st>>>(w->data, xp, ldx, op, ldo, out_f32, bias, w->N, w->K); \
  else gemv_simt_kernel<MT, false><<<grid, 128, 0, st>>>(w->data, xp, ldx, op, ldo, out_f32, bias, w->N, w->K)
    switch (mt) {
      case 1: DLV_GEMV(1); break;
      case 2: DLV_GEMV(2); break;
      case 3: DLV_GEMV(3); break;
      default: DLV_GEMV(4); break;
    }
#undef DLV_GEMV
  }
}

}  // namespace dlv
