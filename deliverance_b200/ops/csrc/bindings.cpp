// torch <-> kernel-launcher glue. Every entry validates device, dtype, contiguity and alignment on the host before a
// launch (no kernel is started on arguments that could fault), and launches on the current CUDA stream.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <memory>
#include <mutex>
#include <unordered_map>

#include "chain_api.h"
#include "gemm_api.h"

namespace {

using torch::Tensor;

inline cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }

void check_cuda(const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
  TORCH_CHECK(t.is_contiguous(), name, " must be contiguous");
}
void check_bf16(const Tensor& t, const char* name) {
  check_cuda(t, name);
  TORCH_CHECK(t.scalar_type() == at::kBFloat16, name, " must be bfloat16");
}
void check_last_error(const char* what) {
  cudaError_t e = cudaGetLastError();
  TORCH_CHECK(e == cudaSuccess, what, ": ", cudaGetErrorString(e));
}
int act_code(const std::string& a) {
  if (a == "silu" || a == "swish") return 0;
  if (a == "gelu_pytorch_tanh" || a == "gelu_new" || a == "gelu_tanh" || a == "gelu_fast") return 1;
  if (a == "gelu") return 2;
  if (a == "relu") return 3;
  if (a == "tanh") return 4;
  TORCH_CHECK(false, "unknown activation ", a);
}

// ---- output allocation with optional guard areas ---------------------------------------------------------------------
// Bounds checking (set_bounds_check(true), or DLV_BOUNDS_CHECK=1 in the environment when the module loads): every tensor a
// kernel of this extension writes its result into is cut out of a larger buffer, between two 4 KB guard areas filled with a byte
// pattern. check_guards() compares all guard areas written since the last call with the pattern and reports the outputs
// whose neighbourhood a kernel overwrote. Off (the default), an output is a plain torch::empty.
constexpr int64_t kGuardBytes = 4096;
constexpr uint8_t kGuardByte = 0xA5;
struct GuardRecord {
  Tensor buf;
  int64_t body_bytes;
  std::string what;
};
bool g_bounds_check = false;
std::vector<GuardRecord> g_guards;

Tensor new_out(c10::IntArrayRef sizes, const torch::TensorOptions& opt) {
  if (!g_bounds_check) return torch::empty(sizes, opt);
  const std::vector<int64_t> shape(sizes.begin(), sizes.end());  // (the caller's list is a temporary)
  const at::ScalarType dt = c10::typeMetaToScalarType(opt.dtype());
  int64_t n = 1;
  for (int64_t v : shape) n *= v;
  const int64_t body = n * static_cast<int64_t>(c10::elementSize(dt));
  if (body == 0) return torch::empty(shape, opt);
  const int64_t padded = (body + 255) / 256 * 256;
  const std::vector<int64_t> total{kGuardBytes + padded + kGuardBytes};
  Tensor buf = torch::empty(total, opt.dtype(at::kByte));
  buf.fill_(static_cast<int64_t>(kGuardByte));
  Tensor out = buf.narrow(0, kGuardBytes, body).view(dt).view(shape);
  std::string what = "output " + std::to_string(g_guards.size()) + " [";
  for (size_t i = 0; i < shape.size(); ++i) what += (i ? ", " : "") + std::to_string(shape[i]);
  what += std::string("] ") + c10::toString(dt);
  GuardRecord rec;
  rec.buf = buf;
  rec.body_bytes = body;
  rec.what = what;
  g_guards.push_back(std::move(rec));
  return out;
}
void set_bounds_check(bool on) {
  g_bounds_check = on;
  if (!on) g_guards.clear();
}
// Names of the outputs whose guard areas no longer hold the pattern (the records are dropped either way).
std::vector<std::string> check_guards() {
  std::vector<std::string> bad;
  for (auto& r : g_guards) {
    const int64_t total = r.buf.numel();
    Tensor lo = r.buf.narrow(0, 0, kGuardBytes), hi = r.buf.narrow(0, kGuardBytes + r.body_bytes, total - kGuardBytes - r.body_bytes);
    if (lo.ne(kGuardByte).any().item<bool>() || hi.ne(kGuardByte).any().item<bool>()) bad.push_back(r.what);
  }
  g_guards.clear();
  return bad;
}
// Test hook: overwrite one guard byte of the newest output from the host side, to show that check_guards() sees it.
void poke_last_guard() {
  TORCH_CHECK(!g_guards.empty(), "no guarded output yet");
  g_guards.back().buf.narrow(0, kGuardBytes + g_guards.back().body_bytes + 7, 1).fill_(0);
}

// ---- per-device scratch for split-K partials, tile counters and the kernel status word ---------------------------
struct DeviceScratch {
  Tensor ws;        // fp32
  Tensor counters;  // int32, zero between launches
  Tensor status;    // int32 [1]
};
DeviceScratch& scratch_for(int device) {
  static std::unordered_map<int, DeviceScratch> table;
  auto it = table.find(device);
  if (it == table.end()) {
    DeviceScratch s;
    auto fopt = torch::TensorOptions().device(torch::kCUDA, device).dtype(torch::kFloat32);
    auto iopt = torch::TensorOptions().device(torch::kCUDA, device).dtype(torch::kInt32);
    s.ws = torch::empty({static_cast<long>(8) * 1024 * 1024}, fopt);  // 32 MB
    s.counters = torch::zeros({8192}, iopt);
    s.status = torch::zeros({1}, iopt);
    it = table.emplace(device, std::move(s)).first;
  }
  return it->second;
}

// ---- peer-memory state for the fused GEMM + all-reduce ------------------------------------------------------------
class TpComm {
 public:
  // recv_ptrs / flag_ptrs: device addresses of every rank's receive area and flag matrix as mapped in this process
  TpComm(int64_t rank, int64_t size, std::vector<int64_t> recv_ptrs, std::vector<int64_t> flag_ptrs, int64_t slab, int64_t ncta_max,
         Tensor rounds, Tensor call) {
    TORCH_CHECK(size >= 2 && size <= 8 && rank >= 0 && rank < size, "tensor-parallel size must be 2..8");
    TORCH_CHECK(static_cast<int64_t>(recv_ptrs.size()) == size && static_cast<int64_t>(flag_ptrs.size()) == size, "one pointer per rank");
    TORCH_CHECK(rounds.is_cuda() && rounds.scalar_type() == at::kInt && rounds.numel() >= ncta_max, "rounds must be int32 [ncta_max]");
    TORCH_CHECK(call.is_cuda() && call.scalar_type() == at::kInt && call.numel() >= 2, "call must be int32 [2]");
    args_.size = static_cast<int>(size);
    args_.rank = static_cast<int>(rank);
    args_.slab = slab;
    args_.ncta_max = static_cast<int>(ncta_max);
    for (int r = 0; r < 8; ++r) {
      args_.recv[r] = r < size ? static_cast<unsigned long long>(recv_ptrs[r]) : 0ull;
      args_.flags[r] = r < size ? static_cast<unsigned long long>(flag_ptrs[r]) : 0ull;
      TORCH_CHECK(r >= size || ((args_.recv[r] & 15) == 0 && (args_.flags[r] & 3) == 0 && args_.recv[r] != 0 && args_.flags[r] != 0), "bad peer pointer");
    }
    rounds_ = rounds;
    call_ = call;
    args_.rounds = reinterpret_cast<unsigned int*>(rounds.data_ptr<int>());
    args_.call = reinterpret_cast<unsigned int*>(call.data_ptr<int>());
  }
  const dlv::GemmTpArgs* args() const { return &args_; }
  // Bound of the peer-flag waits of the comm.cu kernels launched with this state, in milliseconds at a nominal 2 GHz (0: default).
  void set_wait_limit_ms(double ms) { args_.wait_limit_cycles = ms > 0 ? static_cast<long long>(ms * 2.0e6) : 0; }
  // NVSwitch multicast address of the receive area (every rank's area bound to one multicast object), 0 = not available
  void set_multicast(int64_t mc_recv) {
    TORCH_CHECK((mc_recv & 15) == 0, "multicast address must be 16-byte aligned");
    args_.mc_recv = static_cast<unsigned long long>(mc_recv);
  }
  bool has_multicast() const { return args_.mc_recv != 0; }
  dlv::GemmTpArgs with_mode(int mode) const {
    dlv::GemmTpArgs a = args_;
    a.mode = mode;
    return a;
  }

 private:
  dlv::GemmTpArgs args_;
  Tensor rounds_, call_;
};

// ---- peer-memory state for GEMM -> reduce-scatter -> all-gather (prefill-size batches) -----------------------------------
class TpScatter {
 public:
  // recv / gather / flag pointers: device addresses of every rank's areas as mapped in this process; capacities in bf16 elements
  TpScatter(int64_t rank, int64_t size, std::vector<int64_t> recv_ptrs, std::vector<int64_t> gather_ptrs, std::vector<int64_t> flag_ptrs,
            int64_t recv_elems, int64_t gather_elems) {
    TORCH_CHECK(size >= 2 && size <= 8 && rank >= 0 && rank < size, "tensor-parallel size must be 2..8");
    TORCH_CHECK(static_cast<int64_t>(recv_ptrs.size()) == size && static_cast<int64_t>(gather_ptrs.size()) == size &&
                    static_cast<int64_t>(flag_ptrs.size()) == size, "one pointer per rank");
    args_.size = static_cast<int>(size);
    args_.rank = static_cast<int>(rank);
    args_.recv_elems = recv_elems;
    args_.gather_elems = gather_elems;
    for (int r = 0; r < 8; ++r) {
      args_.recv[r] = r < size ? static_cast<unsigned long long>(recv_ptrs[r]) : 0ull;
      args_.gather[r] = r < size ? static_cast<unsigned long long>(gather_ptrs[r]) : 0ull;
      args_.flags[r] = r < size ? static_cast<unsigned long long>(flag_ptrs[r]) : 0ull;
      TORCH_CHECK(r >= size || ((args_.recv[r] & 15) == 0 && (args_.gather[r] & 15) == 0 && (args_.flags[r] & 3) == 0 && args_.recv[r] != 0 &&
                                args_.gather[r] != 0 && args_.flags[r] != 0), "bad peer pointer");
      group_cum_[r] = 0;
      gather_cum_[r] = 0;
    }
  }
  const dlv::GemmScatterArgs* args() const { return &args_; }
  // Advances the cumulative counters by one launch of this shape (every rank runs the same launches in the same order).
  void advance(const dlv::GemmScatterPlan& plan, bool gathered) {
    tile_cum_ += static_cast<unsigned>(plan.tiles[args_.rank]);
    if (gathered)
      for (int r = 0; r < args_.size; ++r) group_cum_[r] += static_cast<unsigned>(plan.groups[r]);
  }
  unsigned tile_target() const { return tile_cum_; }
  const unsigned* group_targets() const { return group_cum_; }
  // the same for one all-gather -> GEMM launch (its counters are separate from the reduce-scatter ones)
  void advance_gather(const dlv::GemmScatterPlan& plan) {
    for (int r = 0; r < args_.size; ++r) gather_cum_[r] += static_cast<unsigned>(plan.groups[r]);
  }
  const unsigned* gather_targets() const { return gather_cum_; }

 private:
  dlv::GemmScatterArgs args_;
  unsigned tile_cum_ = 0;
  unsigned group_cum_[8];
  unsigned gather_cum_[8];
};

// rows_per_rank, then rows / tiles / groups per rank: the cut of a launch of M rows and N columns over `size` ranks
std::vector<int64_t> scatter_plan(int64_t M, int64_t N, int64_t size) {
  TORCH_CHECK(size >= 1 && size <= 8 && M >= 0 && N > 0, "bad plan arguments");
  const dlv::GemmScatterPlan plan = dlv::gemm_scatter_plan(static_cast<int>(M), static_cast<int>(N), static_cast<int>(size));
  std::vector<int64_t> v{plan.rows_per_rank};
  for (int r = 0; r < size; ++r) v.push_back(plan.rows[r]);
  for (int r = 0; r < size; ++r) v.push_back(plan.tiles[r]);
  for (int r = 0; r < size; ++r) v.push_back(plan.groups[r]);
  return v;
}

// ---- GEMM weight handle -------------------------------------------------------------------------------------------
class GemmWeight {
 public:
  // dense: w bf16 [N, K]; JQ4: tile-packed uint8 [ceil(N/128), ceil(K/128), 10240] (ops.prepack_q4) with logical N, K
  GemmWeight(Tensor w, bool is_q4, int64_t N, int64_t K) {
    check_cuda(w, "weight");
    desc_.is_q4 = is_q4;
    if (is_q4) {
      TORCH_CHECK(w.scalar_type() == at::kByte && w.dim() == 3 && w.size(2) == dlv::kQ4StageBytes, "JQ4 weight must be tile-packed uint8 [nt, kb, 10240]");
      TORCH_CHECK(w.size(0) == (N + 127) / 128 && w.size(1) == (K + 127) / 128, "tile-packed shape does not match N, K");
    } else {
      TORCH_CHECK(w.scalar_type() == at::kBFloat16 && w.dim() == 2 && w.size(0) == N && w.size(1) == K, "dense weight must be bf16 [N, K]");
    }
    w_ = w;
    desc_.N = static_cast<int>(N);
    desc_.K = static_cast<int>(K);
    desc_.data = w.data_ptr();
    c10::cuda::CUDAGuard guard(w.device());
    dlv::gemm_weight_init(&desc_);
  }

  // out[m, :] = x[m, :] @ W^T (+ bias). impl: 0 = auto, 1 = tcgen05, 2 = CUDA-core GEMV
  Tensor run(const Tensor& x, c10::optional<Tensor> out_opt, c10::optional<Tensor> bias, bool out_f32, int64_t impl,
             int64_t force_splits) {
    TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kBFloat16 && x.dim() == 2, "x must be bf16 [M, K] on CUDA");
    TORCH_CHECK(x.size(1) == desc_.K && x.stride(1) == 1, "x inner dimension must be K and dense");
    TORCH_CHECK(x.stride(0) % 8 == 0 && (reinterpret_cast<uintptr_t>(x.data_ptr()) & 15) == 0, "x rows must be 16-byte aligned");
    TORCH_CHECK(x.device() == w_.device(), "x and weight live on different devices");
    c10::cuda::CUDAGuard guard(x.device());
    const int M = static_cast<int>(x.size(0));
    Tensor out;
    if (out_opt.has_value()) {
      out = out_opt.value();
      TORCH_CHECK(out.is_cuda() && out.dim() == 2 && out.size(0) == M && out.size(1) == desc_.N && out.stride(1) == 1, "bad out shape");
      TORCH_CHECK(out.scalar_type() == (out_f32 ? at::kFloat : at::kBFloat16), "bad out dtype");
    } else {
      out = new_out({M, desc_.N}, x.options().dtype(out_f32 ? at::kFloat : at::kBFloat16));
    }
    const float* bptr = nullptr;
    if (bias.has_value()) {
      const Tensor& b = bias.value();
      TORCH_CHECK(b.is_cuda() && b.scalar_type() == at::kFloat && b.numel() == desc_.N && b.is_contiguous(), "bias must be fp32 [N]");
      bptr = b.data_ptr<float>();
    }
    if (M == 0) return out;
    const bool simt = impl == 2 || (impl == 0 && M <= 1 && !desc_.is_q4);
    if (simt) {
      dlv::gemv_simt_run(&desc_, x.data_ptr(), M, static_cast<int>(x.stride(0)), out.data_ptr(), static_cast<int>(out.stride(0)), out_f32,
                         bptr, cur_stream());
    } else {
      DeviceScratch& s = scratch_for(x.device().index());
      dlv::gemm_tc_run(&desc_, x.data_ptr(), M, static_cast<int>(x.stride(0)), out.data_ptr(), static_cast<int>(out.stride(0)), out_f32,
                       bptr, s.ws.data_ptr<float>(), static_cast<size_t>(s.ws.numel()), s.counters.data_ptr<int>(),
                       static_cast<int>(s.counters.numel()), s.status.data_ptr<int>(), static_cast<int>(force_splits), cur_stream());
    }
    check_last_error("gemm launch");
    return out;
  }
  // Gate | up projection with act(gate) * up in the epilogue. `this` holds the gate and up rows interleaved per 128-row tile (64 gate
  // rows followed by the 64 up rows of the same outputs); returns [M, N / 2]. act: 1 = SiLU, 2 = tanh-approximated GELU.
  Tensor run_act(const Tensor& x, int64_t act) {
    TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kBFloat16 && x.dim() == 2 && x.size(1) == desc_.K && x.stride(1) == 1, "x must be bf16 [M, K]");
    TORCH_CHECK(x.stride(0) % 8 == 0 && (reinterpret_cast<uintptr_t>(x.data_ptr()) & 15) == 0, "x rows must be 16-byte aligned");
    TORCH_CHECK(desc_.N % 128 == 0, "gate|up rows must be a multiple of 128");
    c10::cuda::CUDAGuard guard(x.device());
    const int M = static_cast<int>(x.size(0));
    Tensor out = new_out({M, desc_.N / 2}, x.options());
    if (M == 0) return out;
    DeviceScratch& s = scratch_for(x.device().index());
    dlv::gemm_tc_run_act(&desc_, x.data_ptr(), M, static_cast<int>(x.stride(0)), out.data_ptr(), static_cast<int>(out.stride(0)), static_cast<int>(act),
                         s.ws.data_ptr<float>(), static_cast<size_t>(s.ws.numel()), s.counters.data_ptr<int>(),
                         static_cast<int>(s.counters.numel()), s.status.data_ptr<int>(), cur_stream());
    check_last_error("gemm (fused activation) launch");
    return out;
  }
  // 1..8 token rows through the mma.sync GEMV with act(gate) * up in its epilogue: `this` holds gate | up rows in plain order
  // (N = 2 I). Returns [M, I], or an undefined tensor when the shape is outside that kernel.
  Tensor run_gemv_act(const Tensor& x, int64_t act) {
    TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kBFloat16 && x.dim() == 2 && x.size(1) == desc_.K && x.stride(1) == 1, "x must be bf16 [M, K]");
    TORCH_CHECK((reinterpret_cast<uintptr_t>(x.data_ptr()) & 15) == 0, "x rows must be 16-byte aligned");
    const int M = static_cast<int>(x.size(0));
    if ((act != 1 && act != 2) || desc_.N % 16 != 0 || !dlv::gemv_dense_supported(&desc_, M, static_cast<int>(x.stride(0)))) return Tensor();
    c10::cuda::CUDAGuard guard(x.device());
    Tensor out = new_out({M, desc_.N / 2}, x.options());
    dlv::gemv_dense_run(&desc_, x.data_ptr(), M, static_cast<int>(x.stride(0)), out.data_ptr(), static_cast<int>(out.stride(0)), false, nullptr,
                        static_cast<int>(act), cur_stream());
    check_last_error("gemv (gated activation) launch");
    return out;
  }
  bool gemv_ok(int64_t M, int64_t ldx) const { return dlv::gemv_dense_supported(&desc_, static_cast<int>(M), static_cast<int>(ldx)); }
  // Grouped (MoE) GEMM: `this` stacks the local experts' weights (n_per_expert rows each; JQ4: whole 128-row tiles per expert),
  // xs holds rows sorted by expert, `items` comes from moe_items with the same token tile.
  Tensor run_grouped(const Tensor& xs, const Tensor& items, int64_t n_per_expert, int64_t bn, int64_t splits, c10::optional<Tensor> out_opt) {
    TORCH_CHECK(xs.is_cuda() && xs.scalar_type() == at::kBFloat16 && xs.dim() == 2 && xs.size(1) == desc_.K && xs.stride(1) == 1, "xs must be bf16 [rows, K]");
    TORCH_CHECK(xs.stride(0) % 8 == 0 && (reinterpret_cast<uintptr_t>(xs.data_ptr()) & 15) == 0, "xs rows must be 16-byte aligned");
    TORCH_CHECK(items.is_cuda() && items.scalar_type() == at::kInt && items.dim() == 2 && items.size(1) == 4 && items.is_contiguous(), "items must be int32 [n, 4]");
    const int64_t per = desc_.is_q4 ? ((n_per_expert + 127) / 128) * 128 : n_per_expert;
    TORCH_CHECK(n_per_expert > 0 && desc_.N % per == 0, "stacked weight rows are not a multiple of the per-expert rows");
    c10::cuda::CUDAGuard guard(xs.device());
    Tensor out = out_opt.has_value() ? out_opt.value() : new_out({xs.size(0), n_per_expert}, xs.options());
    TORCH_CHECK(out.is_cuda() && out.scalar_type() == at::kBFloat16 && out.dim() == 2 && out.size(0) == xs.size(0) && out.size(1) == n_per_expert && out.stride(1) == 1, "bad out");
    if (bn <= 8) {  // decode-size groups: CUDA-core GEMV, one warp per weight row and work item
      dlv::gemv_grouped_run(&desc_, static_cast<int>(n_per_expert), xs.data_ptr(), static_cast<int>(xs.stride(0)), out.data_ptr(),
                            static_cast<int>(out.stride(0)), items.data_ptr<int>(), static_cast<int>(items.size(0)), static_cast<int>(bn), cur_stream());
      check_last_error("grouped gemv launch");
      return out;
    }
    DeviceScratch& s = scratch_for(xs.device().index());
    dlv::gemm_tc_run_grouped(&desc_, static_cast<int>(n_per_expert), xs.data_ptr(), static_cast<int>(xs.size(0)), static_cast<int>(xs.stride(0)),
                             out.data_ptr(), static_cast<int>(out.stride(0)), items.data_ptr<int>(), static_cast<int>(items.size(0)),
                             static_cast<int>(bn), static_cast<int>(splits), s.status.data_ptr<int>(), cur_stream());
    check_last_error("grouped gemm launch");
    return out;
  }
  // Decode-size work items (at most 8 rows each) of a gated MLP: gate | up projection with act(gate) * up in the epilogue on the
  // mma.sync grouped GEMV (plain row order: gate rows, then up rows). Returns [rows, n_per_expert / 2], or an undefined tensor when
  // the shape is outside that kernel.
  // With `perm` (the grouping permutation of moe_route, [rows]) and k, xs is the UNGATHERED activation [tokens, K]: grouped row r
  // reads token perm[r] / k, and the copy into expert order is skipped.
  Tensor run_grouped_gemv_act(const Tensor& xs, const Tensor& items, int64_t n_per_expert, int64_t act, c10::optional<Tensor> perm, int64_t k) {
    TORCH_CHECK(xs.is_cuda() && xs.scalar_type() == at::kBFloat16 && xs.dim() == 2 && xs.size(1) == desc_.K && xs.stride(1) == 1, "xs must be bf16 [rows, K]");
    TORCH_CHECK(xs.stride(0) % 8 == 0 && (reinterpret_cast<uintptr_t>(xs.data_ptr()) & 15) == 0, "xs rows must be 16-byte aligned");
    TORCH_CHECK(items.is_cuda() && items.scalar_type() == at::kInt && items.dim() == 2 && items.size(1) == 4 && items.is_contiguous(), "items must be int32 [n, 4]");
    const int64_t per = desc_.is_q4 ? ((n_per_expert + 127) / 128) * 128 : n_per_expert;
    TORCH_CHECK(n_per_expert > 0 && n_per_expert % 2 == 0 && desc_.N % per == 0, "stacked weight rows are not a multiple of the per-expert rows");
    c10::cuda::CUDAGuard guard(xs.device());
    const int* map = nullptr;
    int64_t rows = xs.size(0);
    if (perm.has_value()) {
      const Tensor& pm = perm.value();
      TORCH_CHECK(pm.is_cuda() && pm.scalar_type() == at::kInt && pm.is_contiguous() && k >= 1 && pm.numel() == xs.size(0) * k, "perm must be int32 [tokens * k]");
      map = pm.data_ptr<int>();
      rows = pm.numel();
    }
    Tensor out = new_out({rows, n_per_expert / 2}, xs.options());
    const bool done = dlv::gemv_grouped_act_run(&desc_, static_cast<int>(n_per_expert), xs.data_ptr(), static_cast<int>(xs.stride(0)), out.data_ptr(),
                                                static_cast<int>(out.stride(0)), items.data_ptr<int>(), static_cast<int>(items.size(0)), static_cast<int>(act),
                                                map, static_cast<int>(k), cur_stream());
    check_last_error("grouped gemv (gated activation) launch");
    return done ? out : Tensor();
  }
  // q | k | v projection with per-head RMSNorm, rotary embedding and the paged KV write in the epilogue (head_dim 128). Returns the
  // query heads [M, H * 128]; K and V go straight into the cache rows `slots`.
  Tensor run_qkv(const Tensor& x, const Tensor& positions, const Tensor& slots, c10::optional<Tensor> q_norm_w, c10::optional<Tensor> k_norm_w,
                 c10::optional<Tensor> cos_t, c10::optional<Tensor> sin_t, Tensor& k_cache, Tensor& v_cache, int64_t H, int64_t KV, double eps,
                 double norm_offset, c10::optional<Tensor> bias) {
    TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kBFloat16 && x.dim() == 2 && x.size(1) == desc_.K && x.stride(1) == 1, "x must be bf16 [M, K]");
    TORCH_CHECK(x.stride(0) % 8 == 0 && (reinterpret_cast<uintptr_t>(x.data_ptr()) & 15) == 0, "x rows must be 16-byte aligned");
    TORCH_CHECK(desc_.N == (H + 2 * KV) * 128, "weight rows must be (H + 2 KV) * 128 (head_dim 128)");
    const int M = static_cast<int>(x.size(0));
    TORCH_CHECK(positions.is_cuda() && positions.scalar_type() == at::kInt && positions.numel() == M, "positions must be int32 [M]");
    TORCH_CHECK(slots.is_cuda() && slots.scalar_type() == at::kLong && slots.numel() == M, "slots must be int64 [M]");
    check_bf16(k_cache, "k_cache");
    check_bf16(v_cache, "v_cache");
    TORCH_CHECK(k_cache.dim() == 4 && k_cache.size(1) == KV && k_cache.size(3) == 128 && k_cache.is_contiguous(), "cache must be contiguous [pages, KV, page, 128]");
    TORCH_CHECK(v_cache.sizes() == k_cache.sizes() && v_cache.is_contiguous(), "k/v cache shape mismatch");
    dlv::GemmQkvArgs a = {};
    a.positions = positions.data_ptr<int>();
    a.slots = reinterpret_cast<const long long*>(slots.data_ptr<int64_t>());
    if (q_norm_w.has_value()) {
      check_bf16(q_norm_w.value(), "q_norm");
      check_bf16(k_norm_w.value(), "k_norm");
      TORCH_CHECK(q_norm_w.value().numel() == 128 && k_norm_w.value().numel() == 128, "q/k norm weights must have 128 entries");
      a.q_norm_w = q_norm_w.value().data_ptr();
      a.k_norm_w = k_norm_w.value().data_ptr();
    }
    a.max_pos = 1;
    if (cos_t.has_value()) {
      check_cuda(cos_t.value(), "cos");
      check_cuda(sin_t.value(), "sin");
      TORCH_CHECK(cos_t.value().scalar_type() == at::kFloat && cos_t.value().dim() == 2 && cos_t.value().is_contiguous() &&
                  sin_t.value().sizes() == cos_t.value().sizes() && sin_t.value().is_contiguous(), "cos/sin must be contiguous fp32 [max_pos, rot/2]");
      a.cos_t = cos_t.value().data_ptr<float>();
      a.sin_t = sin_t.value().data_ptr<float>();
      a.rot_half = static_cast<int>(cos_t.value().size(1));
      a.max_pos = static_cast<int>(cos_t.value().size(0));
      TORCH_CHECK(a.rot_half <= 64, "rotary dimension exceeds head_dim");
    }
    a.k_cache = k_cache.data_ptr();
    a.v_cache = v_cache.data_ptr();
    a.heads = static_cast<int>(H);
    a.kv_heads = static_cast<int>(KV);
    a.block_size = static_cast<int>(k_cache.size(2));
    a.eps = static_cast<float>(eps);
    a.norm_offset = static_cast<float>(norm_offset);
    const float* bptr = nullptr;
    if (bias.has_value()) {
      TORCH_CHECK(bias.value().is_cuda() && bias.value().scalar_type() == at::kFloat && bias.value().numel() == desc_.N && bias.value().is_contiguous(), "bias must be fp32 [N]");
      bptr = bias.value().data_ptr<float>();
    }
    c10::cuda::CUDAGuard guard(x.device());
    Tensor q = new_out({M, H * 128}, x.options());
    if (M == 0) return q;
    DeviceScratch& s = scratch_for(x.device().index());
    dlv::gemm_tc_run_qkv(&desc_, x.data_ptr(), M, static_cast<int>(x.stride(0)), q.data_ptr(), static_cast<int>(q.stride(0)), bptr, &a,
                         s.ws.data_ptr<float>(), static_cast<size_t>(s.ws.numel()), s.counters.data_ptr<int>(),
                         static_cast<int>(s.counters.numel()), s.status.data_ptr<int>(), cur_stream());
    check_last_error("gemm (fused q/k/v epilogue) launch");
    return q;
  }
  // Grouped gate | up projection with act(gate) * up in the epilogue (every expert's rows interleaved per tile); [rows, n / 2].
  Tensor run_grouped_act(const Tensor& xs, const Tensor& items, int64_t n_per_expert, int64_t bn, int64_t splits, int64_t act) {
    TORCH_CHECK(xs.is_cuda() && xs.scalar_type() == at::kBFloat16 && xs.dim() == 2 && xs.size(1) == desc_.K && xs.stride(1) == 1, "xs must be bf16 [rows, K]");
    TORCH_CHECK(xs.stride(0) % 8 == 0 && (reinterpret_cast<uintptr_t>(xs.data_ptr()) & 15) == 0, "xs rows must be 16-byte aligned");
    TORCH_CHECK(items.is_cuda() && items.scalar_type() == at::kInt && items.dim() == 2 && items.size(1) == 4 && items.is_contiguous(), "items must be int32 [n, 4]");
    TORCH_CHECK(n_per_expert > 0 && n_per_expert % 128 == 0 && desc_.N % n_per_expert == 0, "gate|up rows per expert must be a multiple of 128");
    TORCH_CHECK(bn >= 16, "the fused activation needs the tensor-core tiles (token tile >= 16)");
    c10::cuda::CUDAGuard guard(xs.device());
    Tensor out = new_out({xs.size(0), n_per_expert / 2}, xs.options());
    DeviceScratch& s = scratch_for(xs.device().index());
    dlv::gemm_tc_run_grouped_act(&desc_, static_cast<int>(n_per_expert), xs.data_ptr(), static_cast<int>(xs.size(0)), static_cast<int>(xs.stride(0)),
                                 out.data_ptr(), static_cast<int>(out.stride(0)), items.data_ptr<int>(), static_cast<int>(items.size(0)),
                                 static_cast<int>(bn), static_cast<int>(splits), static_cast<int>(act), s.status.data_ptr<int>(), cur_stream());
    check_last_error("grouped gemm (fused activation) launch");
    return out;
  }
  // Row-parallel projection fused with the tensor-parallel sum: every rank calls this with its K-shard; `out` holds the
  // all-reduced result on every rank. Returns false (nothing launched) when the shape is outside the fused path.
  bool run_tp(const Tensor& x, Tensor& out, const TpComm& comm, c10::optional<Tensor> bias) {
    TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kBFloat16 && x.dim() == 2 && x.size(1) == desc_.K && x.stride(1) == 1, "x must be bf16 [M, K]");
    TORCH_CHECK(x.stride(0) % 8 == 0 && (reinterpret_cast<uintptr_t>(x.data_ptr()) & 15) == 0, "x rows must be 16-byte aligned");
    const int M = static_cast<int>(x.size(0));
    TORCH_CHECK(out.is_cuda() && out.scalar_type() == at::kBFloat16 && out.dim() == 2 && out.size(0) == M && out.size(1) == desc_.N && out.stride(1) == 1, "bad out");
    if (!dlv::gemm_tp_supported(&desc_, M, comm.args())) return false;
    const float* bptr = nullptr;
    if (bias.has_value()) {
      TORCH_CHECK(bias.value().is_cuda() && bias.value().scalar_type() == at::kFloat && bias.value().numel() == desc_.N, "bias must be fp32 [N]");
      bptr = bias.value().data_ptr<float>();
    }
    c10::cuda::CUDAGuard guard(x.device());
    DeviceScratch& s = scratch_for(x.device().index());
    dlv::gemm_tc_run(&desc_, x.data_ptr(), M, static_cast<int>(x.stride(0)), out.data_ptr(), static_cast<int>(out.stride(0)), false, bptr,
                     s.ws.data_ptr<float>(), static_cast<size_t>(s.ws.numel()), s.counters.data_ptr<int>(),
                     static_cast<int>(s.counters.numel()), s.status.data_ptr<int>(), 0, cur_stream(), comm.args());
    check_last_error("fused tp gemm launch");
    return true;
  }
  // First half of the split form: the GEMM publishes its partial tiles (mode 1: into every rank's slab, mode 2: into its own slab for
  // the multicast reduction) and does not wait. Returns the number of CTAs launched (0: shape outside the fused path, nothing
  // launched); tp_reduce_norm must follow on the same stream with that number.
  int64_t run_tp_push(const Tensor& x, const TpComm& comm, int64_t mode) {
    TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kBFloat16 && x.dim() == 2 && x.size(1) == desc_.K && x.stride(1) == 1, "x must be bf16 [M, K]");
    TORCH_CHECK(x.stride(0) % 8 == 0 && (reinterpret_cast<uintptr_t>(x.data_ptr()) & 15) == 0, "x rows must be 16-byte aligned");
    TORCH_CHECK(mode == 1 || (mode == 2 && comm.has_multicast()), "mode must be 1 (peer stores) or 2 (multicast reduction, needs the multicast address)");
    const int M = static_cast<int>(x.size(0));
    if (M == 0 || desc_.N % 8 != 0 || !dlv::gemm_tp_supported(&desc_, M, comm.args())) return 0;
    const dlv::GemmTpArgs a = comm.with_mode(static_cast<int>(mode));
    c10::cuda::CUDAGuard guard(x.device());
    DeviceScratch& s = scratch_for(x.device().index());
    dlv::gemm_tc_run(&desc_, x.data_ptr(), M, static_cast<int>(x.stride(0)), nullptr, desc_.N, false, nullptr, s.ws.data_ptr<float>(),
                     static_cast<size_t>(s.ws.numel()), s.counters.data_ptr<int>(), static_cast<int>(s.counters.numel()), s.status.data_ptr<int>(), 0,
                     cur_stream(), &a);
    check_last_error("tp gemm (publish only) launch");
    return a.last_ctas;
  }
  // Row-parallel projection for prefill-size batches: GEMM whose epilogue scatters partial tiles to the ranks that own the token
  // rows, reduction of the owned rows, gather of the others. `out` holds the summed result on every rank. Returns false
  // (nothing launched) when the shape is outside this path. Not for CUDA-graph capture (expected counts are launch arguments).
  // gather = false: plain reduce-scatter, `out` is [rows this rank owns, N]. The caller must then order the ranks before the next
  // scatter launch (an all-gather -> GEMM on the same state does).
  bool run_scatter(const Tensor& x, Tensor& out, TpScatter& comm, c10::optional<Tensor> bias, bool gather) {
    TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kBFloat16 && x.dim() == 2 && x.size(1) == desc_.K && x.stride(1) == 1, "x must be bf16 [M, K]");
    TORCH_CHECK(x.stride(0) % 8 == 0 && (reinterpret_cast<uintptr_t>(x.data_ptr()) & 15) == 0, "x rows must be 16-byte aligned");
    const int M = static_cast<int>(x.size(0));
    TORCH_CHECK(out.is_cuda() && out.scalar_type() == at::kBFloat16 && out.dim() == 2 && out.size(1) == desc_.N && out.is_contiguous() &&
                    (reinterpret_cast<uintptr_t>(out.data_ptr()) & 15) == 0, "bad out");
    if (!dlv::gemm_scatter_supported(&desc_, M, comm.args())) return false;
    TORCH_CHECK(out.size(0) == (gather ? M : dlv::gemm_scatter_plan(M, desc_.N, comm.args()->size).rows[comm.args()->rank]), "out has the wrong number of rows");
    const float* bptr = nullptr;
    if (bias.has_value()) {
      TORCH_CHECK(bias.value().is_cuda() && bias.value().scalar_type() == at::kFloat && bias.value().numel() == desc_.N, "bias must be fp32 [N]");
      bptr = bias.value().data_ptr<float>();
    }
    c10::cuda::CUDAGuard guard(x.device());
    DeviceScratch& s = scratch_for(x.device().index());
    const dlv::GemmScatterPlan plan = dlv::gemm_scatter_plan(M, desc_.N, comm.args()->size);
    dlv::gemm_tc_run_scatter(&desc_, x.data_ptr(), M, static_cast<int>(x.stride(0)), comm.args(), s.status.data_ptr<int>(), cur_stream());
    comm.advance(plan, gather);  // only once the GEMM that publishes these counts is in the stream
    dlv::launch_scatter_reduce(comm.args(), &plan, M, desc_.N, bptr, out.data_ptr(), comm.tile_target(), gather, s.status.data_ptr<int>(), cur_stream());
    if (gather)
      dlv::launch_scatter_finish(comm.args(), &plan, M, desc_.N, out.data_ptr(), comm.group_targets(), s.status.data_ptr<int>(), cur_stream());
    check_last_error("gemm reduce-scatter launch");
    return true;
  }
  // Column-parallel projection of activations whose rows are sharded over the ranks: `x_own` holds this rank's rows (the cut of
  // scatter_plan(M, ., size)); they are pushed to every rank's gather area and the GEMM's activation producers wait per token
  // tile for the owners. `out` = all_gather(x) @ W^T, [M, N]. Between two calls the ranks must have been ordered by another
  // collective (the gather area is a single buffer). Returns false (nothing launched) outside this path.
  bool run_gathered(const Tensor& x_own, int64_t M, Tensor& out, TpScatter& comm, c10::optional<Tensor> bias) {
    TORCH_CHECK(x_own.is_cuda() && x_own.scalar_type() == at::kBFloat16 && x_own.dim() == 2 && x_own.size(1) == desc_.K && x_own.is_contiguous(),
                "x_own must be contiguous bf16 [rows, K]");
    TORCH_CHECK((reinterpret_cast<uintptr_t>(x_own.data_ptr()) & 15) == 0, "x_own must be 16-byte aligned");
    TORCH_CHECK(out.is_cuda() && out.scalar_type() == at::kBFloat16 && out.dim() == 2 && out.size(0) == M && out.size(1) == desc_.N && out.stride(1) == 1, "bad out");
    if (!dlv::gemm_gathered_supported(&desc_, static_cast<int>(M), comm.args())) return false;
    const dlv::GemmScatterPlan plan = dlv::gemm_scatter_plan(static_cast<int>(M), desc_.N, comm.args()->size);
    TORCH_CHECK(x_own.size(0) == plan.rows[comm.args()->rank], "x_own must hold exactly the rows this rank owns");
    const float* bptr = nullptr;
    if (bias.has_value()) {
      TORCH_CHECK(bias.value().is_cuda() && bias.value().scalar_type() == at::kFloat && bias.value().numel() == desc_.N, "bias must be fp32 [N]");
      bptr = bias.value().data_ptr<float>();
    }
    c10::cuda::CUDAGuard guard(x_own.device());
    DeviceScratch& s = scratch_for(x_own.device().index());
    dlv::launch_gather_push(comm.args(), &plan, x_own.data_ptr(), static_cast<int>(M), desc_.K, s.status.data_ptr<int>(), cur_stream());
    comm.advance_gather(plan);
    dlv::gemm_tc_run_gathered(&desc_, static_cast<int>(M), comm.args(), comm.gather_targets(), out.data_ptr(), static_cast<int>(out.stride(0)), bptr,
                              s.ws.data_ptr<float>(), static_cast<size_t>(s.ws.numel()), s.counters.data_ptr<int>(),
                              static_cast<int>(s.counters.numel()), s.status.data_ptr<int>(), cur_stream());
    check_last_error("all-gather gemm launch");
    return true;
  }
  int64_t n() const { return desc_.N; }
  int64_t k() const { return desc_.K; }
  const dlv::GemmWeightDesc* desc() const { return &desc_; }
  const Tensor& data() const { return w_; }
  bool is_q4() const { return desc_.is_q4; }

 private:
  dlv::GemmWeightDesc desc_;
  Tensor w_;
};

// Reads and clears the kernel status word of a device (0 = ok, 1 = barrier wait ran out, 2 = flag wait ran out).
int64_t take_status(int64_t device) {
  DeviceScratch& s = scratch_for(static_cast<int>(device));
  int64_t v = s.status.item<int>();
  if (v != 0) s.status.zero_();
  return v;
}
void init_scratch(int64_t device) { scratch_for(static_cast<int>(device)); }
// ---- elementwise ----------------------------------------------------------------------------------------------------
Tensor rmsnorm(const Tensor& x, const Tensor& w, double eps, double offset) {
  check_bf16(x, "x");
  check_bf16(w, "w");
  const int H = static_cast<int>(x.size(-1));
  TORCH_CHECK(H % 8 == 0 && w.numel() == H, "hidden size must be a multiple of 8");
  c10::cuda::CUDAGuard guard(x.device());
  Tensor y = new_out(x.sizes(), x.options());
  dlv::launch_rmsnorm(x.data_ptr(), nullptr, w.data_ptr(), y.data_ptr(), static_cast<int>(x.numel() / H), H, static_cast<float>(eps),
                      static_cast<float>(offset), 1.f, cur_stream());
  check_last_error("rmsnorm");
  return y;
}
Tensor add_rmsnorm(const Tensor& x, Tensor& residual, const Tensor& w, double eps, double offset, double res_mult) {
  check_bf16(x, "x");
  check_bf16(residual, "residual");
  check_bf16(w, "w");
  const int H = static_cast<int>(x.size(-1));
  TORCH_CHECK(H % 8 == 0 && w.numel() == H && residual.sizes() == x.sizes(), "shape mismatch");
  c10::cuda::CUDAGuard guard(x.device());
  Tensor y = new_out(x.sizes(), x.options());
  dlv::launch_rmsnorm(x.data_ptr(), residual.data_ptr(), w.data_ptr(), y.data_ptr(), static_cast<int>(x.numel() / H), H,
                      static_cast<float>(eps), static_cast<float>(offset), static_cast<float>(res_mult), cur_stream());
  check_last_error("add_rmsnorm");
  return y;
}
Tensor layernorm(const Tensor& x, const Tensor& w, c10::optional<Tensor> b, double eps) {
  check_bf16(x, "x");
  check_bf16(w, "w");
  const int H = static_cast<int>(x.size(-1));
  TORCH_CHECK(w.numel() == H, "shape mismatch");
  const void* bp = nullptr;
  if (b.has_value()) {
    check_bf16(b.value(), "bias");
    bp = b.value().data_ptr();
  }
  c10::cuda::CUDAGuard guard(x.device());
  Tensor y = new_out(x.sizes(), x.options());
  dlv::launch_layernorm(x.data_ptr(), w.data_ptr(), bp, y.data_ptr(), static_cast<int>(x.numel() / H), H, static_cast<float>(eps), cur_stream());
  check_last_error("layernorm");
  return y;
}
Tensor act_mul(const Tensor& gate_up, const std::string& act) {
  check_bf16(gate_up, "gate_up");
  TORCH_CHECK(gate_up.dim() == 2 && gate_up.size(1) % 16 == 0, "gate|up width must be a multiple of 16");
  const int I = static_cast<int>(gate_up.size(1) / 2);
  c10::cuda::CUDAGuard guard(gate_up.device());
  Tensor out = new_out({gate_up.size(0), I}, gate_up.options());
  dlv::launch_act_mul(gate_up.data_ptr(), out.data_ptr(), gate_up.size(0), I, act_code(act), cur_stream());
  check_last_error("act_mul");
  return out;
}
Tensor activation(const Tensor& x, const std::string& act) {
  check_bf16(x, "x");
  c10::cuda::CUDAGuard guard(x.device());
  Tensor out = new_out(x.sizes(), x.options());
  dlv::launch_act(x.data_ptr(), out.data_ptr(), x.numel(), act_code(act), cur_stream());
  check_last_error("activation");
  return out;
}
Tensor embedding(const Tensor& table, const Tensor& ids, double scale, c10::optional<Tensor> pos_table, c10::optional<Tensor> pos,
                 c10::optional<Tensor> type_table, c10::optional<Tensor> types) {
  check_bf16(table, "table");
  check_cuda(ids, "ids");
  TORCH_CHECK(ids.scalar_type() == at::kInt, "ids must be int32");
  const int H = static_cast<int>(table.size(1));
  TORCH_CHECK(H % 8 == 0, "hidden size must be a multiple of 8");
  const void* pt = nullptr;
  const int* pp = nullptr;
  const void* tt = nullptr;
  const int* tp = nullptr;
  if (pos_table.has_value()) {
    check_bf16(pos_table.value(), "pos_table");
    TORCH_CHECK(pos.has_value() && pos.value().scalar_type() == at::kInt && pos.value().numel() == ids.numel(), "positions required");
    check_cuda(pos.value(), "pos");
    pt = pos_table.value().data_ptr();
    pp = pos.value().data_ptr<int>();
  }
  if (type_table.has_value()) {
    check_bf16(type_table.value(), "type_table");
    tt = type_table.value().data_ptr();
    if (types.has_value()) {
      check_cuda(types.value(), "types");
      TORCH_CHECK(types.value().scalar_type() == at::kInt && types.value().numel() == ids.numel(), "bad token types");
      tp = types.value().data_ptr<int>();
    }
  }
  c10::cuda::CUDAGuard guard(table.device());
  Tensor out = new_out({ids.numel(), H}, table.options());
  dlv::launch_embedding(table.data_ptr(), ids.data_ptr<int>(), pt, pp, tt, tp, out.data_ptr(), static_cast<int>(ids.numel()), H,
                        static_cast<int>(table.size(0)), static_cast<float>(scale), cur_stream());
  check_last_error("embedding");
  return out;
}

// qkv [T, (H + 2 KV) * D] modified in place (q heads); k, v scattered into the paged cache [pages, KV, page, D]
void rope_kv(Tensor& qkv, const Tensor& positions, c10::optional<Tensor> slots, c10::optional<Tensor> q_norm_w,
             c10::optional<Tensor> k_norm_w, c10::optional<Tensor> cos_t, c10::optional<Tensor> sin_t, c10::optional<Tensor> k_cache,
             c10::optional<Tensor> v_cache, int64_t H, int64_t KV, int64_t D, double eps, double norm_offset) {
  check_bf16(qkv, "qkv");
  check_cuda(positions, "positions");
  TORCH_CHECK(positions.scalar_type() == at::kInt, "positions must be int32");
  const int T = static_cast<int>(qkv.size(0));
  TORCH_CHECK(qkv.dim() == 2 && qkv.size(1) == (H + 2 * KV) * D && positions.numel() == T, "bad qkv shape");
  const long long* sp = nullptr;
  void *kc = nullptr, *vc = nullptr;
  int page = 1;
  if (slots.has_value()) {
    check_cuda(slots.value(), "slots");
    TORCH_CHECK(slots.value().scalar_type() == at::kLong && slots.value().numel() == T, "slots must be int64 [T]");
    TORCH_CHECK(k_cache.has_value() && v_cache.has_value(), "cache tensors required with slots");
    check_bf16(k_cache.value(), "k_cache");
    check_bf16(v_cache.value(), "v_cache");
    TORCH_CHECK(k_cache.value().dim() == 4 && k_cache.value().size(1) == KV && k_cache.value().size(3) == D, "cache must be [pages, KV, page, D]");
    TORCH_CHECK(v_cache.value().sizes() == k_cache.value().sizes(), "k/v cache shape mismatch");
    sp = reinterpret_cast<const long long*>(slots.value().data_ptr<int64_t>());
    kc = k_cache.value().data_ptr();
    vc = v_cache.value().data_ptr();
    page = static_cast<int>(k_cache.value().size(2));
  }
  const void *qn = nullptr, *kn = nullptr;
  if (q_norm_w.has_value()) {
    check_bf16(q_norm_w.value(), "q_norm");
    check_bf16(k_norm_w.value(), "k_norm");
    TORCH_CHECK(q_norm_w.value().numel() == D && k_norm_w.value().numel() == D, "q/k norm weights must have head_dim entries");
    qn = q_norm_w.value().data_ptr();
    kn = k_norm_w.value().data_ptr();
  }
  const float *ct = nullptr, *stb = nullptr;
  int rot_half = 0, max_pos = 1;
  if (cos_t.has_value()) {
    check_cuda(cos_t.value(), "cos");
    check_cuda(sin_t.value(), "sin");
    TORCH_CHECK(cos_t.value().scalar_type() == at::kFloat && cos_t.value().dim() == 2 && sin_t.value().sizes() == cos_t.value().sizes(), "cos/sin must be fp32 [max_pos, rot/2]");
    ct = cos_t.value().data_ptr<float>();
    stb = sin_t.value().data_ptr<float>();
    rot_half = static_cast<int>(cos_t.value().size(1));
    max_pos = static_cast<int>(cos_t.value().size(0));
    TORCH_CHECK(rot_half * 2 <= D, "rotary dimension exceeds head_dim");
  }
  c10::cuda::CUDAGuard guard(qkv.device());
  int rc = dlv::launch_rope_kv(qkv.data_ptr(), positions.data_ptr<int>(), sp, qn, kn, ct, stb, kc, vc, T, static_cast<int>(H),
                               static_cast<int>(KV), static_cast<int>(D), page, rot_half, static_cast<float>(eps),
                               static_cast<float>(norm_offset), max_pos, cur_stream());
  TORCH_CHECK(rc == 0, "unsupported head_dim ", D, " (64, 128, 256)");
  check_last_error("rope_kv");
}

// ---- attention ------------------------------------------------------------------------------------------------------
// q: view [B, H*D] bf16 with arbitrary row stride (the q part of the fused qkv activation)
// Arrival counters of the split-KV decode kernel (one per sequence and KV head; the CTA that arrives last merges the splits and
// puts its counter back to zero, so the array stays zero between launches). One array per device, made on first use outside any
// stream capture; launches on one device are expected on one stream at a time (the engine's), nullptr means "merge in a second
// kernel" and is what a capture that comes before any eager call gets, as does a batch with more counters than the array holds.
bool g_decode_merge_in_kernel = false;  // measured slower than the merge launch (see ops.set_decode_merge_in_kernel)
constexpr int64_t kSplitCounters = 1 << 16;
int* split_arrival_counters(int device, int64_t needed) {
  static std::mutex mu;
  static std::unordered_map<int, Tensor> per_device;
  if (needed > kSplitCounters) return nullptr;
  std::lock_guard<std::mutex> lock(mu);
  auto it = per_device.find(device);
  if (it == per_device.end()) {
    cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(cur_stream(), &cs) != cudaSuccess || cs != cudaStreamCaptureStatusNone) return nullptr;
    Tensor t = at::zeros({kSplitCounters}, at::TensorOptions().dtype(at::kInt).device(at::kCUDA, device));
    it = per_device.emplace(device, t).first;
  }
  return it->second.data_ptr<int>();
}

Tensor decode_attention(const Tensor& q, const Tensor& k_cache, const Tensor& v_cache, const Tensor& block_tables, const Tensor& ctx_lens,
                        int64_t H, double scale, double softcap, int64_t window, int64_t splits, int64_t impl) {
  TORCH_CHECK(q.is_cuda() && q.scalar_type() == at::kBFloat16 && q.dim() == 2 && q.stride(1) == 1, "q must be bf16 [B, H*D]");
  check_bf16(k_cache, "k_cache");
  check_bf16(v_cache, "v_cache");
  check_cuda(block_tables, "block_tables");
  check_cuda(ctx_lens, "ctx_lens");
  TORCH_CHECK(block_tables.scalar_type() == at::kInt && ctx_lens.scalar_type() == at::kInt, "tables must be int32");
  const int B = static_cast<int>(q.size(0));
  const int KV = static_cast<int>(k_cache.size(1)), page = static_cast<int>(k_cache.size(2)), D = static_cast<int>(k_cache.size(3));
  TORCH_CHECK(q.size(1) == H * D && H % KV == 0 && page % 32 == 0, "shape mismatch (page size must be a multiple of 32)");
  TORCH_CHECK(block_tables.dim() == 2 && block_tables.size(0) >= B && ctx_lens.numel() >= B, "bad table shapes");
  TORCH_CHECK((reinterpret_cast<uintptr_t>(q.data_ptr()) & 3) == 0, "q misaligned");
  c10::cuda::CUDAGuard guard(q.device());
  Tensor out = new_out({B, H * D}, q.options());
  if (splits < 1) splits = 1;
  Tensor po, pml;
  float *pop = nullptr, *pmlp = nullptr;
  if (splits > 1) {
    po = new_out({B, H, splits, D}, q.options().dtype(at::kFloat));
    pml = new_out({B, H, splits, 2}, q.options().dtype(at::kFloat));
    pop = po.data_ptr<float>();
    pmlp = pml.data_ptr<float>();
  }
  int* arrivals = (splits > 1 && g_decode_merge_in_kernel) ? split_arrival_counters(q.device().index(), static_cast<int64_t>(B) * KV) : nullptr;
  int rc = dlv::launch_decode_attention_impl(q.data_ptr(), q.stride(0), k_cache.data_ptr(), v_cache.data_ptr(), block_tables.data_ptr<int>(),
                                             static_cast<int>(block_tables.stride(0)), ctx_lens.data_ptr<int>(), out.data_ptr(), pop, pmlp, arrivals, B,
                                             static_cast<int>(H), KV, D, page, static_cast<float>(scale), static_cast<float>(softcap),
                                             static_cast<int>(window), static_cast<int>(splits), static_cast<int>(impl), cur_stream());
  TORCH_CHECK(rc == 0, "decode attention: unsupported head_dim / group size (code ", rc, ")");
  check_last_error("decode_attention");
  return out;
}

Tensor prefill_attention(const Tensor& q, const Tensor& k_cache, const Tensor& v_cache, const Tensor& block_tables, const Tensor& q_start,
                         const Tensor& q_len, const Tensor& ctx_lens, const Tensor& tile_seq, const Tensor& tile_q0, int64_t H,
                         double scale, double softcap, int64_t window, bool causal) {
  TORCH_CHECK(q.is_cuda() && q.scalar_type() == at::kBFloat16 && q.dim() == 2 && q.stride(1) == 1, "q must be bf16 [T, H*D]");
  TORCH_CHECK(q.stride(0) % 8 == 0 && (reinterpret_cast<uintptr_t>(q.data_ptr()) & 15) == 0, "q rows must be 16-byte aligned");
  check_bf16(k_cache, "k_cache");
  check_bf16(v_cache, "v_cache");
  for (const Tensor* t : {&block_tables, &q_start, &q_len, &ctx_lens, &tile_seq, &tile_q0}) {
    check_cuda(*t, "index tensor");
    TORCH_CHECK(t->scalar_type() == at::kInt, "index tensors must be int32");
  }
  const int T = static_cast<int>(q.size(0));
  const int KV = static_cast<int>(k_cache.size(1)), page = static_cast<int>(k_cache.size(2)), D = static_cast<int>(k_cache.size(3));
  TORCH_CHECK(q.size(1) == H * D && H % KV == 0 && page % 32 == 0, "shape mismatch");
  TORCH_CHECK(tile_seq.numel() == tile_q0.numel(), "tile arrays differ in length");
  c10::cuda::CUDAGuard guard(q.device());
  Tensor out = new_out({T, H * D}, q.options());
  int rc = dlv::launch_prefill_attention(q.data_ptr(), q.stride(0), k_cache.data_ptr(), v_cache.data_ptr(), block_tables.data_ptr<int>(),
                                         static_cast<int>(block_tables.stride(0)), q_start.data_ptr<int>(), q_len.data_ptr<int>(),
                                         ctx_lens.data_ptr<int>(), tile_seq.data_ptr<int>(), tile_q0.data_ptr<int>(),
                                         static_cast<int>(tile_seq.numel()), out.data_ptr(), static_cast<int>(H), KV, D, page,
                                         static_cast<float>(scale), static_cast<float>(softcap), static_cast<int>(window), causal ? 1 : 0,
                                         cur_stream());
  TORCH_CHECK(rc == 0, "prefill attention: unsupported head_dim");
  check_last_error("prefill_attention");
  return out;
}

// Same contract as prefill_attention, on the tcgen05 / TMA kernel; tile arrays cover prefill_tc_tile_rows(head_dim) query rows per tile.
Tensor prefill_attention_tc(const Tensor& q, const Tensor& k_cache, const Tensor& v_cache, const Tensor& block_tables, const Tensor& q_start,
                            const Tensor& q_len, const Tensor& ctx_lens, const Tensor& tile_seq, const Tensor& tile_q0, int64_t H, double scale,
                            double softcap, int64_t window, bool causal) {
  TORCH_CHECK(q.is_cuda() && q.scalar_type() == at::kBFloat16 && q.dim() == 2 && q.stride(1) == 1, "q must be bf16 [T, H*D]");
  TORCH_CHECK(q.stride(0) % 8 == 0 && (reinterpret_cast<uintptr_t>(q.data_ptr()) & 15) == 0, "q rows must be 16-byte aligned");
  check_bf16(k_cache, "k_cache");
  check_bf16(v_cache, "v_cache");
  for (const Tensor* t : {&block_tables, &q_start, &q_len, &ctx_lens, &tile_seq, &tile_q0}) {
    check_cuda(*t, "index tensor");
    TORCH_CHECK(t->scalar_type() == at::kInt, "index tensors must be int32");
  }
  const int T = static_cast<int>(q.size(0));
  const int KV = static_cast<int>(k_cache.size(1)), page = static_cast<int>(k_cache.size(2)), D = static_cast<int>(k_cache.size(3));
  TORCH_CHECK(k_cache.dim() == 4 && v_cache.sizes() == k_cache.sizes() && q.size(1) == H * D && H % KV == 0, "shape mismatch");
  TORCH_CHECK((page == 32 || page == 64 || page == 128) && (D == 64 || D == 128 || D == 256), "page size 32 / 64 / 128 and head_dim 64 / 128 / 256");
  TORCH_CHECK(tile_seq.numel() == tile_q0.numel(), "tile arrays differ in length");
  c10::cuda::CUDAGuard guard(q.device());
  Tensor out = new_out({T, H * D}, q.options());
  DeviceScratch& s = scratch_for(q.device().index());
  int rc = dlv::launch_prefill_attention_tc(q.data_ptr(), q.stride(0), T, k_cache.data_ptr(), v_cache.data_ptr(), k_cache.size(0), block_tables.data_ptr<int>(),
                                            static_cast<int>(block_tables.stride(0)), q_start.data_ptr<int>(), q_len.data_ptr<int>(), ctx_lens.data_ptr<int>(),
                                            tile_seq.data_ptr<int>(), tile_q0.data_ptr<int>(), static_cast<int>(tile_seq.numel()), out.data_ptr(),
                                            static_cast<int>(H), KV, D, page, static_cast<float>(scale), static_cast<float>(softcap),
                                            static_cast<int>(window), causal ? 1 : 0, s.status.data_ptr<int>(), cur_stream());
  TORCH_CHECK(rc == 0, "prefill attention (tcgen05): unsupported shape");
  check_last_error("prefill_attention_tc");
  return out;
}

// ---- sampling ---------------------------------------------------------------------------------------------------------
std::vector<Tensor> argmax(const Tensor& logits, c10::optional<Tensor> mask, double softcap, double inv_scale) {
  TORCH_CHECK(logits.is_cuda() && logits.scalar_type() == at::kFloat && logits.dim() == 2 && logits.stride(1) == 1, "logits must be fp32 [B, V]");
  const int B = static_cast<int>(logits.size(0)), V = static_cast<int>(logits.size(1));
  const uint32_t* mp = nullptr;
  int mld = 0;
  if (mask.has_value()) {
    const Tensor& m = mask.value();
    check_cuda(m, "mask");
    TORCH_CHECK(m.scalar_type() == at::kInt && m.dim() == 2 && m.size(0) == B && m.size(1) * 32 >= V, "mask must be int32 [B, ceil(V/32)]");
    mp = reinterpret_cast<const uint32_t*>(m.data_ptr<int>());
    mld = static_cast<int>(m.size(1));
  }
  c10::cuda::CUDAGuard guard(logits.device());
  Tensor idx = new_out({B}, logits.options().dtype(at::kLong));
  Tensor val = new_out({B}, logits.options());
  dlv::launch_argmax(logits.data_ptr<float>(), static_cast<int>(logits.stride(0)), B, V, mp, mld, static_cast<float>(softcap),
                     static_cast<float>(inv_scale), reinterpret_cast<long long*>(idx.data_ptr<int64_t>()), val.data_ptr<float>(), cur_stream());
  check_last_error("argmax");
  return {idx, val};
}
// Top-k / top-p / uniform-top-p sampling of every row with one kernel launch (histogram select, no vocabulary sort).
// Returns (token ids int64 [B], handled int32 [B]); rows with handled == 0 need the sorting fallback.
std::vector<Tensor> sample_rows(const Tensor& logits, const Tensor& inv_temp, const Tensor& limits, const Tensor& top_p, const Tensor& uniform,
                                const Tensor& us) {
  TORCH_CHECK(logits.is_cuda() && logits.scalar_type() == at::kFloat && logits.dim() == 2 && logits.stride(1) == 1, "logits must be fp32 [B, V]");
  const int B = static_cast<int>(logits.size(0)), V = static_cast<int>(logits.size(1));
  for (const Tensor* t : std::initializer_list<const Tensor*>{&inv_temp, &limits, &top_p, &uniform, &us}) {
    check_cuda(*t, "sampling parameter");
    TORCH_CHECK(t->numel() == B && t->is_contiguous(), "one sampling parameter per row");
  }
  TORCH_CHECK(inv_temp.scalar_type() == at::kFloat && top_p.scalar_type() == at::kFloat && us.scalar_type() == at::kFloat &&
                  limits.scalar_type() == at::kLong && uniform.scalar_type() == at::kByte, "sampling parameter dtypes");
  c10::cuda::CUDAGuard guard(logits.device());
  Tensor tok = torch::zeros({B}, logits.options().dtype(at::kLong));
  Tensor ok = torch::zeros({B}, logits.options().dtype(at::kInt));
  dlv::launch_sample(logits.data_ptr<float>(), static_cast<int>(logits.stride(0)), B, V, inv_temp.data_ptr<float>(),
                     reinterpret_cast<const long long*>(limits.data_ptr<int64_t>()), top_p.data_ptr<float>(), uniform.data_ptr<uint8_t>(),
                     us.data_ptr<float>(), reinterpret_cast<long long*>(tok.data_ptr<int64_t>()), ok.data_ptr<int>(), cur_stream());
  check_last_error("sample_rows");
  return {tok, ok};
}
// The same with every per-row parameter in ONE float32 tensor [6, n] (one host-to-device copy per step instead of six): rows =
// (row of `logits`, 1 / temperature, candidate limit, top_p, uniform flag, uniform random number). Returns int64 [2, n]: the
// token ids and the handled flags (one device-to-host read).
Tensor sample_rows_packed(const Tensor& logits, const Tensor& packed) {
  TORCH_CHECK(logits.is_cuda() && logits.scalar_type() == at::kFloat && logits.dim() == 2 && logits.stride(1) == 1, "logits must be fp32 [B, V]");
  check_cuda(packed, "packed sampling parameters");
  TORCH_CHECK(packed.scalar_type() == at::kFloat && packed.dim() == 2 && packed.size(0) == 6, "packed sampling parameters must be float32 [6, n]");
  const int64_t n = packed.size(1);
  c10::cuda::CUDAGuard guard(logits.device());
  Tensor sub = n == logits.size(0) ? logits : logits.index_select(0, packed[0].to(at::kLong));
  std::vector<Tensor> r = sample_rows(sub, packed[1].contiguous(), packed[2].to(at::kLong), packed[3].contiguous(), packed[4].to(at::kByte), packed[5].contiguous());
  return torch::stack({r[0], r[1].to(at::kLong)}, 0);
}
// Exclude-top-choice picks of every row in one launch: int64 [B], -1 where XTC does not apply (not armed, or no token above the threshold).
Tensor xtc_rows(const Tensor& logits, const Tensor& inv_temp, const Tensor& threshold, const Tensor& fire, const Tensor& special) {
  TORCH_CHECK(logits.is_cuda() && logits.scalar_type() == at::kFloat && logits.dim() == 2 && logits.stride(1) == 1, "logits must be fp32 [B, V]");
  const int B = static_cast<int>(logits.size(0)), V = static_cast<int>(logits.size(1));
  for (const Tensor* t : std::initializer_list<const Tensor*>{&inv_temp, &threshold, &fire}) {
    check_cuda(*t, "xtc parameter");
    TORCH_CHECK(t->numel() == B, "one xtc parameter per row");
  }
  check_cuda(special, "special ids");
  TORCH_CHECK(inv_temp.scalar_type() == at::kFloat && threshold.scalar_type() == at::kFloat && fire.scalar_type() == at::kByte && special.scalar_type() == at::kInt,
              "xtc parameter dtypes");
  c10::cuda::CUDAGuard guard(logits.device());
  Tensor tok = new_out({B}, logits.options().dtype(at::kLong));
  dlv::launch_xtc(logits.data_ptr<float>(), static_cast<int>(logits.stride(0)), B, V, inv_temp.data_ptr<float>(), threshold.data_ptr<float>(),
                  fire.data_ptr<uint8_t>(), special.data_ptr<int>(), static_cast<int>(special.numel()),
                  reinterpret_cast<long long*>(tok.data_ptr<int64_t>()), cur_stream());
  check_last_error("xtc_rows");
  return tok;
}
// Log-probability of the chosen token of every row and the top_n most probable tokens: (chosen [B] f32, top ids [B, top_n] i64, top values [B, top_n] f32).
std::vector<Tensor> logprob_rows(const Tensor& logits, const Tensor& chosen, int64_t top_n) {
  TORCH_CHECK(logits.is_cuda() && logits.scalar_type() == at::kFloat && logits.dim() == 2 && logits.stride(1) == 1, "logits must be fp32 [B, V]");
  const int B = static_cast<int>(logits.size(0)), V = static_cast<int>(logits.size(1));
  check_cuda(chosen, "chosen");
  TORCH_CHECK(chosen.scalar_type() == at::kLong && chosen.numel() == B && top_n >= 0 && top_n <= 64 && top_n <= V, "chosen must be int64 [B]; top_n in 0..64");
  TORCH_CHECK(chosen.min().item<int64_t>() >= 0 && chosen.max().item<int64_t>() < V, "chosen token outside the vocabulary");
  c10::cuda::CUDAGuard guard(logits.device());
  Tensor lp = new_out({B}, logits.options());
  Tensor idx = new_out({B, top_n}, logits.options().dtype(at::kLong));
  Tensor val = new_out({B, top_n}, logits.options());
  dlv::launch_logprobs(logits.data_ptr<float>(), static_cast<int>(logits.stride(0)), B, V, reinterpret_cast<const long long*>(chosen.data_ptr<int64_t>()),
                       static_cast<int>(top_n), lp.data_ptr<float>(), reinterpret_cast<long long*>(idx.data_ptr<int64_t>()), val.data_ptr<float>(), cur_stream());
  check_last_error("logprob_rows");
  return {lp, idx, val};
}
void logits_post(Tensor& logits, c10::optional<Tensor> mask, double softcap, double inv_scale) {
  TORCH_CHECK(logits.is_cuda() && logits.scalar_type() == at::kFloat && logits.dim() == 2 && logits.stride(1) == 1, "logits must be fp32 [B, V]");
  const int B = static_cast<int>(logits.size(0)), V = static_cast<int>(logits.size(1));
  const uint32_t* mp = nullptr;
  int mld = 0;
  if (mask.has_value()) {
    const Tensor& m = mask.value();
    check_cuda(m, "mask");
    TORCH_CHECK(m.scalar_type() == at::kInt && m.dim() == 2 && m.size(0) == B && m.size(1) * 32 >= V, "mask must be int32 [B, ceil(V/32)]");
    mp = reinterpret_cast<const uint32_t*>(m.data_ptr<int>());
    mld = static_cast<int>(m.size(1));
  }
  c10::cuda::CUDAGuard guard(logits.device());
  dlv::launch_logits_post(logits.data_ptr<float>(), static_cast<int>(logits.stride(0)), B, V, mp, mld, static_cast<float>(softcap),
                          static_cast<float>(inv_scale), cur_stream());
  check_last_error("logits_post");
}

// ---- expert-parallel all-to-all -----------------------------------------------------------------------------------------
class ExpertA2A {
 public:
  // recv / meta / flag / ret pointers: device addresses of every rank's areas as mapped in this process
  ExpertA2A(int64_t rank, int64_t size, int64_t ne, int64_t cap, int64_t H, std::vector<int64_t> recv, std::vector<int64_t> meta, std::vector<int64_t> flags,
            std::vector<int64_t> ret) : H_(static_cast<int>(H)) {
    TORCH_CHECK(size >= 2 && size <= 8 && rank >= 0 && rank < size && ne >= 1 && ne <= 128 && cap >= 1 && H % 8 == 0, "bad all-to-all geometry");
    TORCH_CHECK(static_cast<int64_t>(recv.size()) == size && static_cast<int64_t>(meta.size()) == size && static_cast<int64_t>(flags.size()) == size &&
                    static_cast<int64_t>(ret.size()) == size, "one pointer per rank");
    p_ = {};
    p_.size = static_cast<int>(size);
    p_.rank = static_cast<int>(rank);
    p_.ne = static_cast<int>(ne);
    p_.cap = static_cast<int>(cap);
    for (int r = 0; r < size; ++r) {
      p_.recv[r] = static_cast<unsigned long long>(recv[r]);
      p_.meta[r] = static_cast<unsigned long long>(meta[r]);
      p_.flags[r] = static_cast<unsigned long long>(flags[r]);
      p_.ret[r] = static_cast<unsigned long long>(ret[r]);
      TORCH_CHECK((p_.recv[r] & 15) == 0 && (p_.ret[r] & 15) == 0 && (p_.meta[r] & 3) == 0 && (p_.flags[r] & 3) == 0 && p_.recv[r] && p_.ret[r] && p_.meta[r] && p_.flags[r],
                  "bad peer pointer");
    }
  }
  // x [T, H] own token rows; perm / offsets from moe_route over the own tokens (offsets over ALL experts). Pushes the rows and publishes.
  void dispatch(const Tensor& x, const Tensor& perm, const Tensor& offsets, int64_t k) {
    check_bf16(x, "x");
    check_cuda(perm, "perm");
    check_cuda(offsets, "offsets");
    TORCH_CHECK(x.dim() == 2 && x.size(1) == H_ && perm.scalar_type() == at::kInt && offsets.scalar_type() == at::kInt && perm.numel() == x.size(0) * k &&
                    offsets.numel() == static_cast<int64_t>(p_.size) * p_.ne + 1 && perm.numel() <= p_.cap, "dispatch arguments");
    c10::cuda::CUDAGuard guard(x.device());
    dlv::A2AParams p = with_status(x.device().index());
    ++epoch_;
    dlv::launch_a2a_dispatch(&p, x.data_ptr(), perm.data_ptr<int>(), offsets.data_ptr<int>(), static_cast<int>(perm.numel()), static_cast<int>(k), H_, epoch_, cur_stream());
    check_last_error("a2a dispatch");
  }
  // Waits for all sources, returns (xs [max_rows, H] rows grouped by local expert, local_offsets [ne + 1], seg [ne * size, 4]).
  std::vector<Tensor> receive(int64_t max_rows, const Tensor& like) {
    c10::cuda::CUDAGuard guard(like.device());
    auto io = torch::TensorOptions().device(like.device()).dtype(torch::kInt32);
    Tensor local_offsets = torch::zeros({p_.ne + 1}, io), seg = torch::zeros({static_cast<long>(p_.ne) * p_.size, 4}, io);
    Tensor xs = new_out({max_rows, H_}, torch::TensorOptions().device(like.device()).dtype(torch::kBFloat16));
    dlv::A2AParams p = with_status(like.device().index());
    dlv::launch_a2a_receive(&p, epoch_, local_offsets.data_ptr<int>(), seg.data_ptr<int>(), xs.data_ptr(), static_cast<int>(max_rows), H_, cur_stream());
    check_last_error("a2a receive");
    return {xs, local_offsets, seg};
  }
  // Sends the expert outputs back to their senders and returns this rank's own return buffer [cap, H] once every rank has answered.
  Tensor finish(const Tensor& ys, const Tensor& local_offsets, const Tensor& seg, const Tensor& ret_local) {
    check_bf16(ys, "ys");
    TORCH_CHECK(ys.dim() == 2 && ys.size(1) == H_ && ret_local.is_cuda() && ret_local.scalar_type() == at::kBFloat16, "finish arguments");
    c10::cuda::CUDAGuard guard(ys.device());
    dlv::A2AParams p = with_status(ys.device().index());
    dlv::launch_a2a_return(&p, local_offsets.data_ptr<int>(), seg.data_ptr<int>(), ys.data_ptr(), static_cast<int>(ys.size(0)), H_, epoch_, cur_stream());
    dlv::launch_a2a_wait(&p, epoch_, cur_stream());
    check_last_error("a2a return");
    return ret_local;
  }

 private:
  dlv::A2AParams with_status(int device) {
    dlv::A2AParams p = p_;
    p.status = scratch_for(device).status.data_ptr<int>();
    return p;
  }
  dlv::A2AParams p_;
  int H_;
  unsigned epoch_ = 0;
};

// ---- LoRA delta, pooling, classifier softmax, TurboQuant, LZ4 ------------------------------------------------------------------
// y += (x @ A^T) @ Bs^T in place; x [M, K], A [r, K], Bs [N, r] (already scaled), y [M, N], all bf16, r <= 64.
void lora_delta(const Tensor& x, const Tensor& A, const Tensor& Bs, Tensor& y) {
  check_bf16(A, "A");
  check_bf16(Bs, "B");
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kBFloat16 && x.dim() == 2 && x.stride(1) == 1 && x.stride(0) % 2 == 0, "x must be bf16 [M, K]");
  TORCH_CHECK(y.is_cuda() && y.scalar_type() == at::kBFloat16 && y.dim() == 2 && y.stride(1) == 1 && y.size(0) == x.size(0), "y must be bf16 [M, N]");
  const int r = static_cast<int>(A.size(0));
  TORCH_CHECK(A.dim() == 2 && A.size(1) == x.size(1) && Bs.dim() == 2 && Bs.size(0) == y.size(1) && Bs.size(1) == r && r >= 1 && r <= 64 && x.size(1) % 2 == 0,
              "adapter shapes: A [r, K], B [N, r], r <= 64, K even");
  c10::cuda::CUDAGuard guard(x.device());
  dlv::launch_lora_delta(x.data_ptr(), static_cast<int>(x.stride(0)), A.data_ptr(), Bs.data_ptr(), y.data_ptr(), static_cast<int>(y.stride(0)),
                         static_cast<int>(x.size(0)), static_cast<int>(x.size(1)), static_cast<int>(y.size(1)), r, cur_stream());
  check_last_error("lora_delta");
}
// Pools rows [start[s], start[s] + len[s]) of h [T, H] (bf16) into out [S, H] fp32. mode: 0 mean, 1 max, 2 sum, 3 first, 4 last,
// 5 sum / sqrt(len), 6 position-weighted mean.
Tensor pool_rows(const Tensor& h, const Tensor& start, const Tensor& len, int64_t mode, bool normalize) {
  check_bf16(h, "h");
  check_cuda(start, "start");
  check_cuda(len, "len");
  TORCH_CHECK(h.dim() == 2 && start.scalar_type() == at::kInt && len.scalar_type() == at::kInt && start.numel() == len.numel() && mode >= 0 && mode <= 6, "bad pooling arguments");
  TORCH_CHECK((start + len).max().item<int>() <= h.size(0) && start.min().item<int>() >= 0 && len.min().item<int>() >= 0, "segments outside the hidden states");
  c10::cuda::CUDAGuard guard(h.device());
  Tensor out = new_out({start.numel(), h.size(1)}, h.options().dtype(at::kFloat));
  dlv::launch_pool(h.data_ptr(), static_cast<int>(h.size(1)), start.data_ptr<int>(), len.data_ptr<int>(), static_cast<int>(start.numel()), static_cast<int>(mode),
                   normalize ? 1 : 0, out.data_ptr<float>(), cur_stream());
  check_last_error("pool_rows");
  return out;
}
Tensor softmax_rows(const Tensor& x) {
  check_cuda(x, "x");
  TORCH_CHECK(x.scalar_type() == at::kFloat && x.dim() == 2, "x must be fp32 [rows, C]");
  c10::cuda::CUDAGuard guard(x.device());
  Tensor y = new_out(x.sizes(), x.options());
  dlv::launch_softmax_rows(x.data_ptr<float>(), y.data_ptr<float>(), static_cast<int>(x.size(0)), static_cast<int>(x.size(1)), cur_stream());
  check_last_error("softmax_rows");
  return y;
}
// TurboQuant rows: x [rows, dim] (fp32 / bf16) -> (packed codes uint8 [rows, pdim * bits / 8], norms fp32 [rows])
std::vector<Tensor> tq_encode(const Tensor& x, const Tensor& signs, const Tensor& edges, int64_t bits) {
  check_cuda(x, "x");
  check_cuda(signs, "signs");
  check_cuda(edges, "edges");
  TORCH_CHECK(x.dim() == 2 && (x.scalar_type() == at::kFloat || x.scalar_type() == at::kBFloat16), "x must be fp32 / bf16 [rows, dim]");
  const int dim = static_cast<int>(x.size(1)), pdim = static_cast<int>(signs.numel());
  TORCH_CHECK(pdim >= 32 && pdim <= 1024 && (pdim & (pdim - 1)) == 0 && dim <= pdim && bits >= 1 && bits <= 8, "pdim must be a power of two in 32..1024");
  TORCH_CHECK(signs.scalar_type() == at::kFloat && edges.scalar_type() == at::kFloat && edges.numel() == (1 << bits) - 1, "signs [pdim] / edges [2^bits - 1] fp32");
  c10::cuda::CUDAGuard guard(x.device());
  Tensor codes = new_out({x.size(0), pdim * bits / 8}, x.options().dtype(at::kByte));
  Tensor norms = new_out({x.size(0)}, x.options().dtype(at::kFloat));
  dlv::launch_tq_encode(x.data_ptr(), x.scalar_type() == at::kFloat ? 0 : 1, x.size(0), dim, pdim, static_cast<int>(bits), signs.data_ptr<float>(),
                        edges.data_ptr<float>(), codes.data_ptr<uint8_t>(), norms.data_ptr<float>(), cur_stream());
  check_last_error("tq_encode");
  return {codes, norms};
}
Tensor tq_decode(const Tensor& codes, const Tensor& norms, const Tensor& signs, const Tensor& centroids, int64_t dim, int64_t bits, bool to_bf16) {
  check_cuda(codes, "codes");
  check_cuda(norms, "norms");
  check_cuda(signs, "signs");
  check_cuda(centroids, "centroids");
  const int pdim = static_cast<int>(signs.numel());
  TORCH_CHECK(codes.scalar_type() == at::kByte && codes.dim() == 2 && codes.size(1) == pdim * bits / 8 && norms.scalar_type() == at::kFloat && norms.numel() == codes.size(0),
              "codes [rows, pdim * bits / 8] uint8, norms [rows] fp32");
  TORCH_CHECK(pdim >= 32 && pdim <= 1024 && (pdim & (pdim - 1)) == 0 && dim <= pdim && bits >= 1 && bits <= 8 && centroids.numel() == (1 << bits) &&
                  centroids.scalar_type() == at::kFloat && signs.scalar_type() == at::kFloat, "bad codec tables");
  c10::cuda::CUDAGuard guard(codes.device());
  Tensor out = new_out({codes.size(0), dim}, codes.options().dtype(to_bf16 ? at::kBFloat16 : at::kFloat));
  dlv::launch_tq_decode(codes.data_ptr<uint8_t>(), norms.data_ptr<float>(), codes.size(0), static_cast<int>(dim), pdim, static_cast<int>(bits), signs.data_ptr<float>(),
                        centroids.data_ptr<float>(), out.data_ptr(), to_bf16 ? 1 : 0, cur_stream());
  check_last_error("tq_decode");
  return out;
}
py::bytes lz4_compress_bytes(const std::string& raw) {
  std::string out(dlv::lz4_compress_bound(raw.size()), '\0');
  const size_t n = dlv::lz4_compress(reinterpret_cast<const uint8_t*>(raw.data()), raw.size(), reinterpret_cast<uint8_t*>(&out[0]), out.size());
  return py::bytes(out.data(), n);
}
py::bytes lz4_decompress_bytes(const std::string& comp, int64_t n_out) {
  TORCH_CHECK(n_out >= 0, "bad decoded size");
  std::string out(static_cast<size_t>(n_out), '\0');
  dlv::lz4_decompress(reinterpret_cast<const uint8_t*>(comp.data()), comp.size(), reinterpret_cast<uint8_t*>(&out[0]), out.size());
  return py::bytes(out);
}

// ---- MoE --------------------------------------------------------------------------------------------------------------
// returns weights [T, k] f32, expert ids [T, k] i32, counts [E], offsets [E+1], perm [T*k], pos [T*k]
bool g_moe_parallel_sort = true;  // (comparisons: false keeps the single-CTA grouping for every batch size)
std::vector<Tensor> moe_route(const Tensor& logits, int64_t k, int64_t mode, bool renorm) {
  TORCH_CHECK(logits.is_cuda() && logits.scalar_type() == at::kFloat && logits.dim() == 2 && logits.is_contiguous(), "router logits must be fp32 [T, E]");
  const int T = static_cast<int>(logits.size(0)), E = static_cast<int>(logits.size(1));
  TORCH_CHECK(k >= 1 && k <= 16 && k <= E && E <= 1024, "unsupported top-k / expert count");
  c10::cuda::CUDAGuard guard(logits.device());
  auto io = logits.options().dtype(at::kInt);
  Tensor w = new_out({T, k}, logits.options()), idx = new_out({T, k}, io), counts = new_out({E}, io);
  Tensor offsets = new_out({E + 1}, io), perm = new_out({T * k}, io), pos = new_out({T * k}, io);
  Tensor ws;  // per-chunk expert histograms of the parallel grouping (prefill-size batches)
  const size_t ws_ints = g_moe_parallel_sort ? dlv::moe_route_workspace_ints(T, E, static_cast<int>(k)) : 0;
  if (ws_ints > 0) ws = new_out({static_cast<int64_t>(ws_ints)}, io);
  dlv::launch_moe_route(logits.data_ptr<float>(), T, E, static_cast<int>(k), static_cast<int>(mode), renorm ? 1 : 0, w.data_ptr<float>(),
                        idx.data_ptr<int>(), counts.data_ptr<int>(), offsets.data_ptr<int>(), perm.data_ptr<int>(), pos.data_ptr<int>(),
                        ws_ints > 0 ? ws.data_ptr<int>() : nullptr, cur_stream());
  check_last_error("moe_route");
  return {w, idx, counts, offsets, perm, pos};
}
// moe_route and moe_items of a decode-size batch in one launch: {w, idx, counts, offsets, perm, pos, items}; an empty vector when the
// batch is too large for the single-CTA kernel (the caller then uses the two functions).
std::vector<Tensor> moe_route_items(const Tensor& logits, int64_t k, int64_t mode, bool renorm, int64_t e0, int64_t ne, int64_t bn, int64_t max_items) {
  TORCH_CHECK(logits.is_cuda() && logits.scalar_type() == at::kFloat && logits.dim() == 2 && logits.is_contiguous(), "router logits must be fp32 [T, E]");
  const int T = static_cast<int>(logits.size(0)), E = static_cast<int>(logits.size(1));
  TORCH_CHECK(k >= 1 && k <= 16 && k <= E && E <= 1024, "unsupported top-k / expert count");
  TORCH_CHECK(e0 >= 0 && ne >= 1 && e0 + ne <= E && bn >= 1 && max_items >= 1, "bad work-list arguments");
  if (T < 1 || T > 128 || static_cast<int64_t>(T) * k > 8192) return {};  // (the launcher's limits: no allocations for a batch it refuses)
  c10::cuda::CUDAGuard guard(logits.device());
  auto io = logits.options().dtype(at::kInt);
  Tensor w = new_out({T, k}, logits.options()), idx = new_out({T, k}, io), counts = new_out({E}, io);
  Tensor offsets = new_out({E + 1}, io), perm = new_out({T * k}, io), pos = new_out({T * k}, io), items = new_out({max_items, 4}, io);
  const bool ok = dlv::launch_moe_route_small(logits.data_ptr<float>(), T, E, static_cast<int>(k), static_cast<int>(mode), renorm ? 1 : 0,
                                              w.data_ptr<float>(), idx.data_ptr<int>(), counts.data_ptr<int>(), offsets.data_ptr<int>(),
                                              perm.data_ptr<int>(), pos.data_ptr<int>(), static_cast<int>(e0), static_cast<int>(ne),
                                              static_cast<int>(bn), static_cast<int>(max_items), items.data_ptr<int>(), cur_stream());
  check_last_error("moe_route_items");
  if (!ok) return {};
  return {w, idx, counts, offsets, perm, pos, items};
}
Tensor moe_items(const Tensor& offsets, int64_t e0, int64_t ne, int64_t bn, int64_t max_items) {
  check_cuda(offsets, "offsets");
  TORCH_CHECK(offsets.scalar_type() == at::kInt && e0 >= 0 && ne >= 1 && ne <= 1024 && e0 + ne < offsets.numel() + 0 && bn >= 1 && max_items >= 1, "bad work-list arguments");
  c10::cuda::CUDAGuard guard(offsets.device());
  Tensor items = new_out({max_items, 4}, offsets.options());
  dlv::launch_moe_items(offsets.data_ptr<int>(), static_cast<int>(e0), static_cast<int>(ne), static_cast<int>(bn), static_cast<int>(max_items), items.data_ptr<int>(), cur_stream());
  check_last_error("moe_items");
  return items;
}
// offsets / e0 / ne (optional): only rows of the local experts [e0, e0 + ne) are touched
Tensor moe_gather(const Tensor& x, const Tensor& perm, int64_t k, c10::optional<Tensor> offsets, int64_t e0, int64_t ne) {
  check_bf16(x, "x");
  check_cuda(perm, "perm");
  TORCH_CHECK(perm.scalar_type() == at::kInt && x.dim() == 2 && x.size(1) % 8 == 0 && perm.numel() == x.size(0) * k, "bad gather arguments");
  c10::cuda::CUDAGuard guard(x.device());
  Tensor xs = new_out({perm.numel(), x.size(1)}, x.options());
  const int* off = nullptr;
  if (offsets.has_value()) {
    TORCH_CHECK(offsets.value().is_cuda() && offsets.value().scalar_type() == at::kInt && e0 + ne < offsets.value().numel(), "bad expert range");
    off = offsets.value().data_ptr<int>();
  }
  dlv::launch_moe_gather(x.data_ptr(), perm.data_ptr<int>(), static_cast<int>(perm.numel()), static_cast<int>(k), static_cast<int>(x.size(1)), xs.data_ptr(), off, static_cast<int>(e0), static_cast<int>(ne), cur_stream());
  check_last_error("moe_gather");
  return xs;
}
Tensor moe_combine(const Tensor& ys, const Tensor& pos, const Tensor& w, int64_t T, int64_t k, c10::optional<Tensor> offsets, int64_t e0, int64_t ne) {
  check_bf16(ys, "ys");
  check_cuda(pos, "pos");
  check_cuda(w, "w");
  TORCH_CHECK(pos.scalar_type() == at::kInt && w.scalar_type() == at::kFloat && pos.numel() == T * k && w.numel() == T * k && ys.size(0) == T * k && ys.size(1) % 8 == 0, "bad combine arguments");
  c10::cuda::CUDAGuard guard(ys.device());
  Tensor out = new_out({T, ys.size(1)}, ys.options());
  const int* off = nullptr;
  if (offsets.has_value()) {
    TORCH_CHECK(offsets.value().is_cuda() && offsets.value().scalar_type() == at::kInt && e0 + ne < offsets.value().numel(), "bad expert range");
    off = offsets.value().data_ptr<int>();
  }
  dlv::launch_moe_combine(ys.data_ptr(), pos.data_ptr<int>(), w.data_ptr<float>(), static_cast<int>(T), static_cast<int>(k), static_cast<int>(ys.size(1)), out.data_ptr(), off, static_cast<int>(e0), static_cast<int>(ne), cur_stream());
  check_last_error("moe_combine");
  return out;
}

// Expert-parallel combine fused with the all-reduce over peer memory; returns false (nothing launched) outside the fused path.
bool moe_combine_allreduce(const Tensor& ys, const Tensor& pos, const Tensor& w, int64_t T, int64_t k, const Tensor& offsets, int64_t e0,
                           int64_t ne, const TpComm& comm, Tensor& out) {
  check_bf16(ys, "ys");
  check_cuda(pos, "pos");
  check_cuda(w, "w");
  check_cuda(offsets, "offsets");
  const int H = static_cast<int>(ys.size(1));
  TORCH_CHECK(pos.scalar_type() == at::kInt && w.scalar_type() == at::kFloat && offsets.scalar_type() == at::kInt && pos.numel() == T * k &&
                  w.numel() == T * k && ys.size(0) == T * k && e0 + ne < offsets.numel(), "bad combine arguments");
  TORCH_CHECK(out.is_cuda() && out.scalar_type() == at::kBFloat16 && out.dim() == 2 && out.size(0) == T && out.size(1) == H && out.is_contiguous() &&
                  ys.is_contiguous(), "bad out");
  if (!dlv::comm_rows_supported(comm.args(), static_cast<int>(T), H)) return false;
  c10::cuda::CUDAGuard guard(ys.device());
  DeviceScratch& s = scratch_for(ys.device().index());
  dlv::launch_moe_combine_allreduce(ys.data_ptr(), pos.data_ptr<int>(), w.data_ptr<float>(), static_cast<int>(T), static_cast<int>(k), H,
                                    offsets.data_ptr<int>(), static_cast<int>(e0), static_cast<int>(ne), out.data_ptr(), comm.args(),
                                    s.status.data_ptr<int>(), cur_stream());
  check_last_error("moe_combine_allreduce");
  return true;
}
// Second half of the split form (see GemmWeight::run_tp_push): sum over the ranks (+ bias), then kind 0: out = sum; kind 1:
// residual += [RMSNorm(post_w)](sum) * res_mult (in place) and out = RMSNorm(residual, norm_w).
void tp_reduce_norm(const TpComm& comm, int64_t mode, int64_t ctas, int64_t M, int64_t N, int64_t kind, c10::optional<Tensor> bias,
                    c10::optional<Tensor> residual, c10::optional<Tensor> post_w, c10::optional<Tensor> norm_w, Tensor& out, double eps, double offset,
                    double res_mult) {
  TORCH_CHECK(ctas > 0 && M > 0 && M <= 128 && N % 8 == 0 && N <= 12288, "bad reduce shape");
  TORCH_CHECK(out.is_cuda() && out.scalar_type() == at::kBFloat16 && out.dim() == 2 && out.size(0) == M && out.size(1) == N && out.is_contiguous(), "bad out");
  dlv::GemmTpArgs a = comm.with_mode(static_cast<int>(mode));
  a.last_ctas = static_cast<int>(ctas);
  const float* bptr = nullptr;
  if (bias.has_value()) {
    TORCH_CHECK(bias.value().is_cuda() && bias.value().scalar_type() == at::kFloat && bias.value().numel() == N && bias.value().is_contiguous(), "bias must be fp32 [N]");
    bptr = bias.value().data_ptr<float>();
  }
  void* rp = nullptr;
  const void* pw = nullptr;
  const void* nw = nullptr;
  if (kind == 1) {
    TORCH_CHECK(residual.has_value() && norm_w.has_value(), "residual and norm weight are required");
    check_bf16(residual.value(), "residual");
    check_bf16(norm_w.value(), "norm_w");
    TORCH_CHECK(residual.value().dim() == 2 && residual.value().size(0) == M && residual.value().size(1) == N && norm_w.value().numel() == N, "residual / norm shape");
    rp = residual.value().data_ptr();
    nw = norm_w.value().data_ptr();
    if (post_w.has_value()) {
      check_bf16(post_w.value(), "post_w");
      TORCH_CHECK(post_w.value().numel() == N, "post norm shape");
      pw = post_w.value().data_ptr();
    }
  } else {
    TORCH_CHECK(kind == 0, "kind must be 0 or 1");
  }
  c10::cuda::CUDAGuard guard(out.device());
  DeviceScratch& s = scratch_for(out.device().index());
  dlv::launch_tp_reduce_norm(&a, static_cast<int>(M), static_cast<int>(N), static_cast<int>(kind), bptr, rp, pw, nw, out.data_ptr(), static_cast<float>(eps),
                             static_cast<float>(offset), static_cast<float>(res_mult), s.status.data_ptr<int>(), cur_stream());
  check_last_error("tp_reduce_norm");
}
// One-shot all-reduce of a small bf16 tensor [rows <= 128, H] over peer memory; false when the shape is outside the fused path.
bool oneshot_allreduce(const Tensor& x, const TpComm& comm, Tensor& out) {
  check_bf16(x, "x");
  TORCH_CHECK(x.dim() == 2 && x.is_contiguous() && out.is_cuda() && out.scalar_type() == at::kBFloat16 && out.sizes() == x.sizes() && out.is_contiguous(), "bad all-reduce arguments");
  const int rows = static_cast<int>(x.size(0)), H = static_cast<int>(x.size(1));
  if (!dlv::comm_rows_supported(comm.args(), rows, H)) return false;
  c10::cuda::CUDAGuard guard(x.device());
  DeviceScratch& s = scratch_for(x.device().index());
  dlv::launch_oneshot_allreduce(x.data_ptr(), rows, H, out.data_ptr(), comm.args(), s.status.data_ptr<int>(), cur_stream());
  check_last_error("oneshot_allreduce");
  return true;
}

// ---- persistent decode chain ------------------------------------------------------------------------------------------
// A chain is described once (weights, buffers, norm weights are fixed for a model's lifetime) and run once per decode step and
// layer: `run(M, positions, slots)`. All buffers have kChainMaxRows rows; rows >= M are ignored.
class DecodeChain {
 public:
  DecodeChain() {}
  // kind: 0 store, 1 add + norm (unscaled, see chain_api.h), 2 act(gate) * up, 3 q|k|v (set_qkv must follow), 4 add.
  // dep: x is the output of the projection added before this one. scale_src: index of the add + norm stage whose row factor applies.
  void add_op(const GemmWeight& w, const Tensor& x, int64_t kind, bool dep, int64_t scale_src, c10::optional<Tensor> bias,
              c10::optional<Tensor> residual, c10::optional<Tensor> norm_w, c10::optional<Tensor> out, double eps, double offset, double res_mult,
              const std::string& act) {
    TORCH_CHECK(static_cast<int>(ops_.size()) < dlv::kChainMaxOps, "a chain holds at most 4 projections");
    TORCH_CHECK(!sync_.defined(), "the chain is sealed by its first run");
    const dlv::GemmWeightDesc* d = w.desc();
    TORCH_CHECK(d->is_q4, "the decode chain takes JQ4 weights");
    TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kBFloat16 && x.dim() == 2 && x.size(1) == d->K && x.is_contiguous() && x.size(0) >= dlv::kChainMaxRows,
                "chain input must be contiguous bf16 [>= 64, K]");
    TORCH_CHECK((reinterpret_cast<uintptr_t>(x.data_ptr()) & 15) == 0 && d->K % 64 == 0 && d->N % 8 == 0, "chain input alignment / shape");
    TORCH_CHECK(kind >= 0 && kind <= 4, "unknown tile stage");
    dlv::ChainOp o;
    o.wq = d->data;
    o.N = d->N;
    o.K = d->K;
    o.x = x.data_ptr();
    o.x_rows = static_cast<int>(x.size(0));
    o.dep = dep;
    o.scale_src = static_cast<int>(scale_src);
    c10::cuda::CUDAGuard guard(x.device());
    auto fopt = torch::TensorOptions().device(x.device()).dtype(torch::kFloat32);
    Tensor ws = torch::empty({static_cast<long>(dlv::chain_ws_floats(d->N, d->K, dlv::chain_ctas()))}, fopt);
    o.ws = ws.data_ptr<float>();
    keep_.push_back(ws);
    o.kind = static_cast<int>(kind);
    if (bias.has_value()) {
      TORCH_CHECK(bias.value().is_cuda() && bias.value().scalar_type() == at::kFloat && bias.value().numel() == d->N && bias.value().is_contiguous() && d->N % 4 == 0, "bias must be fp32 [N]");
      TORCH_CHECK(kind != 2, "the activation stage takes no bias");
      o.bias = bias.value().data_ptr<float>();
    }
    if (kind == 1 || kind == 4) {
      TORCH_CHECK(residual.has_value(), "the stage needs the residual rows");
      check_bf16(residual.value(), "residual");
      TORCH_CHECK(residual.value().dim() == 2 && residual.value().size(0) >= dlv::kChainMaxRows && residual.value().size(1) == d->N && d->N % 4 == 0, "residual shape");
      o.residual = residual.value().data_ptr();
    }
    if (kind == 1) {
      TORCH_CHECK(norm_w.has_value(), "add + norm needs the norm weight");
      check_bf16(norm_w.value(), "norm_w");
      TORCH_CHECK(norm_w.value().numel() == d->N, "norm weight shape");
      o.norm_w = norm_w.value().data_ptr();
      Tensor ssq = torch::zeros({static_cast<long>((d->N + 127) / 128) * 64}, fopt);
      o.ssq = ssq.data_ptr<float>();
      keep_.push_back(ssq);
    }
    if (kind != 4) {
      TORCH_CHECK(out.has_value(), "the stage needs an output buffer");
      check_bf16(out.value(), "out");
      const int64_t out_cols = kind == 2 ? d->N / 2 : (kind == 3 ? -1 : d->N);
      TORCH_CHECK(out.value().dim() == 2 && out.value().size(0) >= dlv::kChainMaxRows && (out_cols < 0 || out.value().size(1) == out_cols),
                  "chain output must be bf16 [>= 64, cols]");
      o.out = out.value().data_ptr();
    }
    o.eps = static_cast<float>(eps);
    o.offset = static_cast<float>(offset);
    o.res_mult = static_cast<float>(res_mult);
    o.act = act_code(act);
    ops_.push_back(o);
    keep_.push_back(x);
    keep_.push_back(w.data());
    for (auto& t : {bias, residual, norm_w, out})
      if (t.has_value()) keep_.push_back(t.value());
  }
  void set_qkv(c10::optional<Tensor> q_norm_w, c10::optional<Tensor> k_norm_w, c10::optional<Tensor> cos_t, c10::optional<Tensor> sin_t, Tensor& k_cache,
               Tensor& v_cache, int64_t H, int64_t KV, double eps, double norm_offset) {
    check_bf16(k_cache, "k_cache");
    check_bf16(v_cache, "v_cache");
    TORCH_CHECK(k_cache.dim() == 4 && k_cache.size(1) == KV && k_cache.is_contiguous() && v_cache.sizes() == k_cache.sizes() && v_cache.is_contiguous(),
                "cache must be contiguous [pages, KV, page, head_dim]");
    const int D = static_cast<int>(k_cache.size(3));
    TORCH_CHECK(D == 64 || D == 128, "head_dim must be 64 or 128");
    qkv_ = {};
    if (q_norm_w.has_value()) {
      check_bf16(q_norm_w.value(), "q_norm");
      check_bf16(k_norm_w.value(), "k_norm");
      TORCH_CHECK(q_norm_w.value().numel() == D && k_norm_w.value().numel() == D, "q/k norm weights must have head_dim entries");
      qkv_.q_norm_w = reinterpret_cast<const __nv_bfloat16*>(q_norm_w.value().data_ptr());
      qkv_.k_norm_w = reinterpret_cast<const __nv_bfloat16*>(k_norm_w.value().data_ptr());
      keep_.push_back(q_norm_w.value());
      keep_.push_back(k_norm_w.value());
    }
    qkv_.max_pos = 1;
    if (cos_t.has_value()) {
      TORCH_CHECK(cos_t.value().is_cuda() && cos_t.value().scalar_type() == at::kFloat && cos_t.value().dim() == 2 && cos_t.value().is_contiguous() &&
                  sin_t.value().sizes() == cos_t.value().sizes() && sin_t.value().is_contiguous() && sin_t.value().is_cuda(), "cos/sin must be contiguous fp32 [max_pos, rot/2]");
      qkv_.cos_t = cos_t.value().data_ptr<float>();
      qkv_.sin_t = sin_t.value().data_ptr<float>();
      qkv_.rot_half = static_cast<int>(cos_t.value().size(1));
      qkv_.max_pos = static_cast<int>(cos_t.value().size(0));
      TORCH_CHECK(qkv_.rot_half == D / 2, "the chain applies full rotary embeddings only");
      keep_.push_back(cos_t.value());
      keep_.push_back(sin_t.value());
    }
    qkv_.k_cache = reinterpret_cast<__nv_bfloat16*>(k_cache.data_ptr());
    qkv_.v_cache = reinterpret_cast<__nv_bfloat16*>(v_cache.data_ptr());
    qkv_.heads = static_cast<int>(H);
    qkv_.kv_heads = static_cast<int>(KV);
    qkv_.head_dim = D;
    qkv_.block_size = static_cast<int>(k_cache.size(2));
    qkv_.eps = static_cast<float>(eps);
    qkv_.norm_offset = static_cast<float>(norm_offset);
    keep_.push_back(k_cache);
    keep_.push_back(v_cache);
    has_qkv_ = true;
  }
  void run(int64_t M, c10::optional<Tensor> positions, c10::optional<Tensor> slots) {
    TORCH_CHECK(!ops_.empty() && M >= 0 && M <= dlv::kChainMaxRows, "chain: 0..64 rows");
    if (M == 0) return;
    const int dev = static_cast<const Tensor&>(keep_.front()).device().index();
    c10::cuda::CUDAGuard guard(keep_.front().device());
    if (!sync_.defined()) {
      sync_words_ = dlv::chain_sync_words(ops_.data(), static_cast<int>(ops_.size()));
      sync_ = torch::zeros({sync_words_}, torch::TensorOptions().device(keep_.front().device()).dtype(torch::kInt32));
    }
    bool needs_qkv = false;
    for (auto& o : ops_) needs_qkv = needs_qkv || o.kind == dlv::kChainRowQkvRope;
    dlv::ChainQkvArgs a = qkv_;
    if (needs_qkv) {
      TORCH_CHECK(has_qkv_ && positions.has_value(), "the q|k|v stage needs set_qkv and positions");
      TORCH_CHECK(positions.value().is_cuda() && positions.value().scalar_type() == at::kInt && positions.value().numel() >= M, "positions must be int32 [M]");
      a.positions = positions.value().data_ptr<int>();
      a.slots = nullptr;
      if (slots.has_value()) {
        TORCH_CHECK(slots.value().is_cuda() && slots.value().scalar_type() == at::kLong && slots.value().numel() >= M, "slots must be int64 [M]");
        a.slots = reinterpret_cast<const long long*>(slots.value().data_ptr<int64_t>());
      }
    }
    DeviceScratch& s = scratch_for(dev);
    dlv::chain_run(ops_.data(), static_cast<int>(ops_.size()), needs_qkv ? &a : nullptr, static_cast<int>(M),
                   reinterpret_cast<unsigned*>(sync_.data_ptr<int>()), sync_words_, s.status.data_ptr<int>(), cur_stream());
    check_last_error("decode chain launch");
  }
  // after a launch that ended with a status error the counters may be left non-zero: clear them before the next launch
  void reset() {
    if (sync_.defined()) sync_.zero_();
  }
  Tensor counters() const { return sync_; }

 private:
  std::vector<dlv::ChainOp> ops_;
  dlv::ChainQkvArgs qkv_ = {};
  bool has_qkv_ = false;
  Tensor sync_;
  int sync_words_ = 0;
  std::vector<Tensor> keep_;
};

// ---- Mamba2 -----------------------------------------------------------------------------------------------------------
// meta: int32 tensors prepared on the host (row_seq [T], chunk_* [n_chunks], seq_chunk0 / seq_nchunks [S])
Tensor mamba2_forward(const Tensor& zx, const Tensor& conv_w, c10::optional<Tensor> conv_b, const Tensor& dt_bias, const Tensor& A_log,
                      const Tensor& D, const Tensor& norm_w, Tensor& conv_state, Tensor& ssm_state, const Tensor& slots, const Tensor& q_start,
                      const Tensor& q_len, const Tensor& positions, const Tensor& row_seq, const Tensor& chunk_seq, const Tensor& chunk_row0,
                      const Tensor& chunk_len, const Tensor& chunk_first, const Tensor& chunk_last, const Tensor& seq_chunk0,
                      const Tensor& seq_nchunks, bool multi_chunk, int64_t H, int64_t d_head, int64_t G, int64_t S, double eps) {
  check_bf16(zx, "zx");
  const int T = static_cast<int>(zx.size(0));
  const int I = static_cast<int>(H * d_head), conv_dim = static_cast<int>(I + 2 * G * S);
  TORCH_CHECK(zx.dim() == 2 && zx.size(1) == I + conv_dim + H, "in_proj output has the wrong width");
  for (const Tensor* t : std::initializer_list<const Tensor*>{&conv_w, &dt_bias, &A_log, &D, &norm_w, &conv_state, &ssm_state}) {
    check_cuda(*t, "mamba parameter");
    TORCH_CHECK(t->scalar_type() == at::kFloat, "mamba parameters and states are fp32");
  }
  const int K = static_cast<int>(conv_w.numel() / conv_dim);
  TORCH_CHECK(conv_state.dim() == 3 && conv_state.size(1) == conv_dim && conv_state.size(2) == K - 1, "conv_state must be [slots, convDim, K-1]");
  TORCH_CHECK(ssm_state.dim() == 4 && ssm_state.size(1) == H && ssm_state.size(2) == d_head && ssm_state.size(3) == S, "ssm_state must be [slots, H, d_head, S]");
  check_cuda(slots, "slots");
  TORCH_CHECK(slots.scalar_type() == at::kLong, "slots must be int64");
  for (const Tensor* t : {&q_start, &q_len, &positions, &row_seq, &chunk_seq, &chunk_row0, &chunk_len, &chunk_first, &chunk_last, &seq_chunk0, &seq_nchunks}) {
    check_cuda(*t, "index tensor");
    TORCH_CHECK(t->scalar_type() == at::kInt, "index tensors must be int32");
  }
  const int num_seqs = static_cast<int>(q_len.numel()), n_chunks = static_cast<int>(chunk_seq.numel());
  c10::cuda::CUDAGuard guard(zx.device());
  auto fo = zx.options().dtype(at::kFloat);
  Tensor xbc = new_out({T, conv_dim}, fo), ybuf = new_out({T, I}, fo);
  Tensor cstate = new_out({std::max(1, n_chunks), H, d_head, S}, fo), cdecay = new_out({std::max(1, n_chunks), H}, fo);
  Tensor out = new_out({T, I}, zx.options());
  const float* cb = conv_b.has_value() ? conv_b.value().data_ptr<float>() : nullptr;
  int rc = dlv::launch_mamba2(zx.data_ptr(), static_cast<int>(zx.stride(0)), T, num_seqs, I, conv_dim, K, static_cast<int>(H), static_cast<int>(d_head),
                              static_cast<int>(G), static_cast<int>(S), conv_w.data_ptr<float>(), cb, dt_bias.data_ptr<float>(), A_log.data_ptr<float>(),
                              D.data_ptr<float>(), norm_w.data_ptr<float>(), static_cast<float>(eps), conv_state.data_ptr<float>(), ssm_state.data_ptr<float>(),
                              reinterpret_cast<const long long*>(slots.data_ptr<int64_t>()), row_seq.data_ptr<int>(), q_start.data_ptr<int>(),
                              q_len.data_ptr<int>(), positions.data_ptr<int>(), n_chunks, chunk_seq.data_ptr<int>(), chunk_row0.data_ptr<int>(),
                              chunk_len.data_ptr<int>(), chunk_first.data_ptr<int>(), chunk_last.data_ptr<int>(), seq_chunk0.data_ptr<int>(),
                              seq_nchunks.data_ptr<int>(), multi_chunk ? 1 : 0, xbc.data_ptr<float>(), ybuf.data_ptr<float>(), cstate.data_ptr<float>(),
                              cdecay.data_ptr<float>(), out.data_ptr(), cur_stream());
  TORCH_CHECK(rc == 0, "mamba2: unsupported shape (code ", rc, ")");
  check_last_error("mamba2_forward");
  return out;
}

// ---- JQ4 ------------------------------------------------------------------------------------------------------------
std::vector<Tensor> q4_quantize(const Tensor& w) {
  check_cuda(w, "w");
  TORCH_CHECK(w.size(-1) % 32 == 0, "last dimension must be a multiple of 32");
  int code = w.scalar_type() == at::kFloat ? 0 : w.scalar_type() == at::kBFloat16 ? 1 : w.scalar_type() == at::kHalf ? 2 : -1;
  TORCH_CHECK(code >= 0, "unsupported dtype for quantisation");
  c10::cuda::CUDAGuard guard(w.device());
  auto shape = w.sizes().vec();
  auto pshape = shape, sshape = shape;
  pshape.back() = shape.back() / 2;
  sshape.back() = shape.back() / 32;
  Tensor packed = new_out(pshape, w.options().dtype(at::kByte));
  Tensor scales = new_out(sshape, w.options().dtype(at::kFloat));
  dlv::launch_q4_quantize(w.data_ptr(), code, w.numel() / 32, packed.data_ptr<uint8_t>(), scales.data_ptr<float>(), cur_stream());
  check_last_error("q4_quantize");
  return {packed, scales};
}
Tensor q4_dequantize(const Tensor& packed, const Tensor& scales, bool to_bf16) {
  check_cuda(packed, "packed");
  check_cuda(scales, "scales");
  TORCH_CHECK(packed.scalar_type() == at::kByte && scales.scalar_type() == at::kFloat, "packed uint8 + fp32 scales expected");
  TORCH_CHECK(packed.numel() == scales.numel() * 16, "packed / scale sizes do not match");
  c10::cuda::CUDAGuard guard(packed.device());
  auto shape = packed.sizes().vec();
  shape.back() *= 2;
  Tensor out = new_out(shape, packed.options().dtype(to_bf16 ? at::kBFloat16 : at::kFloat));
  dlv::launch_q4_dequantize(packed.data_ptr<uint8_t>(), scales.data_ptr<float>(), scales.numel(), out.data_ptr(), to_bf16 ? 1 : 0, cur_stream());
  check_last_error("q4_dequantize");
  return out;
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  py::class_<TpComm, std::shared_ptr<TpComm>>(m, "TpComm")
      .def(py::init<int64_t, int64_t, std::vector<int64_t>, std::vector<int64_t>, int64_t, int64_t, Tensor, Tensor>())
      .def("set_wait_limit_ms", &TpComm::set_wait_limit_ms)
      .def("set_multicast", &TpComm::set_multicast)
      .def("has_multicast", &TpComm::has_multicast);
  py::class_<ExpertA2A, std::shared_ptr<ExpertA2A>>(m, "ExpertA2A")
      .def(py::init<int64_t, int64_t, int64_t, int64_t, int64_t, std::vector<int64_t>, std::vector<int64_t>, std::vector<int64_t>, std::vector<int64_t>>())
      .def("dispatch", &ExpertA2A::dispatch)
      .def("receive", &ExpertA2A::receive)
      .def("finish", &ExpertA2A::finish);
  py::class_<DecodeChain, std::shared_ptr<DecodeChain>>(m, "DecodeChain")
      .def(py::init<>())
      .def("add_op", &DecodeChain::add_op, py::arg("w"), py::arg("x"), py::arg("kind"), py::arg("dep") = false, py::arg("scale_src") = -1,
           py::arg("bias") = py::none(), py::arg("residual") = py::none(), py::arg("norm_w") = py::none(), py::arg("out") = py::none(),
           py::arg("eps") = 1e-6, py::arg("offset") = 0.0, py::arg("res_mult") = 1.0, py::arg("act") = "silu")
      .def("set_qkv", &DecodeChain::set_qkv)
      .def("run", &DecodeChain::run, py::arg("M"), py::arg("positions") = py::none(), py::arg("slots") = py::none())
      .def("reset", &DecodeChain::reset)
      .def("counters", &DecodeChain::counters);
  py::class_<TpScatter, std::shared_ptr<TpScatter>>(m, "TpScatter")
      .def(py::init<int64_t, int64_t, std::vector<int64_t>, std::vector<int64_t>, std::vector<int64_t>, int64_t, int64_t>());
  m.def("scatter_plan", &scatter_plan);
  py::class_<GemmWeight, std::shared_ptr<GemmWeight>>(m, "GemmWeight")
      .def(py::init<Tensor, bool, int64_t, int64_t>(), py::arg("w"), py::arg("is_q4"), py::arg("N"), py::arg("K"))
      .def("run", &GemmWeight::run, py::arg("x"), py::arg("out") = py::none(), py::arg("bias") = py::none(), py::arg("out_f32") = false,
           py::arg("impl") = 0, py::arg("force_splits") = 0)
      .def("run_tp", &GemmWeight::run_tp, py::arg("x"), py::arg("out"), py::arg("comm"), py::arg("bias") = py::none())
      .def("run_tp_push", &GemmWeight::run_tp_push, py::arg("x"), py::arg("comm"), py::arg("mode") = 1)
      .def("run_scatter", &GemmWeight::run_scatter, py::arg("x"), py::arg("out"), py::arg("comm"), py::arg("bias") = py::none(),
           py::arg("gather") = true)
      .def("run_gathered", &GemmWeight::run_gathered, py::arg("x_own"), py::arg("M"), py::arg("out"), py::arg("comm"), py::arg("bias") = py::none())
      .def("run_act", &GemmWeight::run_act, py::arg("x"), py::arg("act"))
      .def("run_qkv", &GemmWeight::run_qkv)
      .def("run_grouped_act", &GemmWeight::run_grouped_act, py::arg("xs"), py::arg("items"), py::arg("n_per_expert"), py::arg("bn"), py::arg("splits"),
           py::arg("act"))
      .def("run_grouped_gemv_act", &GemmWeight::run_grouped_gemv_act, py::arg("xs"), py::arg("items"), py::arg("n_per_expert"), py::arg("act"),
           py::arg("perm") = py::none(), py::arg("k") = 1)
      .def("run_gemv_act", &GemmWeight::run_gemv_act)
      .def("gemv_ok", &GemmWeight::gemv_ok)
      .def("run_grouped", &GemmWeight::run_grouped, py::arg("xs"), py::arg("items"), py::arg("n_per_expert"), py::arg("bn"), py::arg("splits") = 1,
           py::arg("out") = py::none())
      .def_property_readonly("N", &GemmWeight::n)
      .def_property_readonly("K", &GemmWeight::k)
      .def_property_readonly("is_q4", &GemmWeight::is_q4);
  m.def("take_status", &take_status);
  m.def("init_scratch", &init_scratch);
  m.def("gemm_pdl", [](bool on) { dlv::gemm_set_pdl(on); });
  m.def("num_sms", &dlv::gemm_num_sms);
  m.def("rmsnorm", &rmsnorm);
  m.def("add_rmsnorm", &add_rmsnorm);
  m.def("layernorm", &layernorm);
  m.def("act_mul", &act_mul);
  m.def("activation", &activation);
  m.def("embedding", &embedding, py::arg("table"), py::arg("ids"), py::arg("scale") = 1.0, py::arg("pos_table") = py::none(),
        py::arg("pos") = py::none(), py::arg("type_table") = py::none(), py::arg("types") = py::none());
  m.def("rope_kv", &rope_kv);
  m.def("decode_attention", &decode_attention, py::arg("q"), py::arg("k_cache"), py::arg("v_cache"), py::arg("block_tables"), py::arg("ctx_lens"),
        py::arg("H"), py::arg("scale"), py::arg("softcap") = 0.0, py::arg("window") = 0, py::arg("splits") = 1, py::arg("impl") = 0);
  m.def("prefill_attention", &prefill_attention);
  m.def("prefill_attention_tc", &prefill_attention_tc);
  m.def("prefill_tc_tile_rows", &dlv::prefill_attention_tc_tile_rows);
  m.def("gemv_simt_only", [](bool on) { dlv::g_gemv_simt_only = on; });
  m.def("gemv_dense", [](bool on) { dlv::g_gemv_dense = on; });
  m.def(
      "gemm_persist",
      [](bool on, bool all, bool ordered) {
        dlv::g_gemm_persist = on;
        dlv::g_gemm_persist_all = all;
        dlv::g_gemm_persist_ordered = ordered;
      },
      py::arg("on"), py::arg("all") = false, py::arg("ordered") = true);
  m.def("decode_merge_in_kernel", [](bool on) { g_decode_merge_in_kernel = on; });
  m.def("gemv_max_rows", [](int64_t n) { dlv::g_gemv_max_rows = static_cast<int>(n); });
  m.def("gemv_force_split", [](int64_t s) { dlv::g_gemv_force_split = static_cast<int>(s); });
  m.def("gemm_force_bn", [](int64_t bn) { dlv::g_gemm_force_bn = static_cast<int>(bn); });
  m.def("set_bounds_check", &set_bounds_check);
  m.def("check_guards", &check_guards);
  m.def("poke_last_guard", &poke_last_guard);
  m.def("guarded_empty", [](std::vector<int64_t> sizes, const Tensor& like) { return new_out(sizes, like.options()); });
  m.def("argmax", &argmax, py::arg("logits"), py::arg("mask") = py::none(), py::arg("softcap") = 0.0, py::arg("inv_scale") = 1.0);
  m.def("sample_rows", &sample_rows);
  m.def("sample_rows_packed", &sample_rows_packed);
  m.def("xtc_rows", &xtc_rows);
  m.def("lora_delta", &lora_delta);
  m.def("pool_rows", &pool_rows);
  m.def("softmax_rows", &softmax_rows);
  m.def("tq_encode", &tq_encode);
  m.def("tq_decode", &tq_decode, py::arg("codes"), py::arg("norms"), py::arg("signs"), py::arg("centroids"), py::arg("dim"), py::arg("bits"), py::arg("to_bf16") = false);
  m.def("lz4_compress", &lz4_compress_bytes);
  m.def("lz4_decompress", &lz4_decompress_bytes);
  m.def("logprob_rows", &logprob_rows);
  m.def("logits_post", &logits_post, py::arg("logits"), py::arg("mask") = py::none(), py::arg("softcap") = 0.0, py::arg("inv_scale") = 1.0);
  m.def("moe_route", &moe_route);
  m.def("moe_parallel_sort", [](bool on) { g_moe_parallel_sort = on; });
  m.def("moe_items", &moe_items);
  m.def("moe_route_items", &moe_route_items);
  m.def("moe_gather", &moe_gather, py::arg("x"), py::arg("perm"), py::arg("k"), py::arg("offsets") = py::none(), py::arg("e0") = 0, py::arg("ne") = 0);
  m.def("moe_combine", &moe_combine, py::arg("ys"), py::arg("pos"), py::arg("w"), py::arg("T"), py::arg("k"), py::arg("offsets") = py::none(),
        py::arg("e0") = 0, py::arg("ne") = 0);
  m.def("moe_combine_allreduce", &moe_combine_allreduce);
  m.def("oneshot_allreduce", &oneshot_allreduce);
  m.def("tp_reduce_norm", &tp_reduce_norm, py::arg("comm"), py::arg("mode"), py::arg("ctas"), py::arg("M"), py::arg("N"), py::arg("kind"),
        py::arg("bias") = py::none(), py::arg("residual") = py::none(), py::arg("post_w") = py::none(), py::arg("norm_w") = py::none(), py::arg("out"),
        py::arg("eps") = 1e-6, py::arg("offset") = 0.0, py::arg("res_mult") = 1.0);
  m.def("mamba2_forward", &mamba2_forward);
  m.def("q4_quantize", &q4_quantize);
  m.def("q4_dequantize", &q4_dequantize, py::arg("packed"), py::arg("scales"), py::arg("to_bf16") = false);
}
