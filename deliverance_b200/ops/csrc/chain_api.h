// Host interface of the persistent decode chain (chain.cu): up to four JQ4 projections and the row-wise stages between them in
// one launch. No torch types below this line.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace dlv {

constexpr int kChainMaxOps = 4;
constexpr int kChainMaxRows = 64;   // token rows of a launch (decode batches)

// what the tile stage behind a projection does with the projection's output y (after the optional per-row scale and bias)
enum ChainRowKind {
  kChainRowStore = 0,    // out[m, :N] = y
  kChainRowAddNorm = 1,  // residual += y * res_mult ; out = residual * (norm_w + offset) ; the tile's share of sum(residual^2) -> ssq.
                         // The row factor rsqrt(mean(residual^2) + eps) is NOT applied here: the projection that reads `out` names
                         // this stage as its scale_src and its own tile stage multiplies by it
  kChainRowActMul = 2,   // out[m, :N/2] = act(y[:N/2]) * y[N/2:]
  kChainRowQkvRope = 3,  // per head: q / k RMSNorm (optional), rotary embedding (optional); q -> out, k / v -> paged cache
  kChainRowAdd = 4,      // residual += y * res_mult (nothing else; the last stage of a chain)
};

struct ChainOp {
  const void* wq = nullptr;  // tile-packed JQ4 weight [N, K]
  int N = 0, K = 0;
  const void* x = nullptr;   // bf16 [x_rows, K] input rows of this projection (16-byte aligned, row pitch K); rows >= M are ignored
  int x_rows = 0;
  bool dep = false;          // x is the `out` of the projection in front of this one in the same chain
  int scale_src = -1;        // index of the kChainRowAddNorm stage whose row factor scales y, or -1
  float* ws = nullptr;       // chain_ws_floats(N, K, chain_ctas()) floats of workspace for the partial tiles
  float* ssq = nullptr;      // kChainRowAddNorm: ceil(N / 128) * 64 floats
  int kind = kChainRowStore;
  const float* bias = nullptr;   // [N] fp32 or nullptr
  void* residual = nullptr;      // bf16 [rows, N], updated in place (kChainRowAddNorm, kChainRowAdd)
  const void* norm_w = nullptr;  // bf16 [N]
  void* out = nullptr;           // bf16, see ChainRowKind
  float eps = 1e-6f, offset = 0.f, res_mult = 1.f;
  int act = 0;  // 0 SiLU, 1 GELU (tanh), 2 GELU (erf), 3 ReLU, 4 tanh
};

struct ChainQkvArgs {
  const int* positions;            // [M]
  const long long* slots;          // [M] flat cache rows (< 0: no cache write) or nullptr
  const __nv_bfloat16* q_norm_w;   // [head_dim] or nullptr
  const __nv_bfloat16* k_norm_w;
  const float* cos_t;              // [max_pos, rot_half] or nullptr
  const float* sin_t;
  __nv_bfloat16* k_cache;          // [blocks, kv_heads, block_size, head_dim]
  __nv_bfloat16* v_cache;
  int heads, kv_heads, head_dim, block_size, rot_half, max_pos;
  float eps, norm_offset;
};

int chain_ctas();                                  // CTAs of a chain launch (one per SM)
size_t chain_ws_floats(int N, int K, int ctas);    // workspace floats of one projection
int chain_sync_words(const ChainOp* ops, int n_ops);  // uint32 words of counters this chain needs
// Launch the chain on `st`. `sync`: chain_sync_words() zero-initialised uint32 on the device; the kernel leaves them zero, so one
// array serves every launch of the same chain (and of chains of the same shapes) on a stream. M <= kChainMaxRows token rows.
void chain_run(const ChainOp* ops, int n_ops, const ChainQkvArgs* qkv, int M, unsigned* sync, int sync_words, int* status, cudaStream_t st);

}  // namespace dlv
