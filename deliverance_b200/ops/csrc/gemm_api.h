// C++ interface between the torch bindings and the kernel launchers (no torch types below this line).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace dlv {

// JQ4 weights are held tile-packed on the device: [ceil(N/128)][ceil(K/128)][10240] bytes. One 10240-byte stage holds a
// 128-row x 128-k tile: 8192 bytes of packed nibbles, row r at r*64, its four 16-byte blocks (32 elements each, split-half
// nibble order) stored at chunk position (block ^ ((r >> 1) & 3)), followed by 2048 bytes of fp32 scales [row][4].
// Rows / k beyond N / K are zero (zero scale).
constexpr int kQ4StageBytes = 10240;

struct GemmWeightDesc {
  int N = 0, K = 0;
  bool is_q4 = false;
  const void* data = nullptr;  // bf16 [N, K] or the tile-packed JQ4 bytes
  CUtensorMap map_w;           // dense: [N, K] (3-D chunked form when w3d); JQ4: the packed stages as rows of 1 KB
  bool w3d = false;
};

// Peer-memory state of the fused GEMM + all-reduce epilogue (all pointers are device addresses mapped in this process).
struct GemmTpArgs {
  int size = 1, rank = 0;
  int ncta_max = 0;              // flag matrix row length
  long long slab = 0;            // bf16 elements per (parity, source) receive slab
  unsigned long long recv[8];    // receive area of every rank
  unsigned long long flags[8];   // flag matrix of every rank
  unsigned int* rounds = nullptr;  // local [ncta_max]
  unsigned int* call = nullptr;    // local [2]
  long long wait_limit_cycles = 0; // bound of every peer-flag wait in SM cycles (0: the default of about 2 s)
  // What the row-parallel GEMM epilogue does with its partial tile: 0 = store it into every rank's slab, wait for the peers and
  // reduce (GEMM + all-reduce in one kernel); 1 = store it into every rank's slab, publish and leave (launch_tp_reduce_norm waits,
  // sums the ranks and applies the residual add and the norm that follow the projection); 2 = store it into this rank's own slab,
  // publish and leave (the reduce kernel sums through the NVSwitch multicast address mc_recv with multimem.ld_reduce).
  int mode = 0;
  unsigned long long mc_recv = 0;  // multicast (NVLS) address of the receive area, 0 when not bound
  mutable int last_ctas = 0;       // CTAs of the last fused launch (the reduce kernel waits for that many publications per rank)
};

// Peer-memory state of the GEMM -> reduce-scatter -> all-gather path for prefill-size batches (see gemm_tc_run_scatter).
struct GemmScatterArgs {
  int size = 1, rank = 0;
  long long recv_elems = 0;      // capacity of a receive area in bf16 elements: size * rows_per_rank * N must fit
  long long gather_elems = 0;    // capacity of a gather area: M * N must fit
  unsigned long long recv[8];    // every rank's receive area, bf16 [size sources][rows_per_rank][N] for the launch at hand
  unsigned long long gather[8];  // every rank's gather area, bf16 [M][N]: rows arrive reduced from their owners
  unsigned long long flags[8];   // every rank's u32 [24], cumulative: [src] partial tiles from src, [8 + src] reduced row groups from
                                 // src, [16 + src] row groups src pushed for an all-gather -> GEMM
};
// How a launch of M token rows is cut over the ranks: rank r owns rows [r * rows_per_rank, min(M, (r + 1) * rows_per_rank)).
struct GemmScatterPlan {
  int rows_per_rank;  // a multiple of kScatterGroupRows
  int rows[8];        // rows owned per rank (0 for ranks beyond the end)
  int tiles[8];       // GEMM CTAs that publish to rank r, per source rank
  int groups[8];      // reduce CTAs of rank r (kScatterGroupRows rows each)
};
constexpr int kScatterGroupRows = 8;
GemmScatterPlan gemm_scatter_plan(int M, int N, int size);
bool gemm_scatter_supported(const GemmWeightDesc* w, int M, const GemmScatterArgs* a);

void gemm_weight_init(GemmWeightDesc* w);
int gemm_num_sms();
void gemm_set_pdl(bool on);  // programmatic dependent launch of the GEMM kernels (on by default)
void gemm_tc_run(const GemmWeightDesc* w, const void* x, int M, int ldx, void* out, int ldo, bool out_f32, const float* bias,
                 float* ws, size_t ws_floats, int* counters, int n_counters, int* status, int force_splits, cudaStream_t st,
                 const GemmTpArgs* tp = nullptr);
// Grouped (mixture-of-experts) GEMM over rows sorted by expert; `w` stacks the local experts (JQ4: each expert padded to whole
// 128-row tiles), `items` is the device work list of launch_moe_items built with the same token tile `bn`.
// arguments of the q | k | v epilogue (per-head RMSNorm, rotary embedding, paged KV write); see gemm_tc_run_qkv
struct GemmQkvArgs {
  const int* positions;        // [M]
  const long long* slots;      // [M] flat cache rows, < 0: skip the cache write
  const void* q_norm_w;        // bf16 [128] or nullptr
  const void* k_norm_w;
  const float* cos_t;          // [max_pos, rot_half] or nullptr
  const float* sin_t;
  void* k_cache;               // bf16 [blocks, KV, block_size, 128]
  void* v_cache;
  int heads, kv_heads, block_size, rot_half, max_pos;
  float eps, norm_offset;
};
void gemm_tc_run_qkv(const GemmWeightDesc* w, const void* x, int M, int ldx, void* q_out, int ldo, const float* bias, const GemmQkvArgs* a,
                     float* ws, size_t ws_floats, int* counters, int n_counters, int* status, cudaStream_t st);
void gemm_tc_run_grouped_act(const GemmWeightDesc* w, int n_per_expert, const void* x, int rows, int ldx, void* out, int ldo,
                             const int* items, int max_items, int bn, int splits, int act, int* status, cudaStream_t st);
// gate | up projection with act(gate) * up computed in the epilogue (weights interleaved per tile; see gemm.cu)
void gemm_tc_run_act(const GemmWeightDesc* w, const void* x, int M, int ldx, void* out, int ldo, int act, float* ws, size_t ws_floats,
                     int* counters, int n_counters, int* status, cudaStream_t st);
void gemm_tc_run_grouped(const GemmWeightDesc* w, int n_per_expert, const void* x, int rows, int ldx, void* out, int ldo,
                         const int* items, int max_items, int bn, int splits, int* status, cudaStream_t st);
// CUDA-core variant for decode-size groups (at most `mt` = 4 or 8 rows per work item; items built with bn == mt)
void gemv_grouped_run(const GemmWeightDesc* w, int n_per_expert, const void* x, int ldx, void* out, int ldo, const int* items,
                      int max_items, int mt, cudaStream_t st);
// row_map / row_div (optional): grouped row r reads x row row_map[r] / row_div (x ungathered, row_map the grouping permutation)
bool gemv_grouped_act_run(const GemmWeightDesc* w, int n_per_expert, const void* x, int ldx, void* out, int ldo, const int* items, int max_items,
                          int act, const int* row_map, int row_div, cudaStream_t st);
// Row-parallel projection whose partial tiles go straight to the rank that owns their token rows (epilogue EPI = 3, no waiting
// inside the GEMM). Follow it with launch_scatter_reduce and launch_scatter_finish on the same stream.
void gemm_tc_run_scatter(const GemmWeightDesc* w, const void* x, int M, int ldx, const GemmScatterArgs* a, int* status, cudaStream_t st);
// all-gather -> GEMM: every rank holds the rows it owns (the cut of gemm_scatter_plan) of the activations [M, K]. launch_gather_push
// copies them into every rank's gather area and publishes one count per CTA; gemm_tc_run_gathered multiplies the local gather
// area by `w`, its activation producers wait per token tile for the owners' counts (group_targets[src], cumulative).
bool gemm_gathered_supported(const GemmWeightDesc* w, int M, const GemmScatterArgs* a);
void launch_gather_push(const GemmScatterArgs* a, const GemmScatterPlan* plan, const void* x_own, int M, int K, int* status, cudaStream_t st);
void gemm_tc_run_gathered(const GemmWeightDesc* w, int M, const GemmScatterArgs* a, const unsigned* group_targets, void* out, int ldo,
                          const float* bias, float* ws, size_t ws_floats, int* counters, int n_counters, int* status, cudaStream_t st);
// true when the fused all-reduce epilogue can take this problem (one wave of CTAs, rows and columns inside the slab)
bool gemm_tp_supported(const GemmWeightDesc* w, int M, const GemmTpArgs* tp);
void gemv_simt_run(const GemmWeightDesc* w, const void* x, int M, int ldx, void* out, int ldo, bool out_f32, const float* bias,
                   cudaStream_t st);

// elementwise.cu
void launch_rmsnorm(const void* x, void* residual, const void* w, void* y, int T, int H, float eps, float offset, float res_mult,
                    cudaStream_t st);
void launch_layernorm(const void* x, const void* w, const void* b, void* y, int T, int H, float eps, cudaStream_t st);
void launch_act_mul(const void* in, void* out, long long T, int I, int act, cudaStream_t st);
void launch_act(const void* in, void* out, long long n, int act, cudaStream_t st);
void launch_embedding(const void* table, const int* ids, const void* pos_table, const int* pos, const void* type_table,
                      const int* types, void* out, int T, int H, int vocab, float scale, cudaStream_t st);
int launch_rope_kv(void* qkv, const int* positions, const long long* slots, const void* qn, const void* kn, const float* cos_t,
                   const float* sin_t, void* k_cache, void* v_cache, int T, int H, int KV, int D, int block_size, int rot_half,
                   float eps, float norm_offset, int max_pos, cudaStream_t st);

// attention.cu
int launch_decode_attention(const void* q, long long q_stride, const void* kc, const void* vc, const int* bt, int bt_stride,
                            const int* ctx, void* out, float* po, float* pml, int B, int H, int KV, int D, int page, float scale,
                            float cap, int window, int splits, cudaStream_t st);
int launch_decode_attention_impl(const void* q, long long q_stride, const void* kc, const void* vc, const int* bt, int bt_stride,
                                 const int* ctx, void* out, float* po, float* pml, int* arrivals, int B, int H, int KV, int D, int page,
                                 float scale, float cap, int window, int splits, int impl, cudaStream_t st);
int launch_prefill_attention(const void* q, long long q_stride, const void* kc, const void* vc, const int* bt, int bt_stride,
                             const int* q_start, const int* q_len, const int* ctx, const int* tile_seq, const int* tile_q0,
                             int num_tiles, void* out, int H, int KV, int D, int page, float scale, float cap, int window,
                             int causal, cudaStream_t st);

// attention_tc.cu: tcgen05 / TMA prefill attention; tile arrays hold prefill_attention_tc_tile_rows(D) query rows per tile
int prefill_attention_tc_tile_rows(int D);
extern bool g_gemm_persist;    // gemm_persist.cu: prefill-size JQ4 projections on the persistent kernel (off by default)
extern bool g_gemm_persist_ordered;  // its issuers take turns in k-block order (bit-reproducible; default) or race
bool gemm_persist_supported(const GemmWeightDesc* w, int M, int ldx);
bool gemm_persist_preferred(const GemmWeightDesc* w, int M);
void gemm_persist_run(const GemmWeightDesc* w, const void* x, int M, int ldx, void* out, int ldo, bool out_f32, const float* bias, int* status,
                      cudaStream_t st);
extern bool g_gemm_persist_all;
extern int g_gemm_force_bn;    // gemm.cu: token tile for prefill-size batches (tests, comparisons)
extern int g_gemv_max_rows;     // gemm.cu: most token rows the small-batch GEMV takes (default 8; up to 16)
extern int g_gemv_force_split;  // gemm.cu: warps per CTA of the small-batch GEMV (0: chosen per shape)
extern bool g_gemv_dense;      // gemm.cu: <= 8-row JQ4 projections on the mma.sync GEMV (default on)
bool gemv_dense_supported(const GemmWeightDesc* w, int M, int ldx);
void gemv_dense_run(const GemmWeightDesc* w, const void* x, int M, int ldx, void* out, int ldo, bool out_f32, const float* bias, int act,
                    cudaStream_t st);
extern bool g_gemv_simt_only;  // gemm.cu: grouped JQ4 GEMV on CUDA cores instead of mma.sync (comparisons)
int launch_prefill_attention_tc(const void* q, long long q_stride, long long T, const void* kc, const void* vc, long long num_pages, const int* bt,
                                int bt_stride, const int* q_start, const int* q_len, const int* ctx, const int* tile_seq, const int* tile_q0,
                                int num_tiles, void* out, int H, int KV, int D, int page, float scale, float cap, int window, int causal, int* status,
                                cudaStream_t st);

// sampling.cu
void launch_argmax(const float* logits, int ld, int B, int V, const uint32_t* mask, int mask_ld, float softcap, float inv_scale,
                   long long* out_idx, float* out_val, cudaStream_t st);
void launch_logits_post(float* logits, int ld, int B, int V, const uint32_t* mask, int mask_ld, float softcap, float inv_scale,
                        cudaStream_t st);

void launch_sample(const float* logits, int ld, int B, int V, const float* inv_temp, const long long* limits, const float* top_p,
                   const unsigned char* uniform, const float* us, long long* out_tok, int* out_ok, cudaStream_t st);

// exclude-top-choice pick per row (-1: XTC does not apply) and log-probabilities (chosen token + top_n) per row; see sampling.cu
void launch_xtc(const float* logits, int ld, int B, int V, const float* inv_temp, const float* threshold, const unsigned char* fire,
                const int* special, int n_special, long long* out_tok, cudaStream_t st);
void launch_logprobs(const float* logits, int ld, int B, int V, const long long* chosen, int top_n, float* out_chosen, long long* out_idx,
                     float* out_val, cudaStream_t st);

// moe.cu
size_t moe_route_workspace_ints(int T, int E, int k);  // ints of `ws` for the parallel grouping of large batches (0: not needed)
void launch_moe_route(const float* logits, int T, int E, int k, int mode, int renorm, float* w, int* idx, int* counts, int* offsets,
                      int* perm, int* pos, int* ws, cudaStream_t st);
// `range` (optional) = offsets + first local expert and the count of local experts: rows outside
// [offsets[e0], offsets[e0 + ne]) are skipped (expert parallelism: other ranks own them)
void launch_moe_gather(const void* x, const int* perm, int rows, int k, int H, void* xs, const int* offsets, int e0, int ne,
                       cudaStream_t st);
void launch_moe_combine(const void* ys, const int* pos, const float* w, int T, int k, int H, void* out, const int* offsets, int e0,
                        int ne, cudaStream_t st);
void launch_moe_items(const int* offsets, int e0, int ne, int bn, int max_items, int* items, cudaStream_t st);
bool launch_moe_route_small(const float* logits, int T, int E, int k, int mode, int renorm, float* w, int* idx, int* counts, int* offsets,
                            int* perm, int* pos, int e0, int ne, int bn, int max_items, int* items, cudaStream_t st);

// comm.cu: fused compute + collective kernels over peer memory (same protocol as the GEMM all-reduce epilogue)
bool comm_rows_supported(const GemmTpArgs* tp, int rows, int H);
void launch_moe_combine_allreduce(const void* ys, const int* pos, const float* w, int T, int k, int H, const int* offsets, int e0, int ne,
                                  void* out, const GemmTpArgs* tp, int* status, cudaStream_t st);
void launch_oneshot_allreduce(const void* x, int rows, int H, void* out, const GemmTpArgs* tp, int* status, cudaStream_t st);
// Second half of a row-parallel projection launched with GemmTpArgs::mode 1 or 2 (see comm.cu): wait for the ranks, sum them, then
// kind 0: out = sum; kind 1: residual += [RMSNorm(post_w)](sum) * res_mult, out = RMSNorm(residual, norm_w). N % 8 == 0, N <= 12288.
void launch_tp_reduce_norm(const GemmTpArgs* tp, int M, int N, int kind, const float* bias, void* residual, const void* post_w, const void* norm_w,
                           void* out, float eps, float offset, float res_mult, int* status, cudaStream_t st);

// Sum the size partial slabs of this rank's rows (+ bias). push: write them to out [M, N] and to every peer's gather area and
// publish (all-reduce, follow with launch_scatter_finish); !push: write them to out [own rows, N] only (reduce-scatter).
// gemm_target: cumulative number of partial tiles every source must have published to this rank.
void launch_scatter_reduce(const GemmScatterArgs* a, const GemmScatterPlan* plan, int M, int N, const float* bias, void* out,
                           unsigned gemm_target, bool push, int* status, cudaStream_t st);
// Wait for the other ranks' reduced rows and copy them from the gather area into out. group_targets[src]: cumulative row groups.
void launch_scatter_finish(const GemmScatterArgs* a, const GemmScatterPlan* plan, int M, int N, void* out, const unsigned* group_targets,
                           int* status, cudaStream_t st);

// mamba.cu
int launch_mamba2(const void* zx, int ld, int T, int num_seqs, int I, int conv_dim, int K, int H, int d_head, int G, int S,
                  const float* conv_w, const float* conv_b, const float* dt_bias, const float* A_log, const float* D, const float* norm_w,
                  float eps, float* conv_state, float* ssm_state, const long long* slots, const int* row_seq, const int* q_start,
                  const int* q_len, const int* positions, int n_chunks, const int* chunk_seq, const int* chunk_row0, const int* chunk_len,
                  const int* chunk_first, const int* chunk_last, const int* seq_chunk0, const int* seq_nchunks, int multi_chunk,
                  float* xbc, float* ybuf, float* chunk_state, float* chunk_decay, void* out, cudaStream_t st);

// a2a.cu: expert-parallel all-to-all over peer memory (see the file comment for the protocol)
struct A2AParams {
  int size, rank;
  int ne;                        // experts per rank (<= 128)
  int cap;                       // rows of a receive region = most (token, slot) pairs one rank can send (its rows * k)
  unsigned long long recv[8];    // every rank's receive area: bf16 [size regions][cap][H]
  unsigned long long meta[8];    // every rank's int32 [size][2 * ne]: rows per expert and first grouped row at the sender
  unsigned long long flags[8];   // every rank's uint32 [16]: dispatch epochs [0..8), return epochs [8..16)
  unsigned long long ret[8];     // every rank's return buffer: bf16 [cap][H]
  int* status;
};
void launch_a2a_dispatch(const A2AParams* p, const void* x, const int* perm, const int* offsets, int rows, int k, int H, unsigned epoch, cudaStream_t st);
void launch_a2a_receive(const A2AParams* p, unsigned epoch, int* local_offsets, int* seg, void* xs, int max_rows, int H, cudaStream_t st);
void launch_a2a_return(const A2AParams* p, const int* local_offsets, const int* seg, const void* ys, int max_rows, int H, unsigned epoch, cudaStream_t st);
void launch_a2a_wait(const A2AParams* p, unsigned epoch, cudaStream_t st);

// aux.cu
void launch_lora_delta(const void* x, int ldx, const void* A, const void* Bs, void* y, int ldy, int M, int K, int N, int r, cudaStream_t st);
void launch_pool(const void* h, int H, const int* start, const int* len, int S, int mode, int normalize, float* out, cudaStream_t st);
void launch_softmax_rows(const float* x, float* y, int rows, int C, cudaStream_t st);
void launch_tq_encode(const void* x, int src_dtype, long long rows, int dim, int pdim, int bits, const float* signs, const float* edges, uint8_t* codes,
                      float* norms, cudaStream_t st);
void launch_tq_decode(const uint8_t* codes, const float* norms, long long rows, int dim, int pdim, int bits, const float* signs, const float* centroids,
                      void* out, int dst_dtype, cudaStream_t st);
// lz4_block.cpp (host)
size_t lz4_compress_bound(size_t n);
size_t lz4_compress(const uint8_t* src, size_t n, uint8_t* dst, size_t cap);
size_t lz4_decompress(const uint8_t* src, size_t n, uint8_t* dst, size_t n_out);

// quant.cu
void launch_q4_quantize(const void* w, int src_dtype, long long n_blocks, uint8_t* packed, float* scales, cudaStream_t st);
void launch_q4_dequantize(const uint8_t* packed, const float* scales, long long n_blocks, void* out, int dst_dtype, cudaStream_t st);

}  // namespace dlv
