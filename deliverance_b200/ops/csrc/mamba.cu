// Mamba2 mixer core for granitemoehybrid (fp32 state, bf16 activations).
//   zxbcdt [T, I + convDim + H] = [gate (I) | x (I) | B (G*S) | C (G*S) | dt (H)]  ->  y [T, I]
// Steps: causal depthwise conv1d over x|B|C with a rolling per-sequence state + SiLU; dt = softplus(dt + dt_bias);
// state = state * exp(dt * A) + B * (dt * x); y = C . state + D * x; y *= silu(gate); RMSNorm over the whole intermediate.
// The scan is chunked: every chunk of 128 tokens first computes its local end state from zero and its cumulative decay
// (all chunks of all sequences in parallel), a carry pass folds the chunk states left to right, and the output pass
// re-runs each chunk from its true initial state. Decode and short chunks skip the first two passes.
// Reference (token-by-token): core/.../model/granitemoehybrid/GraniteMoeHybridMambaLayer.java:130-252.
#include "common.cuh"

namespace dlv {

constexpr int kMambaChunk = 128;

__device__ __forceinline__ float silu_f(float v) { return v / (1.f + __expf(-v)); }
__device__ __forceinline__ float softplus_f(float v) { return v > 20.f ? v : log1pf(__expf(v)); }

// conv: one thread per (row, channel). xbc_out [T, convDim] fp32 (activated).
__global__ void __launch_bounds__(256) mamba_conv_kernel(const __nv_bfloat16* __restrict__ zx, int ld, int I, int conv_dim, int K,
                                                         const float* __restrict__ conv_w, const float* __restrict__ conv_b,
                                                         const float* __restrict__ conv_state, const long long* __restrict__ slots,
                                                         const int* __restrict__ row_seq, const int* __restrict__ q_start,
                                                         const int* __restrict__ positions, float* __restrict__ out, int T) {
  pdl_wait();     // no-op unless launched with programmatic stream serialization: the kernel in front has completed
  pdl_trigger();  // the next kernel may start its prologue (and a GEMM its weight prefetch) under this kernel's tail
  const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= static_cast<long long>(T) * conv_dim) return;
  const int row = static_cast<int>(idx / conv_dim), c = static_cast<int>(idx % conv_dim);
  const int s = row_seq[row];
  const int j = row - q_start[s];
  const bool fresh = positions[q_start[s]] == 0;  // a sequence that starts at position 0 starts from a zero state
  const float* st = conv_state + (static_cast<size_t>(slots[s]) * conv_dim + c) * (K - 1);
  float acc = conv_b ? conv_b[c] : 0.f;
  for (int i = 0; i < K; ++i) {  // weight index K-1-i multiplies the input i steps back
    const int jj = j - i;
    float v;
    if (jj >= 0) v = bf2f(zx[static_cast<size_t>(row - i) * ld + I + c]);
    else v = fresh ? 0.f : st[(K - 1) + jj];
    acc += conv_w[c * K + (K - 1 - i)] * v;
  }
  out[static_cast<size_t>(row) * conv_dim + c] = silu_f(acc);
}

// rolling state update: one thread per (sequence, channel)
__global__ void __launch_bounds__(256) mamba_conv_state_kernel(const __nv_bfloat16* __restrict__ zx, int ld, int I, int conv_dim, int K,
                                                               float* __restrict__ conv_state, const long long* __restrict__ slots,
                                                               const int* __restrict__ q_start, const int* __restrict__ q_len,
                                                               const int* __restrict__ positions, int S) {
  pdl_wait();     // no-op unless launched with programmatic stream serialization: the kernel in front has completed
  pdl_trigger();  // the next kernel may start its prologue (and a GEMM its weight prefetch) under this kernel's tail
  const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= static_cast<long long>(S) * conv_dim) return;
  const int s = static_cast<int>(idx / conv_dim), c = static_cast<int>(idx % conv_dim);
  const int n = q_len[s];
  if (n == 0) return;
  const bool fresh = positions[q_start[s]] == 0;
  float* st = conv_state + (static_cast<size_t>(slots[s]) * conv_dim + c) * (K - 1);
  float old[8];
  for (int m = 0; m < K - 1; ++m) old[m] = fresh ? 0.f : st[m];
  for (int m = 0; m < K - 1; ++m) {
    const int jj = n - (K - 1) + m;  // local index of the input that lands in slot m
    st[m] = jj >= 0 ? bf2f(zx[static_cast<size_t>(q_start[s] + jj) * ld + I + c]) : old[(K - 1) + jj];
  }
}

// Scan passes. grid = (chunks_total, H); block = d_head * PARTS threads; thread (d, part) owns SPT = S / PARTS states.
// mode 0: local end state of the chunk from zero -> chunk_state, cumulative decay -> chunk_decay (no output)
// mode 1: output pass, every sequence is a single chunk: initial state = sequence state (or zero at position 0)
// mode 2: output pass after the carry pass: the initial state of every chunk is in chunk_state
template <int SPT>
__global__ void mamba_scan_kernel(const __nv_bfloat16* __restrict__ zx, int ld, int I, int conv_dim, const float* __restrict__ xbc,
                                  const float* __restrict__ dt_bias, const float* __restrict__ A_log, const float* __restrict__ Dp,
                                  float* __restrict__ ssm_state, const long long* __restrict__ slots, const int* __restrict__ chunk_seq,
                                  const int* __restrict__ chunk_row0, const int* __restrict__ chunk_len, const int* __restrict__ chunk_first,
                                  const int* __restrict__ chunk_last, const int* __restrict__ positions, float* __restrict__ chunk_state,
                                  float* __restrict__ chunk_decay, float* __restrict__ y, int H, int d_head, int G, int S, int parts, int mode) {
  pdl_wait();     // no-op unless launched with programmatic stream serialization: the kernel in front has completed
  pdl_trigger();  // the next kernel may start its prologue (and a GEMM its weight prefetch) under this kernel's tail
  extern __shared__ float sh[];  // B [S] | C [S]
  float* sB = sh;
  float* sC = sh + S;
  const int ck = blockIdx.x, h = blockIdx.y;
  const int d = threadIdx.x / parts, part = threadIdx.x % parts;
  const int seq = chunk_seq[ck], row0 = chunk_row0[ck], len = chunk_len[ck];
  const int g = h / (H / G);
  const int GS = G * S;
  const float A = -__expf(A_log[h]);
  const float Dh = Dp[h];
  const float dtb = dt_bias[h];
  float st[SPT];
  const size_t state_off = ((static_cast<size_t>(slots[seq]) * H + h) * d_head + d) * S + part * SPT;
  const size_t cstate_off = ((static_cast<size_t>(ck) * H + h) * d_head + d) * S + part * SPT;
  if (mode == 0) {
#pragma unroll
    for (int i = 0; i < SPT; ++i) st[i] = 0.f;
  } else if (mode == 1 && chunk_first[ck]) {
    const bool fresh = positions[row0] == 0;
#pragma unroll
    for (int i = 0; i < SPT; ++i) st[i] = fresh ? 0.f : ssm_state[state_off + i];
  } else {
#pragma unroll
    for (int i = 0; i < SPT; ++i) st[i] = chunk_state[cstate_off + i];
  }
  float cum = 1.f;
  for (int j = 0; j < len; ++j) {
    const int row = row0 + j;
    __syncthreads();
    for (int i = threadIdx.x; i < 2 * S; i += blockDim.x) {
      const int which = i / S, sidx = i % S;
      sh[i] = xbc[static_cast<size_t>(row) * conv_dim + I + which * GS + g * S + sidx];
    }
    __syncthreads();
    const float dt = softplus_f(bf2f(zx[static_cast<size_t>(row) * ld + I + conv_dim + h]) + dtb);
    const float decay = __expf(dt * A);
    const float xv = xbc[static_cast<size_t>(row) * conv_dim + h * d_head + d];
    const float dx = dt * xv;
    float acc = 0.f;
#pragma unroll
    for (int i = 0; i < SPT; ++i) {
      st[i] = st[i] * decay + sB[part * SPT + i] * dx;
      acc += st[i] * sC[part * SPT + i];
    }
    cum *= decay;
    if (mode >= 1) {
      for (int o = 1; o < parts; o <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
      if (part == 0) {
        const float gate = bf2f(zx[static_cast<size_t>(row) * ld + h * d_head + d]);
        y[static_cast<size_t>(row) * I + h * d_head + d] = (acc + Dh * xv) * silu_f(gate);
      }
    }
  }
  if (mode == 0) {
#pragma unroll
    for (int i = 0; i < SPT; ++i) chunk_state[cstate_off + i] = st[i];
    if (threadIdx.x == 0) chunk_decay[static_cast<size_t>(ck) * H + h] = cum;
  } else if (chunk_last[ck]) {
#pragma unroll
    for (int i = 0; i < SPT; ++i) ssm_state[state_off + i] = st[i];
  }
}

// carry: for each sequence walk its chunks left to right: init(c) = init(c-1) * decay(c-1) + local(c-1).
// On entry chunk_state[c] = local end state of chunk c; on exit chunk_state[c] = initial state of chunk c.
__global__ void __launch_bounds__(256) mamba_carry_kernel(float* __restrict__ chunk_state, const float* __restrict__ chunk_decay,
                                                          const float* __restrict__ ssm_state, const long long* __restrict__ slots,
                                                          const int* __restrict__ seq_chunk0, const int* __restrict__ seq_nchunks,
                                                          const int* __restrict__ q_start, const int* __restrict__ positions, int H,
                                                          int per_head) {
  pdl_wait();     // no-op unless launched with programmatic stream serialization: the kernel in front has completed
  pdl_trigger();  // the next kernel may start its prologue (and a GEMM its weight prefetch) under this kernel's tail
  const int seq = blockIdx.x, h = blockIdx.y;
  const int c0 = seq_chunk0[seq], nc = seq_nchunks[seq];
  const bool fresh = positions[q_start[seq]] == 0;
  for (int e = threadIdx.x; e < per_head; e += blockDim.x) {
    float carry = fresh ? 0.f : ssm_state[(static_cast<size_t>(slots[seq]) * H + h) * per_head + e];
    for (int c = 0; c < nc; ++c) {
      const size_t off = (static_cast<size_t>(c0 + c) * H + h) * per_head + e;
      const float local = chunk_state[off];
      chunk_state[off] = carry;  // initial state of chunk c (chunk 0: the sequence state, so that the output pass never reads
                                 // ssm_state while the last chunk of the same sequence overwrites it)
      carry = carry * chunk_decay[static_cast<size_t>(c0 + c) * H + h] + local;
    }
  }
}

// gated RMSNorm over the whole intermediate: one CTA per row, y fp32 -> out bf16
__global__ void __launch_bounds__(256) mamba_norm_kernel(const float* __restrict__ y, const float* __restrict__ w, __nv_bfloat16* __restrict__ out,
                                                         int I, float eps) {
  pdl_wait();     // no-op unless launched with programmatic stream serialization: the kernel in front has completed
  pdl_trigger();  // the next kernel may start its prologue (and a GEMM its weight prefetch) under this kernel's tail
  __shared__ float red[32];
  const size_t base = static_cast<size_t>(blockIdx.x) * I;
  float ss = 0.f;
  for (int i = threadIdx.x; i < I; i += blockDim.x) ss += y[base + i] * y[base + i];
  ss = block_sum(ss, red);
  const float inv = rsqrtf(ss / I + eps);
  for (int i = threadIdx.x; i < I; i += blockDim.x) out[base + i] = f2bf(y[base + i] * inv * w[i]);
}

int launch_mamba2(const void* zx, int ld, int T, int num_seqs, int I, int conv_dim, int K, int H, int d_head, int G, int S,
                  const float* conv_w, const float* conv_b, const float* dt_bias, const float* A_log, const float* D, const float* norm_w,
                  float eps, float* conv_state, float* ssm_state, const long long* slots, const int* row_seq, const int* q_start,
                  const int* q_len, const int* positions, int n_chunks, const int* chunk_seq, const int* chunk_row0, const int* chunk_len,
                  const int* chunk_first, const int* chunk_last, const int* seq_chunk0, const int* seq_nchunks, int multi_chunk,
                  float* xbc, float* ybuf, float* chunk_state, float* chunk_decay, void* out, cudaStream_t st) {
  if (T == 0) return 0;
  if (K > 9 || K < 2) return 1;
  int spt = S >= 32 ? 32 : S;
  if (S % spt != 0) return 2;
  const int parts = S / spt;
  if (parts > 32 || (parts & (parts - 1)) != 0 || d_head * parts > 1024) return 3;
  const auto* zxp = static_cast<const __nv_bfloat16*>(zx);
  const long long nconv = static_cast<long long>(T) * conv_dim;
  mamba_conv_kernel<<<static_cast<unsigned>((nconv + 255) / 256), 256, 0, st>>>(zxp, ld, I, conv_dim, K, conv_w, conv_b, conv_state, slots,
                                                                                 row_seq, q_start, positions, xbc, T);
  dim3 grid(n_chunks, H);
  const int threads = d_head * parts;
  const size_t smem = 2 * S * sizeof(float);
#define DLV_SCAN(SPT, MODE)                                                                                                             \
  mamba_scan_kernel<SPT><<<grid, threads, smem, st>>>(zxp, ld, I, conv_dim, xbc, dt_bias, A_log, D, ssm_state, slots, chunk_seq, chunk_row0, \
                                                      chunk_len, chunk_first, chunk_last, positions, chunk_state, chunk_decay, ybuf, H,  \
                                                      d_head, G, S, parts, MODE)
  if (multi_chunk) {
    if (spt == 32) DLV_SCAN(32, 0); else if (spt == 16) DLV_SCAN(16, 0); else if (spt == 8) DLV_SCAN(8, 0); else return 2;
    dim3 g2(num_seqs, H);
    mamba_carry_kernel<<<g2, 256, 0, st>>>(chunk_state, chunk_decay, ssm_state, slots, seq_chunk0, seq_nchunks, q_start, positions, H,
                                           d_head * S);
  }
  const int out_mode = multi_chunk ? 2 : 1;
  if (spt == 32) DLV_SCAN(32, out_mode); else if (spt == 16) DLV_SCAN(16, out_mode); else if (spt == 8) DLV_SCAN(8, out_mode); else return 2;
#undef DLV_SCAN
  const long long nst = static_cast<long long>(num_seqs) * conv_dim;
  mamba_conv_state_kernel<<<static_cast<unsigned>((nst + 255) / 256), 256, 0, st>>>(zxp, ld, I, conv_dim, K, conv_state, slots, q_start, q_len,
                                                                                     positions, num_seqs);
  mamba_norm_kernel<<<T, 256, 0, st>>>(ybuf, norm_w, static_cast<__nv_bfloat16*>(out), I, eps);
  return 0;
}

}  // namespace dlv
