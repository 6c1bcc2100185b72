// Fused compute + collective kernels over NVLink peer memory that are not GEMM epilogues.
//
//   moe_combine_allreduce: expert parallelism with replicated tokens. Every rank holds the outputs of ITS experts for the
//     (token, slot) pairs routed to them. One CTA per token forms the weighted sum over the local slots (fp32), stores it as
//     bf16 into the receive slab of EVERY rank with plain peer stores, publishes it with one release-add per rank, waits
//     (bounded) until all ranks have published the same token to it, and adds the partial sums in rank order: the top-k
//     combine and the all-reduce over the expert-parallel group are one kernel, no intermediate [T, H] tensor and no NCCL call.
//   oneshot_allreduce: the same exchange for an existing bf16 tensor (small decode-size tensors that no GEMM produces).
//
// Protocol (shared with the GEMM all-reduce epilogue in gemm_tc.cuh, so launches of both kinds can interleave): receive slabs
// are double-buffered on the parity of a per-rank launch counter; flags are cumulative per (source rank, CTA index) and the
// expected value is kept per CTA index, so CUDA-graph replays need no reset; the last CTA of a grid advances the launch
// counter. Every rank must launch the same sequence of fused kernels with the same grids. All CTAs of a launch are resident at
// once (grid <= 148, small CTAs), otherwise waiting CTAs could keep a peer's publishers from being scheduled.
// Plain peer loads / stores only: no multimem, no TMA.
//
// The reference keeps every expert on one host and combines their outputs locally, token by token (scale + accumulate,
// core/.../model/MixtureOfExpertsBlock.java:78-112; Qwen3MoeFeedForward.java:175-183 scatterAdd); it has no expert parallelism.
#include "common.cuh"
#include "gemm_api.h"

namespace dlv {

struct CommParams {
  int size, rank, ncta_max;
  long long slab;
  unsigned long long recv[8];
  unsigned long long flags[8];
  unsigned int* rounds;
  unsigned int* call;
  int* status;
  long long wait_limit;  // SM cycles a peer-flag wait may take before the kernel gives up and sets the status word
};

// Publish this CTA's region to every rank and wait until every rank has published the same region to this rank.
// Call with all threads of the CTA; returns a CTA-uniform flag (false: a wait ran out, the status word is set).
__device__ __forceinline__ bool exchange_barrier(const CommParams& p, unsigned cta_id, int* s_flag) {
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x < 32) {
    // one lane per peer: release-adds and flag waits of all peers proceed side by side
    const int lane = threadIdx.x;
    const unsigned round = p.rounds[cta_id];
    bool ok_lane = true;
    if (lane < p.size) {
      const int dst = (p.rank + lane) % p.size;
      red_release_sys_add(reinterpret_cast<uint32_t*>(p.flags[dst]) + static_cast<size_t>(p.rank) * p.ncta_max + cta_id, 1u);
      const uint32_t* mine = reinterpret_cast<const uint32_t*>(p.flags[p.rank]);
      ok_lane = flag_wait_ge(mine + static_cast<size_t>(lane) * p.ncta_max + cta_id, round + 1u, p.status, p.wait_limit);
    }
    const bool all = __all_sync(0xffffffffu, ok_lane);
    if (lane == 0) {
      p.rounds[cta_id] = round + 1u;
      *s_flag = all ? 1 : 0;
    }
  }
  __syncthreads();
  return *s_flag != 0;
}

__device__ __forceinline__ void finish_launch(const CommParams& p, unsigned call) {
  __syncthreads();
  if (threadIdx.x == 0) {
    if (atomicAdd(p.call + 1, 1u) == gridDim.x - 1u) {
      p.call[1] = 0u;
      __threadfence();
      p.call[0] = call + 1u;
    }
  }
}

// grid = T tokens (<= ncta_max, all resident), 128 threads. ys: expert outputs in expert-grouped row order [T * k, H].
__global__ void __launch_bounds__(128) moe_combine_allreduce_kernel(const __nv_bfloat16* __restrict__ ys, const int* __restrict__ pos,
                                                                    const float* __restrict__ w, int k, int H,
                                                                    const int* __restrict__ offsets, int e0, int ne,
                                                                    __nv_bfloat16* __restrict__ out, const CommParams p) {
  pdl_wait();     // no-op unless launched with programmatic stream serialization: the kernel in front has completed
  pdl_trigger();  // the next kernel may start its prologue (and a GEMM its weight prefetch) under this kernel's tail
  __shared__ int s_flag;
  const int t = blockIdx.x;
  const unsigned cta_id = blockIdx.x;
  const unsigned call = *reinterpret_cast<volatile unsigned*>(p.call);
  const long long par_off = static_cast<long long>(call & 1u) * p.size * p.slab;
  const int lo = offsets[e0], hi = offsets[e0 + ne];
  // phase A: weighted sum over the slots whose expert lives here -> every rank's slab [parity][my rank][t, :]
  for (int i = threadIdx.x; i < H / 8; i += blockDim.x) {
    float acc[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = 0.f;
    for (int j = 0; j < k; ++j) {
      const int prow = pos[static_cast<size_t>(t) * k + j];
      if (prow < lo || prow >= hi) continue;
      const float wt = w[static_cast<size_t>(t) * k + j];
      const uint4 v = reinterpret_cast<const uint4*>(ys + static_cast<size_t>(prow) * H)[i];
      const uint32_t* vu = reinterpret_cast<const uint32_t*>(&v);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = unpack_bf162(vu[e]);
        acc[2 * e] += wt * f.x;
        acc[2 * e + 1] += wt * f.y;
      }
    }
    uint4 o;
    uint32_t* ou = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
    for (int e = 0; e < 4; ++e) ou[e] = pack_bf162(acc[2 * e], acc[2 * e + 1]);
    const long long off = par_off + static_cast<long long>(p.rank) * p.slab + static_cast<long long>(t) * H + i * 8;
    for (int r = 0; r < p.size; ++r)
      *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.recv[(p.rank + r) % p.size]) + off) = o;
  }
  const bool ok = exchange_barrier(p, cta_id, &s_flag);
  // phase B: add the partial sums of all ranks in rank order (identical result on every rank)
  if (ok) {
    const __nv_bfloat16* rbase = reinterpret_cast<const __nv_bfloat16*>(p.recv[p.rank]) + par_off + static_cast<long long>(t) * H;
    for (int i = threadIdx.x; i < H / 8; i += blockDim.x) {
      float acc[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] = 0.f;
      for (int src = 0; src < p.size; ++src) {
        const uint4 v = __ldcg(reinterpret_cast<const uint4*>(rbase + static_cast<long long>(src) * p.slab) + i);
        const uint32_t* vu = reinterpret_cast<const uint32_t*>(&v);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = unpack_bf162(vu[e]);
          acc[2 * e] += f.x;
          acc[2 * e + 1] += f.y;
        }
      }
      uint4 o;
      uint32_t* ou = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
      for (int e = 0; e < 4; ++e) ou[e] = pack_bf162(acc[2 * e], acc[2 * e + 1]);
      reinterpret_cast<uint4*>(out + static_cast<size_t>(t) * H)[i] = o;
    }
  }
  finish_launch(p, call);
}

// grid = rows (<= ncta_max, all resident), 128 threads: x [rows, H] bf16 -> out = sum over ranks
__global__ void __launch_bounds__(128) oneshot_allreduce_kernel(const __nv_bfloat16* __restrict__ x, int H, __nv_bfloat16* __restrict__ out,
                                                                const CommParams p) {
  pdl_wait();     // no-op unless launched with programmatic stream serialization: the kernel in front has completed
  pdl_trigger();  // the next kernel may start its prologue (and a GEMM its weight prefetch) under this kernel's tail
  __shared__ int s_flag;
  const int t = blockIdx.x;
  const unsigned call = *reinterpret_cast<volatile unsigned*>(p.call);
  const long long par_off = static_cast<long long>(call & 1u) * p.size * p.slab;
  const long long off = par_off + static_cast<long long>(p.rank) * p.slab + static_cast<long long>(t) * H;
  for (int i = threadIdx.x; i < H / 8; i += blockDim.x) {
    const uint4 v = reinterpret_cast<const uint4*>(x + static_cast<size_t>(t) * H)[i];
    for (int r = 0; r < p.size; ++r)
      reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.recv[(p.rank + r) % p.size]) + off)[i] = v;
  }
  const bool ok = exchange_barrier(p, blockIdx.x, &s_flag);
  if (ok) {
    const __nv_bfloat16* rbase = reinterpret_cast<const __nv_bfloat16*>(p.recv[p.rank]) + par_off + static_cast<long long>(t) * H;
    for (int i = threadIdx.x; i < H / 8; i += blockDim.x) {
      float acc[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] = 0.f;
      for (int src = 0; src < p.size; ++src) {
        const uint4 v = __ldcg(reinterpret_cast<const uint4*>(rbase + static_cast<long long>(src) * p.slab) + i);
        const uint32_t* vu = reinterpret_cast<const uint32_t*>(&v);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = unpack_bf162(vu[e]);
          acc[2 * e] += f.x;
          acc[2 * e + 1] += f.y;
        }
      }
      uint4 o;
      uint32_t* ou = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
      for (int e = 0; e < 4; ++e) ou[e] = pack_bf162(acc[2 * e], acc[2 * e + 1]);
      reinterpret_cast<uint4*>(out + static_cast<size_t>(t) * H)[i] = o;
    }
  }
  finish_launch(p, call);
}

static CommParams make_params(const GemmTpArgs* tp, int* status) {
  CommParams p = {};
  p.size = tp->size;
  p.rank = tp->rank;
  p.ncta_max = tp->ncta_max;
  p.slab = tp->slab;
  for (int r = 0; r < 8; ++r) {
    p.recv[r] = tp->recv[r];
    p.flags[r] = tp->flags[r];
  }
  p.rounds = tp->rounds;
  p.call = tp->call;
  p.status = status;
  p.wait_limit = tp->wait_limit_cycles > 0 ? tp->wait_limit_cycles : kWaitLimitCycles;
  return p;
}

bool comm_rows_supported(const GemmTpArgs* tp, int rows, int H) {
  return tp != nullptr && tp->size > 1 && tp->size <= 8 && rows > 0 && rows <= 128 && rows <= tp->ncta_max && H % 8 == 0 &&
         static_cast<long long>(rows) * H <= tp->slab;
}

void launch_moe_combine_allreduce(const void* ys, const int* pos, const float* w, int T, int k, int H, const int* offsets, int e0, int ne,
                                  void* out, const GemmTpArgs* tp, int* status, cudaStream_t st) {
  if (T == 0) return;
  moe_combine_allreduce_kernel<<<T, 128, 0, st>>>(static_cast<const __nv_bfloat16*>(ys), pos, w, k, H, offsets, e0, ne,
                                                  static_cast<__nv_bfloat16*>(out), make_params(tp, status));
}

void launch_oneshot_allreduce(const void* x, int rows, int H, void* out, const GemmTpArgs* tp, int* status, cudaStream_t st) {
  if (rows == 0) return;
  oneshot_allreduce_kernel<<<rows, 128, 0, st>>>(static_cast<const __nv_bfloat16*>(x), H, static_cast<__nv_bfloat16*>(out),
                                                 make_params(tp, status));
}

// ------------------------------------------------------------------------------------------------ tensor-parallel sum + residual + norm
// Second half of a row-parallel projection whose GEMM epilogue only published its partial tiles (GemmTpArgs::mode 1 or 2) and left:
// one CTA per token row waits (bounded) until every rank's GEMM CTAs have published, sums the ranks' partial rows in rank order
// (mode 1: from this rank's receive slabs; mode 2: one multimem.ld_reduce per 16 bytes through the NVSwitch multicast address, the
// switch adds the eight ranks' values on the way), adds the bias, and then does what follows the projection in the layer:
//   kind 0: out = sum                                  (a plain all-reduce)
//   kind 1: [sum = RMSNorm(sum, post_w)] ; residual += sum * res_mult ; out = RMSNorm(residual, norm_w)
// so the peer wait sits in a kernel of M small CTAs instead of in the GEMM's 148 large ones, the weight stream of the next GEMM
// (launched with programmatic stream serialization) runs underneath it, and the separate add + norm launch disappears.
// Replaces the all-reduce call sites core/.../generator/CausalSelfAttention.java:403-405,448-452 and
// core/.../model/tensorparallel/TensorParallelMlp.java:169-171 together with the residual add and norm of TransformerBlock.java:161-200.
__device__ __forceinline__ uint4 multimem_ld_reduce_bf16x8(const void* mc_addr) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(mc_addr)
               : "memory");
  return v;
}

__global__ void __launch_bounds__(256) tp_reduce_norm_kernel(const CommParams p, int N, int ncta, int mode, unsigned long long mc_recv, int kind,
                                                             const float* __restrict__ bias, __nv_bfloat16* residual,
                                                             const __nv_bfloat16* __restrict__ post_w, const __nv_bfloat16* __restrict__ norm_w,
                                                             __nv_bfloat16* __restrict__ out, float eps, float offset, float res_mult) {
  pdl_wait();     // the GEMM in front of this kernel has completed on this rank: its round counters and launch counter are final
  pdl_trigger();
  extern __shared__ float row[];  // N floats
  __shared__ float red[32];
  __shared__ int s_ok;
  const int m = blockIdx.x;
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  // every rank's GEMM CTAs have published this call (the GEMM left rounds[cta] at the value its peers' counters must reach)
  const uint32_t* mine = reinterpret_cast<const uint32_t*>(p.flags[p.rank]);
  for (int idx = threadIdx.x; idx < p.size * ncta; idx += blockDim.x) {
    const int src = idx / ncta, cta = idx - src * ncta;
    if (!flag_wait_ge(mine + static_cast<size_t>(src) * p.ncta_max + cta, p.rounds[cta], p.status, p.wait_limit)) s_ok = 0;
  }
  __syncthreads();
  if (s_ok == 0) return;
  const unsigned call = *reinterpret_cast<volatile unsigned*>(p.call) - 1u;  // the GEMM's last CTA has already advanced the counter
  const long long par_off = static_cast<long long>(call & 1u) * p.size * p.slab;
  float ss = 0.f;
  for (int i = threadIdx.x * 8; i < N; i += blockDim.x * 8) {
    float acc[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = 0.f;
    if (mode == 2) {
      const uint4 v = multimem_ld_reduce_bf16x8(reinterpret_cast<const __nv_bfloat16*>(mc_recv) + par_off + static_cast<long long>(m) * N + i);
      const uint32_t* vu = reinterpret_cast<const uint32_t*>(&v);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = unpack_bf162(vu[e]);
        acc[2 * e] = f.x;
        acc[2 * e + 1] = f.y;
      }
    } else {
      const __nv_bfloat16* rbase = reinterpret_cast<const __nv_bfloat16*>(p.recv[p.rank]) + par_off + static_cast<long long>(m) * N + i;
      for (int src = 0; src < p.size; ++src) {
        const uint4 v = __ldcg(reinterpret_cast<const uint4*>(rbase + static_cast<long long>(src) * p.slab));
        const uint32_t* vu = reinterpret_cast<const uint32_t*>(&v);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = unpack_bf162(vu[e]);
          acc[2 * e] += f.x;
          acc[2 * e + 1] += f.y;
        }
      }
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float v = bf2f(f2bf(acc[e] + (bias != nullptr ? bias[i + e] : 0.f)));  // rounded like the output of the fused GEMM + all-reduce
      row[i + e] = v;
      ss += v * v;
    }
  }
  if (kind == 0) {
    __syncthreads();
    for (int i = threadIdx.x * 8; i < N; i += blockDim.x * 8) {
      uint4 o;
      uint32_t* ou = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
      for (int e = 0; e < 4; ++e) ou[e] = pack_bf162(row[i + 2 * e], row[i + 2 * e + 1]);
      *reinterpret_cast<uint4*>(out + static_cast<size_t>(m) * N + i) = o;
    }
    return;
  }
  if (post_w != nullptr) {  // gemma2: norm on the block output before it joins the residual stream
    ss = block_sum(ss, red);
    const float inv = rsqrtf(ss / N + eps);
    for (int i = threadIdx.x * 8; i < N; i += blockDim.x * 8) {
#pragma unroll
      for (int e = 0; e < 8; ++e) row[i + e] = bf2f(f2bf(row[i + e] * inv * (bf2f(post_w[i + e]) + offset)));
    }
  }
  ss = 0.f;
  for (int i = threadIdx.x * 8; i < N; i += blockDim.x * 8) {
    __nv_bfloat16* rp = residual + static_cast<size_t>(m) * N + i;
    const uint4 rv = *reinterpret_cast<const uint4*>(rp);
    const uint32_t* ru = reinterpret_cast<const uint32_t*>(&rv);
    uint4 ov;
    uint32_t* ou = reinterpret_cast<uint32_t*>(&ov);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 f = unpack_bf162(ru[e]);
      ou[e] = pack_bf162(f.x + row[i + 2 * e] * res_mult, f.y + row[i + 2 * e + 1] * res_mult);
      const float2 back = unpack_bf162(ou[e]);  // the norm sees the stored (rounded) residual
      row[i + 2 * e] = back.x;
      row[i + 2 * e + 1] = back.y;
      ss += back.x * back.x + back.y * back.y;
    }
    *reinterpret_cast<uint4*>(rp) = ov;
  }
  ss = block_sum(ss, red);
  const float inv = rsqrtf(ss / N + eps);
  for (int i = threadIdx.x * 8; i < N; i += blockDim.x * 8) {
    const uint4 wv = *reinterpret_cast<const uint4*>(norm_w + i);
    const uint32_t* wu = reinterpret_cast<const uint32_t*>(&wv);
    uint4 o;
    uint32_t* ou = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 f = unpack_bf162(wu[e]);
      ou[e] = pack_bf162(row[i + 2 * e] * inv * (f.x + offset), row[i + 2 * e + 1] * inv * (f.y + offset));
    }
    *reinterpret_cast<uint4*>(out + static_cast<size_t>(m) * N + i) = o;
  }
}

void launch_tp_reduce_norm(const GemmTpArgs* tp, int M, int N, int kind, const float* bias, void* residual, const void* post_w, const void* norm_w,
                           void* out, float eps, float offset, float res_mult, int* status, cudaStream_t st) {
  if (M == 0) return;
  launch_pdl(tp_reduce_norm_kernel, dim3(M), dim3(256), static_cast<size_t>(N) * sizeof(float), st, make_params(tp, status), N, tp->last_ctas, tp->mode,
             tp->mc_recv, kind, bias, static_cast<__nv_bfloat16*>(residual), static_cast<const __nv_bfloat16*>(post_w),
             static_cast<const __nv_bfloat16*>(norm_w), static_cast<__nv_bfloat16*>(out), eps, offset, res_mult);
}

// ------------------------------------------------------------------------------------------------ reduce-scatter + all-gather
// Second and third step of the prefill-size tensor-parallel projection (the first is the GEMM with epilogue EPI = 3, which has
// stored every rank's partial sums of MY token rows into my receive area [size sources][rows_per_rank][N]).
//   scatter_reduce_kernel: waits (bounded) until every source has published all its tiles for my rows, sums the slabs in rank
//     order (+ bias), writes the rows to `out` and, with plain peer stores, into the gather area of every other rank, then
//     publishes one count per CTA and peer.
//   scatter_finish_kernel: one CTA per row group of the OTHER ranks: waits (bounded) for that source's groups, copies the rows
//     from my gather area into `out`.
// Who waits for whom: a reduce CTA waits only for GEMM kernels (which never wait), a finish CTA only for reduce kernels, and on
// one GPU the three run in stream order, so no launch needs to be resident at once. Buffers are single: a rank's next GEMM comes
// after its finish kernel, i.e. after every peer has pushed its reduced rows and therefore has read its receive area; a peer's
// next reduce waits for this rank's next GEMM, which comes after this rank's finish kernel has drained the gather area.
// Counters are cumulative; the host passes the expected totals, so these launches are not captured in CUDA graphs.
struct ScatterParams {
  int size, rank, rows_per_rank, M, N;
  unsigned long long recv, gather[8], flags[8];
  unsigned int targets[8];
  int* status;
};

// push = 0: plain reduce-scatter, `out` holds only this rank's rows [rows, N] (row 0 = first owned row) and nothing is sent on.
__global__ void __launch_bounds__(256) scatter_reduce_kernel(const ScatterParams p, const float* __restrict__ bias, __nv_bfloat16* __restrict__ out,
                                                             int push) {
  __shared__ int s_ok;
  if (threadIdx.x < 32) {
    const int lane = threadIdx.x;
    bool ok_lane = true;
    if (lane < p.size) ok_lane = flag_wait_ge(reinterpret_cast<const uint32_t*>(p.flags[p.rank]) + lane, p.targets[0], p.status);
    const bool all = __all_sync(0xffffffffu, ok_lane);
    if (lane == 0) s_ok = all ? 1 : 0;
  }
  __syncthreads();
  if (s_ok == 0) return;
  const int first = p.rank * p.rows_per_rank;
  const int end = min(p.M, first + p.rows_per_rank);
  const int row0 = first + blockIdx.x * kScatterGroupRows;
  const int vec = p.N / 8;
  const __nv_bfloat16* slabs = reinterpret_cast<const __nv_bfloat16*>(p.recv);
  for (int idx = threadIdx.x; idx < kScatterGroupRows * vec; idx += blockDim.x) {
    const int r = idx / vec, i = idx - r * vec;
    const int m = row0 + r;
    if (m >= end) break;
    float acc[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = bias != nullptr ? bias[i * 8 + e] : 0.f;
    for (int src = 0; src < p.size; ++src) {
      const uint4 v = __ldcg(reinterpret_cast<const uint4*>(slabs + (static_cast<long long>(src) * p.rows_per_rank + (m - first)) * p.N) + i);
      const uint32_t* vu = reinterpret_cast<const uint32_t*>(&v);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = unpack_bf162(vu[e]);
        acc[2 * e] += f.x;
        acc[2 * e + 1] += f.y;
      }
    }
    uint4 o;
    uint32_t* ou = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
    for (int e = 0; e < 4; ++e) ou[e] = pack_bf162(acc[2 * e], acc[2 * e + 1]);
    const long long off = static_cast<long long>(m) * p.N;
    if (!push) {
      reinterpret_cast<uint4*>(out + static_cast<long long>(m - first) * p.N)[i] = o;
      continue;
    }
    reinterpret_cast<uint4*>(out + off)[i] = o;
    for (int d = 1; d < p.size; ++d)
      reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.gather[(p.rank + d) % p.size]) + off)[i] = o;
  }
  if (!push) return;
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x >= 1 && threadIdx.x < p.size)
    red_release_sys_add(reinterpret_cast<uint32_t*>(p.flags[(p.rank + threadIdx.x) % p.size]) + 8 + p.rank, 1u);
}

__global__ void __launch_bounds__(256) scatter_finish_kernel(const ScatterParams p, int groups_per_rank, __nv_bfloat16* __restrict__ out) {
  __shared__ int s_ok;
  const int src = blockIdx.x / groups_per_rank, g = blockIdx.x - src * groups_per_rank;
  if (src == p.rank || src >= p.size) return;
  const int first = src * p.rows_per_rank;
  const int end = min(p.M, first + p.rows_per_rank);
  const int row0 = first + g * kScatterGroupRows;
  if (row0 >= end) return;
  if (threadIdx.x == 0)
    s_ok = flag_wait_ge(reinterpret_cast<const uint32_t*>(p.flags[p.rank]) + 8 + src, p.targets[src], p.status) ? 1 : 0;
  __syncthreads();
  if (s_ok == 0) return;
  const int vec = p.N / 8;
  const __nv_bfloat16* mine = reinterpret_cast<const __nv_bfloat16*>(p.gather[p.rank]);
  for (int idx = threadIdx.x; idx < kScatterGroupRows * vec; idx += blockDim.x) {
    const int r = idx / vec, i = idx - r * vec;
    const int m = row0 + r;
    if (m >= end) break;
    const long long off = static_cast<long long>(m) * p.N;
    reinterpret_cast<uint4*>(out + off)[i] = __ldcg(reinterpret_cast<const uint4*>(mine + off) + i);
  }
}

// all-gather by push: this rank's rows of x [rows, K] go into every rank's gather area (own included) at their global row
// offset; one release-add per CTA and rank on flags[dst][16 + my rank]. The consumer is the GEMM with the gather prologue.
__global__ void __launch_bounds__(256) gather_push_kernel(const ScatterParams p, const __nv_bfloat16* __restrict__ x_own) {
  const int first = p.rank * p.rows_per_rank;
  const int end = min(p.M, first + p.rows_per_rank);
  const int row0 = first + blockIdx.x * kScatterGroupRows;
  const int vec = p.N / 8;  // N holds the row length K here
  for (int idx = threadIdx.x; idx < kScatterGroupRows * vec; idx += blockDim.x) {
    const int r = idx / vec, i = idx - r * vec;
    const int m = row0 + r;
    if (m >= end) break;
    const uint4 v = reinterpret_cast<const uint4*>(x_own + static_cast<long long>(m - first) * p.N)[i];
    const long long off = static_cast<long long>(m) * p.N;
    for (int d = 0; d < p.size; ++d)
      reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.gather[(p.rank + d) % p.size]) + off)[i] = v;
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x < p.size)
    red_release_sys_add(reinterpret_cast<uint32_t*>(p.flags[(p.rank + threadIdx.x) % p.size]) + 16 + p.rank, 1u);
}

static ScatterParams make_scatter_params(const GemmScatterArgs* a, const GemmScatterPlan* plan, int M, int N, int* status) {
  ScatterParams p = {};
  p.size = a->size;
  p.rank = a->rank;
  p.rows_per_rank = plan->rows_per_rank;
  p.M = M;
  p.N = N;
  p.recv = a->recv[a->rank];
  for (int r = 0; r < 8; ++r) {
    p.gather[r] = a->gather[r];
    p.flags[r] = a->flags[r];
  }
  p.status = status;
  return p;
}

void launch_scatter_reduce(const GemmScatterArgs* a, const GemmScatterPlan* plan, int M, int N, const float* bias, void* out,
                           unsigned gemm_target, bool push, int* status, cudaStream_t st) {
  const int groups = plan->groups[a->rank];
  if (groups == 0) return;
  ScatterParams p = make_scatter_params(a, plan, M, N, status);
  p.targets[0] = gemm_target;
  scatter_reduce_kernel<<<groups, 256, 0, st>>>(p, bias, static_cast<__nv_bfloat16*>(out), push ? 1 : 0);
}

void launch_scatter_finish(const GemmScatterArgs* a, const GemmScatterPlan* plan, int M, int N, void* out, const unsigned* group_targets,
                           int* status, cudaStream_t st) {
  const int groups_per_rank = plan->rows_per_rank / kScatterGroupRows;
  ScatterParams p = make_scatter_params(a, plan, M, N, status);
  for (int r = 0; r < 8; ++r) p.targets[r] = group_targets[r];
  scatter_finish_kernel<<<groups_per_rank * a->size, 256, 0, st>>>(p, groups_per_rank, static_cast<__nv_bfloat16*>(out));
}

void launch_gather_push(const GemmScatterArgs* a, const GemmScatterPlan* plan, const void* x_own, int M, int K, int* status, cudaStream_t st) {
  const int groups = plan->groups[a->rank];
  if (groups == 0) return;
  ScatterParams p = make_scatter_params(a, plan, M, K, status);
  gather_push_kernel<<<groups, 256, 0, st>>>(p, static_cast<const __nv_bfloat16*>(x_own));
}

}  // namespace dlv
