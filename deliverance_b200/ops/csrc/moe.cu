// Mixture-of-experts routing and token shuffling.
//   moe_route:   router logits [T, E] fp32 -> top-k weights / expert ids per token (softmax-all -> top-k -> optional
//                renormalise, or top-k -> softmax over the k), per-expert histogram, exclusive offsets and the permutation
//                that groups (token, slot) pairs by expert — one kernel launch + one small scan kernel.
//   moe_gather:  x [T, H] -> xs [T*k, H] rows in expert-grouped order.
//   moe_combine: ys [T*k, H] (expert outputs in grouped order) -> out [T, H] = sum_j w[t, j] * ys[pos(t, j)]  (fp32 sum in
//                slot order: deterministic, no atomics).
// Reference semantics: core/.../model/MixtureOfExpertsBlock.java:78-112, qwen3/Qwen3MoeFeedForward.java:107-301,
// granitemoehybrid/GraniteMoeHybridMoeFeedForward.java:112-141.
#include "common.cuh"

namespace dlv {

constexpr int kMaxTopK = 16;

// Top-k of one token by one warp (E <= 1024): softmax statistics, k rounds of "every lane proposes its best remaining expert"
// (ties -> lower index), weights by `mode` (0: softmax over all experts, then top-k, optional renormalisation; 1: softmax over
// the k chosen). Lane 0 stores weights and expert ids, adds to the histogram `counts` (global or shared memory) and, when
// `idx_copy` is given, keeps a second copy of the ids there.
__device__ __forceinline__ void moe_topk_token(const float* __restrict__ row, int E, int k, int mode, int renorm, int lane,
                                               float* __restrict__ w_out, int* __restrict__ idx_out, int* counts, int* idx_copy) {
  float mx = -INFINITY;
  for (int e = lane; e < E; e += 32) mx = fmaxf(mx, row[e]);
  mx = warp_max(mx);
  float den = 0.f;
  for (int e = lane; e < E; e += 32) den += __expf(row[e] - mx);
  den = warp_sum(den);
  float sel_v[kMaxTopK];
  int sel_i[kMaxTopK];
  unsigned long long taken_lo = 0ull;  // bitmask of this lane's taken slots (expert e = lane + 32 * j -> bit j)
  for (int r = 0; r < k; ++r) {
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int e = lane, j = 0; e < E; e += 32, ++j) {
      if ((taken_lo >> j) & 1ull) continue;
      const float v = row[e];
      if (v > bv || (v == bv && e < bi)) {
        bv = v;
        bi = e;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) {
        bv = ov;
        bi = oi;
      }
    }
    sel_v[r] = bv;
    sel_i[r] = bi;
    if ((bi & 31) == lane) taken_lo |= 1ull << (bi >> 5);
  }
  if (lane == 0) {
    float wts[kMaxTopK];
    float s = 0.f;
    if (mode == 0) {
      for (int r = 0; r < k; ++r) {
        wts[r] = __expf(sel_v[r] - mx) / den;
        s += wts[r];
      }
      if (renorm)
        for (int r = 0; r < k; ++r) wts[r] /= s;
    } else {
      for (int r = 0; r < k; ++r) {
        wts[r] = __expf(sel_v[r] - sel_v[0]);
        s += wts[r];
      }
      for (int r = 0; r < k; ++r) wts[r] /= s;
    }
    for (int r = 0; r < k; ++r) {
      w_out[r] = wts[r];
      idx_out[r] = sel_i[r];
      if (idx_copy != nullptr) idx_copy[r] = sel_i[r];
      atomicAdd(&counts[sel_i[r]], 1);
    }
  }
}

// one warp per token
__global__ void __launch_bounds__(256) moe_topk_kernel(const float* __restrict__ logits, int T, int E, int k, int mode, int renorm,
                                                       float* __restrict__ w_out, int* __restrict__ idx_out, int* __restrict__ counts) {
  pdl_wait();     // no-op unless launched with programmatic stream serialization: the kernel in front has completed
  pdl_trigger();  // the next kernel may start its prologue (and a GEMM its weight prefetch) under this kernel's tail
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (t >= T) return;
  moe_topk_token(logits + static_cast<size_t>(t) * E, E, k, mode, renorm, lane, w_out + static_cast<size_t>(t) * k,
                 idx_out + static_cast<size_t>(t) * k, counts, nullptr);
}

// Routing of a decode-size batch in ONE launch of one CTA (32 warps): top-k per token, expert histogram and offsets, the stable
// permutation that groups (token, slot) pairs by expert, and the grouped GEMM's work list for the local experts [e0, e0 + ne)
// with `bn` rows per item. It replaces a memset and four launches (moe_topk, moe_sort, moe_items and, where the grouped GEMV reads
// token rows through `perm`, moe_gather), which cost more than the work at a few hundred pairs. Shared memory: T k + 2 E + ne + 3
// ints. Same results as the separate kernels (same tie rule, same stable order).
constexpr int kRouteSmallMaxPairs = 8192;
constexpr int kRouteSmallMaxTokens = 128;  // a warp takes every 32nd token: beyond a few tokens per warp the many-CTA kernels win
__device__ __forceinline__ int warp_incl_scan(int v, int lane) {
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int n = __shfl_up_sync(0xffffffffu, v, o);
    if (lane >= o) v += n;
  }
  return v;
}
__global__ void __launch_bounds__(1024) moe_route_small_kernel(const float* __restrict__ logits, int T, int E, int k, int mode, int renorm,
                                                               float* __restrict__ w_out, int* __restrict__ idx_out, int* __restrict__ counts,
                                                               int* __restrict__ offsets, int* __restrict__ perm, int* __restrict__ pos, int e0,
                                                               int ne, int bn, int max_items, int4* __restrict__ items) {
  pdl_wait();
  pdl_trigger();
  extern __shared__ int rs[];
  const int P = T * k;
  int* idx_s = rs;              // [P] expert of every (token, slot) pair
  int* cnt_s = idx_s + P;       // [E]
  int* off_s = cnt_s + E;       // [E + 1]
  int* first_s = off_s + E + 1; // [ne + 1] first work item of every local expert
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  for (int e = tid; e < E; e += 1024) cnt_s[e] = 0;
  __syncthreads();
  for (int t = warp; t < T; t += 32)
    moe_topk_token(logits + static_cast<size_t>(t) * E, E, k, mode, renorm, lane, w_out + static_cast<size_t>(t) * k,
                   idx_out + static_cast<size_t>(t) * k, cnt_s, idx_s + t * k);
  __syncthreads();
  if (warp == 0) {  // exclusive scan of the histogram: lane l owns a contiguous chunk of experts
    const int chunk = (E + 31) / 32, lo = min(E, lane * chunk), hi = min(E, lo + chunk);
    int sum = 0;
    for (int e = lo; e < hi; ++e) sum += cnt_s[e];
    const int incl = warp_incl_scan(sum, lane);
    int acc = incl - sum;
    for (int e = lo; e < hi; ++e) {
      off_s[e] = acc;
      acc += cnt_s[e];
    }
    if (lane == 31) off_s[E] = incl;
  } else if (warp == 1 && items != nullptr) {  // the same over the local experts' item counts
    const int chunk = (ne + 31) / 32, lo = min(ne, lane * chunk), hi = min(ne, lo + chunk);
    int sum = 0;
    for (int e = lo; e < hi; ++e) sum += (cnt_s[e0 + e] + bn - 1) / bn;
    const int incl = warp_incl_scan(sum, lane);
    int acc = incl - sum;
    for (int e = lo; e < hi; ++e) {
      first_s[e] = acc;
      acc += (cnt_s[e0 + e] + bn - 1) / bn;
    }
    if (lane == 31) first_s[ne] = incl;
  }
  __syncthreads();
  for (int e = tid; e <= E; e += 1024) offsets[e] = off_s[e];
  for (int e = tid; e < E; e += 1024) counts[e] = cnt_s[e];
  // stable grouping: a warp takes an expert and walks the pairs 32 at a time (ballot + prefix count keeps ascending pair order)
  for (int e = warp; e < E; e += 32) {
    if (cnt_s[e] == 0) continue;
    int row = off_s[e];
    for (int p0 = 0; p0 < P; p0 += 32) {
      const int p = p0 + lane;
      const bool mine = p < P && idx_s[p] == e;
      const unsigned m = __ballot_sync(0xffffffffu, mine);
      if (mine) {
        const int r = row + __popc(m & ((1u << lane) - 1u));
        perm[r] = p;
        pos[p] = r;
      }
      row += __popc(m);
    }
  }
  if (items != nullptr) {
    for (int e = tid; e < ne; e += 1024) {
      const int lo = off_s[e0 + e], hi = off_s[e0 + e + 1];
      int it = first_s[e];
      for (int r = lo; r < hi && it < max_items; r += bn, ++it) items[it] = make_int4(e, r, hi, 0);
    }
    for (int it = first_s[ne] + tid; it < max_items; it += 1024) items[it] = make_int4(-1, 0, 0, 0);
  }
}

// single CTA: exclusive scan of counts -> offsets[E + 1]; then a stable counting sort of (token, slot) pairs by expert.
// pos[t * k + j] = row of that pair in the grouped order; perm[row] = t * k + j.
__global__ void __launch_bounds__(1024) moe_sort_kernel(const int* __restrict__ idx, const int* __restrict__ counts, int T, int E, int k,
                                                        int* __restrict__ offsets, int* __restrict__ perm, int* __restrict__ pos) {
  pdl_wait();     // no-op unless launched with programmatic stream serialization: the kernel in front has completed
  pdl_trigger();  // the next kernel may start its prologue (and a GEMM its weight prefetch) under this kernel's tail
  extern __shared__ int sh[];  // E + 1 offsets
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int e = 0; e < E; ++e) {
      sh[e] = acc;
      acc += counts[e];
    }
    sh[E] = acc;
  }
  __syncthreads();
  for (int e = threadIdx.x; e <= E; e += blockDim.x) offsets[e] = sh[e];
  // stable order inside an expert: ascending (token, slot). One thread per expert walks the pairs of its expert.
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int row = sh[e];
    if (counts[e] == 0) continue;
    for (int p = 0; p < T * k; ++p) {
      if (idx[p] == e) {
        perm[row] = p;
        pos[p] = row;
        ++row;
      }
    }
  }
}

// The same grouping for prefill-size batches, in parallel. The single-CTA kernel above walks all T k pairs once per expert (one
// thread each): 2.5 ms for the 65,536 pairs of an 8,192-token chunk with 128 experts, two thirds of the whole MoE block at prefill.
// Here the pairs are cut into chunks of kSortChunk: (a) every chunk counts its pairs per expert, (b) one CTA turns the expert
// histogram into offsets and the chunk counts into the first row of every (chunk, expert), (c) one warp per chunk hands out the
// rows in pair order (__match_any_sync groups the lanes of one expert; the group's first lane advances the running row). The
// order is the stable one: ascending pair index inside an expert.
constexpr int kSortChunk = 1024;
constexpr int kSortSerialMaxPairs = 1024;  // up to here the single-CTA kernel is used
__global__ void __launch_bounds__(256) moe_chunk_hist_kernel(const int* __restrict__ idx, int P, int E, int* __restrict__ chunk_hist) {
  pdl_wait();
  pdl_trigger();
  extern __shared__ int hs[];  // [E]
  for (int e = threadIdx.x; e < E; e += blockDim.x) hs[e] = 0;
  __syncthreads();
  const int p0 = blockIdx.x * kSortChunk, p1 = min(P, p0 + kSortChunk);
  for (int p = p0 + threadIdx.x; p < p1; p += blockDim.x) atomicAdd(&hs[idx[p]], 1);
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) chunk_hist[static_cast<size_t>(blockIdx.x) * E + e] = hs[e];
}
// chunk_hist [C, E]: counts on entry, first grouped row of the (chunk, expert) on exit
__global__ void __launch_bounds__(1024) moe_chunk_scan_kernel(const int* __restrict__ counts, int E, int C, int* __restrict__ offsets,
                                                              int* __restrict__ chunk_hist) {
  pdl_wait();
  pdl_trigger();
  extern __shared__ int sh[];  // [E + 1]
  const int lane = threadIdx.x & 31;
  if (threadIdx.x < 32) {
    const int chunk = (E + 31) / 32, lo = min(E, lane * chunk), hi = min(E, lo + chunk);
    int sum = 0;
    for (int e = lo; e < hi; ++e) sum += counts[e];
    const int incl = warp_incl_scan(sum, lane);
    int acc = incl - sum;
    for (int e = lo; e < hi; ++e) {
      sh[e] = acc;
      acc += counts[e];
    }
    if (lane == 31) sh[E] = incl;
  }
  __syncthreads();
  for (int e = threadIdx.x; e <= E; e += blockDim.x) offsets[e] = sh[e];
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int acc = sh[e];
    for (int c = 0; c < C; ++c) {
      const int h = chunk_hist[static_cast<size_t>(c) * E + e];
      chunk_hist[static_cast<size_t>(c) * E + e] = acc;
      acc += h;
    }
  }
}
__global__ void __launch_bounds__(32) moe_chunk_rank_kernel(const int* __restrict__ idx, int P, int E, const int* __restrict__ chunk_base,
                                                            int* __restrict__ perm, int* __restrict__ pos) {
  pdl_wait();
  pdl_trigger();
  extern __shared__ int rk[];  // [E] running row per expert, then [kSortChunk] the chunk's expert ids
  int* run_s = rk;
  int* idx_s = rk + E;
  const int lane = threadIdx.x;
  const int p0 = blockIdx.x * kSortChunk, n = min(P - p0, kSortChunk);
  for (int e = lane; e < E; e += 32) run_s[e] = chunk_base[static_cast<size_t>(blockIdx.x) * E + e];
  for (int i = lane; i < n; i += 32) idx_s[i] = idx[p0 + i];
  __syncwarp();
  for (int q = 0; q < n; q += 32) {
    const int i = q + lane;
    const bool valid = i < n;
    const int e = valid ? idx_s[i] : -1 - lane;  // (lanes past the end each form a group of their own)
    const unsigned m = __match_any_sync(0xffffffffu, e);
    const int r = __popc(m & ((1u << lane) - 1u));
    const int base = valid ? run_s[e] : 0;
    __syncwarp();
    if (valid && r == 0) run_s[e] = base + __popc(m);
    __syncwarp();
    if (valid) {
      perm[base + r] = p0 + i;
      pos[p0 + i] = base + r;
    }
  }
}

__global__ void __launch_bounds__(128) moe_gather_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ perm, int k, int H,
                                                         __nv_bfloat16* __restrict__ xs, const int* __restrict__ offsets, int e0, int ne) {
  pdl_wait();     // no-op unless launched with programmatic stream serialization: the kernel in front has completed
  pdl_trigger();  // the next kernel may start its prologue (and a GEMM its weight prefetch) under this kernel's tail
  const int row = blockIdx.x;
  if (offsets != nullptr && (row < offsets[e0] || row >= offsets[e0 + ne])) return;  // another rank's expert
  const int t = perm[row] / k;
  const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<size_t>(t) * H);
  uint4* dst = reinterpret_cast<uint4*>(xs + static_cast<size_t>(row) * H);
  for (int i = threadIdx.x; i < H / 8; i += blockDim.x) dst[i] = src[i];
}

__global__ void __launch_bounds__(128) moe_combine_kernel(const __nv_bfloat16* __restrict__ ys, const int* __restrict__ pos,
                                                          const float* __restrict__ w, int k, int H, __nv_bfloat16* __restrict__ out,
                                                          const int* __restrict__ offsets, int e0, int ne) {
  pdl_wait();     // no-op unless launched with programmatic stream serialization: the kernel in front has completed
  pdl_trigger();  // the next kernel may start its prologue (and a GEMM its weight prefetch) under this kernel's tail
  const int t = blockIdx.x;
  const int lo = offsets != nullptr ? offsets[e0] : 0, hi = offsets != nullptr ? offsets[e0 + ne] : 0x7fffffff;
  for (int i = threadIdx.x; i < H / 8; i += blockDim.x) {
    float acc[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = 0.f;
    for (int j = 0; j < k; ++j) {
      const float wt = w[static_cast<size_t>(t) * k + j];
      const int prow = pos[static_cast<size_t>(t) * k + j];
      if (prow < lo || prow >= hi) continue;  // computed on another rank; the all-reduce adds it
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
    reinterpret_cast<uint4*>(out + static_cast<size_t>(t) * H)[i] = o;
  }
}

// Ints of workspace launch_moe_route needs for T tokens (0: none, the single-CTA grouping is used)
size_t moe_route_workspace_ints(int T, int E, int k) {
  const long long P = static_cast<long long>(T) * k;
  return P > kSortSerialMaxPairs ? static_cast<size_t>((P + kSortChunk - 1) / kSortChunk) * E : 0;
}
void launch_moe_route(const float* logits, int T, int E, int k, int mode, int renorm, float* w, int* idx, int* counts, int* offsets,
                      int* perm, int* pos, int* ws, cudaStream_t st) {
  cudaMemsetAsync(counts, 0, sizeof(int) * E, st);
  if (T == 0) {
    cudaMemsetAsync(offsets, 0, sizeof(int) * (E + 1), st);
    return;
  }
  moe_topk_kernel<<<(T + 7) / 8, 256, 0, st>>>(logits, T, E, k, mode, renorm, w, idx, counts);
  const int P = T * k;
  if (ws != nullptr && moe_route_workspace_ints(T, E, k) > 0) {
    const int C = (P + kSortChunk - 1) / kSortChunk;
    moe_chunk_hist_kernel<<<C, 256, sizeof(int) * E, st>>>(idx, P, E, ws);
    moe_chunk_scan_kernel<<<1, 1024, sizeof(int) * (E + 1), st>>>(counts, E, C, offsets, ws);
    moe_chunk_rank_kernel<<<C, 32, sizeof(int) * (E + kSortChunk), st>>>(idx, P, E, ws, perm, pos);
    return;
  }
  moe_sort_kernel<<<1, 1024, sizeof(int) * (E + 1), st>>>(idx, counts, T, E, k, offsets, perm, pos);
}
// Decode-size batches: everything of launch_moe_route + launch_moe_items in one launch. False when the batch is too large for it.
bool launch_moe_route_small(const float* logits, int T, int E, int k, int mode, int renorm, float* w, int* idx, int* counts, int* offsets,
                            int* perm, int* pos, int e0, int ne, int bn, int max_items, int* items, cudaStream_t st) {
  if (T < 1 || T > kRouteSmallMaxTokens || T * k > kRouteSmallMaxPairs || E > 1024 || ne > 1024) return false;
  const size_t smem = sizeof(int) * (static_cast<size_t>(T) * k + 2 * E + ne + 3);
  return launch_pdl(moe_route_small_kernel, dim3(1), dim3(1024), smem, st, logits, T, E, k, mode, renorm, w, idx, counts, offsets, perm, pos, e0,
                    ne, bn, max_items, reinterpret_cast<int4*>(items)) == cudaSuccess;
}
void launch_moe_gather(const void* x, const int* perm, int rows, int k, int H, void* xs, const int* offsets, int e0, int ne,
                       cudaStream_t st) {
  if (rows == 0) return;
  moe_gather_kernel<<<rows, 128, 0, st>>>(static_cast<const __nv_bfloat16*>(x), perm, k, H, static_cast<__nv_bfloat16*>(xs), offsets, e0, ne);
}
void launch_moe_combine(const void* ys, const int* pos, const float* w, int T, int k, int H, void* out, const int* offsets, int e0,
                        int ne, cudaStream_t st) {
  if (T == 0) return;
  moe_combine_kernel<<<T, 128, 0, st>>>(static_cast<const __nv_bfloat16*>(ys), pos, w, k, H, static_cast<__nv_bfloat16*>(out), offsets, e0, ne);
}

// Work list of the grouped GEMM: one item {local expert, first row, end row, 0} per `bn` rows of every local expert that has
// rows, in expert order; the rest of the `max_items` slots get expert = -1. Single CTA (at most a few hundred items).
__global__ void __launch_bounds__(256) moe_items_kernel(const int* __restrict__ offsets, int e0, int ne, int bn, int max_items,
                                                        int4* __restrict__ items) {
  pdl_wait();     // no-op unless launched with programmatic stream serialization: the kernel in front has completed
  pdl_trigger();  // the next kernel may start its prologue (and a GEMM its weight prefetch) under this kernel's tail
  __shared__ int first[1025];
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int e = 0; e < ne; ++e) {
      first[e] = acc;
      acc += (offsets[e0 + e + 1] - offsets[e0 + e] + bn - 1) / bn;
    }
    first[ne] = acc;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < ne; e += blockDim.x) {
    const int lo = offsets[e0 + e], hi = offsets[e0 + e + 1];
    int it = first[e];
    for (int r = lo; r < hi && it < max_items; r += bn, ++it) items[it] = make_int4(e, r, hi, 0);
  }
  for (int it = first[ne] + threadIdx.x; it < max_items; it += blockDim.x) items[it] = make_int4(-1, 0, 0, 0);
}
void launch_moe_items(const int* offsets, int e0, int ne, int bn, int max_items, int* items, cudaStream_t st) {
  if (ne > 1024) return;
  moe_items_kernel<<<1, 256, 0, st>>>(offsets, e0, ne, bn, max_items, reinterpret_cast<int4*>(items));
}

}  // namespace dlv
