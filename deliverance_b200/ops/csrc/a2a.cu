// Expert-parallel all-to-all over NVLink peer memory: token rows that live sharded over the ranks (sequence-parallel residual
// stream) travel to the ranks that own their experts, are multiplied there by the grouped expert GEMMs, and travel back.
//
// Sender (rank s), per mixture-of-experts layer: moe_route has sorted its (token, slot) pairs by expert, so the pairs of the
// experts a destination rank d owns are one contiguous run of grouped rows. a2a_push_kernel stores every row of that run straight
// into d's receive area, region s, in the same order (plain 16-byte peer stores, one CTA per row); a2a_publish_kernel then tells d
// how many rows each of its experts got from s and where s keeps them (count and first grouped row per expert) and raises d's
// dispatch flag for s with a release store.
// Receiver (rank d): a2a_plan_kernel waits (bounded) for the dispatch flags of all sources, lays the rows out expert-major and
// source-major inside an expert (the row offsets per local expert feed the grouped GEMM's work list) and writes the segment table;
// a2a_gather_kernel copies the segments out of the receive regions into that layout. After the two grouped GEMMs
// a2a_return_kernel stores every output row into its sender's return buffer AT THE SENDER'S OWN GROUPED ROW INDEX, and a second
// publish raises the sender's return flag. The sender waits for all return flags (a2a_wait_kernel) and runs the ordinary top-k
// weighted combine over its return buffer: nothing is summed across ranks, so the result does not depend on arrival order.
// Buffer reuse needs no extra handshake: a rank dispatches layer L + 1 only after its combine of layer L, which waited for every
// peer's return of layer L, which those peers issued after reading their receive areas.
// Counters are cumulative launch epochs passed by the host (these launches are not captured in CUDA graphs).
//
// The reference runs every expert on one host (core/.../model/qwen3/Qwen3MoeFeedForward.java:107-183: group by expert, per-expert
// GEMMs, weighted scatter-add; MixtureOfExpertsBlock.java:78-112); it has no expert parallelism to compare with.
#include "common.cuh"
#include "gemm_api.h"

namespace dlv {

__device__ __forceinline__ void st_release_sys_u32(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// grid = grouped rows of this rank (T_own * k), 128 threads. offsets: the sender's exclusive expert offsets [E + 1].
__global__ void __launch_bounds__(128) a2a_push_kernel(const A2AParams p, const __nv_bfloat16* __restrict__ x, const int* __restrict__ perm,
                                                       const int* __restrict__ offsets, int k, int H) {
  const int g = blockIdx.x;
  // destination = owner of the expert whose run contains grouped row g (ranks own ne consecutive experts)
  int d = 0;
  while (d + 1 < p.size && g >= offsets[(d + 1) * p.ne]) ++d;
  const int pidx = g - offsets[d * p.ne];
  if (pidx >= p.cap) return;  // cannot happen: the host sizes cap for all of a rank's pairs
  const int t = perm[g] / k;
  const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<size_t>(t) * H);
  uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.recv[d]) + (static_cast<size_t>(p.rank) * p.cap + pidx) * H);
  for (int i = threadIdx.x; i < H / 8; i += blockDim.x) dst[i] = src[i];
  __threadfence_system();
}

// one CTA per destination: per-expert counts and first grouped rows, then the flag. which: 0 dispatch, 1 return.
__global__ void __launch_bounds__(128) a2a_publish_kernel(const A2AParams p, const int* __restrict__ offsets, int which, unsigned epoch) {
  const int d = blockIdx.x;
  if (which == 0) {
    int* meta = reinterpret_cast<int*>(p.meta[d]) + static_cast<size_t>(p.rank) * 2 * p.ne;
    for (int e = threadIdx.x; e < p.ne; e += blockDim.x) {
      meta[e] = offsets[d * p.ne + e + 1] - offsets[d * p.ne + e];
      meta[p.ne + e] = offsets[d * p.ne + e];
    }
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) st_release_sys_u32(reinterpret_cast<uint32_t*>(p.flags[d]) + which * 8 + p.rank, epoch);
}

// single CTA. Waits for every source's dispatch flag, then: local_offsets[ne + 1] (rows per local expert, expert-major),
// seg[(e * size + s)] = {first row in region s, first row in the grouped layout, rows, first grouped row at the sender}.
__global__ void __launch_bounds__(256) a2a_plan_kernel(const A2AParams p, unsigned epoch, int* __restrict__ local_offsets, int4* __restrict__ seg) {
  __shared__ int s_ok;
  __shared__ int cnt[8][128], soff[8][128];
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  if (threadIdx.x < p.size) {
    if (!flag_wait_ge(reinterpret_cast<const uint32_t*>(p.flags[p.rank]) + threadIdx.x, epoch, p.status)) s_ok = 0;
  }
  __syncthreads();
  if (s_ok == 0) return;
  const int* meta = reinterpret_cast<const int*>(p.meta[p.rank]);
  for (int i = threadIdx.x; i < p.size * p.ne; i += blockDim.x) {
    const int s = i / p.ne, e = i - s * p.ne;
    cnt[s][e] = __ldcg(meta + static_cast<size_t>(s) * 2 * p.ne + e);
    soff[s][e] = __ldcg(meta + static_cast<size_t>(s) * 2 * p.ne + p.ne + e);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int acc = 0;
    int in_region[8] = {0, 0, 0, 0, 0, 0, 0, 0};  // rows of the experts in front of e that source s sent: they precede e's rows in region s
    for (int e = 0; e < p.ne; ++e) {
      local_offsets[e] = acc;
      for (int s = 0; s < p.size; ++s) {
        seg[e * p.size + s] = make_int4(in_region[s], acc, cnt[s][e], soff[s][e]);
        in_region[s] += cnt[s][e];
        acc += cnt[s][e];
      }
    }
    local_offsets[p.ne] = acc;
  }
}

// grid = upper bound of received rows, 128 threads: grouped row r -> its segment (binary search over the grouped starts) -> copy
__device__ __forceinline__ int a2a_find_seg(const int4* seg, int n_seg, int r) {
  int lo = 0, hi = n_seg - 1;  // last segment with start <= r (segments are in grouped order; empty ones share a start)
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (seg[mid].y <= r) lo = mid; else hi = mid - 1;
  }
  return lo;  // never an empty segment: the segment behind an empty one starts at the same row and is found instead
}

__global__ void __launch_bounds__(128) a2a_gather_kernel(const A2AParams p, const int* __restrict__ local_offsets, const int4* __restrict__ seg,
                                                         __nv_bfloat16* __restrict__ xs, int H) {
  const int r = blockIdx.x;
  if (r >= local_offsets[p.ne]) return;
  const int n_seg = p.ne * p.size;
  const int si = a2a_find_seg(seg, n_seg, r);
  const int4 sg = seg[si];
  const int s = si % p.size;
  const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(p.recv[p.rank]) +
                                                    (static_cast<size_t>(s) * p.cap + sg.x + (r - sg.y)) * H);
  uint4* dst = reinterpret_cast<uint4*>(xs + static_cast<size_t>(r) * H);
  for (int i = threadIdx.x; i < H / 8; i += blockDim.x) dst[i] = __ldcg(src + i);
}

// grid = upper bound of received rows: expert output row r goes to its sender's return buffer at the sender's grouped row index
__global__ void __launch_bounds__(128) a2a_return_kernel(const A2AParams p, const int* __restrict__ local_offsets, const int4* __restrict__ seg,
                                                         const __nv_bfloat16* __restrict__ ys, int H) {
  const int r = blockIdx.x;
  if (r >= local_offsets[p.ne]) return;
  const int n_seg = p.ne * p.size;
  const int si = a2a_find_seg(seg, n_seg, r);
  const int4 sg = seg[si];
  const int s = si % p.size;
  const uint4* src = reinterpret_cast<const uint4*>(ys + static_cast<size_t>(r) * H);
  uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.ret[s]) + (static_cast<size_t>(sg.w) + (r - sg.y)) * H);
  for (int i = threadIdx.x; i < H / 8; i += blockDim.x) dst[i] = src[i];
  __threadfence_system();
}

// single warp: every rank has returned this rank's rows
__global__ void __launch_bounds__(32) a2a_wait_kernel(const A2AParams p, unsigned epoch) {
  if (threadIdx.x < p.size) flag_wait_ge(reinterpret_cast<const uint32_t*>(p.flags[p.rank]) + 8 + threadIdx.x, epoch, p.status);
}

void launch_a2a_dispatch(const A2AParams* p, const void* x, const int* perm, const int* offsets, int rows, int k, int H, unsigned epoch, cudaStream_t st) {
  if (rows > 0) a2a_push_kernel<<<rows, 128, 0, st>>>(*p, static_cast<const __nv_bfloat16*>(x), perm, offsets, k, H);
  a2a_publish_kernel<<<p->size, 128, 0, st>>>(*p, offsets, 0, epoch);
}
void launch_a2a_receive(const A2AParams* p, unsigned epoch, int* local_offsets, int* seg, void* xs, int max_rows, int H, cudaStream_t st) {
  a2a_plan_kernel<<<1, 256, 0, st>>>(*p, epoch, local_offsets, reinterpret_cast<int4*>(seg));
  if (max_rows > 0) a2a_gather_kernel<<<max_rows, 128, 0, st>>>(*p, local_offsets, reinterpret_cast<const int4*>(seg), static_cast<__nv_bfloat16*>(xs), H);
}
void launch_a2a_return(const A2AParams* p, const int* local_offsets, const int* seg, const void* ys, int max_rows, int H, unsigned epoch, cudaStream_t st) {
  if (max_rows > 0) a2a_return_kernel<<<max_rows, 128, 0, st>>>(*p, local_offsets, reinterpret_cast<const int4*>(seg), static_cast<const __nv_bfloat16*>(ys), H);
  a2a_publish_kernel<<<p->size, 128, 0, st>>>(*p, nullptr, 1, epoch);
}
void launch_a2a_wait(const A2AParams* p, unsigned epoch, cudaStream_t st) { a2a_wait_kernel<<<1, 32, 0, st>>>(*p, epoch); }

}  // namespace dlv
