// Sampler-side kernels over fp32 logits [B, V] (V up to 256k): greedy argmax with "first maximum wins", logit
// post-processing (Granite logits scaling, final-logit softcap cap*tanh(v/cap), guided-decoding allow-bitmask -> -inf).
// Reference order of operations: core/.../model/AbstractGeneratorSampler.java:117-155, GuideLogitsProcessor.java:23-41.
#include "common.cuh"

namespace dlv {

__device__ __forceinline__ float post_logit(float v, float softcap, float inv_scale) {
  v *= inv_scale;
  if (softcap > 0.f) v = softcap * tanhf(v / softcap);
  return v;
}
__device__ __forceinline__ bool mask_allows(const uint32_t* mask_row, int i) {
  return mask_row == nullptr || ((mask_row[i >> 5] >> (i & 31)) & 1u);
}

// one CTA per row
__global__ void __launch_bounds__(1024) argmax_kernel(const float* __restrict__ logits, int ld, int V,
                                                      const uint32_t* __restrict__ mask, int mask_ld, float softcap,
                                                      float inv_scale, long long* __restrict__ out_idx, float* __restrict__ out_val) {
  pdl_wait();     // no-op unless launched with programmatic stream serialization: the kernel in front has completed
  pdl_trigger();  // the next kernel may start its prologue (and a GEMM its weight prefetch) under this kernel's tail
  __shared__ float sv[32];
  __shared__ int si[32];
  const int b = blockIdx.x;
  const float* row = logits + static_cast<size_t>(b) * ld;
  const uint32_t* mrow = mask ? mask + static_cast<size_t>(b) * mask_ld : nullptr;
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    if (!mask_allows(mrow, i)) continue;
    const float v = row[i];
    if (v > best || (v == best && i < bi)) {
      best = v;
      bi = i;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) {
      best = ov;
      bi = oi;
    }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) {
    sv[warp] = best;
    si[warp] = bi;
  }
  __syncthreads();
  if (warp == 0) {
    const int nw = blockDim.x >> 5;
    best = lane < nw ? sv[lane] : -INFINITY;
    bi = lane < nw ? si[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) {
        best = ov;
        bi = oi;
      }
    }
    if (lane == 0) {
      if (bi == 0x7fffffff) bi = 0;  // every token masked or all logits -inf / NaN
      out_idx[b] = bi;
      if (out_val) out_val[b] = post_logit(row[bi], softcap, inv_scale);
    }
  }
}

// Two-stage argmax for large vocabularies and few rows: one CTA per row reads 600 KB alone (64 CTAs on 148 SMs, ~0.5 TB/s);
// here kArgmaxSeg CTAs share a row and a second small kernel keeps the first maximum. The partial results live in a static
// device buffer (rows <= kArgmaxRows): launches on different streams of one device must not overlap.
constexpr int kArgmaxSeg = 8;
constexpr int kArgmaxRows = 1024;
static __device__ float g_argmax_val[kArgmaxRows * kArgmaxSeg];
static __device__ int g_argmax_idx[kArgmaxRows * kArgmaxSeg];

__global__ void __launch_bounds__(512) argmax_part_kernel(const float* __restrict__ logits, int ld, int V, const uint32_t* __restrict__ mask,
                                                          int mask_ld) {
  pdl_wait();
  pdl_trigger();
  __shared__ float sv[16];
  __shared__ int si[16];
  const int b = blockIdx.x, seg = blockIdx.y;
  const int per = (((V + kArgmaxSeg - 1) / kArgmaxSeg) + 3) & ~3;
  const int lo = seg * per, hi = min(V, lo + per);
  const float* row = logits + static_cast<size_t>(b) * ld;
  const uint32_t* mrow = mask ? mask + static_cast<size_t>(b) * mask_ld : nullptr;
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) {
    if (!mask_allows(mrow, i)) continue;
    const float v = row[i];
    if (v > best || (v == best && i < bi)) {
      best = v;
      bi = i;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) {
      best = ov;
      bi = oi;
    }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) {
    sv[warp] = best;
    si[warp] = bi;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < static_cast<int>(blockDim.x >> 5); ++w) {
      if (sv[w] > best || (sv[w] == best && si[w] < bi)) {
        best = sv[w];
        bi = si[w];
      }
    }
    g_argmax_val[b * kArgmaxSeg + seg] = best;
    g_argmax_idx[b * kArgmaxSeg + seg] = bi;
  }
}

__global__ void __launch_bounds__(32) argmax_final_kernel(const float* __restrict__ logits, int ld, float softcap, float inv_scale,
                                                          long long* __restrict__ out_idx, float* __restrict__ out_val) {
  pdl_wait();
  pdl_trigger();
  const int b = blockIdx.x;
  if (threadIdx.x != 0) return;
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int s = 0; s < kArgmaxSeg; ++s) {
    const float v = g_argmax_val[b * kArgmaxSeg + s];
    const int i = g_argmax_idx[b * kArgmaxSeg + s];
    if (v > best || (v == best && i < bi)) {
      best = v;
      bi = i;
    }
  }
  if (bi == 0x7fffffff) bi = 0;  // every token masked or all logits -inf / NaN
  out_idx[b] = bi;
  if (out_val) out_val[b] = post_logit(logits[static_cast<size_t>(b) * ld + bi], softcap, inv_scale);
}

__global__ void __launch_bounds__(256) logits_post_kernel(float* __restrict__ logits, int ld, int V, const uint32_t* __restrict__ mask,
                                                          int mask_ld, float softcap, float inv_scale) {
  pdl_wait();     // no-op unless launched with programmatic stream serialization: the kernel in front has completed
  pdl_trigger();  // the next kernel may start its prologue (and a GEMM its weight prefetch) under this kernel's tail
  const int b = blockIdx.y;
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= V) return;
  float* row = logits + static_cast<size_t>(b) * ld;
  const uint32_t* mrow = mask ? mask + static_cast<size_t>(b) * mask_ld : nullptr;
  row[i] = mask_allows(mrow, i) ? post_logit(row[i], softcap, inv_scale) : -INFINITY;
}

// =====================================================================================================================
// Top-k / top-p / uniform-top-p sampling without sorting the vocabulary
// =====================================================================================================================
// Semantics (core/.../model/AbstractGeneratorSampler.java:100-323 as restated in engine/sampler.py): order the tokens by
// s = logit / T descending (ties: lower id first); keep the first L (top-k); softmax over the kept set; the nucleus is the
// shortest prefix whose mass reaches top_p; then either a uniform pick inside the nucleus or the inverse-CDF walk with one
// uniform u. Only three positions of that order matter (the L-th element, the nucleus end, the picked element), so the row
// is never sorted: one pass builds a 2048-bin histogram (count, weight) over a linear map of [min, max] (clamped to the top
// 40 nats), prefix sums locate the bin of each position, and only that bin's elements are gathered and sorted in shared
// memory. Weights are exp(s - max) in 40-bit fixed point and summed with integer atomics: the result does not depend on the
// order of the additions, so every tensor-parallel rank draws the same token. A bin with more than 4096 elements (or a
// position inside the clamped tail) makes the row report "not handled" and the caller falls back to the sorting path.
constexpr int kSampBins = 2048;
constexpr int kSampCand = 4096;
constexpr float kSampRange = 40.f;
constexpr double kSampOne = 1099511627776.0;  // 2^40

struct SampShared {
  unsigned int cnt[kSampBins];
  unsigned long long wsum[kSampBins];
  float ckey[kSampCand];
  int cidx[kSampCand];
  unsigned long long cw[kSampCand];
  float red_f[32];
  float red_g[32];
  unsigned int ncand;
  int bin_sel;
  unsigned int rank_sel;         // count-based: elements of the bin before the position
  unsigned long long w_before;   // weight-based: weight in front of the bin
  int result, fail;
};

__device__ __forceinline__ unsigned long long samp_weight(float s, float mx) {
  if (s == -INFINITY) return 0ull;
  return static_cast<unsigned long long>(exp(static_cast<double>(s) - static_cast<double>(mx)) * kSampOne + 0.5);
}
__device__ __forceinline__ int samp_bin(float s, float mx, float scale) {
  if (s == -INFINITY) return kSampBins - 1;
  const float d = (mx - s) * scale;
  return d >= static_cast<float>(kSampBins - 1) ? kSampBins - 1 : static_cast<int>(d);
}
// (a sorts before b) in the sampling order: larger key first, then lower index
__device__ __forceinline__ bool samp_before(float ka, int ia, float kb, int ib) { return ka > kb || (ka == kb && ia < ib); }

// Gather the elements of bin `b` into shared memory and sort them in sampling order. Returns false on overflow.
__device__ bool samp_collect_sort(SampShared& sh, const float* __restrict__ row, int V, float inv_t, float mx, float scale, int b) {
  __syncthreads();
  if (threadIdx.x == 0) sh.ncand = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const float s = row[i] * inv_t;
    if (samp_bin(s, mx, scale) == b) {
      const unsigned int slot = atomicAdd(&sh.ncand, 1u);
      if (slot < kSampCand) {
        sh.ckey[slot] = s;
        sh.cidx[slot] = i;
      }
    }
  }
  __syncthreads();
  const unsigned int n = sh.ncand;
  if (n > kSampCand) return false;
  unsigned int np2 = 1;
  while (np2 < n) np2 <<= 1;
  for (unsigned int i = n + threadIdx.x; i < np2; i += blockDim.x) {
    sh.ckey[i] = -INFINITY;
    sh.cidx[i] = 0x7fffffff;  // padding sorts last
  }
  __syncthreads();
  for (unsigned int k = 2; k <= np2; k <<= 1) {
    for (unsigned int j = k >> 1; j > 0; j >>= 1) {
      for (unsigned int i = threadIdx.x; i < np2; i += blockDim.x) {
        const unsigned int l = i ^ j;
        if (l > i) {
          const bool up = (i & k) == 0;
          const float ka = sh.ckey[i], kb = sh.ckey[l];
          const int ia = sh.cidx[i], ib = sh.cidx[l];
          const bool swap = up ? samp_before(kb, ib, ka, ia) : samp_before(ka, ia, kb, ib);
          if (swap) {
            sh.ckey[i] = kb;
            sh.cidx[i] = ib;
            sh.ckey[l] = ka;
            sh.cidx[l] = ia;
          }
        }
      }
      __syncthreads();
    }
  }
  for (unsigned int i = threadIdx.x; i < n; i += blockDim.x) sh.cw[i] = samp_weight(sh.ckey[i], mx);
  __syncthreads();
  return true;
}

// one CTA (1024 threads) per row. out_ok[b] = 0: the row needs the sorting fallback (out_tok[b] is then undefined).
__global__ void __launch_bounds__(1024) sample_kernel(const float* __restrict__ logits, int ld, int V, const float* __restrict__ inv_temp,
                                                      const long long* __restrict__ limits, const float* __restrict__ top_p,
                                                      const unsigned char* __restrict__ uniform, const float* __restrict__ us,
                                                      long long* __restrict__ out_tok, int* __restrict__ out_ok) {
  pdl_wait();
  pdl_trigger();
  extern __shared__ __align__(16) unsigned char samp_raw[];
  SampShared& sh = *reinterpret_cast<SampShared*>(samp_raw);
  const int b = blockIdx.x;
  const float* row = logits + static_cast<size_t>(b) * ld;
  const float inv_t = inv_temp[b];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  // ---- pass 1: max and smallest finite value of s
  float mx = -INFINITY, mn = INFINITY;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const float s = row[i] * inv_t;
    if (s != -INFINITY) {
      mx = fmaxf(mx, s);
      mn = fminf(mn, s);
    }
  }
  mx = warp_max(mx);
  mn = -warp_max(-mn);
  if (lane == 0) {
    sh.red_f[warp] = mx;
    sh.red_g[warp] = mn;
  }
  for (int i = threadIdx.x; i < kSampBins; i += blockDim.x) {
    sh.cnt[i] = 0u;
    sh.wsum[i] = 0ull;
  }
  if (threadIdx.x == 0) {
    sh.fail = 0;
    sh.result = 0;
  }
  __syncthreads();
  mx = -INFINITY;
  mn = INFINITY;
  for (int w = 0; w < 32; ++w) {
    mx = fmaxf(mx, sh.red_f[w]);
    mn = fminf(mn, sh.red_g[w]);
  }
  if (mx == -INFINITY) {  // every token masked out
    if (threadIdx.x == 0) out_ok[b] = 0;
    return;
  }
  const float range = fminf(kSampRange, fmaxf(mx - mn, 1e-6f));
  const float scale = static_cast<float>(kSampBins - 1) / range;
  // ---- pass 2: histogram of counts and fixed-point weights
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const float s = row[i] * inv_t;
    const int bin = samp_bin(s, mx, scale);
    atomicAdd(&sh.cnt[bin], 1u);
    const unsigned long long w = samp_weight(s, mx);
    if (w) atomicAdd(&sh.wsum[bin], w);
  }
  __syncthreads();
  // ---- inclusive prefix sums over the bins (warp 0: 64 consecutive bins per lane)
  if (warp == 0) {
    constexpr int PER = kSampBins / 32;
    unsigned int c = 0;
    unsigned long long w = 0;
    for (int j = 0; j < PER; ++j) {
      c += sh.cnt[lane * PER + j];
      w += sh.wsum[lane * PER + j];
    }
    unsigned int ci = c;
    unsigned long long wi = w;
    for (int o = 1; o < 32; o <<= 1) {
      const unsigned int oc = __shfl_up_sync(0xffffffffu, ci, o);
      const unsigned long long ow = __shfl_up_sync(0xffffffffu, wi, o);
      if (lane >= o) {
        ci += oc;
        wi += ow;
      }
    }
    unsigned int cb = ci - c;
    unsigned long long wb = wi - w;
    for (int j = 0; j < PER; ++j) {
      cb += sh.cnt[lane * PER + j];
      wb += sh.wsum[lane * PER + j];
      sh.cnt[lane * PER + j] = cb;
      sh.wsum[lane * PER + j] = wb;
    }
  }
  __syncthreads();
  auto cum_c = [&](int bin) -> unsigned int { return bin < 0 ? 0u : sh.cnt[bin]; };
  auto cum_w = [&](int bin) -> unsigned long long { return bin < 0 ? 0ull : sh.wsum[bin]; };
  const long long Lraw = limits[b];
  const unsigned int L = static_cast<unsigned int>(Lraw < 1 ? 1 : (Lraw > V ? V : Lraw));
  // ---- (a) top-k: bin and in-bin count of the L-th element, mass of the kept set
  int bL = kSampBins;            // bin that holds the L-th element (kSampBins: everything is kept)
  unsigned int rL = 0;           // kept elements of that bin
  unsigned long long total = cum_w(kSampBins - 1);
  if (L < static_cast<unsigned int>(V)) {
    int lo = 0, hi = kSampBins - 1;
    while (lo < hi) {
      const int mid = (lo + hi) >> 1;
      if (sh.cnt[mid] >= L) hi = mid; else lo = mid + 1;
    }
    bL = lo;
    rL = L - cum_c(bL - 1);
    if (bL == kSampBins - 1 || !samp_collect_sort(sh, row, V, inv_t, mx, scale, bL)) {
      if (threadIdx.x == 0) out_ok[b] = 0;
      return;
    }
    if (threadIdx.x == 0) {
      unsigned long long acc = cum_w(bL - 1);
      for (unsigned int j = 0; j < rL; ++j) acc += sh.cw[j];
      sh.w_before = acc;
    }
    __syncthreads();
    total = sh.w_before;
    __syncthreads();
  }
  // ---- (b) nucleus end
  const float tp = top_p[b];
  unsigned int n = L;                 // candidates the pick may come from
  unsigned long long nuc_total = total;
  int b_end = bL;                      // bin that holds the last candidate (kSampBins: none, all bins complete)
  unsigned int r_end = rL;             // candidates of that bin
  if (tp > 0.f) {
    const unsigned long long target = static_cast<unsigned long long>(static_cast<double>(tp) * static_cast<double>(total));
    int lo = 0, hi = bL < kSampBins ? bL : kSampBins - 1;
    while (lo < hi) {
      const int mid = (lo + hi) >> 1;
      const unsigned long long kw = (mid < bL) ? sh.wsum[mid] : total;
      if (kw >= target) hi = mid; else lo = mid + 1;
    }
    const int bp = lo;
    if (bp == kSampBins - 1 || !samp_collect_sort(sh, row, V, inv_t, mx, scale, bp)) {
      if (threadIdx.x == 0) out_ok[b] = 0;
      return;
    }
    if (threadIdx.x == 0) {
      const unsigned int lim = (bp == bL) ? rL : sh.ncand;
      unsigned long long acc = cum_w(bp - 1);
      unsigned int r = lim;
      for (unsigned int j = 0; j < lim; ++j) {
        acc += sh.cw[j];
        if (acc >= target) {
          r = j + 1;
          break;
        }
      }
      sh.rank_sel = r;
      sh.w_before = acc;
    }
    __syncthreads();
    b_end = bp;
    r_end = sh.rank_sel;
    n = cum_c(bp - 1) + r_end;
    nuc_total = sh.w_before;
    __syncthreads();
  }
  // ---- (c) the pick
  const float u = us[b];
  int bq;
  if (uniform[b]) {
    long long pos = static_cast<long long>(u * static_cast<float>(n));
    if (pos > static_cast<long long>(n) - 1) pos = static_cast<long long>(n) - 1;
    if (pos < 0) pos = 0;
    int lo = 0, hi = kSampBins - 1;
    while (lo < hi) {
      const int mid = (lo + hi) >> 1;
      if (sh.cnt[mid] > static_cast<unsigned int>(pos)) hi = mid; else lo = mid + 1;
    }
    bq = lo;
    if (bq == kSampBins - 1 || !samp_collect_sort(sh, row, V, inv_t, mx, scale, bq)) {
      if (threadIdx.x == 0) out_ok[b] = 0;
      return;
    }
    if (threadIdx.x == 0) sh.result = sh.cidx[static_cast<unsigned int>(pos) - cum_c(bq - 1)];
  } else {
    const unsigned long long t2 = static_cast<unsigned long long>(static_cast<double>(u) * static_cast<double>(nuc_total));
    int lo = 0, hi = b_end < kSampBins ? b_end : kSampBins - 1;
    while (lo < hi) {
      const int mid = (lo + hi) >> 1;
      const unsigned long long kw = (mid < b_end) ? sh.wsum[mid] : nuc_total;
      if (kw >= t2) hi = mid; else lo = mid + 1;
    }
    bq = lo;
    if (bq == kSampBins - 1 || !samp_collect_sort(sh, row, V, inv_t, mx, scale, bq)) {
      if (threadIdx.x == 0) out_ok[b] = 0;
      return;
    }
    if (threadIdx.x == 0) {
      const unsigned int lim = (bq == b_end) ? r_end : sh.ncand;
      unsigned long long acc = cum_w(bq - 1);
      int tok = sh.cidx[lim > 0 ? lim - 1 : 0];
      for (unsigned int j = 0; j < lim; ++j) {
        acc += sh.cw[j];
        if (acc >= t2) {
          tok = sh.cidx[j];
          break;
        }
      }
      sh.result = tok;
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    out_tok[b] = sh.result;
    out_ok[b] = 1;
  }
}

// ------------------------------------------------------------------------------------------------ exclude-top-choice (XTC)
// One CTA per row. probs = softmax(logits * inv_temp). When `fire[b]` is set and at least one token has a probability above
// `threshold[b]`: the most probable token if it is a special token, otherwise the LEAST probable token above the threshold (first
// index on ties); -1 when XTC does not apply to the row (the caller then samples normally). Reference:
// core/.../model/ExcludeTopChoicePicker.java:42-86.
__global__ void __launch_bounds__(1024) xtc_kernel(const float* __restrict__ logits, int ld, int V, const float* __restrict__ inv_temp,
                                                   const float* __restrict__ threshold, const unsigned char* __restrict__ fire,
                                                   const int* __restrict__ special, int n_special, long long* __restrict__ out_tok) {
  pdl_wait();
  pdl_trigger();
  __shared__ float red_f[32];
  __shared__ int red_i[32];
  __shared__ float s_val;
  __shared__ int s_idx;
  const int b = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (!fire[b]) {
    if (threadIdx.x == 0) out_tok[b] = -1;
    return;
  }
  const float* row = logits + static_cast<size_t>(b) * ld;
  const float it = inv_temp[b];
  // block-wide (value, first index) reduction; want_max: largest value, else smallest
  auto reduce = [&](float v, int i, bool want_max) {
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, v, o);
      const int oi = __shfl_xor_sync(0xffffffffu, i, o);
      const bool take = want_max ? (ov > v || (ov == v && oi < i)) : (ov < v || (ov == v && oi < i));
      if (take) { v = ov; i = oi; }
    }
    __syncthreads();
    if (lane == 0) { red_f[warp] = v; red_i[warp] = i; }
    __syncthreads();
    if (warp == 0) {
      v = red_f[lane];
      i = red_i[lane];
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, o);
        const int oi = __shfl_xor_sync(0xffffffffu, i, o);
        const bool take = want_max ? (ov > v || (ov == v && oi < i)) : (ov < v || (ov == v && oi < i));
        if (take) { v = ov; i = oi; }
      }
      if (lane == 0) { s_val = v; s_idx = i; }
    }
    __syncthreads();
  };
  float mx = -INFINITY;
  int mi = 0x7fffffff;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const float v = row[i] * it;
    if (v > mx) { mx = v; mi = i; }
  }
  reduce(mx, mi, true);
  const float gmx = s_val;
  const int top = s_idx;
  if (gmx == -INFINITY) {
    if (threadIdx.x == 0) out_tok[b] = -1;
    return;
  }
  float sum = 0.f;
  for (int i = threadIdx.x; i < V; i += blockDim.x) sum += __expf(row[i] * it - gmx);
  sum = warp_sum(sum);
  __syncthreads();
  if (lane == 0) red_f[warp] = sum;
  __syncthreads();
  sum = 0.f;
  for (int w = 0; w < 32; ++w) sum += red_f[w];
  const float thr = threshold[b];
  // least probable token whose probability exceeds the threshold
  float lo = INFINITY;
  int li = 0x7fffffff;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const float pr = __expf(row[i] * it - gmx) / sum;
    if (pr > thr && pr < lo) { lo = pr; li = i; }
  }
  reduce(lo, li, false);
  if (threadIdx.x == 0) {
    long long r = -1;
    if (s_val != INFINITY) {
      r = s_idx;
      for (int j = 0; j < n_special; ++j)
        if (special[j] == top) r = top;
    }
    out_tok[b] = r;
  }
}

void launch_xtc(const float* logits, int ld, int B, int V, const float* inv_temp, const float* threshold, const unsigned char* fire,
                const int* special, int n_special, long long* out_tok, cudaStream_t st) {
  if (B == 0) return;
  launch_pdl(xtc_kernel, dim3(B), dim3(1024), 0, st, logits, ld, V, inv_temp, threshold, fire, special, n_special, out_tok);
}

// ------------------------------------------------------------------------------------------------ log-probabilities
// One CTA per row: log-sum-exp of the row, the log-probability of the chosen token and the `top_n` most probable tokens (value
// descending, first index on ties) with their log-probabilities. Reference: core/.../model/AbstractGeneratorSampler.java:135-155,
// tensor/.../VectorTensorMathUtils.java:91-107.
__global__ void __launch_bounds__(1024) logprob_kernel(const float* __restrict__ logits, int ld, int V, const long long* __restrict__ chosen,
                                                       int top_n, float* __restrict__ out_chosen, long long* __restrict__ out_idx,
                                                       float* __restrict__ out_val) {
  pdl_wait();
  pdl_trigger();
  __shared__ float red_f[32];
  __shared__ int red_i[32];
  __shared__ float s_val;
  __shared__ int s_idx;
  const int b = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const float* row = logits + static_cast<size_t>(b) * ld;
  float prev_v = INFINITY;
  int prev_i = -1;
  float lse = 0.f;
  for (int r = 0; r < (top_n < 1 ? 1 : top_n); ++r) {
    // the largest (value, -index) strictly behind the previous pick
    float v = -INFINITY;
    int vi = 0x7fffffff;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      const float x = row[i];
      const bool behind = x < prev_v || (x == prev_v && i > prev_i);
      if (behind && (x > v || (x == v && i < vi))) { v = x; vi = i; }
    }
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, v, o);
      const int oi = __shfl_xor_sync(0xffffffffu, vi, o);
      if (ov > v || (ov == v && oi < vi)) { v = ov; vi = oi; }
    }
    __syncthreads();
    if (lane == 0) { red_f[warp] = v; red_i[warp] = vi; }
    __syncthreads();
    if (warp == 0) {
      v = red_f[lane];
      vi = red_i[lane];
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, o);
        const int oi = __shfl_xor_sync(0xffffffffu, vi, o);
        if (ov > v || (ov == v && oi < vi)) { v = ov; vi = oi; }
      }
      if (lane == 0) { s_val = v; s_idx = vi; }
    }
    __syncthreads();
    prev_v = s_val;
    prev_i = s_idx;
    if (r == 0) {
      const float mx = prev_v;
      float sum = 0.f;
      if (mx != -INFINITY)
        for (int i = threadIdx.x; i < V; i += blockDim.x) sum += __expf(row[i] - mx);
      sum = warp_sum(sum);
      __syncthreads();
      if (lane == 0) red_f[warp] = sum;
      __syncthreads();
      sum = 0.f;
      for (int w = 0; w < 32; ++w) sum += red_f[w];
      lse = mx + logf(sum);
      if (threadIdx.x == 0) out_chosen[b] = row[chosen[b]] - lse;
    }
    if (top_n > 0 && threadIdx.x == 0) {
      out_idx[static_cast<size_t>(b) * top_n + r] = prev_i == 0x7fffffff ? -1 : prev_i;
      out_val[static_cast<size_t>(b) * top_n + r] = prev_v - lse;
    }
  }
}

void launch_logprobs(const float* logits, int ld, int B, int V, const long long* chosen, int top_n, float* out_chosen, long long* out_idx,
                     float* out_val, cudaStream_t st) {
  if (B == 0) return;
  launch_pdl(logprob_kernel, dim3(B), dim3(1024), 0, st, logits, ld, V, chosen, top_n, out_chosen, out_idx, out_val);
}

void launch_sample(const float* logits, int ld, int B, int V, const float* inv_temp, const long long* limits, const float* top_p,
                   const unsigned char* uniform, const float* us, long long* out_tok, int* out_ok, cudaStream_t st) {
  if (B == 0) return;
  static PerDeviceOnce attr_once;
  if (attr_once.first()) cudaFuncSetAttribute(sample_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(sizeof(SampShared)));
  launch_pdl(sample_kernel, dim3(B), dim3(1024), sizeof(SampShared), st, logits, ld, V, inv_temp, limits, top_p, uniform, us, out_tok, out_ok);
}

void launch_argmax(const float* logits, int ld, int B, int V, const uint32_t* mask, int mask_ld, float softcap, float inv_scale,
                   long long* out_idx, float* out_val, cudaStream_t st) {
  if (B == 0) return;
  if (V >= 32768 && B <= kArgmaxRows && B * 2 <= 296) {  // few long rows: split each row over several CTAs
    launch_pdl(argmax_part_kernel, dim3(B, kArgmaxSeg), dim3(512), 0, st, logits, ld, V, mask, mask_ld);
    launch_pdl(argmax_final_kernel, dim3(B), dim3(32), 0, st, logits, ld, softcap, inv_scale, out_idx, out_val);
    return;
  }
  launch_pdl(argmax_kernel, dim3(B), dim3(1024), 0, st, logits, ld, V, mask, mask_ld, softcap, inv_scale, out_idx, out_val);
}
void launch_logits_post(float* logits, int ld, int B, int V, const uint32_t* mask, int mask_ld, float softcap, float inv_scale,
                        cudaStream_t st) {
  if (B == 0) return;
  dim3 grid((V + 255) / 256, B);
  logits_post_kernel<<<grid, 256, 0, st>>>(logits, ld, V, mask, mask_ld, softcap, inv_scale);
}

}  // namespace dlv
