// Stand-alone micro-benchmark of tcgen05.mma issue on sm_100a (zeros in shared memory; timing only, nothing is checked).
//   part 1: cycles per MMA for back-to-back instructions of several shapes and operand forms, issued by one elected thread;
//   part 2: cycles per group of 8 MMAs (128 x 128 x 16) when the issuing thread also commits to 0..4 mbarriers per group, or
//           waits between groups on a barrier that the previous group's commit completes.
// Build and run (one GPU):
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 -o /tmp/mma_issue_bench deliverance_b200/bench/mma_issue_bench.cu -lcuda
//   /tmp/mma_issue_bench
// Every wait is bounded (common.cuh); a wait that runs out is reported in the "ok" column.
#include <cstdio>
#include <cuda_runtime.h>
#include "../ops/csrc/common.cuh"
using namespace dlv;


__device__ __forceinline__ bool elect_one() {
  uint32_t pred = 0;
  asm volatile("{\n\t.reg .pred P;\n\telect.sync _|P, 0xffffffff;\n\tselp.u32 %0, 1, 0, P;\n\t}" : "=r"(pred));
  return pred != 0;
}
// accumulate always on: no predicate register set-up per instruction
__device__ __forceinline__ void mma_ss_acc(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.eq.u32 p, 1, 1;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d), "l"(a), "l"(b), "r"(idesc) : "memory");
}
__device__ __forceinline__ void mma_ts_acc(uint32_t d, uint32_t a, uint64_t b, uint32_t idesc) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.eq.u32 p, 1, 1;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d), "r"(a), "l"(b), "r"(idesc) : "memory");
}

template <int V>
__global__ void __launch_bounds__(128, 1) shape_kernel(int groups, long long* out, int* status) {
  extern __shared__ uint8_t raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~uintptr_t(1023));
  __shared__ uint64_t bar;
  __shared__ uint32_t slot;
  __shared__ int abort_flag;
  for (int i = threadIdx.x; i < 160 * 1024 / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(smem)[i] = 0;
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&bar), 1);
    abort_flag = 0;
    mbar_fence_init();
  }
  if (threadIdx.x < 32) tmem_alloc(smem_u32(&slot), 512);
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tm = slot;
  if (threadIdx.x < 32) {
    if (elect_one()) {
      const uint64_t da = umma_desc_k_sw128(smem_u32(smem));
      const uint64_t db = umma_desc_k_sw128(smem_u32(smem + 64 * 1024));
      constexpr uint32_t id128 = umma_idesc_bf16(128, 128), id256 = umma_idesc_bf16(128, 256), id64 = umma_idesc_bf16(128, 64);
      const long long t0 = clock64();
      for (int g = 0; g < groups; ++g) {
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          constexpr int dummy = 0;
          const uint64_t adv = static_cast<uint64_t>(((k >> 2) * (128 * 128) + (k & 3) * 32) >> 4);
          const uint64_t adv256 = static_cast<uint64_t>(((k >> 2) * (256 * 128) + (k & 3) * 32) >> 4);
          if (V == 0) mma_ss_acc(tm, da + adv, db + adv, id128);
          if (V == 1) mma_ss_acc(tm, da + adv, db + adv256, id256);
          if (V == 2) mma_ts_acc(tm, tm + 256 + k * 8, db + adv, id128);
          if (V == 3) mma_ss_acc(tm, da + adv, db + adv, id64);
          if (V == 4) mma_ts_acc(tm, tm + 256 + k * 8, db + adv256, id256);
          if (V == 5) mma_ss_acc(tm + (k & 3) * 128, da + adv, db + adv, id128);  // four accumulators in turn
          (void)dummy;
        }
      }
      const long long t_issue = clock64() - t0;
      umma_commit(smem_u32(&bar));
      const bool ok = mbar_wait(smem_u32(&bar), 0, &abort_flag, status);
      const long long t1 = clock64();
      if (blockIdx.x == 0) {
        out[0] = t1 - t0;
        out[1] = t_issue;
        out[2] = ok ? 1 : 0;
      }
    }
    __syncwarp();
  }
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x < 32) {
    tc_fence_after();
    tmem_dealloc(tm, 512);
  }
}

template <int V>
int run_shape(const char* name, long long* out, int* status) {
  cudaFuncSetAttribute(shape_kernel<V>, cudaFuncAttributeMaxDynamicSharedMemorySize, 162 * 1024);
  const int groups = 64;
  shape_kernel<V><<<148, 128, 162 * 1024>>>(groups, out, status);
  cudaError_t e = cudaDeviceSynchronize();
  long long h[3];
  cudaMemcpy(h, out, 24, cudaMemcpyDeviceToHost);
  printf("%-28s  cycles/mma %.1f  issue cycles/mma %.1f  ok %lld  (%s)\n", name, double(h[0]) / (groups * 8), double(h[1]) / (groups * 8), h[2], cudaGetErrorString(e));
  return e == cudaSuccess ? 0 : 1;
}



// C = commits per group (to distinct barriers nobody waits on), W = 1: after each group wait on a barrier that the previous group's commit completes
template <int C, int W>
__global__ void __launch_bounds__(128, 1) group_kernel(int groups, long long* out, int* status) {
  extern __shared__ uint8_t raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~uintptr_t(1023));
  __shared__ uint64_t bars[8];
  __shared__ uint64_t bar_end;
  __shared__ uint32_t slot;
  __shared__ int abort_flag;
  for (int i = threadIdx.x; i < 160 * 1024 / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(smem)[i] = 0;
  if (threadIdx.x == 0) {
    for (int i = 0; i < 8; ++i) mbar_init(smem_u32(&bars[i]), 1);
    mbar_init(smem_u32(&bar_end), 1);
    abort_flag = 0;
    mbar_fence_init();
  }
  if (threadIdx.x < 32) tmem_alloc(smem_u32(&slot), 512);
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tm = slot;
  if (threadIdx.x == 0) {
    const uint64_t da = umma_desc_k_sw128(smem_u32(smem)), db = umma_desc_k_sw128(smem_u32(smem + 64 * 1024));
    constexpr uint32_t id = umma_idesc_bf16(128, 128);
    bool ok = true;
    const long long t0 = clock64();
    for (int g = 0; g < groups && ok; ++g) {
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const uint64_t adv = static_cast<uint64_t>(((k >> 2) * (128 * 128) + (k & 3) * 32) >> 4);
        umma_bf16(tm + (g & 1) * 128, da + adv, db + adv, id, 1u);
      }
      if (W == 1 && g > 0) {
        // the commit of group g - 1 went to bars[0]: phase g - 1 (waited for before this group's commit, so at most one phase is open)
        ok = mbar_wait(smem_u32(&bars[0]), (g - 1) & 1, &abort_flag, status);
        tc_fence_after();
      }
#pragma unroll
      for (int c = 0; c < C; ++c) umma_commit(smem_u32(&bars[c]));
    }
    const long long t_issue = clock64() - t0;
    umma_commit(smem_u32(&bar_end));
    ok = ok && mbar_wait(smem_u32(&bar_end), 0, &abort_flag, status);
    const long long t1 = clock64();
    if (blockIdx.x == 0) {
      out[0] = t1 - t0;
      out[1] = t_issue;
      out[2] = ok ? 1 : 0;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x < 32) {
    tc_fence_after();
    tmem_dealloc(tm, 512);
  }
}

template <int C, int W>
int run_group(const char* name, long long* out, int* status) {
  cudaFuncSetAttribute(group_kernel<C, W>, cudaFuncAttributeMaxDynamicSharedMemorySize, 162 * 1024);
  const int groups = 64;
  group_kernel<C, W><<<148, 128, 162 * 1024>>>(groups, out, status);
  cudaError_t e = cudaDeviceSynchronize();
  long long h[3];
  cudaMemcpy(h, out, 24, cudaMemcpyDeviceToHost);
  printf("%-44s  cycles/group %.1f  (8 MMAs = 520 at full rate)  ok %lld  (%s)\n", name, double(h[0]) / groups, h[2], cudaGetErrorString(e));
  return e == cudaSuccess ? 0 : 1;
}

int main() {
  long long* out;
  int* status;
  cudaMalloc(&out, 64);
  cudaMalloc(&status, 4);
  cudaMemset(status, 0, 4);
  if (run_shape<0>("SS N128", out, status)) return 1;
  if (run_shape<1>("SS N256", out, status)) return 1;
  if (run_shape<2>("TS N128", out, status)) return 1;
  if (run_shape<3>("SS N64", out, status)) return 1;
  if (run_shape<4>("TS N256", out, status)) return 1;
  if (run_shape<5>("SS N128 four accumulators", out, status)) return 1;
  if (run_group<0, 0>("no commit", out, status)) return 1;
  if (run_group<1, 0>("1 commit per group", out, status)) return 1;
  if (run_group<2, 0>("2 commits per group", out, status)) return 1;
  if (run_group<4, 0>("4 commits per group", out, status)) return 1;
  if (run_group<1, 1>("1 commit + wait for the previous group", out, status)) return 1;
  return 0;
}
