// Micro-benchmark: how often one thread can issue tcgen05.mma (cta_group::1), for
// kind::f16 and kind::f8f6f4, M in {64, 128}, N in {16 .. 256}, with one or two independent
// accumulators and one or two issuing warps. One CTA, operands are zero-filled shared memory, 4096 instructions per case.
//
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 --expt-relaxed-constexpr \
//        -I arcticinference_b200/csrc benchmarks/mma_issue_rate.cu -o /tmp/mma_issue_rate
//   /tmp/mma_issue_rate
//
// Result on B200: 185-186 SM cycles per instruction in every case, so a k-loop whose
// instructions carry little work (few columns) is bound by instruction count, not by bytes.
#include <cstdio>
#include <cuda_runtime.h>
#include "common/ptx.cuh"
using namespace ab200;

__global__ void __launch_bounds__(128, 1)
rate_kernel(int m, int n, int fp8, int reps, int chains, int issuers, long long* out, int* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  __shared__ uint64_t bar[4];
  __shared__ uint32_t slot;
  __shared__ int abort_flag;
  for (int i = threadIdx.x; i < (16384 + 32768) / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(smem)[i] = 0;
  if (threadIdx.x == 0) { for (int i = 0; i < 4; ++i) mbar_init(smem_u32(&bar[i]), 1); abort_flag = 0; fence_barrier_init(); }
  if (threadIdx.x < 32) { tmem_alloc(smem_u32(&slot), 512); tmem_relinquish(); }
  fence_proxy_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tm = slot;
  const int who = threadIdx.x >> 5;
  if ((threadIdx.x & 31) == 0 && who < issuers) {
    const uint32_t idesc = make_idesc(m, n, fp8 ? 0 : 1, fp8 ? 0 : 1, 0, 0);
    const uint64_t ad = make_desc_kmajor_sw128(smem_u32(smem));
    const uint64_t bd = make_desc_kmajor_sw128(smem_u32(smem) + 16384);
    const long long t0 = clock64();
    for (int i = 0; i < reps; ++i) {
      const uint32_t d = tm + (uint32_t)(who * chains + i % chains) * (uint32_t)n;
      if (fp8) umma_f8_ss(d, ad + 2u * (i & 3), bd + 2u * (i & 3), idesc, i >= chains);
      else umma_f16_ss(d, ad + 2u * (i & 3), bd + 2u * (i & 3), idesc, i >= chains);
    }
    const long long t1 = clock64();
    tc_commit(smem_u32(&bar[who]));
    mbar_wait(smem_u32(&bar[who]), 0, &abort_flag, status, 9000, 0);
    const long long t2 = clock64();
    out[2 * who] = t1 - t0;
    out[2 * who + 1] = t2 - t0;
  }
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x < 32) { tc_fence_after(); tmem_dealloc(tm, 512); }
}

int main() {
  long long* out; int* status;
  cudaMalloc(&out, 64); cudaMalloc(&status, 64); cudaMemset(status, 0, 64);
  cudaFuncSetAttribute(rate_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024);
  const int reps = 4096;
  for (int fp8 = 0; fp8 < 2; ++fp8)
    for (int m : {64, 128})
      for (int n : {16, 32, 64, 128, 256})
        for (int chains : {1, 2})
          for (int issuers : {1, 2}) {
            if (issuers * chains * n > 512) continue;
            for (int w = 0; w < 2; ++w)
              rate_kernel<<<1, 128, 64 * 1024>>>(m, n, fp8, reps, chains, issuers, out, status);
            cudaError_t e = cudaDeviceSynchronize();
            long long h[4]; cudaMemcpy(h, out, 32, cudaMemcpyDeviceToHost);
            int st[8]; cudaMemcpy(st, status, 32, cudaMemcpyDeviceToHost);
            // cycles per instruction seen by issuing thread 0; with two issuing warps the SM
            // retires two instructions in that time
            printf("%s M=%3d N=%3d chains=%d issuers=%d: issue %.1f, complete %.1f cycles per instruction per issuer (err %d status %d)\n",
                   fp8 ? "f8 " : "f16", m, n, chains, issuers, (double)h[0] / reps, (double)h[1] / reps,
                   (int)e, st[0]);
          }
  return 0;
}
