// Tensor-pipe issue-rate microbenchmark: the B200 counterpart of the reference's VNNI peak probe
// (poc/vnni/micro.cc:16-51, which times back-to-back vpdpbusd on registers).  Every SM runs one
// CTA whose operands never leave shared memory; 1-4 threads (one per warp) each issue `iters`
// back-to-back tcgen05.mma of 128 x N x 32 bytes (kind::i8, u8 x s8 -> s32, or kind::f16 with fp32
// accumulation) into their own accumulator in tensor memory.  What comes out is the rate the
// tensor cores sustain when nothing but the MMA instruction stream limits them: the measured
// denominator for the roofline of the contraction kernels.
#pragma once
#include "igemm_sm100.cuh"

namespace unit {

constexpr int kPeakABufs = 4, kPeakBBufs = 2;
constexpr uint32_t kPeakABytes = 128u * 32u;  // one K step of A: 128 rows x 32 bytes
constexpr int kPeakThreads = 160;             // warps 0-3 issue, warp 4 owns the tensor memory

template <bool F16>
__global__ void __launch_bounds__(kPeakThreads, 1)
    tensor_peak_kernel(int n, int iters, int issuers, unsigned int *err, unsigned long long limit_ns) {
  extern __shared__ __align__(1024) uint8_t smem[];
  __shared__ uint32_t tbase;
  __shared__ unsigned long long bar;
  __shared__ int abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t b_bytes = (uint32_t)n * 32u;
  const uint32_t total = kPeakABufs * kPeakABytes + kPeakBBufs * b_bytes;
  // operand bytes: a hash of the position (varied data, so that the power drawn is that of real
  // operands); for fp16 every half-word is a finite value in +-[1, 2)
  for (uint32_t i = threadIdx.x; i < total / 4; i += blockDim.x) {
    uint32_t h = (i + 1u) * 2654435761u + blockIdx.x * 40503u;
    h ^= h >> 15; h *= 2246822519u; h ^= h >> 13;
    if (F16) h = (h & 0x83ff83ffu) | 0x3c003c00u;
    reinterpret_cast<uint32_t *>(smem)[i] = h;
  }
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&bar), (uint32_t)issuers);
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 4) {
    tmem_alloc(smem_u32(&tbase), 512);
    tmem_relinquish();
  }
  fence_proxy_async();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (lane == 0 && warp < issuers) {
    const uint32_t idesc = make_idesc<F16>(n, 0);
    const uint32_t base = smem_u32(smem);
    // K-major, no swizzle: the two 16-byte columns of a K step are 128 (A) or n (B) rows apart
    const uint64_t adesc0 = make_smem_desc(0u, 128u * 16u, 128u);
    const uint64_t bdesc0 = make_smem_desc(0u, (uint32_t)n * 16u, 128u);
    const uint32_t d_tmem = tbase + (uint32_t)warp * (uint32_t)n;
    for (int it = 0; it < iters; ++it) {
      const uint64_t ad = adesc0 | (uint64_t)((base + (uint32_t)(it & (kPeakABufs - 1)) * kPeakABytes) >> 4);
      const uint64_t bd = bdesc0 | (uint64_t)((base + kPeakABufs * kPeakABytes + (uint32_t)(it & (kPeakBBufs - 1)) * b_bytes) >> 4);
      tc_mma<F16>(d_tmem, ad, bd, idesc, it ? 1u : 0u);
    }
    tc_commit(smem_u32(&bar));
    const WaitCtx wc{&abort_flag, err, limit_ns};
    mbar_wait(smem_u32(&bar), 0u, wc, kErrWaitTmemFull);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 4) {
    tc_fence_after();
    tmem_dealloc(tbase, 512);
  }
}

// Runs the probe on every SM of the current device and returns operations per second
// (2 x 128 x N x K-elements per MMA) through *ops_per_second.  Synchronous: times one launch with
// CUDA events on `st`.  Returns a unit_status value.
static int run_tensor_peak(bool f16, int n, int issuers, int iters, unsigned int *err_word, double *ops_per_second,
                           cudaStream_t st) {
  if (n < 16 || n > 256 || n % 16 || issuers < 1 || issuers > 4 || issuers * n > 512 || iters < 1 || iters > (1 << 24) ||
      !ops_per_second)
    return -2;  // UNIT_ERR_SHAPE
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return -6;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (sms < 1) return -6;
  const size_t smem_bytes = kPeakABufs * kPeakABytes + kPeakBBufs * (size_t)n * 32;
  cudaEvent_t e0, e1;
  if (cudaEventCreate(&e0) != cudaSuccess || cudaEventCreate(&e1) != cudaSuccess) return -6;
  // a 10 s bound: the probe's own run time is iters x ~140 cycles
  const unsigned long long limit = 10000000000ull;
  cudaEventRecord(e0, st);
  if (f16) tensor_peak_kernel<true><<<sms, kPeakThreads, smem_bytes, st>>>(n, iters, issuers, err_word, limit);
  else tensor_peak_kernel<false><<<sms, kPeakThreads, smem_bytes, st>>>(n, iters, issuers, err_word, limit);
  const cudaError_t le = cudaGetLastError();
  cudaEventRecord(e1, st);
  const cudaError_t se = cudaEventSynchronize(e1);
  float ms = 0.f;
  cudaEventElapsedTime(&ms, e0, e1);
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  if (le != cudaSuccess || se != cudaSuccess || ms <= 0.f) return -6;
  const double k_elems = f16 ? 16.0 : 32.0;
  *ops_per_second = 2.0 * 128.0 * n * k_elems * (double)iters * issuers * sms / (ms * 1e-3);
  return 0;
}

}  // namespace unit
