// Measured issue-to-completion rate of tcgen05.mma (kind::f16, bf16 operands, M = 128, K = 16) on
// this GPU, for the instruction shapes the attention kernels use.
//
// The tensor pipe does not run every shape at the nominal 8192 flop/clock/SM: an instruction
// carries a fixed cost of about a dozen clocks, and an A operand read from shared memory (the SS
// form) is fetched before the math starts instead of under it.  TMEM's 512 columns decide which
// shapes a kernel can afford (score blocks of N = 64 or 128, update matmuls with A in shared
// memory), so the honest ceiling of a kernel is the sum of these measured instruction times over
// the instructions it has to execute per tile, not the nominal peak.  This probe measures them:
// one CTA, one issuing warp, kProbeMmas back-to-back instructions accumulating into one TMEM block,
// clock() from the first issue to the arrival of the tcgen05.commit.  Operands are zeros (timing
// does not depend on the data).  Every wait is bounded.
#pragma once
#include "tc_kernels.cuh"

namespace moda {
namespace tc {

constexpr int kProbeMmas = 64;
constexpr uint32_t kProbeSmem = 16384 + 32768 + 1024;   // A tile [128 x 64], B tile [256 x 64], alignment

template <int N, bool kTs>
__global__ void __launch_bounds__(128, 1) mma_rate_kernel(float* out) {
  extern __shared__ __align__(1024) unsigned char probe_smem[];
  __shared__ __align__(8) unsigned long long bar;
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  const uint32_t base = (smem_u32(probe_smem) + 1023u) & ~1023u;
  unsigned char* gbase = probe_smem + (base - smem_u32(probe_smem));
  const uint32_t sA = base, sB = base + 16384, bar_addr = smem_u32(&bar);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < (16384 + 32768) / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(gbase)[i] = 0u;
  if (threadIdx.x == 0) {
    mbar_init(bar_addr, 1);
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 0) {
    tmem_alloc(smem_u32(&tmem_slot), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_slot;
  const uint32_t tD = tmem, tA = tmem + 448;             // accumulator [0, N), 16-bit A operand [448, 512)
  {                                                       // zero the A operand: thread = TMEM lane
    uint32_t z[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) z[i] = 0u;
    const uint32_t lane_addr = (uint32_t)(warp * 32) << 16;
    tmem_st32<0>(tA + lane_addr, z);
    tmem_st32<0>(tA + lane_addr + 32, z);
    tmem_wait_st();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 0) {
    constexpr uint32_t idesc = instr_desc(1u, N, false);
    const unsigned t0 = clock();
    if (elect_one()) {
      for (int i = 0; i < kProbeMmas; i += 4) {
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
          if (kTs) mma_ts(tD, tA + kk * 8, smem_desc_sw128(sB + kk * 32, 16, 1024), idesc, 1u);
          else mma_ss(tD, smem_desc_sw128(sA + kk * 32, 16, 1024), smem_desc_sw128(sB + kk * 32, 16, 1024), idesc, 1u);
        }
      }
      tc_commit(bar_addr);
    }
    __syncwarp();
    const bool ok = mbar_wait(bar_addr, 0, &abort_flag, 0);
    const unsigned t1 = clock();
    if (lane == 0) *out = ok ? (float)(t1 - t0) / kProbeMmas : -1.f;
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

template <int N, bool kTs>
inline cudaError_t launch_mma_rate(float* out, cudaStream_t st) {
  auto kern = mma_rate_kernel<N, kTs>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kProbeSmem);
  if (e != cudaSuccess) return e;
  kern<<<1, 128, kProbeSmem, st>>>(out);   // twice: the first launch pays for instruction-cache misses
  kern<<<1, 128, kProbeSmem, st>>>(out);
  return cudaGetLastError();
}

// out (device, 6 floats): clocks per instruction for SS N = 64, 128, 256 and TS N = 64, 128, 256.
inline cudaError_t mma_rates(float* out, cudaStream_t st) {
  cudaError_t e;
  if ((e = launch_mma_rate<64, false>(out + 0, st)) != cudaSuccess) return e;
  if ((e = launch_mma_rate<128, false>(out + 1, st)) != cudaSuccess) return e;
  if ((e = launch_mma_rate<256, false>(out + 2, st)) != cudaSuccess) return e;
  if ((e = launch_mma_rate<64, true>(out + 3, st)) != cudaSuccess) return e;
  if ((e = launch_mma_rate<128, true>(out + 4, st)) != cudaSuccess) return e;
  return launch_mma_rate<256, true>(out + 5, st);
}

}  // namespace tc
}  // namespace moda
