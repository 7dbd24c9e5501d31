// tcgen05 / TMEM / TMA backward of MoDA over the sequence keys as ONE key-stationary kernel that
// executes the five matmuls of the algorithm once each (D = 128, bf16 or fp16):
//
//     S^T = K Q^T,  dP^T = V dO^T,  dV += P^T dO,  dK += dS^T Q,  dQ^T = K^T dS^T
//
// The reference (moda_v14.py:1609,1658-1828) and the two-kernel backward of tc_bwd_kernels.cuh
// compute S and dP twice - once in a query-parallel dq kernel, once in a key-parallel dk/dv kernel -
// i.e. seven matmuls for five.  Here a CTA owns 128 sequence keys of one (batch, KV head), walks the
// 64-row query steps that can see them exactly like dkv_kernel, and additionally forms each step's
// contribution to dQ.  That contribution leaves the SM every step, and the contributions of all key
// tiles to one query row have to be summed in global memory.  Floating-point atomics would make the
// result depend on the order in which CTAs happen to run; instead the partial sums are FIXED-POINT:
// every 64-row query block has a power-of-two scale 2^e chosen from a bound on its rows' |dQ| so
// that the scaled values fit 30 bits, each contribution is rounded to int32 once and added with an
// integer bulk reduction (cp.reduce.async.bulk ... add.s32).  Integer addition is associative, so the accumulated value - and with it dq -
// is bit-identical from run to run whatever the order.  The quantisation step is 2^-29 of the
// bound, far below the 16-bit rounding of dq.  A later pass (dq_kernel walking only the depth keys)
// adds the depth keys' share in fp32 and writes dq.
//
// Bound used for the scale of a query row i (computed by bound_kernel from exact quantities):
//   |dQ_i[d]| = |sum_j dS_ij K_j[d]| <= max_j|K_j[d]| * sum_j P_ij |dP_ij - delta_i|
//            <= Kmax * (max_j |dO_i . V_j| + |delta_i|) <= Kmax * (|dO_i| |V|max + |delta_i|)
// with the maxima over the sequence keys of the (batch, head), times a safety factor for the
// rounding of P and dS to 16 bits.
//
// Where this stands.  At T = 65536 (G = 4, D = 128, 8 KV heads) this kernel takes as long as the
// dq and dk/dv kernels together although it executes 5/7 of their matmuls: with one CTA per MMA
// (cta_group::1) every kernel here is bound by shared-memory bandwidth, not by the tensor pipe, and
// what decides the time is the bytes of shared memory moved per 128 x 64 block of scores.  Two
// kernels have 2 x 512 TMEM columns and keep Q, dO, K and V as TMEM operands; one kernel has 512,
// keeps V only, and additionally stages the dQ contribution through shared memory.  It is therefore
// an alternative (MODA_PATH_TCGEN05_FUSED_BWD), not the default.
//
// Warp roles as in dkv_kernel (TMA warp, score-MMA warp, update-MMA warp, two softmax warpgroups on
// alternate steps).  TMEM (512 columns): [0,64) S^T, [64,128) dP^T (one fp32 score stage),
// [128,256) dV, [256,384) dK, [384,448) V rows as the 16-bit A operand of dP^T, [448,512) dQ^T
// (fp32, lanes = head dim, columns = the step's 64 query rows).  K stays in shared memory: it is the
// K-major A operand of S^T and the MN-major A operand of dQ^T.  The warpgroup that formed dS^T of
// step j takes dQ^T(j) out of TMEM at the start of its next step (j + 2), scales, rounds and adds it
// to the accumulator; the update warp issues dQ^T(j + 1) only after that read (one TMEM block).
#pragma once
#include "tc_bwd_kernels.cuh"

namespace moda {
namespace tc {

constexpr int kFuRing = 3;                                  // ring of {Q, dO, lse, delta, scale} step slots
constexpr uint32_t kFuStat = 768;                           // 64 lse, 64 delta, one float4 {scale, 1/scale, -, -}
struct FuBars {   // barrier indices
  static constexpr int res = 0, kfull = 1, full0 = 2, empty0 = 2 + kFuRing, s0 = 2 + 2 * kFuRing, p0 = s0 + 2,
                       r0 = p0 + 2, t0 = r0 + 2, done = t0 + 2, qfree = done + 1, ws0 = qfree + 1, qd0 = ws0 + 2, count = qd0 + 2;
};
static_assert(FuBars::count <= kMaxBars, "control block too small");
constexpr uint32_t kFuSmem = kTileBytes + kFuRing * 2 * step_tile<128>() + 2 * kDkvPairBytes + kFuRing * kFuStat + kCtlBytes;

// Instruction descriptor with both operand layouts selectable (bit 15: A is MN-major, bit 16: B is).
__host__ __device__ constexpr uint32_t instr_desc_ab(uint32_t fmt, uint32_t n, bool a_mn_major, bool b_mn_major) {
  return (1u << 4) | (fmt << 7) | (fmt << 10) | ((a_mn_major ? 1u : 0u) << 15) | ((b_mn_major ? 1u : 0u) << 16) |
         ((n >> 3) << 17) | ((128u >> 4) << 24);
}

// ------------------------------------------------------------------ bounds for the fixed-point scale
// kvmax[2 (b H + h)] = max_j |V_j|^2, kvmax[.. + 1] = max_{j,d} |K_j[d]| over the sequence keys, as
// the bit patterns of non-negative floats (atomicMax on them as integers is exact and
// order-independent).  Eight lanes per row, 32 rows per block iteration.
template <typename T>
__global__ void __launch_bounds__(256) kvmax_kernel(const __grid_constant__ Params p, int* kvmax) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, sub = lane & 7, grp = lane >> 3;
  const uint32_t groups_per_bh = ((uint32_t)p.T_kv + 31u) / 32u;
  const int64_t n_groups = (int64_t)p.B * p.H * groups_per_bh;
  for (int64_t gidx = blockIdx.x; gidx < n_groups; gidx += gridDim.x) {
    const uint32_t bh = (uint32_t)(gidx / groups_per_bh);
    const int j = (int)((uint32_t)(gidx - (int64_t)bh * groups_per_bh) * 32u) + w * 4 + grp;
    const int b = (int)(bh / (uint32_t)p.H), h = (int)(bh % (uint32_t)p.H);
    float v2 = 0.f, ka = 0.f;
    if (j < p.T_kv) {
      const T* pk = reinterpret_cast<const T*>(p.k.ptr) + p.k.off(b, j, h);
      const T* pv = reinterpret_cast<const T*>(p.v.ptr) + p.v.off(b, j, h);
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const uint4 k4 = *reinterpret_cast<const uint4*>(pk + 64 * i + sub * 8);
        const uint4 v4 = *reinterpret_cast<const uint4*>(pv + 64 * i + sub * 8);
        const uint32_t kw[4] = {k4.x, k4.y, k4.z, k4.w}, vw[4] = {v4.x, v4.y, v4.z, v4.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 x = Pack<T>::unpack(kw[e]), y = Pack<T>::unpack(vw[e]);
          ka = fmaxf(ka, fmaxf(fabsf(x.x), fabsf(x.y)));
          v2 = fmaf(y.x, y.x, fmaf(y.y, y.y, v2));
        }
      }
    }
    v2 += __shfl_xor_sync(0xffffffffu, v2, 1);
    v2 += __shfl_xor_sync(0xffffffffu, v2, 2);
    v2 += __shfl_xor_sync(0xffffffffu, v2, 4);
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      v2 = fmaxf(v2, __shfl_xor_sync(0xffffffffu, v2, o));
      ka = fmaxf(ka, __shfl_xor_sync(0xffffffffu, ka, o));
    }
    if (lane == 0) {
      if (!(v2 == v2) || v2 > 3.0e38f) v2 = 3.0e38f;       // NaN / inf inputs: keep the word an ordered, finite float
      if (!(ka == ka) || ka > 3.0e38f) ka = 3.0e38f;
      atomicMax(&kvmax[2 * bh], __float_as_int(v2));
      atomicMax(&kvmax[2 * bh + 1], __float_as_int(ka));
    }
  }
}

// scale_blk[(b H + h) * T_qp / 64 + blk] = {2^e, 2^-e, 0, 0} for the 64-row query block blk, with
// 2^e * (bound of any of its rows) < 2^29.  One warp per block; norm_t holds |dO_i| (pre_kernel).
__global__ void __launch_bounds__(256) scale_kernel(const float* delta_t, const float* norm_t, const int* kvmax,
                                                    float4* scale_blk, int T_qp, int64_t n_blk) {
  const int lane = threadIdx.x & 31;
  const int blocks_per_bh = T_qp / 64;
  const int64_t wstride = (int64_t)gridDim.x * (blockDim.x >> 5);
  for (int64_t idx = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); idx < n_blk; idx += wstride) {
    const int64_t bh = idx / blocks_per_bh;
    const int blk = (int)(idx % blocks_per_bh);
    const float vmax = sqrtf(__int_as_float(kvmax[2 * bh])), kmax = __int_as_float(kvmax[2 * bh + 1]);
    const int64_t r0 = bh * T_qp + (int64_t)blk * 64;        // rows past T_q hold zeros
    float bound = fmaxf((norm_t[r0 + lane] * vmax + fabsf(delta_t[r0 + lane])) * kmax,
                        (norm_t[r0 + 32 + lane] * vmax + fabsf(delta_t[r0 + 32 + lane])) * kmax);
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) bound = fmaxf(bound, __shfl_xor_sync(0xffffffffu, bound, o));
    if (lane == 0) {
      bound *= 1.25f;                                   // P and dS are rounded to 16 bits before the matmuls
      int ex = -60;
      if (bound > 0.f && bound < 3.0e38f) frexpf(bound, &ex);
      else if (bound > 0.f || !(bound == bound)) ex = 128;
      int e = 29 - ex;                                  // bound < 2^ex  =>  bound * 2^e < 2^29
      e = max(-96, min(96, e));
      scale_blk[idx] = make_float4(ldexpf(1.f, e), ldexpf(1.f, -e), 0.f, 0.f);
    }
  }
}

// =========================================================================== fused backward
// grid (ceil(T_kv/128), H, B), 352 threads.
template <typename T>
__global__ void __launch_bounds__(kFusedBwdThreads, 1)
bwd_fused_kernel(const __grid_constant__ Params p, const __grid_constant__ DkvMaps maps, const float* delta_t,
                 const float* lse_t, const float4* scale_blk, int* dq_acc, int T_qp) {
  constexpr int D = 128;
  constexpr int R = kFuRing;
  using B_ = FuBars;
  constexpr uint32_t kStepTile = step_tile<D>();
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  const uint32_t base = smem_u32(smem_raw);
  if (base & 1023u) {
    if (threadIdx.x == 0) record_failure(2 << 8);
    return;
  }
  const uint32_t sK = base;                                   // [128 keys x 128] K tile, resident
  const uint32_t ring_off = kTileBytes;
  const uint32_t sRing = base + ring_off;
  const uint32_t pt_off = ring_off + R * 2 * kStepTile;
  const uint32_t sPT = base + pt_off;
  const uint32_t stat_off = pt_off + 2 * kDkvPairBytes;
  const uint32_t sStat = base + stat_off;
  const uint32_t ctl_off = stat_off + R * kFuStat;
  const uint32_t bars = base + ctl_off;
  unsigned char* gctl = smem_raw + ctl_off;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gctl + 8 * kMaxBars);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gctl + 8 * kMaxBars + 4);
  volatile int* drain_flag = reinterpret_cast<volatile int*>(gctl + 8 * kMaxBars + 8);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (*reinterpret_cast<volatile int*>(&g_tc_status) != 0) return;

  const int h = blockIdx.y, b = blockIdx.z;
  const int c0 = (int)blockIdx.x * kBN;        // key tile 0 is seen by every query row: heaviest tiles first
  const int n_keys = p.T_kv;
  const int c_last = min(c0 + kBN, n_keys) - 1;

  // query rows that can see a key of this tile: [q_begin, T_q), walked in steps of 64
  int q_begin = (p.mode == kNonCausal) ? 0 : c0 * p.G;
  q_begin = (q_begin / kStep) * kStep;
  const int n = (p.T_q - q_begin + kStep - 1) / kStep;

  if (tid == 0) {
    mbar_init(bars + 8 * B_::res, 128);
    mbar_init(bars + 8 * B_::kfull, 1);
    mbar_init(bars + 8 * B_::done, 1);
    mbar_init(bars + 8 * B_::qfree, 128);
    for (int i = 0; i < R; ++i) { mbar_init(bars + 8 * (B_::full0 + i), 1); mbar_init(bars + 8 * (B_::empty0 + i), 1); }
    for (int i = 0; i < 2; ++i) {
      mbar_init(bars + 8 * (B_::s0 + i), 1); mbar_init(bars + 8 * (B_::p0 + i), 128);
      mbar_init(bars + 8 * (B_::r0 + i), 128); mbar_init(bars + 8 * (B_::t0 + i), 1);
      mbar_init(bars + 8 * (B_::ws0 + i), 128);
      mbar_init(bars + 8 * (B_::qd0 + i), 1);
    }
    *abort_flag = 0;
    *drain_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 0) {
    tmem_alloc(bars + 8 * kMaxBars, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tmem_S = tmem, tmem_P = tmem + 64, tmem_dV = tmem + 128, tmem_dK = tmem + 256;
  const uint32_t tmem_V = tmem + 384, tmem_dQ = tmem + 448;
  constexpr uint32_t fmt = std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;
  const int64_t stat_base = ((int64_t)b * p.H + h) * T_qp;
  const int64_t blk_base = ((int64_t)b * p.H + h) * (T_qp / 64);

  if (warp == 9) {
    // ---------------------------------------------------------------- TMA warp
    if (n > 0) {
      if (elect_one()) {
        prefetch_map(&maps.q); prefetch_map(&maps.dout); prefetch_map(&maps.k);
        mbar_expect_tx(bars + 8 * B_::kfull, kTileBytes);
        tma_load_tile<D>(sK, &maps.k, bars + 8 * B_::kfull, kHalfBytes, h, c0, b);
      }
      __syncwarp();
      bool ok = true;
      int issued = 0;
      for (int i = 0; ok && i < n; ++i) {
        const uint32_t slot = i % R;
        if (i >= R && !(ok = mbar_wait(bars + 8 * (B_::empty0 + slot), ((i / R) - 1) & 1, abort_flag, B_::empty0 + slot))) break;
        const int row = q_begin + i * kStep;
        const uint32_t dst = sRing + slot * 2 * kStepTile, bar = bars + 8 * (B_::full0 + slot);
        const uint32_t st = sStat + slot * kFuStat;
        if (elect_one()) {
          mbar_expect_tx(bar, 2 * kStepTile + 512 + 16);
          tma_load_tile<D>(dst, &maps.q, bar, kStepHalf, h, row, b);
          tma_load_tile<D>(dst + kStepTile, &maps.dout, bar, kStepHalf, h, row, b);
          bulk_load(st, lse_t + stat_base + row, 256, bar);
          bulk_load(st + 256, delta_t + stat_base + row, 256, bar);
          bulk_load(st + 512, scale_blk + blk_base + row / kStep, 16, bar);
        }
        __syncwarp();
        issued = i + 1;
      }
      // every load issued must have landed before the CTA's shared memory is released
      mbar_wait(bars + 8 * B_::kfull, 0, drain_flag, B_::kfull);
      if (!ok) {
        for (int i = max(0, issued - R); i < issued; ++i)
          mbar_wait(bars + 8 * (B_::full0 + i % R), (i / R) & 1, drain_flag, B_::full0 + i % R);
      }
    }
  } else if (warp == 8) {
    // ---------------------------------------------------------------- score-MMA warp
    // S^T(i) = K Q(i)^T (A = K in shared memory) and dP^T(i) = V dO(i)^T (A = V in TMEM) into the
    // score stage, as soon as the previous step's scores are in registers and the step tiles landed.
    if (n > 0) {
      constexpr uint32_t idesc_s = instr_desc(fmt, 64, false);
      bool ok = mbar_wait(bars + 8 * B_::res, 0, abort_flag, B_::res);        // V is in TMEM
      if (ok) ok = mbar_wait(bars + 8 * B_::kfull, 0, abort_flag, B_::kfull); // K is in shared memory
      tc_fence_after();
      const uint64_t dka = desc_kmajor(sK);
      for (int i = 0; ok && i < n; ++i) {
        const uint32_t slot = i % R;
        if (i >= 1 && !(ok = mbar_wait(bars + 8 * (B_::r0 + ((i - 1) & 1)), ((i - 1) >> 1) & 1, abort_flag, B_::r0 + ((i - 1) & 1)))) break;
        if (!(ok = mbar_wait(bars + 8 * (B_::full0 + slot), (i / R) & 1, abort_flag, B_::full0 + slot))) break;
        tc_fence_after();
        const uint32_t sQ = sRing + slot * 2 * kStepTile;
        const uint64_t dq = desc_kmajor(sQ), ddo = desc_kmajor(sQ + kStepTile);
        if (elect_one()) {
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk) {
            mma_ss(tmem_S, desc_add(dka, (kk >> 2) * kHalfBytes + (kk & 3) * 32), desc_add(dq, (kk >> 2) * kStepHalf + (kk & 3) * 32), idesc_s, kk > 0);
            mma_ts(tmem_P, tmem_V + kk * 8, desc_add(ddo, (kk >> 2) * kStepHalf + (kk & 3) * 32), idesc_s, kk > 0);
          }
          tc_commit(bars + 8 * (B_::s0 + (i & 1)));
        }
        __syncwarp();
      }
    }
  } else if (warp == 10) {
    // ---------------------------------------------------------------- update-MMA warp
    // dV += P^T(j) dO(j), dK += dS^T(j) Q(j) (A = tiles written by warpgroup j & 1, B = the step tiles
    // read MN-major), then dQ^T(j) = K^T dS^T(j) (A = K tile read MN-major, B = the dS^T tile read
    // MN-major) into the single dQ^T block once warpgroup (j - 1) & 1 has taken dQ^T(j - 1) out of it.
    if (n > 0) {
      constexpr uint32_t idesc_t = instr_desc(fmt, D, true);
      constexpr uint32_t idesc_q = instr_desc_ab(fmt, 64, true, true);
      const uint64_t dkt = desc_mnmajor(sK, kHalfBytes);
      bool ok = mbar_wait(bars + 8 * B_::kfull, 0, abort_flag, B_::kfull);     // K is in shared memory
      for (int j = 0; ok && j < n; ++j) {
        if (!(ok = mbar_wait(bars + 8 * (B_::p0 + (j & 1)), (j >> 1) & 1, abort_flag, B_::p0 + (j & 1)))) break;
        tc_fence_after();
        const uint32_t slot = j % R, sQ = sRing + slot * 2 * kStepTile;
        const uint64_t dq = desc_mnmajor(sQ, kStepHalf), ddo = desc_mnmajor(sQ + kStepTile, kStepHalf);
        const uint32_t pair = sPT + (j & 1) * kDkvPairBytes;
        const uint64_t dpt = desc_kmajor(pair), dst = desc_kmajor(pair + kScoreTile);
        const uint64_t dsb = desc_mnmajor(pair + kScoreTile, kScoreTile);
        // dQ^T first: while dV / dK of this step run, the warpgroup takes dQ^T(j) out of TMEM, so the
        // block is free again by the time the next step's dQ^T is issued
        if (j >= 1 && !(ok = mbar_wait(bars + 8 * B_::qfree, (j - 1) & 1, abort_flag, B_::qfree))) break;
        tc_fence_after();
        if (elect_one()) {
#pragma unroll
          for (int kk = 0; kk < 8; ++kk)
            mma_ss(tmem_dQ, desc_add(dkt, kk * 2048), desc_add(dsb, kk * 2048), idesc_q, kk > 0);
          tc_commit(bars + 8 * (B_::qd0 + (j & 1)));      // dQ^T(j) is complete
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) {
            mma_ss(tmem_dV, desc_add(dpt, kk * 32), desc_add(ddo, kk * 2048), idesc_t, (j > 0 || kk > 0) ? 1u : 0u);
            mma_ss(tmem_dK, desc_add(dst, kk * 32), desc_add(dq, kk * 2048), idesc_t, (j > 0 || kk > 0) ? 1u : 0u);
          }
          tc_commit(bars + 8 * (B_::empty0 + slot));      // ring slot j may be refilled
          tc_commit(bars + 8 * (B_::t0 + (j & 1)));       // tile pair j & 1 may be rewritten
          if (j == n - 1) tc_commit(bars + 8 * B_::done);
        }
        __syncwarp();
      }
    }
  } else {
    // ---------------------------------------------------------------- softmax warpgroups
    const int wg = warp >> 2, quarter = warp & 3;   // warpgroup g takes steps i with (i & 1) == g
    const int row = quarter * 32 + lane;             // key row of the tile == TMEM lane == head-dim index of dQ^T
    const int key = c0 + row;
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    if (wg == 1) {   // stage this thread's V row into TMEM as the A operand of dP^T
      uint32_t regs[D / 2];
      if (key < n_keys) {
        const uint4* g4 = reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(p.v.ptr) + p.v.off(b, key, h));
#pragma unroll
        for (int i = 0; i < D / 8; ++i) {
          const uint4 v4 = g4[i];
          regs[4 * i] = v4.x; regs[4 * i + 1] = v4.y; regs[4 * i + 2] = v4.z; regs[4 * i + 3] = v4.w;
        }
      } else {
#pragma unroll
        for (int i = 0; i < D / 2; ++i) regs[i] = 0u;
      }
      tmem_st32<0>(tmem_V + lane_addr, regs);
      tmem_st32<32>(tmem_V + lane_addr + 32, regs);
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(bars + 8 * B_::res);
    }
    // query rows [rlo, rhi) that see this key (the visibility rule of common.cuh, inverted)
    int rlo = 0, rhi = 0;
    if (key < n_keys) { rlo = (p.mode == kNonCausal) ? 0 : key * p.G; rhi = p.T_q; }
    // a step [q0, q0+64) needs no mask iff every valid key of the tile sees all 64 rows
    const int tile_rlo_max = (p.mode == kNonCausal) ? 0 : c_last * p.G;
    const bool tail_keys = (c0 + kBN > n_keys);
    const float c = p.scale_log2;
    bool ok = true;
    float esc_prev = 0.f;     // fixed-point scale of this warpgroup's previous step
    uint32_t wphase = 0;      // phase of this warpgroup's own barrier
    // All 128 threads of the warpgroup meet (a bounded mbarrier wait, like every other wait here: a
    // named bar.sync would spin forever if one warp of the group had left through the abort path).
    auto wg_sync = [&]() -> bool {
      mbar_arrive(bars + 8 * (B_::ws0 + wg));
      const bool r = __all_sync(0xffffffffu, mbar_wait(bars + 8 * (B_::ws0 + wg), wphase & 1, abort_flag, B_::ws0 + wg));
      ++wphase;
      return r;
    };

    // dQ^T of step j (this warpgroup's previous step): out of TMEM, scaled and rounded to int32,
    // transposed into [64 query rows][128] in shared memory - the warpgroup's own P^T / dS^T tile
    // pair, which update(j) has finished reading and which is exactly 32 KB - and added to the
    // accumulator rows with ONE bulk reduction (an L2-side integer add of 32 KB).
    auto dq_out = [&](int j, float esc) -> bool {
      if (!__all_sync(0xffffffffu, mbar_wait(bars + 8 * (B_::qd0 + (j & 1)), (j >> 1) & 1, abort_flag, B_::qd0 + (j & 1)))) return false;
      tc_fence_after();
      uint32_t qv[64];
      tmem_ld32<0>(tmem_dQ + lane_addr, qv);
      tmem_ld32<32>(tmem_dQ + lane_addr + 32, qv);
      tmem_wait_ld();
      tc_fence_before();
      mbar_arrive(bars + 8 * B_::qfree);
      // the tile pair is the staging buffer: dV / dK of step j must have finished reading it
      if (!__all_sync(0xffffffffu, mbar_wait(bars + 8 * (B_::t0 + (j & 1)), (j >> 1) & 1, abort_flag, B_::t0 + (j & 1)))) return false;
      int* stage = reinterpret_cast<int*>(smem_raw + pt_off + (j & 1) * kDkvPairBytes);
#pragma unroll
      for (int q = 0; q < 64; ++q) stage[q * D + row] = __float2int_rn(__uint_as_float(qv[q]) * esc);
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      if (!wg_sync()) return false;
      if (quarter == 0 && lane == 0) {
        int* dst = dq_acc + (stat_base + q_begin + (int64_t)j * kStep) * D;
        asm volatile("cp.reduce.async.bulk.global.shared::cta.bulk_group.add.s32 [%0], [%1], %2;"
                     :: "l"(dst), "r"(sPT + (uint32_t)(j & 1) * kDkvPairBytes), "r"(kDkvPairBytes) : "memory");
        bulk_commit();
      }
      return true;
    };
    // the bulk reduction issued by dq_out must have read the tile pair before it is written again
    auto pair_free = [&]() -> bool {
      if (quarter == 0 && lane == 0) bulk_wait_read_all();
      return wg_sync();
    };

    for (int i = wg; i < n; i += 2) {
      if (i >= 2 && !(ok = dq_out(i - 2, esc_prev))) break;
      const uint32_t slot = i % R;
      ok = __all_sync(0xffffffffu, mbar_wait(bars + 8 * (B_::full0 + slot), (i / R) & 1, abort_flag, B_::full0 + slot));
      if (!ok) break;
      ok = __all_sync(0xffffffffu, mbar_wait(bars + 8 * (B_::s0 + (i & 1)), (i >> 1) & 1, abort_flag, B_::s0 + (i & 1)));
      if (!ok) break;
      tc_fence_after();
      const int q0 = q_begin + i * kStep;
      const bool masked = tail_keys || q0 < tile_rlo_max || q0 + kStep > p.T_q;
      const float4* st4 = reinterpret_cast<const float4*>(smem_raw + stat_off + slot * kFuStat);
      esc_prev = st4[32].x;
      uint32_t su[64], du[64];
      tmem_ld32<0>(tmem_S + lane_addr, su);
      tmem_ld32<32>(tmem_S + lane_addr + 32, su);
      tmem_ld32<0>(tmem_P + lane_addr, du);
      tmem_ld32<32>(tmem_P + lane_addr + 32, du);
      tmem_wait_ld();
      tc_fence_before();
      mbar_arrive(bars + 8 * (B_::r0 + (i & 1)));      // scores are in registers: the stage is free
      float pr[64], dd[64];
#pragma unroll
      for (int j4 = 0; j4 < 16; ++j4) {
        const float4 l4 = st4[j4], d4 = st4[16 + j4];
        pr[4 * j4 + 0] = fast_exp2(fmaf(__uint_as_float(su[4 * j4 + 0]), c, -l4.x));
        pr[4 * j4 + 1] = fast_exp2(fmaf(__uint_as_float(su[4 * j4 + 1]), c, -l4.y));
        pr[4 * j4 + 2] = fast_exp2(fmaf(__uint_as_float(su[4 * j4 + 2]), c, -l4.z));
        pr[4 * j4 + 3] = fast_exp2(fmaf(__uint_as_float(su[4 * j4 + 3]), c, -l4.w));
        dd[4 * j4 + 0] = __uint_as_float(du[4 * j4 + 0]) - d4.x;
        dd[4 * j4 + 1] = __uint_as_float(du[4 * j4 + 1]) - d4.y;
        dd[4 * j4 + 2] = __uint_as_float(du[4 * j4 + 2]) - d4.z;
        dd[4 * j4 + 3] = __uint_as_float(du[4 * j4 + 3]) - d4.w;
      }
      if (masked) {
#pragma unroll
        for (int jj = 0; jj < 64; ++jj) {
          const int rr = q0 + jj;
          pr[jj] = (rr >= rlo && rr < rhi) ? pr[jj] : 0.f;
        }
      }
      uint32_t pp[32], pd[32];
#pragma unroll
      for (int jj = 0; jj < 32; ++jj) {
        pp[jj] = Pack<T>::pack(pr[2 * jj], pr[2 * jj + 1]);
        pd[jj] = Pack<T>::pack(pr[2 * jj] * dd[2 * jj], pr[2 * jj + 1] * dd[2 * jj + 1]);
      }
      // the update of step i - 2 has finished reading this warpgroup's tile pair (dq_out waited for
      // it), and so has the reduction of dQ^T(i - 2) that was staged in it
      if (!(ok = pair_free())) break;
      {   // rows of the K-major, 128B-swizzled [128 x 64] tiles: 16-byte chunk c lives at chunk c ^ (row & 7)
        unsigned char* prow = smem_raw + pt_off + (i & 1) * kDkvPairBytes + row * 128;
#pragma unroll
        for (int ch = 0; ch < 8; ++ch) {
          const uint32_t o = (uint32_t)((ch ^ (row & 7)) << 4);
          *reinterpret_cast<uint4*>(prow + o) = make_uint4(pp[4 * ch], pp[4 * ch + 1], pp[4 * ch + 2], pp[4 * ch + 3]);
          *reinterpret_cast<uint4*>(prow + kScoreTile + o) = make_uint4(pd[4 * ch], pd[4 * ch + 1], pd[4 * ch + 2], pd[4 * ch + 3]);
        }
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      mbar_arrive(bars + 8 * (B_::p0 + (i & 1)));
    }
    // this warpgroup's last step still has its dQ^T in TMEM
    if (ok && n > wg) {
      const int j_last = ((n - 1 - wg) / 2) * 2 + wg;
      ok = dq_out(j_last, esc_prev);
    }
    if (quarter == 0 && lane == 0) bulk_wait_read_all();     // staged rows are read before the CTA's smem goes
    if (ok && n > 0) ok = __all_sync(0xffffffffu, mbar_wait(bars + 8 * B_::done, 0, abort_flag, B_::done));
    if (ok && n > 0) {
      tc_fence_after();
      const View& ov = (wg == 0) ? p.dv : p.dk;
      T* gout = reinterpret_cast<T*>(ov.ptr) + ov.off(b, key, h);
      const uint32_t tsrc = (wg == 0) ? tmem_dV : tmem_dK;      // warpgroup 0 stores dV, warpgroup 1 dK
      const float mul = (wg == 0) ? 1.f : p.scale;
#pragma unroll
      for (int q4 = 0; q4 < D / 32; ++q4) {
        uint32_t ov32[32];
        tmem_ld32<0>(tsrc + lane_addr + q4 * 32, ov32);
        tmem_wait_ld();
        if (key < n_keys) {
#pragma unroll
          for (int i = 0; i < 4; ++i) *reinterpret_cast<uint4*>(gout + q4 * 32 + i * 8) = pack8_scaled<T>(ov32 + i * 8, mul);
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

}  // namespace tc
}  // namespace moda
