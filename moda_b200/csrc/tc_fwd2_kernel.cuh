// tcgen05 / TMEM / TMA forward of MoDA, pipelined form (D = 128, bf16 or fp16).
//
// One CTA per SM owns 128 folded query rows of one (batch, KV head) and walks the keys they can
// see - sequence K/V, then the tile's depth K/V window - in tiles of 128 keys.
//
//   warp 10 (TMA)    keeps a ring of {K tile, V tile} full.
//   warp 8  (scores) S(i) = Q K(i)^T into TMEM stage i&1.  Q sits in TMEM as a 16-bit A operand
//                    for the whole CTA, so a score MMA reads only 4 KB of K from shared memory
//                    and runs at the tensor rate; S(i+1) is computed while the softmax warps work
//                    on S(i).
//   warps 0-7        softmax: thread pair (w, w+4) shares a query row = TMEM lane, each takes 64
//                    of the tile's 128 columns (and reads the partner's 64 for the row maximum).
//                    tcgen05.ld the scores, release the stage, exp2 with lazy rescaling
//                    (O is touched only when a row maximum grows by more than 2^8), write P as
//                    packed 16-bit pairs into the P buffer in TMEM.
//   warp 9  (PV)     O += P(i) V(i): A = P buffer in TMEM, B = V tile read MN-major.
//
// TMEM (512 columns): [0,128) and [128,256) score stages, [256,320) P buffer, [320,448) O (fp32),
// [448,512) Q.  Every wait is bounded, as in the other tcgen05 kernels.
#pragma once
#include "tc_bwd_kernels.cuh"

namespace moda {
namespace tc {

constexpr int kF2Ring = 3;
constexpr int kF2Threads = 352;
// barriers: res, full[R], empty[R], s[2], r[2], p[2], t[2], done
struct F2Bars {
  static constexpr int res = 0, full0 = 1, empty0 = 1 + kF2Ring, s0 = 1 + 2 * kF2Ring, r0 = s0 + 2, p0 = s0 + 4,
                       t0 = s0 + 6, done = s0 + 8, count = s0 + 9;
};
static_assert(F2Bars::count <= kMaxBars, "control block too small");
constexpr uint32_t kF2XchgBytes = 2 * 2 * 128 * 8;       // [parity][half][row] {value, tag} exchange slots
constexpr uint32_t kF2Smem = kF2Ring * 2 * kTileBytes + kF2XchgBytes + kCtlBytes;

struct Fwd2Maps { CUtensorMap k, v, kd, vd; };           // 128-row boxes

// Exchange one float per step between the two threads that share a query row (same TMEM lane
// quarter, different column half).  Slots are {tag, value} words written with one 8-byte store and
// double-buffered by step parity; the reader polls for the step's tag a bounded number of times
// (a named barrier would have no way out if the partner warp had given up on an expired wait).
__device__ __forceinline__ bool pair_exchange(volatile unsigned long long* xchg, int parity, int half, int row,
                                              uint32_t tag, float mine, float& theirs, volatile int* abort_flag) {
  xchg[(parity * 2 + half) * 128 + row] = ((unsigned long long)tag << 32) | __float_as_uint(mine);
  volatile unsigned long long* src = xchg + (parity * 2 + (half ^ 1)) * 128 + row;
  for (uint32_t spin = 0; spin < (1u << 24); ++spin) {
    const unsigned long long v = *src;
    if ((uint32_t)(v >> 32) == tag) { theirs = __uint_as_float((uint32_t)v); return true; }
    if ((spin & 255u) == 255u && *abort_flag != 0) return false;
  }
  *abort_flag = 1;
  atomicCAS(&g_tc_status, 0, (4 << 8));
  return false;
}
template <typename T, int kF2PolyEvery>
__global__ void __launch_bounds__(kF2Threads, 1)
fwd2_kernel(const __grid_constant__ Params p, const __grid_constant__ Fwd2Maps maps) {
  constexpr int R = kF2Ring;
  using B_ = F2Bars;
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  const uint32_t base = smem_u32(smem_raw);
  if (base & 1023u) {
    if (threadIdx.x == 0) atomicCAS(&g_tc_status, 0, (2 << 8));
    return;
  }
  const uint32_t sRing = base;
  const uint32_t xchg_off = R * 2 * kTileBytes;
  const uint32_t ctl_off = xchg_off + kF2XchgBytes;
  const uint32_t bars = base + ctl_off;
  unsigned char* gctl = smem_raw + ctl_off;
  volatile unsigned long long* xchg = reinterpret_cast<volatile unsigned long long*>(smem_raw + xchg_off);
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gctl + 8 * kMaxBars);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gctl + 8 * kMaxBars + 4);
  volatile int* drain_flag = reinterpret_cast<volatile int*>(gctl + 8 * kMaxBars + 8);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (*reinterpret_cast<volatile int*>(&g_tc_status) != 0) return;

  const int n_qt = (p.T_q + kBM - 1) / kBM;
  const int qt = n_qt - 1 - (int)blockIdx.x;     // heaviest causal tiles first
  const int h = blockIdx.y, b = blockIdx.z;
  const int r0 = qt * kBM;
  const Walk walk = make_walk(p, r0);               // key walk in tiles of 128
  const int n_seq = walk.n_seq, n_dep = walk.n_dep, dep_c0 = walk.dep_c0, seq_full_hi = walk.seq_full_hi;
  const int n = n_seq + n_dep;
  (void)n_dep;

  if (tid == 0) {
    mbar_init(bars + 8 * B_::res, 128);
    mbar_init(bars + 8 * B_::done, 1);
    for (int i = 0; i < R; ++i) { mbar_init(bars + 8 * (B_::full0 + i), 1); mbar_init(bars + 8 * (B_::empty0 + i), 1); }
    for (int i = 0; i < 2; ++i) {
      mbar_init(bars + 8 * (B_::s0 + i), 1); mbar_init(bars + 8 * (B_::r0 + i), 256);
      mbar_init(bars + 8 * (B_::p0 + i), 256); mbar_init(bars + 8 * (B_::t0 + i), 1);
    }
    *abort_flag = 0;
    *drain_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  for (int i = tid; i < (int)(kF2XchgBytes / 8); i += kF2Threads) xchg[i] = 0ull;   // tags start at 0
  if (warp == 0) {
    tmem_alloc(bars + 8 * kMaxBars, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tmem_Pb = tmem + 256, tmem_O = tmem + 320, tmem_Q = tmem + 448;
  constexpr uint32_t fmt = std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;

  if (warp == 10) {
    // ---------------------------------------------------------------- TMA warp
    if (elect_one()) { prefetch_map(&maps.k); prefetch_map(&maps.v); }
    bool ok = true;
    int issued = 0;
    for (int i = 0; ok && i < n; ++i) {
      const uint32_t slot = i % R;
      if (i >= R && !(ok = mbar_wait(bars + 8 * (B_::empty0 + slot), ((i / R) - 1) & 1, abort_flag, B_::empty0 + slot))) break;
      const bool dep = i >= n_seq;
      const int row = dep ? dep_c0 + (i - n_seq) * kBN : i * kBN;
      const uint32_t dst = sRing + slot * 2 * kTileBytes, bar = bars + 8 * (B_::full0 + slot);
      const CUtensorMap* mk = dep ? &maps.kd : &maps.k;
      const CUtensorMap* mv = dep ? &maps.vd : &maps.v;
      if (elect_one()) {
        mbar_expect_tx(bar, 2 * kTileBytes);
        tma_load_4d(dst, mk, bar, 0, h, row, b);
        tma_load_4d(dst + kHalfBytes, mk, bar, 64, h, row, b);
        tma_load_4d(dst + kTileBytes, mv, bar, 0, h, row, b);
        tma_load_4d(dst + kTileBytes + kHalfBytes, mv, bar, 64, h, row, b);
      }
      __syncwarp();
      issued = i + 1;
    }
    if (!ok) {   // let loads in flight land before the CTA's shared memory is released
      for (int i = max(0, issued - R); i < issued; ++i)
        mbar_wait(bars + 8 * (B_::full0 + i % R), (i / R) & 1, drain_flag, B_::full0 + i % R);
    }
  } else if (warp == 8) {
    // ---------------------------------------------------------------- score-MMA warp
    if (n > 0) {
      constexpr uint32_t idesc_s = instr_desc(fmt, 128, false);
      bool ok = mbar_wait(bars + 8 * B_::res, 0, abort_flag, B_::res);   // Q is in TMEM
      tc_fence_after();
      for (int i = 0; ok && i < n; ++i) {
        const uint32_t slot = i % R;
        if (i >= 2 && !(ok = mbar_wait(bars + 8 * (B_::r0 + (i & 1)), ((i - 2) >> 1) & 1, abort_flag, B_::r0 + (i & 1)))) break;
        if (!(ok = mbar_wait(bars + 8 * (B_::full0 + slot), (i / R) & 1, abort_flag, B_::full0 + slot))) break;
        tc_fence_after();
        const uint64_t dk = desc_kmajor(sRing + slot * 2 * kTileBytes);
        const uint32_t tS = tmem + (i & 1) * 128;
        if (elect_one()) {
#pragma unroll
          for (int kk = 0; kk < 8; ++kk)
            mma_ts(tS, tmem_Q + kk * 8, desc_add(dk, (kk >> 2) * kHalfBytes + (kk & 3) * 32), idesc_s, kk > 0);
          tc_commit(bars + 8 * (B_::s0 + (i & 1)));
        }
        __syncwarp();
      }
    }
  } else if (warp == 9) {
    // ---------------------------------------------------------------- PV-MMA warp
    if (n > 0) {
      constexpr uint32_t idesc_pv = instr_desc(fmt, 128, true);
      bool ok = true;
      for (int j = 0; ok && j < n; ++j) {
        if (!(ok = mbar_wait(bars + 8 * B_::p0, j & 1, abort_flag, B_::p0))) break;
        tc_fence_after();
        const uint32_t slot = j % R;
        const uint64_t dv = desc_mnmajor(sRing + slot * 2 * kTileBytes + kTileBytes, kHalfBytes);
        if (elect_one()) {
#pragma unroll
          for (int kk = 0; kk < 8; ++kk)
            mma_ts(tmem_O, tmem_Pb + kk * 8, desc_add(dv, kk * 2048), idesc_pv, (j > 0 || kk > 0) ? 1u : 0u);
          tc_commit(bars + 8 * (B_::empty0 + slot));     // ring slot j may be refilled
          tc_commit(bars + 8 * B_::t0);                  // the P buffer may be rewritten; O holds tiles <= j
          if (j == n - 1) tc_commit(bars + 8 * B_::done);
        }
        __syncwarp();
      }
    }
  } else {
    // ---------------------------------------------------------------- softmax warps
    const int half = warp >> 2, quarter = warp & 3;   // column half of each step, TMEM lane quarter
    const int row = quarter * 32 + lane;
    const int r = r0 + row;
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    if (half == 0) {   // stage this thread's Q row into TMEM as an A operand
      uint32_t regs[64];
      if (r < p.T_q) {
        const uint4* g4 = reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(p.q.ptr) + p.q.off(b, r, h));
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const uint4 v4 = g4[i];
          regs[4 * i] = v4.x; regs[4 * i + 1] = v4.y; regs[4 * i + 2] = v4.z; regs[4 * i + 3] = v4.w;
        }
      } else {
#pragma unroll
        for (int i = 0; i < 64; ++i) regs[i] = 0u;
      }
      tmem_st32<0>(tmem_Q + lane_addr, regs);
      tmem_st32<32>(tmem_Q + lane_addr + 32, regs);
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(bars + 8 * B_::res);
    }
    int slo, shi, dlo, dhi;
    seq_interval(p, r, slo, shi);
    dep_interval(p, r, dlo, dhi);
    float m_used = -INFINITY;   // maximum the accumulators are currently scaled by (same in both threads of a row)
    float l = 0.f;              // this thread's share of the row sum
    const float c = p.scale_log2;
    bool ok = true;

    for (int i = 0; i < n; ++i) {
      const int st = i & 1;
      ok = __all_sync(0xffffffffu, mbar_wait(bars + 8 * (B_::s0 + st), (i >> 1) & 1, abort_flag, B_::s0 + st));
      if (!ok) break;
      tc_fence_after();
      const bool is_dep = i >= n_seq;
      const int t0c = is_dep ? dep_c0 + (i - n_seq) * kBN : i * kBN;
      const int c0 = t0c + half * 64;
      const bool masked = is_dep || (t0c + kBN > seq_full_hi);
      const int lo = is_dep ? dlo : slo, hi = is_dep ? dhi : shi;
      // own 64 columns, plus the partner's 64 for the row maximum only: both threads of a row
      // then derive the same maximum from the same numbers, with no exchange on the critical path
      uint32_t su[64], so[64];
      tmem_ld32<0>(tmem + st * 128 + half * 64 + lane_addr, su);
      tmem_ld32<32>(tmem + st * 128 + half * 64 + 32 + lane_addr, su);
      tmem_ld32<0>(tmem + st * 128 + (half ^ 1) * 64 + lane_addr, so);
      tmem_ld32<32>(tmem + st * 128 + (half ^ 1) * 64 + 32 + lane_addr, so);
      tmem_wait_ld();
      tc_fence_before();
      mbar_arrive(bars + 8 * (B_::r0 + st));          // scores are in registers: the stage is free
      float s[64];
#pragma unroll
      for (int k = 0; k < 64; ++k) s[k] = __uint_as_float(su[k]);
      if (masked) {
#pragma unroll
        for (int k = 0; k < 64; ++k) {
          const int col = c0 + k;
          s[k] = (col >= lo && col < hi) ? s[k] : -INFINITY;
        }
      }
      // row maximum over own and partner columns: 8 chains of three-input max
      float so_f[64];
      if (masked) {
        const int co = t0c + (half ^ 1) * 64;
#pragma unroll
        for (int k = 0; k < 64; ++k) {
          const int col = co + k;
          so_f[k] = (col >= lo && col < hi) ? __uint_as_float(so[k]) : -INFINITY;
        }
      } else {
#pragma unroll
        for (int k = 0; k < 64; ++k) so_f[k] = __uint_as_float(so[k]);
      }
      float mx8[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float m = fmaxf(s[j], so_f[j]);
#pragma unroll
        for (int k = 1; k < 8; ++k) m = fmax3(m, s[j + 8 * k], so_f[j + 8 * k]);
        mx8[j] = m;
      }
      // (max is exact and order-independent, so both threads of the row get the same value)
      const float mx = fmaxf(fmax3(mx8[0], mx8[1], mx8[2]), fmax3(fmax3(mx8[3], mx8[4], mx8[5]), mx8[6], mx8[7]));
      const float m_new = fmaxf(m_used, mx * c);   // scale > 0 is required by this path
      float alpha = 1.f;
      bool grow = false;
      if (m_new > m_used + 8.f) {        // lazy rescale; also the first finite maximum (m_used = -inf)
        alpha = (m_used == -INFINITY) ? 0.f : fast_exp2(m_used - m_new);
        grow = (m_used != -INFINITY);    // nothing accumulated yet => nothing to rescale
        m_used = m_new;
      }
      const float m_sub = (m_used == -INFINITY) ? 0.f : m_used;
      l *= alpha;
      const float2 c2 = make_float2(c, c), nm2 = make_float2(-m_sub, -m_sub);
      float2 sum2[4] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
      uint32_t pk[32];
#pragma unroll
      for (int k = 0; k < 32; ++k) {
        const float2 x = __ffma2_rn(make_float2(s[2 * k], s[2 * k + 1]), c2, nm2);
        float2 pp;
        if (kF2PolyEvery > 0 && (k % (kF2PolyEvery > 0 ? kF2PolyEvery : 1)) == (kF2PolyEvery > 0 ? kF2PolyEvery : 1) - 1) {
          pp = exp2x2_fma(x);
        } else {
          pp.x = fast_exp2(x.x);
          pp.y = fast_exp2(x.y);
        }
        sum2[k & 3] = __fadd2_rn(sum2[k & 3], pp);
        pk[k] = Pack<T>::pack(pp.x, pp.y);
      }
      {
        const float2 tot = __fadd2_rn(__fadd2_rn(sum2[0], sum2[1]), __fadd2_rn(sum2[2], sum2[3]));
        l += tot.x + tot.y;
      }
      // the P buffer was last read by PV(i-1), after which O is final through tile i-1
      if (i >= 1) {
        ok = __all_sync(0xffffffffu, mbar_wait(bars + 8 * B_::t0, (i - 1) & 1, abort_flag, B_::t0));
        if (!ok) break;
        tc_fence_after();
      }
      tmem_st32<0>(tmem_Pb + half * 32 + lane_addr, pk);
      if (__any_sync(0xffffffffu, grow)) {   // rare: rescale this thread's 64 columns of O
#pragma unroll
        for (int q2 = 0; q2 < 2; ++q2) {
          uint32_t ov[32];
          tmem_ld32<0>(tmem_O + lane_addr + half * 64 + q2 * 32, ov);
          tmem_wait_ld();
#pragma unroll
          for (int k = 0; k < 32; ++k) ov[k] = __float_as_uint(__uint_as_float(ov[k]) * alpha);
          tmem_st32<0>(tmem_O + lane_addr + half * 64 + q2 * 32, ov);
        }
      }
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(bars + 8 * B_::p0);
    }

    if (ok && n > 0) ok = __all_sync(0xffffffffu, mbar_wait(bars + 8 * B_::done, 0, abort_flag, B_::done));
    if (ok && n > 0) {
      tc_fence_after();
      // row sum = the two halves' shares
      float other = 0.f;
      ok = __all_sync(0xffffffffu, pair_exchange(xchg, n & 1, half, row, (uint32_t)(n + 1), l, other, abort_flag));
      const float lt = l + other;
      const float inv = lt > 0.f ? 1.f / lt : 0.f;
      T* go = reinterpret_cast<T*>(p.o.ptr) + p.o.off(b, r, h) + half * 64;
#pragma unroll
      for (int q2 = 0; q2 < 2; ++q2) {
        uint32_t ov[32];
        tmem_ld32<0>(tmem_O + lane_addr + half * 64 + q2 * 32, ov);
        tmem_wait_ld();
        if (ok && r < p.T_q) {
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            uint4 v4;
            v4.x = Pack<T>::pack(__uint_as_float(ov[k * 8 + 0]) * inv, __uint_as_float(ov[k * 8 + 1]) * inv);
            v4.y = Pack<T>::pack(__uint_as_float(ov[k * 8 + 2]) * inv, __uint_as_float(ov[k * 8 + 3]) * inv);
            v4.z = Pack<T>::pack(__uint_as_float(ov[k * 8 + 4]) * inv, __uint_as_float(ov[k * 8 + 5]) * inv);
            v4.w = Pack<T>::pack(__uint_as_float(ov[k * 8 + 6]) * inv, __uint_as_float(ov[k * 8 + 7]) * inv);
            *reinterpret_cast<uint4*>(go + q2 * 32 + k * 8) = v4;
          }
        }
      }
      if (ok && half == 0 && r < p.T_q) p.lse[((int64_t)b * p.T_q + r) * p.H + h] = m_used + log2f(lt);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

inline int fwd2(const Params& p, const moda_problem* pr, cudaStream_t st, int* launches, int* cuda_err) {
  Fwd2Maps maps;
  memset(&maps, 0, sizeof(maps));
  const int64_t TL = (int64_t)p.T_kv * p.L;
  bool ok = make_map_rows(&maps.k, p.k, pr->dtype, p.B, p.T_kv, p.H, 128) &&
            make_map_rows(&maps.v, p.v, pr->dtype, p.B, p.T_kv, p.H, 128);
  if (ok && p.L > 0) {
    ok = make_map_rows(&maps.kd, p.kd, pr->dtype, p.B, TL, p.H, 128) && make_map_rows(&maps.vd, p.vd, pr->dtype, p.B, TL, p.H, 128);
  } else if (ok) {
    maps.kd = maps.k; maps.vd = maps.v;   // never dereferenced (no depth steps)
  }
  if (!ok) return MODA_ERR_UNSUPPORTED;
  void* status_addr = nullptr;
  cudaError_t e = cudaGetSymbolAddress(&status_addr, g_tc_status);
  if (e == cudaSuccess) e = cudaMemsetAsync(status_addr, 0, sizeof(int), st);
  if (e != cudaSuccess) { *cuda_err = (int)e; return MODA_ERR_CUDA; }
  dim3 grid((p.T_q + kBM - 1) / kBM, p.H, p.B);
  auto launch = [&](auto kern) -> cudaError_t {
    cudaError_t er = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kF2Smem);
    if (er != cudaSuccess) return er;
    prof::Scope ps(prof::kFwdTc, st);
    kern<<<grid, kF2Threads, kF2Smem, st>>>(p, maps);
    return cudaGetLastError();
  };
  e = (pr->dtype == MODA_BF16) ? launch(fwd2_kernel<__nv_bfloat16, 4>) : launch(fwd2_kernel<__half, 4>);
  if (e != cudaSuccess) { *cuda_err = (int)e; return MODA_ERR_CUDA; }
  *launches += 1;
  return MODA_OK;
}

}  // namespace tc
}  // namespace moda
