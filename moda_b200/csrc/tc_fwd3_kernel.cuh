// tcgen05 / TMEM / TMA forward of MoDA, two query tiles per CTA (D = 64 or 128, bf16 or fp16).
//
// One CTA per SM owns 256 folded query rows of one (batch, KV head): two tiles of 128 rows, each
// with its own softmax warpgroup (thread = row = TMEM lane), its own score block S_a and its own
// accumulator O_a in TMEM.  One MMA warp issues for both tiles in the order
//
//     QK_0(s+1) after PV_0(s),   QK_1(s+1) after PV_1(s)
//
// so that while warpgroup 0 is busy with the softmax of step s the tensor pipe works on tile 1 and
// vice versa: the exponentials of one tile (the MUFU needs as many clocks per 128 x 128 block as
// the two matmuls need tensor clocks) run under the matmuls of the other, and the two warpgroups
// are kept half a step apart by the issue order instead of drifting into the same phase, which is
// what two independent 128-row CTAs per SM do.  A K/V tile fetched once serves both query tiles.
//
// Steps: the sequence key tiles (a tile past the causal range of query tile 0 is taken by tile 1
// alone), then the depth key tiles of the two query tiles, interleaved (their depth windows are
// different rows, so a depth step belongs to one query tile).
//
//   warp 9 (TMA)   Q_0, Q_1 once; a ring of K tiles and a ring of V tiles with barriers of their own:
//                  a K slot is free again once the scores that read it have run, a softmax earlier
//                  than the V slot of the same step, so the next K tile is on its way that much
//                  sooner (depth tiles come from HBM, not from L2, and are needed right away).
//   warp 8 (MMA)   S_a = Q_a K^T (SS, M128 N128), O_a += P_a V (TS, N = D: P_a packed over S_a in TMEM).
//   warps 0-3 / 4-7  softmax of query tile 0 / 1, lazy O rescale, epilogue.
//
// TMEM (512 columns): S_0 [0,128), S_1 [128,256), O_0 [256,256+D), O_1 [384,384+D).  A softmax warp
// hands P over in two halves (columns [0,32) and [32,64) of the packed block), so the first half of PV
// runs under the last exponentials.  Every wait is bounded, as in the other tcgen05 kernels.
#pragma once
#include "tc_bwd_kernels.cuh"

namespace moda {
namespace tc {

constexpr int kF3Threads = 384;          // 8 softmax warps + MMA warp + TMA warp + 2 idle warps (a whole warpgroup)
// Registers per thread: the CTA starts with 168 (65536 / 384, rounded down to a multiple of 8); after
// the set-up the last warpgroup (MMA, TMA) gives registers back and the softmax warpgroups take
// them, so that a softmax thread holds its 128 scores, the packed P and the partial sums without spills.
constexpr uint32_t kF3SoftmaxRegs = 232, kF3IssueRegs = 40;
static_assert(2 * 128 * kF3SoftmaxRegs + 128 * kF3IssueRegs <= 384 * 168, "register pool of the CTA exceeded");
// P reaches the PV matmul in kF3Parts parts: part i = packed columns [kF3Bound[i], kF3Bound[i+1]) of
// the 64 (multiples of 16: a tcgen05.st of 16 columns, two K = 16 slices of the matmul).
constexpr int kF3Parts = 2;
__device__ constexpr int kF3Bound[5] = {0, 32, 64, 64, 64};
static_assert(kF3Parts >= 1 && kF3Parts <= 4, "one to four parts");
constexpr int kF3KSlots = 2;      // K tiles in flight or in use (three fit and measured the same); V tiles: two
static_assert(kF3KSlots == 2 || kF3KSlots == 3, "two or three K slots");
// barriers: q, fullk[3], fullv[2], emptyk[3], emptyv[2], s[2], done, p[part][2] (part of P stored)
struct F3Bars {
  static constexpr int q = 0, fullk0 = 1, fullv0 = 4, emptyk0 = 6, emptyv0 = 9, s0 = 11, done = 13, p0 = 14, count = 14 + 2 * kF3Parts;
};
static_assert(F3Bars::count <= kMaxBars, "control block too small");
// Q_0, Q_1, the K slots, two V slots
template <int D> __host__ __device__ constexpr uint32_t f3_smem() { return (4 + kF3KSlots) * tile_bytes<D>() + kCtlBytes; }
static_assert(f3_smem<128>() <= 232448, "shared memory of the CTA exceeded");

struct Fwd3Maps { CUtensorMap q, k, v, kd, vd; };        // 128-row boxes

// The key steps of a 256-row CTA.
struct F3Plan {
  Walk w[2];
  int n_s;      // sequence steps
  int n;        // all steps
};
__device__ __forceinline__ F3Plan f3_plan(const Params& p, int r0) {
  F3Plan pl;
  pl.w[0] = make_walk(p, r0);
  if (r0 + kBM < p.T_q) pl.w[1] = make_walk(p, r0 + kBM);
  else { pl.w[1].n_seq = 0; pl.w[1].n_dep = 0; pl.w[1].dep_c0 = 0; pl.w[1].seq_full_hi = 0; }
  pl.n_s = max(pl.w[0].n_seq, pl.w[1].n_seq);
  pl.n = pl.n_s + pl.w[0].n_dep + pl.w[1].n_dep;
  return pl;
}
// Step s: which query tiles take part (bit a), whether it is a depth step, its first key row.
__device__ __forceinline__ void f3_step(const F3Plan& pl, int s, int& part, bool& is_dep, int& row) {
  if (s < pl.n_s) {
    part = (s < pl.w[0].n_seq ? 1 : 0) | (s < pl.w[1].n_seq ? 2 : 0);
    is_dep = false;
    row = s * kBN;
    return;
  }
  const int e = s - pl.n_s, m = min(pl.w[0].n_dep, pl.w[1].n_dep);
  int a, d;
  if (e < 2 * m) { a = e & 1; d = e >> 1; }
  else { a = (pl.w[0].n_dep > pl.w[1].n_dep) ? 0 : 1; d = m + (e - 2 * m); }
  part = 1 << a;
  is_dep = true;
  row = pl.w[a].dep_c0 + d * kBN;
}

// 16 columns of pk starting at column j (j is a compile-time constant after unrolling)
__device__ __forceinline__ void tmem_st16_at(uint32_t taddr, const uint32_t (&pk)[64], int j) {
  if (j == 0) tmem_st16<0>(taddr, pk);
  else if (j == 16) tmem_st16<16>(taddr + 16, pk);
  else if (j == 32) tmem_st16<32>(taddr + 32, pk);
  else tmem_st16<48>(taddr + 48, pk);
}

// Part kPart of a row's P (and the parts after it): exponentials, store into TMEM, signal.
template <typename T, int kPolyEvery, int kPart, typename Ready>
__device__ __forceinline__ void softmax_part(const float (&sc)[128], float c, float m_used, float2 (&sum2)[4], uint32_t (&pk)[64],
                                             uint32_t taddr, Ready& p_ready) {
  if constexpr (kPart < kF3Parts) {
    constexpr int i0 = kF3Bound[kPart], i1 = kF3Bound[kPart + 1];
    static_assert(i0 % 16 == 0 && i1 % 16 == 0 && i0 < i1 && i1 <= 64, "parts are multiples of 16 columns");
    softmax_exps<T, kPolyEvery, i0, i1>(sc, c, m_used, sum2, pk);
    if constexpr (i0 % 32 == 0 && i1 - i0 >= 32) {
      tmem_st32<i0>(taddr + i0, pk);
      if constexpr (i1 - i0 >= 48) tmem_st16<i0 + 32>(taddr + i0 + 32, pk);
      if constexpr (i1 - i0 == 64) tmem_st16<i0 + 48>(taddr + i0 + 48, pk);
    } else {
#pragma unroll
      for (int j = i0; j < i1; j += 16) tmem_st16_at(taddr, pk, j);
    }
    p_ready(F3Bars::p0 + 2 * kPart);
    softmax_part<T, kPolyEvery, kPart + 1>(sc, c, m_used, sum2, pk, taddr, p_ready);
  }
}

template <typename T, int D, int kPolyEvery>
__global__ void __launch_bounds__(kF3Threads, 1)
fwd3_kernel(const __grid_constant__ Params p, const __grid_constant__ Fwd3Maps maps) {
  using B_ = F3Bars;
  constexpr uint32_t kTile = tile_bytes<D>();
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  const uint32_t base = smem_u32(smem_raw);
  if (base & 1023u) {
    if (threadIdx.x == 0) record_failure(2 << 8);
    return;
  }
  const uint32_t sQ = base;                              // Q_a at sQ + a * kTile
  constexpr int KS = kF3KSlots;
  const uint32_t sK = base + 2 * kTile;                  // K slot i at sK + i * kTile
  const uint32_t sV = sK + KS * kTile;                   // V slot i at sV + i * kTile
  const uint32_t ctl_off = (4 + KS) * kTile;
  const uint32_t bars = base + ctl_off;
  unsigned char* gctl = smem_raw + ctl_off;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gctl + 8 * kMaxBars);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gctl + 8 * kMaxBars + 4);
  volatile int* drain_flag = reinterpret_cast<volatile int*>(gctl + 8 * kMaxBars + 8);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (*reinterpret_cast<volatile int*>(&g_tc_status) != 0) return;

  const int n_pairs = (p.T_q + 2 * kBM - 1) / (2 * kBM);
  const BlockId bid = block_order(p, D);
  const int pq = n_pairs - 1 - bid.rank;            // heaviest causal tiles first
  const int h = bid.h, b = bid.b;
  const int r0 = pq * 2 * kBM;
  const F3Plan pl = f3_plan(p, r0);
  const bool two = r0 + kBM < p.T_q;                // the second query tile exists
  const int dep5 = (p.Ls != p.L) ? p.L : 0;         // in-place layer cache: 5-D depth maps

  if (tid == 0) {
    mbar_init(bars + 8 * B_::q, 1);
    mbar_init(bars + 8 * B_::done, 1);
    for (int i = 0; i < KS; ++i) {
      mbar_init(bars + 8 * (B_::fullk0 + i), 1);
      mbar_init(bars + 8 * (B_::emptyk0 + i), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(bars + 8 * (B_::fullv0 + i), 1);
      mbar_init(bars + 8 * (B_::emptyv0 + i), 1);
      mbar_init(bars + 8 * (B_::s0 + i), 1);
      for (int j = 0; j < kF3Parts; ++j) mbar_init(bars + 8 * (B_::p0 + 2 * j + i), 4);   // one arrival per softmax warp
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
  constexpr uint32_t fmt = std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;

  // Warpgroup-wide register reallocation, first thing in every role: all four warps of the last
  // warpgroup release, so the requests of the softmax warpgroups cannot starve.
  if (warp == 9) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" :: "n"(kF3IssueRegs));
    // ---------------------------------------------------------------- TMA warp
    if (pl.n > 0) {
      if (elect_one()) {
        prefetch_map(&maps.q); prefetch_map(&maps.k); prefetch_map(&maps.v);
        mbar_expect_tx(bars + 8 * B_::q, (two ? 2u : 1u) * kTile);
        tma_load_tile<D>(sQ, &maps.q, bars + 8 * B_::q, kHalfBytes, h, r0, b);
        if (two) tma_load_tile<D>(sQ + kTile, &maps.q, bars + 8 * B_::q, kHalfBytes, h, r0 + kBM, b);
      }
      __syncwarp();
      // K tiles run kLead steps ahead of the V tiles: K(s + kLead) waits for the scores of step
      // s + kLead - KS, V(s) for the P V of step s - 2, which finish in that order.
      constexpr int kLead = KS - 2;
      bool ok = true;
      int issued_k = 0, issued_v = 0;
      auto load = [&](int s, bool is_k) -> bool {
        const uint32_t slot = is_k ? s % KS : s & 1;
        const int e_bar = (is_k ? B_::emptyk0 : B_::emptyv0) + slot, f_bar = (is_k ? B_::fullk0 : B_::fullv0) + slot;
        const int use = is_k ? s / KS : s >> 1;           // how often the slot has been filled before
        if (use >= 1 && !mbar_wait(bars + 8 * e_bar, (use - 1) & 1, abort_flag, e_bar)) return false;
        int part, row; bool dep;
        f3_step(pl, s, part, dep, row);
        const uint32_t dst = is_k ? sK + slot * kTile : sV + slot * kTile, bar = bars + 8 * f_bar;
        const CUtensorMap* m = dep ? (is_k ? &maps.kd : &maps.vd) : (is_k ? &maps.k : &maps.v);
        if (elect_one()) {
          mbar_expect_tx(bar, kTile);
          if (dep) tma_load_dep_tile<D>(dst, m, bar, kHalfBytes, h, row, b, dep5);
          else tma_load_tile<D>(dst, m, bar, kHalfBytes, h, row, b);
        }
        __syncwarp();
        (is_k ? issued_k : issued_v) = s + 1;
        return true;
      };
      for (int s = 0; ok && s < kLead && s < pl.n; ++s) ok = load(s, true);
      for (int s = 0; ok && s < pl.n; ++s) {
        if (s + kLead < pl.n) ok = load(s + kLead, true);
        if (ok) ok = load(s, false);
      }
      if (!ok) {   // let loads in flight land before the CTA's shared memory is released
        mbar_wait(bars + 8 * B_::q, 0, drain_flag, B_::q);
        for (int s = max(0, issued_k - KS); s < issued_k; ++s)
          mbar_wait(bars + 8 * (B_::fullk0 + s % KS), (s / KS) & 1, drain_flag, B_::fullk0 + s % KS);
        for (int s = max(0, issued_v - 2); s < issued_v; ++s)
          mbar_wait(bars + 8 * (B_::fullv0 + (s & 1)), (s >> 1) & 1, drain_flag, B_::fullv0 + (s & 1));
      }
    }
  } else if (warp == 8) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" :: "n"(kF3IssueRegs));
    // ---------------------------------------------------------------- MMA warp
    if (pl.n > 0) {
      constexpr uint32_t idesc_qk = instr_desc(fmt, 128, false);
      constexpr uint32_t idesc_pv = instr_desc(fmt, D, true);
      int qk_cnt[2] = {0, 0}, pv_cnt[2] = {0, 0};     // steps tile a has taken part in so far
      bool ok = mbar_wait(bars + 8 * B_::q, 0, abort_flag, B_::q);
      int qk_left = 0;                                // tiles that have yet to read the K tile being read
      // S_a = Q_a K(s)^T; the last tile to read K(s) hands the slot back
      auto qk = [&](int a, int s) -> bool {
        const uint32_t slot = s % KS;
        if (!mbar_wait(bars + 8 * (B_::fullk0 + slot), (s / KS) & 1, abort_flag, B_::fullk0 + slot)) return false;
        tc_fence_after();
        const uint64_t dK = desc_kmajor(sK + slot * kTile), dQa = desc_kmajor(sQ + a * kTile);
        --qk_left;
        const uint32_t tS = tmem + a * 128;
        if (elect_one()) {
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk) {
            const uint32_t off = (kk >> 2) * kHalfBytes + (kk & 3) * 32;
            mma_ss(tS, desc_add(dQa, off), desc_add(dK, off), idesc_qk, kk > 0);
          }
          tc_commit(bars + 8 * (B_::s0 + a));
          if (qk_left == 0) tc_commit(bars + 8 * (B_::emptyk0 + slot));
        }
        __syncwarp();
        ++qk_cnt[a];
        return true;
      };
      // O_a += P_a V(s); `last`: no other MMA of step s follows, the slot may be refilled.  The
      // matmuls over a part of P go out while the softmax still computes the next one.
      auto pv = [&](int a, int s, bool last) -> bool {
        const uint32_t slot = s & 1;
        if (!mbar_wait(bars + 8 * (B_::fullv0 + slot), (s >> 1) & 1, abort_flag, B_::fullv0 + slot)) return false;
        const uint64_t dV = desc_mnmajor(sV + slot * kTile, kHalfBytes);
        const uint32_t tS = tmem + a * 128, tO = tmem + 256 + a * 128;
#pragma unroll
        for (int part = 0; part < kF3Parts; ++part) {
          if (!mbar_wait(bars + 8 * (B_::p0 + 2 * part + a), pv_cnt[a] & 1, abort_flag, B_::p0 + 2 * part + a)) return false;
          tc_fence_after();
          if (elect_one()) {
#pragma unroll
            for (int kk = kF3Bound[part] / 8; kk < kF3Bound[part + 1] / 8; ++kk)
              mma_ts(tO, tS + kk * 8, desc_add(dV, kk * 2048), idesc_pv, (pv_cnt[a] > 0 || kk > 0) ? 1u : 0u);
            if (last && part == kF3Parts - 1) tc_commit(bars + 8 * (B_::emptyv0 + slot));
          }
          __syncwarp();
        }
        ++pv_cnt[a];
        return true;
      };
      int part, row, part_next = 0; bool dep;
      if (ok) {
        f3_step(pl, 0, part, dep, row);
        qk_left = __popc(part);
        for (int a = 0; ok && a < 2; ++a)
          if (part & (1 << a)) ok = qk(a, 0);
      }
      // Steady state: steps that both tiles take part in and whose successor is such a step too
      // (all but the last sequence steps).  The same order as the general loop below, PV_0(s),
      // QK_0(s+1), PV_1(s), QK_1(s+1), as straight runs of instructions: the time this warp spends
      // between two matmuls is time the tensor pipe waits.
      int s = 0;
      const int n_both = min(pl.w[0].n_seq, pl.w[1].n_seq);
      if (ok && n_both > 1) {
        const uint64_t dQ[2] = {desc_kmajor(sQ), desc_kmajor(sQ + kTile)};
        uint32_t kn_slot = 1 % KS, kn_par = 0;            // slot of K(s+1) and the parity of its filling
        for (; ok && s + 1 < n_both; ++s) {
          const uint32_t slot = s & 1, par = s & 1;       // both tiles have taken part in s steps so far
          // V(s) landed long ago: the check costs nothing while the warp waits for P_0 anyway
          if (!(ok = mbar_wait(bars + 8 * (B_::fullv0 + slot), (s >> 1) & 1, abort_flag, B_::fullv0 + slot))) break;
          const uint64_t dV = desc_mnmajor(sV + slot * kTile, kHalfBytes);
          const uint64_t dKn = desc_kmajor(sK + kn_slot * kTile);
          const uint32_t acc = s > 0 ? 1u : 0u;
#pragma unroll
          for (int a = 0; a < 2; ++a) {
            const uint32_t tS = tmem + a * 128, tO = tmem + 256 + a * 128;
#pragma unroll
            for (int part_i = 0; part_i < kF3Parts; ++part_i) {
              if (!(ok = mbar_wait(bars + 8 * (B_::p0 + 2 * part_i + a), par, abort_flag, B_::p0 + 2 * part_i + a))) break;
              tc_fence_after();
              if (elect_one()) {
#pragma unroll
                for (int kk = kF3Bound[part_i] / 8; kk < kF3Bound[part_i + 1] / 8; ++kk)
                  mma_ts(tO, tS + kk * 8, desc_add(dV, kk * 2048), idesc_pv, kk > 0 ? 1u : acc);
                if (a == 1 && part_i == kF3Parts - 1) tc_commit(bars + 8 * (B_::emptyv0 + slot));
              }
              __syncwarp();
            }
            if (!ok) break;
            // K(s+1): one wait serves both tiles
            if (a == 0 && !(ok = mbar_wait(bars + 8 * (B_::fullk0 + kn_slot), kn_par, abort_flag, B_::fullk0 + kn_slot))) break;
            tc_fence_after();
            if (elect_one()) {
#pragma unroll
              for (int kk = 0; kk < D / 16; ++kk) {
                const uint32_t off = (kk >> 2) * kHalfBytes + (kk & 3) * 32;
                mma_ss(tS, desc_add(dQ[a], off), desc_add(dKn, off), idesc_qk, kk > 0);
              }
              tc_commit(bars + 8 * (B_::s0 + a));
              if (a == 1) tc_commit(bars + 8 * (B_::emptyk0 + kn_slot));
            }
            __syncwarp();
          }
          if (++kn_slot == KS) { kn_slot = 0; kn_par ^= 1; }
        }
        qk_cnt[0] = qk_cnt[1] = s + 1;
        pv_cnt[0] = pv_cnt[1] = s;
      }
      for (; ok && s < pl.n; ++s) {
        f3_step(pl, s, part, dep, row);
        part_next = 0;
        if (s + 1 < pl.n) f3_step(pl, s + 1, part_next, dep, row);
        qk_left = __popc(part_next);
        // a tile that joins at s+1 without taking part in s (alternating depth steps) has a free
        // score block: its scores go ahead of this step's PVs and run under the other tile's softmax
#pragma unroll
        for (int a = 0; a < 2; ++a)
          if (ok && ((part_next & ~part) & (1 << a))) ok = qk(a, s + 1);
#pragma unroll
        for (int a = 0; a < 2; ++a) {
          if (ok && (part & (1 << a))) ok = pv(a, s, (part >> (a + 1)) == 0);
          if (ok && ((part_next & part) & (1 << a))) ok = qk(a, s + 1);
        }
      }
      if (ok) {
        if (elect_one()) tc_commit(bars + 8 * B_::done);
        __syncwarp();
      }
    }
  } else if (warp >= 10) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" :: "n"(kF3IssueRegs));
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" :: "n"(kF3SoftmaxRegs));
    // ---------------------------------------------------------------- softmax warps
    const int a = warp >> 2, wq = warp & 3;          // query tile; TMEM lane quarter
    const int row = wq * 32 + lane;                  // row of the tile == TMEM lane
    const int r = r0 + a * kBM + row;
    const uint32_t lane_addr = (uint32_t)(wq * 32) << 16;
    const uint32_t tmem_S = tmem + a * 128, tmem_O = tmem + 256 + a * 128;
    const Walk walk = pl.w[a];
    int slo, shi, dlo, dhi;
    seq_interval(p, r, slo, shi);
    dep_interval(p, r, dlo, dhi);
    float m_used = -INFINITY;   // maximum the accumulators are currently scaled by
    float l = 0.f;
    bool ok = true;
    const float c = p.scale_log2;
    int cnt = 0;                // steps this tile has taken part in

    for (int s = 0; s < pl.n; ++s) {
      int part, c0; bool is_dep;
      f3_step(pl, s, part, is_dep, c0);
      if (!(part & (1 << a))) continue;
      ok = __all_sync(0xffffffffu, mbar_wait(bars + 8 * (B_::s0 + a), cnt & 1, abort_flag, B_::s0 + a));
      if (!ok) break;   // warp-uniform: the tcgen05 loads/stores below are warp-collective
      tc_fence_after();
      const bool masked = is_dep || (c0 + kBN > walk.seq_full_hi);
      const int lo = is_dep ? dlo : slo, hi = is_dep ? dhi : shi;

      // A depth tile holds the rows of several positions; a warp whose 32 query rows see none of
      // its columns contributes an all-zero P block and skips the scores altogether.
      const bool none = is_dep && __all_sync(0xffffffffu, (c0 + kBN <= lo) || (c0 >= hi));
      // P is complete for a group of columns once every lane's stores have finished: one arrival per warp
      auto p_ready = [&](int bar_id) {
        tmem_wait_st();
        tc_fence_before();
        __syncwarp();
#ifdef MODA_WAIT_TEST
        // wait-expiry test build: the arrival for the first part of P is withheld, so the MMA warp's
        // bounded wait on that barrier (which no TMA load targets) runs out and the CTA leaves
        // through the teardown path
        if (bar_id == B_::p0) return;
#endif
        if (lane == 0) mbar_arrive(bars + 8 * (bar_id + a));
      };
      if (none) {
        uint32_t z[64];
#pragma unroll
        for (int i = 0; i < 64; ++i) z[i] = 0u;
        tmem_st32<0>(tmem_S + lane_addr + 0, z);
        tmem_st32<32>(tmem_S + lane_addr + 32, z);
#pragma unroll
        for (int part = 0; part < kF3Parts; ++part) p_ready(B_::p0 + 2 * part);
        ++cnt;
        continue;
      }
      float alpha = 1.f;
      bool grow = false;
      uint32_t pk[64];
      float sc[128];
      {
        uint32_t su[128];
        tmem_ld32<0>(tmem_S + lane_addr + 0, su);
        tmem_ld32<32>(tmem_S + lane_addr + 32, su);
        tmem_ld32<64>(tmem_S + lane_addr + 64, su);
        tmem_ld32<96>(tmem_S + lane_addr + 96, su);
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 128; ++i) sc[i] = __uint_as_float(su[i]);
      }
      softmax_prepare(sc, masked, is_dep && (p.L & 31) == 0, c0, lo, hi, c, m_used, l, alpha, grow);
      // rescale O (TMEM round trip) only when some row of this warp moved its maximum; the PV of
      // this tile's previous step finished before these scores were produced (issue order)
      if (__any_sync(0xffffffffu, grow)) {
#pragma unroll
        for (int q4 = 0; q4 < D / 32; ++q4) {
          uint32_t ov[32];
          tmem_ld32<0>(tmem_O + lane_addr + q4 * 32, ov);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) ov[i] = __float_as_uint(__uint_as_float(ov[i]) * alpha);
          tmem_st32<0>(tmem_O + lane_addr + q4 * 32, ov);
        }
      }
      float2 sum2[4] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
      softmax_part<T, kPolyEvery, 0>(sc, c, m_used, sum2, pk, tmem_S + lane_addr, p_ready);
      l += softmax_total(sum2);
      ++cnt;
    }

    if (ok && cnt > 0) ok = __all_sync(0xffffffffu, mbar_wait(bars + 8 * B_::done, 0, abort_flag, B_::done));
    if (ok && cnt > 0) {
      tc_fence_after();
      float inv = l > 0.f ? 1.f / l : 0.f, w_dep = 0.f, lse_out = m_used + log2f(l);
      const bool merge = p.merge_depth != 0;
      const int64_t lse_idx = ((int64_t)b * p.T_q + (r < p.T_q ? r : 0)) * p.H + h;
      if (merge) merge_partials(m_used, l, p.lse[lse_idx], inv, w_dep, lse_out);
      T* go = reinterpret_cast<T*>(p.o.ptr) + p.o.off(b, r, h);
#pragma unroll
      for (int q4 = 0; q4 < D / 32; ++q4) {
        uint32_t ov[32];
        tmem_ld32<0>(tmem_O + lane_addr + q4 * 32, ov);
        tmem_wait_ld();
        if (r < p.T_q) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint4* dst = reinterpret_cast<uint4*>(go + q4 * 32 + i * 8);
            *dst = merge ? pack8_blend<T>(ov + i * 8, inv, *dst, w_dep) : pack8_scaled<T>(ov + i * 8, inv);
          }
        }
      }
      if (r < p.T_q) p.lse[lse_idx] = lse_out;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

template <typename T, int D>
inline cudaError_t launch_fwd3(const Params& p, const Fwd3Maps& maps, cudaStream_t st) {
  // one pair of exponentials in four goes to the FMA pipe (exp2x2_fma); none, one in eight and
  // one in two were all slower
  auto kern = fwd3_kernel<T, D, 4>;
  constexpr uint32_t smem = f3_smem<D>();
  cudaError_t er = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (er != cudaSuccess) return er;
  dim3 grid((p.T_q + 2 * kBM - 1) / (2 * kBM), p.H, p.B);
  prof::Scope ps(prof::kFwdTc, st);
  kern<<<grid, kF3Threads, smem, st>>>(p, maps);
  return cudaGetLastError();
}

inline int fwd3(const Params& p, const moda_problem* pr, cudaStream_t st, int* launches, int* cuda_err) {
  FwdMaps fm;
  if (!make_fwd_maps(&fm, p, pr)) return MODA_ERR_UNSUPPORTED;
  Fwd3Maps maps{fm.q, fm.k, fm.v, fm.kd, fm.vd};
  cudaError_t e = clear_launch_status(st);
  if (e != cudaSuccess) { *cuda_err = (int)e; return MODA_ERR_CUDA; }
  const bool bf = pr->dtype == MODA_BF16;
  if (pr->D == 128) e = bf ? launch_fwd3<__nv_bfloat16, 128>(p, maps, st) : launch_fwd3<__half, 128>(p, maps, st);
  else e = bf ? launch_fwd3<__nv_bfloat16, 64>(p, maps, st) : launch_fwd3<__half, 64>(p, maps, st);
  if (e != cudaSuccess) { *cuda_err = (int)e; return MODA_ERR_CUDA; }
  *launches += 1;
  return MODA_OK;
}

}  // namespace tc
}  // namespace moda
