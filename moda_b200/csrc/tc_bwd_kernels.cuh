// tcgen05 / TMEM / TMA backward kernels of MoDA for sm_100a (D = 64 or 128, bf16 or fp16).
//
// Like the reference (moda_v14.py:1470-1842) the backward is a row-statistics pass, a
// query-parallel dq kernel and a key-parallel dk/dv kernel; every output row has one
// owning CTA, so there are no atomics and results are bit-reproducible.
//
//   pre_kernel : delta = rowsum(o * dout) (stored o, fp32 accumulate: moda_v14.py:525-539)
//                written, with a copy of lse, as [B, H, T_q rounded up to 64 (+64)] so that
//                a (b, h) slice of 64 rows is one contiguous 256-byte bulk copy.
//   dq_kernel  : CTA = 128 query rows; walks the visible key tiles in steps of 64 keys.
//                Q and dO rows sit in TMEM as 16-bit A operands for the whole CTA, so the
//                score MMAs S = Q K^T, dP = dO V^T (N = 64) read only the K / V step tile
//                from shared memory; softmax warps form dS = P (dP - delta) in TMEM;
//                dQ += dS K (A from TMEM, K tile read MN-major).  dq = scale * dQ.
//   dkv_kernel : CTA = 128 keys of the sequence K/V or of the depth K/V; walks the query
//                rows that can see them in steps of 64 rows.  K and V rows sit in TMEM as
//                A operands; S^T = K Q^T, dP^T = V dO^T (N = 64) -> P^T and dS^T written to
//                shared memory -> dV += P^T dO, dK += dS^T Q (Q/dO tiles read MN-major).
//                The G heads of a KV head are rows of the same folded query tile, so the
//                GQA sum happens inside the MMA.  dk = scale * dK.
//
// Both MMA kernels run one CTA per SM with four roles: a TMA warp that keeps a ring of
// step tiles full, an MMA warp, and two softmax warpgroups that take alternate steps (each
// owns one of the two TMEM score stages).  The tensor pipe executes the MMAs of one issuing
// thread in order, which is what allows step i+2's scores to reuse the TMEM stage the step-i
// update reads from without a wait in between; ring slots are handed back to the TMA warp by
// a tcgen05.commit on the slot's "empty" barrier after the update that last read them.
#pragma once
#include "tc_kernels.cuh"

namespace moda {
namespace tc {

constexpr int kStep = 64;                      // keys (dq) or query rows (dkv) per pipeline step
// Ring depths (step tiles in flight).  A slot is refilled only when the update matmul that reads it
// last has completed, two steps after its scores, and a TMA load of a step's tiles takes longer
// than a step: five slots are needed (four cost dk/dv a fifth of its speed, three a third at
// D = 64; more than five gain nothing).  At D = 128 five (dk/dv) and six (dq) are also what fits
// in shared memory.
template <int D> __host__ __device__ constexpr int dq_ring() { return 6; }                    // {K, V} step tiles
template <int D> __host__ __device__ constexpr int dkv_ring() { return D == 128 ? 5 : 6; }    // {Q, dO, lse, delta} step tiles
constexpr uint32_t kStepHalf = 64 * 64 * 2;    // one TMA box of a step tile: [64 rows x 64 elements]
template <int D> __host__ __device__ constexpr uint32_t step_tile() { return (uint32_t)(D / 64) * kStepHalf; }   // [64 x D] 16-bit tile
constexpr uint32_t kScoreTile = 128 * 64 * 2;  // [128 x 64] 16-bit tile of dS, P^T or dS^T (K-major, 128 B per row)
// 8 softmax warps + S-MMA (8), TMA (9), update-MMA (10) and dP-MMA (11) warps.  The two score matmuls
// of a step have an issuing warp each: a tcgen05.mma occupies its issuing warp for some 30 clocks
// (60 with two shared-memory descriptors), as long as an N = 64 instruction takes to execute, so one
// warp issuing both could not run ahead of the tensor pipe.
constexpr int kDqThreads = 384;
constexpr int kDkvThreads = kDqThreads;
constexpr int kFusedBwdThreads = 352;          // the fused kernel keeps one score-MMA warp

struct DqMaps { CUtensorMap k, v, kd, vd; };               // 64-row boxes
struct DkvMaps { CUtensorMap k, v, kd, vd, q, dout; };     // k, v, kd, vd: 128-row boxes; q, dout 64-row

__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               :: "r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

// Tile store shared -> global through the tensor map (bulk async-group of the issuing thread).
__device__ __forceinline__ void tma_store_4d(const CUtensorMap* map, uint32_t src, int c0, int c1, int c2, int c3) {
  asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
               :: "l"(map), "r"(src), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}
__device__ __forceinline__ void tma_store_5d(const CUtensorMap* map, uint32_t src, int c0, int c1, int c2, int c3, int c4) {
  asm volatile("cp.async.bulk.tensor.5d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5, %6}], [%1];"
               :: "l"(map), "r"(src), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read_all() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// ------------------------------------------------------------------ statistics pass
// delta = rowsum(o * dO) from the stored o, and lse, both transposed to [B, H, T_qp] so that the
// backward kernels fetch 64 rows of one (b, h) with one 256-byte bulk copy.  Eight lanes per row,
// four rows per warp, 32 consecutive rows of one (b, h) per block iteration; each lane has two
// 16-byte loads of o and two of dO in flight (one of each for D = 64).
template <typename T, int D>
__global__ void __launch_bounds__(256) pre_kernel(const __grid_constant__ Params p, float* delta_t, float* lse_t, float* norm_t, int T_qp) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, sub = lane & 7, grp = lane >> 3;
  const uint32_t groups_per_bh = (uint32_t)T_qp / 32u;             // T_qp is a multiple of 64
  const int64_t n_groups = (int64_t)p.B * p.H * groups_per_bh;
  for (int64_t gidx = blockIdx.x; gidx < n_groups; gidx += gridDim.x) {
    const uint32_t bh = (uint32_t)(gidx / groups_per_bh);
    const int r = (int)((uint32_t)(gidx - (int64_t)bh * groups_per_bh) * 32u) + w * 4 + grp;
    const int b = (int)(bh / (uint32_t)p.H), h = (int)(bh % (uint32_t)p.H);
    float s = 0.f, l = 0.f, n2 = 0.f;     // n2: |dO row|^2, for the fixed-point scale of the fused backward
    if (r < p.T_q) {
      const T* po = reinterpret_cast<const T*>(p.o.ptr) + p.o.off(b, r, h);
      const T* pd = reinterpret_cast<const T*>(p.dout.ptr) + p.dout.off(b, r, h);
      uint4 a4[D / 64], d4[D / 64];
#pragma unroll
      for (int i = 0; i < D / 64; ++i) {
        a4[i] = *reinterpret_cast<const uint4*>(po + 64 * i + sub * 8);
        d4[i] = *reinterpret_cast<const uint4*>(pd + 64 * i + sub * 8);
      }
#pragma unroll
      for (int i = 0; i < D / 64; ++i) {
        const uint32_t av[4] = {a4[i].x, a4[i].y, a4[i].z, a4[i].w};
        const uint32_t dv[4] = {d4[i].x, d4[i].y, d4[i].z, d4[i].w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 x = Pack<T>::unpack(av[j]), y = Pack<T>::unpack(dv[j]);
          s = fmaf(x.x, y.x, fmaf(x.y, y.y, s));
          n2 = fmaf(y.x, y.x, fmaf(y.y, y.y, n2));
        }
      }
      if (sub == 0) l = p.lse[((int64_t)b * p.T_q + r) * p.H + h];
    }
    if (norm_t != nullptr) {
      n2 += __shfl_xor_sync(0xffffffffu, n2, 1);
      n2 += __shfl_xor_sync(0xffffffffu, n2, 2);
      n2 += __shfl_xor_sync(0xffffffffu, n2, 4);
      if (sub == 0) norm_t[(int64_t)bh * T_qp + r] = sqrtf(n2);
    }
    s += __shfl_xor_sync(0xffffffffu, s, 1);
    s += __shfl_xor_sync(0xffffffffu, s, 2);
    s += __shfl_xor_sync(0xffffffffu, s, 4);
    if (sub == 0) {
      delta_t[(int64_t)bh * T_qp + r] = s;     // rows in [T_q, T_qp) are written as zeros
      lse_t[(int64_t)bh * T_qp + r] = l;
    }
  }
}

// Control block shared by both kernels (placed after the tiles):
//   [0, 8*kMaxBars) mbarriers; then the TMEM base slot, the abort flag and the drain flag.
constexpr int kMaxBars = 24;
constexpr uint32_t kCtlBytes = 8 * kMaxBars + 32;
struct BwdBars {          // barrier indices for a ring of R slots
  int res, full0, empty0, s0, p0, done, r0, t0, i0;   // i0: "the score matmuls of a step have been issued" (dk/dv)
  __host__ __device__ constexpr explicit BwdBars(int R)
      : res(0), full0(1), empty0(1 + R), s0(1 + 2 * R), p0(3 + 2 * R), done(5 + 2 * R), r0(6 + 2 * R), t0(8 + 2 * R),
        i0(10 + 2 * R) {}
};
// A wait that is only a scheduling hint: a few short tries, then carry on whatever the outcome.
__device__ __forceinline__ void mbar_wait_hint(uint32_t bar, uint32_t parity) {
#pragma unroll 1
  for (int i = 0; i < 6; ++i) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity), "r"(400u) : "memory");
    if (ok) break;
  }
}
static_assert(9 + 2 * dq_ring<128>() < kMaxBars && 11 + 2 * dkv_ring<64>() < kMaxBars, "control block too small");

// Base of a 128-byte-swizzle descriptor for a tile at `addr`; per-MMA offsets (multiples of
// 16 bytes, staying inside the tile) are added to the low word.
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t addr) { return smem_desc_sw128(addr, 16, 1024); }
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t addr, uint32_t block_stride) {
  return smem_desc_sw128(addr, block_stride, 1024);
}
__device__ __forceinline__ uint64_t desc_add(uint64_t d, uint32_t byte_off) { return d + (uint64_t)(byte_off >> 4); }

// ============================================================================ dq
// grid (ceil(T_q/128), H, B), 384 threads.  TMEM (512 columns):
//   stage s in {0,1}: [s*128, +64) S (fp32), [s*128+64, +64) dP (fp32);
//   [256, 256+D) dQ (fp32);  [384, 384+D/2) Q (16-bit A operand);  [448, 448+D/2) dO (16-bit A operand).
// Shared memory: ring of dq_ring<D>() x {K step tile, V step tile} ([64 x D] each), then two
// [128 x 64] dS tiles (K-major, 128-byte swizzle).  A softmax warpgroup releases its TMEM stage
// as soon as it has the scores in registers, so the next-but-one score MMAs overlap its math;
// dS reaches the update MMA through shared memory - at D = 64 through TMEM instead: the 64-column
// accumulator leaves [320, 384) free for the two dS tiles as 16-bit A operands (32 columns each).
constexpr uint32_t kDqDsCol0 = 320;
template <typename T, int D>
__global__ void __launch_bounds__(kDqThreads, 1)
dq_kernel(const __grid_constant__ Params p, const __grid_constant__ DqMaps maps, const float* delta_t,
          const float* lse_t, int T_qp, const int* dq_acc, const float4* scale_blk) {
  constexpr int R = dq_ring<D>();
  constexpr BwdBars B_(R);
  // two issuing warps for the score matmuls at D = 128 (8 instructions each per step); at D = 64 a
  // step has 4 + 4 and one warp issues them faster than two warps take turns on the barriers
  constexpr bool kSplitScores = D == 128;
  constexpr uint32_t kStepTile = step_tile<D>();
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  const uint32_t base = smem_u32(smem_raw);
  if (base & 1023u) {   // the 128-byte swizzle needs 1024-byte aligned tiles
    if (threadIdx.x == 0) record_failure(2 << 8);
    return;
  }
  const uint32_t sRing = base;
  const uint32_t ds_off = R * 2 * kStepTile;            // two dS tiles of kScoreTile bytes
  const uint32_t sDS = base + ds_off;
  const uint32_t ctl_off = ds_off + 2 * kScoreTile;
  const uint32_t bars = base + ctl_off;
  unsigned char* gctl = smem_raw + ctl_off;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gctl + 8 * kMaxBars);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gctl + 8 * kMaxBars + 4);
  volatile int* drain_flag = reinterpret_cast<volatile int*>(gctl + 8 * kMaxBars + 8);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (*reinterpret_cast<volatile int*>(&g_tc_status) != 0) return;

  const int n_qt = (p.T_q + kBM - 1) / kBM;
  const BlockId bid = block_order(p, D);
  const int qt = n_qt - 1 - bid.rank;
  const int h = bid.h, b = bid.b;
  const int r0 = qt * kBM;
  int n_seq, n_dep, dep_c0, seq_full_hi;   // key walk in steps of 64
  {
    const int r_last = min(r0 + kBM, p.T_q) - 1;
    int lo, hi, lo2, hi2;
    seq_interval(p, r_last, lo, hi);
    n_seq = (hi + kStep - 1) / kStep;
    seq_interval(p, r0, lo2, hi2);
    seq_full_hi = hi2;
    dep_interval(p, r0, lo, hi);
    dep_interval(p, r_last, lo2, hi2);
    dep_c0 = lo;
    n_dep = (hi2 - lo + kStep - 1) / kStep;
  }
  // dq_acc != nullptr: the sequence keys' share of dQ is already in the fixed-point accumulator the
  // fused key-stationary kernel filled (tc_bwd_fused_kernel.cuh); this kernel then walks the depth
  // keys only and its epilogue adds the two shares.
  const bool seq_in_acc = dq_acc != nullptr;
  if (seq_in_acc) n_seq = 0;
  const int n = n_seq + n_dep;
  const int dep5 = (p.Ls != p.L) ? p.L : 0;      // in-place layer cache: 5-D depth maps

  if (tid == 0) {
    mbar_init(bars + 8 * B_.res, 256);
    mbar_init(bars + 8 * B_.done, 1);
    for (int i = 0; i < R; ++i) { mbar_init(bars + 8 * (B_.full0 + i), 1); mbar_init(bars + 8 * (B_.empty0 + i), 1); }
    for (int i = 0; i < 2; ++i) {
      mbar_init(bars + 8 * (B_.s0 + i), kSplitScores ? 2 : 1);    // one commit per score-MMA warp
      mbar_init(bars + 8 * (B_.p0 + i), 128);
      mbar_init(bars + 8 * (B_.r0 + i), 128); mbar_init(bars + 8 * (B_.t0 + i), 1);
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
  const uint32_t tmem_dQ = tmem + 256, tmem_Q = tmem + 384, tmem_dO = tmem + 448;
  constexpr uint32_t fmt = std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;

  if (warp == 9) {
    // ---------------------------------------------------------------- TMA warp
    {
      if (elect_one()) { prefetch_map(&maps.k); prefetch_map(&maps.v); }
      bool ok = true;
      int issued = 0;
      for (int i = 0; ok && i < n; ++i) {
        const uint32_t slot = i % R;
        if (i >= R && !(ok = mbar_wait(bars + 8 * (B_.empty0 + slot), ((i / R) - 1) & 1, abort_flag, B_.empty0 + slot))) break;
        const bool dep = i >= n_seq;
        const int row = dep ? dep_c0 + (i - n_seq) * kStep : i * kStep;
        const uint32_t dst = sRing + slot * 2 * kStepTile, bar = bars + 8 * (B_.full0 + slot);
        const CUtensorMap* mk = dep ? &maps.kd : &maps.k;
        const CUtensorMap* mv = dep ? &maps.vd : &maps.v;
        if (elect_one()) {
          mbar_expect_tx(bar, 2 * kStepTile);
          if (dep) {
            tma_load_dep_tile<D>(dst, mk, bar, kStepHalf, h, row, b, dep5);
            tma_load_dep_tile<D>(dst + kStepTile, mv, bar, kStepHalf, h, row, b, dep5);
          } else {
            tma_load_tile<D>(dst, mk, bar, kStepHalf, h, row, b);
            tma_load_tile<D>(dst + kStepTile, mv, bar, kStepHalf, h, row, b);
          }
        }
        __syncwarp();
        issued = i + 1;
      }
      if (!ok) {   // let loads in flight land before the CTA's shared memory is released
        for (int i = max(0, issued - R); i < issued; ++i)
          mbar_wait(bars + 8 * (B_.full0 + i % R), (i / R) & 1, drain_flag, B_.full0 + i % R);
      }
    }
  } else if (warp == 8 || warp == 11) {
    // ---------------------------------------------------------------- score-MMA warps
    // S(i) = Q K(i)^T (warp 8) and dP(i) = dO V(i)^T (warp 11, or warp 8 as well when the scores
    // are not split) into TMEM stage i&1, as soon as the warpgroup that owned the stage has the
    // previous scores in registers and the step tiles have landed.
    const bool is_s = warp == 8;
    if (n > 0 && (is_s || kSplitScores)) {
      constexpr uint32_t idesc_s = instr_desc(fmt, 64, false);
      bool ok = mbar_wait(bars + 8 * B_.res, 0, abort_flag, B_.res);   // Q, dO are in TMEM
      tc_fence_after();
      for (int i = 0; ok && i < n; ++i) {
        const uint32_t slot = i % R;
        if (i >= 2 && !(ok = mbar_wait(bars + 8 * (B_.r0 + (i & 1)), ((i - 2) >> 1) & 1, abort_flag, B_.r0 + (i & 1)))) break;
        if (!(ok = mbar_wait(bars + 8 * (B_.full0 + slot), (i / R) & 1, abort_flag, B_.full0 + slot))) break;
        tc_fence_after();
        const uint32_t sK = sRing + slot * 2 * kStepTile;
        const uint64_t dk = desc_kmajor(sK), dv = desc_kmajor(sK + kStepTile);
        const uint32_t tS = tmem + (i & 1) * 128, tP = tS + 64;
        // (each form is a straight run of instructions: a branch per matmul would cost more issue
        // time than the matmul)
        if (!kSplitScores) {
          if (elect_one()) {
#pragma unroll
            for (int kk = 0; kk < D / 16; ++kk) {
              mma_ts(tS, tmem_Q + kk * 8, desc_add(dk, (kk >> 2) * kStepHalf + (kk & 3) * 32), idesc_s, kk > 0);
              mma_ts(tP, tmem_dO + kk * 8, desc_add(dv, (kk >> 2) * kStepHalf + (kk & 3) * 32), idesc_s, kk > 0);
            }
            tc_commit(bars + 8 * (B_.s0 + (i & 1)));
          }
        } else {
          const uint32_t tAcc = is_s ? tS : tP, tA = is_s ? tmem_Q : tmem_dO;
          const uint64_t db = is_s ? dk : dv;
          if (elect_one()) {
#pragma unroll
            for (int kk = 0; kk < D / 16; ++kk)
              mma_ts(tAcc, tA + kk * 8, desc_add(db, (kk >> 2) * kStepHalf + (kk & 3) * 32), idesc_s, kk > 0);
            tc_commit(bars + 8 * (B_.s0 + (i & 1)));
          }
        }
        __syncwarp();
      }
    }
  } else if (warp == 10) {
    // ---------------------------------------------------------------- update-MMA warp
    // dQ += dS(j) K(j): A = dS tile in shared memory, B = K step tile read MN-major.  A warp of
    // its own, so that an update never waits behind the issue of the next scores.
    if (n > 0) {
      constexpr uint32_t idesc_t = instr_desc(fmt, D, true);
      bool ok = true;
      for (int j = 0; ok && j < n; ++j) {
        if (!(ok = mbar_wait(bars + 8 * (B_.p0 + (j & 1)), (j >> 1) & 1, abort_flag, B_.p0 + (j & 1)))) break;
        tc_fence_after();
        const uint32_t slot = j % R;
        const uint64_t da = desc_kmajor(sDS + (j & 1) * kScoreTile);
        const uint64_t dk = desc_mnmajor(sRing + slot * 2 * kStepTile, kStepHalf);
        const uint32_t tds = tmem + kDqDsCol0 + (j & 1) * 32;      // D = 64: dS in TMEM
        if (elect_one()) {
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) {
            if constexpr (D == 64) mma_ts(tmem_dQ, tds + kk * 8, desc_add(dk, kk * 2048), idesc_t, (j > 0 || kk > 0) ? 1u : 0u);
            else mma_ss(tmem_dQ, desc_add(da, kk * 32), desc_add(dk, kk * 2048), idesc_t, (j > 0 || kk > 0) ? 1u : 0u);
          }
          tc_commit(bars + 8 * (B_.empty0 + slot));      // slot j may be refilled
          tc_commit(bars + 8 * (B_.t0 + (j & 1)));       // dS tile j&1 may be rewritten
          if (j == n - 1) tc_commit(bars + 8 * B_.done);
        }
        __syncwarp();
      }
    }
  } else {
    // ---------------------------------------------------------------- softmax warpgroups
    const int wg = warp >> 2, quarter = warp & 3;   // warpgroup g takes steps i with (i & 1) == g
    const int row = quarter * 32 + lane;
    const int r = r0 + row;
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    {   // stage this thread's Q row (warpgroup 0) or dO row (warpgroup 1) into TMEM as an A operand
      uint32_t regs[D / 2];
      if (r < p.T_q) {
        const View& src = (wg == 0) ? p.q : p.dout;
        const uint4* g4 = reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(src.ptr) + src.off(b, r, h));
#pragma unroll
        for (int i = 0; i < D / 8; ++i) {
          const uint4 v4 = g4[i];
          regs[4 * i] = v4.x; regs[4 * i + 1] = v4.y; regs[4 * i + 2] = v4.z; regs[4 * i + 3] = v4.w;
        }
      } else {
#pragma unroll
        for (int i = 0; i < D / 2; ++i) regs[i] = 0u;
      }
      const uint32_t dst = ((wg == 0) ? tmem_Q : tmem_dO) + lane_addr;
      tmem_st32<0>(dst, regs);
      if constexpr (D == 128) tmem_st32<D / 2 - 32>(dst + 32, regs);
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(bars + 8 * B_.res);
    }
    int slo, shi, dlo, dhi;
    seq_interval(p, r, slo, shi);
    dep_interval(p, r, dlo, dhi);
    float lse_r = 0.f, dl_r = 0.f;
    if (r < p.T_q) {
      const int64_t idx = ((int64_t)b * p.H + h) * T_qp + r;
      lse_r = lse_t[idx]; dl_r = delta_t[idx];
    }
    const float c = p.scale_log2;
    bool ok = true;
    for (int i = wg; i < n; i += 2) {
      ok = __all_sync(0xffffffffu, mbar_wait(bars + 8 * (B_.s0 + (i & 1)), (i >> 1) & 1, abort_flag, B_.s0 + (i & 1)));
      if (!ok) break;
      tc_fence_after();
      const bool is_dep = i >= n_seq;
      const int c0 = is_dep ? dep_c0 + (i - n_seq) * kStep : i * kStep;
      const bool masked = is_dep || (c0 + kStep > seq_full_hi);
      const int lo = is_dep ? dlo : slo, hi = is_dep ? dhi : shi;
      const uint32_t tS = tmem + (i & 1) * 128 + lane_addr;
      uint32_t su[64], du[64];
      tmem_ld32<0>(tS, su);
      tmem_ld32<32>(tS + 32, su);
      tmem_ld32<0>(tS + 64, du);
      tmem_ld32<32>(tS + 96, du);
      tmem_wait_ld();
      tc_fence_before();
      mbar_arrive(bars + 8 * (B_.r0 + (i & 1)));      // scores are in registers: stage is free
      // straight-line passes over the 64 columns (no branches inside, so the scheduler can
      // overlap the exp2 latency of one column with the arithmetic of the others)
      // (packed fp32 pairs: the warps are bound by instruction issue, not by the exp2 unit)
      float pr[64];
      const float2 c2 = make_float2(c, c), nl2 = make_float2(-lse_r, -lse_r), nd2 = make_float2(-dl_r, -dl_r);
#pragma unroll
      for (int jj = 0; jj < 32; ++jj) {
        const float2 x = __ffma2_rn(make_float2(__uint_as_float(su[2 * jj]), __uint_as_float(su[2 * jj + 1])), c2, nl2);
        pr[2 * jj] = fast_exp2(x.x);
        pr[2 * jj + 1] = fast_exp2(x.y);
      }
      if (masked) {
#pragma unroll
        for (int jj = 0; jj < 64; ++jj) {
          const int col = c0 + jj;
          pr[jj] = (col >= lo && col < hi) ? pr[jj] : 0.f;
        }
      }
      uint32_t pk[32];
#pragma unroll
      for (int jj = 0; jj < 32; ++jj) {
        const float2 d = __fadd2_rn(make_float2(__uint_as_float(du[2 * jj]), __uint_as_float(du[2 * jj + 1])), nd2);
        const float2 ds = __fmul2_rn(make_float2(pr[2 * jj], pr[2 * jj + 1]), d);
        pk[jj] = Pack<T>::pack(ds.x, ds.y);
      }
      if (i >= 2) {   // the update of step i-2 must have finished reading this dS tile
        ok = __all_sync(0xffffffffu, mbar_wait(bars + 8 * (B_.t0 + (i & 1)), ((i - 2) >> 1) & 1, abort_flag, B_.t0 + (i & 1)));
        if (!ok) break;
      }
      if constexpr (D == 64) {
        // the 64-column accumulator leaves TMEM columns free at D = 64: dS goes there as the A operand
        // of the update matmul (packed pairs of key columns), not through shared memory
        tmem_st32<0>(tmem + kDqDsCol0 + (i & 1) * 32 + lane_addr, pk);
        tmem_wait_st();
        tc_fence_before();
      } else {   // row of the K-major, 128B-swizzled [128 x 64] tile: 16-byte chunk c lives at chunk c ^ (row & 7)
        unsigned char* prow = smem_raw + ds_off + (i & 1) * kScoreTile + row * 128;
#pragma unroll
        for (int ch = 0; ch < 8; ++ch)
          *reinterpret_cast<uint4*>(prow + ((ch ^ (row & 7)) << 4)) = make_uint4(pk[4 * ch], pk[4 * ch + 1], pk[4 * ch + 2], pk[4 * ch + 3]);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      }
#ifndef MODA_WAIT_TEST
      mbar_arrive(bars + 8 * (B_.p0 + (i & 1)));
#endif
      // (the wait-expiry test build withholds this arrival: the update warp's bounded wait on the
      // "tiles ready" barrier, which no TMA load targets, then runs out and the CTA leaves through
      // the teardown path)
    }
    if (ok && n > 0) ok = __all_sync(0xffffffffu, mbar_wait(bars + 8 * B_.done, 0, abort_flag, B_.done));
    if (ok && (n > 0 || seq_in_acc)) {
      tc_fence_after();
      T* gdq = reinterpret_cast<T*>(p.dq.ptr) + p.dq.off(b, r, h);
      const int64_t bh = (int64_t)b * p.H + h;
      const float inv = (seq_in_acc && r < p.T_q) ? scale_blk[bh * (T_qp / 64) + r / 64].y : 0.f;
      const int4* acc4 = seq_in_acc ? reinterpret_cast<const int4*>(dq_acc + (bh * T_qp + (r < p.T_q ? r : 0)) * D) : nullptr;
#pragma unroll
      for (int q4 = (D / 64) * wg; q4 < (D / 64) * (wg + 1); ++q4) {   // each warpgroup stores half of the row
        uint32_t ov[32];
        if (n > 0) {
          tmem_ld32<0>(tmem_dQ + lane_addr + q4 * 32, ov);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) ov[i] = 0u;
        }
        if (seq_in_acc && r < p.T_q) {
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int4 a = acc4[q4 * 8 + i];
            ov[4 * i + 0] = __float_as_uint(fmaf((float)a.x, inv, __uint_as_float(ov[4 * i + 0])));
            ov[4 * i + 1] = __float_as_uint(fmaf((float)a.y, inv, __uint_as_float(ov[4 * i + 1])));
            ov[4 * i + 2] = __float_as_uint(fmaf((float)a.z, inv, __uint_as_float(ov[4 * i + 2])));
            ov[4 * i + 3] = __float_as_uint(fmaf((float)a.w, inv, __uint_as_float(ov[4 * i + 3])));
          }
        }
        if (r < p.T_q) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint4* dst = reinterpret_cast<uint4*>(gdq + q4 * 32 + i * 8);
            *dst = p.merge_depth ? pack8_blend<T>(ov + i * 8, p.scale, *dst, 1.f) : pack8_scaled<T>(ov + i * 8, p.scale);
          }
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

// =========================================================================== dk / dv
// grid (n_seq_key_tiles + n_dep_key_tiles, H, B), 384 threads; key tiles of 128.
// TMEM (512 columns): [0, 64) S^T and [64, 128) dP^T (one fp32 score stage);
//   [128, 128+D) dV; [256, 256+D) dK; [384, 384+D/2) K and [448, 448+D/2) V rows as 16-bit A operands;
//   at D = 64 also [192, 256) and [320, 384): the two {P^T, dS^T} pairs as 16-bit A operands.
// Shared memory: ring of dkv_ring<D>() x {Q step tile, dO step tile}; two {P^T, dS^T} tile pairs
// ([128 keys x 64 rows], K-major, 128-byte swizzle), one per softmax warpgroup; the ring of
// {64 lse, 64 delta}.  A warpgroup releases the score stage as soon as the scores are in its
// registers, so the next step's score MMAs overlap its math; P^T and dS^T reach the update
// MMAs through shared memory.
constexpr uint32_t kDkvPairBytes = 2 * kScoreTile;   // P^T tile + dS^T tile
// D = 64: the two {P^T, dS^T} pairs live in TMEM columns the 64-column accumulators leave free
// ([192, 256) and [320, 384): P^T in the first 32 columns of a pair, dS^T in the next 32)
constexpr uint32_t kDkvPairCol0 = 192, kDkvPairColStride = 128;

template <typename T, int D>
__global__ void __launch_bounds__(kDkvThreads, 1)
dkv_kernel(const __grid_constant__ Params p, const __grid_constant__ DkvMaps maps, const float* delta_t,
           const float* lse_t, int T_qp, int n_seq_key_tiles) {
  constexpr int R = dkv_ring<D>();
  constexpr BwdBars B_(R);
  constexpr uint32_t kStepTile = step_tile<D>();
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  const uint32_t base = smem_u32(smem_raw);
  if (base & 1023u) {
    if (threadIdx.x == 0) record_failure(2 << 8);
    return;
  }
  const uint32_t sRing = base;
  const uint32_t pt_off = R * 2 * kStepTile;
  const uint32_t sPT = base + pt_off;
  const uint32_t stat_off = pt_off + 2 * kDkvPairBytes;
  const uint32_t sStat = base + stat_off;
  const uint32_t ctl_off = stat_off + R * 512;
  const uint32_t bars = base + ctl_off;
  unsigned char* gctl = smem_raw + ctl_off;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gctl + 8 * kMaxBars);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gctl + 8 * kMaxBars + 4);
  volatile int* drain_flag = reinterpret_cast<volatile int*>(gctl + 8 * kMaxBars + 8);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (*reinterpret_cast<volatile int*>(&g_tc_status) != 0) return;

  const BlockId bid = block_order(p, D);
  const int h = bid.h, b = bid.b;
  const bool is_dep = bid.rank >= n_seq_key_tiles;
  const int c0 = (is_dep ? bid.rank - n_seq_key_tiles : bid.rank) * kBN;
  const int n_keys = is_dep ? p.T_kv * p.L : p.T_kv;
  const int c_last = min(c0 + kBN, n_keys) - 1;

  // query rows that can see a key of this tile: [q_begin, q_end), walked in steps of 64
  int q_begin, q_end;
  if (!is_dep) {
    q_begin = (p.mode == kNonCausal) ? 0 : c0 * p.G;
    q_end = p.T_q;
  } else {
    const int p_lo = c0 / p.L, p_hi = c_last / p.L;
    q_begin = p_lo * p.G;
    const int t_end = (p.mode == kChunkVisible) ? min((p_hi / p.Cb + 1) * p.Cb, p.T_kv) : p_hi + 1;
    q_end = t_end * p.G;
  }
  q_begin = (q_begin / kStep) * kStep;
  const int n = (q_end - q_begin + kStep - 1) / kStep;

  if (tid == 0) {
    mbar_init(bars + 8 * B_.res, 256);
    mbar_init(bars + 8 * B_.done, 1);
    for (int i = 0; i < R; ++i) { mbar_init(bars + 8 * (B_.full0 + i), 1); mbar_init(bars + 8 * (B_.empty0 + i), 1); }
    for (int i = 0; i < 2; ++i) {
      mbar_init(bars + 8 * (B_.s0 + i), 2);    // one commit per score-MMA warp
      mbar_init(bars + 8 * (B_.i0 + i), 2);    // one arrival per score-MMA warp
      mbar_init(bars + 8 * (B_.p0 + i), 128);
      mbar_init(bars + 8 * (B_.r0 + i), 128); mbar_init(bars + 8 * (B_.t0 + i), 1);
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
  const uint32_t tmem_K = tmem + 384, tmem_V = tmem + 448;
  constexpr uint32_t fmt = std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;
  const int64_t stat_base = ((int64_t)b * p.H + h) * T_qp;

  if (warp == 9) {
    // ---------------------------------------------------------------- TMA warp
    if (n > 0) {
      if (elect_one()) { prefetch_map(&maps.q); prefetch_map(&maps.dout); }
      bool ok = true;
      int issued = 0;
      for (int i = 0; ok && i < n; ++i) {
        const uint32_t slot = i % R;
        if (i >= R && !(ok = mbar_wait(bars + 8 * (B_.empty0 + slot), ((i / R) - 1) & 1, abort_flag, B_.empty0 + slot))) break;
        const int row = q_begin + i * kStep;
        const uint32_t dst = sRing + slot * 2 * kStepTile, bar = bars + 8 * (B_.full0 + slot);
        const uint32_t st = sStat + slot * 512;
        if (elect_one()) {
          mbar_expect_tx(bar, 2 * kStepTile + 512);
          tma_load_tile<D>(dst, &maps.q, bar, kStepHalf, h, row, b);
          tma_load_tile<D>(dst + kStepTile, &maps.dout, bar, kStepHalf, h, row, b);
          bulk_load(st, lse_t + stat_base + row, 256, bar);
          bulk_load(st + 256, delta_t + stat_base + row, 256, bar);
        }
        __syncwarp();
        issued = i + 1;
      }
      if (!ok) {   // let loads in flight land before the CTA's shared memory is released
        for (int i = max(0, issued - R); i < issued; ++i)
          mbar_wait(bars + 8 * (B_.full0 + i % R), (i / R) & 1, drain_flag, B_.full0 + i % R);
      }
    }
  } else if (warp == 8 || warp == 11) {
    // ---------------------------------------------------------------- score-MMA warps
    // S^T(i) = K Q(i)^T (warp 8) and dP^T(i) = V dO(i)^T (warp 11), A from TMEM, into the score stage,
    // as soon as the previous step's scores have been read into registers and the step tiles have landed.
    const bool is_s = warp == 8;
    if (n > 0) {
      constexpr uint32_t idesc_s = instr_desc(fmt, 64, false);
      bool ok = mbar_wait(bars + 8 * B_.res, 0, abort_flag, B_.res);   // K, V are in TMEM
      tc_fence_after();
      for (int i = 0; ok && i < n; ++i) {
        const uint32_t slot = i % R;
        if (i >= 1 && !(ok = mbar_wait(bars + 8 * (B_.r0 + ((i - 1) & 1)), ((i - 1) >> 1) & 1, abort_flag, B_.r0 + ((i - 1) & 1)))) break;
        if (!(ok = mbar_wait(bars + 8 * (B_.full0 + slot), (i / R) & 1, abort_flag, B_.full0 + slot))) break;
        tc_fence_after();
        const uint32_t sQ = sRing + slot * 2 * kStepTile;
        const uint64_t db = desc_kmajor(is_s ? sQ : sQ + kStepTile);
        const uint32_t tAcc = is_s ? tmem_S : tmem_P, tA = is_s ? tmem_K : tmem_V;
        if (elect_one()) {
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk)
            mma_ts(tAcc, tA + kk * 8, desc_add(db, (kk >> 2) * kStepHalf + (kk & 3) * 32), idesc_s, kk > 0);
          tc_commit(bars + 8 * (B_.s0 + (i & 1)));
          mbar_arrive(bars + 8 * (B_.i0 + (i & 1)));     // issued, not yet executed (see the update warp)
        }
        __syncwarp();
      }
    }
  } else if (warp == 10) {
    // ---------------------------------------------------------------- update-MMA warp
    // dV += P^T(j) dO(j) and dK += dS^T(j) Q(j): A = tiles written by warpgroup j&1, B = the
    // step tiles read MN-major.
    if (n > 0) {
      constexpr uint32_t idesc_t = instr_desc(fmt, D, true);
      bool ok = true;
      for (int j = 0; ok && j < n; ++j) {
        if (!(ok = mbar_wait(bars + 8 * (B_.p0 + (j & 1)), (j >> 1) & 1, abort_flag, B_.p0 + (j & 1)))) break;
        // The tensor pipe executes matmuls in the order they arrive.  The scores of step j+2 become
        // issuable at about the time these tiles become ready, and they are what the single score
        // stage - and with it the softmax warps - waits for, while nothing waits for this update:
        // let the scores go first.  A hint, not a dependency: the wait is short and falls through.
        if (j + 2 < n) mbar_wait_hint(bars + 8 * (B_.i0 + (j & 1)), ((j + 2) >> 1) & 1);
        tc_fence_after();
        const uint32_t slot = j % R, sQ = sRing + slot * 2 * kStepTile;
        const uint64_t dq = desc_mnmajor(sQ, kStepHalf), ddo = desc_mnmajor(sQ + kStepTile, kStepHalf);
        const uint64_t dpt = desc_kmajor(sPT + (j & 1) * kDkvPairBytes), dst = desc_kmajor(sPT + (j & 1) * kDkvPairBytes + kScoreTile);
        const uint32_t tpair = tmem + kDkvPairCol0 + (j & 1) * kDkvPairColStride;   // D = 64: P^T, dS^T in TMEM
        if (elect_one()) {
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) {
            if constexpr (D == 64) {
              mma_ts(tmem_dV, tpair + kk * 8, desc_add(ddo, kk * 2048), idesc_t, (j > 0 || kk > 0) ? 1u : 0u);
              mma_ts(tmem_dK, tpair + 32 + kk * 8, desc_add(dq, kk * 2048), idesc_t, (j > 0 || kk > 0) ? 1u : 0u);
            } else {
              mma_ss(tmem_dV, desc_add(dpt, kk * 32), desc_add(ddo, kk * 2048), idesc_t, (j > 0 || kk > 0) ? 1u : 0u);
              mma_ss(tmem_dK, desc_add(dst, kk * 32), desc_add(dq, kk * 2048), idesc_t, (j > 0 || kk > 0) ? 1u : 0u);
            }
          }
          tc_commit(bars + 8 * (B_.empty0 + slot));      // ring slot j may be refilled
          tc_commit(bars + 8 * (B_.t0 + (j & 1)));       // tile pair j&1 may be rewritten
          if (j == n - 1) tc_commit(bars + 8 * B_.done);
        }
        __syncwarp();
      }
    }
  } else {
    // ---------------------------------------------------------------- softmax warpgroups
    const int wg = warp >> 2, quarter = warp & 3;   // warpgroup g takes steps i with (i & 1) == g
    const int row = quarter * 32 + lane;             // key row of the tile == TMEM lane
    const int key = c0 + row;
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    {   // stage this thread's K row (warpgroup 0) or V row (warpgroup 1) into TMEM as an A operand
      uint32_t regs[D / 2];
      if (key < n_keys) {
        const View& src = (wg == 0) ? (is_dep ? p.kd : p.k) : (is_dep ? p.vd : p.v);
        const uint4* g4 = reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(src.ptr) +
                                                         src.off(b, is_dep ? dep_mem_row(p, key) : (int64_t)key, h));
#pragma unroll
        for (int i = 0; i < D / 8; ++i) {
          const uint4 v4 = g4[i];
          regs[4 * i] = v4.x; regs[4 * i + 1] = v4.y; regs[4 * i + 2] = v4.z; regs[4 * i + 3] = v4.w;
        }
      } else {
#pragma unroll
        for (int i = 0; i < D / 2; ++i) regs[i] = 0u;
      }
      const uint32_t dst = ((wg == 0) ? tmem_K : tmem_V) + lane_addr;
      tmem_st32<0>(dst, regs);
      if constexpr (D == 128) tmem_st32<D / 2 - 32>(dst + 32, regs);
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(bars + 8 * B_.res);
    }
    // query rows [rlo, rhi) that see this key (the visibility rule of common.cuh, inverted)
    int rlo, rhi;
    if (key >= n_keys) { rlo = 0; rhi = 0; }
    else if (!is_dep) { rlo = (p.mode == kNonCausal) ? 0 : key * p.G; rhi = p.T_q; }
    else {
      const int tp = key / p.L;
      rlo = tp * p.G;
      rhi = ((p.mode == kChunkVisible) ? min((tp / p.Cb + 1) * p.Cb, p.T_kv) : tp + 1) * p.G;
    }
    // a step [q0, q0+64) needs no mask iff every valid key of the tile sees all 64 rows
    const int tile_rlo_max = is_dep ? 0x7fffffff : ((p.mode == kNonCausal) ? 0 : c_last * p.G);
    const bool tail_keys = (c0 + kBN > n_keys);
    const float c = p.scale_log2;
    bool ok = true;
    for (int i = wg; i < n; i += 2) {
      const uint32_t slot = i % R;
      ok = __all_sync(0xffffffffu, mbar_wait(bars + 8 * (B_.full0 + slot), (i / R) & 1, abort_flag, B_.full0 + slot));
      if (!ok) break;
      ok = __all_sync(0xffffffffu, mbar_wait(bars + 8 * (B_.s0 + (i & 1)), (i >> 1) & 1, abort_flag, B_.s0 + (i & 1)));
      if (!ok) break;
      tc_fence_after();
      const int q0 = q_begin + i * kStep;
      const bool masked = is_dep || tail_keys || q0 < tile_rlo_max || q0 + kStep > p.T_q;
      const float4* st4 = reinterpret_cast<const float4*>(smem_raw + stat_off + slot * 512);
      uint32_t su[64], du[64];
      tmem_ld32<0>(tmem_S + lane_addr, su);
      tmem_ld32<32>(tmem_S + lane_addr + 32, su);
      tmem_ld32<0>(tmem_P + lane_addr, du);
      tmem_ld32<32>(tmem_P + lane_addr + 32, du);
      tmem_wait_ld();
      tc_fence_before();
      mbar_arrive(bars + 8 * (B_.r0 + (i & 1)));      // scores are in registers: the stage is free
      // (packed fp32 pairs: the warps are bound by instruction issue, not by the exp2 unit)
      float pr[64], dd[64];
      const float2 c2 = make_float2(c, c);
#pragma unroll
      for (int j4 = 0; j4 < 16; ++j4) {
        const float4 l4 = st4[j4], d4 = st4[16 + j4];
        const float2 x0 = __ffma2_rn(make_float2(__uint_as_float(su[4 * j4 + 0]), __uint_as_float(su[4 * j4 + 1])), c2, make_float2(-l4.x, -l4.y));
        const float2 x1 = __ffma2_rn(make_float2(__uint_as_float(su[4 * j4 + 2]), __uint_as_float(su[4 * j4 + 3])), c2, make_float2(-l4.z, -l4.w));
        pr[4 * j4 + 0] = fast_exp2(x0.x);
        pr[4 * j4 + 1] = fast_exp2(x0.y);
        pr[4 * j4 + 2] = fast_exp2(x1.x);
        pr[4 * j4 + 3] = fast_exp2(x1.y);
        const float2 e0 = __fadd2_rn(make_float2(__uint_as_float(du[4 * j4 + 0]), __uint_as_float(du[4 * j4 + 1])), make_float2(-d4.x, -d4.y));
        const float2 e1 = __fadd2_rn(make_float2(__uint_as_float(du[4 * j4 + 2]), __uint_as_float(du[4 * j4 + 3])), make_float2(-d4.z, -d4.w));
        dd[4 * j4 + 0] = e0.x; dd[4 * j4 + 1] = e0.y; dd[4 * j4 + 2] = e1.x; dd[4 * j4 + 3] = e1.y;
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
        const float2 ds = __fmul2_rn(make_float2(pr[2 * jj], pr[2 * jj + 1]), make_float2(dd[2 * jj], dd[2 * jj + 1]));
        pd[jj] = Pack<T>::pack(ds.x, ds.y);
      }
      if (i >= 2) {   // the update of step i-2 must have finished reading this warpgroup's tile pair
        ok = __all_sync(0xffffffffu, mbar_wait(bars + 8 * (B_.t0 + (i & 1)), ((i - 2) >> 1) & 1, abort_flag, B_.t0 + (i & 1)));
        if (!ok) break;
      }
      if constexpr (D == 64) {
        // the accumulators leave TMEM columns free at D = 64: P^T and dS^T go there as the A operands
        // of the update matmuls (packed pairs of query columns, 32 columns each), not through shared memory
        const uint32_t tpair = tmem + kDkvPairCol0 + (i & 1) * kDkvPairColStride + lane_addr;
        tmem_st32<0>(tpair, pp);
        tmem_st32<0>(tpair + 32, pd);
        tmem_wait_st();
        tc_fence_before();
      } else {   // rows of the K-major, 128B-swizzled [128 x 64] tiles: 16-byte chunk c lives at chunk c ^ (row & 7)
        unsigned char* prow = smem_raw + pt_off + (i & 1) * kDkvPairBytes + row * 128;
#pragma unroll
        for (int ch = 0; ch < 8; ++ch) {
          const uint32_t o = (uint32_t)((ch ^ (row & 7)) << 4);
          *reinterpret_cast<uint4*>(prow + o) = make_uint4(pp[4 * ch], pp[4 * ch + 1], pp[4 * ch + 2], pp[4 * ch + 3]);
          *reinterpret_cast<uint4*>(prow + kScoreTile + o) = make_uint4(pd[4 * ch], pd[4 * ch + 1], pd[4 * ch + 2], pd[4 * ch + 3]);
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      }
#ifndef MODA_WAIT_TEST
      mbar_arrive(bars + 8 * (B_.p0 + (i & 1)));
#endif
      // (the wait-expiry test build withholds this arrival: the update warp's bounded wait on the
      // "tiles ready" barrier, which no TMA load targets, then runs out and the CTA leaves through
      // the teardown path)
    }
    if (ok && n > 0) ok = __all_sync(0xffffffffu, mbar_wait(bars + 8 * B_.done, 0, abort_flag, B_.done));
    if (ok && n > 0) {
      tc_fence_after();
      const View& ov = (wg == 0) ? (is_dep ? p.dvd : p.dv) : (is_dep ? p.dkd : p.dk);
      T* gout = reinterpret_cast<T*>(ov.ptr) + ov.off(b, is_dep ? dep_mem_row(p, key) : (int64_t)key, h);
      const bool acc = is_dep && p.acc_depth != 0;   // depth gradients added to a cache shared by several layers
      const uint32_t tsrc = (wg == 0) ? tmem_dV : tmem_dK;      // warpgroup 0 stores dV, warpgroup 1 dK
      const float mul = (wg == 0) ? 1.f : p.scale;
#pragma unroll
      for (int q4 = 0; q4 < D / 32; ++q4) {
        uint32_t ov32[32];
        tmem_ld32<0>(tsrc + lane_addr + q4 * 32, ov32);
        tmem_wait_ld();
        if (key < n_keys) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint4 v4;
            v4.x = Pack<T>::pack(__uint_as_float(ov32[i * 8 + 0]) * mul, __uint_as_float(ov32[i * 8 + 1]) * mul);
            v4.y = Pack<T>::pack(__uint_as_float(ov32[i * 8 + 2]) * mul, __uint_as_float(ov32[i * 8 + 3]) * mul);
            v4.z = Pack<T>::pack(__uint_as_float(ov32[i * 8 + 4]) * mul, __uint_as_float(ov32[i * 8 + 5]) * mul);
            v4.w = Pack<T>::pack(__uint_as_float(ov32[i * 8 + 6]) * mul, __uint_as_float(ov32[i * 8 + 7]) * mul);
            uint4* dst = reinterpret_cast<uint4*>(gout + q4 * 32 + i * 8);
            *dst = acc ? pack8_blend<T>(ov32 + i * 8, mul, *dst, 1.f) : v4;
          }
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

// ==================================================================== depth dk / dv
// Gradients of the depth K/V, query-stationary: the depth rows a block of 64 query rows can
// see (its chunk's rows, or its positions' rows) are seen by no other query row when 64 is a
// multiple of G (and of the chunk), so one CTA per (64-row block, h, b) owns them outright.
// The CTA keeps the block's Q, dO, lse, delta in shared memory and streams its depth keys in
// tiles of 128 (TMA, two buffers): S^T = Kd Q^T, dP^T = Vd dO^T (SS, N = 64) -> softmax
// threads (thread = key row) write P^T and dS^T over the scores in TMEM -> dVd = P^T dO,
// dKd = dS^T Q (TS, fresh accumulators) -> rows stored.  A key-tile CTA of dkv_kernel would
// spend its whole life in set-up for the one or two steps such keys have; here the set-up is
// paid once per 64 query rows.
//
// Two score stages in TMEM let the scores of tile i+1 be issued ahead of the updates of tile i,
// and the softmax threads work in the order softmax(i+1), then store(i): the tensor pipe runs
// the updates of tile i under softmax(i+1) and the scores of tile i+2 under store(i).
//
// The two [128 x 128] gradient tiles of a key tile leave through shared memory and TMA tile
// stores, one 32-row box per warp (a warp stages and stores its own rows, so no barrier is
// involved, only the issuing lane's bulk-group wait before the rows are reused).  Stored
// row-wise instead - a thread owns one key row, 32 threads each writing 16 bytes of their own
// row per instruction - every store instruction half-fills 32 sectors, and the stores were the
// longest phase of a tile.  A warp whose 32 rows are not all this block's (window not a multiple
// of 32 rows) keeps the row-wise stores, masked per row.
// Eight softmax / store warps: warp w and warp w + 4 share TMEM lanes 32 (w & 3) .. + 31 (key
// rows); warps 0-3 take query columns [0,32) of the scores and stage dVd, warps 4-7 take query
// columns [32,64) and stage dKd.
// Persistent: one CTA per SM walks the (64-row block, h, b) list with a stride of the grid, so
// the TMEM allocation and barrier set-up are paid once per SM and the key tiles of the next
// block are already on their way while the current one finishes; only Q, dO and the row
// statistics (single-buffered) wait for the previous block's last update MMAs.
// grid (min(blocks, SMs)), 320 threads.  TMEM (512 columns): stage s at [128 s, 128 s + 64)
// S^T / P^T and [128 s + 64, 128 s + 128) dP^T / dS^T (the packed 16-bit P^T / dS^T of query
// columns 32 g .. + 31 sit in the first 16 columns of that group's 32 fp32 columns);
// [256,256+D) dVd, [384,384+D) dKd.
enum DgBar : int { kDgRes = 0, kDgFull0 = 1, kDgEmpty0 = 3, kDgS0 = 5, kDgP0 = 7, kDgU = 9, kDgE = 10, kDgQFree = 11, kDgCount = 12 };
template <int D> __host__ __device__ constexpr uint32_t dg_out_off() { return 2 * step_tile<D>() + 1024 + 2 * 2 * tile_bytes<D>(); }   // {dVd tile, dKd tile} staging
template <int D> __host__ __device__ constexpr uint32_t dg_smem() { return dg_out_off<D>() + 2 * tile_bytes<D>() + 128; }
struct DgOutMaps { CUtensorMap dkd, dvd; };                                     // 32-row boxes
constexpr int kDgThreads = 320;                                                 // 8 softmax/store warps, MMA warp, TMA warp

// One 64-row query block of the depth-gradient kernel.
struct DgBlock { int q0, h, b, k_lo, k_hi, n; int64_t stat_base; };
__device__ __forceinline__ DgBlock dg_block(const Params& p, int idx, int n_xb, int T_qp) {
  DgBlock k;
  const int xb = idx % n_xb, hb = idx / n_xb;
  k.h = hb % p.H;
  k.b = hb / p.H;
  k.q0 = xb * kStep;
  const int r_last = min(k.q0 + kStep, p.T_q) - 1;
  int tmp;
  dep_interval(p, k.q0, k.k_lo, tmp);
  dep_interval(p, r_last, tmp, k.k_hi);
  k.n = (k.k_hi - k.k_lo + kBN - 1) / kBN;              // key tiles of 128
  k.stat_base = ((int64_t)k.b * p.H + k.h) * T_qp;
  return k;
}

template <typename T, int D>
__global__ void __launch_bounds__(kDgThreads, 1)
depth_grad_kernel(const __grid_constant__ Params p, const __grid_constant__ DkvMaps maps,
                  const __grid_constant__ DgOutMaps omaps, const float* delta_t, const float* lse_t, int T_qp) {
  constexpr uint32_t kStepTile = step_tile<D>(), kTile = tile_bytes<D>(), kDgOutOff = dg_out_off<D>();
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  const uint32_t base = smem_u32(smem_raw);
  if (base & 1023u) {
    if (threadIdx.x == 0) record_failure(2 << 8);
    return;
  }
  const uint32_t sQ = base, sDO = base + kStepTile, sStat = base + 2 * kStepTile;
  const uint32_t sKV = base + 2 * kStepTile + 1024;          // 2 x {Kd tile, Vd tile}
  const uint32_t sOut = base + kDgOutOff;
  const uint32_t ctl_off = kDgOutOff + 2 * kTile;
  const uint32_t bars = base + ctl_off;
  unsigned char* gctl = smem_raw + ctl_off;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gctl + 104);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gctl + 108);
  volatile int* drain_flag = reinterpret_cast<volatile int*>(gctl + 112);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (*reinterpret_cast<volatile int*>(&g_tc_status) != 0) return;

  const int n_xb = (p.T_q + kStep - 1) / kStep;
  const int total = n_xb * p.H * p.B;                   // 64-row blocks; this CTA takes blockIdx.x, + gridDim.x, ...
  const int dep5 = (p.Ls != p.L) ? p.L : 0;             // in-place layer cache: 5-D depth maps

  if (tid == 0) {
    mbar_init(bars + 8 * kDgRes, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(bars + 8 * (kDgFull0 + i), 1);
      mbar_init(bars + 8 * (kDgEmpty0 + i), 1);
      mbar_init(bars + 8 * (kDgS0 + i), 1);
      mbar_init(bars + 8 * (kDgP0 + i), 256);
    }
    mbar_init(bars + 8 * kDgU, 1);
    mbar_init(bars + 8 * kDgE, 256);
    mbar_init(bars + 8 * kDgQFree, 1);
    *abort_flag = 0;
    *drain_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 0) {
    tmem_alloc(bars + 104, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tmem_dV = tmem + 256, tmem_dK = tmem + 384;   // score stage s: tmem + 128 s (+ 64 for dP^T)
  constexpr uint32_t fmt = std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;

  // Every role walks the same blocks in the same order; g counts key tiles and kb blocks since the
  // CTA started, and all slot / stage / phase choices derive from them.
  if (warp == 9) {
    // ---------------------------------------------------------------- TMA warp
    if (elect_one()) { prefetch_map(&maps.q); prefetch_map(&maps.dout); prefetch_map(&maps.kd); prefetch_map(&maps.vd); }
    __syncwarp();
    bool ok = true;
    int g = 0, kb = 0;
    int issued = 0, res_kb = -1;                        // key tiles / block loads issued so far
    for (int idx = blockIdx.x; ok && idx < total; idx += gridDim.x) {
      const DgBlock k = dg_block(p, idx, n_xb, T_qp);
      if (k.n <= 0) continue;
      auto load_tile = [&](int i) -> bool {
        const int gi = g + i;
        const uint32_t slot = gi & 1;
        if (gi >= 2 && !mbar_wait(bars + 8 * (kDgEmpty0 + slot), ((gi >> 1) - 1) & 1, abort_flag, kDgEmpty0 + slot)) return false;
        const int row = k.k_lo + i * kBN;
        const uint32_t dst = sKV + slot * 2 * kTile, bar = bars + 8 * (kDgFull0 + slot);
        if (elect_one()) {
          mbar_expect_tx(bar, 2 * kTile);
          tma_load_dep_tile<D>(dst, &maps.kd, bar, kHalfBytes, k.h, row, k.b, dep5);
          tma_load_dep_tile<D>(dst + kTile, &maps.vd, bar, kHalfBytes, k.h, row, k.b, dep5);
        }
        __syncwarp();
        issued = gi + 1;
        return true;
      };
      // the first two key tiles only need free slots; Q, dO and the row statistics replace the
      // previous block's, which its last update MMAs still read
      int i = 0;
      for (; ok && i < min(k.n, 2); ++i) ok = load_tile(i);
      if (!ok) break;
      if (kb >= 1 && !(ok = mbar_wait(bars + 8 * kDgQFree, (kb - 1) & 1, abort_flag, kDgQFree))) break;
      if (elect_one()) {
        mbar_expect_tx(bars + 8 * kDgRes, 2 * kStepTile + 512);
        tma_load_tile<D>(sQ, &maps.q, bars + 8 * kDgRes, kStepHalf, k.h, k.q0, k.b);
        tma_load_tile<D>(sDO, &maps.dout, bars + 8 * kDgRes, kStepHalf, k.h, k.q0, k.b);
        bulk_load(sStat, lse_t + k.stat_base + k.q0, 256, bars + 8 * kDgRes);
        bulk_load(sStat + 256, delta_t + k.stat_base + k.q0, 256, bars + 8 * kDgRes);
      }
      __syncwarp();
      res_kb = kb;
      for (; ok && i < k.n; ++i) ok = load_tile(i);
      if (!ok) break;
      g += k.n;
      ++kb;
    }
    if (!ok) {   // let what is in flight land before the CTA's smem goes
      if (res_kb >= 0) mbar_wait(bars + 8 * kDgRes, res_kb & 1, drain_flag, kDgRes);
      for (int gi = max(0, issued - 2); gi < issued; ++gi)
        mbar_wait(bars + 8 * (kDgFull0 + (gi & 1)), (gi >> 1) & 1, drain_flag, kDgFull0 + (gi & 1));
    }
  } else if (warp == 8) {
    // ---------------------------------------------------------------- MMA warp
    constexpr uint32_t idesc_s = instr_desc(fmt, 64, false);
    constexpr uint32_t idesc_t = instr_desc(fmt, D, true);
    const uint64_t dq_k = desc_kmajor(sQ), ddo_k = desc_kmajor(sDO);
    const uint64_t dq_mn = desc_mnmajor(sQ, kStepHalf), ddo_mn = desc_mnmajor(sDO, kStepHalf);
    // scores of tile gj into stage gj & 1; the updates that read that stage last (tile gj - 2) were
    // issued before, and the pipe runs in issue order
    auto scores = [&](int gj) -> bool {
      const uint32_t slot = gj & 1;
      if (!mbar_wait(bars + 8 * (kDgFull0 + slot), (gj >> 1) & 1, abort_flag, kDgFull0 + slot)) return false;
      tc_fence_after();
      const uint64_t dK = desc_kmajor(sKV + slot * 2 * kTile), dV = desc_kmajor(sKV + slot * 2 * kTile + kTile);
      const uint32_t tS = tmem + slot * 128, tP = tS + 64;
      if (elect_one()) {
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          mma_ss(tS, desc_add(dK, (kk >> 2) * kHalfBytes + (kk & 3) * 32), desc_add(dq_k, (kk >> 2) * kStepHalf + (kk & 3) * 32), idesc_s, kk > 0);
          mma_ss(tP, desc_add(dV, (kk >> 2) * kHalfBytes + (kk & 3) * 32), desc_add(ddo_k, (kk >> 2) * kStepHalf + (kk & 3) * 32), idesc_s, kk > 0);
        }
        tc_commit(bars + 8 * (kDgS0 + slot));
        tc_commit(bars + 8 * (kDgEmpty0 + slot));      // Kd/Vd tile gj has been read
      }
      __syncwarp();
      return true;
    };
    bool ok = true;
    int g = 0, kb = 0;
    for (int idx = blockIdx.x; ok && idx < total; idx += gridDim.x) {
      const DgBlock k = dg_block(p, idx, n_xb, T_qp);
      if (k.n <= 0) continue;
      if (!(ok = mbar_wait(bars + 8 * kDgRes, kb & 1, abort_flag, kDgRes))) break;
      if (!(ok = scores(g))) break;
      for (int i = 0; ok && i < k.n; ++i) {
        const int gi = g + i;
        if (i + 1 < k.n && !(ok = scores(gi + 1))) break;
        if (!(ok = mbar_wait(bars + 8 * (kDgP0 + (gi & 1)), (gi >> 1) & 1, abort_flag, kDgP0 + (gi & 1)))) break;   // P^T, dS^T written
        if (gi >= 1 && !(ok = mbar_wait(bars + 8 * kDgE, (gi - 1) & 1, abort_flag, kDgE))) break;   // accumulators of tile gi-1 read
        tc_fence_after();
        const uint32_t tS = tmem + (gi & 1) * 128, tP = tS + 64;
        if (elect_one()) {
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) {
            const uint32_t acol = (kk >> 1) * 32 + (kk & 1) * 8;   // query rows 16 kk .. + 15 of P^T / dS^T
            mma_ts(tmem_dV, tS + acol, desc_add(ddo_mn, kk * 2048), idesc_t, kk > 0);
            mma_ts(tmem_dK, tP + acol, desc_add(dq_mn, kk * 2048), idesc_t, kk > 0);
          }
          tc_commit(bars + 8 * kDgU);
          if (i + 1 == k.n) tc_commit(bars + 8 * kDgQFree);   // the block's Q, dO, statistics are done with
        }
        __syncwarp();
      }
      g += k.n;
      ++kb;
    }
  } else {
    // ---------------------------------------------------------------- softmax / store warps
    const int wq = warp & 3, wg = warp >> 2;          // TMEM lane quarter; column half / output tensor
    const int row = wq * 32 + lane;                   // key row of the tile == TMEM lane
    const uint32_t lane_addr = (uint32_t)(wq * 32) << 16;
    const float c = p.scale_log2;
    bool ok = true;
    int g = 0, kb = 0;
    for (int idx = blockIdx.x; ok && idx < total; idx += gridDim.x) {
      const DgBlock k = dg_block(p, idx, n_xb, T_qp);
      if (k.n <= 0) continue;

      // this warp's 32 query columns of P^T and dS^T of the block's tile i (tile g + i of the CTA),
      // over its scores
      auto softmax = [&](int i) -> bool {
        const int gj = g + i;
        const int key = k.k_lo + i * kBN + row;
        int jlo = 0, jn = 0;                            // query rows [q0 + jlo, q0 + jlo + jn) see this key
        if (key < k.k_hi) {
          const int tp = key / p.L;
          const int rlo = tp * p.G;
          const int rhi = ((p.mode == kChunkVisible) ? min((tp / p.Cb + 1) * p.Cb, p.T_kv) : tp + 1) * p.G;
          jlo = rlo - k.q0 - 32 * wg;
          jn = rhi - rlo;
        }
        if (!__all_sync(0xffffffffu, mbar_wait(bars + 8 * (kDgS0 + (gj & 1)), (gj >> 1) & 1, abort_flag, kDgS0 + (gj & 1)))) return false;
        tc_fence_after();
        const uint32_t tS = tmem + (gj & 1) * 128 + lane_addr, tP = tS + 64;
        const float4* st4 = reinterpret_cast<const float4*>(smem_raw + 2 * kStepTile) + 8 * wg;
        uint32_t su[32], du[32];
        tmem_ld32<0>(tS + 32 * wg, su);
        tmem_ld32<0>(tP + 32 * wg, du);
        tmem_wait_ld();
        float pr[32], dd[32];
#pragma unroll
        for (int j4 = 0; j4 < 8; ++j4) {
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
#pragma unroll
        for (int jj = 0; jj < 32; ++jj) pr[jj] = ((unsigned)(jj - jlo) < (unsigned)jn) ? pr[jj] : 0.f;
        uint32_t pp[16], pd[16];
#pragma unroll
        for (int jj = 0; jj < 16; ++jj) {
          pp[jj] = Pack<T>::pack(pr[2 * jj], pr[2 * jj + 1]);
          pd[jj] = Pack<T>::pack(pr[2 * jj] * dd[2 * jj], pr[2 * jj + 1] * dd[2 * jj + 1]);
        }
        // 16-bit pairs over the first half of the warp's own fp32 columns (the other warpgroup may
        // still be reading its columns): query columns 32 wg .. + 31 at TMEM columns 32 wg .. + 15
        tmem_st16<0>(tS + 32 * wg, pp);
        tmem_st16<0>(tP + 32 * wg, pd);
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive(bars + 8 * (kDgP0 + (gj & 1)));
        return true;
      };

      ok = __all_sync(0xffffffffu, mbar_wait(bars + 8 * kDgRes, kb & 1, abort_flag, kDgRes));   // statistics landed
      if (ok) ok = softmax(0);
      for (int i = 0; ok && i < k.n; ++i) {
        if (i + 1 < k.n && !(ok = softmax(i + 1))) break;
        ok = __all_sync(0xffffffffu, mbar_wait(bars + 8 * kDgU, (g + i) & 1, abort_flag, kDgU));
        if (!ok) break;
        tc_fence_after();
        const int key0 = k.k_lo + i * kBN + wq * 32;         // first key row of this warp
        const uint32_t tacc = (wg ? tmem_dK : tmem_dV) + lane_addr;
        const float f = wg ? p.scale : 1.f;
        if (key0 + 32 <= k.k_hi && !p.acc_depth) {           // every row of the warp is this block's
          if (lane == 0) bulk_wait_read_all();               // this warp's previous store has read its rows
          __syncwarp();
          // staging = the TMA box layout: two [128 rows x 128 B] halves per tensor, 16-byte chunk c of
          // row r at chunk c ^ (r & 7)
          unsigned char* orow = smem_raw + kDgOutOff + wg * kTile + row * 128;
          uint32_t ov[D];
          tmem_ld32<0>(tacc, ov);
          tmem_ld32<32>(tacc + 32, ov);
          if constexpr (D == 128) {
            tmem_ld32<D - 64>(tacc + 64, ov);
            tmem_ld32<D - 32>(tacc + 96, ov);
          }
          tmem_wait_ld();
          tc_fence_before();
          mbar_arrive(bars + 8 * kDgE);                      // accumulator values are in registers
#pragma unroll
          for (int ch = 0; ch < D / 8; ++ch)
            *reinterpret_cast<uint4*>(orow + (ch >> 3) * kHalfBytes + (((ch & 7) ^ (row & 7)) << 4)) = pack8_scaled<T>(ov + ch * 8, f);
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          __syncwarp();
          if (lane == 0) {
            const uint32_t src = sOut + wg * kTile + wq * 32 * 128;
            const CUtensorMap* om = wg ? &omaps.dkd : &omaps.dvd;
#pragma unroll
            for (int bx = 0; bx < D / 64; ++bx) {
              if (dep5 == 0) tma_store_4d(om, src + bx * kHalfBytes, 64 * bx, k.h, key0, k.b);
              else tma_store_5d(om, src + bx * kHalfBytes, 64 * bx, k.h, 0, key0 / dep5, k.b);
            }
            bulk_commit();
          }
          __syncwarp();
        } else {
          const int key = key0 + lane;
          const bool valid = key < k.k_hi;
          const int64_t mrow = dep_mem_row(p, valid ? key : k.k_lo);
          T* gout = wg ? reinterpret_cast<T*>(p.dkd.ptr) + p.dkd.off(k.b, mrow, k.h) : reinterpret_cast<T*>(p.dvd.ptr) + p.dvd.off(k.b, mrow, k.h);
#pragma unroll
          for (int q4 = 0; q4 < D / 32; ++q4) {
            uint32_t ov[32];
            tmem_ld32<0>(tacc + q4 * 32, ov);
            tmem_wait_ld();
            if (valid) {
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                uint4* dst = reinterpret_cast<uint4*>(gout + q4 * 32 + e * 8);
                *dst = p.acc_depth ? pack8_blend<T>(ov + e * 8, f, *dst, 1.f) : pack8_scaled<T>(ov + e * 8, f);
              }
            }
          }
          tc_fence_before();
          mbar_arrive(bars + 8 * kDgE);
        }
      }
      g += k.n;
      ++kb;
    }
    if (lane == 0) bulk_wait_read_all();                   // staged rows are read before the CTA's smem goes
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

// The query-stationary depth-gradient kernel owns its depth rows only when a 64-row block
// holds whole positions (64 % G == 0) and, for chunk-visible, whole chunks.
inline bool depth_grad_applies(const Params& p, const moda_problem* pr) {
  if (p.L <= 0 || (kStep % p.G) != 0) return false;
  if (pr->mode == MODA_CHUNK_VISIBLE && (kStep % pr->chunk_rows) != 0) return false;
  return true;
}

}  // namespace tc
}  // namespace moda
