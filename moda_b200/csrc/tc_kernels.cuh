// tcgen05 / TMEM / TMA MoDA kernels for sm_100a (head dim D = 64 or 128, bf16 or fp16).
//
// Forward.  One CTA owns 128 folded query rows of one (batch, KV head) and walks the
// key tiles they can see: sequence K/V first, then the depth K/V window of the tile
// (the same walk and the same visibility intervals as the mma.sync kernels).  Two CTAs
// are resident per SM so that one CTA's softmax overlaps the other's MMAs.
//
//   warp 5           : TMA loads (128B-swizzled [128 x 64] boxes) of Q once and of each K and
//                      V tile into single-stage buffers, refilled as soon as the MMA that read
//                      them has completed.
//   warp 4           : issues S = Q K^T (M=128, N=128) and O += P V (M=128, N=D) as tcgen05.mma
//                      in K=16 steps with fp32 accumulators in TMEM.
//   warps 0-3        : softmax.  Thread = query row = TMEM lane.  tcgen05.ld of the S
//                      row, visibility mask on masked tiles only, online softmax in
//                      base 2 with lazy rescaling of O (O is touched only when a row
//                      maximum grows by more than 2^8), P written back to TMEM over S
//                      as packed 16-bit pairs and consumed by the PV MMA straight from
//                      TMEM.
//
// TMEM (256 columns per CTA): [0,128) S (fp32) / P (16-bit, first 64 columns),
// [128,128+D) O (fp32).  Shared memory: Q, K, V tiles of [128 x D] 16-bit values each, stored
// as D/64 boxes of [128 rows x 64 elements] (one 128-byte swizzle atom per row).
//
// Every mbarrier wait is bounded: on expiry the CTA records an error in a device
// status word, drains its outstanding TMA loads (bounded again), frees its TMEM and
// returns; later CTAs of the launch see the status word and return at once.
#pragma once
#include <cuda.h>

#include <cstring>
#include <type_traits>

#include "../../include/moda_b200.h"
#include "common.cuh"
#include "profiler.cuh"

namespace moda {
namespace tc {

constexpr int kBM = 128;
constexpr int kBN = 128;
constexpr uint32_t kWaitHintNs = 20000;        // one try_wait may sleep this long (ns)
#ifdef MODA_WAIT_TEST
constexpr uint32_t kWaitTries = 50;            // wait-expiry test build: give up after about 1 ms
#else
constexpr uint32_t kWaitTries = 10000;         // tries per wait before giving up (<= 0.2 s)
#endif
constexpr uint32_t kHalfBytes = 128 * 64 * 2;  // one TMA box: [128 rows x 64 elements] of 16 bits
constexpr uint32_t kTileBytes = 2 * kHalfBytes; // a [128 x 128] 16-bit tile (two boxes)
template <int D> __host__ __device__ constexpr uint32_t tile_bytes() { return (uint32_t)(D / 64) * kHalfBytes; }   // [128 x D]

// 0 = ok; otherwise (code << 8) | barrier id of the first wait that expired.  g_tc_status is the
// abort flag of the launch in flight: it is cleared when a launch is enqueued and lets the CTAs
// that start after a failure return at once.  g_tc_sticky keeps the first failure of any launch
// until the host reads it (moda_b200_device_status), so that a later call cannot erase it.
__device__ int g_tc_status;
__device__ int g_tc_sticky;

__device__ __forceinline__ void record_failure(int code) {
  atomicCAS(&g_tc_status, 0, code);
  atomicCAS(&g_tc_sticky, 0, code);
}

struct FwdMaps { CUtensorMap q, k, v, kd, vd; };

// ------------------------------------------------------------------ PTX wrappers
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" :: "r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
// Bounded wait.  Returns false when the limit expired or another thread of the CTA
// already gave up (abort flag); the caller must then leave through the teardown path.
// The wait sleeps in hardware (mbarrier.try_wait with a suspend-time hint) instead of
// spinning: a spinning warp takes issue slots from the producer lane and from the softmax
// warp that shares its SM sub-partition.  Bound: kWaitTries x kWaitHintNs of sleeping.
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(bar), "r"(parity), "r"(kWaitHintNs) : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int bar_id) {
  if (mbar_test(bar, parity)) return true;
  for (uint32_t i = 0; i < kWaitTries; ++i) {
    if (mbar_try(bar, parity)) return true;
    if (*abort_flag != 0) return false;
  }
  *abort_flag = 1;
  record_failure((1 << 8) | bar_id);
  return false;
}

// One lane of a converged warp.  The TMA and MMA warps run their control flow with all 32
// lanes (so descriptors and addresses stay in uniform registers) and only the asynchronous
// instruction itself is issued by the elected lane - always the same one, which matters because
// tcgen05.commit tracks the MMAs of the issuing thread.
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(pred));
  return pred != 0;
}

__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      :: "r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}
__device__ __forceinline__ void tma_load_5d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, int c2, int c3, int c4) {
  asm volatile(
      "cp.async.bulk.tensor.5d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
      :: "r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4) : "memory");
}
__device__ __forceinline__ void prefetch_map(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" :: "l"(map) : "memory");
}

__device__ __forceinline__ void tmem_alloc(uint32_t slot_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" :: "r"(slot_smem), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" :: "r"(bar) : "memory");
}
// D[tmem] (+)= A[smem desc] * B[smem desc]
__device__ __forceinline__ void mma_ss(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      :: "r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem desc]
__device__ __forceinline__ void mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      :: "r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// 32 lanes x 32 columns of 32 bits: thread (lane i of warp w) <-> TMEM lane 32w+i; register k <->
// column k.  OFF selects which 32 registers of a larger per-thread array take part, so that
// the array stays in registers (all indices are compile-time constants).
template <int OFF, int N>
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[N]) {
  static_assert(OFF + 32 <= N, "register window out of range");
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[OFF + 0]), "=r"(r[OFF + 1]), "=r"(r[OFF + 2]), "=r"(r[OFF + 3]), "=r"(r[OFF + 4]), "=r"(r[OFF + 5]),
        "=r"(r[OFF + 6]), "=r"(r[OFF + 7]), "=r"(r[OFF + 8]), "=r"(r[OFF + 9]), "=r"(r[OFF + 10]), "=r"(r[OFF + 11]),
        "=r"(r[OFF + 12]), "=r"(r[OFF + 13]), "=r"(r[OFF + 14]), "=r"(r[OFF + 15]), "=r"(r[OFF + 16]), "=r"(r[OFF + 17]),
        "=r"(r[OFF + 18]), "=r"(r[OFF + 19]), "=r"(r[OFF + 20]), "=r"(r[OFF + 21]), "=r"(r[OFF + 22]), "=r"(r[OFF + 23]),
        "=r"(r[OFF + 24]), "=r"(r[OFF + 25]), "=r"(r[OFF + 26]), "=r"(r[OFF + 27]), "=r"(r[OFF + 28]), "=r"(r[OFF + 29]),
        "=r"(r[OFF + 30]), "=r"(r[OFF + 31])
      : "r"(taddr) : "memory");
}
template <int OFF, int N>
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[N]) {
  static_assert(OFF + 32 <= N, "register window out of range");
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
      :: "r"(taddr),
         "r"(r[OFF + 0]), "r"(r[OFF + 1]), "r"(r[OFF + 2]), "r"(r[OFF + 3]), "r"(r[OFF + 4]), "r"(r[OFF + 5]),
         "r"(r[OFF + 6]), "r"(r[OFF + 7]), "r"(r[OFF + 8]), "r"(r[OFF + 9]), "r"(r[OFF + 10]), "r"(r[OFF + 11]),
         "r"(r[OFF + 12]), "r"(r[OFF + 13]), "r"(r[OFF + 14]), "r"(r[OFF + 15]), "r"(r[OFF + 16]), "r"(r[OFF + 17]),
         "r"(r[OFF + 18]), "r"(r[OFF + 19]), "r"(r[OFF + 20]), "r"(r[OFF + 21]), "r"(r[OFF + 22]), "r"(r[OFF + 23]),
         "r"(r[OFF + 24]), "r"(r[OFF + 25]), "r"(r[OFF + 26]), "r"(r[OFF + 27]), "r"(r[OFF + 28]), "r"(r[OFF + 29]),
         "r"(r[OFF + 30]), "r"(r[OFF + 31])
      : "memory");
}
template <int OFF, int N>
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[N]) {
  static_assert(OFF + 16 <= N, "register window out of range");
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
      :: "r"(taddr), "r"(r[OFF + 0]), "r"(r[OFF + 1]), "r"(r[OFF + 2]), "r"(r[OFF + 3]), "r"(r[OFF + 4]), "r"(r[OFF + 5]),
         "r"(r[OFF + 6]), "r"(r[OFF + 7]), "r"(r[OFF + 8]), "r"(r[OFF + 9]), "r"(r[OFF + 10]), "r"(r[OFF + 11]),
         "r"(r[OFF + 12]), "r"(r[OFF + 13]), "r"(r[OFF + 14]), "r"(r[OFF + 15])
      : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Packed fp32 pairs (sm_100 has two-wide fp32 FMA / ADD / MUL on register pairs - the float2
// intrinsics - and a three-input max): the softmax of a 128 x 128 block is bound by instruction
// issue, so every fp32 instruction saved in it counts.
__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float d; asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c)); return d;
}

// exp2 of two values on the FMA pipe: x = n + f with n = round(x), f in [-0.5, 0.5]; degree-4
// polynomial for 2^f (relative error < 4e-6, far inside the 16-bit rounding of P); 2^n goes into
// the exponent field.  Inputs below -126 (masked columns: -inf) are clamped and come out as 2^-126
// times the polynomial, which the 16-bit rounding turns into 0 or the smallest normal.
__device__ __forceinline__ float2 exp2x2_fma(float2 x) {
  const float2 xc = make_float2(fmaxf(x.x, -126.f), fmaxf(x.y, -126.f));
  const float2 t = __fadd2_rn(xc, make_float2(12582912.f, 12582912.f));   // 1.5 * 2^23: low mantissa bits = round(x)
  const float2 r = __fadd2_rn(t, make_float2(-12582912.f, -12582912.f));
  const float2 f = __ffma2_rn(r, make_float2(-1.f, -1.f), xc);
  float2 q = __ffma2_rn(make_float2(0.009676037f, 0.009676037f), f, make_float2(0.055922035f, 0.055922035f));
  q = __ffma2_rn(q, f, make_float2(0.24022107f, 0.24022107f));
  q = __ffma2_rn(q, f, make_float2(0.6931210f, 0.6931210f));
  q = __ffma2_rn(q, f, make_float2(1.0000001f, 1.0000001f));
  return make_float2(__int_as_float(__float_as_int(q.x) + (__float_as_int(t.x) << 23)),
                     __int_as_float(__float_as_int(q.y) + (__float_as_int(t.y) << 23)));
}

// One row's online-softmax step over the 128 scores of a key tile (thread = query row), in two
// parts so that a caller can hand the first columns of P to the PV matmul before the last ones
// are computed.  scale > 0 is required (the maximum is taken before scaling).
//
// softmax_prepare: masks columns outside [lo, hi) when `masked` (`uniform32`: [lo, hi) and the tile
// are aligned to 32 columns), takes the row maximum, keeps the old reference maximum unless the
// new one is more than 2^8 larger (lazy rescale: alpha / grow tell the caller to rescale O) and
// scales the running row sum l by alpha.
__device__ __forceinline__ void softmax_prepare(float (&s)[128], bool masked, bool uniform32, int c0, int lo, int hi, float c,
                                                float& m_used, float& l, float& alpha, bool& grow) {
  if (masked && uniform32) {
    // depth tile with L a multiple of 32: a row sees whole positions, so each aligned group of 32
    // columns is visible or not as a whole - four tests instead of 128
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      const int col = c0 + 32 * g;
      const bool vis = col >= lo && col < hi;
#pragma unroll
      for (int i = 0; i < 32; ++i) s[32 * g + i] = vis ? s[32 * g + i] : -INFINITY;
    }
  } else if (masked) {
#pragma unroll
    for (int i = 0; i < 128; ++i) {
      const int col = c0 + i;
      s[i] = (col >= lo && col < hi) ? s[i] : -INFINITY;
    }
  }
  // row maximum: 8 independent chains of three-input max (a single running maximum would be a
  // 128-deep dependent chain for the one warp this sub-partition has on the job)
  float mx8[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    float m = s[j];
#pragma unroll
    for (int k = 1; k + 1 < 16; k += 2) m = fmax3(m, s[j + 8 * k], s[j + 8 * (k + 1)]);
    mx8[j] = fmaxf(m, s[j + 8 * 15]);
  }
  const float mx = fmaxf(fmax3(mx8[0], mx8[1], mx8[2]), fmax3(fmax3(mx8[3], mx8[4], mx8[5]), mx8[6], mx8[7]));
  const float m_new = fmaxf(m_used, mx * c);
  alpha = 1.f;
  grow = false;
  if (m_new > m_used + 8.f) {        // also true for the first finite maximum (m_used = -inf)
    alpha = (m_used == -INFINITY) ? 0.f : fast_exp2(m_used - m_new);
    grow = (m_used != -INFINITY);    // nothing accumulated yet => nothing to rescale
    m_used = m_new;
  }
  l *= alpha;
}

// softmax_exps: P = exp2(s * c - m) for the column pairs [I0, I1) as packed 16-bit pairs in pk, their
// sums added to the four partial sums.  One pair in kPolyEvery takes its two exponentials on the FMA
// pipe (exp2x2_fma) instead of the exp2 unit.
template <typename T, int kPolyEvery, int I0, int I1>
__device__ __forceinline__ void softmax_exps(const float (&s)[128], float c, float m_used, float2 (&sum2)[4], uint32_t (&pk)[64]) {
  const float m_sub = (m_used == -INFINITY) ? 0.f : m_used;
  const float2 c2 = make_float2(c, c), nm2 = make_float2(-m_sub, -m_sub);
#pragma unroll
  for (int i = I0; i < I1; ++i) {
    const float2 x = __ffma2_rn(make_float2(s[2 * i], s[2 * i + 1]), c2, nm2);
    float2 pp;
    if (kPolyEvery > 0 && (i % (kPolyEvery > 0 ? kPolyEvery : 1)) == (kPolyEvery > 0 ? kPolyEvery : 1) - 1) {
      pp = exp2x2_fma(x);
    } else {
      pp.x = fast_exp2(x.x);
      pp.y = fast_exp2(x.y);
    }
    sum2[i & 3] = __fadd2_rn(sum2[i & 3], pp);
    pk[i] = Pack<T>::pack(pp.x, pp.y);
  }
}
__device__ __forceinline__ float softmax_total(const float2 (&sum2)[4]) {
  const float2 tot = __fadd2_rn(__fadd2_rn(sum2[0], sum2[1]), __fadd2_rn(sum2[2], sum2[3]));
  return tot.x + tot.y;
}

// The whole step at once.
template <typename T, int kPolyEvery>
__device__ __forceinline__ void softmax_row128(const uint32_t (&su)[128], bool masked, bool uniform32, int c0, int lo, int hi, float c,
                                               float& m_used, float& l, float& alpha, bool& grow, uint32_t (&pk)[64]) {
  float s[128];
#pragma unroll
  for (int i = 0; i < 128; ++i) s[i] = __uint_as_float(su[i]);
  softmax_prepare(s, masked, uniform32, c0, lo, hi, c, m_used, l, alpha, grow);
  float2 sum2[4] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
  softmax_exps<T, kPolyEvery, 0, 64>(s, c, m_used, sum2, pk);
  l += softmax_total(sum2);
}

// Shared-memory matrix descriptor, 128-byte swizzle, descriptor version 1.
//   K-major operand  ([rows][64 elem] boxes, 128 B per row):   lbo = 16,   sbo = 1024
//   MN-major operand ([k rows][64 elem] boxes, second 64-wide
//   block of the MN extent in the next box):                    lbo = box bytes, sbo = 1024
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = (uint64_t)((saddr & 0x3FFFFu) >> 4);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
// Instruction descriptor, kind::f16, fp32 accumulate, M = 128.
//   fmt: 0 = f16, 1 = bf16.  b_mn_major: B operand is MN-major (V tile) instead of K-major.
__host__ __device__ constexpr uint32_t instr_desc(uint32_t fmt, uint32_t n, bool b_mn_major) {
  return (1u << 4) | (fmt << 7) | (fmt << 10) | ((b_mn_major ? 1u : 0u) << 16) | ((n >> 3) << 17) | ((128u >> 4) << 24);
}

enum BarId : int { kBarQ = 0, kBarK, kBarV, kBarS, kBarP, kBarO, kBarKFree, kBarVFree, kBarCount };

// Tile walk of a 128-row query tile (same construction as simt::make_walk).
struct Walk { int n_seq, n_dep, dep_c0, seq_full_hi; };
__device__ __forceinline__ Walk make_walk(const Params& p, int r0) {
  Walk w;
  const int r_last = min(r0 + kBM, p.T_q) - 1;
  int lo, hi, lo2, hi2;
  seq_interval(p, r_last, lo, hi);
  w.n_seq = (hi + kBN - 1) / kBN;
  seq_interval(p, r0, lo2, hi2);
  w.seq_full_hi = hi2;
  dep_interval(p, r0, lo, hi);
  dep_interval(p, r_last, lo2, hi2);
  w.dep_c0 = lo;
  w.n_dep = (hi2 - lo + kBN - 1) / kBN;
  return w;
}

// Loads a [rows x D] tile as D/64 boxes; the caller has armed `bar` with the byte count.
template <int D>
__device__ __forceinline__ void tma_load_tile(uint32_t dst, const CUtensorMap* map, uint32_t bar, uint32_t box_bytes,
                                              int h, int row, int b) {
#pragma unroll
  for (int bx = 0; bx < D / 64; ++bx) tma_load_4d(dst + bx * box_bytes, map, bar, 64 * bx, h, row, b);
}

// The same for a tile of depth K/V rows [row, row + rows).  L5 == 0: the packed layout, a 4-D map
// like every other tensor.  L5 == L > 0: the depth tensor is an in-place layer cache
// (Params::Ls > L), its map is 5-D (D, H, L, T, B) with a box of L layers x rows / L positions,
// which lands in shared memory in the same row order (position-major, layer-minor) as the packed
// tile; `row` is a multiple of L because depth windows start at position boundaries.
template <int D>
__device__ __forceinline__ void tma_load_dep_tile(uint32_t dst, const CUtensorMap* map, uint32_t bar, uint32_t box_bytes,
                                                  int h, int row, int b, int L5) {
  if (L5 == 0) { tma_load_tile<D>(dst, map, bar, box_bytes, h, row, b); return; }
  const int pos = row / L5;
#pragma unroll
  for (int bx = 0; bx < D / 64; ++bx) tma_load_5d(dst + bx * box_bytes, map, bar, 64 * bx, h, 0, pos, b);
}

// ======================================================================= forward
// grid (ceil(T_q/128), H, B); 192 threads (4 softmax warps, MMA warp, TMA warp); two CTAs per SM.
template <typename T, int D>
__global__ void __launch_bounds__(192, 2)
fwd_kernel(const __grid_constant__ Params p, const __grid_constant__ FwdMaps maps) {
  constexpr uint32_t kTile = tile_bytes<D>();
  extern __shared__ unsigned char smem_raw[];
  const uint32_t raw_u32 = smem_u32(smem_raw);
  const uint32_t base = (raw_u32 + 1023u) & ~1023u;
  unsigned char* gbase = smem_raw + (base - raw_u32);
  const uint32_t sQ = base, sK = base + kTile, sV = base + 2 * kTile;
  const uint32_t ctl = base + 3 * kTile;
  unsigned char* gctl = gbase + 3 * kTile;
  const uint32_t bars = ctl;                                    // kBarCount x 8 bytes
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gctl + 64);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gctl + 72);
  volatile int* drain_flag = reinterpret_cast<volatile int*>(gctl + 76);   // never set: lets the drain waits run

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (*reinterpret_cast<volatile int*>(&g_tc_status) != 0) return;   // an earlier CTA failed: do nothing

  const int n_qt = (p.T_q + kBM - 1) / kBM;
  const BlockId bid = block_order(p, D);
  const int qt = n_qt - 1 - bid.rank;            // heaviest causal tiles first
  const int h = bid.h, b = bid.b;
  const int r0 = qt * kBM;
  const Walk walk = make_walk(p, r0);
  const int n_tiles = walk.n_seq + walk.n_dep;
  const int dep5 = (p.Ls != p.L) ? p.L : 0;      // in-place layer cache: 5-D depth maps

  if (tid == 0) {
    mbar_init(bars + 8 * kBarQ, 1);
    mbar_init(bars + 8 * kBarK, 1);
    mbar_init(bars + 8 * kBarV, 1);
    mbar_init(bars + 8 * kBarS, 1);
    mbar_init(bars + 8 * kBarP, 128);
    mbar_init(bars + 8 * kBarO, 1);
    mbar_init(bars + 8 * kBarKFree, 1);
    mbar_init(bars + 8 * kBarVFree, 1);
    *abort_flag = 0;
    *drain_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 0) {
    tmem_alloc(ctl + 64, 256);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tmem_S = tmem, tmem_O = tmem + 128;
  constexpr uint32_t fmt = std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;

  if (warp == 5) {
    // ------------------------------------------------------------- TMA warp
    // All lanes run the control flow; one elected lane issues.  K(j+1) is loaded as soon as
    // QK(j) has finished reading the K buffer, V(j+1) as soon as PV(j) has finished reading V.
    if (n_tiles > 0) {
      bool pend_k = false, pend_v = false;
      uint32_t pend_k_par = 0, pend_v_par = 0;
      auto load_kv = [&](int i, bool is_k) {
        const bool dep = i >= walk.n_seq;
        const int row = dep ? walk.dep_c0 + (i - walk.n_seq) * kBN : i * kBN;
        const CUtensorMap* m = is_k ? (dep ? &maps.kd : &maps.k) : (dep ? &maps.vd : &maps.v);
        const uint32_t dst = is_k ? sK : sV;
        const uint32_t bar = bars + 8 * (is_k ? kBarK : kBarV);
        if (elect_one()) {
          mbar_expect_tx(bar, kTile);
          if (dep) tma_load_dep_tile<D>(dst, m, bar, kHalfBytes, h, row, b, dep5);
          else tma_load_tile<D>(dst, m, bar, kHalfBytes, h, row, b);
        }
        __syncwarp();
        if (is_k) { pend_k = true; pend_k_par = i & 1; } else { pend_v = true; pend_v_par = i & 1; }
      };
      if (elect_one()) {
        prefetch_map(&maps.q); prefetch_map(&maps.k); prefetch_map(&maps.v);
        mbar_expect_tx(bars + 8 * kBarQ, kTile);
        tma_load_tile<D>(sQ, &maps.q, bars + 8 * kBarQ, kHalfBytes, h, r0, b);
      }
      __syncwarp();
      load_kv(0, true);
      load_kv(0, false);
      bool ok = true;
      for (int j = 0; ok && j + 1 < n_tiles; ++j) {
        if (!(ok = mbar_wait(bars + 8 * kBarKFree, j & 1, abort_flag, kBarKFree))) break;
        load_kv(j + 1, true);
        if (!(ok = mbar_wait(bars + 8 * kBarVFree, j & 1, abort_flag, kBarVFree))) break;
        load_kv(j + 1, false);
      }
      // Every load this warp issued must have landed before the CTA's shared memory is released,
      // whether the walk completed (the last tiles are about to be consumed anyway) or a wait gave
      // up somewhere in the CTA: wait (bounded) for the latest Q, K and V loads.
      mbar_wait(bars + 8 * kBarQ, 0, drain_flag, kBarQ);
      if (pend_k) mbar_wait(bars + 8 * kBarK, pend_k_par, drain_flag, kBarK);
      if (pend_v) mbar_wait(bars + 8 * kBarV, pend_v_par, drain_flag, kBarV);
    }
  } else if (warp == 4) {
    // ------------------------------------------------------------- MMA warp
    if (n_tiles > 0) {
      constexpr uint32_t idesc_qk = instr_desc(fmt, 128, false);
      constexpr uint32_t idesc_pv = instr_desc(fmt, D, true);
      bool ok = mbar_wait(bars + 8 * kBarQ, 0, abort_flag, kBarQ);
      for (int j = 0; ok && j < n_tiles; ++j) {
        const uint32_t par = j & 1;
        if (!(ok = mbar_wait(bars + 8 * kBarK, par, abort_flag, kBarK))) break;
        tc_fence_after();
        if (elect_one()) {
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk) {
            const uint32_t off = (kk >> 2) * kHalfBytes + (kk & 3) * 32;
            mma_ss(tmem_S, smem_desc_sw128(sQ + off, 16, 1024), smem_desc_sw128(sK + off, 16, 1024), idesc_qk, kk > 0);
          }
          tc_commit(bars + 8 * kBarS);
          tc_commit(bars + 8 * kBarKFree);
        }
        __syncwarp();
        if (!(ok = mbar_wait(bars + 8 * kBarP, par, abort_flag, kBarP))) break;
        if (!(ok = mbar_wait(bars + 8 * kBarV, par, abort_flag, kBarV))) break;
        tc_fence_after();
        if (elect_one()) {
#pragma unroll
          for (int kk = 0; kk < 8; ++kk)
            mma_ts(tmem_O, tmem_S + kk * 8, smem_desc_sw128(sV + kk * 2048, kHalfBytes, 1024), idesc_pv,
                   (j > 0 || kk > 0) ? 1u : 0u);
          tc_commit(bars + 8 * kBarO);
          tc_commit(bars + 8 * kBarVFree);
        }
        __syncwarp();
      }
    }
  } else {
    // ------------------------------------------------------------- softmax warps
    const int row = warp * 32 + lane;          // row of the tile == TMEM lane
    const int r = r0 + row;
    const uint32_t lane_addr = (uint32_t)(warp * 32) << 16;
    int slo, shi, dlo, dhi;
    seq_interval(p, r, slo, shi);
    dep_interval(p, r, dlo, dhi);
    float m_used = -INFINITY;   // maximum the accumulators are currently scaled by
    float l = 0.f;
    bool ok = true;
    const float c = p.scale_log2;

    for (int j = 0; j < n_tiles; ++j) {
      ok = __all_sync(0xffffffffu, mbar_wait(bars + 8 * kBarS, j & 1, abort_flag, kBarS));
      if (!ok) break;   // warp-uniform: the tcgen05 loads/stores below are warp-collective
      tc_fence_after();
      const bool is_dep = j >= walk.n_seq;
      const int c0 = is_dep ? walk.dep_c0 + (j - walk.n_seq) * kBN : j * kBN;
      const bool masked = is_dep || (c0 + kBN > walk.seq_full_hi);
      const int lo = is_dep ? dlo : slo, hi = is_dep ? dhi : shi;

      // A depth tile holds the rows of several positions; a warp whose 32 query rows see none of
      // its columns contributes an all-zero P block and skips the scores altogether.
      const bool none = is_dep && __all_sync(0xffffffffu, (c0 + kBN <= lo) || (c0 >= hi));
      float alpha = 1.f;
      bool grow = false;
      uint32_t pk[64];
      if (none) {
#pragma unroll
        for (int i = 0; i < 64; ++i) pk[i] = 0u;
      } else {
        uint32_t su[128];
        tmem_ld32<0>(tmem_S + lane_addr + 0, su);
        tmem_ld32<32>(tmem_S + lane_addr + 32, su);
        tmem_ld32<64>(tmem_S + lane_addr + 64, su);
        tmem_ld32<96>(tmem_S + lane_addr + 96, su);
        tmem_wait_ld();
        // same arithmetic as fwd3_kernel, so that a result does not depend on which of the two ran
        softmax_row128<T, 4>(su, masked, is_dep && (p.L & 31) == 0, c0, lo, hi, c, m_used, l, alpha, grow, pk);
      }
      tmem_st32<0>(tmem_S + lane_addr + 0, pk);
      tmem_st32<32>(tmem_S + lane_addr + 32, pk);
      // rescale O (TMEM round trip) only when some row of this warp moved its maximum
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
      tmem_wait_st();
      tc_fence_before();
#ifndef MODA_WAIT_TEST
      mbar_arrive(bars + 8 * kBarP);
#endif
      // (the wait-expiry test build withholds this arrival: the MMA warp's bounded wait on the
      // P-ready barrier, which no TMA load targets, then runs out and the CTA leaves through the
      // teardown path)
    }

    if (ok && n_tiles > 0) ok = __all_sync(0xffffffffu, mbar_wait(bars + 8 * kBarO, (n_tiles - 1) & 1, abort_flag, kBarO));
    if (ok && n_tiles > 0) {
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
    tmem_dealloc(tmem, 256);
  }
}

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = []() -> EncodeTiledFn {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return nullptr;
    return reinterpret_cast<EncodeTiledFn>(f);
  }();
  return fn;
}

// [B, T, H, D] view -> 4-D tensor map (D, H, T, B), box [64, 1, box_rows, 1], 128B swizzle, zero
// fill.  A dimension of extent 1 may carry any stride (it is never multiplied by a non-zero
// index) and gets a placeholder TMA accepts; every other stride must be a positive multiple of
// 8 elements, which the entry points have checked.
inline bool make_map_rows(CUtensorMap* m, const View& v, int dtype, int B, int64_t T, int H, int D, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr || v.ptr == nullptr) return false;
  bool bad = false;
  auto stride = [&bad](int64_t s, int64_t extent) -> cuuint64_t {
    if (extent <= 1) return (cuuint64_t)16;
    if (s <= 0) { bad = true; return (cuuint64_t)16; }
    return (cuuint64_t)(s * 2);
  };
  cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)H, (cuuint64_t)T, (cuuint64_t)B};
  cuuint64_t strides[3] = {stride(v.sh, H), stride(v.st, T), stride(v.sb, B)};
  if (bad) return false;
  cuuint32_t box[4] = {64, 1, (cuuint32_t)box_rows, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  return fn(m, dtype == MODA_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, v.ptr,
            dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Depth K/V (or their gradients) of an in-place layer cache: rows (t, l), l < L, at memory row
// t * Ls + l.  5-D map (D, H, L, T, B), box [64, 1, L, box_rows / L, 1]: a tile of box_rows
// consecutive depth rows of the operator.  box_rows must be a multiple of L.
inline bool make_map_dep5(CUtensorMap* m, const View& v, int dtype, int B, int T, int L, int Ls, int H, int D, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr || v.ptr == nullptr || L <= 0 || box_rows % L != 0) return false;
  if ((H > 1 && v.sh <= 0) || v.st <= 0 || (B > 1 && v.sb <= 0)) return false;
  cuuint64_t dims[5] = {(cuuint64_t)D, (cuuint64_t)H, (cuuint64_t)L, (cuuint64_t)T, (cuuint64_t)B};
  cuuint64_t strides[4] = {(cuuint64_t)((H > 1 ? v.sh : 8) * 2), (cuuint64_t)(v.st * 2), (cuuint64_t)(v.st * 2 * Ls),
                           (cuuint64_t)((B > 1 ? v.sb : 8) * 2)};
  cuuint32_t box[5] = {64, 1, (cuuint32_t)L, (cuuint32_t)(box_rows / L), 1};
  cuuint32_t estr[5] = {1, 1, 1, 1, 1};
  return fn(m, dtype == MODA_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 5, v.ptr,
            dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}
// Map of a depth tensor in whichever of the two layouts the problem uses.
inline bool make_map_depth(CUtensorMap* m, const View& v, int dtype, const Params& p, int D, int box_rows) {
  if (p.Ls == p.L) return make_map_rows(m, v, dtype, p.B, (int64_t)p.T_kv * p.L, p.H, D, box_rows);
  return make_map_dep5(m, v, dtype, p.B, p.T_kv, p.L, p.Ls, p.H, D, box_rows);
}

// The tcgen05 kernels take a positive scale (the row maximum is taken before scaling) and, for an
// in-place layer cache (depth_rows_per_pos > L), a layer count that divides the 32-row boxes.
inline bool depth_layout_supported(const moda_problem* pr) {
  return pr->L == 0 || pr->depth_rows_per_pos <= pr->L || (32 % pr->L) == 0;
}
inline bool fwd_supported(const moda_problem* pr) {
  return (pr->D == 128 || pr->D == 64) && pr->mode != MODA_DEPTH_ONLY && pr->scale > 0.f && depth_layout_supported(pr);
}

// Clears the abort flag of the launch about to be enqueued (the sticky word is left alone).
inline cudaError_t clear_launch_status(cudaStream_t st) {
  void* status_addr = nullptr;
  cudaError_t e = cudaGetSymbolAddress(&status_addr, g_tc_status);
  if (e == cudaSuccess) e = cudaMemsetAsync(status_addr, 0, sizeof(int), st);
  return e;
}

inline bool make_fwd_maps(FwdMaps* maps, const Params& p, const moda_problem* pr) {
  memset(maps, 0, sizeof(*maps));
  const int D = pr->D;
  bool ok = make_map_rows(&maps->q, p.q, pr->dtype, p.B, p.T_q, p.H, D, 128) &&
            make_map_rows(&maps->k, p.k, pr->dtype, p.B, p.T_kv, p.H, D, 128) &&
            make_map_rows(&maps->v, p.v, pr->dtype, p.B, p.T_kv, p.H, D, 128);
  if (ok && p.L > 0) {
    ok = make_map_depth(&maps->kd, p.kd, pr->dtype, p, D, 128) && make_map_depth(&maps->vd, p.vd, pr->dtype, p, D, 128);
  } else if (ok) {
    maps->kd = maps->k; maps->vd = maps->v;   // never dereferenced (no depth tiles)
  }
  return ok;
}

template <typename T, int D>
inline cudaError_t launch_fwd(const Params& p, const FwdMaps& maps, cudaStream_t st) {
  auto kern = fwd_kernel<T, D>;
  const size_t smem = 3 * (size_t)tile_bytes<D>() + 1024 + 128;
  cudaError_t er = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (er != cudaSuccess) return er;
  dim3 grid((p.T_q + kBM - 1) / kBM, p.H, p.B);
  prof::Scope ps(prof::kFwdTc, st);
  kern<<<grid, 192, smem, st>>>(p, maps);
  return cudaGetLastError();
}

inline int fwd(const Params& p, const moda_problem* pr, cudaStream_t st, int* launches, int* cuda_err) {
  FwdMaps maps;
  if (!make_fwd_maps(&maps, p, pr)) return MODA_ERR_UNSUPPORTED;
  cudaError_t e = clear_launch_status(st);
  if (e != cudaSuccess) { *cuda_err = (int)e; return MODA_ERR_CUDA; }
  const bool bf = pr->dtype == MODA_BF16;
  if (pr->D == 128) e = bf ? launch_fwd<__nv_bfloat16, 128>(p, maps, st) : launch_fwd<__half, 128>(p, maps, st);
  else e = bf ? launch_fwd<__nv_bfloat16, 64>(p, maps, st) : launch_fwd<__half, 64>(p, maps, st);
  if (e != cudaSuccess) { *cuda_err = (int)e; return MODA_ERR_CUDA; }
  *launches += 1;
  return MODA_OK;
}

// Reads the sticky status word of the tcgen05 kernels (synchronises) and clears it when set.
inline int read_status(int* out) {
  int v = 0;
  cudaError_t e = cudaMemcpyFromSymbol(&v, g_tc_sticky, sizeof(int));
  if (e != cudaSuccess) return (int)e;
  if (v != 0) {
    const int zero = 0;
    e = cudaMemcpyToSymbol(g_tc_sticky, &zero, sizeof(int));
    if (e != cudaSuccess) return (int)e;
  }
  *out = v;
  return 0;
}

}  // namespace tc
}  // namespace moda
