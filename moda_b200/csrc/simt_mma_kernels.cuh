// Warp-level mma.sync (m16n8k16) MoDA kernels: forward, dq, and key-parallel dk/dv
// (sequence and depth keys in one launch), for every mode, any T, D in {64,128},
// bf16/fp16.  They are the library's coverage path: shapes the tcgen05 kernels do
// not take (D=64, ragged T, fp16 ...) run here.  No atomics anywhere: every output
// row has exactly one owning CTA, so results are bit-reproducible.
//
// Numerics follow the reference kernels: scores are scaled by scale*log2(e) after
// the fp32-accumulated dot (moda_v14.py:188), probabilities use exp2, P and dS are
// rounded to the input dtype before the second matmul (moda_v14.py:209,712),
// o = acc / l and lse = m + log2(l) (moda_v14.py:372-374), dq and dk are multiplied
// by scale once at the end (moda_v14.py:860,1019).
#pragma once
#include "common.cuh"

namespace moda {
namespace simt {

// ------------------------------------------------------------------ primitives
template <typename T> struct Mma;
template <> struct Mma<__nv_bfloat16> {
  static __device__ __forceinline__ void run(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
};
template <> struct Mma<__half> {
  static __device__ __forceinline__ void run(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
};

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" :: "r"(dst), "l"(src));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" :: "n"(N));
}

// Shared-memory tile of ROWS x D elements, row stride D+8 (keeps ldmatrix rows on
// distinct banks).  Loaded with 16-byte cp.async; rows outside [0, nrows) are zeroed.
template <typename T, int D> struct Tile {
  static constexpr int LD = D + 8;
  // L, Ls: rows come in groups of L that sit Ls rows apart in memory (the depth K/V of an in-place
  // layer cache, Params::Ls); L == Ls is the plain contiguous case.
  template <int ROWS, int NT>
  static __device__ __forceinline__ void load(T* s, const T* g, int64_t row_stride, int64_t row0,
                                              int64_t nrows, int tid, int L = 1, int Ls = 1) {
    constexpr int CH = D / 8;
    for (int i = tid; i < ROWS * CH; i += NT) {
      const int r = i / CH, c = i % CH;
      T* dst = s + r * LD + c * 8;
      const int64_t row = row0 + r;
      if (row >= 0 && row < nrows) {
        const int64_t mrow = (L == Ls) ? row : (row / L) * Ls + (row % L);
        cp_async16(smem_u32(dst), g + mrow * row_stride + c * 8);
      } else {
        *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
      }
    }
  }
  // A fragment (16 rows x 16 k) at (row0, k0) of a row-major tile.
  static __device__ __forceinline__ void ldA(uint32_t (&a)[4], const T* s, int row0, int k0, int lane) {
    ldsm_x4(a, smem_u32(s + (row0 + (lane & 15)) * LD + k0 + (lane >> 4) * 8));
  }
  // B fragments for two n-blocks (n0..n0+15) x 16 k, tile stored [n][k] (k contiguous).
  // r[0],r[1] = n-block 0; r[2],r[3] = n-block 1.
  static __device__ __forceinline__ void ldB_nk(uint32_t (&r)[4], const T* s, int n0, int k0, int lane) {
    ldsm_x4(r, smem_u32(s + (n0 + (lane & 7) + (lane >> 4) * 8) * LD + k0 + ((lane >> 3) & 1) * 8));
  }
  // B fragments for two n-blocks x 16 k, tile stored [k][n] (n contiguous).
  static __device__ __forceinline__ void ldB_kn(uint32_t (&r)[4], const T* s, int k0, int n0, int lane) {
    ldsm_x4_t(r, smem_u32(s + (k0 + (lane & 7) + ((lane >> 3) & 1) * 8) * LD + n0 + (lane >> 4) * 8));
  }
};

// Key segments a query tile walks: sequence keys first, depth rows second.
struct KeyWalk {
  int n_seq_tiles, n_dep_tiles;
  int dep_c0;        // first depth row of the tile's window
  int seq_full_hi;   // sequence keys below this bound are visible to every row of the tile
};
template <int BM, int BN>
__device__ __forceinline__ KeyWalk make_walk(const Params& p, int r0) {
  KeyWalk w;
  const int r_last = min(r0 + BM, p.T_q) - 1;
  int lo, hi, lo2, hi2;
  seq_interval(p, r_last, lo, hi);
  w.n_seq_tiles = (hi + BN - 1) / BN;
  seq_interval(p, r0, lo2, hi2);
  w.seq_full_hi = hi2;
  dep_interval(p, r0, lo, hi);
  dep_interval(p, r_last, lo2, hi2);
  w.dep_c0 = lo;
  w.n_dep_tiles = (hi2 - lo + BN - 1) / BN;
  return w;
}

// =================================================================== forward
// grid (ceil(T_q/64), H, B), 128 threads; warp w owns query rows [16w, 16w+16).
template <typename T, int D>
__global__ void __launch_bounds__(128) fwd_kernel(const __grid_constant__ Params p) {
  constexpr int BM = 64, BN = 64, NT = 128;
  using TL = Tile<T, D>;
  constexpr int LD = TL::LD;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  T* sQ = reinterpret_cast<T*>(smem_raw);
  T* sK = sQ + BM * LD;       // 2 stages
  T* sV = sK + 2 * BN * LD;   // 2 stages

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, tq = lane & 3;
  const int n_qt = (p.T_q + BM - 1) / BM;
  const int qt = n_qt - 1 - (int)blockIdx.x;   // heaviest (latest) causal tiles first
  const int h = blockIdx.y, b = blockIdx.z;
  const int r0 = qt * BM;
  const KeyWalk walk = make_walk<BM, BN>(p, r0);
  const int n_tiles = walk.n_seq_tiles + walk.n_dep_tiles;

  const T* gq = reinterpret_cast<const T*>(p.q.ptr) + p.q.off(b, 0, h);
  const T* gk = reinterpret_cast<const T*>(p.k.ptr) + p.k.off(b, 0, h);
  const T* gv = reinterpret_cast<const T*>(p.v.ptr) + p.v.off(b, 0, h);
  const T* gkd = reinterpret_cast<const T*>(p.kd.ptr) + p.kd.off(b, 0, h);
  const T* gvd = reinterpret_cast<const T*>(p.vd.ptr) + p.vd.off(b, 0, h);

  auto issue = [&](int i) {
    const int st = i & 1;
    if (i < walk.n_seq_tiles) {
      TL::template load<BN, NT>(sK + st * BN * LD, gk, p.k.st, (int64_t)i * BN, p.T_kv, tid);
      TL::template load<BN, NT>(sV + st * BN * LD, gv, p.v.st, (int64_t)i * BN, p.T_kv, tid);
    } else {
      const int64_t c0 = walk.dep_c0 + (int64_t)(i - walk.n_seq_tiles) * BN;
      const int64_t n = (int64_t)p.T_kv * p.L;
      TL::template load<BN, NT>(sK + st * BN * LD, gkd, p.kd.st, c0, n, tid, p.L, p.Ls);
      TL::template load<BN, NT>(sV + st * BN * LD, gvd, p.vd.st, c0, n, tid, p.L, p.Ls);
    }
  };

  TL::template load<BM, NT>(sQ, gq, p.q.st, r0, p.T_q, tid);
  if (n_tiles > 0) issue(0);
  cp_async_commit();

  const int rA = r0 + warp * 16 + g, rB = rA + 8;
  int sloA, shiA, sloB, shiB, dloA, dhiA, dloB, dhiB;
  seq_interval(p, rA, sloA, shiA); seq_interval(p, rB, sloB, shiB);
  dep_interval(p, rA, dloA, dhiA); dep_interval(p, rB, dloB, dhiB);
  // warp-wide visible windows (first row's lo, last row's hi)
  int wslo, wshi, wdlo, wdhi, tmp;
  seq_interval(p, r0 + warp * 16, wslo, tmp); seq_interval(p, min(r0 + warp * 16 + 15, p.T_q - 1), tmp, wshi);
  dep_interval(p, r0 + warp * 16, wdlo, tmp); dep_interval(p, min(r0 + warp * 16 + 15, p.T_q - 1), tmp, wdhi);
  if (r0 + warp * 16 >= p.T_q) { wshi = 0; wdhi = 0; wslo = 0; wdlo = 0; }

  float mA = -INFINITY, mB = -INFINITY, lA = 0.f, lB = 0.f;
  float acc[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) { acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f; }

  for (int it = 0; it < n_tiles; ++it) {
    if (it + 1 < n_tiles) issue(it + 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    const T* cK = sK + (it & 1) * BN * LD;
    const T* cV = sV + (it & 1) * BN * LD;

    const bool is_dep = it >= walk.n_seq_tiles;
    const int c0 = is_dep ? walk.dep_c0 + (it - walk.n_seq_tiles) * BN : it * BN;
    const bool masked = is_dep || (c0 + BN > walk.seq_full_hi);
    const int loA = is_dep ? dloA : sloA, hiA = is_dep ? dhiA : shiA;
    const int loB = is_dep ? dloB : sloB, hiB = is_dep ? dhiB : shiB;
    const int wlo = is_dep ? wdlo : wslo, whi = is_dep ? wdhi : wshi;

    // 16-key groups of this tile the warp can skip entirely
    unsigned live = 0xF;
    if (masked) {
      live = 0;
#pragma unroll
      for (int j = 0; j < BN / 16; ++j)
        if (c0 + j * 16 < whi && c0 + j * 16 + 16 > wlo) live |= 1u << j;
    }

    if (live) {
      float s[BN / 8][4];
#pragma unroll
      for (int i = 0; i < BN / 8; ++i) { s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f; }
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) {
        uint32_t a[4];
        TL::ldA(a, sQ, warp * 16, kk * 16, lane);
#pragma unroll
        for (int j = 0; j < BN / 16; ++j) {
          if (live & (1u << j)) {
            uint32_t bb[4];
            TL::ldB_nk(bb, cK, j * 16, kk * 16, lane);
            Mma<T>::run(s[2 * j], a, bb[0], bb[1]);
            Mma<T>::run(s[2 * j + 1], a, bb[2], bb[3]);
          }
        }
      }
      float mxA = -INFINITY, mxB = -INFINITY;
#pragma unroll
      for (int nb = 0; nb < BN / 8; ++nb) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          float xa = s[nb][e] * p.scale_log2, xb = s[nb][2 + e] * p.scale_log2;
          if (masked) {
            const int col = c0 + nb * 8 + tq * 2 + e;
            if (col < loA || col >= hiA) xa = -INFINITY;
            if (col < loB || col >= hiB) xb = -INFINITY;
          }
          s[nb][e] = xa; s[nb][2 + e] = xb;
          mxA = fmaxf(mxA, xa); mxB = fmaxf(mxB, xb);
        }
      }
      mxA = fmaxf(mxA, __shfl_xor_sync(0xffffffffu, mxA, 1));
      mxA = fmaxf(mxA, __shfl_xor_sync(0xffffffffu, mxA, 2));
      mxB = fmaxf(mxB, __shfl_xor_sync(0xffffffffu, mxB, 1));
      mxB = fmaxf(mxB, __shfl_xor_sync(0xffffffffu, mxB, 2));
      const float nmA = fmaxf(mA, mxA), nmB = fmaxf(mB, mxB);
      const float safeA = (nmA == -INFINITY) ? 0.f : nmA, safeB = (nmB == -INFINITY) ? 0.f : nmB;
      const float alA = fast_exp2(mA - safeA), alB = fast_exp2(mB - safeB);
      mA = nmA; mB = nmB;
      float sumA = 0.f, sumB = 0.f;
#pragma unroll
      for (int nb = 0; nb < BN / 8; ++nb) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const float pa = fast_exp2(s[nb][e] - safeA), pb = fast_exp2(s[nb][2 + e] - safeB);
          s[nb][e] = pa; s[nb][2 + e] = pb;
          sumA += pa; sumB += pb;
        }
      }
      lA = lA * alA + sumA; lB = lB * alB + sumB;
#pragma unroll
      for (int i = 0; i < D / 8; ++i) { acc[i][0] *= alA; acc[i][1] *= alA; acc[i][2] *= alB; acc[i][3] *= alB; }
#pragma unroll
      for (int j = 0; j < BN / 16; ++j) {
        if (live & (1u << j)) {
          uint32_t a[4];
          a[0] = Pack<T>::pack(s[2 * j][0], s[2 * j][1]);
          a[1] = Pack<T>::pack(s[2 * j][2], s[2 * j][3]);
          a[2] = Pack<T>::pack(s[2 * j + 1][0], s[2 * j + 1][1]);
          a[3] = Pack<T>::pack(s[2 * j + 1][2], s[2 * j + 1][3]);
#pragma unroll
          for (int d2 = 0; d2 < D / 16; ++d2) {
            uint32_t bb[4];
            TL::ldB_kn(bb, cV, j * 16, d2 * 16, lane);
            Mma<T>::run(acc[2 * d2], a, bb[0], bb[1]);
            Mma<T>::run(acc[2 * d2 + 1], a, bb[2], bb[3]);
          }
        }
      }
    }
    __syncthreads();
  }
  cp_async_wait<0>();

  lA += __shfl_xor_sync(0xffffffffu, lA, 1); lA += __shfl_xor_sync(0xffffffffu, lA, 2);
  lB += __shfl_xor_sync(0xffffffffu, lB, 1); lB += __shfl_xor_sync(0xffffffffu, lB, 2);
  float invA = lA > 0.f ? 1.f / lA : 0.f, invB = lB > 0.f ? 1.f / lB : 0.f;
  float depA = 0.f, depB = 0.f, lseA = mA + log2f(lA), lseB = mB + log2f(lB);
  const bool merge = p.merge_depth != 0;
  if (merge) {   // fold this kernel's sequence part into the stored depth-only partial
    if (rA < p.T_q) merge_partials(mA, lA, p.lse[((int64_t)b * p.T_q + rA) * p.H + h], invA, depA, lseA);
    if (rB < p.T_q) merge_partials(mB, lB, p.lse[((int64_t)b * p.T_q + rB) * p.H + h], invB, depB, lseB);
    __syncwarp();   // every lane of a row's quad has read the stored lse before lane 0 replaces it
  }
  T* go = reinterpret_cast<T*>(p.o.ptr) + p.o.off(b, 0, h);
  if (rA < p.T_q) {
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
      uint32_t* dst = reinterpret_cast<uint32_t*>(go + (int64_t)rA * p.o.st + i * 8 + tq * 2);
      float x = acc[i][0] * invA, y = acc[i][1] * invA;
      if (merge) { const float2 prev = Pack<T>::unpack(*dst); x = fmaf(prev.x, depA, x); y = fmaf(prev.y, depA, y); }
      *dst = Pack<T>::pack(x, y);
    }
    if (tq == 0) p.lse[((int64_t)b * p.T_q + rA) * p.H + h] = lseA;
  }
  if (rB < p.T_q) {
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
      uint32_t* dst = reinterpret_cast<uint32_t*>(go + (int64_t)rB * p.o.st + i * 8 + tq * 2);
      float x = acc[i][2] * invB, y = acc[i][3] * invB;
      if (merge) { const float2 prev = Pack<T>::unpack(*dst); x = fmaf(prev.x, depB, x); y = fmaf(prev.y, depB, y); }
      *dst = Pack<T>::pack(x, y);
    }
    if (tq == 0) p.lse[((int64_t)b * p.T_q + rB) * p.H + h] = lseB;
  }
}

// ============================================================ delta preprocess
// delta[b, r, h] = sum_d o * dout with the stored (rounded) o, fp32 accumulate
// (moda_v14.py:525-539).  One warp per row; grid-stride.
template <typename T, int D>
__global__ void __launch_bounds__(256) delta_kernel(const __grid_constant__ Params p) {
  const int lane = threadIdx.x & 31;
  const int64_t n_rows = (int64_t)p.B * p.T_q * p.H;
  const int64_t wstride = (int64_t)gridDim.x * (blockDim.x >> 5);
  for (int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); row < n_rows; row += wstride) {
    const int h = (int)(row % p.H);
    const int64_t bt = row / p.H;
    const int r = (int)(bt % p.T_q), b = (int)(bt / p.T_q);
    const T* po = reinterpret_cast<const T*>(p.o.ptr) + p.o.off(b, r, h);
    const T* pd = reinterpret_cast<const T*>(p.dout.ptr) + p.dout.off(b, r, h);
    float s = 0.f;
    for (int c = lane * 2; c < D; c += 64) {
      const float2 a = Pack<T>::unpack(*reinterpret_cast<const uint32_t*>(po + c));
      const float2 d = Pack<T>::unpack(*reinterpret_cast<const uint32_t*>(pd + c));
      s += a.x * d.x + a.y * d.y;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0) p.delta[row] = s;
  }
}

// ======================================================================== dq
// Same walk as the forward.  P = exp2(S*c - lse), dP = dO V^T, dS = P (dP - delta),
// dq = scale * dS K  (moda_v14.py:542-871).
template <typename T, int D>
__global__ void __launch_bounds__(128) dq_kernel(const __grid_constant__ Params p) {
  constexpr int BM = 64, BN = 64, NT = 128;
  using TL = Tile<T, D>;
  constexpr int LD = TL::LD;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  T* sQ = reinterpret_cast<T*>(smem_raw);
  T* sDO = sQ + BM * LD;
  T* sK = sDO + BM * LD;      // 2 stages
  T* sV = sK + 2 * BN * LD;   // 2 stages

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, tq = lane & 3;
  const int n_qt = (p.T_q + BM - 1) / BM;
  const int qt = n_qt - 1 - (int)blockIdx.x;
  const int h = blockIdx.y, b = blockIdx.z;
  const int r0 = qt * BM;
  const KeyWalk walk = make_walk<BM, BN>(p, r0);
  const int n_tiles = walk.n_seq_tiles + walk.n_dep_tiles;

  const T* gq = reinterpret_cast<const T*>(p.q.ptr) + p.q.off(b, 0, h);
  const T* gdo = reinterpret_cast<const T*>(p.dout.ptr) + p.dout.off(b, 0, h);
  const T* gk = reinterpret_cast<const T*>(p.k.ptr) + p.k.off(b, 0, h);
  const T* gv = reinterpret_cast<const T*>(p.v.ptr) + p.v.off(b, 0, h);
  const T* gkd = reinterpret_cast<const T*>(p.kd.ptr) + p.kd.off(b, 0, h);
  const T* gvd = reinterpret_cast<const T*>(p.vd.ptr) + p.vd.off(b, 0, h);

  auto issue = [&](int i) {
    const int st = i & 1;
    if (i < walk.n_seq_tiles) {
      TL::template load<BN, NT>(sK + st * BN * LD, gk, p.k.st, (int64_t)i * BN, p.T_kv, tid);
      TL::template load<BN, NT>(sV + st * BN * LD, gv, p.v.st, (int64_t)i * BN, p.T_kv, tid);
    } else {
      const int64_t c0 = walk.dep_c0 + (int64_t)(i - walk.n_seq_tiles) * BN;
      const int64_t n = (int64_t)p.T_kv * p.L;
      TL::template load<BN, NT>(sK + st * BN * LD, gkd, p.kd.st, c0, n, tid, p.L, p.Ls);
      TL::template load<BN, NT>(sV + st * BN * LD, gvd, p.vd.st, c0, n, tid, p.L, p.Ls);
    }
  };

  TL::template load<BM, NT>(sQ, gq, p.q.st, r0, p.T_q, tid);
  TL::template load<BM, NT>(sDO, gdo, p.dout.st, r0, p.T_q, tid);
  if (n_tiles > 0) issue(0);
  cp_async_commit();

  const int rA = r0 + warp * 16 + g, rB = rA + 8;
  int sloA, shiA, sloB, shiB, dloA, dhiA, dloB, dhiB;
  seq_interval(p, rA, sloA, shiA); seq_interval(p, rB, sloB, shiB);
  dep_interval(p, rA, dloA, dhiA); dep_interval(p, rB, dloB, dhiB);
  int wslo, wshi, wdlo, wdhi, tmp;
  seq_interval(p, r0 + warp * 16, wslo, tmp); seq_interval(p, min(r0 + warp * 16 + 15, p.T_q - 1), tmp, wshi);
  dep_interval(p, r0 + warp * 16, wdlo, tmp); dep_interval(p, min(r0 + warp * 16 + 15, p.T_q - 1), tmp, wdhi);
  if (r0 + warp * 16 >= p.T_q) { wshi = 0; wdhi = 0; wslo = 0; wdlo = 0; }

  float lseA = 0.f, lseB = 0.f, dlA = 0.f, dlB = 0.f;
  if (rA < p.T_q) { const int64_t i = ((int64_t)b * p.T_q + rA) * p.H + h; lseA = p.lse[i]; dlA = p.delta[i]; }
  if (rB < p.T_q) { const int64_t i = ((int64_t)b * p.T_q + rB) * p.H + h; lseB = p.lse[i]; dlB = p.delta[i]; }

  float acc[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) { acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f; }

  for (int it = 0; it < n_tiles; ++it) {
    if (it + 1 < n_tiles) issue(it + 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    const T* cK = sK + (it & 1) * BN * LD;
    const T* cV = sV + (it & 1) * BN * LD;

    const bool is_dep = it >= walk.n_seq_tiles;
    const int c0 = is_dep ? walk.dep_c0 + (it - walk.n_seq_tiles) * BN : it * BN;
    const bool masked = is_dep || (c0 + BN > walk.seq_full_hi);
    const int loA = is_dep ? dloA : sloA, hiA = is_dep ? dhiA : shiA;
    const int loB = is_dep ? dloB : sloB, hiB = is_dep ? dhiB : shiB;
    const int wlo = is_dep ? wdlo : wslo, whi = is_dep ? wdhi : wshi;
    unsigned live = 0xF;
    if (masked) {
      live = 0;
#pragma unroll
      for (int j = 0; j < BN / 16; ++j)
        if (c0 + j * 16 < whi && c0 + j * 16 + 16 > wlo) live |= 1u << j;
    }
    if (live) {
      float s[BN / 8][4], dp[BN / 8][4];
#pragma unroll
      for (int i = 0; i < BN / 8; ++i) {
        s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
        dp[i][0] = dp[i][1] = dp[i][2] = dp[i][3] = 0.f;
      }
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) {
        uint32_t a[4], ad[4];
        TL::ldA(a, sQ, warp * 16, kk * 16, lane);
        TL::ldA(ad, sDO, warp * 16, kk * 16, lane);
#pragma unroll
        for (int j = 0; j < BN / 16; ++j) {
          if (live & (1u << j)) {
            uint32_t bb[4];
            TL::ldB_nk(bb, cK, j * 16, kk * 16, lane);
            Mma<T>::run(s[2 * j], a, bb[0], bb[1]);
            Mma<T>::run(s[2 * j + 1], a, bb[2], bb[3]);
            TL::ldB_nk(bb, cV, j * 16, kk * 16, lane);
            Mma<T>::run(dp[2 * j], ad, bb[0], bb[1]);
            Mma<T>::run(dp[2 * j + 1], ad, bb[2], bb[3]);
          }
        }
      }
#pragma unroll
      for (int nb = 0; nb < BN / 8; ++nb) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          float pa = fast_exp2(s[nb][e] * p.scale_log2 - lseA);
          float pb = fast_exp2(s[nb][2 + e] * p.scale_log2 - lseB);
          if (masked) {
            const int col = c0 + nb * 8 + tq * 2 + e;
            if (col < loA || col >= hiA) pa = 0.f;
            if (col < loB || col >= hiB) pb = 0.f;
          }
          s[nb][e] = pa * (dp[nb][e] - dlA);
          s[nb][2 + e] = pb * (dp[nb][2 + e] - dlB);
        }
      }
#pragma unroll
      for (int j = 0; j < BN / 16; ++j) {
        if (live & (1u << j)) {
          uint32_t a[4];
          a[0] = Pack<T>::pack(s[2 * j][0], s[2 * j][1]);
          a[1] = Pack<T>::pack(s[2 * j][2], s[2 * j][3]);
          a[2] = Pack<T>::pack(s[2 * j + 1][0], s[2 * j + 1][1]);
          a[3] = Pack<T>::pack(s[2 * j + 1][2], s[2 * j + 1][3]);
#pragma unroll
          for (int d2 = 0; d2 < D / 16; ++d2) {
            uint32_t bb[4];
            TL::ldB_kn(bb, cK, j * 16, d2 * 16, lane);
            Mma<T>::run(acc[2 * d2], a, bb[0], bb[1]);
            Mma<T>::run(acc[2 * d2 + 1], a, bb[2], bb[3]);
          }
        }
      }
    }
    __syncthreads();
  }
  cp_async_wait<0>();

  T* gdq = reinterpret_cast<T*>(p.dq.ptr) + p.dq.off(b, 0, h);
  const bool merge = p.merge_depth != 0;   // dq already holds the depth rows' share
  if (rA < p.T_q) {
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
      uint32_t* dst = reinterpret_cast<uint32_t*>(gdq + (int64_t)rA * p.dq.st + i * 8 + tq * 2);
      float x = acc[i][0] * p.scale, y = acc[i][1] * p.scale;
      if (merge) { const float2 prev = Pack<T>::unpack(*dst); x += prev.x; y += prev.y; }
      *dst = Pack<T>::pack(x, y);
    }
  }
  if (rB < p.T_q) {
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
      uint32_t* dst = reinterpret_cast<uint32_t*>(gdq + (int64_t)rB * p.dq.st + i * 8 + tq * 2);
      float x = acc[i][2] * p.scale, y = acc[i][3] * p.scale;
      if (merge) { const float2 prev = Pack<T>::unpack(*dst); x += prev.x; y += prev.y; }
      *dst = Pack<T>::pack(x, y);
    }
  }
}

// ===================================================================== dk / dv
// Key-parallel: one CTA owns 64 keys (warp w owns 16) of either the sequence K/V or
// the depth K/V and walks the query tiles that can see them; the G heads of a KV head
// are rows of the same folded query tile, so their contributions are summed inside
// the MMAs (the reference needs a [B,T,H,G,K] scratch and a host-side sum for this:
// moda_v14.py:1715-1752).  Computes transposed scores S^T = K Q^T so that P^T and
// dS^T come out as A operands:  dv = P^T dO,  dk = scale * dS^T Q
// (moda_v14.py:1042-1248 sequence keys, moda_v14.py:1251-1454 depth keys).
// grid (n_seq_key_tiles + n_dep_key_tiles, H, B), 128 threads.
template <typename T, int D>
__global__ void __launch_bounds__(128) dkv_kernel(const __grid_constant__ Params p, int n_seq_key_tiles) {
  constexpr int BN = 64;                  // keys per CTA
  constexpr int BM = (D == 128) ? 32 : 64;  // query rows per step
  constexpr int NT = 128;
  using TL = Tile<T, D>;
  constexpr int LD = TL::LD;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  T* sK = reinterpret_cast<T*>(smem_raw);
  T* sV = sK + BN * LD;
  T* sQ = sV + BN * LD;        // 2 stages of BM rows
  T* sDO = sQ + 2 * BM * LD;   // 2 stages
  float* sLse = reinterpret_cast<float*>(sDO + 2 * BM * LD);  // 2 x BM
  float* sDel = sLse + 2 * BM;
  int* sLo = reinterpret_cast<int*>(sDel + 2 * BM);
  int* sHi = sLo + 2 * BM;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, tq = lane & 3;
  const int h = blockIdx.y, b = blockIdx.z;
  const bool is_dep = (int)blockIdx.x >= n_seq_key_tiles;
  const int c0 = (is_dep ? (int)blockIdx.x - n_seq_key_tiles : (int)blockIdx.x) * BN;
  const int n_keys = is_dep ? p.T_kv * p.L : p.T_kv;
  const int c_last = min(c0 + BN, n_keys) - 1;

  // query rows that can see any key of this tile: [q_begin, q_end)
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
  q_begin = (q_begin / BM) * BM;
  const int n_steps = (q_end - q_begin + BM - 1) / BM;

  const View& kv_k = is_dep ? p.kd : p.k;
  const View& kv_v = is_dep ? p.vd : p.v;
  const T* gk = reinterpret_cast<const T*>(kv_k.ptr) + kv_k.off(b, 0, h);
  const T* gv = reinterpret_cast<const T*>(kv_v.ptr) + kv_v.off(b, 0, h);
  const T* gq = reinterpret_cast<const T*>(p.q.ptr) + p.q.off(b, 0, h);
  const T* gdo = reinterpret_cast<const T*>(p.dout.ptr) + p.dout.off(b, 0, h);

  auto issue = [&](int i) {
    const int st = i & 1;
    const int q0 = q_begin + i * BM;
    TL::template load<BM, NT>(sQ + st * BM * LD, gq, p.q.st, q0, p.T_q, tid);
    TL::template load<BM, NT>(sDO + st * BM * LD, gdo, p.dout.st, q0, p.T_q, tid);
    if (tid < BM) {
      const int r = q0 + tid;
      float l = 0.f, d = 0.f;
      int lo, hi;
      if (is_dep) dep_interval(p, r, lo, hi); else seq_interval(p, r, lo, hi);
      if (r < p.T_q) { const int64_t idx = ((int64_t)b * p.T_q + r) * p.H + h; l = p.lse[idx]; d = p.delta[idx]; }
      sLse[st * BM + tid] = l; sDel[st * BM + tid] = d;
      sLo[st * BM + tid] = lo; sHi[st * BM + tid] = hi;
    }
  };

  const int grpL = is_dep ? p.L : 1, grpLs = is_dep ? p.Ls : 1;   // memory layout of the key rows
  TL::template load<BN, NT>(sK, gk, kv_k.st, c0, n_keys, tid, grpL, grpLs);
  TL::template load<BN, NT>(sV, gv, kv_v.st, c0, n_keys, tid, grpL, grpLs);
  if (n_steps > 0) issue(0);
  cp_async_commit();

  float dk[D / 8][4], dv[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) {
    dk[i][0] = dk[i][1] = dk[i][2] = dk[i][3] = 0.f;
    dv[i][0] = dv[i][1] = dv[i][2] = dv[i][3] = 0.f;
  }
  const int keyA = c0 + warp * 16 + g, keyB = keyA + 8;   // this thread's two key rows
  const int wk0 = c0 + warp * 16;                          // warp's first key

  for (int it = 0; it < n_steps; ++it) {
    if (it + 1 < n_steps) issue(it + 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    const int st = it & 1;
    const T* cQ = sQ + st * BM * LD;
    const T* cDO = sDO + st * BM * LD;
    const float* cLse = sLse + st * BM;
    const float* cDel = sDel + st * BM;
    const int* cLo = sLo + st * BM;
    const int* cHi = sHi + st * BM;

    // 16-row groups of this step that can see the warp's 16 keys
    // (intervals are monotone over valid rows only, so clamp to the last valid row)
    unsigned live = 0;
    const int last_valid = p.T_q - 1 - (q_begin + it * BM);
#pragma unroll
    for (int j = 0; j < BM / 16; ++j) {
      const int jl = min(j * 16 + 15, last_valid);
      if (jl >= j * 16 && cLo[j * 16] < wk0 + 16 && cHi[jl] > wk0) live |= 1u << j;
    }

    if (live) {
      float s[BM / 8][4], dp[BM / 8][4];
#pragma unroll
      for (int i = 0; i < BM / 8; ++i) {
        s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
        dp[i][0] = dp[i][1] = dp[i][2] = dp[i][3] = 0.f;
      }
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) {
        uint32_t a[4], av[4];
        TL::ldA(a, sK, warp * 16, kk * 16, lane);
        TL::ldA(av, sV, warp * 16, kk * 16, lane);
#pragma unroll
        for (int j = 0; j < BM / 16; ++j) {
          if (live & (1u << j)) {
            uint32_t bb[4];
            TL::ldB_nk(bb, cQ, j * 16, kk * 16, lane);
            Mma<T>::run(s[2 * j], a, bb[0], bb[1]);
            Mma<T>::run(s[2 * j + 1], a, bb[2], bb[3]);
            TL::ldB_nk(bb, cDO, j * 16, kk * 16, lane);
            Mma<T>::run(dp[2 * j], av, bb[0], bb[1]);
            Mma<T>::run(dp[2 * j + 1], av, bb[2], bb[3]);
          }
        }
      }
      // element (key row, query col): regs 0,1 -> keyA, cols 2tq,2tq+1; regs 2,3 -> keyB
#pragma unroll
      for (int nb = 0; nb < BM / 8; ++nb) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int rr = nb * 8 + tq * 2 + e;
          const float l = cLse[rr], d = cDel[rr];
          const int lo = cLo[rr], hi = cHi[rr];
          float pa = (keyA >= lo && keyA < hi) ? fast_exp2(s[nb][e] * p.scale_log2 - l) : 0.f;
          float pb = (keyB >= lo && keyB < hi) ? fast_exp2(s[nb][2 + e] * p.scale_log2 - l) : 0.f;
          s[nb][e] = pa; s[nb][2 + e] = pb;
          dp[nb][e] = pa * (dp[nb][e] - d);
          dp[nb][2 + e] = pb * (dp[nb][2 + e] - d);
        }
      }
#pragma unroll
      for (int j = 0; j < BM / 16; ++j) {
        if (live & (1u << j)) {
          uint32_t ap[4], ads[4];
          ap[0] = Pack<T>::pack(s[2 * j][0], s[2 * j][1]);
          ap[1] = Pack<T>::pack(s[2 * j][2], s[2 * j][3]);
          ap[2] = Pack<T>::pack(s[2 * j + 1][0], s[2 * j + 1][1]);
          ap[3] = Pack<T>::pack(s[2 * j + 1][2], s[2 * j + 1][3]);
          ads[0] = Pack<T>::pack(dp[2 * j][0], dp[2 * j][1]);
          ads[1] = Pack<T>::pack(dp[2 * j][2], dp[2 * j][3]);
          ads[2] = Pack<T>::pack(dp[2 * j + 1][0], dp[2 * j + 1][1]);
          ads[3] = Pack<T>::pack(dp[2 * j + 1][2], dp[2 * j + 1][3]);
#pragma unroll
          for (int d2 = 0; d2 < D / 16; ++d2) {
            uint32_t bb[4];
            TL::ldB_kn(bb, cDO, j * 16, d2 * 16, lane);
            Mma<T>::run(dv[2 * d2], ap, bb[0], bb[1]);
            Mma<T>::run(dv[2 * d2 + 1], ap, bb[2], bb[3]);
            TL::ldB_kn(bb, cQ, j * 16, d2 * 16, lane);
            Mma<T>::run(dk[2 * d2], ads, bb[0], bb[1]);
            Mma<T>::run(dk[2 * d2 + 1], ads, bb[2], bb[3]);
          }
        }
      }
    }
    __syncthreads();
  }
  cp_async_wait<0>();

  const View& ok = is_dep ? p.dkd : p.dk;
  const View& ov = is_dep ? p.dvd : p.dv;
  T* gdk = reinterpret_cast<T*>(ok.ptr) + ok.off(b, 0, h);
  T* gdv = reinterpret_cast<T*>(ov.ptr) + ov.off(b, 0, h);
  const bool acc = is_dep && p.acc_depth != 0;   // depth gradients added to a cache shared by several layers
  auto store2 = [&](T* dst, float a, float b2) {
    uint32_t* w = reinterpret_cast<uint32_t*>(dst);
    if (acc) { const float2 old = Pack<T>::unpack(*w); a += old.x; b2 += old.y; }
    *w = Pack<T>::pack(a, b2);
  };
  if (keyA < n_keys) {
    const int64_t rowA = is_dep ? dep_mem_row(p, keyA) : keyA;
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
      store2(gdk + rowA * ok.st + i * 8 + tq * 2, dk[i][0] * p.scale, dk[i][1] * p.scale);
      store2(gdv + rowA * ov.st + i * 8 + tq * 2, dv[i][0], dv[i][1]);
    }
  }
  if (keyB < n_keys) {
    const int64_t rowB = is_dep ? dep_mem_row(p, keyB) : keyB;
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
      store2(gdk + rowB * ok.st + i * 8 + tq * 2, dk[i][2] * p.scale, dk[i][3] * p.scale);
      store2(gdv + rowB * ov.st + i * 8 + tq * 2, dv[i][2], dv[i][3]);
    }
  }
}

template <typename T, int D> constexpr size_t fwd_smem() { return (size_t)(64 + 4 * 64) * (D + 8) * sizeof(T); }
template <typename T, int D> constexpr size_t dq_smem() { return (size_t)(2 * 64 + 4 * 64) * (D + 8) * sizeof(T); }
template <typename T, int D> constexpr size_t dkv_smem() {
  constexpr int BM = (D == 128) ? 32 : 64;
  return (size_t)(2 * 64 + 4 * BM) * (D + 8) * sizeof(T) + 2 * BM * (2 * sizeof(float) + 2 * sizeof(int));
}

}  // namespace simt
}  // namespace moda
