// Shared definitions of the MoDA kernels: the launch parameter block, the visibility
// rule (one place for every mask in the library), and small device primitives.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace moda {

enum Mode : int { kCausal = 0, kNonCausal = 1, kChunkVisible = 2, kDepthOnly = 3 };

// Element strides of a [B, T, H, D] tensor (innermost stride 1).
struct View {
  void* ptr;
  int64_t sb, st, sh;
  __host__ __device__ __forceinline__ int64_t off(int b, int64_t t, int h) const {
    return (int64_t)b * sb + t * st + (int64_t)h * sh;
  }
};

struct Params {
  View q, k, v, kd, vd, o;          // forward
  View dout, dq, dk, dv, dkd, dvd;  // backward
  float* lse;                       // [B, T_q, H] fp32 (base-2)
  float* delta;                     // [B, T_q, H] fp32 rowsum(o * dout)
  int B, H, T_kv, T_q, G, L;
  int mode;
  int Cb;                           // chunk-visible: base positions per chunk (chunk_rows / G)
  float scale;                      // softmax scale
  float scale_log2;                 // scale * log2(e); reference constant 1.4426950216 (moda_v14.py:109)
  // Split evaluation of the own-position depth modes: the bandwidth kernels have already written
  // the depth-only partial (forward: o = softmax over the depth rows alone, lse = its log-sum-exp;
  // backward: dq = the depth rows' share) and this launch, run with L = 0, folds its sequence
  // part into it in the epilogue.
  int merge_depth;
  // Depth rows per position IN MEMORY.  Ls == L: the packed [B, T*L, H, D] layout (row t*L + l).
  // Ls > L: rows (t, l), l < L, of an in-place cache [B, T, Ls, H, D] written layer by layer,
  // i.e. depth row c = t*L + l of the operator lives at memory row t*Ls + l; the depth gradients
  // use the same layout.  acc_depth: add d_depth_k / d_depth_v to what the buffers hold instead of
  // overwriting (every depth row has one owning thread block, so this stays deterministic).
  int Ls;
  int acc_depth;
};

// Memory row of depth row c (see Params::Ls).
__host__ __device__ __forceinline__ int64_t dep_mem_row(const Params& p, int64_t c) {
  return (p.Ls == p.L) ? c : (c / p.L) * p.Ls + (c % p.L);
}

// Order in which a grid (tiles, H, B) is worked through.  Thread blocks are handed out x-fastest,
// so by default a wave of them works on the tiles of ONE (batch, head), whose K/V then stay in L2.
// When the sequence K/V of all heads together are small against L2 that locality comes for free
// and the causal imbalance between tiles is what matters: `rank` then runs over the tiles of
// every head alike, so that the heaviest tiles of ALL heads start first and the light ones fill
// the tail of a short launch.  (Depth rows are read once, by one block: they do not count.)
struct BlockId { int rank, h, b; };
__device__ __forceinline__ BlockId block_order(const Params& p, int head_dim) {
  const int64_t seq_kv_bytes = (int64_t)p.B * p.H * p.T_kv * head_dim * 4;     // K and V, 16-bit
  if (seq_kv_bytes > ((int64_t)48 << 20)) return {(int)blockIdx.x, (int)blockIdx.y, (int)blockIdx.z};
  const int hb = (int)(gridDim.y * gridDim.z);
  const int lin = (int)(blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z));
  const int r = lin / hb, w = lin - r * hb;
  return {r, w % (int)gridDim.y, w / (int)gridDim.y};
}

// ---------------------------------------------------------------------------
// Visibility.  A query row r (base position t = r / G) sees
//   sequence key j     iff  seq_lo <= j < seq_hi
//   depth row c=t'*L+l iff  dep_lo <= c < dep_hi
// Both intervals are monotone non-decreasing in r, which the kernels rely on to
// derive tile ranges from a tile's first and last row.
//   causal / chunk-visible: seq [0, t+1)            moda_v14.py:250, moda_v16.py:2553
//   non-causal:             seq [0, T_kv)           moda_v14.py:259-300
//   own-position depth:     dep [t*L, (t+1)*L)      moda_v14.py:352-356
//   chunk-visible depth:    dep [chunk_start(t)*L, (t+1)*L)   moda_v16.py:325-328
// Rows r >= T_q see nothing.
// ---------------------------------------------------------------------------
__host__ __device__ __forceinline__ void seq_interval(const Params& p, int r, int& lo, int& hi) {
  lo = 0;
  if (r >= p.T_q || p.mode == kDepthOnly) { hi = 0; return; }
  hi = (p.mode == kNonCausal) ? p.T_kv : (r / p.G + 1);
}
__host__ __device__ __forceinline__ void dep_interval(const Params& p, int r, int& lo, int& hi) {
  if (r >= p.T_q || p.L == 0) { lo = 0; hi = 0; return; }
  const int t = r / p.G;
  const int t0 = (p.mode == kChunkVisible) ? (t / p.Cb) * p.Cb : t;
  lo = t0 * p.L;
  hi = (t + 1) * p.L;
}

// ---------------------------------------------------------------------------
// dtype traits
// ---------------------------------------------------------------------------
template <typename T> struct Pack;
template <> struct Pack<__nv_bfloat16> {
  static __device__ __forceinline__ uint32_t pack(float a, float b) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
  }
  static __device__ __forceinline__ float2 unpack(uint32_t u) {
    return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&u));
  }
};
template <> struct Pack<__half> {
  static __device__ __forceinline__ uint32_t pack(float a, float b) {
    __half2 v = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
  }
  static __device__ __forceinline__ float2 unpack(uint32_t u) {
    return __half22float2(*reinterpret_cast<__half2*>(&u));
  }
};

// Eight fp32 values (as register bits) times a, optionally plus eight stored 16-bit values times b.
template <typename T> __device__ __forceinline__ uint4 pack8_scaled(const uint32_t* x, float a) {
  return make_uint4(Pack<T>::pack(__uint_as_float(x[0]) * a, __uint_as_float(x[1]) * a),
                    Pack<T>::pack(__uint_as_float(x[2]) * a, __uint_as_float(x[3]) * a),
                    Pack<T>::pack(__uint_as_float(x[4]) * a, __uint_as_float(x[5]) * a),
                    Pack<T>::pack(__uint_as_float(x[6]) * a, __uint_as_float(x[7]) * a));
}
template <typename T> __device__ __forceinline__ uint4 pack8_blend(const uint32_t* x, float a, const uint4& prev, float b) {
  const float2 p0 = Pack<T>::unpack(prev.x), p1 = Pack<T>::unpack(prev.y), p2 = Pack<T>::unpack(prev.z), p3 = Pack<T>::unpack(prev.w);
  return make_uint4(Pack<T>::pack(fmaf(__uint_as_float(x[0]), a, p0.x * b), fmaf(__uint_as_float(x[1]), a, p0.y * b)),
                    Pack<T>::pack(fmaf(__uint_as_float(x[2]), a, p1.x * b), fmaf(__uint_as_float(x[3]), a, p1.y * b)),
                    Pack<T>::pack(fmaf(__uint_as_float(x[4]), a, p2.x * b), fmaf(__uint_as_float(x[5]), a, p2.y * b)),
                    Pack<T>::pack(fmaf(__uint_as_float(x[6]), a, p3.x * b), fmaf(__uint_as_float(x[7]), a, p3.y * b)));
}

// Softmax partials over two disjoint key sets: this kernel's (unnormalised accumulator, running
// max m, row sum l; lse_self = m + log2 l) and a stored, normalised one with log-sum-exp lse_other.
// Returns the factor for the accumulator (includes 1/l), the factor for the stored row and the
// combined lse.  lse_other must be finite.
__device__ __forceinline__ void merge_partials(float m, float l, float lse_other, float& w_acc, float& w_other, float& lse_out) {
  if (!(l > 0.f)) { w_acc = 0.f; w_other = 1.f; lse_out = lse_other; return; }
  const float lse_self = m + log2f(l);
  const float mx = fmaxf(lse_self, lse_other);
  const float a = exp2f(lse_self - mx), c = exp2f(lse_other - mx);
  const float inv = 1.f / (a + c);
  w_acc = a * inv / l;
  w_other = c * inv;
  lse_out = mx + log2f(a + c);
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// exp2 on the FMA pipe (no MUFU): round-to-nearest split x = n + f, f in [-0.5, 0.5], degree-4
// polynomial for 2^f (max relative error 3.6e-6), 2^n applied through the exponent field.
// Valid for x <= 126; x below -126 (including -inf) is clamped, giving a value <= 2^-126.
// The MUFU unit delivers 16 exp2 per clock per SM against 128 FMAs, and the softmax of one
// 128 x 128 score tile needs as many MUFU cycles as its two matmuls need tensor cycles; moving
// part of the exponentials here takes the MUFU off the critical path.
__device__ __forceinline__ float poly_exp2(float x) {
  x = fmaxf(x, -126.0f);
  const float t = x + 12582912.0f;   // 1.5 * 2^23: the low mantissa bits now hold round(x)
  const float f = x - (t - 12582912.0f);
  float p = fmaf(0.009676037f, f, 0.055922035f);
  p = fmaf(p, f, 0.24022107f);
  p = fmaf(p, f, 0.6931210f);
  p = fmaf(p, f, 1.0000001f);
  return __int_as_float(__float_as_int(p) + (__float_as_int(t) << 23));
}

}  // namespace moda
