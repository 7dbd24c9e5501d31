// Depth-only attention (parallel_fda, fda_v12.py:1346) as HBM-bandwidth kernels.
//
// Each query position attends only to the L depth K/V rows of its own position, so the
// operator moves 2*L*D elements per position for 4*G*L*D flops: about 1 flop per byte.  The
// attention-tile pipeline (tensor cores, 128-row tiles) would multiply every query against
// the depth rows of 127 other positions; here one warp owns one (batch, position, head),
// streams its L K rows and L V rows once with 16-byte loads (8 lanes per 256-byte row, four
// rows per pass, sixteen rows per online-softmax block), keeps scores, softmax and accumulators in fp32 registers, and writes o /
// lse (forward) or dq, d_depth_k, d_depth_v (backward; rows are owner-exclusive, no atomics).
// Numerics as in the other kernels: scores scaled by scale*log2(e), exp2, lse = m + log2(l),
// delta from the stored o, dq and dk scaled by `scale` at the end.
#pragma once
#include "common.cuh"

namespace moda {
namespace fda {

template <typename T> __device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
  const float2 a = Pack<T>::unpack(u.x), b = Pack<T>::unpack(u.y), c = Pack<T>::unpack(u.z), d = Pack<T>::unpack(u.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}
// f += the eight stored 16-bit values of u
template <typename T> __device__ __forceinline__ void add8(float (&f)[8], const uint4& u) {
  float g[8];
  unpack8<T>(u, g);
#pragma unroll
  for (int e = 0; e < 8; ++e) f[e] += g[e];
}
template <typename T> __device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  return make_uint4(Pack<T>::pack(f[0], f[1]), Pack<T>::pack(f[2], f[3]), Pack<T>::pack(f[4], f[5]), Pack<T>::pack(f[6], f[7]));
}
__device__ __forceinline__ float group8_sum(float x) {   // sum over the 8 lanes that share a row
  x += __shfl_xor_sync(0xffffffffu, x, 1);
  x += __shfl_xor_sync(0xffffffffu, x, 2);
  x += __shfl_xor_sync(0xffffffffu, x, 4);
  return x;
}
__device__ __forceinline__ float cross4_sum(float x) {   // sum over the 4 row groups of a warp
  x += __shfl_xor_sync(0xffffffffu, x, 8);
  x += __shfl_xor_sync(0xffffffffu, x, 16);
  return x;
}
__device__ __forceinline__ float cross4_max(float x) {
  x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, 8));
  x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, 16));
  return x;
}

// (b, t, h) of a flattened unit index; 32-bit division when the index fits (64-bit division
// costs hundreds of clocks, which a unit with a few KB of depth rows does not hide).
__device__ __forceinline__ void decode_unit(int64_t unit, int H, int T_kv, int& b, int& t, int& h) {
  if (unit <= 0x7fffffffLL) {
    const unsigned u = (unsigned)unit, uh = u / (unsigned)H;
    h = (int)(u - uh * (unsigned)H);
    b = (int)(uh / (unsigned)T_kv);
    t = (int)(uh - (unsigned)b * (unsigned)T_kv);
  } else {
    h = (int)(unit % H);
    t = (int)((unit / H) % T_kv);
    b = (int)(unit / ((int64_t)H * T_kv));
  }
}

// Lane layout: sub = lane & 7 picks the 16-byte chunks {sub, sub + 8, ...} of a row (CH = D/64
// chunks per lane), grp = lane >> 3 picks which of the 4 rows of a pass the lane works on.

// ------------------------------------------------------------------------- forward
// One warp per (b, t, h); all G query rows of the position reuse the K/V rows (L1-resident on
// the second and later reads).  With 128-byte rows (D = 64) a unit is a few KB and the kernels are
// bound by latency and instruction issue rather than by HBM, so more warps are kept resident there.
template <typename T, int D>
__global__ void __launch_bounds__(256, D == 64 ? 3 : 2) fwd_kernel(const __grid_constant__ Params p) {
  constexpr int CH = D / 64;
  const int lane = threadIdx.x & 31, sub = lane & 7, grp = lane >> 3;
  const int64_t n_units = (int64_t)p.B * p.T_kv * p.H;
  const int64_t wstride = (int64_t)gridDim.x * (blockDim.x >> 5);
  for (int64_t unit = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); unit < n_units; unit += wstride) {
    int b, t, h;
    decode_unit(unit, p.H, p.T_kv, b, t, h);
    const T* kb = reinterpret_cast<const T*>(p.kd.ptr) + p.kd.off(b, (int64_t)t * p.Ls, h);
    const T* vb = reinterpret_cast<const T*>(p.vd.ptr) + p.vd.off(b, (int64_t)t * p.Ls, h);
    for (int g = 0; g < p.G; ++g) {
      const int r = t * p.G + g;
      float qf[CH][8];
      {
        const T* qp = reinterpret_cast<const T*>(p.q.ptr) + p.q.off(b, r, h);
#pragma unroll
        for (int c = 0; c < CH; ++c) {
          unpack8<T>(*reinterpret_cast<const uint4*>(qp + (sub + 8 * c) * 8), qf[c]);
#pragma unroll
          for (int e = 0; e < 8; ++e) qf[c][e] *= p.scale_log2;
        }
      }
      float m = -INFINITY, lsum = 0.f;
      float acc[CH][8];
#pragma unroll
      for (int c = 0; c < CH; ++c)
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[c][e] = 0.f;

      for (int l0 = 0; l0 < p.L; l0 += 16) {
        uint4 raw[4][CH];
        uint4 vraw[4][1];                         // D = 64: the V rows travel with the K rows
        float s[4];
#pragma unroll
        for (int ps = 0; ps < 4; ++ps) {          // all K loads of the block in flight together
          const int key = l0 + ps * 4 + grp;
#pragma unroll
          for (int c = 0; c < CH; ++c)
            raw[ps][c] = (key < p.L) ? *reinterpret_cast<const uint4*>(kb + (int64_t)key * p.kd.st + (sub + 8 * c) * 8)
                                     : make_uint4(0, 0, 0, 0);
          if constexpr (CH == 1)
            vraw[ps][0] = (key < p.L) ? *reinterpret_cast<const uint4*>(vb + (int64_t)key * p.vd.st + sub * 8)
                                      : make_uint4(0, 0, 0, 0);
        }
        float bm = -INFINITY;
#pragma unroll
        for (int ps = 0; ps < 4; ++ps) {
          float d = 0.f;
#pragma unroll
          for (int c = 0; c < CH; ++c) {
            float kf[8];
            unpack8<T>(raw[ps][c], kf);
#pragma unroll
            for (int e = 0; e < 8; ++e) d = fmaf(qf[c][e], kf[e], d);
          }
          d = group8_sum(d);
          s[ps] = (l0 + ps * 4 + grp < p.L) ? d : -INFINITY;
          bm = fmaxf(bm, s[ps]);
        }
        bm = cross4_max(bm);
        const float m_new = fmaxf(m, bm);          // finite: key l0 of the block is always valid
        const float alpha = fast_exp2(m - m_new);
        m = m_new;
        lsum *= alpha;
#pragma unroll
        for (int c = 0; c < CH; ++c)
#pragma unroll
          for (int e = 0; e < 8; ++e) acc[c][e] *= alpha;
        if constexpr (CH == 1) {
#pragma unroll
          for (int ps = 0; ps < 4; ++ps) raw[ps][0] = vraw[ps][0];
        } else {
#pragma unroll
          for (int ps = 0; ps < 4; ++ps) {          // V loads of the block
            const int key = l0 + ps * 4 + grp;
#pragma unroll
            for (int c = 0; c < CH; ++c)
              raw[ps][c] = (key < p.L) ? *reinterpret_cast<const uint4*>(vb + (int64_t)key * p.vd.st + (sub + 8 * c) * 8)
                                       : make_uint4(0, 0, 0, 0);
          }
        }
#pragma unroll
        for (int ps = 0; ps < 4; ++ps) {
          const float pw = fast_exp2(s[ps] - m);  // 0 for invalid keys (s = -inf)
          lsum += pw;
#pragma unroll
          for (int c = 0; c < CH; ++c) {
            float vf[8];
            unpack8<T>(raw[ps][c], vf);
#pragma unroll
            for (int e = 0; e < 8; ++e) acc[c][e] = fmaf(pw, vf[e], acc[c][e]);
          }
        }
      }
      lsum = cross4_sum(lsum);
      const float inv = 1.f / lsum;
#pragma unroll
      for (int c = 0; c < CH; ++c)
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[c][e] = cross4_sum(acc[c][e]) * inv;
      if (grp == 0) {
        T* op = reinterpret_cast<T*>(p.o.ptr) + p.o.off(b, r, h);
#pragma unroll
        for (int c = 0; c < CH; ++c) *reinterpret_cast<uint4*>(op + (sub + 8 * c) * 8) = pack8<T>(acc[c]);
        if (sub == 0) p.lse[((int64_t)b * p.T_q + r) * p.H + h] = m + log2f(lsum);
      }
    }
  }
}

// ------------------------------------------------------------------------- backward
// One warp per (b, t, h), G query rows held in registers (G is a template parameter).
template <typename T, int D, int G>
__global__ void __launch_bounds__(128, (G == 1) ? (D == 64 ? 5 : 3) : 2) bwd_kernel(const __grid_constant__ Params p) {
  constexpr int CH = D / 64;
  const int lane = threadIdx.x & 31, sub = lane & 7, grp = lane >> 3;
  const int64_t n_units = (int64_t)p.B * p.T_kv * p.H;
  const int64_t wstride = (int64_t)gridDim.x * (blockDim.x >> 5);
  for (int64_t unit = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); unit < n_units; unit += wstride) {
    int b, t, h;
    decode_unit(unit, p.H, p.T_kv, b, t, h);
    const T* kb = reinterpret_cast<const T*>(p.kd.ptr) + p.kd.off(b, (int64_t)t * p.Ls, h);
    const T* vb = reinterpret_cast<const T*>(p.vd.ptr) + p.vd.off(b, (int64_t)t * p.Ls, h);
    T* dkb = reinterpret_cast<T*>(p.dkd.ptr) + p.dkd.off(b, (int64_t)t * p.Ls, h);
    T* dvb = reinterpret_cast<T*>(p.dvd.ptr) + p.dvd.off(b, (int64_t)t * p.Ls, h);

    uint4 qraw[G][CH], doraw[G][CH];
    float lse_g[G], delta_g[G];
    float dq[G][CH][8];
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const int r = t * G + g;
      const T* qp = reinterpret_cast<const T*>(p.q.ptr) + p.q.off(b, r, h);
      const T* dp_ = reinterpret_cast<const T*>(p.dout.ptr) + p.dout.off(b, r, h);
      const T* op = reinterpret_cast<const T*>(p.o.ptr) + p.o.off(b, r, h);
      float dl = 0.f;
#pragma unroll
      for (int c = 0; c < CH; ++c) {
        qraw[g][c] = *reinterpret_cast<const uint4*>(qp + (sub + 8 * c) * 8);
        doraw[g][c] = *reinterpret_cast<const uint4*>(dp_ + (sub + 8 * c) * 8);
        float of[8], df[8];
        unpack8<T>(*reinterpret_cast<const uint4*>(op + (sub + 8 * c) * 8), of);
        unpack8<T>(doraw[g][c], df);
#pragma unroll
        for (int e = 0; e < 8; ++e) { dl = fmaf(of[e], df[e], dl); dq[g][c][e] = 0.f; }
      }
      delta_g[g] = group8_sum(dl);
      lse_g[g] = p.lse[((int64_t)b * p.T_q + r) * p.H + h];
    }

    for (int l0 = 0; l0 < p.L; l0 += 16) {
      uint4 kraw[4][CH], vraw[4][CH];
#pragma unroll
      for (int ps = 0; ps < 4; ++ps) {
        const int key = l0 + ps * 4 + grp;
#pragma unroll
        for (int c = 0; c < CH; ++c) {
          const bool valid = key < p.L;
          kraw[ps][c] = valid ? *reinterpret_cast<const uint4*>(kb + (int64_t)key * p.kd.st + (sub + 8 * c) * 8) : make_uint4(0, 0, 0, 0);
          vraw[ps][c] = valid ? *reinterpret_cast<const uint4*>(vb + (int64_t)key * p.vd.st + (sub + 8 * c) * 8) : make_uint4(0, 0, 0, 0);
        }
      }
#pragma unroll
      for (int ps = 0; ps < 4; ++ps) {
        const int key = l0 + ps * 4 + grp;
        const bool valid = key < p.L;
        float kf[CH][8], vf[CH][8], dkr[CH][8], dvr[CH][8];
#pragma unroll
        for (int c = 0; c < CH; ++c) {
          unpack8<T>(kraw[ps][c], kf[c]);
          unpack8<T>(vraw[ps][c], vf[c]);
#pragma unroll
          for (int e = 0; e < 8; ++e) { dkr[c][e] = 0.f; dvr[c][e] = 0.f; }
        }
#pragma unroll
        for (int g = 0; g < G; ++g) {
          float s = 0.f, dpv = 0.f;
          float qf[CH][8], df[CH][8];
#pragma unroll
          for (int c = 0; c < CH; ++c) {
            unpack8<T>(qraw[g][c], qf[c]);
            unpack8<T>(doraw[g][c], df[c]);
#pragma unroll
            for (int e = 0; e < 8; ++e) { s = fmaf(qf[c][e], kf[c][e], s); dpv = fmaf(df[c][e], vf[c][e], dpv); }
          }
          s = group8_sum(s);
          dpv = group8_sum(dpv);
          const float pw = valid ? fast_exp2(fmaf(s, p.scale_log2, -lse_g[g])) : 0.f;
          const float ds = pw * (dpv - delta_g[g]);
#pragma unroll
          for (int c = 0; c < CH; ++c)
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              dq[g][c][e] = fmaf(ds, kf[c][e], dq[g][c][e]);
              dkr[c][e] = fmaf(ds, qf[c][e], dkr[c][e]);
              dvr[c][e] = fmaf(pw, df[c][e], dvr[c][e]);
            }
        }
        if (valid) {
#pragma unroll
          for (int c = 0; c < CH; ++c) {
#pragma unroll
            for (int e = 0; e < 8; ++e) dkr[c][e] *= p.scale;
            uint4* gk4 = reinterpret_cast<uint4*>(dkb + (int64_t)key * p.dkd.st + (sub + 8 * c) * 8);
            uint4* gv4 = reinterpret_cast<uint4*>(dvb + (int64_t)key * p.dvd.st + (sub + 8 * c) * 8);
            if (p.acc_depth) {   // gradient cache shared by several layers: add to what earlier calls left
              add8<T>(dkr[c], *gk4);
              add8<T>(dvr[c], *gv4);
            }
            *gk4 = pack8<T>(dkr[c]);
            *gv4 = pack8<T>(dvr[c]);
          }
        }
      }
    }
#pragma unroll
    for (int g = 0; g < G; ++g) {
#pragma unroll
      for (int c = 0; c < CH; ++c)
#pragma unroll
        for (int e = 0; e < 8; ++e) dq[g][c][e] = cross4_sum(dq[g][c][e]) * p.scale;
      if (grp == 0) {
        T* qp = reinterpret_cast<T*>(p.dq.ptr) + p.dq.off(b, t * G + g, h);
#pragma unroll
        for (int c = 0; c < CH; ++c) *reinterpret_cast<uint4*>(qp + (sub + 8 * c) * 8) = pack8<T>(dq[g][c]);
      }
    }
  }
}

// G query rows of a position are held in registers: up to 2 at D = 128, up to 4 at D = 64.
inline bool bwd_supported(int G, int D) { return G == 1 || G == 2 || (G == 4 && D == 64); }

}  // namespace fda
}  // namespace moda
