// Host side of the tcgen05 backward: workspace layout, tensor maps and the launch sequences.
//
// Two sequences exist.  The default TWO-KERNEL one is the reference's structure: a query-parallel
// dq kernel and a key-parallel dk/dv kernel that both recompute the scores (seven executed matmuls).
// The FUSED one (D = 128, selected with MODA_PATH_TCGEN05_FUSED_BWD) runs
//     bounds (kvmax, pre, scale)  ->  bwd_fused_kernel over the sequence key tiles (dK, dV and the
//     sequence keys' share of dQ in a fixed-point accumulator)  ->  dq_kernel over the depth keys only,
//     which adds the two shares and writes dq  ->  depth gradients
// and executes the five matmuls of the backward once each; measured, it is no faster (see
// tc_bwd_fused_kernel.cuh), which is why it is not the default.
#pragma once
#include "tc_bwd_fused_kernel.cuh"

namespace moda {
namespace tc {

inline int padded_rows(int T_q) { return (T_q + 63) / 64 * 64 + 64; }

inline bool bwd_supported(const moda_problem* pr) {
  return (pr->D == 128 || pr->D == 64) && pr->mode != MODA_DEPTH_ONLY && pr->scale > 0.f && depth_layout_supported(pr);
}
inline bool bwd_is_fused(const moda_problem* pr) {
  return bwd_supported(pr) && pr->D == 128 && pr->path == MODA_PATH_TCGEN05_FUSED_BWD;
}

inline size_t align256(size_t n) { return (n + 255) & ~(size_t)255; }

// Workspace after the per-row delta of the generic path: delta_t, lse_t [B, H, T_qp] fp32 and, for
// the fused sequence, norm_t [B, H, T_qp] fp32, scale_blk [B, H, T_qp / 64] float4, kvmax [B, H, 2]
// and the dQ accumulator [B, H, T_qp, 128] int32.
struct BwdWorkspace {
  size_t stat = 0, scale = 0, kvmax = 0, acc = 0, total = 0;
  explicit BwdWorkspace(const moda_problem* pr) {
    if (!bwd_supported(pr)) return;
    const size_t rows = (size_t)pr->B * pr->H * padded_rows(pr->T_kv * pr->G);
    stat = align256(rows * sizeof(float));
    total = 2 * stat;
    if (bwd_is_fused(pr)) {
      scale = align256(rows / 64 * sizeof(float4));
      kvmax = align256((size_t)pr->B * pr->H * 2 * sizeof(int));
      acc = align256(rows * 128 * sizeof(int));
      total += stat + scale + kvmax + acc;
    }
  }
};
inline size_t bwd_extra_workspace_bytes(const moda_problem* pr) { return BwdWorkspace(pr).total; }

struct BwdMaps { DqMaps dq; DkvMaps dkv; DgOutMaps out; };
struct BwdBuffers { float *delta_t, *lse_t, *norm_t; float4* scale_blk; int* kvmax; int* dq_acc; size_t acc_bytes, kvmax_bytes; };

template <typename T, int D>
inline cudaError_t launch_bwd(const Params& p, const BwdMaps& m, const BwdBuffers& w, int T_qp, bool dg, bool fused,
                              int n_sm, cudaStream_t st, int* launches) {
  cudaError_t e;
  float* delta_t = w.delta_t;
  float* lse_t = w.lse_t;
  const int n_seq = (p.T_kv + kBN - 1) / kBN;
  const int n_dep_tiles = (int)(((int64_t)p.T_kv * p.L + kBN - 1) / kBN);
  if (fused) {
    if constexpr (D == 128) {
      if ((e = cudaMemsetAsync(w.kvmax, 0, w.kvmax_bytes, st)) != cudaSuccess) return e;
      const int64_t groups = (int64_t)p.B * p.H * ((p.T_kv + 31) / 32);
      const int64_t cap = (int64_t)n_sm * 16;
      prof::Scope ps(prof::kBwdBoundsTc, st);
      kvmax_kernel<T><<<(int)(groups < cap ? groups : cap), 256, 0, st>>>(p, w.kvmax);
      if ((e = cudaGetLastError()) != cudaSuccess) return e;
      *launches += 1;
    }
  }
  {
    const int64_t groups = (int64_t)p.B * p.H * (T_qp / 32);
    const int64_t cap = (int64_t)n_sm * 16;
    const int blocks = (int)(groups < cap ? groups : cap);
    prof::Scope ps(prof::kPreTc, st);
    pre_kernel<T, D><<<blocks, 256, 0, st>>>(p, delta_t, lse_t, fused ? w.norm_t : nullptr, T_qp);
  }
  if ((e = cudaGetLastError()) != cudaSuccess) return e;
  *launches += 1;
  const size_t dq_smem = dq_ring<D>() * 2 * (size_t)step_tile<D>() + 2 * (size_t)kScoreTile + kCtlBytes;
  const size_t dkv_smem = dkv_ring<D>() * (2 * (size_t)step_tile<D>() + 512) + 2 * (size_t)kDkvPairBytes + kCtlBytes;
  if (fused) {
    if constexpr (D == 128) {
      {
        const int64_t n_blk = (int64_t)p.B * p.H * (T_qp / 64);
        const int64_t want = (n_blk + 7) / 8, cap = (int64_t)n_sm * 8;
        prof::Scope ps(prof::kBwdBoundsTc, st);
        scale_kernel<<<(int)(want < cap ? want : cap), 256, 0, st>>>(delta_t, w.norm_t, w.kvmax, w.scale_blk, T_qp, n_blk);
      }
      if ((e = cudaGetLastError()) != cudaSuccess) return e;
      *launches += 1;
      if ((e = cudaMemsetAsync(w.dq_acc, 0, w.acc_bytes, st)) != cudaSuccess) return e;
      {
        auto kern = bwd_fused_kernel<T>;
        if ((e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kFuSmem)) != cudaSuccess) return e;
        dim3 grid(n_seq, p.H, p.B);
        prof::Scope ps(prof::kBwdFusedTc, st);
        kern<<<grid, kFusedBwdThreads, kFuSmem, st>>>(p, m.dkv, delta_t, lse_t, w.scale_blk, w.dq_acc, T_qp);
      }
      if ((e = cudaGetLastError()) != cudaSuccess) return e;
      *launches += 1;
      {   // depth keys' share of dQ, added to the accumulated sequence share; writes dq
        auto kern = dq_kernel<T, D>;
        if ((e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dq_smem)) != cudaSuccess) return e;
        dim3 grid((p.T_q + kBM - 1) / kBM, p.H, p.B);
        prof::Scope ps(prof::kDqTc, st);
        kern<<<grid, kDqThreads, dq_smem, st>>>(p, m.dq, delta_t, lse_t, T_qp, w.dq_acc, w.scale_blk);
      }
      if ((e = cudaGetLastError()) != cudaSuccess) return e;
      *launches += 1;
      if (!dg && n_dep_tiles > 0) {   // depth key tiles the query-stationary kernel cannot own: key-parallel kernel on them alone
        auto kern = dkv_kernel<T, D>;
        if ((e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dkv_smem)) != cudaSuccess) return e;
        dim3 grid(n_dep_tiles, p.H, p.B);
        prof::Scope ps(prof::kDkvTc, st);
        kern<<<grid, kDkvThreads, dkv_smem, st>>>(p, m.dkv, delta_t, lse_t, T_qp, 0);
        if ((e = cudaGetLastError()) != cudaSuccess) return e;
        *launches += 1;
      }
    }
  } else {
    {
      auto kern = dq_kernel<T, D>;
      if ((e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dq_smem)) != cudaSuccess) return e;
      dim3 grid((p.T_q + kBM - 1) / kBM, p.H, p.B);
      prof::Scope ps(prof::kDqTc, st);
      kern<<<grid, kDqThreads, dq_smem, st>>>(p, m.dq, delta_t, lse_t, T_qp, nullptr, nullptr);
    }
    if ((e = cudaGetLastError()) != cudaSuccess) return e;
    *launches += 1;
    {
      auto kern = dkv_kernel<T, D>;
      if ((e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dkv_smem)) != cudaSuccess) return e;
      dim3 grid(n_seq + (dg ? 0 : n_dep_tiles), p.H, p.B);
      prof::Scope ps(prof::kDkvTc, st);
      kern<<<grid, kDkvThreads, dkv_smem, st>>>(p, m.dkv, delta_t, lse_t, T_qp, n_seq);
    }
    if ((e = cudaGetLastError()) != cudaSuccess) return e;
    *launches += 1;
  }
  if (dg) {
    auto kern = depth_grad_kernel<T, D>;
    constexpr uint32_t smem = dg_smem<D>();
    if ((e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)) != cudaSuccess) return e;
    const int64_t n_blocks = (int64_t)((p.T_q + kStep - 1) / kStep) * p.H * p.B;
    dim3 grid((unsigned)(n_blocks < n_sm ? n_blocks : n_sm));
    {
      prof::Scope ps(prof::kDepthGradTc, st);
      kern<<<grid, kDgThreads, smem, st>>>(p, m.dkv, m.out, delta_t, lse_t, T_qp);
    }
    if ((e = cudaGetLastError()) != cudaSuccess) return e;
    *launches += 1;
  }
  return cudaSuccess;
}

inline int bwd(const Params& p, const moda_problem* pr, void* extra, int n_sm, cudaStream_t st, int* launches, int* cuda_err) {
  const int T_qp = padded_rows(p.T_q);
  const BwdWorkspace ws(pr);
  const bool fused = bwd_is_fused(pr);
  unsigned char* base = reinterpret_cast<unsigned char*>(extra);
  BwdBuffers w{};
  w.delta_t = reinterpret_cast<float*>(base);
  w.lse_t = reinterpret_cast<float*>(base + ws.stat);
  if (fused) {
    w.norm_t = reinterpret_cast<float*>(base + 2 * ws.stat);
    w.scale_blk = reinterpret_cast<float4*>(base + 3 * ws.stat);
    w.kvmax = reinterpret_cast<int*>(base + 3 * ws.stat + ws.scale);
    w.dq_acc = reinterpret_cast<int*>(base + 3 * ws.stat + ws.scale + ws.kvmax);
    w.acc_bytes = ws.acc;
    w.kvmax_bytes = ws.kvmax;
  }
  const bool dep = p.L > 0;
  const int D = pr->D, dt = pr->dtype;

  BwdMaps m;
  memset(&m, 0, sizeof(m));
  bool ok = make_map_rows(&m.dq.k, p.k, dt, p.B, p.T_kv, p.H, D, 64) &&
            make_map_rows(&m.dq.v, p.v, dt, p.B, p.T_kv, p.H, D, 64) &&
            make_map_rows(&m.dkv.k, p.k, dt, p.B, p.T_kv, p.H, D, 128) &&
            make_map_rows(&m.dkv.v, p.v, dt, p.B, p.T_kv, p.H, D, 128) &&
            make_map_rows(&m.dkv.q, p.q, dt, p.B, p.T_q, p.H, D, 64) &&
            make_map_rows(&m.dkv.dout, p.dout, dt, p.B, p.T_q, p.H, D, 64);
  if (ok && dep) {
    ok = make_map_depth(&m.dq.kd, p.kd, dt, p, D, 64) && make_map_depth(&m.dq.vd, p.vd, dt, p, D, 64) &&
         make_map_depth(&m.dkv.kd, p.kd, dt, p, D, 128) && make_map_depth(&m.dkv.vd, p.vd, dt, p, D, 128);
  } else if (ok) {
    m.dq.kd = m.dq.k; m.dq.vd = m.dq.v; m.dkv.kd = m.dkv.k; m.dkv.vd = m.dkv.v;
  }
  if (!ok) return MODA_ERR_UNSUPPORTED;
  const bool dg = depth_grad_applies(p, pr);
  if (dg && !(make_map_depth(&m.out.dkd, p.dkd, dt, p, D, 32) && make_map_depth(&m.out.dvd, p.dvd, dt, p, D, 32)))
    return MODA_ERR_UNSUPPORTED;
  if ((int64_t)((p.T_q + kStep - 1) / kStep) * p.H * p.B > 0x7fffffff || n_sm <= 0) return MODA_ERR_UNSUPPORTED;

  cudaError_t e = clear_launch_status(st);
  if (e == cudaSuccess) {
    const bool bf = dt == MODA_BF16;
    if (D == 128) e = bf ? launch_bwd<__nv_bfloat16, 128>(p, m, w, T_qp, dg, fused, n_sm, st, launches)
                         : launch_bwd<__half, 128>(p, m, w, T_qp, dg, fused, n_sm, st, launches);
    else e = bf ? launch_bwd<__nv_bfloat16, 64>(p, m, w, T_qp, dg, false, n_sm, st, launches)
                : launch_bwd<__half, 64>(p, m, w, T_qp, dg, false, n_sm, st, launches);
  }
  if (e != cudaSuccess) { *cuda_err = (int)e; return MODA_ERR_CUDA; }
  return MODA_OK;
}

}  // namespace tc
}  // namespace moda
