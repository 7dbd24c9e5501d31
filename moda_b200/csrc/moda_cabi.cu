// C ABI of libmoda_b200.so: argument validation, parameter-block set-up and kernel
// dispatch.  Declarations and the reference functions each entry point replaces are
// in include/moda_b200.h.  No torch headers; pure CUDA runtime.
#include "../../include/moda_b200.h"

#include <cuda_runtime.h>

#include "common.cuh"
#include "profiler.cuh"
#include "simt_mma_kernels.cuh"
#include "fda_kernels.cuh"
#include "depth_cache_kernels.cuh"
#ifndef MODA_NO_TCGEN05
#include "tc_kernels.cuh"
#include "tc_bwd_kernels.cuh"
#include "tc_fwd3_kernel.cuh"
#include "tc_bwd_launch.cuh"
#include "mma_rate_probe.cuh"
#endif

namespace {

using namespace moda;

thread_local int g_last_launches = 0;
thread_local int g_last_cuda_error = 0;

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// A tensor of extents [B, T, H, D].  A dimension of extent 1 may carry any stride (its index is
// always 0); every other stride must be a positive multiple of 8 elements.  Zero or negative
// strides (expanded / flipped views) are refused: the TMA tensor maps cannot express them and a
// gradient written through one would alias.
int check_tensor(const moda_tensor4* t, bool required, int64_t B, int64_t T, int64_t H) {
  if (t == nullptr || t->data == nullptr) return required ? MODA_ERR_NULL : MODA_OK;
  if (!aligned16(t->data)) return MODA_ERR_ALIGNMENT;
  const int64_t ext[3] = {B, T, H}, str[3] = {t->stride_b, t->stride_t, t->stride_h};
  for (int i = 0; i < 3; ++i)
    if (ext[i] > 1 && (str[i] <= 0 || (str[i] % 8) != 0)) return MODA_ERR_ALIGNMENT;
  return MODA_OK;
}

// Multiprocessor count of a device (queried once per device).
int sm_count(int device) {
  static std::mutex mu;
  static int cached[64] = {0};
  std::lock_guard<std::mutex> lk(mu);
  if (device >= 0 && device < 64 && cached[device] > 0) return cached[device];
  int n = 0;
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || n <= 0) return 0;
  if (device >= 0 && device < 64) cached[device] = n;
  return n;
}

View to_view(const moda_tensor4* t) {
  View v{nullptr, 0, 0, 0};
  if (t != nullptr) { v.ptr = t->data; v.sb = t->stride_b; v.st = t->stride_t; v.sh = t->stride_h; }
  return v;
}

int check_problem(const moda_problem* pr) {
  if (pr == nullptr) return MODA_ERR_NULL;
  if (pr->B < 1 || pr->T_kv < 1 || pr->H < 1 || pr->G < 1 || pr->L < 0) return MODA_ERR_SHAPE;
  if (pr->B > 65535 || pr->H > 65535) return MODA_ERR_SHAPE;
  if ((int64_t)pr->T_kv * pr->G > (int64_t)1 << 30) return MODA_ERR_SHAPE;
  if ((int64_t)pr->T_kv * pr->L > (int64_t)1 << 30) return MODA_ERR_SHAPE;
  if (pr->D != 64 && pr->D != 128) return MODA_ERR_HEAD_DIM;
  if (pr->dtype != MODA_BF16 && pr->dtype != MODA_FP16) return MODA_ERR_DTYPE;
  if (pr->mode < MODA_CAUSAL || pr->mode > MODA_DEPTH_ONLY) return MODA_ERR_MODE;
  if (pr->mode == MODA_DEPTH_ONLY && pr->L < 1) return MODA_ERR_MODE;
  if (pr->mode == MODA_CHUNK_VISIBLE) {
    if (pr->chunk_rows < 1 || pr->chunk_rows % pr->G != 0) return MODA_ERR_CHUNK;
  }
  if (pr->path < MODA_PATH_AUTO || pr->path > MODA_PATH_TCGEN05_FUSED_BWD) return MODA_ERR_MODE;
  if (!(pr->scale == pr->scale)) return MODA_ERR_SHAPE;  // NaN scale
  if (pr->depth_rows_per_pos < 0 || (pr->depth_rows_per_pos > 0 && pr->depth_rows_per_pos < pr->L)) return MODA_ERR_SHAPE;
  if ((int64_t)pr->T_kv * pr->depth_rows_per_pos > (int64_t)1 << 30) return MODA_ERR_SHAPE;
  return MODA_OK;
}

void fill_common(Params& p, const moda_problem* pr) {
  p.B = pr->B; p.H = pr->H; p.T_kv = pr->T_kv; p.T_q = pr->T_kv * pr->G; p.G = pr->G; p.L = pr->L;
  p.mode = pr->mode;
  p.Cb = (pr->mode == MODA_CHUNK_VISIBLE) ? pr->chunk_rows / pr->G : 1;
  p.scale = pr->scale;
  p.scale_log2 = pr->scale * 1.4426950216f;
  p.Ls = (pr->depth_rows_per_pos > pr->L) ? pr->depth_rows_per_pos : pr->L;
  p.acc_depth = pr->accumulate_depth_grads != 0;
}

int cuda_fail(cudaError_t e) { g_last_cuda_error = (int)e; return MODA_ERR_CUDA; }

#define MODA_CUDA(x) do { cudaError_t e__ = (x); if (e__ != cudaSuccess) return cuda_fail(e__); } while (0)

template <typename K> int opt_in_smem(K kernel, size_t bytes) {
  MODA_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
  return MODA_OK;
}

// ----------------------------------------------------------------- mma.sync path
template <typename T, int D>
int simt_fwd(const Params& p, cudaStream_t st) {
  auto kern = simt::fwd_kernel<T, D>;
  constexpr size_t smem = simt::fwd_smem<T, D>();
  if (int rc = opt_in_smem(kern, smem)) return rc;
  dim3 grid((p.T_q + 63) / 64, p.H, p.B);
  {
    prof::Scope ps(prof::kFwdSimt, st);
    kern<<<grid, 128, smem, st>>>(p);
  }
  MODA_CUDA(cudaGetLastError());
  g_last_launches += 1;
  return MODA_OK;
}

template <typename T, int D>
int simt_delta(const Params& p, int n_sm, cudaStream_t st) {
  const int64_t rows = (int64_t)p.B * p.T_q * p.H;
  const int64_t want = (rows + 7) / 8, cap = (int64_t)n_sm * 16;
  const int blocks = (int)(want < cap ? want : cap);
  {
    prof::Scope ps(prof::kDelta, st);
    simt::delta_kernel<T, D><<<blocks, 256, 0, st>>>(p);
  }
  MODA_CUDA(cudaGetLastError());
  g_last_launches += 1;
  return MODA_OK;
}

template <typename T, int D>
int simt_bwd(const Params& p, int n_sm, cudaStream_t st) {
  if (int rc = simt_delta<T, D>(p, n_sm, st)) return rc;
  {
    auto kern = simt::dq_kernel<T, D>;
    constexpr size_t smem = simt::dq_smem<T, D>();
    if (int rc = opt_in_smem(kern, smem)) return rc;
    dim3 grid((p.T_q + 63) / 64, p.H, p.B);
    {
      prof::Scope ps(prof::kDqSimt, st);
      kern<<<grid, 128, smem, st>>>(p);
    }
    MODA_CUDA(cudaGetLastError());
    g_last_launches += 1;
  }
  {
    auto kern = simt::dkv_kernel<T, D>;
    constexpr size_t smem = simt::dkv_smem<T, D>();
    if (int rc = opt_in_smem(kern, smem)) return rc;
    const int n_seq = (p.mode == kDepthOnly) ? 0 : (p.T_kv + 63) / 64;
    const int n_dep = (int)(((int64_t)p.T_kv * p.L + 63) / 64);
    if (n_seq + n_dep > 0) {
      dim3 grid(n_seq + n_dep, p.H, p.B);
      prof::Scope ps(prof::kDkvSimt, st);
      kern<<<grid, 128, smem, st>>>(p, n_seq);
      MODA_CUDA(cudaGetLastError());
      g_last_launches += 1;
    }
  }
  return MODA_OK;
}

template <typename T>
int simt_fwd_d(const Params& p, int D, cudaStream_t st) {
  return D == 64 ? simt_fwd<T, 64>(p, st) : simt_fwd<T, 128>(p, st);
}
template <typename T>
int simt_bwd_d(const Params& p, int D, int n_sm, cudaStream_t st) {
  return D == 64 ? simt_bwd<T, 64>(p, n_sm, st) : simt_bwd<T, 128>(p, n_sm, st);
}

// ----------------------------------------------------------------- depth-only (FDA) bandwidth path
bool use_fda(const moda_problem* pr, bool is_bwd) {
  if (pr->mode != MODA_DEPTH_ONLY || pr->path != MODA_PATH_AUTO) return false;
  return !is_bwd || fda::bwd_supported(pr->G, pr->D);
}

// Own-position depth (parallel_moda, causal or not) with one query row per position (G = 1) as
// two launches: a query's depth keys are the L rows of its own position, so that part of the
// softmax is the depth-only operator and runs at HBM rate in the bandwidth kernels; the attention
// kernels then run on the sequence keys alone and fold their part into the stored partial in the
// epilogue (Params::merge_depth).  Inside the attention kernels a 128-row query tile at G = 1
// spans 128 positions and has to multiply against 128 L depth columns of which each row uses L
// (L extra key tiles per query tile; at T = 197, L = 11 that is 11 tiles beside 2 sequence
// tiles).  With G = 4 the tile spans 32 positions, the extra tiles are a small share of the
// sequence tiles, and one launch is faster.
bool split_depth(const moda_problem* pr, bool is_bwd) {
  if (pr->path != MODA_PATH_AUTO || pr->L <= 0 || pr->G != 1) return false;
  if (pr->mode != MODA_CAUSAL && pr->mode != MODA_NONCAUSAL) return false;
  return !is_bwd || fda::bwd_supported(pr->G, pr->D);
}
Params sequence_part(const Params& p) {
  Params s = p;
  s.L = 0;
  s.kd = View{}; s.vd = View{}; s.dkd = View{}; s.dvd = View{};
  s.merge_depth = 1;
  return s;
}

template <typename T, int D>
int fda_fwd(const Params& p, int n_sm, cudaStream_t st) {
  const int64_t units = (int64_t)p.B * p.T_kv * p.H;
  const int64_t want = (units + 7) / 8, cap = (int64_t)n_sm * 32;
  const int blocks = (int)(want < cap ? want : cap);
  {
    prof::Scope ps(prof::kFdaFwd, st);
    fda::fwd_kernel<T, D><<<blocks, 256, 0, st>>>(p);
  }
  MODA_CUDA(cudaGetLastError());
  g_last_launches += 1;
  return MODA_OK;
}

template <typename T, int D>
int fda_bwd(const Params& p, int n_sm, cudaStream_t st) {
  const int64_t units = (int64_t)p.B * p.T_kv * p.H;
  const int64_t want = (units + 3) / 4, cap = (int64_t)n_sm * 64;
  const int blocks = (int)(want < cap ? want : cap);
  {
    prof::Scope ps(prof::kFdaBwd, st);
    if (p.G == 1) fda::bwd_kernel<T, D, 1><<<blocks, 128, 0, st>>>(p);
    else if (p.G == 2) fda::bwd_kernel<T, D, 2><<<blocks, 128, 0, st>>>(p);
    else if constexpr (D == 64) fda::bwd_kernel<T, D, 4><<<blocks, 128, 0, st>>>(p);
  }
  MODA_CUDA(cudaGetLastError());
  g_last_launches += 1;
  return MODA_OK;
}

template <typename T>
int fda_dispatch(const Params& p, int D, bool is_bwd, int n_sm, cudaStream_t st) {
  if (is_bwd) return D == 64 ? fda_bwd<T, 64>(p, n_sm, st) : fda_bwd<T, 128>(p, n_sm, st);
  return D == 64 ? fda_fwd<T, 64>(p, n_sm, st) : fda_fwd<T, 128>(p, n_sm, st);
}

int resolve_path(const moda_problem* pr, bool is_bwd) {
#ifndef MODA_NO_TCGEN05
  const bool ok = is_bwd ? tc::bwd_supported(pr) : tc::fwd_supported(pr);
#else
  const bool ok = false;
#endif
  if (pr->path == MODA_PATH_SIMT_MMA) return MODA_PATH_SIMT_MMA;
  if (pr->path >= MODA_PATH_TCGEN05) return ok ? MODA_PATH_TCGEN05 : -MODA_ERR_UNSUPPORTED;
  return ok ? MODA_PATH_TCGEN05 : MODA_PATH_SIMT_MMA;
}

#ifndef MODA_NO_TCGEN05
int tc_forward(const Params& p, const moda_problem* prob, int n_sm, cudaStream_t st) {
  // Two forwards.  tc::fwd3 (two 128-row query tiles per CTA, one CTA per SM, one MMA warp
  // ordering the work of both tiles) is the faster one once its grid fills the GPU; tc::fwd
  // (one query tile per CTA, two CTAs per SM) has twice as many, smaller CTAs and serves the
  // small problems.  Both use the same softmax arithmetic, so a result does not depend on the
  // choice.  MODA_PATH_TCGEN05_ONE_TILE / _TWO_TILES force one of them.
  bool two_tiles = prob->path == MODA_PATH_TCGEN05_TWO_TILES;
  if (prob->path != MODA_PATH_TCGEN05_ONE_TILE && prob->path != MODA_PATH_TCGEN05_TWO_TILES) {
    const int64_t n_cta = (int64_t)((p.T_q + 255) / 256) * p.H * p.B;
    two_tiles = n_sm > 0 && n_cta >= n_sm;
  }
  if (two_tiles) return tc::fwd3(p, prob, st, &g_last_launches, &g_last_cuda_error);
  return tc::fwd(p, prob, st, &g_last_launches, &g_last_cuda_error);
}
#endif

size_t delta_bytes(const moda_problem* pr) {
  const size_t n = (size_t)pr->B * pr->T_kv * pr->G * pr->H * sizeof(float);
  return (n + 255) & ~(size_t)255;
}

struct DeviceGuard {
  int prev = -1; bool ok = true; cudaError_t err = cudaSuccess;
  explicit DeviceGuard(int dev) {
    err = cudaGetDevice(&prev);
    if (err == cudaSuccess && prev != dev) err = cudaSetDevice(dev);
    ok = (err == cudaSuccess);
  }
  ~DeviceGuard() { int cur = -1; if (cudaGetDevice(&cur) == cudaSuccess && cur != prev && prev >= 0) cudaSetDevice(prev); }
};

}  // namespace

extern "C" {

int moda_b200_check_problem(const moda_problem* prob) { return check_problem(prob); }

int moda_b200_resolve_path(const moda_problem* prob, int is_bwd) {
  if (int rc = check_problem(prob)) return -rc;
  return resolve_path(prob, is_bwd != 0);
}

int moda_b200_fwd(const moda_problem* prob, const moda_tensor4* q, const moda_tensor4* k,
                  const moda_tensor4* v, const moda_tensor4* depth_k, const moda_tensor4* depth_v,
                  const moda_tensor4* o, float* lse, void* stream) {
  if (int rc = check_problem(prob)) return rc;
  const bool need_seq = prob->mode != MODA_DEPTH_ONLY;
  const bool need_dep = prob->L > 0;
  const int64_t Tq = (int64_t)prob->T_kv * prob->G, Tk = prob->T_kv;
  const int64_t Td = (int64_t)prob->T_kv * (prob->depth_rows_per_pos > prob->L ? prob->depth_rows_per_pos : prob->L);
  if (int rc = check_tensor(q, true, prob->B, Tq, prob->H)) return rc;
  if (int rc = check_tensor(k, need_seq, prob->B, Tk, prob->H)) return rc;
  if (int rc = check_tensor(v, need_seq, prob->B, Tk, prob->H)) return rc;
  if (int rc = check_tensor(depth_k, need_dep, prob->B, Td, prob->H)) return rc;
  if (int rc = check_tensor(depth_v, need_dep, prob->B, Td, prob->H)) return rc;
  if (int rc = check_tensor(o, true, prob->B, Tq, prob->H)) return rc;
  if (lse == nullptr) return MODA_ERR_NULL;
  const int path = resolve_path(prob, false);
  if (path < 0) return -path;

  Params p{};
  fill_common(p, prob);
  p.q = to_view(q); p.k = to_view(need_seq ? k : nullptr); p.v = to_view(need_seq ? v : nullptr);
  p.kd = to_view(need_dep ? depth_k : nullptr); p.vd = to_view(need_dep ? depth_v : nullptr);
  p.o = to_view(o); p.lse = lse;

  DeviceGuard guard(prob->device);
  if (!guard.ok) return cuda_fail(guard.err);
  g_last_launches = 0;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int n_sm = sm_count(prob->device);
  if (n_sm <= 0) return cuda_fail(cudaErrorInvalidDevice);
  if (use_fda(prob, false))
    return prob->dtype == MODA_BF16 ? fda_dispatch<__nv_bfloat16>(p, prob->D, false, n_sm, st)
                                    : fda_dispatch<__half>(p, prob->D, false, n_sm, st);
  if (split_depth(prob, false)) {
    if (int rc = prob->dtype == MODA_BF16 ? fda_dispatch<__nv_bfloat16>(p, prob->D, false, n_sm, st)
                                          : fda_dispatch<__half>(p, prob->D, false, n_sm, st)) return rc;
    p = sequence_part(p);
  }
#ifndef MODA_NO_TCGEN05
  if (path == MODA_PATH_TCGEN05) return tc_forward(p, prob, n_sm, st);
#endif
  return prob->dtype == MODA_BF16 ? simt_fwd_d<__nv_bfloat16>(p, prob->D, st)
                                  : simt_fwd_d<__half>(p, prob->D, st);
}

int moda_b200_bwd_workspace_bytes(const moda_problem* prob, size_t* bytes) {
  if (bytes == nullptr) return MODA_ERR_NULL;
  if (int rc = check_problem(prob)) return rc;
  size_t n = delta_bytes(prob);
#ifndef MODA_NO_TCGEN05
  n += tc::bwd_extra_workspace_bytes(prob);
#endif
  *bytes = n;
  return MODA_OK;
}

int moda_b200_bwd(const moda_problem* prob, const moda_tensor4* q, const moda_tensor4* k,
                  const moda_tensor4* v, const moda_tensor4* depth_k, const moda_tensor4* depth_v,
                  const moda_tensor4* o, const float* lse, const moda_tensor4* dout,
                  const moda_tensor4* dq, const moda_tensor4* dk, const moda_tensor4* dv,
                  const moda_tensor4* d_depth_k, const moda_tensor4* d_depth_v, void* workspace,
                  size_t workspace_bytes, void* stream) {
  if (int rc = check_problem(prob)) return rc;
  const bool need_seq = prob->mode != MODA_DEPTH_ONLY;
  const bool need_dep = prob->L > 0;
  const int64_t Tq = (int64_t)prob->T_kv * prob->G, Tk = prob->T_kv;
  const int64_t Td = (int64_t)prob->T_kv * (prob->depth_rows_per_pos > prob->L ? prob->depth_rows_per_pos : prob->L);
  const int Bn = prob->B, Hn = prob->H;
  if (int rc = check_tensor(q, true, Bn, Tq, Hn)) return rc;
  if (int rc = check_tensor(k, need_seq, Bn, Tk, Hn)) return rc;
  if (int rc = check_tensor(v, need_seq, Bn, Tk, Hn)) return rc;
  if (int rc = check_tensor(depth_k, need_dep, Bn, Td, Hn)) return rc;
  if (int rc = check_tensor(depth_v, need_dep, Bn, Td, Hn)) return rc;
  if (int rc = check_tensor(o, true, Bn, Tq, Hn)) return rc;
  if (int rc = check_tensor(dout, true, Bn, Tq, Hn)) return rc;
  if (int rc = check_tensor(dq, true, Bn, Tq, Hn)) return rc;
  if (int rc = check_tensor(dk, need_seq, Bn, Tk, Hn)) return rc;
  if (int rc = check_tensor(dv, need_seq, Bn, Tk, Hn)) return rc;
  if (int rc = check_tensor(d_depth_k, need_dep, Bn, Td, Hn)) return rc;
  if (int rc = check_tensor(d_depth_v, need_dep, Bn, Td, Hn)) return rc;
  if (lse == nullptr) return MODA_ERR_NULL;
  size_t need = 0;
  if (int rc = moda_b200_bwd_workspace_bytes(prob, &need)) return rc;
  if (workspace == nullptr || workspace_bytes < need) return MODA_ERR_WORKSPACE;
  if (reinterpret_cast<uintptr_t>(workspace) & 255u) return MODA_ERR_ALIGNMENT;
  const int path = resolve_path(prob, true);
  if (path < 0) return -path;

  Params p{};
  fill_common(p, prob);
  p.q = to_view(q); p.k = to_view(need_seq ? k : nullptr); p.v = to_view(need_seq ? v : nullptr);
  p.kd = to_view(need_dep ? depth_k : nullptr); p.vd = to_view(need_dep ? depth_v : nullptr);
  p.o = to_view(o); p.lse = const_cast<float*>(lse);
  p.dout = to_view(dout); p.dq = to_view(dq);
  p.dk = to_view(need_seq ? dk : nullptr); p.dv = to_view(need_seq ? dv : nullptr);
  p.dkd = to_view(need_dep ? d_depth_k : nullptr); p.dvd = to_view(need_dep ? d_depth_v : nullptr);
  p.delta = reinterpret_cast<float*>(workspace);

  DeviceGuard guard(prob->device);
  if (!guard.ok) return cuda_fail(guard.err);
  g_last_launches = 0;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int n_sm = sm_count(prob->device);
  if (n_sm <= 0) return cuda_fail(cudaErrorInvalidDevice);
  if (use_fda(prob, true))
    return prob->dtype == MODA_BF16 ? fda_dispatch<__nv_bfloat16>(p, prob->D, true, n_sm, st)
                                    : fda_dispatch<__half>(p, prob->D, true, n_sm, st);
  if (split_depth(prob, true)) {   // depth rows' dq share, d_depth_k, d_depth_v; then the sequence part
    if (int rc = prob->dtype == MODA_BF16 ? fda_dispatch<__nv_bfloat16>(p, prob->D, true, n_sm, st)
                                          : fda_dispatch<__half>(p, prob->D, true, n_sm, st)) return rc;
    p = sequence_part(p);
  }
#ifndef MODA_NO_TCGEN05
  if (path == MODA_PATH_TCGEN05) {
    void* extra = reinterpret_cast<unsigned char*>(workspace) + delta_bytes(prob);
    return tc::bwd(p, prob, extra, n_sm, st, &g_last_launches, &g_last_cuda_error);
  }
#endif
  return prob->dtype == MODA_BF16 ? simt_bwd_d<__nv_bfloat16>(p, prob->D, n_sm, st)
                                  : simt_bwd_d<__half>(p, prob->D, n_sm, st);
}

int moda_b200_depth_append(const moda_problem* prob, const moda_tensor4* k, const moda_tensor4* v,
                           const moda_tensor4* cache_k, const moda_tensor4* cache_v, int32_t layer, void* stream) {
  if (prob == nullptr) return MODA_ERR_NULL;
  if (prob->B < 1 || prob->T_kv < 1 || prob->H < 1 || prob->B > 65535 || prob->H > 65535) return MODA_ERR_SHAPE;
  if (prob->D != 64 && prob->D != 128) return MODA_ERR_HEAD_DIM;
  if (prob->dtype != MODA_BF16 && prob->dtype != MODA_FP16) return MODA_ERR_DTYPE;
  const int Lmax = prob->depth_rows_per_pos;
  if (Lmax < 1 || layer < 0 || layer >= Lmax || (int64_t)prob->T_kv * Lmax > (int64_t)1 << 30) return MODA_ERR_SHAPE;
  if (int rc = check_tensor(k, true, prob->B, prob->T_kv, prob->H)) return rc;
  if (int rc = check_tensor(v, true, prob->B, prob->T_kv, prob->H)) return rc;
  if (int rc = check_tensor(cache_k, true, prob->B, (int64_t)prob->T_kv * Lmax, prob->H)) return rc;
  if (int rc = check_tensor(cache_v, true, prob->B, (int64_t)prob->T_kv * Lmax, prob->H)) return rc;
  DeviceGuard guard(prob->device);
  if (!guard.ok) return cuda_fail(guard.err);
  g_last_launches = 0;
  const int n_sm = sm_count(prob->device);
  if (n_sm <= 0) return cuda_fail(cudaErrorInvalidDevice);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int64_t n = (int64_t)prob->B * prob->T_kv * prob->H * (prob->D / 8);
  const int64_t want = (n + 255) / 256, cap = (int64_t)n_sm * 16;
  const int blocks = (int)(want < cap ? want : cap);
  {
    prof::Scope ps(prof::kDepthAppend, st);
    if (prob->D == 128)
      cache::append_kernel<16><<<blocks, 256, 0, st>>>(to_view(k), to_view(v), to_view(cache_k), to_view(cache_v),
                                                      prob->B, prob->T_kv, prob->H, Lmax, layer);
    else
      cache::append_kernel<8><<<blocks, 256, 0, st>>>(to_view(k), to_view(v), to_view(cache_k), to_view(cache_v),
                                                     prob->B, prob->T_kv, prob->H, Lmax, layer);
  }
  MODA_CUDA(cudaGetLastError());
  g_last_launches += 1;
  return MODA_OK;
}

int moda_b200_profile_begin(void) {
  prof::State& ps = prof::state();
  std::lock_guard<std::mutex> lk(ps.mu);
  for (auto& e : ps.entries) { cudaEventDestroy(e.a); cudaEventDestroy(e.b); }
  ps.entries.clear();
  ps.on = true;
  return MODA_OK;
}

int moda_b200_profile_end(int max_entries, int* n_entries, int* kernel_ids, int* launches, float* total_ms) {
  if (n_entries == nullptr || kernel_ids == nullptr || launches == nullptr || total_ms == nullptr) return MODA_ERR_NULL;
  prof::State& ps = prof::state();
  std::lock_guard<std::mutex> lk(ps.mu);
  ps.on = false;
  int cnt[prof::kCount] = {0};
  float ms[prof::kCount] = {0.f};
  int rc = MODA_OK;
  for (auto& e : ps.entries) {
    float t = 0.f;
    cudaError_t err = cudaEventSynchronize(e.b);
    if (err == cudaSuccess) err = cudaEventElapsedTime(&t, e.a, e.b);
    if (err != cudaSuccess) { g_last_cuda_error = (int)err; rc = MODA_ERR_CUDA; }
    cnt[e.id] += 1; ms[e.id] += t;
    cudaEventDestroy(e.a); cudaEventDestroy(e.b);
  }
  ps.entries.clear();
  int n = 0;
  for (int i = 0; i < prof::kCount && n < max_entries; ++i) {
    if (cnt[i] == 0) continue;
    kernel_ids[n] = i; launches[n] = cnt[i]; total_ms[n] = ms[i]; ++n;
  }
  *n_entries = n;
  return rc;
}

const char* moda_b200_kernel_name(int kernel_id) { return prof::kernel_name(kernel_id); }

int moda_b200_device_status(int* status) {
  if (status == nullptr) return MODA_ERR_NULL;
#ifndef MODA_NO_TCGEN05
  int v = 0;
  const int e = tc::read_status(&v);
  if (e != 0) { g_last_cuda_error = e; return MODA_ERR_CUDA; }
  *status = v;
#else
  *status = 0;
#endif
  return MODA_OK;
}

// ---- backward without any caller-provided or library-allocated scratch ---------------
// The scratch of the backward lives in this file-scope device array.  In host code the
// name g_static_scratch is only a handle for the runtime; the address kernels can use is
// obtained per device with cudaGetSymbolAddress and cached below.
static __device__ __align__(256) unsigned char g_static_scratch[MODA_B200_STATIC_SCRATCH_BYTES];

namespace {
constexpr int kMaxDevices = 64;
std::mutex g_scratch_mu;
void* g_scratch_ptr[kMaxDevices] = {nullptr};

// Device address of g_static_scratch on the CURRENT device (resolved once per device).
int static_scratch_address(int device, void** out) {
  if (device < 0 || device >= kMaxDevices) return MODA_ERR_SHAPE;
  std::lock_guard<std::mutex> lk(g_scratch_mu);
  if (g_scratch_ptr[device] == nullptr) {
    void* ptr = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&ptr, g_static_scratch);
    if (e != cudaSuccess || ptr == nullptr) return cuda_fail(e != cudaSuccess ? e : cudaErrorInvalidSymbol);
    g_scratch_ptr[device] = ptr;
  }
  *out = g_scratch_ptr[device];
  return MODA_OK;
}
}  // namespace

int moda_b200_bwd_static_scratch(const moda_problem* prob, const moda_tensor4* q, const moda_tensor4* k,
                                 const moda_tensor4* v, const moda_tensor4* depth_k,
                                 const moda_tensor4* depth_v, const moda_tensor4* o, const float* lse,
                                 const moda_tensor4* dout, const moda_tensor4* dq, const moda_tensor4* dk,
                                 const moda_tensor4* dv, const moda_tensor4* d_depth_k,
                                 const moda_tensor4* d_depth_v, void* stream) {
  size_t need = 0;
  if (int rc = moda_b200_bwd_workspace_bytes(prob, &need)) return rc;
  if (need > (size_t)MODA_B200_STATIC_SCRATCH_BYTES) return MODA_ERR_TOO_LARGE;
  DeviceGuard guard(prob->device);          // the symbol address is per device: resolve it with
  if (!guard.ok) return cuda_fail(guard.err);  // the problem's device current
  void* scratch = nullptr;
  if (int rc = static_scratch_address(prob->device, &scratch)) return rc;
  return moda_b200_bwd(prob, q, k, v, depth_k, depth_v, o, lse, dout, dq, dk, dv, d_depth_k, d_depth_v,
                       scratch, (size_t)MODA_B200_STATIC_SCRATCH_BYTES, stream);
}

int moda_b200_tensor_pipe_rates(int device, float* clocks_per_mma, void* stream) {
  if (!clocks_per_mma) return MODA_ERR_NULL;
  DeviceGuard guard(device);
  if (!guard.ok) return cuda_fail(guard.err);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  MODA_CUDA(tc::clear_launch_status(st));
  MODA_CUDA(tc::mma_rates(clocks_per_mma, st));
  g_last_launches = 12;
  return MODA_OK;
}

int moda_b200_last_launch_count(void) { return g_last_launches; }
int moda_b200_last_cuda_error(void) { return g_last_cuda_error; }

const char* moda_b200_status_string(int status) {
  switch (status) {
    case MODA_OK: return "ok";
    case MODA_ERR_NULL: return "required pointer is NULL";
    case MODA_ERR_SHAPE: return "invalid shape";
    case MODA_ERR_HEAD_DIM: return "head dim must be 64 or 128";
    case MODA_ERR_DTYPE: return "dtype must be bf16 or fp16";
    case MODA_ERR_ALIGNMENT: return "pointer or stride alignment";
    case MODA_ERR_MODE: return "invalid mode";
    case MODA_ERR_CHUNK: return "chunk_rows must be a positive multiple of G";
    case MODA_ERR_WORKSPACE: return "workspace missing or too small";
    case MODA_ERR_CUDA: return "CUDA call failed";
    case MODA_ERR_UNSUPPORTED: return "kernel path does not support this problem";
    case MODA_ERR_TOO_LARGE: return "problem exceeds the entry point's fixed capacity";
    default: return "unknown status";
  }
}

int moda_b200_version(void) { return 100; }

}  // extern "C"
