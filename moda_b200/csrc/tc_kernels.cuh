// tcgen05 / TMEM / TMA kernels (placeholder interface; filled in next).
#pragma once
#include "../../include/moda_b200.h"
#include "common.cuh"
namespace moda { namespace tc {
inline bool fwd_supported(const moda_problem*) { return false; }
inline bool bwd_supported(const moda_problem*) { return false; }
inline size_t bwd_extra_workspace_bytes(const moda_problem*) { return 0; }
inline int fwd(const Params&, const moda_problem*, cudaStream_t, int*, int*) { return MODA_ERR_UNSUPPORTED; }
inline int bwd(const Params&, const moda_problem*, void*, cudaStream_t, int*, int*) { return MODA_ERR_UNSUPPORTED; }
}}
