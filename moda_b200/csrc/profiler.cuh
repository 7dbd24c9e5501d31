// Optional per-kernel device timing: cudaEvents recorded on the launch stream around
// each kernel launch while profiling is switched on (moda_b200_profile_begin/_end).
#pragma once
#include <cuda_runtime.h>

#include <mutex>
#include <vector>

namespace moda {
namespace prof {

enum KernelId : int {
  kFwdSimt = 0, kDelta, kDqSimt, kDkvSimt, kFwdTc, kPreTc, kDqTc, kDkvTc, kFdaFwd, kFdaBwd, kDepthGradTc, kDepthAppend, kBwdFusedTc, kBwdBoundsTc, kCount
};
inline const char* kernel_name(int id) {
  static const char* const names[kCount] = {"simt_fwd", "delta", "simt_dq", "simt_dkv", "tc_fwd",
                                            "tc_bwd_pre", "tc_dq", "tc_dkv", "fda_fwd", "fda_bwd", "tc_depth_grad",
                                            "depth_append", "tc_bwd_fused", "tc_bwd_bounds"};
  return (id >= 0 && id < kCount) ? names[id] : "unknown";
}

struct Entry { int id; cudaEvent_t a, b; };
struct State {
  std::mutex mu;
  bool on = false;
  std::vector<Entry> entries;
};
inline State& state() { static State s; return s; }

// Brackets one launch.  Construct before the <<<>>>, let it go out of scope after.
struct Scope {
  cudaStream_t st; cudaEvent_t a = nullptr, b = nullptr; int id; bool on;
  Scope(int id_, cudaStream_t st_) : st(st_), id(id_), on(state().on) {
    if (on) {
      if (cudaEventCreate(&a) != cudaSuccess || cudaEventCreate(&b) != cudaSuccess) { on = false; return; }
      cudaEventRecord(a, st);
    }
  }
  ~Scope() {
    if (on) {
      cudaEventRecord(b, st);
      std::lock_guard<std::mutex> lk(state().mu);
      state().entries.push_back({id, a, b});
    }
  }
};

}  // namespace prof
}  // namespace moda
