// In-place depth-KV cache: one layer's K and V rows are copied into their slot of a persistent
// [B, T, Lmax, H, D] cache, which later layers read as depth K/V through Params::Ls.  Replaces the
// reference caller's per-layer rebuild of the whole cache (torch.stack over all earlier layers,
// reshape, contiguous: vision_tasks/deit/models.py:361-375), whose copies grow with the square of
// the layer count; here every K/V row is copied once.
#pragma once
#include "common.cuh"

namespace moda {
namespace cache {

// One thread per 16-byte chunk of a (b, t, h) row of k and of v.  chunks = D / 8.
template <int kChunks>
__global__ void __launch_bounds__(256) append_kernel(View k, View v, View ck, View cv, int B, int T, int H, int Ls, int slot) {
  const int64_t n = (int64_t)B * T * H * kChunks;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const int c = (int)(i % kChunks);
    int64_t r = i / kChunks;
    const int h = (int)(r % H); r /= H;
    const int t = (int)(r % T);
    const int b = (int)(r / T);
    const int64_t dst_row = (int64_t)t * Ls + slot;
    const uint4 kv4 = *reinterpret_cast<const uint4*>(reinterpret_cast<const unsigned char*>(k.ptr) + 2 * (k.off(b, t, h) + c * 8));
    const uint4 vv4 = *reinterpret_cast<const uint4*>(reinterpret_cast<const unsigned char*>(v.ptr) + 2 * (v.off(b, t, h) + c * 8));
    *reinterpret_cast<uint4*>(reinterpret_cast<unsigned char*>(ck.ptr) + 2 * (ck.off(b, dst_row, h) + c * 8)) = kv4;
    *reinterpret_cast<uint4*>(reinterpret_cast<unsigned char*>(cv.ptr) + 2 * (cv.off(b, dst_row, h) + c * 8)) = vv4;
  }
}

}  // namespace cache
}  // namespace moda
