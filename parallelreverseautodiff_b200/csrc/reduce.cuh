// Deterministic block reduction in double: warp shuffles, then the warp totals in warp
// order.  Same launch shape => same bits, run after run.
#pragma once

#include <cuda_runtime.h>

namespace prad {

__device__ __forceinline__ double warp_sum_d(double v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// all threads of the block must call; result valid in thread 0 (and broadcast to all)
template <int THREADS>
__device__ __forceinline__ double block_sum_d(double v) {
  __shared__ double warp_tot[THREADS / 32];
  __shared__ double total;
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  v = warp_sum_d(v);
  __syncthreads();  // protects warp_tot/total across back-to-back calls
  if (lane == 0) warp_tot[w] = v;
  __syncthreads();
  if (threadIdx.x == 0) {
    double s = 0.0;
#pragma unroll
    for (int k = 0; k < THREADS / 32; ++k) s += warp_tot[k];
    total = s;
  }
  __syncthreads();
  return total;
}

}  // namespace prad
