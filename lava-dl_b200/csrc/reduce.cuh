// Folding of per-warp / per-row parameter-gradient partials (fp64) into the
// fp32 gradient the reference returns (torch.sum over batch, space and time:
// leaky_integrator.py:248-257, resonator.py:449-465).
//
// Scratch layout handed in by the caller (doubles):
//   [0, nparts)                    partials written by the backward kernel
//                                  (nparts = ceil(rows/32) for a shared
//                                  parameter, rows for a per-channel one)
//   [nparts, nparts + slices * n)  stage buffer of the two-step fold
// Both steps use a fixed summation order, so results are deterministic.
#pragma once

#include "common.cuh"

namespace sb {

constexpr int kFoldSlices = 64;

int64_t scratch_slots(int64_t rows, int64_t n);
int fold_param_grad(double* scratch, float* out, const RowGeom& g, int64_t n, cudaStream_t st);

__device__ __forceinline__ double block_sum(double v) {
  __shared__ double red[32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  if (lane == 0) red[warp] = v;
  __syncthreads();
  const int nw = (blockDim.x + 31) >> 5;
  v = (threadIdx.x < nw) ? red[threadIdx.x] : 0.0;
  if (warp == 0) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  }
  return v;
}

}  // namespace sb
