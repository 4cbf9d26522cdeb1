// Measurement aid, not part of the hot path: a plain streaming kernel with R
// input and W output streams (coalesced 128-bit grid-stride accesses).  HBM
// delivers different bandwidth for different read:write mixes, so the row-scan
// kernels are put next to this kernel at their own mix (bench.py, workloads
// stream_<R>r<W>w).
#include "api_util.cuh"

using namespace sb;

namespace {

template <int R, int W>
__global__ void __launch_bounds__(512)
stream_kernel(const float4* __restrict__ in, float4* __restrict__ out, size_t n4) {
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const float4 v = __ldg(in + r * n4 + i);
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
#pragma unroll
    for (int w = 0; w < W; ++w) {
      float4 o = acc;
      o.x += (float)w;
      out[w * n4 + i] = o;
    }
  }
}

template <int R>
int dispatch_w(int W, const float4* in, float4* out, size_t n4, unsigned grid, cudaStream_t st) {
  switch (W) {
    case 1: stream_kernel<R, 1><<<grid, 512, 0, st>>>(in, out, n4); break;
    case 2: stream_kernel<R, 2><<<grid, 512, 0, st>>>(in, out, n4); break;
    case 3: stream_kernel<R, 3><<<grid, 512, 0, st>>>(in, out, n4); break;
    case 4: stream_kernel<R, 4><<<grid, 512, 0, st>>>(in, out, n4); break;
    default: set_error("writes must be 1..4"); return SB_ERR_INVALID_ARG;
  }
  return SB_OK;
}

}  // namespace

extern "C" int sb_probe_stream(const float* in, float* out, int64_t n, int reads, int writes, void* stream) {
  SB_REQUIRE(n >= 0 && (n & 3) == 0, "element count must be a multiple of 4");
  SB_REQUIRE(reads >= 1 && reads <= 4 && writes >= 1 && writes <= 4, "reads and writes must be 1..4");
  if (n == 0) return SB_OK;
  SB_REQUIRE(in && out && ((((uintptr_t)in) | ((uintptr_t)out)) & 15u) == 0, "buffers must be 16-byte aligned");
  const unsigned grid = (unsigned)sm_count() * 16;
  cudaStream_t st = (cudaStream_t)stream;
  const float4* a = reinterpret_cast<const float4*>(in);
  float4* b = reinterpret_cast<float4*>(out);
  int rc;
  switch (reads) {
    case 1: rc = dispatch_w<1>(writes, a, b, (size_t)n / 4, grid, st); break;
    case 2: rc = dispatch_w<2>(writes, a, b, (size_t)n / 4, grid, st); break;
    case 3: rc = dispatch_w<3>(writes, a, b, (size_t)n / 4, grid, st); break;
    default: rc = dispatch_w<4>(writes, a, b, (size_t)n / 4, grid, st); break;
  }
  if (rc != SB_OK) return rc;
  SB_CUDA(cudaGetLastError());
  return SB_OK;
}
