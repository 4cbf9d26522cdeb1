// Sum-pooling synapse over NCHWT spike tensors (synapse/layer.py:326-508): the
// reference runs it as a Conv3d with an all-equal (kh, kw, 1) kernel and stride
// = kernel, which cuDNN serves with a grouped direct convolution several times
// slower than the memory roof.  It is a pure gather-and-add with the time axis
// contiguous, so here every thread owns four consecutive time steps of one
// output neuron and adds the kh x kw input rows that feed it (128-bit coalesced
// loads along time).  Weights stay a (kh, kw) table so a non-uniform kernel
// still gives conv3d's result; with 0/1 spikes and quantised weights the sums
// are exact whatever the order.
#include "api_util.cuh"

using namespace sb;

namespace {

constexpr int kMaxPoolTaps = 64;

struct PoolGeom {
  int NC, H, W, Ho, Wo, kh, kw, T;
};

template <bool VEC>
__global__ void __launch_bounds__(256)
pool_fwd_kernel(const float* __restrict__ x, const float* __restrict__ wgt, float* __restrict__ y, PoolGeom g) {
  __shared__ float w[kMaxPoolTaps];
  for (int i = threadIdx.x; i < g.kh * g.kw; i += blockDim.x) w[i] = __ldg(wgt + i);
  __syncthreads();
  constexpr int V = VEC ? 4 : 1;
  const int TV = g.T / V;
  const int64_t total = (int64_t)g.NC * g.Ho * g.Wo * TV;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int tv = (int)(idx % TV);
    int64_t r = idx / TV;
    const int wo = (int)(r % g.Wo); r /= g.Wo;
    const int ho = (int)(r % g.Ho);
    const int64_t nc = r / g.Ho;
    float acc[V];
#pragma unroll
    for (int v = 0; v < V; ++v) acc[v] = 0.f;
    for (int i = 0; i < g.kh; ++i) {
      const int h = ho * g.kh + i;
      if (h >= g.H) break;  // rows past the tensor are the zero padding
      for (int j = 0; j < g.kw; ++j) {
        const int ww = wo * g.kw + j;
        if (ww >= g.W) break;
        const float* src = x + ((nc * g.H + h) * (int64_t)g.W + ww) * g.T + (int64_t)tv * V;
        const float wv = w[i * g.kw + j];
        if (VEC) {
          const float4 a = __ldg(reinterpret_cast<const float4*>(src));
          acc[0] = fmaf(wv, a.x, acc[0]); acc[1] = fmaf(wv, a.y, acc[1]);
          acc[2] = fmaf(wv, a.z, acc[2]); acc[3] = fmaf(wv, a.w, acc[3]);
        } else {
          acc[0] = fmaf(wv, __ldg(src), acc[0]);
        }
      }
    }
    float* dst = y + idx * V;
    if (VEC) *reinterpret_cast<float4*>(dst) = make_float4(acc[0], acc[1], acc[2], acc[3]);
    else dst[0] = acc[0];
  }
}

// One block per input image row (nc, h), looping over the row's words: the only divisions are
// 32-bit and per thread, not per element (a flat index over NC * H * W * T costs four 64-bit
// divisions per word).
template <bool VEC>
__global__ void __launch_bounds__(256)
pool_bwd_kernel(const float* __restrict__ gy, const float* __restrict__ wgt, float* __restrict__ gx, PoolGeom g) {
  constexpr int V = VEC ? 4 : 1;
  const int TV = g.T / V;
  const int per_row = g.W * TV;                        // words of one input row
  const int64_t nrows = (int64_t)g.NC * g.H;
  for (int64_t row = blockIdx.y; row < nrows; row += gridDim.y) {
    const int64_t nc = row / g.H;                      // once per row
    const int h = (int)(row - nc * g.H);
    const int ho = h / g.kh, hk = h - ho * g.kh;
    float* drow = gx + row * (int64_t)g.W * g.T;
    const float* srow = gy + (nc * g.Ho + ho) * (int64_t)g.Wo * g.T;
    for (int q = blockIdx.x * blockDim.x + threadIdx.x; q < per_row; q += gridDim.x * blockDim.x) {
      const int ww = q / TV, tv = q - ww * TV;
      const int wo = ww / g.kw;
      float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
      if (ho < g.Ho && wo < g.Wo) {  // inputs past the last full window feed nothing
        const float wv = __ldg(wgt + hk * g.kw + (ww - wo * g.kw));
        const float* src = srow + (int64_t)wo * g.T + tv * V;
        if (VEC) {
          const float4 a = __ldg(reinterpret_cast<const float4*>(src));
          o = make_float4(__fmul_rn(wv, a.x), __fmul_rn(wv, a.y), __fmul_rn(wv, a.z), __fmul_rn(wv, a.w));
        } else {
          o.x = __fmul_rn(wv, __ldg(src));
        }
      }
      float* dst = drow + (int64_t)q * V;
      if (VEC) *reinterpret_cast<float4*>(dst) = o;
      else dst[0] = o.x;
    }
  }
}

int check_pool(const void* a, const void* wgt, const void* b, int64_t NC, int64_t H, int64_t W, int64_t Ho,
               int64_t Wo, int64_t kh, int64_t kw, int64_t T, PoolGeom* g) {
  SB_REQUIRE(NC >= 0 && H >= 0 && W >= 0 && T >= 0 && Ho >= 0 && Wo >= 0, "negative geometry");
  SB_REQUIRE(kh >= 1 && kw >= 1 && kh * kw <= kMaxPoolTaps, "pool window %lldx%lld outside 1..%d taps", (long long)kh,
             (long long)kw, kMaxPoolTaps);
  SB_REQUIRE(H < (1 << 30) && W < (1 << 30) && T < (1 << 30) && NC < (1LL << 40), "geometry too large");
  SB_REQUIRE(Ho * kh <= H + kh - 1 && Wo * kw <= W + kw - 1, "output size does not fit the input");
  if (NC * H * W * T == 0 || NC * Ho * Wo * T == 0) return 1;  // nothing to do
  SB_REQUIRE(a && wgt && b, "null tensor pointer");
  *g = PoolGeom{(int)0, (int)H, (int)W, (int)Ho, (int)Wo, (int)kh, (int)kw, (int)T};
  return SB_OK;
}

inline bool vec_ok(const void* a, const void* b, int64_t T) {
  return (T & 3) == 0 && ((((uintptr_t)a) | ((uintptr_t)b)) & 15u) == 0;
}

}  // namespace

extern "C" {

int sb_pool_fwd(const float* x, const float* weight, float* y, int64_t NC, int64_t H, int64_t W, int64_t Ho,
                int64_t Wo, int64_t kh, int64_t kw, int64_t T, void* stream) {
  PoolGeom g;
  const int rc = check_pool(x, weight, y, NC, H, W, Ho, Wo, kh, kw, T, &g);
  if (rc == 1) return SB_OK;
  if (rc != SB_OK) return rc;
  SB_REQUIRE(NC < (1LL << 31), "too many channel planes");
  g.NC = (int)NC;
  const bool vec = vec_ok(x, y, T);
  const int64_t total = NC * Ho * Wo * (vec ? T / 4 : T);
  int64_t blocks = (total + 255) / 256;
  const int64_t cap = (int64_t)sm_count() * 32;
  if (blocks > cap) blocks = cap;
  cudaStream_t st = (cudaStream_t)stream;
  if (vec) pool_fwd_kernel<true><<<(unsigned)blocks, 256, 0, st>>>(x, weight, y, g);
  else pool_fwd_kernel<false><<<(unsigned)blocks, 256, 0, st>>>(x, weight, y, g);
  SB_CUDA(cudaGetLastError());
  return SB_OK;
}

int sb_pool_bwd(const float* grad_y, const float* weight, float* grad_x, int64_t NC, int64_t H, int64_t W,
                int64_t Ho, int64_t Wo, int64_t kh, int64_t kw, int64_t T, void* stream) {
  PoolGeom g;
  const int rc = check_pool(grad_y, weight, grad_x, NC, H, W, Ho, Wo, kh, kw, T, &g);
  if (rc == 1) {
    if (NC * H * W * T > 0 && grad_x) SB_CUDA(cudaMemsetAsync(grad_x, 0, sizeof(float) * NC * H * W * T, (cudaStream_t)stream));
    return SB_OK;
  }
  if (rc != SB_OK) return rc;
  SB_REQUIRE(NC < (1LL << 31), "too many channel planes");
  g.NC = (int)NC;
  const bool vec = vec_ok(grad_y, grad_x, T);
  SB_REQUIRE(W * (vec ? T / 4 : T) < (1LL << 31), "input row too long");
  const int64_t per_row = W * (vec ? T / 4 : T);
  // whole rows per block; a row is split over several blocks only when there are too few rows to fill the GPU
  int64_t gyr = NC * H;
  if (gyr > 65535) gyr = 65535;
  int64_t gx = ((int64_t)sm_count() * 8 + gyr - 1) / gyr;
  const int64_t gx_max = (per_row + 255) / 256;
  if (gx > gx_max) gx = gx_max;
  if (gx < 1) gx = 1;
  const dim3 grid((unsigned)gx, (unsigned)gyr);
  cudaStream_t st = (cudaStream_t)stream;
  if (vec) pool_bwd_kernel<true><<<grid, 256, 0, st>>>(grad_y, weight, grad_x, g);
  else pool_bwd_kernel<false><<<grid, 256, 0, st>>>(grad_y, weight, grad_x, g);
  SB_CUDA(cudaGetLastError());
  return SB_OK;
}

}  // extern "C"
