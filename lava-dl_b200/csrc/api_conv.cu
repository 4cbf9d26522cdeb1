// Spatial convolution synapse over NCHWT tensors with a unit time kernel
// (synapse/layer.py:178-323), stride 1, no dilation, one group.  The reference
// hands this to cuDNN as a Conv3d; with time innermost cuDNN first transposes to
// channels-last and back, and the whole call is several times slower than the
// arithmetic needs.  Here time stays the vector axis: a thread owns four
// consecutive time steps of one output pixel for a tile of 16 output channels
// (64 accumulators), walks the (ci, kh, kw) taps with one coalesced 128-bit
// load of the input per tap and the 16 tap weights broadcast from shared memory:
// 64 FMAs per load.  With 0/1 spikes and weights on the 1/32 grid every partial
// sum is exact, so the result is bit-identical to cuDNN's and to the CPU's.
#include "api_util.cuh"

using namespace sb;

namespace {

constexpr int kCoTile = 16;
constexpr int kConvThreads = 128;

struct ConvGeom {
  int N, Ci, Co, H, W, Ho, Wo, kh, kw, ph, pw, T;
};

// KW > 0 fixes the kernel width at compile time so that the KW input loads of a
// kernel row are issued together before their FMAs (memory-level parallelism);
// KW = 0 is the run-time width.
template <bool VEC, int KW>
__global__ void __launch_bounds__(kConvThreads)
conv_fwd_kernel(const float* __restrict__ x, const float* __restrict__ wgt, float* __restrict__ y, ConvGeom g) {
  extern __shared__ float ws[];  // [Ci * kh * kw][kCoTile], output channel fastest
  constexpr int V = VEC ? 4 : 1;
  const int taps = g.Ci * g.kh * g.kw;
  const int co0 = blockIdx.z * kCoTile;
  for (int i = threadIdx.x; i < taps * kCoTile; i += kConvThreads) {
    const int c = i % kCoTile, tap = i / kCoTile;
    const int co = co0 + c;
    ws[i] = (co < g.Co) ? __ldg(wgt + (int64_t)co * taps + tap) : 0.f;
  }
  __syncthreads();

  const int TV = g.T / V;
  const int n = blockIdx.y / g.Ho, ho = blockIdx.y % g.Ho;
  const int q = blockIdx.x * kConvThreads + threadIdx.x;  // flattened (wo, time vector)
  if (q >= g.Wo * TV) return;
  const int wo = q / TV, tv = q - wo * TV;

  float acc[kCoTile][V];
#pragma unroll
  for (int c = 0; c < kCoTile; ++c)
#pragma unroll
    for (int v = 0; v < V; ++v) acc[c][v] = 0.f;

  if (KW > 0) {
    // Software pipeline over the Ci * kh kernel rows: the KW input words of row
    // r + 1 are requested before the FMAs of row r run (one register set in
    // flight), so the loads' L1/L2 latency hides behind 64 * KW FMAs.
    constexpr int KWc = KW > 0 ? KW : 1;
    const int rows = g.Ci * g.kh;
    auto load_row = [&](int r, float (&xv)[KWc][V]) -> bool {
      const int ci = r / g.kh, i = r - ci * g.kh;
      const int h = ho + i - g.ph;
      const bool row_in = r < rows && h >= 0 && h < g.H;
      const float* row = x + (((int64_t)n * g.Ci + ci) * g.H + (row_in ? h : 0)) * (int64_t)g.W * g.T + (int64_t)tv * V;
#pragma unroll
      for (int j = 0; j < KWc; ++j) {
        const int wsrc = wo + j - g.pw;
        const bool in = row_in && wsrc >= 0 && wsrc < g.W;
        if (VEC) {
          float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
          if (in) a = __ldg(reinterpret_cast<const float4*>(row + (int64_t)wsrc * g.T));
          xv[j][0] = a.x; xv[j][1 % V] = a.y; xv[j][2 % V] = a.z; xv[j][3 % V] = a.w;
        } else {
          xv[j][0] = in ? __ldg(row + (int64_t)wsrc * g.T) : 0.f;
        }
      }
      return row_in;  // uniform over the block
    };
    auto fma_row = [&](int r, const float (&xv)[KWc][V]) {
      const float* wrow = ws + r * KWc * kCoTile;
#pragma unroll
      for (int j = 0; j < KWc; ++j) {
#pragma unroll
        for (int c4 = 0; c4 < kCoTile / 4; ++c4) {
          const float4 w4 = *reinterpret_cast<const float4*>(wrow + j * kCoTile + 4 * c4);
#pragma unroll
          for (int v = 0; v < V; ++v) {
            acc[4 * c4 + 0][v] = fmaf(w4.x, xv[j][v], acc[4 * c4 + 0][v]);
            acc[4 * c4 + 1][v] = fmaf(w4.y, xv[j][v], acc[4 * c4 + 1][v]);
            acc[4 * c4 + 2][v] = fmaf(w4.z, xv[j][v], acc[4 * c4 + 2][v]);
            acc[4 * c4 + 3][v] = fmaf(w4.w, xv[j][v], acc[4 * c4 + 3][v]);
          }
        }
      }
    };
    float xa[KWc][V], xb[KWc][V];
    bool in_a = load_row(0, xa), in_b = false;
    for (int r = 0; r < rows; r += 2) {
      in_b = load_row(r + 1, xb);
      if (in_a) fma_row(r, xa);
      in_a = load_row(r + 2, xa);
      if (in_b) fma_row(r + 1, xb);
    }
  } else
  for (int ci = 0; ci < g.Ci; ++ci) {
    for (int i = 0; i < g.kh; ++i) {
      const int h = ho + i - g.ph;
      if (h < 0 || h >= g.H) continue;
      const float* row = x + (((int64_t)n * g.Ci + ci) * g.H + h) * (int64_t)g.W * g.T + (int64_t)tv * V;
      const float* wrow = ws + (ci * g.kh + i) * g.kw * kCoTile;
      for (int j = 0; j < g.kw; ++j) {
        const int wsrc = wo + j - g.pw;
        if (wsrc < 0 || wsrc >= g.W) continue;
        float xv[V];
        if (VEC) {
          const float4 a = __ldg(reinterpret_cast<const float4*>(row + (int64_t)wsrc * g.T));
          xv[0] = a.x; xv[1 % V] = a.y; xv[2 % V] = a.z; xv[3 % V] = a.w;
        } else {
          xv[0] = __ldg(row + (int64_t)wsrc * g.T);
        }
        const float* wt = wrow + j * kCoTile;
#pragma unroll
        for (int c4 = 0; c4 < kCoTile / 4; ++c4) {
          const float4 w4 = *reinterpret_cast<const float4*>(wt + 4 * c4);
#pragma unroll
          for (int v = 0; v < V; ++v) {
            acc[4 * c4 + 0][v] = fmaf(w4.x, xv[v], acc[4 * c4 + 0][v]);
            acc[4 * c4 + 1][v] = fmaf(w4.y, xv[v], acc[4 * c4 + 1][v]);
            acc[4 * c4 + 2][v] = fmaf(w4.z, xv[v], acc[4 * c4 + 2][v]);
            acc[4 * c4 + 3][v] = fmaf(w4.w, xv[v], acc[4 * c4 + 3][v]);
          }
        }
      }
    }
  }
#pragma unroll
  for (int c = 0; c < kCoTile; ++c) {
    const int co = co0 + c;
    if (co >= g.Co) break;
    float* dst = y + ((((int64_t)n * g.Co + co) * g.Ho + ho) * (int64_t)g.Wo) * g.T + (int64_t)q * V;
    if (VEC) *reinterpret_cast<float4*>(dst) = make_float4(acc[c][0], acc[c][1 % V], acc[c][2 % V], acc[c][3 % V]);
    else dst[0] = acc[c][0];
  }
}

}  // namespace

namespace sb {
int conv_tc_try(const float* x, const float* weight, float* y, int64_t N, int64_t Ci, int64_t Co, int64_t H, int64_t W,
                int64_t kh, int64_t kw, int64_t ph, int64_t pw, int64_t T, cudaStream_t st, bool* taken);
}

extern "C" int sb_conv_fwd_path(const float* x, const float* weight, float* y, int64_t N, int64_t Ci, int64_t Co,
                                int64_t H, int64_t W, int64_t kh, int64_t kw, int64_t ph, int64_t pw, int64_t T,
                                int path, void* stream) {
  SB_REQUIRE(path >= -1 && path <= 1, "path is -1 (automatic), 0 (fp32 kernel) or 1 (tensor cores)");
  SB_REQUIRE(N >= 0 && Ci >= 1 && Co >= 1 && H >= 0 && W >= 0 && T >= 0, "bad geometry");
  SB_REQUIRE(kh >= 1 && kw >= 1 && ph >= 0 && pw >= 0, "bad kernel geometry");
  const int64_t Ho = H + 2 * ph - kh + 1, Wo = W + 2 * pw - kw + 1;
  SB_REQUIRE(Ho >= 0 && Wo >= 0, "kernel larger than the padded input");
  if (N * Co * Ho * Wo * T == 0) return SB_OK;
  SB_REQUIRE(x && weight && y, "null tensor pointer");
  const bool aligned = ((((uintptr_t)x) | ((uintptr_t)y)) & 15u) == 0;
  if (path == 1 || (path == -1 && aligned && sb_conv_uses_tensor_cores(N, Ci, Co, H, W, kh, kw, ph, pw, T))) {
    // implicit GEMM on the tensor cores (api_conv_tc.cu)
    bool taken = false;
    SB_TRY(conv_tc_try(x, weight, y, N, Ci, Co, H, W, kh, kw, ph, pw, T, (cudaStream_t)stream, &taken));
    if (taken) return SB_OK;
    if (path == 1) {
      set_error("the tensor-core convolution does not take this geometry or alignment");
      return SB_ERR_UNSUPPORTED;
    }
  }
  SB_REQUIRE(N * Ho <= 65535 * 32767LL && H < (1 << 20) && W < (1 << 20) && T < (1 << 24) && Ci * kh * kw < (1 << 20),
             "geometry too large");
  const size_t smem = sizeof(float) * (size_t)(Ci * kh * kw) * kCoTile;
  SB_REQUIRE(smem <= 96 * 1024, "Ci * kh * kw = %lld taps do not fit shared memory", (long long)(Ci * kh * kw));
  const bool vec = (T & 3) == 0 && ((((uintptr_t)x) | ((uintptr_t)y)) & 15u) == 0;
  const int64_t per_row = Wo * (vec ? T / 4 : T);
  const int64_t gx = (per_row + kConvThreads - 1) / kConvThreads;
  SB_REQUIRE(gx < (1LL << 31) && N * Ho <= 65535, "geometry outside the launch grid (N * Ho = %lld)", (long long)(N * Ho));
  const dim3 grid((unsigned)gx, (unsigned)(N * Ho), (unsigned)((Co + kCoTile - 1) / kCoTile));
  ConvGeom g{(int)N, (int)Ci, (int)Co, (int)H, (int)W, (int)Ho, (int)Wo, (int)kh, (int)kw, (int)ph, (int)pw, (int)T};
  cudaStream_t st = (cudaStream_t)stream;
#define SB_GO(VECF, KWF)                                                                                      \
  {                                                                                                           \
    auto fn = conv_fwd_kernel<VECF, KWF>;                                                                     \
    if (smem > 48 * 1024)                                                                                     \
      SB_CUDA(cudaFuncSetAttribute((const void*)fn, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024)); \
    fn<<<grid, kConvThreads, smem, st>>>(x, weight, y, g);                                                    \
  }
  if (vec) {
    if (kw == 3) SB_GO(true, 3) else if (kw == 5) SB_GO(true, 5) else if (kw == 1) SB_GO(true, 1) else SB_GO(true, 0)
  } else {
    SB_GO(false, 0)
  }
#undef SB_GO
  SB_CUDA(cudaGetLastError());
  return SB_OK;
}

extern "C" int sb_conv_fwd(const float* x, const float* weight, float* y, int64_t N, int64_t Ci, int64_t Co,
                           int64_t H, int64_t W, int64_t kh, int64_t kw, int64_t ph, int64_t pw, int64_t T,
                           void* stream) {
  return sb_conv_fwd_path(x, weight, y, N, Ci, Co, H, W, kh, kw, ph, pw, T, -1, stream);
}
