// Weight gradient of the convolution synapse (the backward of the Conv3d call of
// synapse/layer.py:297-323 with respect to its weight), stride 1, no dilation,
// one group, fp32 throughout:
//   dW[co][ci][i][j] = sum_{n, ho, wo, t} dz[n, co, ho, wo, t] * x[n, ci, ho + i - ph, wo + j - pw, t]
// cuDNN runs this as a TF32 implicit GEMM after transposing both tensors to
// channels-last (time innermost is not a layout it has); here time stays the
// vector axis.  A CTA owns one output row (n, ho) and reduces over (wo, t): it
// stages 16-step chunks of the dz row [Co][Wo] and of the kh input rows
// [Ci * kh][Wo + kw - 1] in shared memory (cp.async, double buffered); a thread owns an 8 x 8 tile of
// (output channel, tap) accumulators for every wg-th output column and reads
// operands as 128-bit words of four time steps: 256 FMAs per 16 shared loads.
// The threads of the column groups are then summed in shared memory and the
// CTA's partial goes to scratch; a second kernel adds the N * Ho partials in a
// fixed order, so the result does not depend on scheduling.
#include "api_util.cuh"

using namespace sb;

namespace {

constexpr int kTc = 16;            // time steps per staged chunk
constexpr int kQ = kTc / 4;        // 128-bit words per chunk
constexpr int kTile = 8;           // accumulator tile edge (channels and taps)
constexpr int kMaxThreads = 384;

struct WgradGeom {
  int N, Ci, Co, H, W, Ho, Wo, kh, kw, ph, pw, T;
  int taps, ncog, ntapg, owners, wgroups, Wp;
  int dz_row, x_row;               // shared-memory row strides in 128-bit words (skewed)
};

__global__ void __launch_bounds__(kMaxThreads)
conv_wgrad_kernel(const float* __restrict__ x, const float* __restrict__ dz, float* __restrict__ partial,
                  WgradGeom g) {
  extern __shared__ float4 sm4[];   // two staging buffers: dz rows [ncog * 8][dz_row], then x rows [Ci * kh][x_row]
  const int tid = threadIdx.x, nthreads = blockDim.x;
  const int n = blockIdx.x / g.Ho, ho = blockIdx.x % g.Ho;
  const int owner = tid % g.owners, wg = tid / g.owners;
  const int cog = owner % g.ncog, tapg = owner / g.ncog;
  const bool active = wg < g.wgroups;

  // This thread's 8 taps are tapg, tapg + ntapg, ...: for a given k the threads of a warp then read
  // consecutive taps, and with x_s laid out [row][time word][column] and a row stride that is kw
  // (mod 8) 128-bit words, consecutive taps sit in consecutive banks.  xoff: offset of tap k in x_s.
  int xoff[kTile];
#pragma unroll
  for (int k = 0; k < kTile; ++k) {
    const int tap = tapg + g.ntapg * k;
    const bool ok = tap < g.taps;
    const int r = ok ? tap / g.kw : 0, j = ok ? tap - r * g.kw : 0;
    xoff[k] = r * g.x_row + j;
  }
  // dz rows are stored channel-tile interleaved (row = (co % 8) * ncog + co / 8) with an odd stride,
  // so the ncog different rows a warp reads at once fall into different banks.
  float acc[kTile][kTile];
#pragma unroll
  for (int c = 0; c < kTile; ++c)
#pragma unroll
    for (int k = 0; k < kTile; ++k) acc[c][k] = 0.f;

  const int TV = g.T / 4;
  const int rows_x = g.Ci * g.kh, rows_dz = g.ncog * kTile;
  const int buf_words = rows_dz * g.dz_row + rows_x * g.x_row;   // one staging buffer, in 128-bit words
  const uint32_t sm_base = smem_u32(sm4);

  // Staging with cp.async, double buffered: a thread keeps one (column, time word) position of
  // the row and walks down the rows, so the loop has no divisions; positions outside the tensor
  // (channels past Co, rows and columns of the zero padding, time past T) are zero filled.
  // A row has P = columns x time words positions.  With at least P threads, tid / P rows are staged side by
  // side; with fewer (a narrow layer with few accumulator tiles, or a wide image) every thread takes
  // several positions of a row.
  const int dz_P = g.Wo * kQ, x_P = g.Wp * kQ;
  const bool dz_wide = nthreads >= dz_P, x_wide = nthreads >= x_P;
  const int dz_lane0 = dz_wide ? tid % dz_P : tid, dz_r0 = dz_wide ? tid / dz_P : 0;
  const int dz_rstep = dz_wide ? nthreads / dz_P : 1, dz_lstep = dz_wide ? dz_P : nthreads;
  const int x_lane0 = x_wide ? tid % x_P : tid, x_r0 = x_wide ? tid / x_P : 0;
  const int x_rstep = x_wide ? nthreads / x_P : 1, x_lstep = x_wide ? x_P : nthreads;
  auto stage = [&](int q0, int buf) {
    const uint32_t dst0 = sm_base + (uint32_t)(buf * buf_words) * 16u;
    if (dz_r0 < dz_rstep) {
      for (int lane = dz_lane0; lane < dz_P; lane += dz_lstep) {
        const int q = lane % kQ, w = lane / kQ;
        const bool tin = q0 + q < TV;
        const float* src = dz + (((int64_t)n * g.Co * g.Ho + ho) * g.Wo + w) * g.T + (int64_t)(q0 + q) * 4;
        for (int co = dz_r0; co < rows_dz; co += dz_rstep) {
          const bool ok = tin && co < g.Co;
          const float* p = ok ? src + (int64_t)co * g.Ho * g.Wo * g.T : dz;
          const int row = (co % kTile) * g.ncog + co / kTile;
          asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst0 + (uint32_t)(row * g.dz_row + lane) * 16u),
                       "l"(p), "r"(ok ? 16 : 0) : "memory");
        }
      }
    }
    if (x_r0 < x_rstep) {
      for (int lane = x_lane0; lane < x_P; lane += x_lstep) {
        const int q = lane % kQ, wp = lane / kQ, win = wp - g.pw;
        const bool cin = q0 + q < TV && win >= 0 && win < g.W;
        const float* src = x + ((int64_t)n * g.Ci * g.H * g.W + win) * g.T + (int64_t)(q0 + q) * 4;
        for (int r = x_r0; r < rows_x; r += x_rstep) {
          const int ci = r / g.kh, hin = ho + (r - ci * g.kh) - g.ph;
          const bool ok = cin && hin >= 0 && hin < g.H;
          const float* p = ok ? src + ((int64_t)ci * g.H + hin) * g.W * g.T : x;
          asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;"
                       ::"r"(dst0 + (uint32_t)(rows_dz * g.dz_row + r * g.x_row + q * g.Wp + wp) * 16u), "l"(p), "r"(ok ? 16 : 0)
                       : "memory");
        }
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };

  const int nchunks = (TV + kQ - 1) / kQ;
  stage(0, 0);
  for (int c = 0; c < nchunks; ++c) {
    if (c + 1 < nchunks) {
      stage((c + 1) * kQ, (c + 1) & 1);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    const float4* dz_s = sm4 + (size_t)(c & 1) * buf_words;
    const float4* x_s = dz_s + (size_t)rows_dz * g.dz_row;
    if (active) {
      for (int w = wg; w < g.Wo; w += g.wgroups) {
#pragma unroll 1
        for (int q = 0; q < kQ; ++q) {
          float4 b[kTile];
#pragma unroll
          for (int k = 0; k < kTile; ++k) b[k] = x_s[xoff[k] + q * g.Wp + w];
#pragma unroll
          for (int cc = 0; cc < kTile; ++cc) {
            const float4 a = dz_s[(cc * g.ncog + cog) * g.dz_row + w * kQ + q];
#pragma unroll
            for (int k = 0; k < kTile; ++k) {
              acc[cc][k] = fmaf(a.x, b[k].x, acc[cc][k]);
              acc[cc][k] = fmaf(a.y, b[k].y, acc[cc][k]);
              acc[cc][k] = fmaf(a.z, b[k].z, acc[cc][k]);
              acc[cc][k] = fmaf(a.w, b[k].w, acc[cc][k]);
            }
          }
        }
      }
    }
    __syncthreads();   // the buffer just read is refilled two chunks later
  }
  // sum the column groups: red[wg][owner][64], then the first `owners` threads per output add them up
  float* red = reinterpret_cast<float*>(sm4);
  if (active) {
#pragma unroll
    for (int c = 0; c < kTile; ++c)
#pragma unroll
      for (int k = 0; k < kTile; ++k) red[((size_t)wg * g.owners + owner) * 64 + c * kTile + k] = acc[c][k];
  }
  __syncthreads();
  float* out = partial + (size_t)blockIdx.x * g.Co * g.taps;
  for (int i = tid; i < g.owners * 64; i += nthreads) {
    const int o = i / 64, e = i % 64;
    const int co = (o % g.ncog) * kTile + e / kTile, tap = (o / g.ncog) + g.ntapg * (e % kTile);
    if (co < g.Co && tap < g.taps) {
      float s = 0.f;
      for (int wgi = 0; wgi < g.wgroups; ++wgi) s += red[((size_t)wgi * g.owners + o) * 64 + e];
      out[(size_t)co * g.taps + tap] = s;
    }
  }
}

// Sum of the N * Ho partial gradients in a fixed order.  A 32 x 8 thread block owns 32 neighbouring
// outputs: thread (x, y) adds every eighth partial of output x (coalesced across x), the eight
// slices meet in shared memory.  (One thread per output walking all partials left 18 blocks of
// latency-bound threads: 0.05 ms per layer.)
__global__ void conv_wgrad_fold_kernel(const float* __restrict__ partial, float* __restrict__ grad_w, int nparts,
                                       int nout) {
  __shared__ double part[8][33];
  const int i = blockIdx.x * 32 + threadIdx.x;
  double s = 0.0;
  if (i < nout)
    for (int p = threadIdx.y; p < nparts; p += 8) s += (double)partial[(size_t)p * nout + i];
  part[threadIdx.y][threadIdx.x] = s;
  __syncthreads();
  if (threadIdx.y == 0 && i < nout) {
#pragma unroll
    for (int y = 1; y < 8; ++y) s += part[y][threadIdx.x];
    grad_w[i] = (float)s;
  }
}

int wgrad_plan(int64_t N, int64_t Ci, int64_t Co, int64_t H, int64_t W, int64_t kh, int64_t kw, int64_t ph,
               int64_t pw, int64_t T, WgradGeom* g, size_t* smem) {
  const int64_t Ho = H + 2 * ph - kh + 1, Wo = W + 2 * pw - kw + 1;
  SB_REQUIRE(Ho >= 1 && Wo >= 1, "kernel larger than the padded input");
  g->N = (int)N; g->Ci = (int)Ci; g->Co = (int)Co; g->H = (int)H; g->W = (int)W; g->Ho = (int)Ho; g->Wo = (int)Wo;
  g->kh = (int)kh; g->kw = (int)kw; g->ph = (int)ph; g->pw = (int)pw; g->T = (int)T;
  g->taps = (int)(Ci * kh * kw);
  g->ncog = (int)((Co + kTile - 1) / kTile);
  g->ntapg = (g->taps + kTile - 1) / kTile;
  g->owners = g->ncog * g->ntapg;
  SB_REQUIRE(g->owners <= kMaxThreads, "Co * Ci * kh * kw = %lld outputs exceed one CTA's accumulators",
             (long long)(Co * g->taps));
  int wgroups = kMaxThreads / g->owners;
  if (wgroups > g->Wo) wgroups = g->Wo;
  while (wgroups > 1 && g->Wo % wgroups != 0) --wgroups;   // equal work per column group
  g->wgroups = wgroups;
  g->Wp = (int)(Wo + kw - 1);
  g->dz_row = g->Wo * kQ + 1;                       // odd: interleaved channel tiles on different banks
  g->x_row = g->Wp * kQ;
  while ((g->x_row & 7) != (g->kw & 7)) ++g->x_row;  // consecutive taps on consecutive banks
  const size_t stage = 2 * sizeof(float4) * ((size_t)g->ncog * kTile * g->dz_row + (size_t)Ci * kh * g->x_row);
  const size_t red = sizeof(float) * (size_t)wgroups * g->owners * 64;
  *smem = stage > red ? stage : red;
  SB_REQUIRE(*smem <= 200 * 1024, "one output row (%lld bytes staged) does not fit shared memory", (long long)*smem);
  return SB_OK;
}

}  // namespace

extern "C" int64_t sb_conv_wgrad_scratch_bytes(int64_t N, int64_t Ci, int64_t Co, int64_t H, int64_t kh, int64_t kw,
                                               int64_t ph) {
  const int64_t Ho = H + 2 * ph - kh + 1;
  if (N <= 0 || Ho <= 0) return 0;
  return N * Ho * Co * Ci * kh * kw * (int64_t)sizeof(float);
}

extern "C" int sb_conv_wgrad_fits(int64_t N, int64_t Ci, int64_t Co, int64_t H, int64_t W, int64_t kh, int64_t kw,
                                  int64_t ph, int64_t pw, int64_t T) {
  if (N < 0 || Ci < 1 || Co < 1 || H < 0 || W < 0 || T < 0 || kh < 1 || kw < 1 || ph < 0 || pw < 0 || (T & 3)) return 0;
  const int64_t Ho = H + 2 * ph - kh + 1, Wo = W + 2 * pw - kw + 1;
  if (Ho < 1 || Wo < 1 || N * Ho >= (1LL << 31) || Co * Ci * kh * kw >= (1LL << 31)) return 0;
  if (((Co + kTile - 1) / kTile) * ((Ci * kh * kw + kTile - 1) / kTile) > kMaxThreads) return 0;
  WgradGeom g;
  size_t smem;
  return wgrad_plan(N, Ci, Co, H, W, kh, kw, ph, pw, T, &g, &smem) == SB_OK ? 1 : 0;
}

extern "C" int sb_conv_wgrad(const float* x, const float* grad_y, float* grad_weight, void* scratch, int64_t N,
                             int64_t Ci, int64_t Co, int64_t H, int64_t W, int64_t kh, int64_t kw, int64_t ph,
                             int64_t pw, int64_t T, void* stream) {
  SB_REQUIRE(N >= 0 && Ci >= 1 && Co >= 1 && H >= 0 && W >= 0 && T >= 0, "bad geometry");
  SB_REQUIRE(kh >= 1 && kw >= 1 && ph >= 0 && pw >= 0, "bad kernel geometry");
  SB_REQUIRE(grad_weight != nullptr, "null weight gradient");
  cudaStream_t st = (cudaStream_t)stream;
  const int64_t nout = Co * Ci * kh * kw;
  const int64_t Ho = H + 2 * ph - kh + 1, Wo = W + 2 * pw - kw + 1;
  if (N == 0 || T == 0 || Ho <= 0 || Wo <= 0) {
    SB_CUDA(cudaMemsetAsync(grad_weight, 0, sizeof(float) * nout, st));
    return SB_OK;
  }
  SB_REQUIRE(x && grad_y && scratch, "null tensor pointer");
  SB_REQUIRE((T & 3) == 0 && ((((uintptr_t)x) | ((uintptr_t)grad_y)) & 15u) == 0,
             "the weight-gradient kernel needs T %% 4 == 0 and 16-byte aligned tensors");
  SB_REQUIRE(N * Ho < (1LL << 31) && nout < (1LL << 31), "geometry too large");
  WgradGeom g;
  size_t smem;
  SB_TRY(wgrad_plan(N, Ci, Co, H, W, kh, kw, ph, pw, T, &g, &smem));
  if (smem > 48 * 1024)
    SB_CUDA(cudaFuncSetAttribute((const void*)conv_wgrad_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 200 * 1024));
  const int threads = ((g.owners * g.wgroups + 31) / 32) * 32;
  conv_wgrad_kernel<<<(unsigned)(N * Ho), threads, smem, st>>>(x, grad_y, (float*)scratch, g);
  SB_CUDA(cudaGetLastError());
  conv_wgrad_fold_kernel<<<(unsigned)((nout + 31) / 32), dim3(32, 8), 0, st>>>((const float*)scratch, grad_weight,
                                                                                (int)(N * Ho), (int)nout);
  SB_CUDA(cudaGetLastError());
  return SB_OK;
}
