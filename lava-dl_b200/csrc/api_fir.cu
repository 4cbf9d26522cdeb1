// Causal temporal filter (utils/filter/conv.py:48-97) as a shared-memory
// sliding-window kernel, optionally fused with the per-neuron delay
// (utils/time/shift.py) on its input (forward) or output (adjoint) side.
//
// One formulation covers conv, corr and both fused forms:
//     z[u]   = Ts * sum_m h[m] * S(u + m - off)            u in [0, T)
//     S(v)   = x[v - d_in]  if 0 <= v < T and 0 <= v - d_in < T else 0
//     out[t] = z[t + d_out] if 0 <= t + d_out < T else 0
//   conv : h = reversed filter, off = K - 1, d_in = d_out = 0
//   corr : h = filter,          off = 0
//   conv(shift(x, d)) : d_in = d;   shift(corr(g), -d) : d_out = d
//
// A block owns one row segment of 1024 outputs: it stages the
// 1024 + K window in shared memory once (every input element is read from HBM
// once), then each thread produces 16 consecutive outputs from registers, 16
// taps at a time (a 32-word window per tap group, read as 128-bit words).
// Shared memory is skewed by 4 words every 16 so that those 128-bit reads,
// 64 bytes apart between neighbouring threads, are bank-conflict free.
// At 64 taps the kernel does 64 FMAs per 8 bytes of HBM traffic, which puts it
// at the FP32 issue limit rather than the HBM limit.  K is capped at 4096 so the
// window always fits the default 48 KB of dynamic shared memory.
#include "api_util.cuh"

using namespace sb;

namespace sb {
// api_fir_tc.cu: tensor-core path for K <= 64, T % 4 == 0, rows >= 128.
int fir_tc_try(const float* x, const float* filt, int64_t K, bool corr, const float* lut, int64_t n_lut, float shift,
               float shift_ts, int mode, float ts, float* out, int64_t rows, int64_t T, cudaStream_t st,
               bool* taken);
}

namespace {

constexpr int kOutPerThread = 16;
constexpr int kFirThreads = 64;
constexpr int kSeg = kOutPerThread * kFirThreads;  // outputs per block
constexpr int kTapGroup = 16;
constexpr int kFillBatch = 9;  // 17 window words per thread at 64 taps: two batches

// 4 pad words after every 16: thread j's 16-output window then starts at word
// 20 * j, so the eight threads of a 128-bit access phase hit distinct banks, and
// offsets relative to that start are the same for every thread.
__host__ __device__ constexpr int skew(int i) { return i + ((i >> 4) << 2); }

template <bool SHIFT_IN, bool SHIFT_OUT>
__global__ void __launch_bounds__(kFirThreads)
fir_kernel(const float* __restrict__ x, const float* __restrict__ filt, int K, int Kp, bool reverse_taps, int off,
           const float* __restrict__ lut, int64_t n_lut, float shift, float shift_ts, float ts,
           float* __restrict__ out, int64_t rows, int T) {
  extern __shared__ float sm[];
  float* h = sm;         // Kp taps (zero padded)
  float* win = sm + Kp;  // skewed window of kSeg + Kp words
  const int nwin = kSeg + Kp;
  const int tid = threadIdx.x;

  for (int i = tid; i < Kp; i += kFirThreads) {
    float v = 0.f;
    if (i < K) v = __ldg(filt + (reverse_taps ? (K - 1 - i) : i));
    h[i] = v;
  }
  const int c0 = tid * kOutPerThread;
  const float* wthread = win + skew(c0);
  const int t0 = blockIdx.x * kSeg;

  for (int64_t row = blockIdx.y; row < rows; row += gridDim.y) {
    int d = 0;
    if (SHIFT_IN || SHIFT_OUT) {
      const float sv = lut ? __ldg(lut + (row % n_lut)) : shift;
      d = __float2int_rz(__fdiv_rn(sv, shift_ts));
      d = max(-T - 8, min(T + 8, d));
    }
    const int d_in = SHIFT_IN ? d : 0;
    const int d_out = SHIFT_OUT ? d : 0;
    const int v0 = t0 + d_out - off;  // S index of window word 0
    // window word i holds x[v0 + i - d_in] when both v0 + i and v0 + i - d_in lie in [0, T)
    const int lo = max(0, max(-v0, d_in - v0));
    const int hi = min(nwin, min(T - v0, T + d_in - v0));
    const float* src = x + row * (int64_t)T + (v0 - d_in);

    __syncthreads();  // previous row's window fully consumed (and taps visible)
    // kFillBatch independent loads in flight per thread before the first store
    for (int i0 = tid; i0 < nwin; i0 += kFillBatch * kFirThreads) {
      float val[kFillBatch];
#pragma unroll
      for (int k = 0; k < kFillBatch; ++k) {
        const int i = i0 + k * kFirThreads;
        val[k] = (i >= lo && i < hi) ? __ldg(src + i) : 0.f;
      }
#pragma unroll
      for (int k = 0; k < kFillBatch; ++k) {
        const int i = i0 + k * kFirThreads;
        if (i < nwin) win[skew(i)] = val[k];
      }
    }
    __syncthreads();

    float acc[kOutPerThread];
#pragma unroll
    for (int c = 0; c < kOutPerThread; ++c) acc[c] = 0.f;

    const float* wp = wthread;
    for (int m0 = 0; m0 < Kp; m0 += kTapGroup, wp += skew(kTapGroup)) {
      float hv[kTapGroup];
#pragma unroll
      for (int q = 0; q < kTapGroup / 4; ++q) {
        const float4 f4 = *reinterpret_cast<const float4*>(h + m0 + 4 * q);
        hv[4 * q] = f4.x; hv[4 * q + 1] = f4.y; hv[4 * q + 2] = f4.z; hv[4 * q + 3] = f4.w;
      }
      float xv[kOutPerThread + kTapGroup];
#pragma unroll
      for (int q = 0; q < (kOutPerThread + kTapGroup) / 4; ++q) {
        const float4 x4 = *reinterpret_cast<const float4*>(wp + skew(4 * q));
        xv[4 * q] = x4.x; xv[4 * q + 1] = x4.y; xv[4 * q + 2] = x4.z; xv[4 * q + 3] = x4.w;
      }
#pragma unroll
      for (int m = 0; m < kTapGroup; ++m) {
#pragma unroll
        for (int c = 0; c < kOutPerThread; ++c) acc[c] = fmaf(hv[m], xv[c + m], acc[c]);
      }
    }

    const int t = t0 + c0;
    if (t >= T) continue;
    float* dst = out + row * (int64_t)T + t;
#pragma unroll
    for (int c = 0; c < kOutPerThread; ++c) {
      acc[c] = __fmul_rn(acc[c], ts);
      if (SHIFT_OUT) {
        const int u = t + c + d_out;
        if (u < 0 || u >= T) acc[c] = 0.f;
      }
    }
    if (((((uintptr_t)dst) & 15u) == 0) && (t + kOutPerThread <= T)) {
#pragma unroll
      for (int q = 0; q < kOutPerThread / 4; ++q)
        reinterpret_cast<float4*>(dst)[q] = make_float4(acc[4 * q], acc[4 * q + 1], acc[4 * q + 2], acc[4 * q + 3]);
    } else {
#pragma unroll
      for (int c = 0; c < kOutPerThread; ++c)
        if (t + c < T) dst[c] = acc[c];
    }
  }
}

// ---------------------------------------------------------------------------
// Two rows per block with packed FP32 math.  The window holds float2 entries
// (row a, row b) side by side, the taps are stored duplicated (h, h), and every
// multiply-add is one fma.rn.f32x2 on (acc_a, acc_b): half the FMA issue slots
// for the same arithmetic, which is what this kernel is short of.  Results are
// bit-identical to the one-row kernel (same operation order per lane).
// ---------------------------------------------------------------------------
__host__ __device__ constexpr int skew2(int i) { return 2 * i + ((i >> 4) << 2); }  // in words

template <bool SHIFT_IN, bool SHIFT_OUT>
__global__ void __launch_bounds__(kFirThreads)
fir2_kernel(const float* __restrict__ x, const float* __restrict__ filt, int K, int Kp, bool reverse_taps, int off,
            const float* __restrict__ lut, int64_t n_lut, float shift, float shift_ts, float ts,
            float* __restrict__ out, int64_t rows, int T) {
  extern __shared__ float sm[];
  float* h2 = sm;             // Kp duplicated taps: 2 * Kp words
  float* win = sm + 2 * Kp;   // skewed window of float2 entries
  const int nwin = kSeg + Kp;
  const int tid = threadIdx.x;

  for (int i = tid; i < Kp; i += kFirThreads) {
    float v = 0.f;
    if (i < K) v = __ldg(filt + (reverse_taps ? (K - 1 - i) : i));
    reinterpret_cast<float2*>(h2)[i] = make_float2(v, v);
  }
  const int c0 = tid * kOutPerThread;
  const float* wthread = win + skew2(c0);
  const int t0 = blockIdx.x * kSeg;
  const int64_t npairs = (rows + 1) >> 1;

  for (int64_t pair = blockIdx.y; pair < npairs; pair += gridDim.y) {
    const int64_t row_a = pair * 2, row_b = row_a + 1;
    const bool has_b = row_b < rows;
    int d_a = 0, d_b = 0;
    if (SHIFT_IN || SHIFT_OUT) {
      const float sa = lut ? __ldg(lut + (row_a % n_lut)) : shift;
      const float sb = lut ? __ldg(lut + ((has_b ? row_b : row_a) % n_lut)) : shift;
      d_a = max(-T - 8, min(T + 8, __float2int_rz(__fdiv_rn(sa, shift_ts))));
      d_b = max(-T - 8, min(T + 8, __float2int_rz(__fdiv_rn(sb, shift_ts))));
    }
    const int din_a = SHIFT_IN ? d_a : 0, din_b = SHIFT_IN ? d_b : 0;
    const int dout_a = SHIFT_OUT ? d_a : 0, dout_b = SHIFT_OUT ? d_b : 0;
    const int v0a = t0 + dout_a - off, v0b = t0 + dout_b - off;
    const int lo_a = max(0, max(-v0a, din_a - v0a)), hi_a = min(nwin, min(T - v0a, T + din_a - v0a));
    const int lo_b = max(0, max(-v0b, din_b - v0b));
    const int hi_b = has_b ? min(nwin, min(T - v0b, T + din_b - v0b)) : 0;
    const float* src_a = x + row_a * (int64_t)T + (v0a - din_a);
    const float* src_b = x + row_b * (int64_t)T + (v0b - din_b);

    __syncthreads();
    for (int i0 = tid; i0 < nwin; i0 += kFillBatch * kFirThreads) {
      float va[kFillBatch], vb[kFillBatch];
#pragma unroll
      for (int k = 0; k < kFillBatch; ++k) {
        const int i = i0 + k * kFirThreads;
        va[k] = (i >= lo_a && i < hi_a) ? __ldg(src_a + i) : 0.f;
        vb[k] = (i >= lo_b && i < hi_b) ? __ldg(src_b + i) : 0.f;
      }
#pragma unroll
      for (int k = 0; k < kFillBatch; ++k) {
        const int i = i0 + k * kFirThreads;
        if (i < nwin) *reinterpret_cast<float2*>(win + skew2(i)) = make_float2(va[k], vb[k]);
      }
    }
    __syncthreads();

    float2 acc[kOutPerThread];
#pragma unroll
    for (int c = 0; c < kOutPerThread; ++c) acc[c] = make_float2(0.f, 0.f);

    const float* wp = wthread;
    for (int m0 = 0; m0 < Kp; m0 += kTapGroup, wp += skew2(kTapGroup)) {
      float2 hv[kTapGroup];
#pragma unroll
      for (int q = 0; q < kTapGroup / 2; ++q) {
        const float4 f4 = *reinterpret_cast<const float4*>(h2 + 2 * m0 + 4 * q);
        hv[2 * q] = make_float2(f4.x, f4.y);
        hv[2 * q + 1] = make_float2(f4.z, f4.w);
      }
      float2 xv[kOutPerThread + kTapGroup];
#pragma unroll
      for (int q = 0; q < (kOutPerThread + kTapGroup) / 2; ++q) {
        const float4 x4 = *reinterpret_cast<const float4*>(wp + skew2(2 * q));
        xv[2 * q] = make_float2(x4.x, x4.y);
        xv[2 * q + 1] = make_float2(x4.z, x4.w);
      }
#pragma unroll
      for (int m = 0; m < kTapGroup; ++m) {
#pragma unroll
        for (int c = 0; c < kOutPerThread; ++c) acc[c] = __ffma2_rn(hv[m], xv[c + m], acc[c]);
      }
    }

    const int t = t0 + c0;
    if (t >= T) continue;
    float ra[kOutPerThread], rb[kOutPerThread];
#pragma unroll
    for (int c = 0; c < kOutPerThread; ++c) {
      ra[c] = __fmul_rn(acc[c].x, ts);
      rb[c] = __fmul_rn(acc[c].y, ts);
      if (SHIFT_OUT) {
        const int ua = t + c + dout_a, ub = t + c + dout_b;
        if (ua < 0 || ua >= T) ra[c] = 0.f;
        if (ub < 0 || ub >= T) rb[c] = 0.f;
      }
    }
    float* dst_a = out + row_a * (int64_t)T + t;
    float* dst_b = out + row_b * (int64_t)T + t;
    const bool full = t + kOutPerThread <= T;
    if (full && ((((uintptr_t)dst_a) & 15u) == 0)) {
#pragma unroll
      for (int q = 0; q < kOutPerThread / 4; ++q)
        reinterpret_cast<float4*>(dst_a)[q] = make_float4(ra[4 * q], ra[4 * q + 1], ra[4 * q + 2], ra[4 * q + 3]);
    } else {
#pragma unroll
      for (int c = 0; c < kOutPerThread; ++c)
        if (t + c < T) dst_a[c] = ra[c];
    }
    if (has_b) {
      if (full && ((((uintptr_t)dst_b) & 15u) == 0)) {
#pragma unroll
        for (int q = 0; q < kOutPerThread / 4; ++q)
          reinterpret_cast<float4*>(dst_b)[q] = make_float4(rb[4 * q], rb[4 * q + 1], rb[4 * q + 2], rb[4 * q + 3]);
      } else {
#pragma unroll
        for (int c = 0; c < kOutPerThread; ++c)
          if (t + c < T) dst_b[c] = rb[c];
      }
    }
  }
}

int launch_fir(const float* x, const float* filt, int64_t K, bool corr, const float* lut, int64_t n_lut, float shift,
               float shift_ts, bool shift_in, bool shift_out, float ts, float* out, int64_t rows, int64_t T,
               void* stream) {
  SB_REQUIRE(rows >= 0 && T >= 0 && T <= 2147483647LL - 4096, "bad geometry");
  SB_REQUIRE(K >= 1 && K <= 4096, "filter length %lld outside [1, 4096]", (long long)K);
  if (rows == 0 || T == 0) return SB_OK;
  SB_REQUIRE(x && filt && out, "null tensor pointer");
  SB_REQUIRE(x != out, "the filter cannot run in place");
  if (shift_in || shift_out) {
    SB_REQUIRE(shift_ts != 0.f, "shift sampling_time must be non-zero");
    if (lut) SB_REQUIRE(n_lut > 0 && rows % n_lut == 0, "lut of %lld entries does not tile %lld rows",
                        (long long)n_lut, (long long)rows);
  }
  const int Kp = (int)((K + kTapGroup - 1) / kTapGroup) * kTapGroup;
  const int nwin = kSeg + Kp;
  const unsigned gx = (unsigned)((T + kSeg - 1) / kSeg);
  const int off = corr ? 0 : (int)K - 1;
  cudaStream_t st = (cudaStream_t)stream;
  {
    bool taken = false;
    const int rc = fir_tc_try(x, filt, K, corr, lut, n_lut, shift, shift_ts, shift_in ? 1 : (shift_out ? -1 : 0), ts,
                              out, rows, T, st, &taken);
    if (rc != SB_OK || taken) return rc;
  }
  // The packed two-row kernel needs twice the shared memory; filters too long
  // for its 48 KB take the one-row kernel (as does a single row).
  const size_t smem2 = sizeof(float) * (size_t)(2 * Kp + skew2(nwin) + 8);
  if (rows >= 2 && smem2 <= 48 * 1024) {
    const int64_t npairs = (rows + 1) / 2;
    const dim3 grid(gx, (unsigned)(npairs < 65535 ? npairs : 65535));
#define SB_GO(SI, SO)                                                                                            \
  fir2_kernel<SI, SO><<<grid, kFirThreads, smem2, st>>>(x, filt, (int)K, Kp, !corr, off, lut, n_lut, shift, shift_ts, \
                                                         ts, out, rows, (int)T);
    if (shift_in) SB_GO(true, false)
    else if (shift_out) SB_GO(false, true)
    else SB_GO(false, false)
#undef SB_GO
    SB_CUDA(cudaGetLastError());
    return SB_OK;
  }
  const size_t smem = sizeof(float) * (size_t)(Kp + skew(nwin) + 8);
  const dim3 grid(gx, (unsigned)(rows < 65535 ? rows : 65535));
#define SB_GO(SI, SO)                                                                                          \
  fir_kernel<SI, SO><<<grid, kFirThreads, smem, st>>>(x, filt, (int)K, Kp, !corr, off, lut, n_lut, shift, shift_ts, \
                                                       ts, out, rows, (int)T);
  if (shift_in) SB_GO(true, false)
  else if (shift_out) SB_GO(false, true)
  else SB_GO(false, false)
#undef SB_GO
  SB_CUDA(cudaGetLastError());
  return SB_OK;
}

}  // namespace

extern "C" {

int sb_fir_conv(const float* x, const float* filter, int64_t K, float sampling_time, float* out, int64_t rows,
                int64_t T, void* stream) {
  return launch_fir(x, filter, K, false, nullptr, 0, 0.f, 1.f, false, false, sampling_time, out, rows, T, stream);
}

int sb_fir_corr(const float* x, const float* filter, int64_t K, float sampling_time, float* out, int64_t rows,
                int64_t T, void* stream) {
  return launch_fir(x, filter, K, true, nullptr, 0, 0.f, 1.f, false, false, sampling_time, out, rows, T, stream);
}

int sb_shift_fir_fwd(const float* x, const float* lut, int64_t n_lut, float shift, float shift_ts,
                     const float* filter, int64_t K, float sampling_time, float* out, int64_t rows, int64_t T,
                     void* stream) {
  return launch_fir(x, filter, K, false, lut, n_lut, shift, shift_ts, true, false, sampling_time, out, rows, T,
                    stream);
}

int sb_shift_fir_bwd(const float* grad_out, const float* lut, int64_t n_lut, float shift, float shift_ts,
                     const float* filter, int64_t K, float sampling_time, float* grad_x, int64_t rows, int64_t T,
                     void* stream) {
  return launch_fir(grad_out, filter, K, true, lut, n_lut, shift, shift_ts, false, true, sampling_time, grad_x, rows,
                    T, stream);
}

}  // extern "C"
