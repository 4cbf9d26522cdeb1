// Element-wise pieces of the hot path: the spike functions with their
// surrogate gradients (spike/spike.py, spike/complex.py) and the time shift
// (utils/time/shift.py).  No recurrence, so no transposition: threads walk the
// contiguous time axis directly.
#include "api_util.cuh"

using namespace sb;

namespace {

constexpr int kThreads = 256;

inline unsigned grid_for(int64_t items, int per_block) {
  int64_t b = (items + per_block - 1) / per_block;
  const int64_t cap = (int64_t)sm_count() * 16;
  if (b > cap) b = cap;
  if (b < 1) b = 1;
  return (unsigned)b;
}

inline bool aligned16(const void* p) { return (((uintptr_t)p) & 15u) == 0; }

// ---------------------------------------------------------------------------
// Spike forward: spike/spike.py:86-88
// ---------------------------------------------------------------------------
template <bool TT, bool GRADED>
__device__ __forceinline__ float spike_one(float v, float th, float scale) {
  const bool s = v >= th;
  if (GRADED) return __fdiv_rn(__fmul_rn(s ? 1.f : 0.f, v), scale);
  return s ? 1.f : 0.f;
}

template <bool TT, bool GRADED, bool VEC>
__global__ void spike_fwd_kernel(const float* __restrict__ v, const float* __restrict__ tht, float thr,
                                 float* __restrict__ out, int64_t n, float scale) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (VEC) {
    const int64_t n4 = n >> 2;
    for (; i < n4; i += stride) {
      const float4 a = __ldg(reinterpret_cast<const float4*>(v) + i);
      float4 t = make_float4(thr, thr, thr, thr);
      if (TT) t = __ldg(reinterpret_cast<const float4*>(tht) + i);
      float4 o;
      o.x = spike_one<TT, GRADED>(a.x, t.x, scale);
      o.y = spike_one<TT, GRADED>(a.y, t.y, scale);
      o.z = spike_one<TT, GRADED>(a.z, t.z, scale);
      o.w = spike_one<TT, GRADED>(a.w, t.w, scale);
      reinterpret_cast<float4*>(out)[i] = o;
    }
    i = (n4 << 2) + (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  }
  for (; i < n; i += stride) out[i] = spike_one<TT, GRADED>(__ldg(v + i), TT ? __ldg(tht + i) : thr, scale);
}

// Spike backward: spike/spike.py:10-23,112-126
template <bool TT, bool GRADED, bool VEC>
__global__ void spike_bwd_kernel(const float* __restrict__ v, const float* __restrict__ tht, float thr,
                                 const float* __restrict__ gs, float* __restrict__ gv, int64_t n, Surrogate sg) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (VEC) {
    const int64_t n4 = n >> 2;
    for (; i < n4; i += stride) {
      const float4 a = __ldg(reinterpret_cast<const float4*>(v) + i);
      const float4 g = __ldg(reinterpret_cast<const float4*>(gs) + i);
      float4 t = make_float4(thr, thr, thr, thr);
      if (TT) t = __ldg(reinterpret_cast<const float4*>(tht) + i);
      float4 o;
      o.x = __fmul_rn(surrogate<GRADED>(sg, a.x, t.x), g.x);
      o.y = __fmul_rn(surrogate<GRADED>(sg, a.y, t.y), g.y);
      o.z = __fmul_rn(surrogate<GRADED>(sg, a.z, t.z), g.z);
      o.w = __fmul_rn(surrogate<GRADED>(sg, a.w, t.w), g.w);
      reinterpret_cast<float4*>(gv)[i] = o;
    }
    i = (n4 << 2) + (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  }
  for (; i < n; i += stride)
    gv[i] = __fmul_rn(surrogate<GRADED>(sg, __ldg(v + i), TT ? __ldg(tht + i) : thr), __ldg(gs + i));
}

// ---------------------------------------------------------------------------
// Complex spike forward: spike/complex.py:66-92.  Needs im[t-1] (imag_last at
// t = 0), so threads are mapped (row, t) without any division: blockIdx.y
// strides over rows, a block covers 4 * blockDim.x consecutive steps.
// ---------------------------------------------------------------------------
template <bool TT, bool GRADED>
__global__ void cspike_fwd_kernel(const float* __restrict__ re, const float* __restrict__ im,
                                  const float* __restrict__ tht, float thr, const float* __restrict__ imag_last,
                                  float* __restrict__ out, int64_t rows, int T, float scale) {
  for (int64_t row = blockIdx.y; row < rows; row += gridDim.y) {
    const int64_t base = row * (int64_t)T;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int t = (blockIdx.x * 4 + k) * blockDim.x + threadIdx.x;
      if (t >= T) break;
      const float r = __ldg(re + base + t);
      const float m = __ldg(im + base + t);
      const float mp = (t == 0) ? __ldg(imag_last + row) : __ldg(im + base + t - 1);
      const float th = TT ? __ldg(tht + base + t) : thr;
      const bool s = (r >= th) && (mp < 0.f) && (m >= 0.f);
      out[base + t] = GRADED ? __fdiv_rn(__fmul_rn(s ? 1.f : 0.f, r), scale) : (s ? 1.f : 0.f);
    }
  }
}

// The same on 128-bit words (T % 4 == 0, aligned tensors): a thread owns four consecutive steps of
// one row and needs one extra value, the imaginary part just before its word.
template <bool TT, bool GRADED>
__global__ void cspike_fwd_vec_kernel(const float* __restrict__ re, const float* __restrict__ im,
                                      const float* __restrict__ tht, float thr, const float* __restrict__ imag_last,
                                      float* __restrict__ out, int64_t rows, int T, float scale) {
  const int T4 = T >> 2;
  for (int64_t row = blockIdx.y; row < rows; row += gridDim.y) {
    const int64_t base = row * (int64_t)T;
    for (int q = blockIdx.x * blockDim.x + threadIdx.x; q < T4; q += gridDim.x * blockDim.x) {
      const float4 r = __ldg(reinterpret_cast<const float4*>(re + base) + q);
      const float4 m = __ldg(reinterpret_cast<const float4*>(im + base) + q);
      const float mp = (q == 0) ? __ldg(imag_last + row) : __ldg(im + base + 4 * q - 1);
      float4 th = make_float4(thr, thr, thr, thr);
      if (TT) th = __ldg(reinterpret_cast<const float4*>(tht + base) + q);
      const bool s0 = (r.x >= th.x) && (mp < 0.f) && (m.x >= 0.f);
      const bool s1 = (r.y >= th.y) && (m.x < 0.f) && (m.y >= 0.f);
      const bool s2 = (r.z >= th.z) && (m.y < 0.f) && (m.z >= 0.f);
      const bool s3 = (r.w >= th.w) && (m.z < 0.f) && (m.w >= 0.f);
      float4 o;
      o.x = GRADED ? __fdiv_rn(__fmul_rn(s0 ? 1.f : 0.f, r.x), scale) : (s0 ? 1.f : 0.f);
      o.y = GRADED ? __fdiv_rn(__fmul_rn(s1 ? 1.f : 0.f, r.y), scale) : (s1 ? 1.f : 0.f);
      o.z = GRADED ? __fdiv_rn(__fmul_rn(s2 ? 1.f : 0.f, r.z), scale) : (s2 ? 1.f : 0.f);
      o.w = GRADED ? __fdiv_rn(__fmul_rn(s3 ? 1.f : 0.f, r.w), scale) : (s3 ? 1.f : 0.f);
      reinterpret_cast<float4*>(out + base)[q] = o;
    }
  }
}

// Complex spike backward: spike/complex.py:144-167 (element-wise)
template <bool TT, bool GRADED>
__global__ void cspike_bwd_kernel(const float* __restrict__ re, const float* __restrict__ im,
                                  const float* __restrict__ tht, float thr, const float* __restrict__ gs,
                                  float* __restrict__ gre, float* __restrict__ gim, int64_t n, CSurrogate sg) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    float dre, dim;
    csurrogate<GRADED>(sg, __ldg(re + i), __ldg(im + i), TT ? __ldg(tht + i) : thr, dre, dim);
    const float g = __ldg(gs + i);
    gre[i] = __fmul_rn(g, dre);
    gim[i] = __fmul_rn(g, dim);
  }
}

// 128-bit form for n % 4 == 0 and 16-byte aligned tensors: three loads and two stores of four values
// per thread and trip (0.85 -> 0.96 of copy bandwidth against one value per thread).
template <bool TT, bool GRADED>
__global__ void cspike_bwd_vec_kernel(const float4* __restrict__ re, const float4* __restrict__ im,
                                      const float4* __restrict__ tht, float thr, const float4* __restrict__ gs,
                                      float4* __restrict__ gre, float4* __restrict__ gim, int64_t n4, CSurrogate sg) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
    const float4 r = __ldg(re + i), m = __ldg(im + i), g = __ldg(gs + i);
    float4 th = make_float4(thr, thr, thr, thr);
    if (TT) th = __ldg(tht + i);
    float4 a, b;
    float dre, dim;
    csurrogate<GRADED>(sg, r.x, m.x, th.x, dre, dim); a.x = __fmul_rn(g.x, dre); b.x = __fmul_rn(g.x, dim);
    csurrogate<GRADED>(sg, r.y, m.y, th.y, dre, dim); a.y = __fmul_rn(g.y, dre); b.y = __fmul_rn(g.y, dim);
    csurrogate<GRADED>(sg, r.z, m.z, th.z, dre, dim); a.z = __fmul_rn(g.z, dre); b.z = __fmul_rn(g.z, dim);
    csurrogate<GRADED>(sg, r.w, m.w, th.w, dre, dim); a.w = __fmul_rn(g.w, dre); b.w = __fmul_rn(g.w, dim);
    gre[i] = a;
    gim[i] = b;
  }
}

// ---------------------------------------------------------------------------
// Shift: a delay gather, one launch for all batches (shift.cu:130-154 launches
// once per batch element).  out[r, t] = in[r, t - d(r)] or 0.
// ---------------------------------------------------------------------------
__global__ void shift_kernel(const float* __restrict__ x, const float* __restrict__ lut, int64_t n_lut, float shift,
                             float ts, float* __restrict__ out, int64_t rows, int T) {
  for (int64_t row = blockIdx.y; row < rows; row += gridDim.y) {
    const float sv = lut ? __ldg(lut + (row % n_lut)) : shift;
    const int d = __float2int_rz(__fdiv_rn(sv, ts));
    const int64_t base = row * (int64_t)T;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int t = (blockIdx.x * 4 + k) * blockDim.x + threadIdx.x;
      if (t >= T) break;
      const int s = t - d;
      out[base + t] = (s >= 0 && s < T) ? __ldg(x + base + s) : 0.f;
    }
  }
}

// Vector form for T % 4 == 0 and 16-byte aligned tensors: a thread writes two
// aligned float4; the source window starts (t - d), in general not aligned, so
// it is assembled from the aligned float4 words that cover it (neighbouring
// threads read overlapping words: L1 serves the second touch).
constexpr int kShiftVecPerThread = 2;

__device__ __forceinline__ float4 ld4_or_zero(const float4* p, int q, int nq) {
  return (q >= 0 && q < nq) ? __ldg(p + q) : make_float4(0.f, 0.f, 0.f, 0.f);
}

__global__ void __launch_bounds__(128)
shift_vec_kernel(const float* __restrict__ x, const float* __restrict__ lut, int64_t n_lut, float shift, float ts,
                 float* __restrict__ out, int64_t rows, int T) {
  const int nq = T >> 2;  // float4 words per row
  for (int64_t row = blockIdx.y; row < rows; row += gridDim.y) {
    const float sv = lut ? __ldg(lut + (row % n_lut)) : shift;
    int d = __float2int_rz(__fdiv_rn(sv, ts));
    d = max(-T - 8, min(T + 8, d));  // beyond +-T everything is zero anyway; keeps the arithmetic below in range
    const float4* src = reinterpret_cast<const float4*>(x + row * (int64_t)T);
    float4* dst = reinterpret_cast<float4*>(out + row * (int64_t)T);
    // source element index of output element 4*q is 4*q - d = 4*(q - dq) + r, 0 <= r < 4
    const int dq = (d + 3) >> 2;             // ceil(d / 4) for either sign (arithmetic shift floors)
    const int r = (dq << 2) - d;             // 0..3
#pragma unroll
    for (int k = 0; k < kShiftVecPerThread; ++k) {
      const int q = (blockIdx.x * kShiftVecPerThread + k) * blockDim.x + threadIdx.x;
      if (q >= nq) break;
      const int s0 = q - dq;
      const float4 a = ld4_or_zero(src, s0, nq);
      float4 o = a;
      if (r != 0) {
        const float4 b = ld4_or_zero(src, s0 + 1, nq);
        if (r == 1) o = make_float4(a.y, a.z, a.w, b.x);
        else if (r == 2) o = make_float4(a.z, a.w, b.x, b.y);
        else o = make_float4(a.w, b.x, b.y, b.z);
      }
      dst[q] = o;
    }
  }
}

Surrogate surrogate_consts(float tau_rho, float scale_rho, bool graded) {
  Surrogate s;
  s.k2 = (float)(1.4426950408889634 / (double)tau_rho);
  volatile float half = scale_rho / 2.0f;
  volatile float c = half / tau_rho;
  s.c0 = graded ? scale_rho : c;
  return s;
}

CSurrogate csurrogate_consts(float tau_rho, float scale_rho) {
  CSurrogate s;
  s.k2 = (float)(1.4426950408889634 / (double)tau_rho);
  s.scale_rho = scale_rho;
  volatile float a = 0.5f / tau_rho;
  volatile float b = 2.0f * tau_rho;
  volatile float c = (-scale_rho) / tau_rho;
  s.half_over_tau = a;
  s.two_tau = b;
  s.neg_scale_over_tau = c;
  return s;
}

inline dim3 row_grid(int64_t rows, int64_t T, int threads) {
  unsigned gx = (unsigned)((T + 4 * threads - 1) / (4 * threads));
  unsigned gy = (unsigned)(rows < 65535 ? rows : 65535);
  return dim3(gx ? gx : 1, gy ? gy : 1, 1);
}

}  // namespace

extern "C" {

int sb_spike_fwd(const float* v, const float* thr_tensor, float thr, float* spike, int64_t n, int graded,
                 float scale, void* stream) {
  SB_REQUIRE(n >= 0, "negative element count");
  if (n == 0) return SB_OK;
  SB_REQUIRE(v && spike, "null tensor pointer");
  cudaStream_t st = (cudaStream_t)stream;
  const bool vec = aligned16(v) && aligned16(spike) && (!thr_tensor || aligned16(thr_tensor));
  const unsigned grid = grid_for(vec ? (n + 3) / 4 : n, kThreads);
#define SB_GO(TT, G)                                                                                          \
  {                                                                                                           \
    if (vec) spike_fwd_kernel<TT, G, true><<<grid, kThreads, 0, st>>>(v, thr_tensor, thr, spike, n, scale);   \
    else spike_fwd_kernel<TT, G, false><<<grid, kThreads, 0, st>>>(v, thr_tensor, thr, spike, n, scale);      \
  }
  if (thr_tensor) { if (graded) SB_GO(true, true) else SB_GO(true, false) }
  else            { if (graded) SB_GO(false, true) else SB_GO(false, false) }
#undef SB_GO
  SB_CUDA(cudaGetLastError());
  return SB_OK;
}

int sb_spike_bwd(const float* v, const float* thr_tensor, float thr, const float* grad_spike, float* grad_v,
                 int64_t n, float tau_rho, float scale_rho, int graded, void* stream) {
  SB_REQUIRE(n >= 0, "negative element count");
  if (n == 0) return SB_OK;
  SB_REQUIRE(v && grad_spike && grad_v, "null tensor pointer");
  cudaStream_t st = (cudaStream_t)stream;
  const Surrogate sg = surrogate_consts(tau_rho, scale_rho, graded != 0);
  const bool vec = aligned16(v) && aligned16(grad_spike) && aligned16(grad_v) && (!thr_tensor || aligned16(thr_tensor));
  const unsigned grid = grid_for(vec ? (n + 3) / 4 : n, kThreads);
#define SB_GO(TT, G)                                                                                               \
  {                                                                                                                \
    if (vec) spike_bwd_kernel<TT, G, true><<<grid, kThreads, 0, st>>>(v, thr_tensor, thr, grad_spike, grad_v, n, sg); \
    else spike_bwd_kernel<TT, G, false><<<grid, kThreads, 0, st>>>(v, thr_tensor, thr, grad_spike, grad_v, n, sg); \
  }
  if (thr_tensor) { if (graded) SB_GO(true, true) else SB_GO(true, false) }
  else            { if (graded) SB_GO(false, true) else SB_GO(false, false) }
#undef SB_GO
  SB_CUDA(cudaGetLastError());
  return SB_OK;
}

int sb_cspike_fwd(const float* re, const float* im, const float* thr_tensor, float thr, const float* imag_last,
                  float* spike, int64_t rows, int64_t T, int graded, float scale, void* stream) {
  SB_REQUIRE(rows >= 0 && T >= 0 && T <= 2147483647LL, "bad geometry");
  if (rows == 0 || T == 0) return SB_OK;
  SB_REQUIRE(re && im && imag_last && spike, "null tensor pointer");
  cudaStream_t st = (cudaStream_t)stream;
  const dim3 grid = row_grid(rows, T, kThreads);
  const bool vec = (T & 3) == 0 && ((((uintptr_t)re) | ((uintptr_t)im) | ((uintptr_t)spike) | ((uintptr_t)thr_tensor)) & 15u) == 0;
  const dim3 vgrid((unsigned)((T / 4 + kThreads - 1) / kThreads > 0 ? (T / 4 + kThreads - 1) / kThreads : 1), grid.y);
#define SB_GO(TT, G)                                                                                                   \
  if (vec)                                                                                                             \
    cspike_fwd_vec_kernel<TT, G><<<vgrid, kThreads, 0, st>>>(re, im, thr_tensor, thr, imag_last, spike, rows, (int)T, scale); \
  else                                                                                                                 \
    cspike_fwd_kernel<TT, G><<<grid, kThreads, 0, st>>>(re, im, thr_tensor, thr, imag_last, spike, rows, (int)T, scale);
  if (thr_tensor) { if (graded) SB_GO(true, true) else SB_GO(true, false) }
  else            { if (graded) SB_GO(false, true) else SB_GO(false, false) }
#undef SB_GO
  SB_CUDA(cudaGetLastError());
  return SB_OK;
}

int sb_cspike_bwd(const float* re, const float* im, const float* thr_tensor, float thr, const float* grad_spike,
                  float* grad_re, float* grad_im, int64_t n, float tau_rho, float scale_rho, int graded,
                  void* stream) {
  SB_REQUIRE(n >= 0, "negative element count");
  if (n == 0) return SB_OK;
  SB_REQUIRE(re && im && grad_spike && grad_re && grad_im, "null tensor pointer");
  cudaStream_t st = (cudaStream_t)stream;
  const CSurrogate sg = csurrogate_consts(tau_rho, scale_rho);
  const unsigned grid = grid_for(n, kThreads);
  const bool vec = (n & 3) == 0 && ((((uintptr_t)re) | ((uintptr_t)im) | ((uintptr_t)thr_tensor) | ((uintptr_t)grad_spike) |
                                     ((uintptr_t)grad_re) | ((uintptr_t)grad_im)) & 15u) == 0;
  const unsigned vgrid = grid_for(n / 4 > 0 ? n / 4 : 1, kThreads);
#define SB_GO(TT, G)                                                                                                  \
  if (vec)                                                                                                            \
    cspike_bwd_vec_kernel<TT, G><<<vgrid, kThreads, 0, st>>>(                                                          \
        reinterpret_cast<const float4*>(re), reinterpret_cast<const float4*>(im),                                     \
        reinterpret_cast<const float4*>(thr_tensor), thr, reinterpret_cast<const float4*>(grad_spike),                \
        reinterpret_cast<float4*>(grad_re), reinterpret_cast<float4*>(grad_im), n / 4, sg);                           \
  else                                                                                                                \
    cspike_bwd_kernel<TT, G><<<grid, kThreads, 0, st>>>(re, im, thr_tensor, thr, grad_spike, grad_re, grad_im, n, sg);
  if (thr_tensor) { if (graded) SB_GO(true, true) else SB_GO(true, false) }
  else            { if (graded) SB_GO(false, true) else SB_GO(false, false) }
#undef SB_GO
  SB_CUDA(cudaGetLastError());
  return SB_OK;
}

int sb_shift(const float* x, const float* lut, int64_t n_lut, float shift, float sampling_time, float* out,
             int64_t rows, int64_t T, void* stream) {
  SB_REQUIRE(rows >= 0 && T >= 0 && T <= 2147483647LL, "bad geometry");
  if (rows == 0 || T == 0) return SB_OK;
  SB_REQUIRE(x && out, "null tensor pointer");
  SB_REQUIRE(x != out, "shift cannot run in place");
  SB_REQUIRE(sampling_time != 0.f, "sampling_time must be non-zero");
  if (lut) SB_REQUIRE(n_lut > 0 && rows % n_lut == 0, "lut of %lld entries does not tile %lld rows", (long long)n_lut,
                      (long long)rows);
  cudaStream_t st = (cudaStream_t)stream;
  const int threads = 128;
  if ((T & 3) == 0 && aligned16(x) && aligned16(out)) {
    const int per_block = threads * kShiftVecPerThread;
    const unsigned gx = (unsigned)(((T >> 2) + per_block - 1) / per_block);
    const unsigned gy = (unsigned)(rows < 65535 ? rows : 65535);
    shift_vec_kernel<<<dim3(gx, gy), threads, 0, st>>>(x, lut, n_lut, shift, sampling_time, out, rows, (int)T);
    SB_CUDA(cudaGetLastError());
    return SB_OK;
  }
  shift_kernel<<<row_grid(rows, T, threads), threads, 0, st>>>(x, lut, n_lut, shift, sampling_time, out, rows, (int)T);
  SB_CUDA(cudaGetLastError());
  return SB_OK;
}

}  // extern "C"

// ---------------------------------------------------------------------------
// out[i] = *value for i < n, value read on the device: materialises a gradient
// that autograd hands over as one broadcast number (the backward of sum() or
// mean()) at memory speed and without a host round trip.
// ---------------------------------------------------------------------------
namespace {
__global__ void broadcast_fill_kernel(const float* __restrict__ value, float* __restrict__ out, int64_t n) {
  const float v = __ldg(value);
  const int64_t n4 = n >> 2;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  const bool aligned = (((uintptr_t)out) & 15u) == 0;
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (aligned) {
    const float4 v4 = make_float4(v, v, v, v);
    for (int64_t k = i; k < n4; k += stride) reinterpret_cast<float4*>(out)[k] = v4;
    for (int64_t k = (n4 << 2) + i; k < n; k += stride) out[k] = v;
  } else {
    for (int64_t k = i; k < n; k += stride) out[k] = v;
  }
}
}  // namespace

extern "C" int sb_broadcast_fill(const float* value, float* out, int64_t n, void* stream) {
  SB_REQUIRE(n >= 0, "negative element count");
  if (n == 0) return SB_OK;
  SB_REQUIRE(value && out, "null pointer");
  broadcast_fill_kernel<<<(unsigned)sb::sm_count() * 8, 512, 0, (cudaStream_t)stream>>>(value, out, n);
  SB_CUDA(cudaGetLastError());
  return SB_OK;
}
