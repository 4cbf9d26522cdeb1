// Dense recurrent CUBA layer in one launch per direction.
//
// The reference (utils/recurrent.py:45-112, used by block/base.py:1460-1488)
// walks over time in Python: per step one matmul for the feedback
// R s[t-1], one addition and one Neuron.forward() call with T = 1 (about a
// dozen launches), and the same again in reverse for the gradient.  Samples
// of a batch never interact, so here one CTA owns one sample, one thread one
// neuron; the neuron state lives in registers, the spikes of the previous step
// in a compact list in shared memory, and only the spiking columns of R are
// read (R stays L2 resident).  Time tiles of 16 steps move through shared
// memory so that global loads and stores are row segments of 64 bytes.
#pragma once

#include "ops.cuh"

namespace sb {

constexpr int kRecTile = 16;        // steps per shared-memory tile
constexpr int kRecPitch = kRecTile + 1;

// rows [row0, row0 + C) x steps [t0, t0 + kRecTile) between global memory and a [C][kRecPitch] tile
template <bool LOAD>
__device__ __forceinline__ void rec_tile_io(float* tile, float* gmem, const float* gmem_in, int64_t row0, int C,
                                            int T, int t0) {
  const int tt = threadIdx.x % kRecTile;
  const int r0 = threadIdx.x / kRecTile;
  const int rstep = blockDim.x / kRecTile;
  const bool ok = t0 + tt < T;
  for (int r = r0; r < C; r += rstep) {
    const int64_t off = (row0 + r) * (int64_t)T + t0 + tt;
    if (LOAD) tile[r * kRecPitch + tt] = ok ? __ldg(gmem_in + off) : 0.f;
    else if (ok) gmem[off] = tile[r * kRecPitch + tt];
  }
}

// Forward.  z [B, C, T]; rec_t [C, C] = R transposed (row j holds R[:, j]);
// outputs voltage and spike [B, C, T].  Dynamic shared memory:
// 2 tiles [C][kRecPitch] floats, then 2 x C spike indices (ushort), 2 x C spike
// values (float), 2 x 32 warp counts.
template <bool GRADED>
__global__ void __launch_bounds__(1024, 1)
cuba_recurrent_fwd_kernel(typename CubaFwd<false, true, GRADED>::Params p, RowGeom g, const float* __restrict__ z,
                          const float* __restrict__ rec_t, float* __restrict__ voltage, float* __restrict__ spike,
                          int C) {
  extern __shared__ __align__(16) unsigned char rec_smem[];
  float* zt = reinterpret_cast<float*>(rec_smem);           // input tile, overwritten by the spikes
  float* vt = zt + (size_t)C * kRecPitch;                   // voltage tile
  float* sval = vt + (size_t)C * kRecPitch;                 // [2][C]
  int* wcount = reinterpret_cast<int*>(sval + 2 * (size_t)C);  // [2][32]
  int* total = wcount + 64;                                 // [2]
  unsigned short* sidx = reinterpret_cast<unsigned short*>(total + 2);  // [2][C]

  const int i = threadIdx.x, lane = i & 31, warp = i >> 5, nwarp = blockDim.x >> 5;
  const bool valid = i < C;
  const int64_t row0 = (int64_t)blockIdx.x * C;
  const int T = g.T;
  CubaFwd<false, true, GRADED> op;
  op.init(p, g, row0 + (valid ? i : 0), valid);
  if (i < 2) total[i] = 0;
  int cur = 0;
  __syncthreads();

  for (int t0 = 0; t0 < T; t0 += kRecTile) {
    rec_tile_io<true>(zt, nullptr, z, row0, C, T, t0);
    __syncthreads();
    const int nstep = min(kRecTile, T - t0);
    for (int tt = 0; tt < nstep; ++tt) {
      // feedback of the spikes of the previous step, in ascending source order
      float fb = 0.f;
      const int ns = total[cur];
      if (valid) {
        const unsigned short* li = sidx + cur * C;
        const float* lv = sval + cur * C;
        // eight columns in flight per round (the loads are L2 latency bound), summed in list order
        int k = 0;
        for (; k + 8 <= ns; k += 8) {
          float r[8];
#pragma unroll
          for (int u = 0; u < 8; ++u) r[u] = __ldg(rec_t + (size_t)li[k + u] * C + i);
#pragma unroll
          for (int u = 0; u < 8; ++u) fb = __fmaf_rn(GRADED ? lv[k + u] : 1.f, r[u], fb);
        }
        for (; k < ns; ++k)
          fb = __fmaf_rn(GRADED ? lv[k] : 1.f, __ldg(rec_t + (size_t)li[k] * C + i), fb);
      }
      float a[1], b[2];
      a[0] = valid ? __fadd_rn(zt[i * kRecPitch + tt], fb) : 0.f;
      op.step(a, b);
      const bool fired = valid && b[1] != 0.f;
      if (valid) {
        vt[i * kRecPitch + tt] = b[0];
        zt[i * kRecPitch + tt] = b[1];
      }
      const int nxt = cur ^ 1;
      const unsigned m = __ballot_sync(0xffffffffu, fired);
      if (lane == 0) wcount[nxt * 32 + warp] = __popc(m);
      __syncthreads();
      int base = 0, all = 0;
      for (int w = 0; w < nwarp; ++w) {
        const int c = wcount[nxt * 32 + w];
        base += (w < warp) ? c : 0;
        all += c;
      }
      if (fired) {
        const int pos = base + __popc(m & ((1u << lane) - 1u));
        sidx[nxt * C + pos] = (unsigned short)i;
        if (GRADED) sval[nxt * C + pos] = b[1];
      }
      if (i == 0) total[nxt] = all;
      __syncthreads();
      cur = nxt;
    }
    rec_tile_io<false>(zt, spike, nullptr, row0, C, T, t0);
    rec_tile_io<false>(vt, voltage, nullptr, row0, C, T, t0);
    __syncthreads();
  }
  op.finish(p, g, row0 + (valid ? i : 0), valid, lane, 0);
}

// Backward (utils/recurrent.py:79-112).  Every forward step was a Neuron call
// with T = 1 whose incoming state carries no gradient, so the time recursion
// runs through R only:
//   g_d[t] = surrogate(v[t]) * (grad_spike[t] + R^T g_d[t + 1]),  grad_z[t] = g_d[t].
// rec [C, C] = R (row i holds the weights into neuron i).  Shared memory per
// sample of the CTA: 2 tiles [C][kRecPitch], C floats for g_d of the current step and
// 4 x C partial sums.
template <bool GRADED, int S, bool VEC>
__global__ void __launch_bounds__(1024, 1)
cuba_recurrent_bwd_kernel(Surrogate sg, float thr, RowGeom g, const float* __restrict__ grad_spike,
                          const float* __restrict__ voltage, const float* __restrict__ rec,
                          float* __restrict__ grad_z, int C, int batch) {
  // S samples per CTA share every load of R (the walk is bound by the L2 traffic of R).
  extern __shared__ __align__(16) unsigned char rec_smem[];
  const size_t tile_floats = (size_t)C * kRecPitch;
  float* gt = reinterpret_cast<float*>(rec_smem);   // [S] grad_spike tiles, overwritten by grad_z
  float* vt = gt + S * tile_floats;                 // [S] voltage tiles
  float* gd = vt + S * tile_floats;                 // [S][C]
  float* part = gd + (size_t)S * C;                 // [S][4][C] partial sums of the vector path

  const int j = threadIdx.x;
  const bool valid = j < C;
  const int b0 = blockIdx.x * S;
  const int ns = min(S, batch - b0);
  const int64_t row0 = (int64_t)b0 * C;
  const int T = g.T;
  float carry[S];
#pragma unroll
  for (int s = 0; s < S; ++s) carry[s] = 0.f;
  const int ntile = (T + kRecTile - 1) / kRecTile;
  for (int tile = ntile - 1; tile >= 0; --tile) {
    const int t0 = tile * kRecTile;
    for (int s = 0; s < ns; ++s) {
      rec_tile_io<true>(gt + s * tile_floats, nullptr, grad_spike, row0 + (int64_t)s * C, C, T, t0);
      rec_tile_io<true>(vt + s * tile_floats, nullptr, voltage, row0 + (int64_t)s * C, C, T, t0);
    }
    __syncthreads();
    const int nstep = min(kRecTile, T - t0);
    for (int tt = nstep - 1; tt >= 0; --tt) {
      if (valid) {
#pragma unroll
        for (int s = 0; s < S; ++s) {
          float d = 0.f;
          if (s < ns) {
            float* gts = gt + s * tile_floats;
            const float gs = __fadd_rn(gts[j * kRecPitch + tt], carry[s]);
            d = __fmul_rn(surrogate<GRADED>(sg, vt[s * tile_floats + j * kRecPitch + tt], thr), gs);
            gts[j * kRecPitch + tt] = d;
          }
          gd[s * C + j] = d;
        }
      }
      __syncthreads();
      const bool more = (t0 + tt) > 0;
      if (VEC) {
        // C % 4 == 0: a thread owns four adjacent columns of R and every fourth row, so each load is
        // 16 bytes (four times the bytes in flight of the scalar path); the four row groups meet in shared memory
        if (valid && more) {
          const int q = C >> 2, jq = j % q, ig = j / q;
          float4 acc[S];
#pragma unroll
          for (int s = 0; s < S; ++s) acc[s] = make_float4(0.f, 0.f, 0.f, 0.f);
          const float4* base = reinterpret_cast<const float4*>(rec) + jq;
          int i = ig;
          for (; i + 12 < C; i += 16) {
            float4 r[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) r[u] = __ldg(base + (size_t)(i + 4 * u) * q);
#pragma unroll
            for (int u = 0; u < 4; ++u)
#pragma unroll
              for (int s = 0; s < S; ++s) {
                const float gv = gd[s * C + i + 4 * u];
                acc[s].x = __fmaf_rn(gv, r[u].x, acc[s].x);
                acc[s].y = __fmaf_rn(gv, r[u].y, acc[s].y);
                acc[s].z = __fmaf_rn(gv, r[u].z, acc[s].z);
                acc[s].w = __fmaf_rn(gv, r[u].w, acc[s].w);
              }
          }
          for (; i < C; i += 4) {
            const float4 r = __ldg(base + (size_t)i * q);
#pragma unroll
            for (int s = 0; s < S; ++s) {
              const float gv = gd[s * C + i];
              acc[s].x = __fmaf_rn(gv, r.x, acc[s].x);
              acc[s].y = __fmaf_rn(gv, r.y, acc[s].y);
              acc[s].z = __fmaf_rn(gv, r.z, acc[s].z);
              acc[s].w = __fmaf_rn(gv, r.w, acc[s].w);
            }
          }
#pragma unroll
          for (int s = 0; s < S; ++s)
            *reinterpret_cast<float4*>(part + ((size_t)(s * 4 + ig) * C) + 4 * jq) = acc[s];
        }
        __syncthreads();
        if (valid && more) {
#pragma unroll
          for (int s = 0; s < S; ++s) {
            const float* ps = part + (size_t)s * 4 * C + j;
            carry[s] = __fadd_rn(__fadd_rn(ps[0], ps[C]), __fadd_rn(ps[2 * C], ps[3 * C]));
          }
        }
      } else if (valid && more) {
        float acc[S][4];
#pragma unroll
        for (int s = 0; s < S; ++s) acc[s][0] = acc[s][1] = acc[s][2] = acc[s][3] = 0.f;
        int i = 0;
        for (; i + 4 <= C; i += 4) {
          float r[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) r[u] = __ldg(rec + (size_t)(i + u) * C + j);
#pragma unroll
          for (int s = 0; s < S; ++s)
#pragma unroll
            for (int u = 0; u < 4; ++u) acc[s][u] = __fmaf_rn(gd[s * C + i + u], r[u], acc[s][u]);
        }
        for (; i < C; ++i) {
          const float r = __ldg(rec + (size_t)i * C + j);
#pragma unroll
          for (int s = 0; s < S; ++s) acc[s][0] = __fmaf_rn(gd[s * C + i], r, acc[s][0]);
        }
#pragma unroll
        for (int s = 0; s < S; ++s)
          carry[s] = __fadd_rn(__fadd_rn(acc[s][0], acc[s][1]), __fadd_rn(acc[s][2], acc[s][3]));
      }
      __syncthreads();
    }
    for (int s = 0; s < ns; ++s)
      rec_tile_io<false>(gt + s * tile_floats, grad_z, nullptr, row0 + (int64_t)s * C, C, T, t0);
    __syncthreads();
  }
}

inline size_t rec_fwd_smem(int C) {
  return 2 * (size_t)C * kRecPitch * 4 + 2 * (size_t)C * 4 + 66 * 4 + 2 * (size_t)C * 2;
}
inline size_t rec_bwd_smem(int C, int S) {
  return (size_t)S * (2 * (size_t)C * kRecPitch * 4 + (size_t)C * 4 + 4 * (size_t)C * 4);
}

}  // namespace sb
