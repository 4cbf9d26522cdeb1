// Row-scan framework: the one kernel skeleton every time-recurrent op uses.
//
// Data layout (fixed by the lava-dl API): tensors are [rows, T] fp32 with time
// contiguous; every row is an independent serial recurrence over T.  One lane
// owns one row and keeps the recurrence state in registers.  A warp therefore
// works on a 32-row band and walks it in 32-step time tiles:
//
//   global --TMA 2-D tile (32 rows x 128 B, swizzle-128B)--> shared
//   lane l reads row l of the tile as 128-bit chunks (bank-conflict free),
//   computes 4 steps per chunk, writes results back IN PLACE into the same
//   tile slots (row l / chunk c is private to lane l)
//   shared --TMA 2-D tile store--> global
//
// so global traffic is always 128-byte row segments although the math runs
// "down the rows".  Warps are fully independent (own stages, own mbarriers, no
// __syncthreads), a CTA is only a packaging unit for shared memory.
//
// Pipeline per warp with S stages of max(NIN, NOUT) tiles: while tile k is
// computed, the loads of tiles k+1 .. k+S-2 are in flight; after the stores of
// tile k are issued the stage used by tile k-1 is recycled for tile k+S-1 once
// its stores have finished reading shared memory (bulk wait_group.read).
//
// Outputs that are 0/1 valued (binary spikes) need not occupy a shared-memory
// tile at all: an op may declare its last NBIT outputs as bit outputs.  Each
// lane then collects one bit per step in a register and, per stage, the warp
// writes those rows straight to global memory (a shuffle hands every lane the
// mask of the row being written: one coalesced row segment per store).  This
// halves the shared memory of the fused CUBA forward, which buys two boxes per
// stage, i.e. 256-byte row segments for every stream.
//
// When a tensor cannot be described to TMA (T not a multiple of 4, base not
// 16-byte aligned, T < 32) the same ops run under rowscan_plain_kernel, which
// fills the same swizzled tiles with plain coalesced loads.
#pragma once

#include "common.cuh"

namespace sb {

template <int N>
struct MapPack {
  CUtensorMap m[N];
};

template <int NIN, int NOUT>
struct RowPtrs {
  const float* in[NIN];
  float* out[NOUT];
};

__host__ __device__ constexpr int cmax(int a, int b) { return a > b ? a : b; }

// An op may offer a second, shorter form of its step for parameters every lane
// of the warp can take (HAS_FAST, fast(), step_t<FAST>): the skeleton asks once
// per warp and runs whole tiles in that form.
template <class Op, class = void>
struct OpHasFast { static constexpr bool value = false; };
template <class Op>
struct OpHasFast<Op, decltype((void)Op::HAS_FAST)> { static constexpr bool value = Op::HAS_FAST; };

template <class Op>
__device__ __forceinline__ bool op_fast(const Op& op) {
  if constexpr (OpHasFast<Op>::value) return op.fast();
  else return false;
}
template <bool FAST, class Op, class A, class B>
__device__ __forceinline__ void op_step(Op& op, const A& a, B& b) {
  if constexpr (OpHasFast<Op>::value) op.template step_t<FAST>(a, b);
  else op.step(a, b);
}

// ---------------------------------------------------------------------------
// One tile: TW / 4 chunks of 4 steps.  nvalid < TW only for the ragged last tile.
// ---------------------------------------------------------------------------
template <class Op, bool FULL, int TW, bool FAST = false>
__device__ __forceinline__ void process_tile(Op& op, uint8_t* stage, int lane, int nvalid,
                                             uint32_t (&bits)[Op::NBIT > 0 ? Op::NBIT : 1]) {
  constexpr int NIN = Op::NIN, NOUT = Op::NOUT, NS = Op::NOUT - Op::NBIT;
  constexpr int kChunks = TW / 4;
  constexpr int kTileBytes = TW * kTileR * 4;
#pragma unroll 2
  for (int cc = 0; cc < kChunks; ++cc) {
    const int c = Op::REVERSE ? kChunks - 1 - cc : cc;
    if (!FULL && c * 4 >= nvalid) {
      if (Op::REVERSE) continue; else break;
    }
    const uint32_t off = swz_chunk<TW>(lane, c);
    float vin[NIN][4];
#pragma unroll
    for (int i = 0; i < NIN; ++i) {
      const float4 v = *reinterpret_cast<const float4*>(stage + i * kTileBytes + off);
      vin[i][0] = v.x; vin[i][1] = v.y; vin[i][2] = v.z; vin[i][3] = v.w;
    }
    float vout[NS > 0 ? NS : 1][4];
#pragma unroll
    for (int jj = 0; jj < 4; ++jj) {
      const int j = Op::REVERSE ? 3 - jj : jj;
      float a[NIN], b[NOUT];
#pragma unroll
      for (int i = 0; i < NIN; ++i) a[i] = vin[i][j];
      if (FULL || c * 4 + j < nvalid) {
        op_step<FAST>(op, a, b);
      } else {
#pragma unroll
        for (int o = 0; o < NOUT; ++o) b[o] = 0.f;
      }
#pragma unroll
      for (int o = 0; o < NS; ++o) vout[o][j] = b[o];
#pragma unroll
      for (int d = 0; d < Op::NBIT; ++d)
        if (b[NS + d] != 0.f) bits[d] |= 1u << (c * 4 + j);
    }
#pragma unroll
    for (int o = 0; o < NS; ++o) {
      *reinterpret_cast<float4*>(stage + o * kTileBytes + off) =
          make_float4(vout[o][0], vout[o][1], vout[o][2], vout[o][3]);
    }
  }
}

// ---------------------------------------------------------------------------
// Bit outputs: lane r holds, per box, the mask of row r (bit t = step t of the
// box).  Row by row, every lane fetches that row's masks and the warp writes
// the row's NB * TW steps as coalesced 0.f / 1.f values.
// ---------------------------------------------------------------------------
// delay = 1 writes every bit output one step late (out[t] = bit[t - 1]): the
// one-step inter-layer delay of lava-dl's blocks (block/base.py:15-39) folded
// into the store.  The bit that enters at t = 0 is head[row] != 0 (the spike a
// persistent-state block carried over from its previous call), 0 without head.
// lut adds a per-row axonal delay on top (axon/delay.py:150-175 after the step
// delay, block/base.py:549-552): row r is written int(lut[r % n_lut] / lut_ts)
// steps later still, 0 .. 62.  A lane keeps the masks of its row's last two
// boxes and takes each output word out of that 96-bit window with a funnel
// shift, so the delay costs no memory traffic.
// packed (bit output 0 only): the same bits as 32-bit words instead of, or next to, the 0.f / 1.f
// values: word w of row r holds steps 32 w .. 32 w + 31 (bit i = step 32 w + i), packed_words words per row.
template <int N>
struct BitPtrs {
  float* p[N > 0 ? N : 1];
  uint32_t* packed;
  int64_t packed_words;
  const float* head;
  int delay;
  const float* lut;
  int64_t n_lut;
  float lut_ts;
};

struct BitDelay {
  int steps;          // 0 or 1
  const float* head;  // [rows] or null
  const float* lut;   // per-row delays or null
  int64_t n_lut;
  float lut_ts;
  uint32_t* packed = nullptr;  // [rows, ceil(T / 32)] or null: bit output 0 as 32-step words
};

constexpr int kMaxBitDelay = 62;  // per-row delay; with the step delay the window shift stays below 64

// Total shift of a row's bit stream (step delay + per-row delay); a delay outside
// 0 .. kMaxBitDelay is clamped and reported in the device status word.
__device__ __forceinline__ int bit_shift_of_row(int steps, const float* lut, int64_t n_lut, float lut_ts, int64_t row,
                                                bool valid, unsigned int* status) {
  int sh = steps;
  if (lut != nullptr && valid) {
    int d = __float2int_rz(__fdiv_rn(__ldg(lut + (row % n_lut)), lut_ts));
    if (d < 0 || d > kMaxBitDelay) {
      dev_flag(status, SB_DEV_BAD_DELAY);
      d = d < 0 ? 0 : kMaxBitDelay;
    }
    sh += d;
  }
  return sh;
}
// Output word of the current box: bits [64 - sh, 96 - sh) of (m : prev1 : prev2).
__device__ __forceinline__ uint32_t delayed_word(uint32_t m, uint32_t prev1, uint32_t prev2, int sh) {
  return sh < 32 ? __funnelshift_l(prev1, m, sh) : __funnelshift_l(prev2, prev1, sh - 32);
}

template <int NB, int TW>
__device__ __forceinline__ void store_bit_rows(float* __restrict__ base, int64_t T, int nrows, int nvalid,
                                               const uint32_t (&mask)[NB], int lane, bool vec_ok) {
  constexpr int kSpan = NB * TW;
  if (TW == 32 && vec_ok && nrows == kTileR && nvalid >= kSpan) {
    // 128-bit stores: eight lanes cover one row's 32 steps, four rows per instruction
    const int sub = lane >> 3, chunk = lane & 7;
#pragma unroll
    for (int i = 0; i < kTileR / 4; ++i) {
      const int r = sub + 4 * i;
      float* dst = base + (int64_t)r * T + chunk * 4;
#pragma unroll
      for (int b = 0; b < NB; ++b) {
        const uint32_t m = __shfl_sync(0xffffffffu, mask[b], r) >> (chunk * 4);
        *reinterpret_cast<float4*>(dst + b * TW) =
            make_float4((m & 1u) ? 1.f : 0.f, (m & 2u) ? 1.f : 0.f, (m & 4u) ? 1.f : 0.f, (m & 8u) ? 1.f : 0.f);
      }
    }
    return;
  }
#pragma unroll 4
  for (int r = 0; r < kTileR; ++r) {
    uint32_t mrow[NB];
#pragma unroll
    for (int b = 0; b < NB; ++b) mrow[b] = __shfl_sync(0xffffffffu, mask[b], r);
    if (r >= nrows) continue;
    float* dst = base + (int64_t)r * T;
#pragma unroll
    for (int q = 0; q < (kSpan + 31) / 32; ++q) {
      const int pos = q * 32 + lane;
      if (pos < kSpan && pos < nvalid) {
        const int box = pos / TW, bit = pos % TW;
        uint32_t m = mrow[0];
#pragma unroll
        for (int b = 1; b < NB; ++b) m = (box == b) ? mrow[b] : m;
        dst[pos] = ((m >> bit) & 1u) ? 1.f : 0.f;
      }
    }
  }
}

// ---------------------------------------------------------------------------
// TMA-pipelined kernel
// ---------------------------------------------------------------------------
template <class Op, int STAGES, int NB, int TW, bool FAST>
__device__ __forceinline__ void rowscan_tma_body(const MapPack<Op::NIN + Op::NOUT - Op::NBIT>& maps,
                                                 const BitPtrs<Op::NBIT>& bitout, const typename Op::Params& p,
                                                 const RowGeom& g, unsigned int* status, Op& op, uint8_t* wsm,
                                                 uint32_t bar0, int64_t row0, int lane, int64_t warp_id) {
  constexpr int NIN = Op::NIN, NOUT = Op::NOUT - Op::NBIT, NBIT = Op::NBIT, NT = cmax(NIN, NOUT);
  constexpr int kTileT = TW;                         // shadows the 32-step default
  constexpr int kTileBytes = TW * kTileR * 4;
  constexpr int kStageBytes = NT * NB * kTileBytes;  // NB boxes of TW steps, side by side in time
  constexpr int kSpan = NB * kTileT;                 // time steps per stage
  const int T = g.T;
  const int ntiles = (T + kSpan - 1) / kSpan;
  const int y = (int)row0;
  const int64_t row = row0 + lane;
  const bool valid = row < g.rows;

  auto tile_t0 = [&](int k) { return (Op::REVERSE ? (ntiles - 1 - k) : k) * kSpan; };
  auto issue_load = [&](int k) {  // lane 0 only
    const int s = k % STAGES;
    const uint32_t bar = bar0 + s * 8;
    const int t0 = tile_t0(k);
    int nb = (T - t0 + kTileT - 1) / kTileT;  // boxes that start inside the tensor
    nb = nb > NB ? NB : nb;
    mbar_expect_tx(bar, NIN * nb * kTileBytes);
    for (int b = 0; b < nb; ++b) {
#pragma unroll
      for (int i = 0; i < NIN; ++i)
        tma_load_2d(smem_u32(wsm + s * kStageBytes + (b * NT + i) * kTileBytes), &maps.m[i], t0 + b * kTileT, y,
                    bar);
    }
  };

  // delayed bit outputs: the masks of the row's last two boxes and the row's shift
  uint32_t prev1 = 0u, prev2 = 0u;
  const bool delayed = NBIT > 0 && (bitout.delay != 0 || bitout.lut != nullptr);
  int sh = 0;
  if (delayed) {
    sh = bit_shift_of_row(bitout.delay, bitout.lut, bitout.n_lut, bitout.lut_ts, row, valid, status);
    if (bitout.delay && bitout.head != nullptr && valid) prev1 = (__ldg(bitout.head + row) != 0.f) ? 0x80000000u : 0u;
  }

  int issued = 0;
  if (lane == 0) {
    for (; issued < STAGES - 1 && issued < ntiles; ++issued) issue_load(issued);
  }

  bool ok = true;
  int k = 0;
  for (; k < ntiles; ++k) {
    const int s = k % STAGES;
    if (!mbar_wait(bar0 + s * 8, (k / STAGES) & 1)) { ok = false; break; }
    uint8_t* stage = wsm + s * kStageBytes;
    const int t0 = tile_t0(k);
    uint32_t bits[NBIT > 0 ? NBIT : 1][NB];
#pragma unroll
    for (int bb = 0; bb < NB; ++bb) {
      const int b = Op::REVERSE ? NB - 1 - bb : bb;
      uint32_t boxbits[NBIT > 0 ? NBIT : 1];
#pragma unroll
      for (int d = 0; d < (NBIT > 0 ? NBIT : 1); ++d) boxbits[d] = 0u;
      const int nvalid = T - (t0 + b * kTileT);
      if (nvalid > 0) {
        uint8_t* box = stage + b * NT * kTileBytes;
        if (nvalid >= kTileT) process_tile<Op, true, TW, FAST>(op, box, lane, kTileT, boxbits);
        else process_tile<Op, false, TW, FAST>(op, box, lane, nvalid, boxbits);
        op.tile_end();
      }
      if (delayed) {  // forward ops only: boxes come in time order (32-step boxes)
        const uint32_t m = boxbits[0];
        boxbits[0] = delayed_word(m, prev1, prev2, sh);
        prev2 = prev1;
        prev1 = m;
      }
#pragma unroll
      for (int d = 0; d < (NBIT > 0 ? NBIT : 1); ++d) bits[d][b] = boxbits[d];
    }
    fence_proxy_async();
    __syncwarp();
    if (lane == 0) {
      for (int b = 0; b < NB; ++b) {
        if (t0 + b * kTileT >= T) break;
#pragma unroll
        for (int o = 0; o < NOUT; ++o)
          tma_store_2d(&maps.m[NIN + o], t0 + b * kTileT, y, smem_u32(stage + (b * NT + o) * kTileBytes));
      }
      tma_commit();
      const int kn = k + STAGES - 1;
      if (kn < ntiles) {
        tma_wait_read<1>();  // stores of tile k-1 have left shared memory
        issue_load(kn);
      }
    }
    __syncwarp();
    if (NBIT > 0) {
      const int64_t left = g.rows - row0;
      if (TW == 32 && bitout.packed != nullptr && valid) {
        uint32_t* dst = bitout.packed + row * bitout.packed_words + t0 / 32;
#pragma unroll
        for (int b = 0; b < NB; ++b) {
          const int left_t = T - (t0 + b * kTileT);  // a delayed word carries the row's last bits past T
          if (left_t > 0) dst[b] = left_t >= 32 ? bits[0][b] : (bits[0][b] & ((1u << left_t) - 1u));
        }
      }
#pragma unroll
      for (int d = 0; d < NBIT; ++d)
        if (bitout.p[d] != nullptr)
          store_bit_rows<NB, TW>(bitout.p[d] + row0 * (int64_t)T + t0, T, left < kTileR ? (int)left : kTileR, T - t0,
                                 bits[d], lane, (reinterpret_cast<uintptr_t>(bitout.p[d]) & 15u) == 0);
    }
  }

  if (lane == 0) tma_wait_all<0>();
  if (!ok) {
    // A load never arrived.  Record it and drain what this warp still has in flight (bounded).
    // The per-row results below are then those of a walk that stopped early: the status bit says
    // so, and every slot a later pass reads (parameter-gradient partials) is still written.
    if (lane == 0) {
      dev_flag(status, SB_DEV_TMA_TIMEOUT);
      const int last = (k + STAGES - 1 < ntiles) ? k + STAGES - 1 : ntiles;
      for (int kk = k + 1; kk < last; ++kk) (void)mbar_wait(bar0 + (kk % STAGES) * 8, (kk / STAGES) & 1);
    }
    __syncwarp();
  }
  op.finish(p, g, row, valid, lane, warp_id);
}

template <class Op, int STAGES, int NB, int TW>
__global__ void __launch_bounds__(128)
rowscan_tma_kernel(const __grid_constant__ MapPack<Op::NIN + Op::NOUT - Op::NBIT> maps,
                   const BitPtrs<Op::NBIT> bitout, const typename Op::Params p, const RowGeom g,
                   unsigned int* status) {
  constexpr int NIN = Op::NIN, NOUT = Op::NOUT - Op::NBIT, NT = cmax(NIN, NOUT);
  constexpr int kWarpBytes = STAGES * NT * NB * (TW * kTileR * 4);
  extern __shared__ uint8_t smem_raw[];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  const int64_t warp_id = (int64_t)blockIdx.x * nwarps + warp;
  const int64_t row0 = warp_id * kTileR;
  if (row0 >= g.rows) return;
  // swizzle-128B tiles need 1024-byte alignment; the launch reserves the slack
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint8_t* wsm = smem + (size_t)warp * kWarpBytes;
  const uint32_t bar0 = smem_u32(smem + (size_t)nwarps * kWarpBytes) + warp * STAGES * 8;

  if (lane == 0) {
#pragma unroll
    for (int s = 0; s < STAGES; ++s) mbar_init(bar0 + s * 8, 1);
    fence_mbar_init();
    fence_proxy_async();
  }
  __syncwarp();

  Op op;
  op.init(p, g, row0 + lane, row0 + lane < g.rows);
  // one warp-uniform choice between the two forms of the op's step for the whole walk
  if (OpHasFast<Op>::value && op_fast(op))
    rowscan_tma_body<Op, STAGES, NB, TW, true>(maps, bitout, p, g, status, op, wsm, bar0, row0, lane, warp_id);
  else
    rowscan_tma_body<Op, STAGES, NB, TW, false>(maps, bitout, p, g, status, op, wsm, bar0, row0, lane, warp_id);
}

// ---------------------------------------------------------------------------
// Plain-load kernel: any T, any alignment.  Same tiles, same ops.
// ---------------------------------------------------------------------------
template <class Op, bool FAST>
__device__ __forceinline__ void rowscan_plain_body(const RowPtrs<Op::NIN, Op::NOUT>& ptrs, const BitDelay& bd,
                                                   const typename Op::Params& p, const RowGeom& g,
                                                   unsigned int* status, Op& op, uint8_t* stage, int64_t wid,
                                                   int lane) {
  constexpr int NIN = Op::NIN, NOUT = Op::NOUT - Op::NBIT, NBIT = Op::NBIT;
  const int64_t row0 = wid * kTileR;
  const int T = g.T;
  const int ntiles = (T + kTileT - 1) / kTileT;
  const int nrows = (int)((g.rows - row0) < kTileR ? (g.rows - row0) : kTileR);
  const int64_t row = row0 + lane;
  const bool valid = row < g.rows;

  uint32_t prev1 = 0u, prev2 = 0u;
  const bool delayed = NBIT > 0 && (bd.steps != 0 || bd.lut != nullptr);
  int sh = 0;
  if (delayed) {
    sh = bit_shift_of_row(bd.steps, bd.lut, bd.n_lut, bd.lut_ts, row, valid, status);
    if (bd.steps && bd.head != nullptr && valid) prev1 = (__ldg(bd.head + row) != 0.f) ? 0x80000000u : 0u;
  }

  for (int k = 0; k < ntiles; ++k) {
    const int t0 = (Op::REVERSE ? (ntiles - 1 - k) : k) * kTileT;
    const int nvalid = T - t0;
    const bool tin = lane < nvalid;
#pragma unroll
    for (int i = 0; i < NIN; ++i) {
      const float* src = ptrs.in[i] + row0 * (int64_t)T + t0 + lane;
#pragma unroll 8
      for (int r = 0; r < kTileR; ++r) {
        float v = 0.f;
        if (tin && r < nrows) v = __ldg(src + (int64_t)r * T);
        *reinterpret_cast<float*>(stage + i * kTileBytes + swz_elem(r, lane)) = v;
      }
    }
    __syncwarp();
    uint32_t bits[NBIT > 0 ? NBIT : 1];
#pragma unroll
    for (int d = 0; d < (NBIT > 0 ? NBIT : 1); ++d) bits[d] = 0u;
    if (nvalid >= kTileT) process_tile<Op, true, 32, FAST>(op, stage, lane, kTileT, bits);
    else process_tile<Op, false, 32, FAST>(op, stage, lane, nvalid, bits);
    op.tile_end();
    if (delayed) {
      const uint32_t m = bits[0];
      bits[0] = delayed_word(m, prev1, prev2, sh);
      prev2 = prev1;
      prev1 = m;
    }
    __syncwarp();
#pragma unroll
    for (int o = 0; o < NOUT; ++o) {
      float* dst = ptrs.out[o] + row0 * (int64_t)T + t0 + lane;
#pragma unroll 8
      for (int r = 0; r < kTileR; ++r) {
        if (tin && r < nrows)
          dst[(int64_t)r * T] = *reinterpret_cast<const float*>(stage + o * kTileBytes + swz_elem(r, lane));
      }
    }
    if (NBIT > 0 && bd.packed != nullptr && valid)
      bd.packed[row * (int64_t)((T + 31) / 32) + t0 / 32] = nvalid >= 32 ? bits[0] : (bits[0] & ((1u << nvalid) - 1u));
#pragma unroll
    for (int d = 0; d < NBIT; ++d) {
      if (ptrs.out[NOUT + d] == nullptr) continue;
      const uint32_t one[1] = {bits[d]};
      store_bit_rows<1, 32>(ptrs.out[NOUT + d] + row0 * (int64_t)T + t0, T, nrows, nvalid, one, lane, false);
    }
    __syncwarp();
  }
  op.finish(p, g, row, valid, lane, wid);
}

template <class Op>
__global__ void __launch_bounds__(128)
rowscan_plain_kernel(const RowPtrs<Op::NIN, Op::NOUT> ptrs, const BitDelay bd, const typename Op::Params p,
                     const RowGeom g, unsigned int* status) {
  constexpr int NT = cmax(Op::NIN, Op::NOUT - Op::NBIT);
  extern __shared__ uint8_t smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  const int64_t wid = (int64_t)blockIdx.x * nwarps + warp;
  if (wid * kTileR >= g.rows) return;
  uint8_t* stage = smem + (size_t)warp * NT * kTileBytes;
  Op op;
  op.init(p, g, wid * kTileR + lane, wid * kTileR + lane < g.rows);
  if (OpHasFast<Op>::value && op_fast(op)) rowscan_plain_body<Op, true>(ptrs, bd, p, g, status, op, stage, wid, lane);
  else rowscan_plain_body<Op, false>(ptrs, bd, p, g, status, op, stage, wid, lane);
}

// ---------------------------------------------------------------------------
// Host launcher
// ---------------------------------------------------------------------------
struct LaunchPlan {
  int warps_per_cta;
  int64_t ctas;
  size_t smem;
};

LaunchPlan plan_rowscan(int64_t rows, size_t bytes_per_warp, size_t fixed_bytes);
int prepare_kernel(const void* fn, size_t smem);

// Pipeline shape of the TMA kernels: each op names its own (ops.cuh).
template <class Op> constexpr int pipe_stages() { return Op::STAGES; }
template <class Op> constexpr int pipe_boxes() { return Op::BOXES; }
template <class Op> constexpr int pipe_tile() { return Op::TILE; }

template <class Op, int STAGES = pipe_stages<Op>(), int NB = pipe_boxes<Op>(), int TW = pipe_tile<Op>()>
int launch_rowscan(const typename Op::Params& p, const RowGeom& g, const float* const* in, float* const* out,
                   cudaStream_t st, BitDelay bit_delay = BitDelay{0, nullptr, nullptr, 0, 1.f}) {
  // NOUT counts the outputs that travel through shared memory; the NBIT bit
  // outputs follow them in `out`.
  constexpr int NIN = Op::NIN, NOUT = Op::NOUT - Op::NBIT, NBIT = Op::NBIT, NT = cmax(NIN, NOUT);
  if (g.rows == 0 || g.T == 0) return SB_OK;
  SB_REQUIRE(g.rows > 0 && g.rows < (int64_t)2147483647 - 64, "rows out of range: %lld", (long long)g.rows);
  SB_REQUIRE(g.T > 0, "T out of range");
  const void* all[NIN + NOUT];
  for (int i = 0; i < NIN; ++i) all[i] = in[i];
  for (int o = 0; o < NOUT; ++o) all[NIN + o] = out[o];
  for (int i = 0; i < NIN + NOUT; ++i) SB_REQUIRE(all[i] != nullptr, "null tensor pointer (slot %d)", i);
  SB_REQUIRE(bit_delay.steps == 0 || (bit_delay.steps == 1 && NBIT == 1 && !Op::REVERSE),
             "a one-step output delay exists only for ops with one bit output");
  SB_REQUIRE(bit_delay.lut == nullptr || (NBIT == 1 && !Op::REVERSE && TW == 32 && bit_delay.n_lut > 0 &&
                                          g.rows % bit_delay.n_lut == 0 && bit_delay.lut_ts != 0.f),
             "a per-row output delay needs one bit output, 32-step tiles and a table that tiles the rows");
  BitPtrs<NBIT> bitout;
  bitout.p[0] = nullptr;
  bitout.packed = bit_delay.packed;
  bitout.packed_words = (g.T + 31) / 32;
  bitout.head = bit_delay.head;
  bitout.delay = bit_delay.steps;
  bitout.lut = bit_delay.lut;
  bitout.n_lut = bit_delay.n_lut;
  bitout.lut_ts = bit_delay.lut_ts;
  SB_REQUIRE(bit_delay.packed == nullptr || (NBIT == 1 && TW == 32 && !Op::REVERSE),
             "packed output exists only for forward ops with one bit output and 32-step tiles");
  for (int d = 0; d < NBIT; ++d) {
    SB_REQUIRE(out[NOUT + d] != nullptr || (d == 0 && bit_delay.packed != nullptr),
               "null tensor pointer (bit output %d)", d);
    bitout.p[d] = out[NOUT + d];
  }
  unsigned int* status = status_ptr();
  if (!status) return SB_ERR_CUDA;

  if (tma_eligible(all, NIN + NOUT, g.T)) {
    MapPack<NIN + NOUT> maps;
    for (int i = 0; i < NIN + NOUT; ++i) {
      int rc = make_row_map(&maps.m[i], all[i], g.rows, g.T, TW);
      if (rc != SB_OK) return rc;
    }
    const size_t per_warp = (size_t)STAGES * NT * NB * (TW * kTileR * 4) + STAGES * 8;
    const LaunchPlan lp = plan_rowscan(g.rows, per_warp, 1024);
    auto fn = rowscan_tma_kernel<Op, STAGES, NB, TW>;
    int rc = prepare_kernel((const void*)fn, lp.smem);
    if (rc != SB_OK) return rc;
    fn<<<(unsigned)lp.ctas, lp.warps_per_cta * 32, lp.smem, st>>>(maps, bitout, p, g, status);
  } else {
    RowPtrs<NIN, Op::NOUT> ptrs;
    for (int i = 0; i < NIN; ++i) ptrs.in[i] = in[i];
    for (int o = 0; o < Op::NOUT; ++o) ptrs.out[o] = out[o];
    const size_t per_warp = (size_t)NT * kTileBytes;
    const LaunchPlan lp = plan_rowscan(g.rows, per_warp, 0);
    auto fn = rowscan_plain_kernel<Op>;
    int rc = prepare_kernel((const void*)fn, lp.smem);
    if (rc != SB_OK) return rc;
    fn<<<(unsigned)lp.ctas, lp.warps_per_cta * 32, lp.smem, st>>>(ptrs, bit_delay, p, g, status);
  }
  SB_CUDA(cudaGetLastError());
  return SB_OK;
}

}  // namespace sb
