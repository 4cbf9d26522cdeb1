// Convolution synapse (synapse/layer.py:178-323: Conv3d with a 1-wide time
// kernel over [N, C, H, W, T]) on the 5th-generation tensor cores, as an implicit
// GEMM with time kept innermost:
//
//   y[n, co, ho, wo, t] = sum_{ci, i, j} w[co, ci, i, j] * x[n, ci, ho + i - ph, wo + j - pw, t]
//   D[m, co]            = sum_k A[m, k] * B[co, k]        m = (wo, t) position, k = (i, j, ci)
//
// A tile is M = 128 positions (4 output columns x 32 time steps) of one output
// row and N = up to 64 output channels.  Nothing gathers the A operand: an input
// row lands in shared memory as [column][channel][32 steps] (a 5-D TMA box whose
// dimensions are listed in that order, 128-byte swizzle over 32-byte chunks), which is exactly the
// M-major TF32 operand layout of tcgen05.mma -- 32 positions contiguous, channels 128
// bytes apart in atoms of four, the next output column one column stride further on.  An
// MMA (K = 8) reads eight consecutive 128-byte (column, channel) rows of the slot of input row
// ho + i: with 8 or more channels per column that is tap (i, j) over channels 8 g .. 8 g + 7
// (the descriptor starts j columns and g atoms into the slot); with 2 or 4 channels per column
// it is 4 or 2 neighbouring taps at once (the weights of taps past kw are zeros), so a
// 2-channel 5 x 5 layer takes 10 MMAs per tile instead of 25 with zero-filled channels.  The
// padding is the zero fill of the TMA box, in space and in the channel count alike.
//
// Spikes are 0 / 1 and block weights sit on a 1/32 grid, both exact in TF32, so
// the fp32 accumulation gives bit for bit the sums of the fp32 kernel and of the
// CPU.  Any other operand is split v = hi + lo (two TF32 values): the scan warps
// look at every row that lands and, if a value has low mantissa bits, leave its
// hi parts in place and write the lo parts to a second slot; the tile then
// accumulates hi*hi + lo*hi + hi*lo, so float inputs keep fp32 accuracy.
//
// Data flow per CTA (persistent over work items, one CTA per SM, 12 warps).  A
// work item is (sample, group of 4 output columns, chunk of 32 steps); the CTA
// walks down its output rows, so every input row is fetched once per item (the
// only re-read is the kw - 1 column halo between neighbouring items):
//   producer (1 thread): one TMA box per input row into a ring of row slots --
//     the kh rows a tile reads plus the rows requested ahead.
//   scan (4 warps): reads each landed row once with 128-bit loads, decides
//     whether it needs lo parts and writes them if so (ring of kh + 2 lo slots, taken only by
//     rows that need one: rows of spikes are scanned as far ahead as the row ring reaches).
//   issue (3 threads, taking tiles in turn): kh x kw x ceil(Ci / 8) MMAs (kind::tf32, M128, N = Co
//     padded to 16) per tile into a ring of TMEM accumulators; B (the weights, split, K-major,
//     128-byte swizzle) is built once per CTA in shared memory.  An MMA with an M-major operand
//     holds its thread for well over a hundred cycles while the pipe accepts the next thread's
//     (16 -> 32 channels, 3 x 3, [32, 16, 16, 16, 300]: 0.42 / 0.23 / 0.19 / 0.31 ms with 1 / 2 / 3 / 4
//     issue threads; 0.11 ms with the MMAs taken out; 0.15 ms with the MMAs of a kernel row in one loop).
//   drain (4 warps): tcgen05.ld of the accumulator, one coalesced 128-byte store
//     per warp and output channel; having seen a tile complete they also hand its
//     oldest row slot back to the producer -- every tcgen05 instruction, commits
//     included, queues behind the MMAs, so the issue thread commits once per tile.
// TMEM holds accumulators only (up to 8 of npad columns).
// Every wait is bounded; a wait that runs out sets a CTA-wide flag that ends all
// other waits, SB_DEV_TMA_TIMEOUT is recorded, loads and MMAs in flight are
// waited for, TMEM is freed.  Tensor maps cover this GPU's memory only; no
// cluster, no multicast.
#include "api_util.cuh"
#include "tc.cuh"

using namespace sb;

namespace sb {
int make_map_5d(CUtensorMap* out, const void* base, const uint64_t (&dims)[5], const uint64_t (&strides)[4],
                const uint32_t (&box)[5], int swizzle);
}

namespace {

constexpr int kM = 128;
constexpr int kWG = 4;                       // output columns per tile
constexpr int kTT = 32;                      // time steps per tile
constexpr int kAccCols = 64;                 // output channels per launch group
constexpr int kTmemCols = 512;
constexpr int kMaxAcc = 8;                   // accumulators at most

constexpr int kNumIssue = 3;                 // MMA-issuing threads, taking tiles in turn
constexpr int kIssueWarp = 8, kProdWarp = kIssueWarp + kNumIssue;
constexpr int kThreads = 32 * (kProdWarp + 1);
constexpr int kMaxRing = 24;                 // row slots: the kh live rows plus the rows in flight
constexpr int kMaxLo = 8;                    // lo slots: kh + 2

struct ConvTc {
  int N, Ci, Co, H, W, Ho, Wo, ph, pw, T;
  int ci0, cib;    // this launch's block of input channels: ci0 .. ci0 + cib - 1 (wide layers take several launches)
  int cpc;         // channels per column of a row slot: 2, 4, or a multiple of 8 (zero filled past the block)
  int nm;          // MMAs per kernel row: each reads 8 consecutive 128-byte (column, channel) rows of the slot
  int box_bytes;   // bytes one TMA box delivers: columns x cpc x 128
  int npad;        // MMA N: output channels of this launch's channel groups, padded to 16
  int nwg, ntc;    // work-item grid: column groups, time chunks
  int slot_bytes;  // stride of the row slots (box_bytes rounded up to 1024)
  int ring;        // row slots: kh live rows + rows requested ahead (the TMA latency to hide)
  int b_bytes;     // one of the two weight factors in shared memory
};

// Position in a ring of n slots: slot index and how often the ring has wrapped (its low bit is the
// mbarrier phase).  Advanced by comparison, because n is a run-time value and the loops of all four
// roles are single-thread latency chains in which an integer division costs as much as four MMAs.
struct Cursor {
  uint32_t slot, wraps;
  __device__ __forceinline__ void next(uint32_t n) {
    if (++slot == n) { slot = 0; ++wraps; }
  }
};

__device__ __forceinline__ void tma_load_5d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, int c3, int c4,
                                            uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.5d.shared::cta.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5, %6}], [%7];"
      ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4), "r"(bar)
      : "memory");
}

// ACC: this launch adds to y (a block of input channels after the first); a kernel of its own, because the
// read-modify-write of the drain warps needs registers the plain kernel should not pay for
template <int KH, int KW, bool ACC>
__global__ void __launch_bounds__(kThreads, 1)
conv_tc_kernel(const __grid_constant__ CUtensorMap xmap, const float* __restrict__ wgt, float* __restrict__ y,
               const ConvTc g, unsigned int* status) {
  constexpr uint32_t RL = KH + 2;              // lo slots
  static_assert(KH + 2 <= kMaxLo && KH + 2 <= kMaxRing, "ring too small for the kernel height");
  const uint32_t R = (uint32_t)g.ring;
  const uint32_t NM = (uint32_t)g.nm;
  const uint32_t col_bytes = (uint32_t)g.cpc * 128u;   // one column of a row slot

  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* sm = smem_raw + (base - smem_u32(smem_raw));
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // layout: weights hi | weights lo | row ring | lo ring | barriers | words
  const int off_bhi = 0, off_blo = g.b_bytes, off_ring = 2 * g.b_bytes;
  const int off_lo = off_ring + R * g.slot_bytes;
  const int off_bar = off_lo + RL * g.slot_bytes;
  const uint32_t bar_full = base + off_bar;                // [R]   a row has landed
  const uint32_t bar_rawfree = bar_full + 8 * kMaxRing;    // [R]   no MMA reads the row any more
  const uint32_t bar_ready = bar_rawfree + 8 * kMaxRing;   // [R]   the row is scanned (and split)
  const uint32_t bar_lofree = bar_ready + 8 * kMaxRing;    // [RL]  a lo slot is read no more
  const uint32_t bar_mma = bar_lofree + 8 * kMaxLo;        // [NACC]
  const uint32_t bar_accfree = bar_mma + 8 * kMaxAcc;      // [NACC]
  constexpr int kBarBytes = 8 * (3 * kMaxRing + kMaxLo + 2 * kMaxAcc);
  volatile uint32_t* tmem_word = reinterpret_cast<volatile uint32_t*>(sm + off_bar + kBarBytes);
  volatile int* dead = reinterpret_cast<volatile int*>(sm + off_bar + kBarBytes + 4);
  // [R] per row slot: 0 = the row is exact in TF32, else 1 + the lo slot that holds its lo parts
  volatile int* has_lo = reinterpret_cast<volatile int*>(sm + off_bar + kBarBytes + 8);
  const uint32_t NACC = (uint32_t)(kTmemCols / g.npad) < (uint32_t)kMaxAcc ? (uint32_t)(kTmemCols / g.npad)
                                                                           : (uint32_t)kMaxAcc;

  if (tid == 0) {
    for (uint32_t i = 0; i < R; ++i) {
      mbar_init(bar_full + 8 * i, 1);
      mbar_init(bar_rawfree + 8 * i, 4);     // one arrival per drain warp
      mbar_init(bar_ready + 8 * i, kM);
    }
    for (uint32_t i = 0; i < RL; ++i) mbar_init(bar_lofree + 8 * i, 4);
    for (int i = 0; i < kMaxAcc; ++i) {
      mbar_init(bar_mma + 8 * i, 1);
      mbar_init(bar_accfree + 8 * i, kM);
    }
    *dead = 0;
    fence_mbar_init();
  }
  if (warp == kIssueWarp) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(base + off_bar + kBarBytes), "r"(kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }

  // Weight factor of this CTA's channel group, split into two TF32 values, K-major with the
  // 128-byte swizzle: rows = output channels, column k' = (i * NM + m) * 8 + r, where MMA m of kernel
  // row i reads the slot's rows 8 m .. 8 m + 7 -- with 8 or more channels per column that is tap
  // j = m / (cpc / 8) over channels 8 (m % (cpc / 8)) + r, with 2 or 4 channels per column it is taps
  // j = m (8 / cpc) + r / cpc over channel r % cpc (taps past KW get zero weights).
  const int co0 = blockIdx.y * kAccCols;
  const int ktot = KH * (int)NM * 8;
  int any_blo = 0;
  for (int e = tid; e < g.npad * ktot; e += kThreads) {
    const int co = e / ktot, kp = e - co * ktot;
    const int q = kp >> 3, r = kp & 7, i = q / (int)NM, m = q - i * (int)NM;
    int j, ci;
    if (g.cpc >= 8) {
      const int G = g.cpc >> 3;
      j = m / G;
      ci = (m - j * G) * 8 + r;
    } else {
      j = m * (8 / g.cpc) + r / g.cpc;
      ci = r % g.cpc;
    }
    const int tap = i * KW + j;
    float v = 0.f;
    if (j < KW && ci < g.cib && co0 + co < g.Co)
      v = __ldg(wgt + ((int64_t)(co0 + co) * g.Ci + g.ci0 + ci) * (KH * KW) + tap);
    const uint32_t hi = tf32_rn(v), lo = tf32_rn(__fsub_rn(v, __uint_as_float(hi)));
    any_blo |= (lo != 0u);
    const int kk = kp & 31;
    const int off = (kp >> 5) * (g.npad * 128) + co * 128 + (((kk >> 2) ^ (co & 7)) << 4) + ((kk & 3) << 2);
    *reinterpret_cast<uint32_t*>(sm + off_bhi + off) = hi;
    *reinterpret_cast<uint32_t*>(sm + off_blo + off) = lo;
  }
  fence_proxy_async();
  tc_fence_before();
  any_blo = __syncthreads_or(any_blo);
  tc_fence_after();
  const uint32_t tmem = *tmem_word;

  const int64_t nitems = (int64_t)g.N * g.nwg * g.ntc;
  const int Q = g.Ho + KH - 1;                  // input rows an item walks through
  const uint32_t idesc = idesc_tf32(kM, g.npad) | kIdescAMajorM;

  if (warp == kProdWarp) {
    // ---------------- producer: one TMA box per input row ----------------
    if (lane == 0) {
      Cursor rq{0, 0};
      bool ok = true;
      for (int64_t item = blockIdx.x; item < nitems && ok; item += gridDim.x) {
        const int tc = (int)(item % g.ntc), wg = (int)((item / g.ntc) % g.nwg), n = (int)(item / ((int64_t)g.ntc * g.nwg));
        for (int q = 0; q < Q; ++q, rq.next(R)) {
          if (rq.wraps >= 1 && !wait_or_dead(bar_rawfree + 8 * rq.slot, (rq.wraps - 1u) & 1u, dead)) { ok = false; break; }
          const uint32_t bar = bar_full + 8 * rq.slot;
          mbar_expect_tx(bar, (uint32_t)g.box_bytes);
          // box dimensions: steps, channels, columns, rows, samples
          tma_load_5d(base + off_ring + rq.slot * g.slot_bytes, &xmap, tc * kTT, g.ci0, wg * kWG - g.pw, q - g.ph, n, bar);
        }
      }
      if (*dead) {
        // loads still in flight must land before the shared memory is given back
        for (uint32_t i = 0; i < R; ++i) { mbar_wait(bar_full + 8 * i, 0); mbar_wait(bar_full + 8 * i, 1); }
      }
    }
    __syncwarp();
  } else if (warp >= kIssueWarp && warp < kIssueWarp + kNumIssue) {
    // ---------------- issue: the MMAs of every kNumIssue-th tile (one thread per warp) ----------------
    // A thread waits well over a hundred cycles on each MMA it issues; the tensor pipe takes the next
    // thread's MMA meanwhile.
    const uint32_t me = (uint32_t)(warp - kIssueWarp);
    if (lane == 0) {
      const uint32_t bhi = desc_lo(base + off_bhi), blo = desc_lo(base + off_blo);
      const uint32_t a_deschi = kDescHiMMajor;
      const uint32_t box16 = (uint32_t)(g.npad * 128) >> 4;   // one 32-column box of the factor, in 16-byte units
      Cursor rq{0, 0}, cd{0, 0};   // oldest live row, accumulators
      uint32_t last_acc = 0, last_phase = 0, tiles = 0, turn = 0;   // turn: whose tile this is
      bool ok = true;
      for (int64_t item = blockIdx.x; item < nitems; item += gridDim.x) {
        for (int ho = 0; ho < g.Ho; ++ho) {
          const bool mine = turn == me;
          if (++turn == (uint32_t)kNumIssue) turn = 0;
          if (!mine) {
            cd.next(NACC);
            rq.next(R);
            continue;
          }
          const uint32_t acc = cd.slot;
          if (cd.wraps >= 1) ok = wait_or_dead(bar_accfree + 8 * acc, (cd.wraps - 1u) & 1u, dead) && ok;
          const uint32_t d_tmem = tmem + acc * (uint32_t)g.npad;
          // rows ho .. ho + KH - 1 of this item (all of them are waited for: the tile before this one was
          // another thread's)
          uint32_t rs[KH];
          {
            Cursor r = rq;
#pragma unroll
            for (int i = 0; i < KH; ++i, r.next(R)) {
              ok = wait_or_dead(bar_ready + 8 * r.slot, r.wraps & 1u, dead) && ok;
              rs[i] = r.slot;
            }
          }
          tc_fence_after();
          if (ok) {
            uint32_t first = 0u;
#pragma unroll
            for (int i = 0; i < KH; ++i) {
              const uint32_t row_hi = base + off_ring + rs[i] * g.slot_bytes;
              const int lo_slot = has_lo[rs[i]] - 1;
              const bool alo = lo_slot >= 0;
              const uint32_t row_lo = base + off_lo + (alo ? lo_slot : 0) * g.slot_bytes;
              // MMA m of this kernel row reads the slot's rows 8 m .. 8 m + 7 (the next output column
              // starts one column further on: the leading offset).  Three loops with run-time trip
              // counts rather than three conditional MMAs per step: a predicated-off MMA still takes
              // its ~46 cycles on the issue path.
              const uint32_t kp0 = (uint32_t)i * NM * 8u;
#pragma unroll 1
              for (uint32_t m = 0; m < NM; ++m) {
                const uint32_t kp = kp0 + m * 8u;
                umma_ss(d_tmem, desc_lo_mmajor(row_hi + m * 1024u, col_bytes),
                        a_deschi, bhi + (kp >> 5) * box16 + ((kp & 31u) >> 2), idesc, first);
                first = 1u;
              }
              const uint32_t nblo = any_blo ? NM : 0u, nalo = alo ? NM : 0u;
#pragma unroll 1
              for (uint32_t m = 0; m < nblo; ++m) {
                const uint32_t kp = kp0 + m * 8u;
                umma_ss(d_tmem, desc_lo_mmajor(row_hi + m * 1024u, col_bytes),
                        a_deschi, blo + (kp >> 5) * box16 + ((kp & 31u) >> 2), idesc, 1u);
              }
#pragma unroll 1
              for (uint32_t m = 0; m < nalo; ++m) {
                const uint32_t kp = kp0 + m * 8u;
                umma_ss(d_tmem, desc_lo_mmajor(row_lo + m * 1024u, col_bytes),
                        a_deschi, bhi + (kp >> 5) * box16 + ((kp & 31u) >> 2), idesc, 1u);
              }
            }
          }
          umma_commit(bar_mma + 8 * acc);
          last_acc = acc; last_phase = cd.wraps & 1u; ++tiles;
          cd.next(NACC);
          rq.next(R);
        }
        // the item's last KH - 1 rows belong to no further tile
        for (int q = g.Ho; q < Q; ++q) rq.next(R);
      }
      // nothing may still be writing TMEM when it is freed: wait for this thread's last tile
      if (tiles >= 1) mbar_wait(bar_mma + 8 * last_acc, last_phase);
    }
    __syncwarp();
  } else if (warp < 4) {
    // ---------------- scan warps: does a landed row need lo parts? ----------------
    // Each thread reads its 16-byte words of the slot (the same offsets in the lo slot: both
    // start on a 1024-byte boundary, so the swizzle pattern is the same).  Only a row that needs
    // lo parts takes a lo slot (the next of their ring) and waits for it; rows of spikes run as far
    // ahead of the tiles as the row ring allows.
    Cursor rq{0, 0}, lq{0, 0};
    for (int64_t item = blockIdx.x; item < nitems; item += gridDim.x) {
      for (int q = 0; q < Q; ++q, rq.next(R)) {
        wait_or_dead(bar_full + 8 * rq.slot, rq.wraps & 1u, dead);
        uint8_t* row = sm + off_ring + rq.slot * g.slot_bytes;
        uint32_t low = 0;
        for (int off = tid * 16; off < g.box_bytes; off += kM * 16) {
          const uint4 v = *reinterpret_cast<const uint4*>(row + off);
          low |= v.x | v.y | v.z | v.w;
        }
        int any;
        asm volatile(
            "{\n\t.reg .pred p, q;\n\t"
            "setp.ne.b32 q, %1, 0;\n\t"
            "bar.red.or.pred p, 1, %2, q;\n\t"
            "selp.s32 %0, 1, 0, p;\n\t}"
            : "=r"(any)
            : "r"(low & ~kTf32Mask), "n"(kM)
            : "memory");
        int flag = 0;
        if (any) {
          // the lo slot's previous row is read no more?
          if (lq.wraps >= 1) wait_or_dead(bar_lofree + 8 * lq.slot, (lq.wraps - 1u) & 1u, dead);
          // hi = x truncated to TF32 stays in the row's own slot, lo = x - hi (exact) goes to the lo slot
          uint8_t* lorow = sm + off_lo + lq.slot * g.slot_bytes;
          for (int off = tid * 16; off < g.box_bytes; off += kM * 16) {
            uint4 v = *reinterpret_cast<const uint4*>(row + off);
            uint4 h, l;
            h.x = v.x & kTf32Mask; l.x = __float_as_uint(__fsub_rn(__uint_as_float(v.x), __uint_as_float(h.x)));
            h.y = v.y & kTf32Mask; l.y = __float_as_uint(__fsub_rn(__uint_as_float(v.y), __uint_as_float(h.y)));
            h.z = v.z & kTf32Mask; l.z = __float_as_uint(__fsub_rn(__uint_as_float(v.z), __uint_as_float(h.z)));
            h.w = v.w & kTf32Mask; l.w = __float_as_uint(__fsub_rn(__uint_as_float(v.w), __uint_as_float(h.w)));
            *reinterpret_cast<uint4*>(row + off) = h;
            *reinterpret_cast<uint4*>(lorow + off) = l;
          }
          fence_proxy_async();   // the MMAs read what these stores wrote
          flag = 1 + (int)lq.slot;
          lq.next(RL);
        }
        if (tid == 0) has_lo[rq.slot] = flag;
        mbar_arrive(bar_ready + 8 * rq.slot);
      }
    }
  } else {
    // ---------------- drain warps: accumulator -> output rows ----------------
    const int m = tid - kM, wl = m >> 5, tl = m & 31;
    const int ew = warp & 3;
    Cursor cd{0, 0}, rq{0, 0};
    const int64_t cstride = (int64_t)g.Ho * g.Wo * g.T;
    const int64_t rstride = (int64_t)g.Wo * g.T;
    const int nco = min(g.npad, g.Co - co0);
    for (int64_t item = blockIdx.x; item < nitems; item += gridDim.x) {
      const int tc = (int)(item % g.ntc), wg = (int)((item / g.ntc) % g.nwg), n = (int)(item / ((int64_t)g.ntc * g.nwg));
      const int wo = wg * kWG + wl, t = tc * kTT + tl;
      const bool live_pos = wo < g.Wo && t < g.T;
      float* dst = y + ((int64_t)n * g.Co + co0) * cstride + (int64_t)(live_pos ? wo : 0) * g.T + (live_pos ? t : 0);
      for (int ho = 0; ho < g.Ho; ++ho, dst += rstride) {
        const uint32_t acc = cd.slot;
        const bool ok = wait_or_dead(bar_mma + 8 * acc, cd.wraps & 1u, dead);
        tc_fence_after();
        // This warp has seen every tile up to this one complete: no MMA reads the tile's oldest
        // row any more, nor, after an item's last tile, its other rows.
        if (lane == 0) {
          const int nfree = (ho == g.Ho - 1) ? KH : 1;
          for (int i = 0; i < nfree; ++i, rq.next(R)) {
            const int lo_slot = has_lo[rq.slot] - 1;    // read before the row slot is handed back
            mbar_arrive(bar_rawfree + 8 * rq.slot);
            if (lo_slot >= 0) mbar_arrive(bar_lofree + 8 * lo_slot);
          }
        }
        const uint32_t taddr = tmem + ((uint32_t)(ew * 32) << 16) + acc * (uint32_t)g.npad;
        // the tile's npad columns in as few loads as their count allows: 32 at a time, then 16
#pragma unroll 1
        for (int cb = 0; cb < g.npad;) {
          uint32_t r[32];
          const int ncol = (g.npad - cb >= 32) ? 32 : 16;
          if (ncol == 32) {
            tmem_ld32(taddr + cb, r);
          } else {
            tmem_ld16(taddr + cb, *reinterpret_cast<uint32_t(*)[16]>(r));
          }
          tmem_ld_wait();
          if (ok && live_pos) {
            if constexpr (ACC) {
              // loads first, sixteen at a time: written as load-add-store per channel the stores would keep
              // each next load waiting (the compiler cannot tell that the channels do not alias)
#pragma unroll
              for (int h = 0; h < 32; h += 16) {
                float prev[16];
#pragma unroll
                for (int e = 0; e < 16; ++e)
                  prev[e] = (h + e < ncol && cb + h + e < nco) ? __ldcg(dst + (cb + h + e) * cstride) : 0.f;
#pragma unroll
                for (int e = 0; e < 16; ++e)
                  if (h + e < ncol && cb + h + e < nco)
                    dst[(cb + h + e) * cstride] = __fadd_rn(prev[e], __uint_as_float(r[h + e]));
              }
            } else {
#pragma unroll
              for (int e = 0; e < 32; ++e)
                if (e < ncol && cb + e < nco) dst[(cb + e) * cstride] = __uint_as_float(r[e]);
            }
          }
          cb += ncol;
        }
        tc_fence_before();
        mbar_arrive(bar_accfree + 8 * acc);
        cd.next(NACC);
      }
    }
  }
  if (*dead && tid == 0) dev_flag(status, SB_DEV_TMA_TIMEOUT);
  tc_fence_before();
  __syncthreads();
  if (warp == kIssueWarp) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
  }
}

struct TcPlan {
  ConvTc g;
  size_t smem;
  bool ok;
};

// Plan for one launch over a block of `cb` input channels (the whole layer when cb == Ci).
TcPlan plan_block(int64_t N, int64_t Ci, int64_t cb, int64_t Co, int64_t H, int64_t W, int64_t kh, int64_t kw, int64_t ph,
                  int64_t pw, int64_t T) {
  TcPlan p{};
  p.ok = false;
  const int64_t Ho = H + 2 * ph - kh + 1, Wo = W + 2 * pw - kw + 1;
  // channels per column of a row slot: few channels are packed 2 or 4 to a column, so that the eight
  // rows an MMA reads span several taps instead of zero-filled channels
  const int cpc = cb <= 2 ? 2 : (cb <= 4 ? 4 : (int)((cb + 7) / 8) * 8);
  const int per = cpc < 8 ? 8 / cpc : 1;                                 // columns (taps) per MMA
  const int nm = cpc < 8 ? (int)((kw + per - 1) / per) : (int)kw * (cpc / 8);
  const int wcols = cpc < 8 ? (kWG - 1) + nm * per : (int)(kWG + kw - 1);
  const int ngroup = (int)((Co + kAccCols - 1) / kAccCols);
  const int64_t co_last = Co - (int64_t)(ngroup - 1) * kAccCols;
  // every channel group is launched with the same MMA N: the widest group, padded to 16
  const int npad = (int)(((ngroup > 1 ? kAccCols : co_last) + 15) & ~15);
  const int64_t box_bytes = (int64_t)wcols * cpc * 128;
  const int64_t slot = (box_bytes + 1023) & ~1023LL;
  const int64_t ktot = kh * nm * 8;
  const int64_t b_bytes = (((ktot + 31) / 32) * npad * 128 + 1023) & ~1023LL;
  const int64_t fixed = 2 * b_bytes + 8 * (3 * kMaxRing + kMaxLo + 2 * kMaxAcc) + 128 + 1024 + (kh + 2) * slot;
  // rows in flight beyond the kh live ones: as many as fit in 224 KB, at most 16, at least 2
  int64_t ahead = (224 * 1024 - fixed) / slot - kh;
  if (ahead > 16) ahead = 16;
  if (ahead < 2 || ngroup > 65535) return p;
  const int R = (int)(kh + ahead);
  const int64_t smem = fixed + (int64_t)R * slot;
  p.g = ConvTc{(int)N, (int)Ci, (int)Co, (int)H, (int)W, (int)Ho, (int)Wo, (int)ph, (int)pw, (int)T, 0, (int)cb, cpc, nm,
               (int)box_bytes, npad, (int)((Wo + kWG - 1) / kWG), (int)((T + kTT - 1) / kTT), (int)slot, R, (int)b_bytes};
  // at least 120 KB so that two CTAs (two TMEM allocations of 512 columns) never share an SM
  p.smem = (size_t)(smem < 120 * 1024 ? 120 * 1024 : smem);
  p.ok = true;
  return p;
}

// The whole layer in one launch when its rings and weights fit shared memory; else in blocks of input
// channels, each launch after the first adding to the output (the fewest blocks, of equal size rounded up
// to 8 channels).  *nblocks says how many launches.
TcPlan plan_conv_tc(int64_t N, int64_t Ci, int64_t Co, int64_t H, int64_t W, int64_t kh, int64_t kw, int64_t ph,
                    int64_t pw, int64_t T, int* nblocks) {
  TcPlan p{};
  p.ok = false;
  *nblocks = 0;
  if (!((kh == 1 && kw == 1) || (kh == 3 && kw == 3) || (kh == 5 && kw == 5))) return p;
  if (T < kTT || (T & 3) || Ci > 1024 || N > 65535 * 16 || H > (1 << 20) || W > (1 << 20) || T > (1 << 28)) return p;
  const int64_t Ho = H + 2 * ph - kh + 1, Wo = W + 2 * pw - kw + 1;
  if (Ho < 1 || Wo < 1) return p;
  p = plan_block(N, Ci, Ci, Co, H, W, kh, kw, ph, pw, T);
  if (p.ok) { *nblocks = 1; return p; }
  for (int nb = 2; nb <= 16 && Ci / nb >= 8; ++nb) {
    const int64_t cb = (((Ci + nb - 1) / nb) + 7) & ~7LL;
    p = plan_block(N, Ci, cb, Co, H, W, kh, kw, ph, pw, T);
    if (p.ok) { *nblocks = (int)((Ci + cb - 1) / cb); return p; }
  }
  p.ok = false;
  return p;
}

}  // namespace

namespace sb {

// Runs the tensor-core convolution when the problem fits it; *taken says whether it did.
int conv_tc_try(const float* x, const float* weight, float* y, int64_t N, int64_t Ci, int64_t Co, int64_t H, int64_t W,
                int64_t kh, int64_t kw, int64_t ph, int64_t pw, int64_t T, cudaStream_t st, bool* taken) {
  *taken = false;
  if ((((uintptr_t)x) | ((uintptr_t)y)) & 15u) return SB_OK;
  int nblocks = 0;
  const TcPlan p = plan_conv_tc(N, Ci, Co, H, W, kh, kw, ph, pw, T, &nblocks);
  if (!p.ok) return SB_OK;
  // The box lists its dimensions as (steps, channels, columns, rows, samples): that is the order a
  // row slot has in shared memory.  Channels past Ci are out of range and read zeros.
  CUtensorMap xmap;
  const uint64_t dims[5] = {(uint64_t)T, (uint64_t)Ci, (uint64_t)W, (uint64_t)H, (uint64_t)N};
  const uint64_t strides[4] = {(uint64_t)(H * W * T * 4), (uint64_t)(T * 4), (uint64_t)(W * T * 4),
                               (uint64_t)(Ci * H * W * T * 4)};
  const uint32_t box[5] = {(uint32_t)kTT, (uint32_t)p.g.cpc, (uint32_t)(p.g.box_bytes / (p.g.cpc * 128)), 1u, 1u};
  int rc = make_map_5d(&xmap, x, dims, strides, box, 2);
  if (rc != SB_OK) return rc;
  const int64_t nitems = (int64_t)p.g.N * p.g.nwg * p.g.ntc;
  const int ngroup = (int)((Co + kAccCols - 1) / kAccCols);
  const int gx = (int)(nitems < sm_count() ? nitems : sm_count());
  const dim3 grid((unsigned)gx, (unsigned)ngroup);
  unsigned int* status = status_ptr();
  if (!status) return SB_ERR_CUDA;
  // one launch per block of input channels; every launch after the first adds to y
#define SB_GO(KH, KW)                                                                                        \
  {                                                                                                          \
    auto fn = conv_tc_kernel<KH, KW, false>;                                                                 \
    auto fn_acc = conv_tc_kernel<KH, KW, true>;                                                              \
    SB_CUDA(cudaFuncSetAttribute((const void*)fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)p.smem)); \
    if (nblocks > 1)                                                                                         \
      SB_CUDA(cudaFuncSetAttribute((const void*)fn_acc, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)p.smem)); \
    ConvTc gb = p.g;                                                                                         \
    const int block = gb.cib;                                                                                \
    for (int b = 0; b < nblocks; ++b) {                                                                      \
      gb.ci0 = b * block;                                                                                    \
      gb.cib = (int)(Ci - gb.ci0 < block ? Ci - gb.ci0 : block);                                             \
      if (b == 0) fn<<<grid, kThreads, p.smem, st>>>(xmap, weight, y, gb, status);                           \
      else fn_acc<<<grid, kThreads, p.smem, st>>>(xmap, weight, y, gb, status);                              \
    }                                                                                                        \
  }
  if (kh == 1) SB_GO(1, 1)
  else if (kh == 3) SB_GO(3, 3)
  else SB_GO(5, 5)
#undef SB_GO
  SB_CUDA(cudaGetLastError());
  *taken = true;
  return SB_OK;
}

}  // namespace sb

// the contraction must be long enough for the tile hand-offs to pay off (2 -> 16 channels, 5 x 5, 50
// taps, at [32, 2, 32, 32, 300]: 0.53 ms on either kernel; 16 -> 32, 3 x 3, 144 taps: 0.15 against 0.79 ms)
constexpr int64_t kMinTapsForAuto = 64;

extern "C" int sb_conv_fits_tensor_cores(int64_t N, int64_t Ci, int64_t Co, int64_t H, int64_t W, int64_t kh,
                                         int64_t kw, int64_t ph, int64_t pw, int64_t T) {
  int nb = 0;
  return plan_conv_tc(N, Ci, Co, H, W, kh, kw, ph, pw, T, &nb).ok ? 1 : 0;
}

extern "C" int sb_conv_uses_tensor_cores(int64_t N, int64_t Ci, int64_t Co, int64_t H, int64_t W, int64_t kh,
                                         int64_t kw, int64_t ph, int64_t pw, int64_t T) {
  int nb = 0;
  return (Ci * kh * kw >= kMinTapsForAuto && plan_conv_tc(N, Ci, Co, H, W, kh, kw, ph, pw, T, &nb).ok) ? 1 : 0;
}
