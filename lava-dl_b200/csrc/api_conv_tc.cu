// Convolution synapse (synapse/layer.py:178-323: Conv3d with a 1-wide time
// kernel over [N, C, H, W, T]) on the 5th-generation tensor cores, as an implicit
// GEMM with time kept innermost:
//
//   y[n, co, ho, wo, t] = sum_{ci, i, j} w[co, ci, i, j] * x[n, ci, ho + i - ph, wo + j - pw, t]
//   D[m, co]            = sum_k A[m, k] * B[co, k]        m = (wo, t) position, k = (ci, i, j)
//
// A tile is M = 128 positions (4 output columns x 32 time steps) of one output
// row, N = up to 64 output channels, and K = Ci * kh * kw in chunks of CIG input
// channels (<= 96 operand columns).  Spikes are 0 / 1 and block weights sit on a
// 1/32 grid, both exact in TF32, so the fp32 accumulation gives bit for bit the
// sums of the fp32 kernel and of the CPU; any other operand is split v = hi + lo
// (two TF32 values) and the tile accumulates hi*hi + lo*hi + hi*lo, as the
// temporal filter does, so float inputs (the input-gradient pass) keep fp32
// accuracy.  A box whose values are all exact skips its lo products.
//
// Data flow per CTA (persistent over work items, one CTA per SM, 10 warps).  A
// work item is (sample, group of 4 output columns, chunk of 32 steps); the CTA
// walks down its output rows, so every input row is fetched once per item (the
// only re-read is the kw - 1 column halo between neighbouring items):
//   producer (1 thread): one 5-D TMA box per input row -- 32 steps x (4 + kw - 1)
//     columns x all Ci channels, zero filled outside the image, which is the
//     padding -- into a ring of row slots in shared memory: the kh rows a tile reads plus up to 16
//     rows requested ahead (a row is a few KB, so the ring has to be deep to cover the TMA latency).
//   split (4 warps, one position per thread): gathers the thread's K values of
//     the chunk from the kh live row slots, splits them, and writes them to TMEM
//     (tcgen05.st): the A operand of the MMAs is read from TMEM, K along columns.
//   issue (1 thread): KC / 8 x tcgen05.mma kind::tf32 (M128, N = Co padded to 16) per chunk into
//     a ring of TMEM accumulators; B (the weights, split, K-major, 128-byte swizzle) is built once
//     per CTA in shared memory.  (Two issue threads on alternating tiles, each with half of the
//     rings, measured slower: the rings get too shallow.)
//   drain (4 warps): tcgen05.ld of the accumulator, one coalesced 128-byte store
//     per warp and output channel.
// TMEM columns: 128 for a ring of accumulators (2 for 64 output channels, 8 for 16), 384 for a
// ring of operand slots of one chunk each (4 to 8 slots).  A chunk of exact values takes one slot;
// a chunk that needs lo parts takes the next slot as well.  The rings are what hides the latency of
// the hand-offs (split -> MMA -> drain take about a microsecond per round trip).
// Every wait is bounded; a wait that runs out sets a CTA-wide flag that ends all
// other waits, SB_DEV_TMA_TIMEOUT is recorded, loads and MMAs in flight are
// waited for, TMEM is freed.  Tensor maps cover this GPU's memory only; no
// cluster, no multicast.
#include "api_util.cuh"
#include "tc.cuh"

using namespace sb;

namespace sb {
int make_map_5d(CUtensorMap* out, const void* base, const uint64_t (&dims)[5], const uint32_t (&box)[5]);
}

namespace {

constexpr int kM = 128;
constexpr int kWG = 4;                       // output columns per tile
constexpr int kTT = 32;                      // time steps per tile
constexpr int kKCmax = 96;                   // operand columns per K-chunk
constexpr int kAccCols = 64;                 // output channels per launch group
constexpr int kAccSpace = 128;               // TMEM columns of the accumulator ring
constexpr int kColA = kAccSpace;             // operand slots start here
constexpr int kTmemCols = 512;
constexpr int kMaxSlots = 8;                 // operand slots / accumulators at most

constexpr int kIssueWarp = 8, kProdWarp = 9;
constexpr int kThreads = 32 * (kProdWarp + 1);
constexpr int kMaxRing = 24;                 // row slots: the kh live rows plus the rows in flight

struct ConvTc {
  int N, Ci, Co, H, W, Ho, Wo, ph, pw, T;
  int nchunk;      // K-chunks per tile
  int npad;        // MMA N: output channels of this launch's channel groups, padded to 16
  int nwg, ntc;    // work-item grid: column groups, time chunks
  int slot_bytes;  // one input row in shared memory: Ci x (4 + kw - 1) x 128 B
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

template <int KH, int KW, int CIG>
__global__ void __launch_bounds__(kThreads, 1)
conv_tc_kernel(const __grid_constant__ CUtensorMap xmap, const float* __restrict__ wgt, float* __restrict__ y,
               const ConvTc g, unsigned int* status) {
  constexpr int KC = CIG * KH * KW;
  constexpr int KCpad = (KC + 7) & ~7;
  constexpr int WB = kWG + KW - 1;
  static_assert(KCpad <= kKCmax && KH + 2 <= kMaxRing, "chunk or ring too large");
  const uint32_t R = (uint32_t)g.ring;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* sm = smem_raw + (base - smem_u32(smem_raw));
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // layout: weights hi | weights lo | row ring | barriers | words
  const int off_bhi = 0, off_blo = g.b_bytes, off_ring = 2 * g.b_bytes;
  const int off_bar = off_ring + R * g.slot_bytes;
  const uint32_t bar_full = base + off_bar;              // [R]
  const uint32_t bar_rawfree = bar_full + 8 * kMaxRing;  // [R]
  const uint32_t bar_aready = bar_rawfree + 8 * kMaxRing;  // [NA]
  const uint32_t bar_afree = bar_aready + 8 * kMaxSlots;   // [NA]
  const uint32_t bar_mma = bar_afree + 8 * kMaxSlots;      // [NACC]
  const uint32_t bar_accfree = bar_mma + 8 * kMaxSlots;    // [NACC]
  constexpr int kBarBytes = 8 * (2 * kMaxRing + 4 * kMaxSlots);
  volatile uint32_t* tmem_word = reinterpret_cast<volatile uint32_t*>(sm + off_bar + kBarBytes);
  volatile int* dead = reinterpret_cast<volatile int*>(sm + off_bar + kBarBytes + 4);
  volatile int* has_lo = reinterpret_cast<volatile int*>(sm + off_bar + kBarBytes + 8);  // [NA]
  // operand slots of KCpad columns; accumulators of npad columns
  constexpr uint32_t NA = (kTmemCols - kColA) / KCpad < kMaxSlots ? (kTmemCols - kColA) / KCpad : kMaxSlots;
  static_assert(NA >= 4, "at least four operand slots");
  const uint32_t NACC = (uint32_t)(kAccSpace / g.npad) < (uint32_t)kMaxSlots ? (uint32_t)(kAccSpace / g.npad)
                                                                             : (uint32_t)kMaxSlots;

  if (tid == 0) {
    for (uint32_t i = 0; i < R; ++i) {
      mbar_init(bar_full + 8 * i, 1);
      mbar_init(bar_rawfree + 8 * i, kM);
    }
    for (int i = 0; i < kMaxSlots; ++i) {
      mbar_init(bar_aready + 8 * i, kM);
      mbar_init(bar_afree + 8 * i, 1);
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
  // 128-byte swizzle: column k' = chunk * KCpad + (cl * KH + i) * KW + j, rows = output channels.
  const int co0 = blockIdx.y * kAccCols;
  const int ktot = g.nchunk * KCpad;
  int any_blo = 0;
  for (int e = tid; e < g.npad * ktot; e += kThreads) {
    const int co = e / ktot, kp = e - co * ktot;
    const int c = kp / KCpad, kl = kp - c * KCpad;
    float v = 0.f;
    if (kl < KC) {
      const int cl = kl / (KH * KW), r = kl - cl * (KH * KW);
      const int ci = c * CIG + cl;
      if (ci < g.Ci && co0 + co < g.Co) v = __ldg(wgt + ((int64_t)(co0 + co) * g.Ci + ci) * (KH * KW) + r);
    }
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
  const uint32_t idesc = idesc_tf32(kM, g.npad);

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
          mbar_expect_tx(bar, (uint32_t)g.slot_bytes);
          tma_load_5d(base + off_ring + rq.slot * g.slot_bytes, &xmap, tc * kTT, wg * kWG - g.pw, q - g.ph, 0, n, bar);
        }
      }
      if (*dead) {
        // loads still in flight must land before the shared memory is given back
        for (uint32_t i = 0; i < R; ++i) { mbar_wait(bar_full + 8 * i, 0); mbar_wait(bar_full + 8 * i, 1); }
      }
    }
    __syncwarp();
  } else if (warp == kIssueWarp) {
    // ---------------- issue: the MMAs of every tile (one thread) ----------------
    if (lane == 0) {
      const uint32_t bhi = desc_lo(base + off_bhi), blo = desc_lo(base + off_blo);
      const uint32_t box16 = (uint32_t)(g.npad * 128) >> 4;   // one 32-column box of the factor, in 16-byte units
      Cursor ca{0, 0}, cd{0, 0};   // operand slots, accumulators
      uint32_t last_acc = 0, last_phase = 0, tiles = 0;
      bool ok = true;
      for (int64_t item = blockIdx.x; item < nitems; item += gridDim.x) {
        for (int ho = 0; ho < g.Ho; ++ho) {
          const uint32_t acc = cd.slot;
          if (cd.wraps >= 1) ok = wait_or_dead(bar_accfree + 8 * acc, (cd.wraps - 1u) & 1u, dead) && ok;
          const uint32_t d_tmem = tmem + acc * (uint32_t)g.npad;
          for (int c = 0; c < g.nchunk; ++c) {
            // the chunk's hi values sit in the next slot; its lo values, if it has any, in the slot after
            uint32_t as = ca.slot;
            ok = wait_or_dead(bar_aready + 8 * as, ca.wraps & 1u, dead) && ok;
            tc_fence_after();
            const bool alo = has_lo[as] != 0;
            if (ok) {
              const uint32_t ah = tmem + kColA + as * KCpad;
#pragma unroll
              for (int ks = 0; ks < KCpad / 8; ++ks) {
                const uint32_t kp = (uint32_t)(c * KCpad + 8 * ks);
                const uint32_t boff = (kp >> 5) * box16 + ((kp & 31u) >> 2);
                umma_ts(d_tmem, ah + 8 * ks, bhi + boff, idesc, (c | ks) ? 1u : 0u);
                if (any_blo) umma_ts(d_tmem, ah + 8 * ks, blo + boff, idesc, 1u);
              }
            }
            umma_commit(bar_afree + 8 * as);
            ca.next(NA);
            if (alo) {
              as = ca.slot;
              ok = wait_or_dead(bar_aready + 8 * as, ca.wraps & 1u, dead) && ok;
              tc_fence_after();
              if (ok) {
                const uint32_t al = tmem + kColA + as * KCpad;
#pragma unroll
                for (int ks = 0; ks < KCpad / 8; ++ks) {
                  const uint32_t kp = (uint32_t)(c * KCpad + 8 * ks);
                  umma_ts(d_tmem, al + 8 * ks, bhi + (kp >> 5) * box16 + ((kp & 31u) >> 2), idesc, 1u);
                }
              }
              umma_commit(bar_afree + 8 * as);
              ca.next(NA);
            }
          }
          umma_commit(bar_mma + 8 * acc);
          last_acc = acc; last_phase = cd.wraps & 1u; ++tiles;
          cd.next(NACC);
        }
      }
      // nothing may still be writing TMEM when it is freed: wait for the last tile's MMAs
      if (tiles >= 1) mbar_wait(bar_mma + 8 * last_acc, last_phase);
    }
    __syncwarp();
  } else if (warp < 4) {
    // ---------------- split warps: row slots -> K values of this position -> TMEM ----------------
    const int wl = tid >> 5, tl = tid & 31;
    const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
    Cursor rq{0, 0};               // oldest live row of the tile
    Cursor ca{0, 0};               // operand slots
    for (int64_t item = blockIdx.x; item < nitems; item += gridDim.x) {
      for (int ho = 0; ho < g.Ho; ++ho) {
        // rows ho .. ho + KH - 1 of this item; only the newest one can still be in flight
        const uint8_t* rowp[KH];
        {
          Cursor r = rq;
#pragma unroll
          for (int i = 0; i < KH; ++i, r.next(R)) {
            if (ho == 0 || i == KH - 1) wait_or_dead(bar_full + 8 * r.slot, r.wraps & 1u, dead);
            rowp[i] = sm + off_ring + r.slot * g.slot_bytes + wl * 128 + tl * 4;
          }
        }
        for (int c = 0; c < g.nchunk; ++c) {
          const int ci0 = c * CIG;
          uint32_t v[KCpad];
          uint32_t low = 0;
#pragma unroll
          for (int k = 0; k < KCpad; ++k) {
            uint32_t val = 0u;
            if (k < KC) {
              constexpr int KK = KH * KW;
              const int cl = k / KK, r = k % KK, i = r / KW, j = r % KW;
              if (ci0 + cl < g.Ci)
                val = *reinterpret_cast<const uint32_t*>(rowp[i] + ((ci0 + cl) * WB + j) * 128);
            }
            v[k] = val;
            low |= val;
          }
          // does any value of the chunk need a lo part?  (spike trains do not)
          int any;
          asm volatile(
              "{\n\t.reg .pred p, q;\n\t"
              "setp.ne.b32 q, %1, 0;\n\t"
              "bar.red.or.pred p, 1, %2, q;\n\t"
              "selp.s32 %0, 1, 0, p;\n\t}"
              : "=r"(any)
              : "r"(low & ~kTf32Mask), "n"(kM)
              : "memory");
          // `any` is the same in every thread of the four warps: one slot for the hi values and, only
          // when some value needs it, the next slot for the lo values
          const uint32_t as = ca.slot;
          if (ca.wraps >= 1) wait_or_dead(bar_afree + 8 * as, (ca.wraps - 1u) & 1u, dead);
          tc_fence_after();
          const uint32_t ah = tmem + lane_base + kColA + as * KCpad;
#pragma unroll
          for (int g8 = 0; g8 < KCpad / 8; ++g8) {
            uint32_t hi[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) hi[e] = v[g8 * 8 + e] & kTf32Mask;
            tmem_st8(ah + g8 * 8, hi);
          }
          tmem_st_wait();
          tc_fence_before();
          if (tid == 0) has_lo[as] = any;
          mbar_arrive(bar_aready + 8 * as);
          ca.next(NA);
          if (any) {
            const uint32_t as2 = ca.slot;
            if (ca.wraps >= 1) wait_or_dead(bar_afree + 8 * as2, (ca.wraps - 1u) & 1u, dead);
            tc_fence_after();
            const uint32_t al = tmem + lane_base + kColA + as2 * KCpad;
#pragma unroll
            for (int g8 = 0; g8 < KCpad / 8; ++g8) {
              uint32_t lo[8];
#pragma unroll
              for (int e = 0; e < 8; ++e) {
                const uint32_t h = v[g8 * 8 + e] & kTf32Mask;
                lo[e] = __float_as_uint(__fsub_rn(__uint_as_float(v[g8 * 8 + e]), __uint_as_float(h)));
              }
              tmem_st8(al + g8 * 8, lo);
            }
            tmem_st_wait();
            tc_fence_before();
            mbar_arrive(bar_aready + 8 * as2);
            ca.next(NA);
          }
        }
        // the oldest row of this tile is not read again
        mbar_arrive(bar_rawfree + 8 * rq.slot);
        rq.next(R);
      }
      // the item's last KH - 1 rows
      for (int q = g.Ho; q < Q; ++q, rq.next(R)) mbar_arrive(bar_rawfree + 8 * rq.slot);
    }
  } else {
    // ---------------- drain warps: accumulator -> output rows ----------------
    const int m = tid - kM, wl = m >> 5, tl = m & 31;
    const int ew = warp & 3;
    Cursor cd{0, 0};
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
        const uint32_t taddr = tmem + ((uint32_t)(ew * 32) << 16) + acc * (uint32_t)g.npad;
#pragma unroll 1
        for (int cb = 0; cb < g.npad; cb += 16) {
          uint32_t r[16];
          tmem_ld16(taddr + cb, r);
          tmem_ld_wait();
          if (ok && live_pos) {
#pragma unroll
            for (int e = 0; e < 16; ++e)
              if (cb + e < nco) dst[(cb + e) * cstride] = __uint_as_float(r[e]);
          }
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

// input channels per K-chunk: 3 x 3 -> 8 (72 columns, nine MMAs), 5 x 5 -> 2 (50 -> 56 columns, seven MMAs),
// 1 x 1 -> 32; picked so that common channel counts fill their chunks
constexpr int cig_for(int kh, int kw) { return kh * kw == 1 ? 32 : (kh * kw == 9 ? 8 : 2); }

struct TcPlan {
  ConvTc g;
  size_t smem;
  int cig;
  bool ok;
};

TcPlan plan_conv_tc(int64_t N, int64_t Ci, int64_t Co, int64_t H, int64_t W, int64_t kh, int64_t kw, int64_t ph,
                    int64_t pw, int64_t T) {
  TcPlan p{};
  p.ok = false;
  if (!((kh == 1 && kw == 1) || (kh == 3 && kw == 3) || (kh == 5 && kw == 5))) return p;
  if (T < kTT || (T & 3) || Ci > 256 || N > 65535 * 16 || H > (1 << 20) || W > (1 << 20) || T > (1 << 28)) return p;
  const int64_t Ho = H + 2 * ph - kh + 1, Wo = W + 2 * pw - kw + 1;
  if (Ho < 1 || Wo < 1) return p;
  const int cig = cig_for((int)kh, (int)kw);
  const int kc = cig * (int)(kh * kw), kcpad = (kc + 7) & ~7;
  const int nchunk = (int)((Ci + cig - 1) / cig);
  const int ngroup = (int)((Co + kAccCols - 1) / kAccCols);
  const int64_t co_last = Co - (int64_t)(ngroup - 1) * kAccCols;
  // every channel group is launched with the same MMA N: the widest group, padded to 16
  const int npad = (int)(((ngroup > 1 ? kAccCols : co_last) + 15) & ~15);
  const int slot = (int)(Ci * (kWG + kw - 1) * 128);
  const int64_t ktot = (int64_t)nchunk * kcpad;
  const int64_t b_bytes = (((ktot + 31) / 32) * npad * 128 + 1023) & ~1023LL;
  const int64_t fixed = 2 * b_bytes + 8 * (2 * kMaxRing + 4 * kMaxSlots) + 128 + 1024;
  // rows in flight beyond the kh live ones: as many as fit in about 200 KB, at most 16, at least 2
  int64_t ahead = (200 * 1024 - fixed) / slot - kh;
  if (ahead > 16) ahead = 16;
  if (ahead < 2 || ngroup > 65535) return p;
  const int R = (int)(kh + ahead);
  const int64_t smem = fixed + (int64_t)R * slot;
  p.g = ConvTc{(int)N, (int)Ci, (int)Co, (int)H, (int)W, (int)Ho, (int)Wo, (int)ph, (int)pw, (int)T, nchunk, npad,
               (int)((Wo + kWG - 1) / kWG), (int)((T + kTT - 1) / kTT), slot, R, (int)b_bytes};
  // at least 120 KB so that two CTAs (two TMEM allocations of 512 columns) never share an SM
  p.smem = (size_t)(smem < 120 * 1024 ? 120 * 1024 : smem);
  p.cig = cig;
  p.ok = true;
  return p;
}

}  // namespace

namespace sb {

// Runs the tensor-core convolution when the problem fits it; *taken says whether it did.
int conv_tc_try(const float* x, const float* weight, float* y, int64_t N, int64_t Ci, int64_t Co, int64_t H, int64_t W,
                int64_t kh, int64_t kw, int64_t ph, int64_t pw, int64_t T, cudaStream_t st, bool* taken) {
  *taken = false;
  if ((((uintptr_t)x) | ((uintptr_t)y)) & 15u) return SB_OK;
  const TcPlan p = plan_conv_tc(N, Ci, Co, H, W, kh, kw, ph, pw, T);
  if (!p.ok) return SB_OK;
  CUtensorMap xmap;
  const uint64_t dims[5] = {(uint64_t)T, (uint64_t)W, (uint64_t)H, (uint64_t)Ci, (uint64_t)N};
  const uint32_t box[5] = {(uint32_t)kTT, (uint32_t)(kWG + kw - 1), 1u, (uint32_t)Ci, 1u};
  int rc = make_map_5d(&xmap, x, dims, box);
  if (rc != SB_OK) return rc;
  const int64_t nitems = (int64_t)p.g.N * p.g.nwg * p.g.ntc;
  const int ngroup = (int)((Co + kAccCols - 1) / kAccCols);
  const int gx = (int)(nitems < sm_count() ? nitems : sm_count());
  const dim3 grid((unsigned)gx, (unsigned)ngroup);
  unsigned int* status = status_ptr();
  if (!status) return SB_ERR_CUDA;
#define SB_GO(KH, KW, CIG)                                                                                   \
  {                                                                                                          \
    auto fn = conv_tc_kernel<KH, KW, CIG>;                                                                   \
    SB_CUDA(cudaFuncSetAttribute((const void*)fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)p.smem)); \
    fn<<<grid, kThreads, p.smem, st>>>(xmap, weight, y, p.g, status);                                        \
  }
  if (kh == 1) SB_GO(1, 1, cig_for(1, 1))
  else if (kh == 3) SB_GO(3, 3, cig_for(3, 3))
  else SB_GO(5, 5, cig_for(5, 5))
#undef SB_GO
  SB_CUDA(cudaGetLastError());
  *taken = true;
  return SB_OK;
}

}  // namespace sb

// the contraction must be long enough for the tile hand-offs to pay off (measured: 5 x 5 over two
// channels, 50 taps, runs faster on the fp32 kernel; 3 x 3 over sixteen, 144 taps, twice as fast here)
constexpr int64_t kMinTapsForAuto = 64;

extern "C" int sb_conv_fits_tensor_cores(int64_t N, int64_t Ci, int64_t Co, int64_t H, int64_t W, int64_t kh,
                                         int64_t kw, int64_t ph, int64_t pw, int64_t T) {
  return plan_conv_tc(N, Ci, Co, H, W, kh, kw, ph, pw, T).ok ? 1 : 0;
}

extern "C" int sb_conv_uses_tensor_cores(int64_t N, int64_t Ci, int64_t Co, int64_t H, int64_t W, int64_t kh,
                                         int64_t kw, int64_t ph, int64_t pw, int64_t T) {
  return (Ci * kh * kw >= kMinTapsForAuto && plan_conv_tc(N, Ci, Co, H, W, kh, kw, ph, pw, T).ok) ? 1 : 0;
}
