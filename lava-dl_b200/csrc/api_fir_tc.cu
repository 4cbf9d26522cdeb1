// Temporal filter (utils/filter/conv.py:48-97) on the 5th-generation tensor
// cores: conv / corr of a [rows, T] tensor with K <= 64 taps as a banded
// (Toeplitz) matrix product, with fp32-level accuracy from three TF32 products.
//
//   y[r, t0 + n] = Ts * sum_k  W[r, k] * B[n, k]        n in [0, 32), k in [0, 96)
//   W[r, k]      = x[r, w0 + k]   (w0 = t0 - 64 for conv, t0 for corr; zero outside [0, T))
//   B[n, k]      = h[n + 64 - k]  (conv)   |   h[k - n]  (corr)       zero outside [0, K)
//
// A tile is 128 rows x 32 outputs: M = 128, N = 32, K = 96 in three 32-step
// boxes.  The SIMT kernel (api_fir.cu) spends 64 FMAs per output and is bound by
// the FP32 pipe at 0.43 of the HBM roof; here the multiply-adds run on
// tcgen05.mma (kind::tf32) and the kernel streams x once and out once.
//
// Accuracy: every operand is split as v = hi + lo with hi a TF32 value (10
// mantissa bits) and lo = v - hi; the tile accumulates hi*hi + hi*lo + lo*hi in
// fp32 (TMEM).  The filter is split once with round-to-nearest (cvt.rna); x is
// split per box by truncation (hi = v & mask, lo = v - hi exactly), and the
// tensor core keeps the top 11 bits of lo.  What is lost per product -- the tail
// of lo and the lo*lo term -- is below 2^-20 of the product.  A box of x whose
// values are all exact in TF32 (spike trains) skips its lo products.
//
// Data flow per CTA (persistent over 128-row blocks, 1 CTA per SM, 10 warps):
//   producer (1 thread): TMA boxes (32 steps x 128 rows, SWIZZLE_128B) into a
//     ring of 11 landing slots in shared memory; a slot is free again as soon as
//     the split warps have read it, so ~10 boxes (160 KB) are in flight per SM.
//   split (4 warps, one row per thread): box -> registers -> hi / lo -> TMEM
//     (tcgen05.st) into a ring of 6 operand slots.  The A operand of the MMAs is
//     read from TMEM, which is what frees the shared memory for the deep ring.
//   issue (1 thread): per tile 3 boxes x 4 K-steps x {A_hi x [B_hi; B_lo] as one
//     N = 64 product, A_lo x B_hi with N = 32} into one of two 64-column TMEM
//     accumulators; B (the Toeplitz factor, 24 KB) stays in shared memory.  An
//     MMA costs ~46 cycles to issue whatever its N <= 64, so merging the two B
//     factors along N saves a third of the instructions.
//   drain (4 warps, one row per thread): tcgen05.ld, add the two halves, scale,
//     stage the row's eight 128-bit words in shared memory (4 KB per warp) and
//     write them with a (4 rows x 128 bytes) per instruction mapping -- one row
//     per lane would cost 32 L1 wavefronts per store instruction.
//   TMEM columns: 2 x 64 accumulators, 6 operand slots of 32 A_hi | 32 A_lo = 512.
// Fused delay (axon.delay): shift(corr(g), -d) shifts the output, and
// conv(shift(x, d)) equals shift(conv(x), d) for d >= 0 (a delay only prepends
// zeros), so both are the same tiles written at a per-row offset s = 4 sq + e.
// The split warps delay the row's operand by e (0..3 steps, the leading values
// carried over from the row's previous box), so the accumulator already holds
// the row shifted by e and the drain moves whole 128-bit words by sq and
// zero-fills what the shift uncovers.  A negative delay on the input side (an
// advance) drops the first |d| samples before the filter sees them; then every
// row takes two more tiles past T, and advanced rows subtract the dropped
// samples' contribution from their first K - 1 outputs.
// Every mbarrier wait is bounded; a wait that runs out sets a CTA-wide flag that
// ends all other waits at once, SB_DEV_TMA_TIMEOUT is recorded, and the CTA
// waits (bounded) for loads and MMAs in flight, frees its TMEM and returns.
#include "api_util.cuh"
#include "tc.cuh"

using namespace sb;

namespace {

// The filter's waits sleep 64 ns from the third failed poll on: the waiting warps of the other roles then
// leave the issue slots of their scheduler to the warp that works (1.7 % faster than with 64 polls before
// the first sleep of 32 ns; sleeping from the first poll on is slower again).
__device__ __forceinline__ bool wait_fir(uint32_t bar, uint32_t parity, volatile int* dead) {
  return wait_or_dead(bar, parity, dead, 1u, 64u);
}

constexpr int kM = 128;                  // rows per block = MMA M
constexpr int kN = 32;                   // outputs per tile = steps per box
constexpr int kBoxBytes = kM * kN * 4;   // 16 KB
constexpr int kNumIssue = 2;             // MMA-issuing threads, one accumulator each
constexpr int kARing = (512 - kNumIssue * 2 * kN) / (2 * kN);   // operand slots in TMEM: 3 in use, the rest ahead
constexpr int kBBoxBytes = 2 * kN * 128; // one 64 x 32 box of the Toeplitz factor: rows 0-31 hi, 32-63 lo
constexpr int kAccCols = 2 * kN;         // hi*hi + lo*hi | hi*lo
constexpr int kColA = kNumIssue * kAccCols;      // operand slot s at kColA + 64 s, hi | lo
constexpr int kTmemCols = 512;

// warps: split 0-3, drain 4-7, two issue warps, producer warp
constexpr int kIssueWarp = 8, kProdWarp = kIssueWarp + kNumIssue;
constexpr int kThreads = 32 * (kProdWarp + 1);
constexpr int kRing = 11;                                // landing slots in shared memory
constexpr int kOffRaw = 0;
constexpr int kOffB = kOffRaw + kRing * kBoxBytes;
constexpr int kOffStage = kOffB + 3 * kBBoxBytes;        // output staging, 4 KB private to each drain warp
constexpr int kOffSq = kOffStage + kBoxBytes;            // 128 row shifts (>> 2)
constexpr int kOffBar = kOffSq + kM * 4;
// barriers: full[kRing], raw_free[kRing], a_ready[kARing], a_free[kARing], mma_done[kNumIssue], acc_free[kNumIssue];
// then the TMEM base word, the dead flag, has_lo[kARing]
constexpr int kNumBars = 2 * kRing + 2 * kARing + 2 * kNumIssue;
constexpr int kSmemBytes = kOffBar + 8 * kNumBars + 8 + 4 * kARing + 8 + 1024;  // + slack to align the base
static_assert(kSmemBytes <= 227 * 1024, "shared memory budget");
static_assert(kColA + kARing * 2 * kN == kTmemCols, "TMEM column budget");

__host__ __device__ constexpr uint32_t idesc_n(int n) { return idesc_tf32(kM, n); }

__global__ void __launch_bounds__(kThreads, 1)
fir_tc_kernel(const __grid_constant__ CUtensorMap xmap, const float* __restrict__ x, const float* __restrict__ filt,
              int K, int corr, const float* __restrict__ lut, int64_t n_lut, float shift, float shift_ts, int mode,
              float ts, float* __restrict__ out, int64_t rows, int T, unsigned int* status) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* sm = smem_raw + (base - smem_u32(smem_raw));
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t bar_full = base + kOffBar;
  const uint32_t bar_rawfree = bar_full + 8 * kRing;
  const uint32_t bar_aready = bar_rawfree + 8 * kRing;
  const uint32_t bar_afree = bar_aready + 8 * kARing;
  const uint32_t bar_mma = bar_afree + 8 * kARing;
  const uint32_t bar_free = bar_mma + 8 * kNumIssue;
  volatile uint32_t* tmem_word = reinterpret_cast<volatile uint32_t*>(sm + kOffBar + 8 * kNumBars);
  volatile int* dead = reinterpret_cast<volatile int*>(sm + kOffBar + 8 * kNumBars + 4);
  volatile int* has_lo = reinterpret_cast<volatile int*>(sm + kOffBar + 8 * kNumBars + 8);  // [kARing]

  if (tid == 0) {
    for (int i = 0; i < kRing; ++i) {
      mbar_init(bar_full + 8 * i, 1);
      mbar_init(bar_rawfree + 8 * i, kM);
    }
    for (int i = 0; i < kARing; ++i) {
      mbar_init(bar_aready + 8 * i, kM);
      mbar_init(bar_afree + 8 * i, 4);   // one arrival per drain warp
    }
    for (int i = 0; i < kNumIssue; ++i) {
      mbar_init(bar_mma + 8 * i, 1);
      mbar_init(bar_free + 8 * i, kM);
    }
    *dead = 0;
    fence_mbar_init();
  }
  if (warp == kIssueWarp) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(base + kOffBar + 8 * kNumBars), "r"(kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }

  // Is any input-side delay negative?  Then filter outputs past T reach the
  // result and two more tiles are computed there.  Every CTA scans the whole
  // table so that all agree without a second kernel or scratch.
  int wrong = 0;
  if (mode > 0) {
    const int64_t n = lut ? n_lut : 1;
    for (int64_t i = tid; i < n; i += kThreads) {
      const float sv = lut ? __ldg(lut + i) : shift;
      wrong |= __float2int_rz(__fdiv_rn(sv, shift_ts)) < 0;
    }
  }
  // Toeplitz factor, split, in the swizzled K-major layout: row n holds the hi
  // part for output n, row 32 + n the lo part.
  for (int e = tid; e < kN * 96; e += kThreads) {
    const int n = e / 96, k = e - n * 96;
    const int m = corr ? (k - n) : (n + 64 - k);
    const float v = (m >= 0 && m < K) ? __fmul_rn(__ldg(filt + m), ts) : 0.f;   // Ts folded into the factor
    const uint32_t hi = tf32_rn(v), lo = tf32_rn(__fsub_rn(v, __uint_as_float(hi)));
    const int kk = k & 31;
    const int off = (k >> 5) * kBBoxBytes + n * 128 + ((((kk >> 2) ^ (n & 7))) << 4) + ((kk & 3) << 2);
    *reinterpret_cast<uint32_t*>(sm + kOffB + off) = hi;
    *reinterpret_cast<uint32_t*>(sm + kOffB + off + kN * 128) = lo;  // row n + 32: same swizzle phase
  }
  fence_proxy_async();
  tc_fence_before();
  wrong = __syncthreads_or(wrong);
  tc_fence_after();
  const uint32_t tmem = *tmem_word;

  // a shifted row's filter output is delayed by up to 3 steps before it is moved by whole words
  const int nt = (T + (mode != 0 ? 3 : 0) + kN - 1) / kN;
  const int ntile = nt + (wrong ? 2 : 0);
  const int narr = ntile + 2;                 // boxes per block
  const int qoff = corr ? 2 : 0;
  const int ngroups = T >> 2;
  const int64_t nblk = (rows + kM - 1) / kM;
  const int64_t my_nblk = blockIdx.x < nblk ? (nblk - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
  const int64_t total = my_nblk * narr;

  if (warp == kProdWarp) {
    // ---------------- producer: TMA requests (one thread) ----------------
    if (lane == 0) {
      int slot = 0, a = 0, row0 = (int)(blockIdx.x * kM);
      uint32_t use = 0;
      int64_t f = 0;
      for (; f < total; ++f) {
        if (use >= 1 && !wait_fir(bar_rawfree + 8 * slot, (use - 1u) & 1u, dead)) break;
        const uint32_t bar = bar_full + 8 * slot;
        mbar_expect_tx(bar, kBoxBytes);
        tma_load_2d(base + kOffRaw + slot * kBoxBytes, &xmap, kN * (a - 2 + qoff), row0, bar);
        if (++a == narr) { a = 0; row0 += (int)(gridDim.x * kM); }
        if (++slot == kRing) { slot = 0; ++use; }
      }
      if (*dead) {
        // loads still in flight must land before the shared memory is given back
        for (int i = 0; i < kRing; ++i) { mbar_wait(bar_full + 8 * i, 0); mbar_wait(bar_full + 8 * i, 1); }
      }
    }
    __syncwarp();
  } else if (warp >= kIssueWarp && warp < kIssueWarp + kNumIssue) {
    // ---------------- issue: the MMAs of every other tile (one thread per warp) ----------------
    // One thread issues an MMA every ~46 cycles whatever its size; two threads do twice that.
    const uint32_t me = (uint32_t)(warp - kIssueWarp);   // this thread's accumulator
    if (lane == 0) {
      const uint32_t b0 = desc_lo(base + kOffB);
      int a = 0, as = 0, as1 = 0, as2 = 0;    // operand slots of this arrival and the two before it
      uint32_t ause = 0, tcount = 0;
      for (int64_t f = 0; f < total; ++f) {
        if (a >= 2) {
          if (tcount % kNumIssue == me) {
            const uint32_t acc = me;
            bool ok2;
            ok2 = wait_fir(bar_aready + 8 * as, ause & 1u, dead);
            if (tcount >= kNumIssue) ok2 = wait_fir(bar_free + 8 * acc, (tcount / kNumIssue - 1u) & 1u, dead) && ok2;
            tc_fence_after();
            if (ok2) {
              const uint32_t d_tmem = tmem + acc * kAccCols;
              const int slots[3] = {as2, as1, as};
#pragma unroll
              for (int c = 0; c < 3; ++c) {
                const uint32_t ah = tmem + kColA + (uint32_t)slots[c] * (2 * kN);
                const uint32_t al = ah + kN;
                const uint32_t bb = b0 + c * (kBBoxBytes >> 4);
                const bool lo = has_lo[slots[c]] != 0;
#pragma unroll
                for (int ks = 0; ks < 4; ++ks) {
                  // columns 0-31 += A_hi B_hi, columns 32-63 += A_hi B_lo; then columns 0-31 += A_lo B_hi
                  umma_ts(d_tmem, ah + 8 * ks, bb + 2 * ks, idesc_n(2 * kN), (c | ks) ? 1u : 0u);
                  if (lo) umma_ts(d_tmem, al + 8 * ks, bb + 2 * ks, idesc_n(kN), 1u);
                }
              }
            }
            umma_commit(bar_mma + 8 * acc);
          }
          ++tcount;
        }
        if (++a == narr) a = 0;
        as2 = as1; as1 = as;
        if (++as == kARing) { as = 0; ++ause; }
      }
      // nothing may still be writing TMEM when it is freed: wait for this thread's last tile
      if (tcount > me) {
        const uint32_t own = (tcount - 1u - me) / kNumIssue + 1u;   // tiles this thread issued
        mbar_wait(bar_mma + 8 * me, (own - 1u) & 1u);
      }
    }
    __syncwarp();
  } else if (warp < 4) {
    // ---------------- split warps: landing slot -> hi / lo in TMEM ----------------
    // A row shifted by s = 4 sq + e (e in 0..3) is filtered from its input delayed by e: the
    // operand row is W[k - e], the e leading values carried over from the previous box of the
    // row, so what the drain sees is already shifted by e and it only moves whole 128-bit words.
    int slot = 0, as = 0, a = 0, e_row = 0;
    uint32_t use = 0, ause = 0;
    uint32_t p0 = 0, p1 = 0, p2 = 0;            // the previous box's values 29..31 of this row
    int64_t blk = blockIdx.x;
    const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
    for (int64_t f = 0; f < total; ++f) {
      if (a == 0) {
        e_row = 0;
        const int64_t row = blk * kM + tid;
        if (mode != 0 && row < rows) {
          const float sv = lut ? __ldg(lut + (row % n_lut)) : shift;
          e_row = (max(-T, min(T, __float2int_rz(__fdiv_rn(sv, shift_ts)))) * mode) & 3;
        }
        p0 = p1 = p2 = 0;
      }
      if (++a == narr) { a = 0; blk += gridDim.x; }
      wait_fir(bar_full + 8 * slot, use & 1u, dead);
      const uint8_t* rowp = sm + kOffRaw + slot * kBoxBytes + tid * 128;
      uint32_t xr[32];
      uint32_t low = 0;
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        const uint4 q = *reinterpret_cast<const uint4*>(rowp + ((c ^ (tid & 7)) << 4));
        xr[4 * c] = q.x; xr[4 * c + 1] = q.y; xr[4 * c + 2] = q.z; xr[4 * c + 3] = q.w;
        low |= q.x | q.y | q.z | q.w;
      }
      low |= p0 | p1 | p2;   // values carried in from the previous box land in this operand too
      // Does any value of the box need a lo part?  (Spike trains do not.)  The
      // barrier also orders every thread's reads of the slot before its release.
      int any;
      asm volatile(
          "{\n\t.reg .pred p, q;\n\t"
          "setp.ne.b32 q, %1, 0;\n\t"
          "bar.red.or.pred p, 1, %2, q;\n\t"
          "selp.s32 %0, 1, 0, p;\n\t}"
          : "=r"(any)
          : "r"(low & ~kTf32Mask), "n"(kM)
          : "memory");
      mbar_arrive(bar_rawfree + 8 * slot);
      if (mode != 0) {
        // delay the row by e steps without diverging: by 2 if (e & 2), then by 1 if (e & 1)
        const uint32_t n0 = xr[29], n1 = xr[30], n2 = xr[31];
        const bool by2 = (e_row & 2) != 0, by1 = (e_row & 1) != 0;
        uint32_t t0 = by2 ? p0 : p2;             // element -1 after the first stage
#pragma unroll
        for (int j = 31; j >= 2; --j) xr[j] = by2 ? xr[j - 2] : xr[j];
        xr[1] = by2 ? p2 : xr[1];
        xr[0] = by2 ? p1 : xr[0];
#pragma unroll
        for (int j = 31; j >= 1; --j) xr[j] = by1 ? xr[j - 1] : xr[j];
        xr[0] = by1 ? t0 : xr[0];
        p0 = n0; p1 = n1; p2 = n2;
      }
      // the MMAs that read this operand slot's previous box have completed?
      if (ause >= 1) wait_fir(bar_afree + 8 * as, (ause - 1u) & 1u, dead);
      tc_fence_after();
      if (any) {
        uint32_t hl[64];
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          // hi = x truncated to TF32 (exact in the operand format), lo = x - hi exactly (13
          // bits, of which the tensor core keeps 11): two instructions per value
          const uint32_t h = xr[j] & kTf32Mask;
          hl[32 + j] = __float_as_uint(__fsub_rn(__uint_as_float(xr[j]), __uint_as_float(h)));
          hl[j] = h;
        }
        tmem_st64(tmem + lane_base + kColA + as * (2 * kN), hl);   // hi | lo side by side: one store
      } else {
        tmem_st32(tmem + lane_base + kColA + as * (2 * kN), xr);
      }
      tmem_st_wait();
      tc_fence_before();
      if (tid == 0) has_lo[as] = any;
      mbar_arrive(bar_aready + 8 * as);
      if (++slot == kRing) { slot = 0; ++use; }
      if (++as == kARing) { as = 0; ++ause; }
    }
  } else {
    // ---------------- drain warps: accumulator -> rows of the result ----------------
    // Rows differ only in the word offset sq of their shift.
    const int et = tid - kM;                     // row inside the block
    const int ew = warp & 3;                     // TMEM lane quarter
    int s_row = 0;
    int64_t blk = blockIdx.x;
    uint32_t tcount = 0;
    int oldest = 0;                              // operand slot of the oldest box of the current tile
    uint8_t* stage = sm + kOffStage;                        // rows 32 ew .. 32 ew + 31 are this warp's
    int* sq_s = reinterpret_cast<int*>(sm + kOffSq);
    for (int64_t b = 0; b < my_nblk; ++b, blk += gridDim.x) {
      const int64_t row = blk * kM + et;
      for (int tile = 0; tile < ntile; ++tile, ++tcount) {
        const int acc = (int)(tcount % kNumIssue);
        bool ok;
        ok = wait_fir(bar_mma + 8 * acc, (tcount / kNumIssue) & 1u, dead);
        tc_fence_after();
        // This warp has now seen every tile up to this one complete, so nothing reads the tile's
        // oldest box any more (nor, after a block's last tile, the two newer ones): the operand
        // slots go back to the split warps from here.  A commit per slot from the issue threads
        // would do the same, but every tcgen05 instruction takes its turn on the issue path that
        // the MMAs need, and three commits per tile cost as much there as five MMAs.
        if (lane == 0) {
          const int nfree = (tile == ntile - 1) ? 3 : 1;
          for (int i = 0; i < nfree; ++i) {
            mbar_arrive(bar_afree + 8 * oldest);
            if (++oldest == kARing) oldest = 0;
          }
        }
        uint32_t r[64];
        const uint32_t taddr = tmem + ((uint32_t)(ew * 32) << 16) + (uint32_t)(acc * kAccCols);
        tmem_ld64(taddr, r);
        tmem_ld_wait();
        tc_fence_before();
        mbar_arrive(bar_free + 8 * acc);
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = __fadd_rn(__uint_as_float(r[j]), __uint_as_float(r[32 + j]));

        const bool live = row < rows && ok;
        float* rowp = out + (live ? row : 0) * (int64_t)T;
        if (tile == 0) {
          s_row = 0;
          if (mode != 0 && live) {
            const float sv = lut ? __ldg(lut + (row % n_lut)) : shift;
            s_row = max(-T, min(T, __float2int_rz(__fdiv_rn(sv, shift_ts)))) * mode;
          }
          sq_s[et] = s_row >> 2;
          if (live) {
            // zeros before the row's first word and after its last one
            const int gfirst = min(ngroups, s_row >> 2);
            for (int G = 0; G < gfirst; ++G) reinterpret_cast<float4*>(rowp)[G] = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int G = max(8 * ntile + (s_row >> 2), 0); G < ngroups; ++G)
              reinterpret_cast<float4*>(rowp)[G] = make_float4(0.f, 0.f, 0.f, 0.f);
          }
        }
        if (mode > 0 && s_row < 0 && live) {
          // advance by nd: outputs 0 .. K-2 must not see x[0 .. nd).  Tile value j sits at
          // output 32 tile + j + s_row - e (the tile is already delayed by e = s_row & 3).
          const int nd = -s_row, tbase = kN * tile - (s_row & 3);
          if (tbase < nd + K - 1 && tbase + kN > nd) {
            const float* xrow = x + row * (int64_t)T;
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const int po = tbase + j - nd;
              if (po >= 0 && po <= K - 2) {
                float c = 0.f;
                for (int q = max(0, po + nd - K + 1); q < nd; ++q)
                  c = fmaf(__ldg(filt + (po + nd - q)), __ldg(xrow + q), c);
                v[j] = __fsub_rn(v[j], __fmul_rn(c, ts));
              }
            }
          }
          if (s_row <= -T) {   // a row advanced by T or more is empty
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = 0.f;
          }
        }
        if (mode < 0 && tile == 0) {
          // corr reaches forward, so its output is not zero before t = 0; the e values the
          // delayed operand puts there belong to the zero fill
          const int e = s_row & 3;
          if (e > 0) v[0] = 0.f;
          if (e > 1) v[1] = 0.f;
          if (e > 2) v[2] = 0.f;
        }
        {
          uint8_t* stage_row = stage + et * 128;
#pragma unroll
          for (int g = 0; g < 8; ++g)
            *reinterpret_cast<float4*>(stage_row + ((g ^ (et & 7)) << 4)) =
                make_float4(v[4 * g], v[4 * g + 1], v[4 * g + 2], v[4 * g + 3]);
        }
        __syncwarp();
        // coalesced write-out of the warp's 32 rows: an instruction covers 4 rows x 128 bytes
        if (ok) {
          const int g = lane & 7;
          const int rl0 = ew * 32 + (lane >> 3);
          float* orow = out + (blk * kM + rl0) * (int64_t)T;
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const int rl = rl0 + 4 * k;
            const float4 w = *reinterpret_cast<const float4*>(stage + rl * 128 + ((g ^ (rl & 7)) << 4));
            const int G = 8 * tile + sq_s[rl] + g;
            if (blk * kM + rl < rows && G >= 0 && G < ngroups)
              reinterpret_cast<float4*>(orow + (int64_t)(4 * k) * T)[G] = w;
          }
        }
        __syncwarp();
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

}  // namespace

static bool tc_shape_ok(int64_t K, int64_t rows, int64_t T) {
  return K >= 1 && K <= 64 && T >= kN && (T & 3) == 0 && rows >= kM && T <= (1 << 30);
}

namespace sb {

// Runs the tensor-core filter when the problem fits it; *taken says whether it
// did.  mode: 0 plain, +1 output shifted by +delay (conv of a delayed input),
// -1 output shifted by -delay (adjoint).
int fir_tc_try(const float* x, const float* filt, int64_t K, bool corr, const float* lut, int64_t n_lut, float shift,
               float shift_ts, int mode, float ts, float* out, int64_t rows, int64_t T, cudaStream_t st,
               bool* taken) {
  *taken = false;
  if (!tc_shape_ok(K, rows, T)) return SB_OK;
  if ((mode > 0 && corr) || (mode < 0 && !corr)) return SB_OK;
  if ((((uintptr_t)x) | ((uintptr_t)out)) & 15u) return SB_OK;
  if (lut && n_lut > (1 << 22)) return SB_OK;
  CUtensorMap xmap;
  int rc = make_row_map_box(&xmap, x, rows, T, kN, kM);
  if (rc != SB_OK) return rc;
  static bool configured[64] = {false};
  int dev = 0;
  SB_CUDA(cudaGetDevice(&dev));
  if (dev < 64 && !configured[dev]) {
    SB_CUDA(cudaFuncSetAttribute(fir_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
    configured[dev] = true;
  }
  const int64_t nblk = (rows + kM - 1) / kM;
  const int grid = (int)(nblk < sm_count() ? nblk : sm_count());
  fir_tc_kernel<<<grid, kThreads, kSmemBytes, st>>>(xmap, x, filt, (int)K, corr ? 1 : 0, lut, n_lut, shift, shift_ts, mode,
                                                    ts, out, rows, (int)T, status_ptr());
  SB_CUDA(cudaGetLastError());
  *taken = true;
  return SB_OK;
}

}  // namespace sb

extern "C" int sb_fir_uses_tensor_cores(int64_t K, int64_t rows, int64_t T) { return tc_shape_ok(K, rows, T) ? 1 : 0; }
