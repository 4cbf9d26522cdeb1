// Shared device/host helpers for the SLAYER hot-path kernels (sm_100a only).
//
// Everything here is plain CUDA C++: no torch headers, no exceptions across the
// C boundary.  Integer semantics follow the CPU implementation of lava-dl
// (src/lava/lib/dl/slayer/neuron/dynamics/*.py), not its .cu files.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/slayer_b200.h"

namespace sb {

// ---------------------------------------------------------------------------
// Host-side error plumbing
// ---------------------------------------------------------------------------
void set_error(const char* fmt, ...);
int cuda_fail(cudaError_t e, const char* what);

#define SB_REQUIRE(cond, ...)                 \
  do {                                        \
    if (!(cond)) {                            \
      ::sb::set_error(__VA_ARGS__);           \
      return SB_ERR_INVALID_ARG;              \
    }                                         \
  } while (0)

#define SB_CUDA(call)                                     \
  do {                                                    \
    cudaError_t e__ = (call);                             \
    if (e__ != cudaSuccess) return ::sb::cuda_fail(e__, #call); \
  } while (0)

// Sticky device-side status word (bit flags, see SB_DEV_* in the public header).
// Kernels only ever OR bits into it; sb_device_status() reads and clears it.
// The word lives in one translation unit; kernels receive its device address
// as an argument (status_ptr() resolves it once per device).
unsigned int* status_ptr();

__device__ __forceinline__ void dev_flag(unsigned int* status, unsigned int bits) { atomicOr(status, bits); }

// ---------------------------------------------------------------------------
// Row -> parameter index.  A "row" is one neuron of one sample (T contiguous
// floats).  Per-channel parameters are indexed the way the reference kernels do
// (neuron/dynamics/leaky_integrator.cu:46-52): channel = (row % rows_per_batch)
// / decay_block, which equals the CPU broadcast for NCT tensors.
// ---------------------------------------------------------------------------
struct RowGeom {
  int64_t rows;            // B * prod(spatial)
  int64_t rows_per_batch;  // prod(spatial)
  int64_t decay_block;     // prod(spatial[1:])
  int T;
};

__device__ __forceinline__ int64_t param_index(const RowGeom& g, int64_t row, int64_t count) {
  if (count <= 1) return 0;
  return (row % g.rows_per_batch) / g.decay_block;
}

// ---------------------------------------------------------------------------
// Loihi fixed-point helpers
// ---------------------------------------------------------------------------

// trunc(a * m / 4096): utils/int_utils.py:9-31 (right_shift_to_zero) applied to
// the 64-bit product, any sign of a and m.
// floor((p + bias) / 4096) with bias = 4095 for a negative product equals
// trunc(p / 4096); the bias depends only on the operand signs, so it is formed
// off the multiply's critical path and rides in as the 64-bit addend of the
// widening multiply-add.
__device__ __forceinline__ int mul_shift12(int a, int m) {
  const long long bias = (long long)(((a ^ m) >> 31) & 4095);
  const long long p = (long long)a * (long long)m + bias;
  return (int)(p >> 12);
}

// Shorter forms of the same value for multipliers of limited size, used on the
// serial chain of the recurrences (every instruction there is latency).
//   trunc(a * m / 4096) = floor((16 * a * m + 65535 * [a * m < 0]) / 65536):
// 16 * a * m is a multiple of 16, so any bias in [65520, 65535] lands on the
// same quotient as 4095 does before the scaling, and 0xFFFF is what one byte
// permute with sign replication makes out of a sign bit.  The multiplier rides
// in pre-shifted (m16 = m << 4), so the chain is PRMT, IMAD.WIDE, SHF.
// sign16(x) = 0x0000FFFF for x < 0, else 0.
__device__ __forceinline__ uint32_t sign16(int x) {
  uint32_t d;
  asm("prmt.b32 %0, %1, 0, 0x44BB;" : "=r"(d) : "r"(x));
  return d;
}
// m16 = m << 4 with 0 <= m: the sign of the product is the sign of a.
__device__ __forceinline__ int mul_shift12_pos(int a, int m16) {
  const long long p = (long long)a * (long long)m16 + (long long)sign16(a);
  return (int)(p >> 16);
}
// m16 = m << 4 with |m| < 2^27, either sign.
__device__ __forceinline__ int mul_shift12_sym(int a, int m16) {
  const long long p = (long long)a * (long long)m16 + (long long)sign16(a ^ m16);
  return (int)(p >> 16);
}
// A multiplier the short forms may take (warp-uniform test at kernel start).
__device__ __forceinline__ bool mul_is_decay(int m) { return m >= 0 && m <= 4096; }

// (w_scale * x).to(int): one fp32 multiply (round to nearest), then truncation.
__device__ __forceinline__ int to_fixed(float w, float x) { return __float2int_rz(__fmul_rn(w, x)); }

// int_state / w_scale: int -> fp32 (round to nearest) then a true IEEE divide.
// With a power-of-two w_scale the multiply by the exact reciprocal is the same
// value; POW2 selects it at compile time.
template <bool POW2>
__device__ __forceinline__ float from_fixed(int v, float w, float inv_w) {
  float f = __int2float_rn(v);
  return POW2 ? __fmul_rn(f, inv_w) : __fdiv_rn(f, w);
}

// ---------------------------------------------------------------------------
// Shared-memory tile layout.  A tile is 32 rows x 32 time steps of fp32
// (128 B per row) stored with the 128-byte TMA swizzle: the 16-byte chunk c of
// row r lives at chunk position c ^ (r & 7).  Lane l owns row l, so a warp
// reading chunk c of every row touches all 32 banks exactly once per quarter
// warp (conflict-free 128-bit accesses), while TMA moves the tile as coalesced
// 128-byte row segments.
// ---------------------------------------------------------------------------
//
// Ops with three or more streams per stage use 16-step tiles instead (64 B per
// row, 64-byte swizzle: chunk c of row r at position c ^ ((r >> 1) & 3), again
// conflict free) to halve shared memory per warp and double resident warps.
constexpr int kTileT = 32;
constexpr int kTileR = 32;
constexpr int kTileBytes = kTileT * kTileR * 4;

template <int TW>
__device__ __forceinline__ uint32_t swz_chunk(int row, int chunk) {
  static_assert(TW == 32 || TW == 16, "tile width is 16 or 32 steps");
  if (TW == 32) return (uint32_t)(row * 128 + ((chunk ^ (row & 7)) << 4));
  return (uint32_t)(row * 64 + ((chunk ^ ((row >> 1) & 3)) << 4));
}
__device__ __forceinline__ uint32_t swz_elem(int row, int t) {
  return swz_chunk<32>(row, t >> 2) + ((t & 3) << 2);
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}

// ---------------------------------------------------------------------------
// mbarrier / TMA (cp.async.bulk.tensor) wrappers
// ---------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: a healthy load lands in microseconds; the limit is seconds.
// Returns false when it gave up (the caller records SB_DEV_TMA_TIMEOUT).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
  for (uint32_t it = 0; it < (1u << 22); ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if (it > 64) __nanosleep(it > 4096 ? 256 : 32);
  }
  return false;
}
__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cta.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, int x, int y, uint32_t src) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%1, %2}], [%3];"
               ::"l"(map), "r"(x), "r"(y), "r"(src)
               : "memory");
}
__device__ __forceinline__ void tma_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void tma_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N>
__device__ __forceinline__ void tma_wait_all() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

// ---------------------------------------------------------------------------
// Host: tensor-map construction and launch helpers (api_common.cu)
// ---------------------------------------------------------------------------

// Encodes a [rows, T] fp32 tensor as a 2-D tiled map with a 32x32 box and the
// 128-byte swizzle.  Fails (returns non-zero, error text set) when the driver
// entry point is missing or the tensor violates TMA's alignment rules; callers
// test tma_eligible() first and take the plain-load kernel otherwise.
int make_row_map(CUtensorMap* out, const void* base, int64_t rows, int64_t T, int tile_steps);
// Same with a box of box_rows rows (<= 256).
int make_row_map_box(CUtensorMap* out, const void* base, int64_t rows, int64_t T, int tile_steps, int box_rows);
bool tma_eligible(const void* const* ptrs, int n, int64_t T);

// Smallest int k with (float)k >= thr (the reference compares an integer tensor
// with a Python float, which PyTorch evaluates in fp32).  INT_MAX if none.
int int_threshold_ge(float thr);
// Smallest int k with (float)k / w >= thr, same reasoning for spike(v/w >= thr).
int int_threshold_ge_scaled(float thr, float w);

int sm_count();
bool is_pow2(int64_t v);

}  // namespace sb
