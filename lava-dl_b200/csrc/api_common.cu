// Host-side plumbing shared by every entry point: error text, the sticky device
// status word, tensor-map encoding, launch planning, the parameter-gradient
// fold kernel.
#include <stdarg.h>
#include <stdio.h>
#include <string.h>
#include <limits.h>

#include <atomic>

#include "common.cuh"
#include "rowscan.cuh"
#include "reduce.cuh"

namespace sb {

// ---------------------------------------------------------------------------
// errors
// ---------------------------------------------------------------------------
static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

int cuda_fail(cudaError_t e, const char* what) {
  set_error("CUDA error %d (%s) in %s", (int)e, cudaGetErrorString(e), what);
  return SB_ERR_CUDA;
}

// ---------------------------------------------------------------------------
// device status word
// ---------------------------------------------------------------------------
__device__ unsigned int g_dev_status = 0;

// Host-side caches are filled lazily and may be reached from several threads at once (autograd
// runs backward passes on worker threads): every cached value is the same whoever computes it, so
// the slots are atomics with release / acquire ordering and a lost race only repeats the lookup.
static constexpr int kMaxDev = 64;
static std::atomic<unsigned int*> g_status_ptr[kMaxDev];

unsigned int* status_ptr() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDev) {
    set_error("no usable CUDA device (cudaGetDevice failed)");
    return nullptr;
  }
  unsigned int* cached = g_status_ptr[dev].load(std::memory_order_acquire);
  if (!cached) {
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_dev_status);
    if (e != cudaSuccess) {
      cuda_fail(e, "cudaGetSymbolAddress(g_dev_status)");
      return nullptr;
    }
    cached = (unsigned int*)p;
    g_status_ptr[dev].store(cached, std::memory_order_release);
  }
  return cached;
}

// ---------------------------------------------------------------------------
// tensor maps
// ---------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn resolve_encode_fn() {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
      q == cudaDriverEntryPointSuccess)
    return (EncodeTiledFn)p;
  return nullptr;
}

static EncodeTiledFn encode_fn() {
  static const EncodeTiledFn fn = resolve_encode_fn();   // initialised once, thread-safe since C++11
  return fn;
}

bool tma_eligible(const void* const* ptrs, int n, int64_t T) {
  if (T < kTileT || (T & 3)) return false;
  for (int i = 0; i < n; ++i)
    if (((uintptr_t)ptrs[i]) & 15u) return false;
  return encode_fn() != nullptr;
}

// The encode call is a driver-API function and wants a context current on the
// calling thread.  A thread that was only handed a device number (an autograd
// worker, say) may have none bound yet.  The primary context of the device is
// retained once per device and made current on such threads; nothing is
// allocated or freed.
typedef CUresult (*CtxGetCurrentFn)(CUcontext*);
typedef CUresult (*CtxSetCurrentFn)(CUcontext);
typedef CUresult (*PrimaryRetainFn)(CUcontext*, CUdevice);
typedef CUresult (*DeviceGetFn)(CUdevice*, int);

static void* driver_fn(const char* name) {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
    return nullptr;
  return p;
}

static void bind_primary_context() {
  static CtxGetCurrentFn get_cur = (CtxGetCurrentFn)driver_fn("cuCtxGetCurrent");
  static CtxSetCurrentFn set_cur = (CtxSetCurrentFn)driver_fn("cuCtxSetCurrent");
  static PrimaryRetainFn retain = (PrimaryRetainFn)driver_fn("cuDevicePrimaryCtxRetain");
  static DeviceGetFn dev_get = (DeviceGetFn)driver_fn("cuDeviceGet");
  static std::atomic<CUcontext> primary[kMaxDev];
  if (!get_cur || !set_cur || !retain || !dev_get) return;
  CUcontext cur = nullptr;
  if (get_cur(&cur) == CUDA_SUCCESS && cur != nullptr) return;
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDev) return;
  CUcontext ctx = primary[dev].load(std::memory_order_acquire);
  if (!ctx) {
    CUdevice cd;
    if (dev_get(&cd, dev) != CUDA_SUCCESS || retain(&ctx, cd) != CUDA_SUCCESS) return;
    primary[dev].store(ctx, std::memory_order_release);
  }
  set_cur(ctx);
}

// L2 fetches 256 bytes per missed 128-byte tile row: the next tile of the same
// row (needed 32 steps later) is then an L2 hit and DRAM sees 256-byte reads.
// Measured: CUBA forward 0.76 -> 0.80 of copy bandwidth, LI forward 0.79 -> 0.84.
static constexpr CUtensorMapL2promotion kL2Promotion = CU_TENSOR_MAP_L2_PROMOTION_L2_256B;

int make_row_map(CUtensorMap* out, const void* base, int64_t rows, int64_t T, int tile_steps) {
  return make_row_map_box(out, base, rows, T, tile_steps, kTileR);
}

int make_row_map_box(CUtensorMap* out, const void* base, int64_t rows, int64_t T, int tile_steps, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) {
    set_error("cuTensorMapEncodeTiled is not available from this driver");
    return SB_ERR_UNSUPPORTED;
  }
  bind_primary_context();
  const cuuint64_t dims[2] = {(cuuint64_t)T, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)T * 4};
  const cuuint32_t box[2] = {(cuuint32_t)tile_steps, (cuuint32_t)box_rows};
  const CUtensorMapSwizzle swizzle = tile_steps == 16 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B;
  const cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, kL2Promotion,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled failed with CUresult %d (rows=%lld T=%lld base=%p)", (int)r, (long long)rows,
              (long long)T, base);
    return SB_ERR_CUDA;
  }
  return SB_OK;
}

// [d4][d3][d2][d1][d0] fp32 tensor, d0 contiguous, dense strides; boxes are stored unswizzled and
// out-of-range elements read as zero (which is how the convolution gets its padding).
// 5-D fp32 tensor map with explicit strides: dims[0] is the contiguous dimension, strides[i] is the
// byte stride of dims[i + 1] (multiples of 16; they need not grow with i, so the dimensions can be
// listed in the order the box should have in shared memory).  swizzle: 0 none, 1 the 128-byte pattern
// over 16-byte chunks, 2 the 128-byte pattern over 32-byte chunks (what an M-major TF32 operand of
// tcgen05.mma wants); the box's inner extent must then be 128 bytes.  Out-of-range coordinates read zeros.
int make_map_5d(CUtensorMap* out, const void* base, const uint64_t (&dims)[5], const uint64_t (&strides)[4],
                const uint32_t (&box)[5], int swizzle) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) {
    set_error("cuTensorMapEncodeTiled is not available from this driver");
    return SB_ERR_UNSUPPORTED;
  }
  bind_primary_context();
  cuuint64_t gdims[5], gstr[4];
  cuuint32_t gbox[5], estr[5];
  for (int i = 0; i < 5; ++i) {
    gdims[i] = dims[i];
    gbox[i] = box[i];
    estr[i] = 1;
    if (i < 4) gstr[i] = strides[i];
  }
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 5, const_cast<void*>(base), gdims, gstr, gbox, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE,
                  swizzle == 2 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B
                               : (swizzle == 1 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE),
                  CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled (5-D) failed with CUresult %d (dims %llu %llu %llu %llu %llu, base %p)", (int)r,
              (unsigned long long)dims[0], (unsigned long long)dims[1], (unsigned long long)dims[2],
              (unsigned long long)dims[3], (unsigned long long)dims[4], base);
    return SB_ERR_CUDA;
  }
  return SB_OK;
}

// ---------------------------------------------------------------------------
// thresholds: integer equivalents of fp32 comparisons
// ---------------------------------------------------------------------------
template <class Pred>
static int first_int_where(Pred pred) {  // pred monotone: false ... false true ... true
  long long lo = INT_MIN, hi = INT_MAX;
  if (!pred((int)hi)) return INT_MAX;
  while (lo < hi) {
    long long mid = lo + (hi - lo) / 2;
    if (pred((int)mid)) hi = mid; else lo = mid + 1;
  }
  return (int)lo;
}

int int_threshold_ge(float thr) {
  return first_int_where([thr](int k) { return (float)k >= thr; });
}
int int_threshold_ge_scaled(float thr, float w) {
  return first_int_where([thr, w](int k) {
    volatile float q = (float)k / w;
    return q >= thr;
  });
}

bool is_pow2(int64_t v) { return v > 0 && (v & (v - 1)) == 0; }

// ---------------------------------------------------------------------------
// launch planning
// ---------------------------------------------------------------------------
struct DevInfo {
  int sms;
  size_t smem_per_sm;
  size_t smem_per_block_optin;
  bool ok;
};
static DevInfo g_dev[kMaxDev];
static std::atomic<bool> g_dev_ready[kMaxDev];

static const DevInfo& dev_info() {
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= kMaxDev) dev = 0;
  DevInfo& d = g_dev[dev];
  if (!g_dev_ready[dev].load(std::memory_order_acquire)) {
    DevInfo n;
    int v = 0;
    n.sms = 148; n.smem_per_sm = 228 * 1024; n.smem_per_block_optin = 227 * 1024;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && v > 0) n.sms = v;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMaxSharedMemoryPerMultiprocessor, dev) == cudaSuccess && v > 0)
      n.smem_per_sm = (size_t)v;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev) == cudaSuccess && v > 0)
      n.smem_per_block_optin = (size_t)v;
    n.ok = true;
    d = n;   // racing threads write the same values
    g_dev_ready[dev].store(true, std::memory_order_release);
  }
  return d;
}

int sm_count() { return dev_info().sms; }

// Warps never talk to each other, so the CTA size only decides how shared
// memory is carved up.  Pick the warps-per-CTA (1..4) that keeps the most warps
// resident per SM (each CTA costs its dynamic bytes plus 1 KB the hardware
// reserves); small problems take one warp per CTA so every SM gets work.
LaunchPlan plan_rowscan(int64_t rows, size_t bytes_per_warp, size_t fixed_bytes) {
  const DevInfo& d = dev_info();
  const int64_t nwarps = (rows + kTileR - 1) / kTileR;
  int best_w = 1;
  long best_res = -1;
  for (int w = 1; w <= 4; ++w) {
    const size_t cta = w * bytes_per_warp + fixed_bytes;
    if (cta > d.smem_per_block_optin) break;
    long ctas = (long)(d.smem_per_sm / (cta + 1024));
    if (ctas > 32) ctas = 32;
    long res = ctas * w;
    if (res > 64) res = 64;
    if (res > best_res) { best_res = res; best_w = w; }
  }
  if (nwarps <= (int64_t)d.sms * best_res) {
    // not even one full wave: spread warps over SMs as evenly as possible
    int w = (int)((nwarps + d.sms - 1) / d.sms);
    if (w < 1) w = 1;
    if (w < best_w) best_w = w;
  }
  LaunchPlan lp;
  lp.warps_per_cta = best_w;
  lp.ctas = (nwarps + best_w - 1) / best_w;
  lp.smem = best_w * bytes_per_warp + fixed_bytes;
  return lp;
}

// Opt a kernel into large dynamic shared memory.  Cheap enough to call per
// launch; the attribute is per device and per function.
int prepare_kernel(const void* fn, size_t smem) {
  SB_CUDA(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  SB_CUDA(cudaFuncSetAttribute(fn, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
  return SB_OK;
}

// ---------------------------------------------------------------------------
// parameter-gradient fold
// ---------------------------------------------------------------------------
int64_t scratch_slots(int64_t rows, int64_t n) {
  const int64_t partials = (n <= 1) ? (rows + kTileR - 1) / kTileR : rows;
  return partials + kFoldSlices * (n < 1 ? 1 : n);
}

__global__ void fold_stage1(const double* __restrict__ partial, double* __restrict__ stage, RowGeom g, int64_t n,
                            int64_t nparts) {
  // grid: (slices, min(n, 65535)).  Block (s, c) sums the partials of channel c that fall in slice s;
  // with more channels than the grid's second dimension allows a block takes every gridDim.y-th one.
  const int s = blockIdx.x;
  for (int64_t c = blockIdx.y; c < (n < 1 ? 1 : n); c += gridDim.y) {
    double acc = 0.0;
    if (n <= 1) {
      for (int64_t i = (int64_t)s * blockDim.x + threadIdx.x; i < nparts; i += (int64_t)gridDim.x * blockDim.x)
        acc += partial[i];
    } else {
      // rows of channel c: for each batch b, [b*rpb + c*blk, b*rpb + (c+1)*blk)
      const int64_t batches = g.rows / g.rows_per_batch;
      const int64_t per = batches * g.decay_block;
      for (int64_t i = (int64_t)s * blockDim.x + threadIdx.x; i < per; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t b = i / g.decay_block, j = i - b * g.decay_block;
        acc += partial[b * g.rows_per_batch + c * g.decay_block + j];
      }
    }
    acc = block_sum(acc);
    if (threadIdx.x == 0) stage[c * gridDim.x + s] = acc;
    __syncthreads();   // block_sum's shared slots are reused by the next channel
  }
}

__global__ void fold_stage2(const double* __restrict__ stage, float* __restrict__ out, int slices, int64_t n) {
  const int64_t c = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (c >= n) return;
  const int lane = threadIdx.x & 31;
  double acc = 0.0;
  for (int s = lane; s < slices; s += 32) acc += stage[c * slices + s];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (lane == 0) out[c] = (float)acc;
}

// One parameter per row of a [batch, n] problem (time-major rows, no spatial block under the
// channel): thread (x, y) of a 32 x 8 block adds every eighth batch entry of channel x, so a warp
// reads 32 neighbouring partials, and the eight slices meet in shared memory.  One launch, no stage
// buffer: with 64 batch entries per channel the sliced fold below would start 64 x n blocks to add
// 64 numbers each.
__global__ void fold_columns(const double* __restrict__ partial, float* __restrict__ out, int64_t n, int64_t batches) {
  __shared__ double part[8][33];
  const int64_t c = (int64_t)blockIdx.x * 32 + threadIdx.x;
  double acc = 0.0;
  if (c < n)
    for (int64_t b = threadIdx.y; b < batches; b += 8) acc += partial[b * n + c];
  part[threadIdx.y][threadIdx.x] = acc;
  __syncthreads();
  if (threadIdx.y == 0 && c < n) {
#pragma unroll
    for (int y = 1; y < 8; ++y) acc += part[y][threadIdx.x];
    out[c] = (float)acc;
  }
}

int fold_param_grad(double* scratch, float* out, const RowGeom& g, int64_t n, cudaStream_t st) {
  if (n < 1) n = 1;
  if (n > 1 && g.decay_block == 1 && g.rows_per_batch == n) {
    fold_columns<<<(unsigned)((n + 31) / 32), dim3(32, 8), 0, st>>>(scratch, out, n, g.rows / g.rows_per_batch);
    SB_CUDA(cudaGetLastError());
    return SB_OK;
  }
  const int64_t nparts = (n <= 1) ? (g.rows + kTileR - 1) / kTileR : g.rows;
  double* stage = scratch + nparts;
  // slices of about 2048 partials each, at most kFoldSlices (the stage buffer's size)
  const int64_t per = (n <= 1) ? nparts : (g.rows / g.rows_per_batch) * g.decay_block;
  int slices = (int)((per + 2047) / 2048);
  slices = slices < 1 ? 1 : (slices > kFoldSlices ? kFoldSlices : slices);
  dim3 grid1(slices, (unsigned)(n > 65535 ? 65535 : n));
  fold_stage1<<<grid1, 256, 0, st>>>(scratch, stage, g, n, nparts);
  SB_CUDA(cudaGetLastError());
  const int wpb = 4;
  fold_stage2<<<(unsigned)((n + wpb - 1) / wpb), wpb * 32, 0, st>>>(stage, out, slices, n);
  SB_CUDA(cudaGetLastError());
  return SB_OK;
}

}  // namespace sb

// ---------------------------------------------------------------------------
// extern "C"
// ---------------------------------------------------------------------------
extern "C" {

int sb_version(void) { return 100; }

const char* sb_last_error_string(void) { return sb::g_err; }

int sb_device_status(unsigned int* bits) {
  SB_REQUIRE(bits != nullptr, "bits is null");
  unsigned int* p = sb::status_ptr();
  if (!p) return SB_ERR_CUDA;
  SB_CUDA(cudaDeviceSynchronize());
  SB_CUDA(cudaMemcpy(bits, p, sizeof(unsigned int), cudaMemcpyDeviceToHost));
  SB_CUDA(cudaMemset(p, 0, sizeof(unsigned int)));
  return SB_OK;
}

int64_t sb_param_grad_scratch_bytes(int64_t rows, int64_t n) {
  if (rows < 0) return 0;
  return sb::scratch_slots(rows, n) * (int64_t)sizeof(double);
}

int sb_uses_tma(const void* base, int64_t T) {
  const void* p[1] = {base};
  return sb::tma_eligible(p, 1, T) ? 1 : 0;
}

}  // extern "C"
