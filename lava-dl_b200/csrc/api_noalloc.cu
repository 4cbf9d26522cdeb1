// sb_li_bwd_noalloc: the leaky-integrator backward with decay gradient for hosts
// that have no way to hand the library a scratch buffer.
//
// Who needs this.  Every other entry point that produces a parameter gradient
// asks the caller for scratch memory, which in practice means the caller runs
// an allocator (cudaMalloc, or torch's caching allocator) right before the
// call.  Some hosts cannot: an operator plugged into a runtime that plans all
// device memory ahead of time and passes a custom op nothing but its input and
// output buffers; a serving process whose memory pool already owns the whole
// GPU, where a raw cudaMalloc fails or stalls the device; a control loop with a
// latency budget that cannot absorb the implicit device synchronisation of an
// allocation.  For them the scratch lives inside the library image instead.
//
// What it costs.  The scratch is one file-scope device array of
// SB_NOALLOC_SCRATCH_BYTES (4 MiB).  Every GPU on which this library is loaded
// holds that array from module load until the process exits, used or not.
//
// Rules for callers.
//  * Problems whose partials do not fit are rejected with SB_ERR_INVALID_ARG
//    (the message names both sizes); use sb_li_bwd with your own scratch then.
//    Shared decay: up to 32 * (capacity/8 - 64) rows (about 16.7 M).
//    Per-channel decay: rows + 64 * n_decay <= capacity/8 = 524288.
//  * The first call on each device resolves the device address of the array
//    (cudaGetSymbolAddress, with that device current) and opts the kernel into
//    its shared-memory size.  Make that first call outside any stream capture.
//  * All calls on one device share the one array, and it keeps whatever the
//    previous call left in it.  Nothing in it has to start at zero: every slot
//    that is read has been written earlier in the same call (each warp or row
//    writes its partial before the fold reads it -- also a warp that gave up
//    waiting for a tile and set SB_DEV_TMA_TIMEOUT, whose partial then covers
//    only the steps it walked -- and the fold writes its stage slots before
//    summing them), so no clearing pass is issued.  After any call check
//    sb_device_status: with SB_DEV_TMA_TIMEOUT set, grad_x and grad_decay of
//    that call are incomplete.
//  * Two calls that overlap on the GPU (different streams, or different host
//    threads on different streams) race on the array and produce garbage in
//    grad_decay.  Serialise them on one stream or with events.
//  * Nothing here calls cudaMalloc, cudaFree or any allocating library routine.
#include <atomic>

#include "api_util.cuh"
#include "reduce.cuh"
#include "rowscan.cuh"

using namespace sb;

static __device__ __align__(256) unsigned char g_noalloc_scratch[SB_NOALLOC_SCRATCH_BYTES];

namespace {

constexpr int kMaxDevices = 64;
// One slot per device ordinal.  Threads may race to fill a slot; they all store the same address
// (release / acquire), so the race only repeats the lookup.
std::atomic<double*> g_scratch_dev_ptr[kMaxDevices];

// In host code `g_noalloc_scratch` is only a handle for the symbol, not an
// address a kernel could use; the address on the current device comes from the
// runtime, once per device.
int noalloc_scratch(double** out) {
  int dev = -1;
  SB_CUDA(cudaGetDevice(&dev));
  SB_REQUIRE(dev >= 0 && dev < kMaxDevices, "device ordinal %d outside [0, %d)", dev, kMaxDevices);
  double* cached = g_scratch_dev_ptr[dev].load(std::memory_order_acquire);
  if (cached == nullptr) {
    void* p = nullptr;
    SB_CUDA(cudaGetSymbolAddress(&p, g_noalloc_scratch));
    SB_REQUIRE(p != nullptr && (((uintptr_t)p) & 255u) == 0, "built-in scratch has an unusable address %p", p);
    cached = (double*)p;
    g_scratch_dev_ptr[dev].store(cached, std::memory_order_release);
  }
  *out = cached;
  return SB_OK;
}

}  // namespace

extern "C" int sb_li_bwd_noalloc(const float* grad_y, const float* y, const float* decay, int64_t n_decay,
                                 float* grad_x, float* grad_decay, const sb_geom* g, void* stream) {
  RowGeom rg;
  SB_TRY(check_count(n_decay, "decay"));
  SB_TRY(check_geom(g, &rg, n_decay));
  SB_REQUIRE(decay && grad_decay, "decay and grad_decay are required (without a decay gradient sb_li_bwd needs no scratch)");
  const int64_t need = scratch_slots(rg.rows, n_decay) * (int64_t)sizeof(double);
  SB_REQUIRE(need <= (int64_t)SB_NOALLOC_SCRATCH_BYTES,
             "this problem needs %lld bytes of scratch but the built-in area holds %lld; call sb_li_bwd with caller scratch",
             (long long)need, (long long)SB_NOALLOC_SCRATCH_BYTES);
  cudaStream_t st = (cudaStream_t)stream;
  if (rg.rows == 0 || rg.T == 0) {
    SB_CUDA(cudaMemsetAsync(grad_decay, 0, sizeof(float) * n_decay, st));
    return SB_OK;
  }
  SB_REQUIRE(grad_y && y && grad_x, "null tensor pointer");
  double* scratch = nullptr;
  SB_TRY(noalloc_scratch(&scratch));
  const float* in[2] = {grad_y, y};
  float* out[1] = {grad_x};
  LiBwd<true>::Params p{{decay, n_decay}, scratch};
  SB_TRY((launch_rowscan<LiBwd<true>>(p, rg, in, out, st)));
  return fold_param_grad(scratch, grad_decay, rg, n_decay, st);
}
