// Host side of the bit-packed spike result (sb_cuba_fwd_packed): expands the 32-step words
// into the fp32 0 / 1 tensor that the neuron's forward() returns, on the CPU.  A result that
// is wanted on the host as fp32 then crosses PCIe as bits (1/32 of the bytes) and is expanded
// where it lands.  No counterpart in the reference, which returns fp32 spikes on the device.
//
// Synchronous (stream_ordered = 0), or enqueued on a stream as a host function
// (stream_ordered = 1): the expansion then runs after the work already queued there (the copy
// of the bits to the host) and before anything queued later, e.g. an event that times the pass.
#include "api_util.cuh"

#include <thread>
#include <vector>

using namespace sb;

namespace {

struct UnpackJob {
  const uint32_t* bits;
  float* out;
  int64_t rows, T;
  int threads;
};

void unpack_rows(const uint32_t* bits, float* out, int64_t r0, int64_t r1, int64_t T) {
  const int64_t words = (T + 31) / 32;
  for (int64_t r = r0; r < r1; ++r) {
    const uint32_t* b = bits + r * words;
    float* o = out + r * T;
    int64_t w = 0;
    for (; w + 1 <= T / 32; ++w) {   // whole words: a loop the compiler vectorises
      const uint32_t m = b[w];
      float* d = o + 32 * w;
      for (int i = 0; i < 32; ++i) d[i] = (float)((m >> i) & 1u);
    }
    if (32 * w < T) {
      const uint32_t m = b[w];
      for (int64_t i = 0; 32 * w + i < T; ++i) o[32 * w + i] = (float)((m >> i) & 1u);
    }
  }
}

void run_job(const UnpackJob& j) {
  int n = j.threads > 0 ? j.threads : (int)std::thread::hardware_concurrency();
  if (n < 1) n = 1;
  if (n > 64) n = 64;
  if ((int64_t)n > j.rows) n = (int)(j.rows < 1 ? 1 : j.rows);
  if (n == 1) {
    unpack_rows(j.bits, j.out, 0, j.rows, j.T);
    return;
  }
  std::vector<std::thread> pool;
  pool.reserve(n);
  const int64_t per = (j.rows + n - 1) / n;
  for (int t = 0; t < n; ++t) {
    const int64_t r0 = t * per, r1 = (r0 + per < j.rows) ? r0 + per : j.rows;
    if (r0 >= r1) break;
    pool.emplace_back(unpack_rows, j.bits, j.out, r0, r1, j.T);
  }
  for (auto& th : pool) th.join();
}

void CUDART_CB unpack_callback(void* p) {
  UnpackJob* j = static_cast<UnpackJob*>(p);
  run_job(*j);
  delete j;
}

}  // namespace

extern "C" int sb_unpack_spikes_host(const uint32_t* bits, float* out, int64_t rows, int64_t T, int threads,
                                     int stream_ordered, void* stream) {
  SB_REQUIRE(rows >= 0 && T >= 0, "bad geometry");
  if (rows == 0 || T == 0) return SB_OK;
  SB_REQUIRE(bits != nullptr && out != nullptr, "null host pointer");
  if (!stream_ordered) {
    run_job(UnpackJob{bits, out, rows, T, threads});
    return SB_OK;
  }
  UnpackJob* j = new UnpackJob{bits, out, rows, T, threads};
  cudaError_t e = cudaLaunchHostFunc((cudaStream_t)stream, unpack_callback, j);
  if (e != cudaSuccess) {
    delete j;
    SB_CUDA(e);
  }
  return SB_OK;
}
