// LayerNorm backward (+ dgamma) as a plain two-kernel call that allocates nothing: the per-task dgamma partials, which the
// scheduler path keeps in a caller-allocated buffer, live here in a file-scope device array of fixed size.
//
// Who needs this: hosts that must not call cudaMalloc on the serving/training path. Two kinds show up in practice:
// processes whose device memory is already owned by another allocator (a framework's caching pool that claimed the GPU at
// start-up, so a raw cudaMalloc either fails or eats into memory the pool believes it has), and latency-sensitive loops
// that share the GPU with a resident persistent kernel - cudaMalloc/cudaFree synchronise the whole device, which would
// stall everything else running on it. Such a host hands in its own input and output buffers and this entry point needs no
// other memory.
//
// Rules that follow from the design:
//   * The scratch array is ONE per device for the life of the process (about 6 MB, held by every GPU that loads the
//     library). Every call uses it and leaves its last partials in it; nothing has to start at zero because each call
//     overwrites every partial it later reads. Two calls that overlap on the GPU (different streams, or another host thread)
//     race on it: serialise them.
//   * The first call on a device looks up the array's device address (a lookup, not an allocation) with that device
//     current. Make that first call before any stream capture starts.
//   * Sizes beyond the compiled-in maximum are rejected with OFA_BAD_ARGUMENT and a message; nothing is launched.
#include "../../include/ofa_b200.h"
#include "elementwise.cuh"
#include <cuda_runtime.h>
#include <mutex>
#include <string>

using namespace ofa;

namespace {

constexpr int NA_D = 768;                                  // model width of the bf16 path
constexpr int NA_MAX_ROWS = 32768;                         // rows (tokens) per call
constexpr int NA_MAX_TASKS = NA_MAX_ROWS / ew::ROWS_PER_TASK;
static __device__ __align__(256) float g_ln_partials[(size_t)NA_MAX_TASKS * NA_D];   // 2048 x 768 floats = 6,291,456 B

constexpr int MAX_DEVICES = 64;
std::mutex g_mu;
float* g_partials_ptr[MAX_DEVICES] = {nullptr};            // device address of g_ln_partials on each device, filled on first use
thread_local std::string g_na_error;

__global__ void __launch_bounds__(NTHR) na_ln_bwd_kernel(bf16* dx, float* part, const bf16* dy, const bf16* x, const float* mean,
                                                          const float* rstd, const bf16* gamma, const bf16* dres, int N) {
  extern __shared__ __align__(16) unsigned char na_smem[];
  ew::ln_bwd_task<bf16, NA_D>((int)blockIdx.x, dx, part, dy, x, mean, rstd, gamma, dres, N, na_smem);
}
__global__ void __launch_bounds__(NTHR) na_ln_dgamma_kernel(float* dgamma, const float* part, int nblk, int accumulate) {
  ew::ln_dgamma_reduce_task<float>((int)blockIdx.x, dgamma, part, nblk, NA_D, accumulate);
}

int na_fail(int code, const std::string& msg) { g_na_error = msg; return code; }

}  // namespace

extern "C" const char* ofa_noalloc_last_error(void) { return g_na_error.c_str(); }
extern "C" int ofa_noalloc_max_rows(void) { return NA_MAX_ROWS; }

extern "C" int ofa_ln_bwd_noalloc(void* dx, float* dgamma, const void* dy, const void* x, const float* mean, const float* rstd,
                                  const void* gamma, const void* dres, int n_rows, int d_model, int accumulate, void* stream) {
  if (!dx || !dgamma || !dy || !x || !mean || !rstd || !gamma) return na_fail(OFA_BAD_ARGUMENT, "null pointer");
  if (d_model != NA_D) return na_fail(OFA_BAD_ARGUMENT, "ofa_ln_bwd_noalloc is built for d_model 768");
  if (n_rows <= 0) return na_fail(OFA_BAD_ARGUMENT, "n_rows must be positive");
  if (n_rows > NA_MAX_ROWS)
    return na_fail(OFA_BAD_ARGUMENT, "n_rows " + std::to_string(n_rows) + " exceeds the fixed scratch of this entry point (max " + std::to_string(NA_MAX_ROWS) + " rows)");
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return na_fail(OFA_CUDA_ERROR, "no current CUDA device");
  float* part = nullptr;
  {
    std::lock_guard<std::mutex> lk(g_mu);
    if (!g_partials_ptr[dev]) {      // once per device, with that device current: the symbol's name is only a host-side handle
      float* p = nullptr;
      const cudaError_t e = cudaGetSymbolAddress((void**)&p, g_ln_partials);
      if (e != cudaSuccess || !p) return na_fail(OFA_CUDA_ERROR, std::string("cudaGetSymbolAddress failed: ") + cudaGetErrorString(e));
      g_partials_ptr[dev] = p;
    }
    part = g_partials_ptr[dev];
  }
  const int ntasks = (n_rows + ew::ROWS_PER_TASK - 1) / ew::ROWS_PER_TASK;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  na_ln_bwd_kernel<<<ntasks, NTHR, (unsigned)ew::ln_bwd_smem_bytes<NA_D>(), s>>>(
      reinterpret_cast<bf16*>(dx), part, reinterpret_cast<const bf16*>(dy), reinterpret_cast<const bf16*>(x), mean, rstd,
      reinterpret_cast<const bf16*>(gamma), reinterpret_cast<const bf16*>(dres), n_rows);
  na_ln_dgamma_kernel<<<(NA_D + NTHR - 1) / NTHR, NTHR, 0, s>>>(dgamma, part, ntasks, accumulate);
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return na_fail(OFA_CUDA_ERROR, std::string("launch failed: ") + cudaGetErrorString(e));
  return OFA_OK;
}
