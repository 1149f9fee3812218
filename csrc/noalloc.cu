// The library's one allocation-free entry point (declared and documented in memarch_noalloc.h): an Instinct "hs" step
// whose scratch statistics live in a file-scope __device__ array instead of memory obtained at call time.
#include <cstdio>

#include "instinct_core.cuh"
#include "memarch_noalloc.h"

namespace {

// Row / column sums of the homeostasis normalisation plus the three step scalars.  One copy per GPU, held until exit.
static __device__ __align__(256) float g_noalloc_scratch[MEMARCH_NOALLOC_SCRATCH_FLOATS];

// In host code `g_noalloc_scratch` is only a stand-in symbol; the address a kernel may use comes from
// cudaGetSymbolAddress on the device that will run it.  Looked up once per device.
static float* g_scratch_addr[64] = {nullptr};

__global__ void noalloc_set_scalars(float* dst, float gain, float stake, float lr) {
  dst[0] = gain; dst[1] = stake; dst[2] = lr;
}

}  // namespace

extern "C" int memarch_instinct_hs_step_noalloc(void* weight, const void* grad, void* momentum, float* master,
                                                int weight_bf16, int grad_bf16, int momentum_bf16, long long rows,
                                                long long cols, float gain, float stake, float lr_scaled, float beta,
                                                float weight_decay, cudaStream_t stream) {
  if (!weight || !grad || !momentum || rows <= 0 || cols <= 0 || cols % 4 != 0) {
    std::fprintf(stderr, "memarch_instinct_hs_step_noalloc: bad argument (null pointer, empty shape or cols %% 4 != 0)\n");
    return MEMARCH_NOALLOC_BAD_ARG;
  }
  const long long need = mb::instinct_scratch_floats(1, rows, cols) + 8;   // <= 3*rows + 2*cols + 21
  if (need > (long long)MEMARCH_NOALLOC_SCRATCH_FLOATS) {
    std::fprintf(stderr,
                 "memarch_instinct_hs_step_noalloc: a %lld x %lld weight needs %lld floats of scratch, the built-in "
                 "array holds %d; use the allocating path for this weight\n",
                 rows, cols, need, (int)MEMARCH_NOALLOC_SCRATCH_FLOATS);
    return MEMARCH_NOALLOC_TOO_LARGE;
  }
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return MEMARCH_NOALLOC_CUDA_ERROR;
  if (!g_scratch_addr[dev]) {                      // first call on this device: resolve the array's device address
    float* ptr = nullptr;
    cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_noalloc_scratch);
    if (e != cudaSuccess || ptr == nullptr) {
      std::fprintf(stderr, "memarch_instinct_hs_step_noalloc: cudaGetSymbolAddress failed: %s\n", cudaGetErrorString(e));
      return MEMARCH_NOALLOC_CUDA_ERROR;
    }
    g_scratch_addr[dev] = ptr;
  }
  float* base = g_scratch_addr[dev];
  float* scalars = base;                           // [gain, stake, lr] then padding to keep the statistics 32-byte aligned
  float* stats = base + 8;
  // the statistics are accumulated with atomics and must start at zero; the array still holds the previous call's
  if (cudaMemsetAsync(stats, 0, sizeof(float) * (size_t)(need - 8), stream) != cudaSuccess) return MEMARCH_NOALLOC_CUDA_ERROR;
  noalloc_set_scalars<<<1, 1, 0, stream>>>(scalars, gain, stake, lr_scaled);
  mb::InstinctArgs a{};
  a.p = weight; a.g = grad; a.m = momentum; a.w = master;
  a.p_bf16 = weight_bf16 ? 1 : 0; a.g_bf16 = grad_bf16 ? 1 : 0; a.m_bf16 = momentum_bf16 ? 1 : 0;
  a.gain = scalars; a.stake = scalars + 1; a.lr = scalars + 2;
  a.beta = beta; a.wd = weight_decay;
  a.sr = 0; a.seed = nullptr; a.salt = 0u;
  a.frozen = nullptr; a.frozen_stride = 1;
  a.E = 1; a.R = rows; a.C = cols;
  a.shadow = nullptr;
  if (mb::instinct_launch(a, /*kind hs*/ 4, stats, nullptr, stream) < 0) {
    std::fprintf(stderr, "memarch_instinct_hs_step_noalloc: a row of %lld columns does not fit the kernels' shared memory\n", cols);
    return MEMARCH_NOALLOC_TOO_LARGE;
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    std::fprintf(stderr, "memarch_instinct_hs_step_noalloc: launch failed: %s\n", cudaGetErrorString(e));
    return MEMARCH_NOALLOC_CUDA_ERROR;
  }
  return MEMARCH_NOALLOC_OK;
}
