// b200_sumsq_static: two-pass fp32 sum of squares whose partial sums live in a static device
// array, so the call path contains no allocation of any kind (see sumsq_static.h for the contract).
#include "sumsq_static.h"

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <mutex>

#include "common.cuh"
#include "runtime.h"

namespace {

// one partial sum per CTA of the first pass; shared by every call on the device
static __device__ __align__(256) float g_sumsq_scratch[B200_SUMSQ_STATIC_SLOTS];

constexpr int kMaxDevices = 64;
float* g_scratch_ptr[kMaxDevices] = {};
std::mutex g_setup_mu;

template <typename G>
__global__ void __launch_bounds__(256)
sumsq_static_partial_kernel(const G* __restrict__ g, long long n, float* __restrict__ partial) {
  __shared__ float red[8];
  float acc = 0.f;
  for (long long i = blockIdx.x * 256ll + threadIdx.x; i < n; i += (long long)gridDim.x * 256) {
    float v;
    if constexpr (sizeof(G) == 2) v = __bfloat162float(g[i]); else v = g[i];
    acc += v * v;
  }
  acc = warp_sum(acc);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x < 32) {
    float r = threadIdx.x < 8 ? red[threadIdx.x] : 0.f;
    r = warp_sum(r);
    if (threadIdx.x == 0) partial[blockIdx.x] = r;
  }
}

__global__ void sumsq_static_final_kernel(const float* __restrict__ partial, int n, float* __restrict__ out,
                                          int accumulate) {
  __shared__ float red[8];
  float acc = 0.f;
  for (int i = threadIdx.x; i < n; i += 256) acc += partial[i];
  acc = warp_sum(acc);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x < 32) {
    float r = threadIdx.x < 8 ? red[threadIdx.x] : 0.f;
    r = warp_sum(r);
    if (threadIdx.x == 0) out[0] = accumulate ? out[0] + r : r;
  }
}

// Address of the scratch array on the current device; looked up once per device.
int scratch_for_current_device(float** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return b200::fail(1400, "sumsq_static: cudaGetDevice failed: %s", cudaGetErrorString(e));
  if (dev < 0 || dev >= kMaxDevices) return b200::fail(1401, "sumsq_static: device index %d out of range", dev);
  std::lock_guard<std::mutex> lk(g_setup_mu);
  if (g_scratch_ptr[dev] == nullptr) {
    float* p = nullptr;
    e = cudaGetSymbolAddress((void**)&p, g_sumsq_scratch);
    if (e != cudaSuccess || p == nullptr) {
      cudaGetLastError();
      return b200::fail(1402, "sumsq_static: cudaGetSymbolAddress failed on device %d: %s", dev, cudaGetErrorString(e));
    }
    g_scratch_ptr[dev] = p;
  }
  *out = g_scratch_ptr[dev];
  return 0;
}

}  // namespace

extern "C" long long b200_sumsq_static_max_elems(void) { return B200_SUMSQ_STATIC_MAX_ELEMS; }

extern "C" int b200_sumsq_static(const void* g, long long n, int g_is_bf16, float* out, int accumulate, void* stream) {
  if (n < 0 || n > B200_SUMSQ_STATIC_MAX_ELEMS)
    return b200::fail(1403, "sumsq_static: n=%lld is outside [0, %lld]; use b200_sumsq with caller-provided scratch",
                      n, (long long)B200_SUMSQ_STATIC_MAX_ELEMS);
  if (g == nullptr || out == nullptr) return b200::fail(1404, "sumsq_static: null pointer argument");
  float* scratch = nullptr;
  if (int rc = scratch_for_current_device(&scratch)) return rc;
  int grid = b200::sm_count() * 4;
  if (grid > B200_SUMSQ_STATIC_SLOTS) grid = B200_SUMSQ_STATIC_SLOTS;
  if ((long long)grid * 256 > n) grid = (int)((n + 255) / 256);
  if (grid < 1) grid = 1;
  cudaStream_t st = (cudaStream_t)stream;
  if (g_is_bf16) sumsq_static_partial_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)g, n, scratch);
  else sumsq_static_partial_kernel<float><<<grid, 256, 0, st>>>((const float*)g, n, scratch);
  sumsq_static_final_kernel<<<1, 256, 0, st>>>(scratch, grid, out, accumulate);
  b200::count_launch(2);
  return b200::check_launch("sumsq_static");
}
