// Host-side runtime: status block, tensor-map encoding, launch counter, error text.
#include "runtime.h"
#include "common.cuh"

#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>

namespace b200 {

static std::mutex g_mu;
static char g_err[1024] = {0};
static std::atomic<long long> g_launches{0};
static int* g_status[64] = {nullptr};
static int g_sms[64] = {0};

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn g_encode = nullptr;

int fail(int code, const char* fmt, ...) {
  std::lock_guard<std::mutex> lk(g_mu);
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

void count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

int* status_ptr() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  if (g_status[dev]) return g_status[dev];
  std::lock_guard<std::mutex> lk(g_mu);
  if (g_status[dev]) return g_status[dev];
  int* p = nullptr;
  if (cudaMalloc(&p, 8 * sizeof(int)) != cudaSuccess) return nullptr;
  cudaMemset(p, 0, 8 * sizeof(int));
  g_status[dev] = p;
  return p;
}

int sm_count() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (g_sms[dev]) return g_sms[dev];
  int n = 0;
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
  g_sms[dev] = n;
  return n;
}

static int ensure_encode() {
  // Driver entry points need a context current on the calling thread.  A thread that has made no
  // runtime call yet (an autograd worker whose first op is one of these GEMMs) has none: bind the
  // primary context of its current device once per thread.
  static thread_local bool bound = false;
  if (!bound) {
    cudaFree(nullptr);
    bound = true;
  }
  if (g_encode) return 0;
  std::lock_guard<std::mutex> lk(g_mu);
  if (g_encode) return 0;
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult qres;
  cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
  if (e != cudaSuccess || fn == nullptr || qres != cudaDriverEntryPointSuccess) {
    snprintf(g_err, sizeof(g_err), "cuTensorMapEncodeTiled entry point unavailable (%s)", cudaGetErrorString(e));
    return 100;
  }
  g_encode = (EncodeTiledFn)fn;
  return 0;
}

static CUtensorMapDataType to_cu(DType dt) {
  switch (dt) {
    case DT_BF16: return CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    case DT_F32: return CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
    case DT_U8: return CU_TENSOR_MAP_DATA_TYPE_UINT8;
    case DT_F16: return CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    case DT_I32: return CU_TENSOR_MAP_DATA_TYPE_INT32;
  }
  return CU_TENSOR_MAP_DATA_TYPE_UINT8;
}
static CUtensorMapSwizzle to_cu(Swizzle s) {
  switch (s) {
    case SWZ_NONE: return CU_TENSOR_MAP_SWIZZLE_NONE;
    case SWZ_32: return CU_TENSOR_MAP_SWIZZLE_32B;
    case SWZ_64: return CU_TENSOR_MAP_SWIZZLE_64B;
    case SWZ_128: return CU_TENSOR_MAP_SWIZZLE_128B;
  }
  return CU_TENSOR_MAP_SWIZZLE_NONE;
}

int make_tmap_2d(CUtensorMap* out, DType dt, const void* base, uint64_t cols, uint64_t rows,
                 uint64_t row_pitch_bytes, uint32_t box_cols, uint32_t box_rows, Swizzle swz) {
  if (int r = ensure_encode()) return r;
  if (((uintptr_t)base & 15) != 0) return fail(101, "tensor map base %p is not 16-byte aligned", base);
  if ((row_pitch_bytes & 15) != 0) return fail(102, "tensor map row pitch %llu is not a multiple of 16 bytes",
                                               (unsigned long long)row_pitch_bytes);
  if (box_cols > 256 || box_rows > 256 || box_cols == 0 || box_rows == 0)
    return fail(103, "tensor map box %u x %u out of range", box_cols, box_rows);
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {row_pitch_bytes};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = g_encode(out, to_cu(dt), 2, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, to_cu(swz), CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(104, "cuTensorMapEncodeTiled(2d) failed: %d (cols=%llu rows=%llu pitch=%llu box=%ux%u)", (int)r,
                (unsigned long long)cols, (unsigned long long)rows, (unsigned long long)row_pitch_bytes, box_cols,
                box_rows);
  return 0;
}

int make_tmap_3d(CUtensorMap* out, DType dt, const void* base, uint64_t d0, uint64_t d1, uint64_t d2,
                 uint64_t pitch1_bytes, uint64_t pitch2_bytes, uint32_t box0, uint32_t box1, uint32_t box2,
                 Swizzle swz) {
  if (int r = ensure_encode()) return r;
  if (((uintptr_t)base & 15) != 0) return fail(101, "tensor map base %p is not 16-byte aligned", base);
  if ((pitch1_bytes & 15) != 0 || (pitch2_bytes & 15) != 0)
    return fail(102, "tensor map pitches %llu/%llu are not multiples of 16 bytes", (unsigned long long)pitch1_bytes,
                (unsigned long long)pitch2_bytes);
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {pitch1_bytes, pitch2_bytes};
  cuuint32_t box[3] = {box0, box1, box2};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = g_encode(out, to_cu(dt), 3, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, to_cu(swz), CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(104, "cuTensorMapEncodeTiled(3d) failed: %d (d=%llu,%llu,%llu box=%u,%u,%u)", (int)r,
                (unsigned long long)d0, (unsigned long long)d1, (unsigned long long)d2, box0, box1, box2);
  return 0;
}

int make_tmap_4d(CUtensorMap* out, DType dt, const void* base, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t d3,
                 uint64_t pitch1_bytes, uint64_t pitch2_bytes, uint64_t pitch3_bytes, uint32_t box0, uint32_t box1,
                 uint32_t box2, uint32_t box3, Swizzle swz) {
  if (int r = ensure_encode()) return r;
  if (((uintptr_t)base & 15) != 0) return fail(101, "tensor map base %p is not 16-byte aligned", base);
  if ((pitch1_bytes & 15) != 0 || (pitch2_bytes & 15) != 0 || (pitch3_bytes & 15) != 0)
    return fail(102, "tensor map pitches %llu/%llu/%llu are not multiples of 16 bytes",
                (unsigned long long)pitch1_bytes, (unsigned long long)pitch2_bytes, (unsigned long long)pitch3_bytes);
  cuuint64_t dims[4] = {d0, d1, d2, d3};
  cuuint64_t strides[3] = {pitch1_bytes, pitch2_bytes, pitch3_bytes};
  cuuint32_t box[4] = {box0, box1, box2, box3};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = g_encode(out, to_cu(dt), 4, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, to_cu(swz), CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(104, "cuTensorMapEncodeTiled(4d) failed: %d (d=%llu,%llu,%llu,%llu pitch=%llu,%llu,%llu box=%u,%u,%u,%u)",
                (int)r, (unsigned long long)d0, (unsigned long long)d1, (unsigned long long)d2, (unsigned long long)d3,
                (unsigned long long)pitch1_bytes, (unsigned long long)pitch2_bytes, (unsigned long long)pitch3_bytes,
                box0, box1, box2, box3);
  return 0;
}

int check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(200, "%s: launch failed: %s", what, cudaGetErrorString(e));
  return 0;
}

}  // namespace b200

// ----------------------------------------------------------------------------------
// exported C API
// ----------------------------------------------------------------------------------
B200_API const char* b200_last_error() { return b200::g_err; }

B200_API long long b200_launch_count() { return b200::g_launches.load(); }
B200_API void b200_launch_count_reset() { b200::g_launches.store(0); }

// Copies the 8 status ints of the current device to `out8` (synchronises the device).
B200_API int b200_status_read(int* out8) {
  int* p = b200::status_ptr();
  if (!p) return b200::fail(110, "status block unavailable");
  cudaError_t e = cudaMemcpy(out8, p, 8 * sizeof(int), cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) return b200::fail(111, "status read failed: %s", cudaGetErrorString(e));
  return 0;
}
B200_API int b200_status_reset() {
  int* p = b200::status_ptr();
  if (!p) return b200::fail(110, "status block unavailable");
  cudaError_t e = cudaMemset(p, 0, 8 * sizeof(int));
  if (e != cudaSuccess) return b200::fail(111, "status reset failed: %s", cudaGetErrorString(e));
  return 0;
}
B200_API int b200_sm_count() { return b200::sm_count(); }

// ----------------------------------------------------------------------------------
// Wait probe: one thread waits (bounded) for `*flag >= want`.  Used by the failure-detection tests
// to see a wait run out and report through the status block while the context stays usable, and
// by hosts that want to block a stream on a device flag with a deadline.
// ----------------------------------------------------------------------------------
namespace {
__global__ void flag_wait_probe_kernel(const int* flag, int want, unsigned long long limit_ns, int* status, int* result) {
  const bool ok = flag_wait_geq(flag, want, limit_ns, status, 99);
  if (result != nullptr) *result = ok ? 1 : 0;
}
}  // namespace

B200_API int b200_flag_wait_probe(const int* flag, int want, long long limit_ns, int* result, void* stream) {
  if (limit_ns <= 0 || limit_ns > (long long)B200_WAIT_LIMIT_NS)
    return b200::fail(120, "flag_wait_probe: limit %lld ns outside (0, %llu]", limit_ns, (unsigned long long)B200_WAIT_LIMIT_NS);
  flag_wait_probe_kernel<<<1, 1, 0, (cudaStream_t)stream>>>(flag, want, (unsigned long long)limit_ns, b200::status_ptr(), result);
  b200::count_launch();
  return b200::check_launch("flag_wait_probe");
}
