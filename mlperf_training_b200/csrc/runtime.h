// Host-side runtime shared by every launcher in this library: per-device status block,
// TMA tensor-map encoding (driver entry point fetched through the runtime, so the library
// does not link libcuda), launch counter and last-error text.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define B200_API extern "C" __attribute__((visibility("default")))

namespace b200 {

enum DType : int { DT_BF16 = 0, DT_F32 = 1, DT_U8 = 2, DT_F16 = 3, DT_I32 = 4 };
enum Swizzle : int { SWZ_NONE = 0, SWZ_32 = 1, SWZ_64 = 2, SWZ_128 = 3 };

// Returns the 8-int status block of the current device (allocated on first use, zeroed).
int* status_ptr();
// Number of SMs of the current device (cached).
int sm_count();
// Record an error message (returned by b200_last_error) and return `code`.
int fail(int code, const char* fmt, ...);
// Count one kernel launch of this library (read by b200_launch_count()).
void count_launch(int n = 1);

// 2-D row-major tensor [rows][cols] of `dt`; box = [box_rows][box_cols]; row pitch in bytes.
// Returns 0 on success.  `cols` is the contiguous dimension.
int make_tmap_2d(CUtensorMap* out, DType dt, const void* base, uint64_t cols, uint64_t rows,
                 uint64_t row_pitch_bytes, uint32_t box_cols, uint32_t box_rows, Swizzle swz);
// 3-D tensor [d2][d1][d0] with pitches (bytes) for d1 and d2.
int make_tmap_3d(CUtensorMap* out, DType dt, const void* base, uint64_t d0, uint64_t d1, uint64_t d2,
                 uint64_t pitch1_bytes, uint64_t pitch2_bytes, uint32_t box0, uint32_t box1, uint32_t box2,
                 Swizzle swz);

// 4-D tensor [d3][d2][d1][d0] with pitches (bytes) for d1, d2, d3.
int make_tmap_4d(CUtensorMap* out, DType dt, const void* base, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t d3,
                 uint64_t pitch1_bytes, uint64_t pitch2_bytes, uint64_t pitch3_bytes, uint32_t box0, uint32_t box1,
                 uint32_t box2, uint32_t box3, Swizzle swz);

// Check the launch of the kernel just issued; returns 0 or a failure code with message.
int check_launch(const char* what);

}  // namespace b200
