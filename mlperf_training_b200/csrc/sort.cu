// Sort / unique / segment machinery of the sparse (embedding) path, all on the device and all
// deterministic:
//
//   sort_ids           stable LSD radix sort of 64-bit ids restricted to the bits the table size needs
//                      (bounded keys: a 400 M-row table sorts 29 bits, not 64), carrying each id's original
//                      position as the value;
//   unique_segments    from the sorted ids: the unique ids, the start of every run of equal ids
//                      (segment offsets), the number of runs, and for every original position the index of
//                      its run (the "inverse" of a dedup);
//   segment_sum_gather rows of a gradient matrix that belong to one run are summed in sorted order -
//                      fixed order, no atomics - straight from their original places (gather by the sort
//                      permutation), into fp32 or bf16.
//
// The digit passes of the sort and the prefix sums are CUB device primitives (cub::DeviceRadixSort,
// cub::DeviceScan) run on caller-provided scratch; the head flags, run bookkeeping, inverse map and the
// reduction are this library's kernels.  Replaces the reference's bounded-key onesweep sort and segment
// reduction (generative_recommenders/ops/onesweep_sort_kernels.hip:39-110,
// generative_recommenders/dlrm_v4/train/ec_segment_reduce.py:1-317).
#include <cub/cub.cuh>

#include "common.cuh"
#include "runtime.h"

namespace {

__global__ void iota_kernel(long long* __restrict__ p, long long n) {
  for (long long i = blockIdx.x * 256ll + threadIdx.x; i < n; i += (long long)gridDim.x * 256) p[i] = i;
}

__global__ void head_flags_kernel(const long long* __restrict__ keys, long long n, int* __restrict__ flags) {
  for (long long i = blockIdx.x * 256ll + threadIdx.x; i < n; i += (long long)gridDim.x * 256)
    flags[i] = (i == 0 || keys[i] != keys[i - 1]) ? 1 : 0;
}

// run[i] = inclusive sum of the head flags = 1-based index of the run of sorted position i
__global__ void runs_kernel(const long long* __restrict__ keys, const long long* __restrict__ perm,
                            const int* __restrict__ run, long long n, long long* __restrict__ uniq,
                            long long* __restrict__ seg_off, long long* __restrict__ inverse, long long* __restrict__ count) {
  for (long long i = blockIdx.x * 256ll + threadIdx.x; i < n; i += (long long)gridDim.x * 256) {
    const int r = run[i] - 1;
    if (i == 0 || run[i] != run[i - 1]) { uniq[r] = keys[i]; seg_off[r] = i; }
    if (inverse != nullptr) inverse[perm[i]] = r;
    if (i == n - 1) { seg_off[r + 1] = n; *count = r + 1; }
  }
}

// ---- segment reduction ----
// out[s, :] = sum over sorted positions r in [seg[s], seg[s + 1]) of src[perm[r], :], in a fixed order.
// Ids of a recommender batch are heavily skewed (a few ids own thousands of positions), so a run longer than
// SEG_CHUNK positions is not summed by one warp: first one warp per block of SEG_CHUNK sorted positions sums
// the part of each long run that falls into its block (at most two long runs touch a block: the one that
// holds its first position and the one that holds its last), then the run's warp adds those partial sums in
// block order.  Short runs are summed directly.  A lane owns 8-element vectors (16-byte loads of bf16 rows).
constexpr int SEG_CHUNK = 64;

struct RowSrc {
  const __nv_bfloat16* bf16;
  const float* f32;
  const long long* perm;
  long long rows;
  int D;
};

B200_DEVICE void add_row(float (&acc)[8], const RowSrc& s, long long row, int v) {
  if (s.bf16 != nullptr) {
    const uint4 u = *reinterpret_cast<const uint4*>(s.bf16 + row * s.D + v * 8);
    const float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
    acc[0] += a.x; acc[1] += a.y; acc[2] += b.x; acc[3] += b.y; acc[4] += c.x; acc[5] += c.y; acc[6] += d.x; acc[7] += d.y;
  } else {
    const float4 a = *reinterpret_cast<const float4*>(s.f32 + row * s.D + v * 8);
    const float4 b = *reinterpret_cast<const float4*>(s.f32 + row * s.D + v * 8 + 4);
    acc[0] += a.x; acc[1] += a.y; acc[2] += a.z; acc[3] += a.w; acc[4] += b.x; acc[5] += b.y; acc[6] += b.z; acc[7] += b.w;
  }
}

// acc += rows of sorted positions [lo, hi) for vector v, in position order; four row indices are fetched at a time
// so that four row loads are in flight.
B200_DEVICE void sum_positions(float (&acc)[8], const RowSrc& s, long long lo, long long hi, int v, int* status) {
  long long r = lo;
  for (; r + 4 <= hi; r += 4) {
    long long row[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) row[j] = s.perm != nullptr ? s.perm[r + j] : r + j;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (row[j] < 0 || row[j] >= s.rows) {               // a permutation entry outside the source matrix
        if (v == 0) B200_BOUNDS_REPORT(status, 1601);
        continue;
      }
      add_row(acc, s, row[j], v);
    }
  }
  for (; r < hi; ++r) {
    const long long row = s.perm != nullptr ? s.perm[r] : r;
    if (row < 0 || row >= s.rows) {
      if (v == 0) B200_BOUNDS_REPORT(status, 1601);
      continue;
    }
    add_row(acc, s, row, v);
  }
}

// run that holds sorted position r (last s with seg[s] <= r)
B200_DEVICE long long run_of(const long long* __restrict__ seg, long long total, long long r) {
  long long lo = 0, hi = total - 1;
  while (lo < hi) {
    const long long mid = (lo + hi + 1) >> 1;
    if (seg[mid] <= r) lo = mid; else hi = mid - 1;
  }
  return lo;
}

// partial[b][0] = sum of the long run that holds position b * SEG_CHUNK over its positions inside block b;
// partial[b][1] = the same for the long run that holds the block's last position, when that is another run.
__global__ void __launch_bounds__(256)
segment_partial_kernel(RowSrc s, const long long* __restrict__ seg, const long long* __restrict__ n_seg, long long n,
                       float* __restrict__ partial, int* status) {
  const long long total = *n_seg;
  if (total <= 0) return;
  const int lane = threadIdx.x & 31;
  const long long b = (blockIdx.x * 256ll + threadIdx.x) >> 5;
  const long long p0 = b * SEG_CHUNK;
  if (p0 >= n) return;
  const long long p1 = p0 + SEG_CHUNK < n ? p0 + SEG_CHUNK : n;
  const long long s0 = run_of(seg, total, p0), s1 = run_of(seg, total, p1 - 1);
  const int nvec = s.D / 8;
  for (int slot = 0; slot < 2; ++slot) {
    const long long run = slot == 0 ? s0 : s1;
    if (slot == 1 && s1 == s0) break;
    const long long rlo = seg[run], rhi = seg[run + 1];
    if (rhi - rlo <= SEG_CHUNK) continue;               // short runs are summed by their own warp
    const long long lo = rlo > p0 ? rlo : p0, hi = rhi < p1 ? rhi : p1;
    for (int v = lane; v < nvec; v += 32) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      sum_positions(acc, s, lo, hi, v, status);
      float* dst = partial + ((b * 2 + slot) * s.D + v * 8);
      *reinterpret_cast<float4*>(dst) = make_float4(acc[0], acc[1], acc[2], acc[3]);
      *reinterpret_cast<float4*>(dst + 4) = make_float4(acc[4], acc[5], acc[6], acc[7]);
    }
  }
}

// one warp per run, runs taken grid-stride
template <typename Out>
__global__ void __launch_bounds__(256)
segment_sum_gather_kernel(RowSrc s, const long long* __restrict__ seg, const long long* __restrict__ n_seg,
                          const float* __restrict__ partial, Out* __restrict__ out, int* status) {
  const long long total = *n_seg;
  const int lane = threadIdx.x & 31;
  const long long warp0 = (blockIdx.x * 256ll + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * 256) >> 5;
  const int nvec = s.D / 8;
  for (long long r = warp0; r < total; r += nwarps) {
    const long long lo = seg[r], hi = seg[r + 1];
    for (int v = lane; v < nvec; v += 32) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      if (hi - lo <= SEG_CHUNK || partial == nullptr) {
        sum_positions(acc, s, lo, hi, v, status);
      } else {
        for (long long b = lo / SEG_CHUNK; b * SEG_CHUNK < hi; ++b) {
          const int slot = b * SEG_CHUNK >= lo ? 0 : 1;   // the run holds the block's first position, or starts inside it
          const float* src = partial + ((b * 2 + slot) * s.D + v * 8);
          const float4 a = *reinterpret_cast<const float4*>(src), c = *reinterpret_cast<const float4*>(src + 4);
          acc[0] += a.x; acc[1] += a.y; acc[2] += a.z; acc[3] += a.w; acc[4] += c.x; acc[5] += c.y; acc[6] += c.z; acc[7] += c.w;
        }
      }
      if constexpr (sizeof(Out) == 2) {
        *reinterpret_cast<uint4*>(out + r * s.D + v * 8) =
            make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]), pack_bf16x2(acc[4], acc[5]), pack_bf16x2(acc[6], acc[7]));
      } else {
        *reinterpret_cast<float4*>(out + r * s.D + v * 8) = make_float4(acc[0], acc[1], acc[2], acc[3]);
        *reinterpret_cast<float4*>(out + r * s.D + v * 8 + 4) = make_float4(acc[4], acc[5], acc[6], acc[7]);
      }
    }
  }
}

}  // namespace

// Scratch bytes that b200_sort_ids / b200_unique_segments need for n elements (one buffer serves both).
B200_API long long b200_sort_scratch_bytes(long long n) {
  size_t a = 0, b = 0;
  cub::DeviceRadixSort::SortPairs(nullptr, a, (const long long*)nullptr, (long long*)nullptr, (const long long*)nullptr,
                                  (long long*)nullptr, (int)n, 0, 64);
  cub::DeviceScan::InclusiveSum(nullptr, b, (const int*)nullptr, (int*)nullptr, (int)n);
  const size_t lib = a > b ? a : b;
  // + positions (n x 8) + flags (n x 4) + runs (n x 4), each 256-byte aligned
  return (long long)(((lib + 255) & ~size_t(255)) + (((size_t)n * 8 + 255) & ~size_t(255)) + 2 * (((size_t)n * 4 + 255) & ~size_t(255)));
}

// keys_out = keys_in sorted ascending on bits [0, end_bit); perm_out[i] = original position of keys_out[i].
B200_API int b200_sort_ids(const long long* keys_in, long long* keys_out, long long* perm_out, long long n, int end_bit,
                           void* scratch, long long scratch_bytes, void* stream) {
  if (n <= 0) return 0;
  if (n > 0x7fffffffll) return b200::fail(1600, "sort_ids: n=%lld exceeds 2^31 - 1", n);
  if (end_bit < 1 || end_bit > 64) return b200::fail(1601, "sort_ids: end_bit %d outside [1, 64]", end_bit);
  if (scratch_bytes < b200_sort_scratch_bytes(n)) return b200::fail(1602, "sort_ids: scratch of %lld bytes is too small", scratch_bytes);
  cudaStream_t st = (cudaStream_t)stream;
  size_t lib = 0;
  cub::DeviceRadixSort::SortPairs(nullptr, lib, keys_in, keys_out, (const long long*)nullptr, perm_out, (int)n, 0, end_bit);
  uint8_t* base = (uint8_t*)scratch;
  long long* iota = (long long*)(base + ((lib + 255) & ~size_t(255)));
  const int grid = (int)((n + 255) / 256 < 4096 ? (n + 255) / 256 : 4096);
  iota_kernel<<<grid, 256, 0, st>>>(iota, n);
  cudaError_t e = cub::DeviceRadixSort::SortPairs(scratch, lib, keys_in, keys_out, iota, perm_out, (int)n, 0, end_bit, st);
  b200::count_launch(2);
  if (e != cudaSuccess) return b200::fail(1603, "sort_ids: radix sort failed: %s", cudaGetErrorString(e));
  return b200::check_launch("sort_ids");
}

// sorted_keys [n] (ascending), perm [n] (from b200_sort_ids; may be null when inverse is null).
// uniq [n], seg_off [n + 1], inverse [n] (may be null), count [1]: device outputs sized for the worst case.
B200_API int b200_unique_segments(const long long* sorted_keys, const long long* perm, long long n, long long* uniq,
                                  long long* seg_off, long long* inverse, long long* count, void* scratch,
                                  long long scratch_bytes, void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  if (n <= 0) {
    cudaMemsetAsync(count, 0, sizeof(long long), st);
    return 0;
  }
  if (scratch_bytes < b200_sort_scratch_bytes(n)) return b200::fail(1602, "unique_segments: scratch of %lld bytes is too small", scratch_bytes);
  size_t a = 0, lib = 0;
  cub::DeviceRadixSort::SortPairs(nullptr, a, (const long long*)nullptr, (long long*)nullptr, (const long long*)nullptr,
                                  (long long*)nullptr, (int)n, 0, 64);
  cub::DeviceScan::InclusiveSum(nullptr, lib, (const int*)nullptr, (int*)nullptr, (int)n);
  if (a > lib) lib = a;
  uint8_t* base = (uint8_t*)scratch;
  uint8_t* p = base + ((lib + 255) & ~size_t(255)) + (((size_t)n * 8 + 255) & ~size_t(255));
  int* flags = (int*)p;
  int* run = (int*)(p + (((size_t)n * 4 + 255) & ~size_t(255)));
  const int grid = (int)((n + 255) / 256 < 4096 ? (n + 255) / 256 : 4096);
  head_flags_kernel<<<grid, 256, 0, st>>>(sorted_keys, n, flags);
  size_t scan_bytes = lib;
  cudaError_t e = cub::DeviceScan::InclusiveSum(scratch, scan_bytes, flags, run, (int)n, st);
  if (e != cudaSuccess) return b200::fail(1604, "unique_segments: scan failed: %s", cudaGetErrorString(e));
  runs_kernel<<<grid, 256, 0, st>>>(sorted_keys, perm, run, n, uniq, seg_off, inverse, count);
  b200::count_launch(3);
  return b200::check_launch("unique_segments");
}

// Floats of the scratch b200_segment_sum_gather needs for n sorted positions of D-wide rows.
B200_API long long b200_segment_sum_scratch_elems(long long n, int D) {
  return ((n + SEG_CHUNK - 1) / SEG_CHUNK) * 2 * (long long)D;
}

// out[s, :] = sum of src[perm[r], :] over the sorted positions r of run s, s < *n_seg (device scalar), summed in a
// fixed order.  src: bf16 or fp32 [src_rows, D]; perm [n] (null: identity); seg [*n_seg + 1] run offsets; out
// [max_seg, D] bf16 or fp32; partial: b200_segment_sum_scratch_elems(n, D) floats (null: every run is summed by one
// warp, whatever its length).
B200_API int b200_segment_sum_gather(const void* src, int src_is_f32, long long src_rows, const long long* perm,
                                     const long long* seg, const long long* n_seg, long long n, long long max_seg, int D,
                                     void* out, int out_bf16, float* partial, void* stream) {
  if (max_seg <= 0 || n <= 0) return 0;
  if (D % 8 != 0 || ((uintptr_t)src & 15) || ((uintptr_t)out & 15) || ((uintptr_t)partial & 15))
    return b200::fail(1605, "segment_sum_gather: D=%d must be a multiple of 8 and the matrices 16-byte aligned", D);
  RowSrc s;
  s.bf16 = src_is_f32 ? nullptr : (const __nv_bfloat16*)src;
  s.f32 = src_is_f32 ? (const float*)src : nullptr;
  s.perm = perm; s.rows = src_rows; s.D = D;
  cudaStream_t st = (cudaStream_t)stream;
  if (partial != nullptr) {
    const long long blocks = (n + SEG_CHUNK - 1) / SEG_CHUNK;
    segment_partial_kernel<<<(unsigned)((blocks + 7) / 8), 256, 0, st>>>(s, seg, n_seg, n, partial, b200::status_ptr());
    b200::count_launch();
    int rc = b200::check_launch("segment_partial");
    if (rc) return rc;
  }
  const long long want = (max_seg + 7) / 8;            // 8 warps (runs) per CTA
  const int grid = (int)(want < 148 * 16 ? want : 148 * 16);
  if (out_bf16)
    segment_sum_gather_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(s, seg, n_seg, partial, (__nv_bfloat16*)out, b200::status_ptr());
  else
    segment_sum_gather_kernel<float><<<grid, 256, 0, st>>>(s, seg, n_seg, partial, (float*)out, b200::status_ptr());
  b200::count_launch();
  return b200::check_launch("segment_sum_gather");
}
