// Expert-parallel token movement over NVLink peer memory.
//
//   scatter_rows_to_peers  (dispatch, and the backward of combine): row i of a local matrix is
//       stored straight into row dst_row[i] of rank dst_rank[i]'s slab - the slab is laid out
//       expert-major on the owner (128-row padded segments, inside a segment the source ranks in
//       order), so the rows arrive already grouped for the grouped GEMM: no send buffer, no
//       all-to-all call, no regrouping pass on the owner.
//   gather_rows_from_peers (combine, and the backward of dispatch): row i of the local result is
//       loaded from row src_row[i] of rank src_rank[i]'s slab.
//   zero_pad_rows          clears the padding rows of every segment (they enter the weight-gradient
//       contraction and must be zero).
//
// The routing tables are computed on the device from the all-gathered per-expert counts; nothing
// in the layer reads a size back to the host.  Rows whose slot is negative (slab capacity
// exceeded) are skipped / returned as zero and counted in `dropped`.
//
// The reference moves tokens with Megatron's all-to-all dispatcher around a library grouped GEMM
// (small_llm_moe_pretraining/primus/conf/gpt_oss_20B-MXFP4-deosc-mlperf-pretrain.yaml:160-167).
#include "common.cuh"
#include "runtime.h"

namespace {

constexpr int MAXW = 16;
struct Peers { uint8_t* p[MAXW]; };

__global__ void __launch_bounds__(256)
scatter_rows_kernel(const __nv_bfloat16* __restrict__ src, const int* __restrict__ src_row, const int* __restrict__ dst_rank,
                    const int* __restrict__ dst_row, long long n, int D, Peers out, int W, long long cap, int* dropped) {
  const int vpr = D / 8;
  const long long total = n * vpr;
  for (long long i = blockIdx.x * 256ll + threadIdx.x; i < total; i += (long long)gridDim.x * 256) {
    const long long r = i / vpr;
    const int v = (int)(i - r * vpr);
    const int rk = dst_rank[r];
    const long long row = dst_row[r];
    if (rk < 0 || rk >= W || row < 0 || row >= cap) {
      if (v == 0 && dropped != nullptr) atomicAdd(dropped, 1);
      continue;
    }
    const long long s = src_row != nullptr ? src_row[r] : r;
    const uint4 u = *reinterpret_cast<const uint4*>(src + s * D + v * 8);
    *reinterpret_cast<uint4*>(out.p[rk] + (row * D + v * 8) * 2) = u;
  }
}

__global__ void __launch_bounds__(256)
gather_rows_kernel(Peers in, const int* __restrict__ src_rank, const int* __restrict__ src_row, long long n, int D,
                   __nv_bfloat16* __restrict__ out, int W, long long cap) {
  const int vpr = D / 8;
  const long long total = n * vpr;
  for (long long i = blockIdx.x * 256ll + threadIdx.x; i < total; i += (long long)gridDim.x * 256) {
    const long long r = i / vpr;
    const int v = (int)(i - r * vpr);
    const int rk = src_rank[r];
    const long long row = src_row[r];
    uint4 u = make_uint4(0, 0, 0, 0);
    if (rk >= 0 && rk < W && row >= 0 && row < cap) {
      const uint8_t* p = in.p[rk] + (row * D + v * 8) * 2;
      asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(u.x), "=r"(u.y), "=r"(u.z), "=r"(u.w) : "l"(p));
    }
    *reinterpret_cast<uint4*>(out + r * D + v * 8) = u;
  }
}

// one CTA per local expert: rows [seg[e] + count[e], seg[e+1]) are padding
__global__ void zero_pad_rows_kernel(__nv_bfloat16* __restrict__ buf, const int* __restrict__ seg,
                                     const int* __restrict__ count, int D, long long cap) {
  const int e = blockIdx.x;
  long long lo = (long long)seg[e] + count[e], hi = seg[e + 1];
  if (hi > cap) hi = cap;
  const int vpr = D / 8;
  for (long long i = threadIdx.x; i < (hi - lo) * vpr; i += blockDim.x)
    *reinterpret_cast<uint4*>(buf + (lo + i / vpr) * D + (i % vpr) * 8) = make_uint4(0, 0, 0, 0);
}

// Routing tables of the peer-memory dispatch from the all-gathered per-expert counts, in one launch.
//   allc [W, E]   pairs every rank routes to every (global) expert
//   seg  [E + 1]  offsets of this rank's pairs sorted by global expert (unpadded)
// Every expert's segment on its owner starts at a multiple of `pad` rows; inside it the sources' rows follow in
// rank order.  Outputs: dst_rank / dst_row [n] for this rank's sorted pairs (row -1 = beyond the slab capacity),
// seg2 [L + 1] / cnt2 [L] / tile_expert [cap / pad] for the experts this rank owns.
constexpr int ROUTE_MAX_E = 1024;
__global__ void __launch_bounds__(256)
ep_route_kernel(const int* __restrict__ allc, const int* __restrict__ seg, int W, int E, int L, int rank, int pad,
                long long cap, long long n, int* __restrict__ dst_rank, int* __restrict__ dst_row, int* __restrict__ seg2,
                int* __restrict__ cnt2, int* __restrict__ tile_expert, int n_tiles) {
  __shared__ long long base[ROUTE_MAX_E];         // first row of this rank's pairs of expert e on the owner
  __shared__ int padded[ROUTE_MAX_E];
  __shared__ int my_seg[ROUTE_MAX_E + 1];
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int tot = 0, before = 0;
    for (int w = 0; w < W; ++w) {
      const int c = allc[w * E + e];
      tot += c;
      if (w < rank) before += c;
    }
    padded[e] = (tot + pad - 1) / pad * pad;
    base[e] = before;
    if (blockIdx.x == 0 && e / L == rank) cnt2[e - rank * L] = tot;
  }
  for (int e = threadIdx.x; e <= E; e += blockDim.x) my_seg[e] = seg[e];
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    long long start = 0;
    for (int j = (e / L) * L; j < e; ++j) start += padded[j];
    base[e] += start;                              // each thread updates only its own entries: no race with the reads of padded[]
  }
  __syncthreads();
  if (blockIdx.x == 0) {
    // this rank's own segments and the expert of every `pad`-row tile of its slab
    __shared__ long long own[ROUTE_MAX_E + 1];
    if (threadIdx.x == 0) {
      long long acc = 0;
      own[0] = 0;
      for (int l = 0; l < L; ++l) { acc += padded[rank * L + l]; own[l + 1] = acc; }
      for (int l = 0; l <= L; ++l) seg2[l] = (int)(own[l] < cap ? own[l] : cap);
    }
    __syncthreads();
    for (int t = threadIdx.x; t < n_tiles; t += blockDim.x) {
      const long long row = (long long)t * pad;
      int e = -1;
      if (row < own[L]) {
        int lo = 0, hi = L - 1;
        while (lo < hi) { const int mid = (lo + hi + 1) >> 1; if (own[mid] <= row) lo = mid; else hi = mid - 1; }
        e = lo;
      }
      tile_expert[t] = e;
    }
  }
  for (long long i = blockIdx.x * 256ll + threadIdx.x; i < n; i += (long long)gridDim.x * 256) {
    int lo = 0, hi = E - 1;                        // last expert whose segment starts at or before pair i and is not empty before i
    while (lo < hi) { const int mid = (lo + hi + 1) >> 1; if (my_seg[mid] <= i) lo = mid; else hi = mid - 1; }
    const int e = lo;
    const long long row = base[e] + (i - my_seg[e]);
    dst_rank[i] = e / L;
    dst_row[i] = row < cap ? (int)row : -1;
  }
}

int grid_for(long long work) {
  long long g = (work + 255) / 256;
  const long long cap = (long long)b200::sm_count() * 16;
  return (int)(g < cap ? (g < 1 ? 1 : g) : cap);
}

}  // namespace

// out_ptrs[r]: base of rank r's slab ([cap, D] bf16).  src_row may be null (row i of src).
B200_API int b200_scatter_rows_to_peers(const void* src, const int* src_row, const int* dst_rank, const int* dst_row,
                                        long long n, int D, const unsigned long long* out_ptrs, int W, long long cap,
                                        int* dropped, void* stream) {
  if (W < 1 || W > MAXW) return b200::fail(1600, "scatter_rows_to_peers: world %d out of range", W);
  if (D % 8 != 0) return b200::fail(1601, "scatter_rows_to_peers: D=%d must be a multiple of 8", D);
  if (n <= 0) return 0;
  Peers pe{};
  for (int r = 0; r < W; ++r) pe.p[r] = reinterpret_cast<uint8_t*>(out_ptrs[r]);
  scatter_rows_kernel<<<grid_for(n * (D / 8)), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)src, src_row, dst_rank, dst_row, n, D, pe, W, cap, dropped);
  b200::count_launch();
  return b200::check_launch("scatter_rows_to_peers");
}

B200_API int b200_gather_rows_from_peers(const unsigned long long* in_ptrs, const int* src_rank, const int* src_row,
                                         long long n, int D, void* out, int W, long long cap, void* stream) {
  if (W < 1 || W > MAXW) return b200::fail(1610, "gather_rows_from_peers: world %d out of range", W);
  if (D % 8 != 0) return b200::fail(1611, "gather_rows_from_peers: D=%d must be a multiple of 8", D);
  if (n <= 0) return 0;
  Peers pe{};
  for (int r = 0; r < W; ++r) pe.p[r] = reinterpret_cast<uint8_t*>(in_ptrs[r]);
  gather_rows_kernel<<<grid_for(n * (D / 8)), 256, 0, (cudaStream_t)stream>>>(pe, src_rank, src_row, n, D,
                                                                              (__nv_bfloat16*)out, W, cap);
  b200::count_launch();
  return b200::check_launch("gather_rows_from_peers");
}

B200_API int b200_zero_pad_rows(void* buf, const int* seg, const int* count, int n_seg, int D, long long cap, void* stream) {
  if (D % 8 != 0) return b200::fail(1620, "zero_pad_rows: D=%d must be a multiple of 8", D);
  if (n_seg <= 0) return 0;
  zero_pad_rows_kernel<<<n_seg, 256, 0, (cudaStream_t)stream>>>((__nv_bfloat16*)buf, seg, count, D, cap);
  b200::count_launch();
  return b200::check_launch("zero_pad_rows");
}

// See ep_route_kernel.  allc [W, E] int32 (all-gathered counts), seg [E + 1] int32; all pointers on the device.
B200_API int b200_ep_route(const int* allc, const int* seg, int W, int E, int rank, int pad, long long cap, long long n,
                           int* dst_rank, int* dst_row, int* seg2, int* cnt2, int* tile_expert, void* stream) {
  if (W < 1 || E < W || E % W != 0 || E > ROUTE_MAX_E || pad < 1 || cap % pad != 0)
    return b200::fail(1630, "ep_route: W=%d E=%d pad=%d cap=%lld", W, E, pad, cap);
  const int n_tiles = (int)(cap / pad);
  ep_route_kernel<<<grid_for(n > 0 ? n : 1), 256, 0, (cudaStream_t)stream>>>(allc, seg, W, E, E / W, rank, pad, cap, n, dst_rank,
                                                                           dst_row, seg2, cnt2, tile_expert, n_tiles);
  b200::count_launch();
  return b200::check_launch("ep_route");
}
