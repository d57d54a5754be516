// Sharded-embedding kernels.
//
//   gather_rows_to_peers : the owner of table rows answers every rank's requests in ONE kernel -
//                          each requested row is read from the local shard and stored directly into
//                          the requesting rank's receive buffer over NVLink (P2P stores), in the
//                          requester's order.  The row all-to-all and the lookup are one pass; there is
//                          no send buffer, no pack / unpack kernel and no collective-library call on
//                          the row traffic (the reference packs rows, calls an RCCL all-to-all and
//                          unpacks: generative_recommenders/dlrm_v4/seq_a2a_fused.py K1-K4,
//                          seq_a2a_rowperm.py:631-807).
//   rowwise_adagrad      : fused sparse optimizer on unique rows: state[r] += mean(g^2),
//                          row -= lr * g / (sqrt(state[r]) + eps)  (TorchRec's RowWiseAdagrad applied
//                          in backward, generative_recommenders/dlrm_v4/train/utils.py:1572-1578).
//   segment_sum_rows     : deterministic reduction of duplicate gradient rows after a sort
//                          (generative_recommenders/dlrm_v4/train/ec_segment_reduce.py).
#include "common.cuh"
#include "runtime.h"

namespace {

constexpr int MAXW = 16;
struct PeerBufs {
  void* p[MAXW];
  long long base_row[MAXW];   // first row of this owner's segment inside rank r's receive buffer
};

// requests are grouped by requesting rank: recv_off[r] .. recv_off[r+1]
__global__ void gather_rows_to_peers_kernel(const __nv_bfloat16* __restrict__ table, long long rows,
                                            const long long* __restrict__ local_idx,
                                            const long long* __restrict__ recv_off, int W, int D, PeerBufs out, int* status) {
  const int vpr = D / 8;
  const long long n = recv_off[W];
  const long long total = n * vpr;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long req = i / vpr;
    const int v = (int)(i % vpr);
    int r = 0;
    while (r + 1 < W && req >= recv_off[r + 1]) ++r;
    const long long id = local_idx[req];
    uint4 u = make_uint4(0, 0, 0, 0);
    if (id >= 0 && id < rows) u = *reinterpret_cast<const uint4*>(table + id * D + v * 8);
    else if (v == 0) B200_BOUNDS_REPORT(status, 1301);
    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(out.p[r]) + (out.base_row[r] + (req - recv_off[r])) * D + v * 8;
    *reinterpret_cast<uint4*>(dst) = u;
  }
}

// one warp per unique row
__global__ void rowwise_adagrad_kernel(__nv_bfloat16* __restrict__ table, float* __restrict__ state,
                                       const long long* __restrict__ ids, const float* __restrict__ grads, long long n,
                                       int D, float lr, float eps, long long rows, int* status) {
  const long long w = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (w >= n) return;
  const long long id = ids[w];
  if (id < 0 || id >= rows) {
    if (lane == 0 && id != -1) B200_BOUNDS_REPORT(status, 1302);   // -1 pads the unique list past the run count
    return;
  }
  const float* g = grads + w * D;
  float ss = 0.f;
  for (int d = lane; d < D; d += 32) ss += g[d] * g[d];
  ss = warp_sum(ss) / D;
  float st = state[id] + ss;
  if (lane == 0) state[id] = st;
  const float step = lr / (sqrtf(st) + eps);
  __nv_bfloat16* row = table + id * D;
  for (int d = lane; d < D; d += 32) row[d] = __float2bfloat16_rn(__bfloat162float(row[d]) - step * g[d]);
}

// out[s, :] = sum of src[seg[s] .. seg[s+1], :] in index order (src rows sorted by key)
__global__ void segment_sum_rows_kernel(const __nv_bfloat16* __restrict__ src, const long long* __restrict__ seg,
                                        long long n_seg, int D, float* __restrict__ out) {
  const long long s = blockIdx.x;
  if (s >= n_seg) return;
  const long long lo = seg[s], hi = seg[s + 1];
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float acc = 0.f;
    for (long long r = lo; r < hi; ++r) acc += __bfloat162float(src[r * D + d]);
    out[s * D + d] = acc;
  }
}

}  // namespace

// local_idx [n] (rows of this shard, grouped by requesting rank), recv_off [W+1] (device),
// out_ptrs[r] = base of rank r's receive buffer, base_rows[r] = first row there for this owner.
B200_API int b200_gather_rows_to_peers(const void* table, long long rows, const long long* local_idx,
                                       const long long* recv_off, long long n_host_upper, int W, int D,
                                       const unsigned long long* out_ptrs, const long long* base_rows, void* stream) {
  if (W > MAXW) return b200::fail(1300, "gather_rows_to_peers: world %d exceeds %d", W, MAXW);
  if (D % 8 != 0) return b200::fail(1301, "gather_rows_to_peers: D=%d must be a multiple of 8", D);
  if (n_host_upper <= 0) return 0;
  PeerBufs pb{};
  for (int r = 0; r < W; ++r) { pb.p[r] = reinterpret_cast<void*>(out_ptrs[r]); pb.base_row[r] = base_rows[r]; }
  long long work = n_host_upper * (D / 8);
  long long g = (work + 255) / 256;
  long long cap = (long long)b200::sm_count() * 16;
  gather_rows_to_peers_kernel<<<(unsigned)(g < cap ? g : cap), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)table, rows, local_idx, recv_off, W, D, pb, b200::status_ptr());
  b200::count_launch();
  return b200::check_launch("gather_rows_to_peers");
}

B200_API int b200_rowwise_adagrad(void* table, float* state, const long long* ids, const float* grads, long long n,
                                  int D, float lr, float eps, long long rows, void* stream) {
  if (n <= 0) return 0;
  const long long threads = n * 32;
  rowwise_adagrad_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
      (__nv_bfloat16*)table, state, ids, grads, n, D, lr, eps, rows, b200::status_ptr());
  b200::count_launch();
  return b200::check_launch("rowwise_adagrad");
}

B200_API int b200_segment_sum_rows(const void* src, const long long* seg, long long n_seg, int D, float* out, void* stream) {
  if (n_seg <= 0) return 0;
  segment_sum_rows_kernel<<<(unsigned)n_seg, 128, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)src, seg, n_seg, D, out);
  b200::count_launch();
  return b200::check_launch("segment_sum_rows");
}
