// Copy roles of the all-gather -> GEMM kernels: CTAs of the SAME launch as the GEMM move the ranks' blocks of the
// gathered operand over NVLink peer memory and publish one counter per block, which the TMA producers of the
// GEMM CTAs wait on.  Shared by the one-CTA-per-tile kernel (gemm_tp.cu) and the CTA-pair kernel (gemm_core.cuh).
//
// `P` provides: W, rank, peer_src[], gdst, chunk_bytes, pieces_per_chunk, chunk_flag, chunk_flag_peer[], status.
// `cta` / `n_cta`: index of this copy CTA among the launch's copy CTAs and their number.
#pragma once
#include "common.cuh"

namespace tpcopy {

constexpr int COPY_PIECE = 32768;     // bytes per bulk copy (pull mode)
constexpr int COPY_STAGES = 6;
constexpr int PUSH_PIECE = 262144;    // bytes per published piece (push mode)

B200_DEVICE void bulk_g2s(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
B200_DEVICE void bulk_s2g(void* gdst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst), "r"(smem_u32(smem_src)),
               "r"(bytes)
               : "memory");
}
B200_DEVICE void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }
B200_DEVICE void red_release_gpu_add(int* p, int v) {
  asm volatile("red.release.gpu.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
B200_DEVICE void red_release_sys_add(int* p, int v) {
  asm volatile("red.release.sys.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
B200_DEVICE uint4 ld_cg_u4(const void* p) {
  uint4 v;
  asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

// One thread drives a ring of bulk copies peer -> shared -> local and publishes a piece two
// stores after it was issued (its bulk group is then complete).
template <class P>
B200_DEVICE void copy_cta(const P& p, int cta, int n_cta, uint8_t* smem, uint64_t* bars) {
  if (threadIdx.x != 0) return;
  for (int i = 0; i < COPY_STAGES; ++i) mbar_init(&bars[i], 1);
  mbar_fence_init();
  const int ppc = p.pieces_per_chunk;
  const int total = (p.W - 1) * ppc;
  const int mine = (total - cta + n_cta - 1) / n_cta;   // pieces cta, cta + n_cta, ...
  volatile int dummy_abort = 0;
  auto piece_of = [&](int i, int& chunk, long long& off, uint32_t& bytes) {
    const int g = cta + i * n_cta;
    chunk = (p.rank + 1 + g / ppc) % p.W;
    off = (long long)(g % ppc) * COPY_PIECE;
    const long long left = p.chunk_bytes - off;
    bytes = (uint32_t)(left < COPY_PIECE ? left : COPY_PIECE);
  };
  auto issue_load = [&](int i) {
    int c; long long off; uint32_t bytes;
    piece_of(i, c, off, bytes);
    const int s = i % COPY_STAGES;
    mbar_expect_tx(&bars[s], bytes);
    bulk_g2s(smem + s * COPY_PIECE, p.peer_src[c] + (long long)c * p.chunk_bytes + off, bytes, &bars[s]);
  };
  auto publish = [&](int i) {
    int c; long long off; uint32_t bytes;
    piece_of(i, c, off, bytes);
    fence_proxy_async_all();
    red_release_gpu_add(p.chunk_flag + c, 1);
  };
  const int ahead = COPY_STAGES - 2;
  for (int i = 0; i < mine && i < ahead; ++i) issue_load(i);
  bool ok = true;
  for (int i = 0; i < mine; ++i) {
    const int s = i % COPY_STAGES;
    if (!mbar_wait(&bars[s], (i / COPY_STAGES) & 1, &dummy_abort, p.status, 40)) { ok = false; break; }
    int c; long long off; uint32_t bytes;
    piece_of(i, c, off, bytes);
    bulk_s2g(p.gdst + (long long)c * p.chunk_bytes + off, smem + s * COPY_PIECE, bytes);
    tma_store_commit();
    tma_store_wait_all<2>();                 // stores up to i-2 are complete
    if (i >= 2) publish(i - 2);
    if (i + ahead < mine) issue_load(i + ahead);   // stage (i-2) % STAGES: its store has completed
  }
  tma_store_wait_all<0>();
  if (ok) {
    if (mine >= 2) publish(mine - 2);
    if (mine >= 1) publish(mine - 1);
  } else {
    // loads that never completed may still land: give them time before shared memory is released
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
}

// Push variant: every thread of the CTA copies 16-byte vectors of this rank's block from local memory
// straight into every peer's buffer (plain posted stores: no round trip per piece), and one thread
// bumps the peers' counters after each PUSH_PIECE bytes, behind a system-scope fence.
template <class P>
B200_DEVICE void copy_cta_push(const P& p, int cta, int n_cta, int nthreads) {
  // Work items are (destination, piece), destination-major: the rank that consumes this block first
  // (rank - 1: it visits its own block, then rank + 1's, ...) receives all of it first.
  const int ppc = (int)((p.chunk_bytes + PUSH_PIECE - 1) / PUSH_PIECE);
  const long long base = (long long)p.rank * p.chunk_bytes;
  const uint8_t* src = p.gdst + base;
  const int items = (p.W - 1) * ppc;
  for (int it = cta; it < items; it += n_cta) {
    const int d = (p.rank - 1 - it / ppc + 2 * p.W) % p.W;
    const long long off = (long long)(it % ppc) * PUSH_PIECE;
    const long long left = p.chunk_bytes - off;
    const int nvec = (int)((left < PUSH_PIECE ? left : PUSH_PIECE) / 16);
    uint8_t* dst = const_cast<uint8_t*>(p.peer_src[d]) + base + off;
    constexpr int U = 16;
    for (int v0 = threadIdx.x; v0 < nvec; v0 += U * nthreads) {
      uint4 q[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int v = v0 + u * nthreads;
        if (v < nvec) q[u] = ld_cg_u4(src + off + (long long)v * 16);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int v = v0 + u * nthreads;
        if (v < nvec) *reinterpret_cast<uint4*>(dst + (long long)v * 16) = q[u];
      }
    }
    __threadfence_system();
    named_bar_sync(3, nthreads);
    if (threadIdx.x == 0) red_release_sys_add(p.chunk_flag_peer[d] + p.rank, 1);
  }
}

}  // namespace tpcopy
