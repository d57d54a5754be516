"""Device-timed comparison of the fused tensor-parallel GEMMs with their NCCL + GEMM baselines.

    torchrun --nproc-per-node W -m mlperf_training_b200.utils.microbench_tp [--tokens 8192] [--hidden 8192] [--ffn 28672]

For each of all-gather->GEMM (column-parallel forward) and GEMM->reduce-scatter (row-parallel
forward) it prints one JSON line: milliseconds (max over ranks, median of the timed launches, L2
flushed between them), achieved TFLOP/s per GPU, the NVLink bytes per GPU and the roofline time
max(FLOPs / measured GEMM peak, bytes / measured per-direction NVLink bandwidth).
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

from ..ops import kernels as K
from ..parallel.tensor import TPContext

GEMM_PEAK_TFLOPS = 1421.6      # measured sustained cuBLAS bf16 on the B200s these numbers were taken on
NVLINK_GBS = 770.0             # measured peer copy, per direction


def timed(fn, iters, warmup, flush):
    for _ in range(warmup):
        fn()
    ts = []
    for _ in range(iters):
        flush.zero_()
        dist.barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b))
    ts.sort()
    t = torch.tensor([ts[len(ts) // 2]], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--hidden", type=int, default=8192)
    ap.add_argument("--ffn", type=int, default=28672)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--n-copy", type=int, default=0, help="copy CTAs of the all-gather kernel (0 = default)")
    ap.add_argument("--n-red", type=int, default=0, help="dedicated reduce CTAs of the reduce-scatter kernel (0 = default)")
    ap.add_argument("--copy-sweep", action="store_true", help="also time the all-gather copies alone for several n_copy")
    args = ap.parse_args(argv)
    rank = int(os.environ.get("RANK", "0"))
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    dist.init_process_group("nccl")
    W = dist.get_world_size()
    dev = torch.device("cuda", torch.cuda.current_device())
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    T, D, Fl = args.tokens, args.hidden, 2 * args.ffn // W
    fused, nccl = TPContext(None, "fused", dev), TPContext(None, "nccl", dev)
    x_shard = torch.randn(T // W, D, device=dev).bfloat16()
    w_col = (torch.randn(Fl, D, device=dev) * 0.02).bfloat16()
    act = torch.randn(T, args.ffn // W, device=dev).bfloat16()
    w_row = (torch.randn(D, args.ffn // W, device=dev) * 0.02).bfloat16()

    def ag_fused():
        buf, full = fused.gather_begin(x_shard)
        return fused.gemm_gather(buf, full, w_col, mode=1)

    def ag_nccl():
        return K.gemm(nccl.all_gather_rows(x_shard), w_col)

    def rs_fused():
        return fused.gemm_reduce_scatter(act, w_row)

    def rs_nccl():
        return nccl.reduce_scatter_rows(K.gemm(act, w_row))

    if args.n_copy:
        fused.n_copy = args.n_copy
    if args.n_red:
        fused.n_red = args.n_red
    err_ag = (ag_fused().float() - ag_nccl().float()).abs().max().item()
    err_rs = (rs_fused().float() - rs_nccl().float()).abs().max().item()
    for name, f_fused, f_nccl, flops, link_bytes, err in (
            ("all_gather_gemm", ag_fused, ag_nccl, 2.0 * T * Fl * D, (W - 1) / W * T * D * 2, err_ag),
            ("gemm_reduce_scatter", rs_fused, rs_nccl, 2.0 * T * D * (args.ffn // W), (W - 1) / W * T * D * 2, err_rs)):
        t_f = timed(f_fused, args.iters, args.warmup, flush)
        t_n = timed(f_nccl, args.iters, args.warmup, flush)
        roof_ms = max(flops / (GEMM_PEAK_TFLOPS * 1e12), link_bytes / (NVLINK_GBS * 1e9)) * 1e3
        if rank == 0:
            print(json.dumps({"kernel": name, "world": W, "n_copy": fused.n_copy, "n_red": fused.n_red, "tokens": T, "hidden": D, "ffn": args.ffn, "fused_ms": round(t_f, 4),
                              "nccl_plus_gemm_ms": round(t_n, 4), "speedup": round(t_n / t_f, 3),
                              "fused_tflops_per_gpu": round(flops / t_f / 1e9, 1), "nvlink_mb_per_gpu": round(link_bytes / 1e6, 1),
                              "roofline_ms": round(roof_ms, 4), "fraction_of_roofline": round(roof_ms / t_f, 3),
                              "max_abs_diff_vs_nccl": err}), flush=True)
    # the same two linears with a frozen weight on per-tensor FP8 operands (quantisation of the activation included)
    from ..ops import fp8 as F8
    from ..ops.linear import _site, fp8_weight_operands, weight_epoch
    f8 = TPContext(None, "fused", dev, precision="fp8")
    if args.n_copy:
        f8.n_copy = args.n_copy
    if args.n_red:
        f8.n_red = args.n_red
    w_col.requires_grad_(False), w_row.requires_grad_(False)

    def ag_fp8():
        st = f8.shared_site(w_col, "x", "e4m3")
        f8.prepare_shared(st, x_shard)
        xq, _ = F8.quantize(x_shard, st)
        buf, full = f8.gather_begin_codes(xq.q)
        return f8.gemm_gather_fp8(buf, full, st.inv_scale, "e4m3", fp8_weight_operands(w_col)[0])

    def rs_fp8():
        st = _site(w_row, "x", "e4m3")
        st.prepare(act, weight_epoch())
        aq, _ = F8.quantize(act, st)
        return f8.gemm_reduce_scatter_fp8(aq, fp8_weight_operands(w_row)[0])

    for name, fn, ref, flops, link_bytes in (
            ("all_gather_gemm_fp8", ag_fp8, ag_nccl, 2.0 * T * Fl * D, (W - 1) / W * T * D),
            ("gemm_reduce_scatter_fp8", rs_fp8, rs_nccl, 2.0 * T * D * (args.ffn // W), (W - 1) / W * T * D * 2)):
        a, b = fn().float(), ref().float()
        rel = ((a - b).norm() / b.norm()).item()
        t_f = timed(fn, args.iters, args.warmup, flush)
        if rank == 0:
            print(json.dumps({"kernel": name, "world": W, "tokens": T, "hidden": D, "ffn": args.ffn, "fused_ms": round(t_f, 4),
                              "fused_tflops_per_gpu": round(flops / t_f / 1e9, 1), "nvlink_mb_per_gpu": round(link_bytes / 1e6, 1),
                              "rel_diff_vs_bf16": round(rel, 4)}), flush=True)
    if args.copy_sweep:
        # all-gather with a negligible GEMM (N = 128): the time is the in-kernel copy of the peers' blocks
        w_small = (torch.randn(128, D, device=dev) * 0.02).bfloat16()
        for n_copy in (4, 8, 16, 32):
            fused.n_copy = n_copy

            def ag_small():
                buf, full = fused.gather_begin(x_shard)
                return fused.gemm_gather(buf, full, w_small, mode=1)
            t = timed(ag_small, args.iters, args.warmup, flush)
            if rank == 0:
                mb = (W - 1) / W * T * D * 2 / 1e6
                print(json.dumps({"kernel": "all_gather_copy_only", "world": W, "n_copy": n_copy, "ms": round(t, 4),
                                  "pulled_mb": round(mb, 1), "gb_per_s": round(mb / t, 1)}), flush=True)
    from ..ops import _lib
    _lib.check_status("microbench_tp")
    dist.barrier()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
