"""Device-timed comparison of the peer-memory token / row movement with its NCCL baselines.

    torchrun --nproc-per-node W -m mlperf_training_b200.utils.microbench_ep

* ``moe_layer``: routed expert MLP forward + backward on GPT-OSS-20B shapes (8192 tokens, hidden 2880,
  32 experts, top-4, expert FFN 2880) with the all-to-all dispatcher and with the fused one.
* ``embedding``: sharded-embedding lookup + backward (row-wise Adagrad) for one HSTU batch
  (128 users, log-normal lengths, Zipf ids) with ``all_to_all_single`` and with the fused gather.

One JSON line per measurement (milliseconds: median of the timed launches, max over ranks).
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

from ..ops import _lib
from ..ops import moe_ops as M
from ..parallel.embedding import ShardedEmbedding
from ..parallel.expert import ExpertParallelDispatcher, FusedExpertDispatcher


def timed(fn, iters, warmup):
    for _ in range(warmup):
        fn()
    ts = []
    for _ in range(iters):
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
    return float(t)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=8)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--table-rows", type=int, default=20_000_000)
    args = ap.parse_args(argv)
    rank = int(os.environ.get("RANK", "0"))
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    dev = torch.device("cuda", torch.cuda.current_device())
    dist.init_process_group("nccl", device_id=dev)
    W = dist.get_world_size()

    # ---------------- MoE layer ----------------
    T, D, E, k, Fh = args.tokens, 2880, 32, 4, 2880
    L = E // W
    torch.manual_seed(rank)
    x = torch.randn(T, D, device=dev).bfloat16().requires_grad_(True)
    logits = torch.randn(T, E, device=dev)
    w1 = (torch.randn(L, 2 * Fh, D, device=dev) * 0.02).bfloat16().requires_grad_(True)
    w2 = (torch.randn(L, D, Fh, device=dev) * 0.02).bfloat16().requires_grad_(True)
    gy = torch.randn(T, D, device=dev).bfloat16()
    w1.main_grad, w2.main_grad = torch.zeros_like(w1, dtype=torch.float32), torch.zeros_like(w2, dtype=torch.float32)
    flops = 3 * 2.0 * T * k * (3 * D * Fh)              # fwd + dgrad + wgrad of fc1 (2F) and fc2 (F), all ranks' tokens land somewhere
    for precision in ("bf16", "mxfp8"):
        disp = {"nccl": ExpertParallelDispatcher(dist.group.WORLD, E),
                "fused": FusedExpertDispatcher(dist.group.WORLD, E, D, T * k, dev, pad=M.pad_rows(precision))}
        res = {}
        for name, d in disp.items():
            def layer():
                idx, w, counts = M.RouterFn.apply(logits, k)
                y = d(x, idx, w, counts, w1, w2, precision)
                y.backward(gy)
                x.grad = None
            res[name] = timed(layer, args.iters, args.warmup)
        if rank == 0:
            print(json.dumps({"kernel": "moe_layer_fwd_bwd", "precision": precision, "world": W, "tokens_per_rank": T, "hidden": D,
                              "experts": E, "top_k": k, "nccl_all_to_all_ms": round(res["nccl"], 3),
                              "fused_peer_ms": round(res["fused"], 3), "speedup": round(res["nccl"] / res["fused"], 3),
                              "expert_gemm_tflops_per_gpu_fused": round(flops / res["fused"] / 1e9, 1),
                              "dropped_pairs": int(disp["fused"].dropped.item())}), flush=True)
        del disp

    # ---------------- sharded embedding ----------------
    from ..data.hstu_synth import HSTUSyntheticData
    data = HSTUSyntheticData(args.table_rows, 128, seed=0)
    ids = data.batch_at(0, rank)["item_ids"].to(dev)
    res = {}
    for comm in ("nccl", "fused"):
        tab = ShardedEmbedding(args.table_rows, 256, device=dev, dtype=torch.bfloat16, lr=0.01, comm=comm, max_requests=1 << 18)
        g = torch.randn(ids.numel(), 256, device=dev).bfloat16()

        def look():
            out = tab.lookup(ids)
            out.backward(g)
        res[comm] = timed(look, args.iters, args.warmup)
    if rank == 0:
        print(json.dumps({"kernel": "sharded_embedding_lookup_bwd", "world": W, "ids_per_rank": int(ids.numel()), "dim": 256,
                          "table_rows": args.table_rows, "nccl_all_to_all_ms": round(res["nccl"], 3),
                          "fused_peer_gather_ms": round(res["fused"], 3), "speedup": round(res["nccl"] / res["fused"], 3)}), flush=True)
    torch.cuda.synchronize()
    _lib.check_status("microbench_ep")
    dist.barrier()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
