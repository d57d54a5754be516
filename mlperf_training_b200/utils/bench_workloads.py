"""Device-timed training throughput of the workloads other than the flagship dense Llama
(``bench.py`` at the repository root covers that one):

    torchrun --nproc-per-node N -m mlperf_training_b200.utils.bench_workloads <workload> [--steps K --warmup W]

    gpt-oss-20b   MoE pre-training, expert parallel over all ranks (tokens/s)
    llama2-70b-lora   LoRA SFT, tensor + sequence parallel over all ranks, loss on the last 1024 positions (tokens/s)
    flux1         MMDiT flow matching, 256 image + 256 text tokens per sample (samples/s)
    hstu          8-layer HSTU ranker with a row-wise sharded item table (samples/s)

Synthetic data of the configured shapes, random-init weights.  ``W`` untimed steps, then ``K`` steps
between a barrier + synchronize, CUDA events on the launching stream, maximum over ranks; one JSON
line from rank 0.  ``--layers`` / ``--scale`` shrink a model for smoke runs (the line then says
``"reduced": true``).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist


def _timed(step_fn, steps: int, warmup: int, world: int):
    for i in range(warmup):
        step_fn(i)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    last = None
    for i in range(steps):
        last = step_fn(warmup + i)
    b.record()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    t = torch.tensor([a.elapsed_time(b)], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t) / steps, (float(last) if last is not None else None)


def bench_gpt_oss(args, rank, world, dev):
    from ..models.gpt import GPT, gpt_oss_20b
    from ..parallel.engine import OptimConfig, ZeroEngine
    cfg = gpt_oss_20b(precision=args.precision if args.precision in ("bf16", "mxfp8") else "bf16", ep_comm=args.comm)
    if args.layers:
        cfg.n_layers = args.layers
    ep = dist.group.WORLD if world > 1 else None
    model = GPT(cfg, dev, seed=0, ep_group=ep)
    eng = ZeroEngine(model, OptimConfig(lr=4e-4, weight_decay=0.1, clip_grad=1.0))
    local = max(args.global_batch // world, 1) if args.global_batch else 2
    g = torch.Generator().manual_seed(rank)
    toks = torch.randint(0, cfg.vocab_size, (local, cfg.seq_len + 1), generator=g).to(dev)

    def step(i):
        tot = None
        for m in range(local):
            loss = model(toks[m:m + 1, :-1], toks[m:m + 1, 1:])
            loss.backward()
            tot = loss.detach() if tot is None else tot + loss.detach()
        eng.step(grad_scale=1.0 / local)
        return tot / local
    ms, loss = _timed(step, args.steps, args.warmup, world)
    tokens = local * cfg.seq_len * world
    return {"metric": "train tokens/s", "value": tokens / (ms / 1e3), "unit": "tokens/s", "ms_per_step": ms, "loss": loss,
            "config": {"model": cfg.name, "layers": cfg.n_layers, "experts": cfg.n_experts, "top_k": cfg.top_k,
                       "global_batch": local * world, "seq_len": cfg.seq_len, "parallelism": f"ep{world} ({args.comm} dispatch) + dp{world} dense",
                       "linears": ("MXFP8 grouped experts on the CTA-pair core (bf16 where a width is not a multiple of 128)"
                                   if cfg.precision == "mxfp8" else "bf16 tcgen05 (grouped experts), bf16 dense")}}


def bench_llama70b_lora(args, rank, world, dev):
    from ..models.gpt import llama2_70b
    from ..parallel.engine import OptimConfig
    from ..parallel.tensor import TPContext
    from ..trainer.pretrain import PretrainTrainer, TrainConfig
    cfg = llama2_70b(precision="bf16", lora_rank=16, lora_alpha=32.0, lora_dropout=0.1)
    if args.layers:
        cfg.n_layers = args.layers
    tp_prec = "fp8" if (args.precision != "bf16" and args.comm == "fused") else "bf16"
    tp = TPContext(dist.group.WORLD, comm="fused" if args.comm == "fused" else "nccl", device=dev, precision=tp_prec) if world > 1 else None
    solo = [dist.new_group([r]) for r in range(world)][rank] if world > 1 else None
    local = args.global_batch or 8                       # data-parallel size 1: every rank sees the whole batch
    tr = PretrainTrainer(cfg, OptimConfig(lr=4e-4, beta2=0.999, eps=1e-8, weight_decay=1e-4, clip_grad=0.3),
                         TrainConfig(micro_batch=args.micro_batch or 4, local_batch=local, warmup_steps=0, seed=0), dev, group=solo, tp=tp,
                         freeze_base=True)
    g = torch.Generator().manual_seed(0)
    toks = torch.randint(0, cfg.vocab_size, (local, cfg.seq_len + 1), generator=g).to(dev)
    x, y = toks[:, :-1].contiguous(), toks[:, 1:].clone()
    y[:, : cfg.seq_len - 1024] = -100
    ms, loss = _timed(lambda i: tr.train_step_device(x, y), args.steps, args.warmup, world)
    tokens = local * cfg.seq_len
    return {"metric": "train tokens/s", "value": tokens / (ms / 1e3), "unit": "tokens/s", "ms_per_step": ms, "loss": loss,
            "config": {"model": cfg.name, "layers": cfg.n_layers, "global_batch": local, "seq_len": cfg.seq_len,
                       "micro_batch": args.micro_batch or 4, "lora": "rank 16 alpha 32 on qkv + proj, base frozen", "loss_positions": 1024,
                       "parallelism": f"tp{world} + sequence parallel ({args.comm} all-gather->GEMM / GEMM->reduce-scatter)",
                       "linears": "frozen base on per-tensor FP8 (e4m3 forward, e5m2 gradients), LoRA bf16" if tp_prec == "fp8" else "bf16 tcgen05"}}


def bench_flux(args, rank, world, dev):
    from ..models.mmdit import flux1_schnell
    from ..parallel.engine import OptimConfig
    from ..trainer.flux import FluxTrainer, SyntheticFluxData
    cfg = flux1_schnell(precision=args.precision)
    if args.layers:
        cfg.n_double, cfg.n_single = args.layers, 2 * args.layers
    local = max((args.global_batch or 256) // world, 1)
    if args.scale:
        local = max(local // args.scale, 1)
    tr = FluxTrainer(cfg, OptimConfig(lr=2.5e-4, beta2=0.95, eps=1e-8, weight_decay=0.1, clip_grad=1.0), dev, local,
                     comm="nccl", seed=0, micro_batch=min(local, args.micro_batch or 8))
    data = SyntheticFluxData(cfg, seed=0)
    lat, txt, vec = (t.to(dev) for t in data.batch(0, rank, local))
    dt = cfg.torch_dtype() if hasattr(cfg, "torch_dtype") else torch.bfloat16
    lat, txt, vec = lat.to(dt), txt.to(dt), vec.to(dt)
    ms, loss = _timed(lambda i: tr.train_step_device(lat, txt, vec), args.steps, args.warmup, world)
    return {"metric": "train samples/s", "value": local * world / (ms / 1e3), "unit": "samples/s", "ms_per_step": ms, "loss": loss,
            "config": {"model": cfg.name, "double_blocks": cfg.n_double, "single_blocks": cfg.n_single, "global_batch": local * world,
                       "tokens_per_sample": cfg.img_tokens + cfg.txt_tokens, "parallelism": f"dp{world} (ZeRO-sharded optimizer)",
                       "linears": getattr(cfg, "precision", "bf16")}}


def bench_hstu(args, rank, world, dev):
    from ..models.hstu import HSTUConfig
    from ..trainer.hstu import HSTUTrainer
    cfg = HSTUConfig(layers=args.layers or 8, dim=512, heads=4, d_qk=128, d_v=128, max_seq_len=4096, emb_dim=256, dtype="bf16",
                     precision="bf16", fuse_glue=args.glue == "fused", attn_precision="fp8" if args.precision == "fp8" else "bf16")
    rows = 400_000_000 // (args.scale or 1)
    bpg = args.global_batch // world if args.global_batch else 128
    tr = HSTUTrainer(cfg, rows, bpg, dev, emb_comm=args.comm, seed=0,
                     data_kw=dict(length_median=512, length_min=16, length_max=4096, zipf_alpha=1.05,
                                  balance_world=world if args.balance else 0))
    ms, loss = _timed(lambda i: tr.train_step(i), args.steps, args.warmup, world)
    return {"metric": "train samples/s", "value": bpg * world / (ms / 1e3), "unit": "samples/s", "ms_per_step": ms, "loss": loss,
            "config": {"model": "hstu", "layers": cfg.layers, "dim": cfg.dim, "heads": cfg.heads, "table_rows": rows, "emb_dim": 256,
                       "users_per_gpu": bpg, "layer_glue": args.glue, "lengths": "lognormal median 512 in [16, 4096]" + (", users dealt to ranks by length (longest first to the least loaded rank)" if args.balance else ""),
                       "ids": "Zipf(1.05)",
                       "parallelism": f"row-wise sharded table over {world} ({args.comm} lookup) + dp{world} dense",
                       "includes": "host batch build, H2D on a side stream, sparse Adagrad in backward"}}


WORKLOADS = {"gpt-oss-20b": bench_gpt_oss, "llama2-70b-lora": bench_llama70b_lora, "flux1": bench_flux, "hstu": bench_hstu}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("workload", choices=sorted(WORKLOADS))
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--scale", type=int, default=0, help="divide table rows / batch by this (smoke runs)")
    ap.add_argument("--global-batch", type=int, default=0)
    ap.add_argument("--micro-batch", type=int, default=0)
    ap.add_argument("--comm", default="fused", choices=["fused", "nccl"])
    ap.add_argument("--balance", type=int, default=1, help="hstu: deal each step's users to the ranks by length (0 = every rank draws its own)")
    ap.add_argument("--glue", default="fused", choices=["fused", "eager"], help="HSTU layer glue: one kernel or torch operators")
    ap.add_argument("--precision", default="bf16", choices=["bf16", "mxfp8", "fp8"],
                    help="flux1 / gpt-oss-20b: linear precision; llama2-70b-lora: mxfp8 or fp8 = frozen base on per-tensor FP8; "
                         "hstu: fp8 = e4m3 attention forward")
    args = ap.parse_args(argv)
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    dev = torch.device("cuda", torch.cuda.current_device())
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    from ..ops import _lib
    l0 = _lib.launch_count()
    out = WORKLOADS[args.workload](args, rank, world, dev)
    torch.cuda.synchronize()
    _lib.check_status(args.workload)
    out.update({"n_gpus": world, "steps": args.steps, "warmup": args.warmup, "higher_is_better": True, "dtype": "bf16",
                "data": "synthetic, random-init weights", "gpu_launches_total": _lib.launch_count() - l0,
                "reduced": bool(args.layers or args.scale), "mem_gb": round(torch.cuda.max_memory_allocated() / 2**30, 1)})
    out["value"], out["ms_per_step"] = round(out["value"], 1), round(out["ms_per_step"], 2)
    if rank == 0:
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
