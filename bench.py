"""Headline benchmark: Llama-3.1-8B-architecture pre-training step, train tokens/s.

    python bench.py --gpus N --steps K --warmup W            (N = 1)
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W

Config (the Llama-3.1-8B row of the benchmark definition): 32 layers, hidden 4096, 32 q / 8 kv
heads of 128, SwiGLU 14336, vocab 128256, seq 8192, 4 sequences per GPU per step (global batch
32 at 8 GPUs, weak scaling), synthetic uniform token ids, random-init weights, bf16 compute,
fp32 gradient accumulation and Adam moments, ZeRO-sharded optimizer over the data-parallel ranks.

Two measurements per run, both K steps after W warm-up steps:
  * ``value``: device-timed (CUDA events, max over ranks) with the step's tokens already on the
    device and no host read inside the loop;
  * ``e2e``: wall-clock around ``PretrainTrainer.train_step`` - the public call - including the
    pinned-host -> device copy of each step's tokens and the device -> host read of its loss.
Inputs (token ids) are tiny; the working set per step (16 GB of weights, 32 GB of gradients)
is far larger than L2, which is what keeps timed iterations cold.

``--impl reference`` would run the unmodified reference; it cannot be installed here (the tree has
no setup.py / pyproject.toml and its stack is ROCm-only), so that arm prints an ``unavailable``
line.  ``--impl baseline`` runs the same step with stock PyTorch modules (cuBLAS / cuBLASLt, SDPA,
fused torch AdamW, DDP or FSDP2) for comparison on the same box.

Because the reference publishes no throughput number and cannot run here, the package's own arm also
times the stock arms in the same invocation (same N, same shapes, a few steps each, after its own
model has been freed) and reports ``stock``: the library stack at bf16 and at the same MXFP8
precision (``torch._scaled_mm`` block-scaled GEMMs), with ``ratio`` = own value / stock value.
``vs_baseline`` is the ratio against the equal-precision stock arm.  ``--stock none`` skips this.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference", "baseline"])
    ap.add_argument("--model", default="llama3.1-8b")
    ap.add_argument("--layers", type=int, default=0, help="override depth (debug only; marks the run reduced)")
    ap.add_argument("--seq-len", type=int, default=0)
    ap.add_argument("--local-batch", type=int, default=4)
    ap.add_argument("--micro-batch", type=int, default=1)
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-overlap", action="store_true",
                    help="do not overlap the gradient reduce-scatter with the last micro-batch's backward")
    ap.add_argument("--comm", default="fused", choices=["fused", "nccl"],
                    help="data-parallel step: in-kernel NVLink peer loads/stores, or NCCL collectives")
    ap.add_argument("--precision", default="mxfp8", choices=["mxfp8", "bf16"],
                    help="GEMM precision of the linears (attention, norms, residual stream stay bf16)")
    ap.add_argument("--zero-stage", type=int, default=1, choices=[1, 3],
                    help="1: optimizer state sharded, parameters replicated; 3: block matrices sharded and gathered per block")
    ap.add_argument("--check", action="store_true",
                    help="instead of timing: 3 steps with the in-kernel (fused / NVLS) data-parallel step and 3 with the "
                         "NCCL step on the same data, compare losses and gradient norms, print RESULT ok=...")
    ap.add_argument("--stock", default="mxfp8,bf16",
                    help="stock-PyTorch arms timed after the package's own arm: comma list of mxfp8, bf16, or none")
    ap.add_argument("--stock-steps", type=int, default=5, help="timed steps of each stock arm (3 warm-up steps)")
    ap.add_argument("--stock-parallel", default="fsdp", choices=["fsdp", "ddp"],
                    help="data parallelism of the stock arms at N > 1 (FSDP2 fully_shard, or DDP)")
    return ap.parse_args()


def time_stock_arm(args, cfg, opt, tc, device, world, rank, precision: str) -> dict:
    """Device-timed tokens/s of the stock-PyTorch trainer at ``precision`` (same shapes, max over ranks)."""
    import copy

    import torch
    import torch.distributed as dist

    from baseline.torch_gpt import BaselineTrainer
    from mlperf_training_b200.trainer.pretrain import synthetic_tokens

    scfg = copy.copy(cfg)
    scfg.precision = precision
    trainer = BaselineTrainer(scfg, opt, tc, device, parallel=args.stock_parallel)
    K_, W_ = max(args.stock_steps, 1), 3
    toks = synthetic_tokens(W_ + K_, args.local_batch, cfg.seq_len, cfg.vocab_size, seed=1, rank=rank).to(device)
    for i in range(W_):
        trainer.train_step_device(toks[i])
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for i in range(K_):
        last = trainer.train_step_device(toks[W_ + i])
    ev1.record()
    torch.cuda.synchronize()
    t = torch.tensor([ev0.elapsed_time(ev1)], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t[0]) / K_
    loss = float(last)
    del trainer, toks
    torch.cuda.empty_cache()
    return {"value": round(args.local_batch * cfg.seq_len * world / (ms / 1e3), 1), "ms_per_step": round(ms, 2),
            "steps": K_, "warmup": W_, "loss_last": round(loss, 4),
            "stack": ("torch._scaled_mm MXFP8 (cuBLASLt block-scaled) linears" if precision == "mxfp8" else "cuBLAS bf16 linears")
                     + ", SDPA, F.rms_norm, F.cross_entropy, torch AdamW(fused), "
                     + (("FSDP2 fully_shard" if args.stock_parallel == "fsdp" else "DDP") if world > 1 else "single GPU")}


def check_comm_paths(args, cfg, opt, device, world, rank) -> int:
    """Correctness of the in-kernel data-parallel step at this N: the same model, seed and batches through
    ``comm=fused`` (peer loads / stores or NVLS multimem) and through ``comm=nccl``; losses and global gradient
    norms of 3 steps must agree."""
    import gc

    import torch
    import torch.distributed as dist

    from mlperf_training_b200.ops import _lib
    from mlperf_training_b200.trainer.pretrain import PretrainTrainer, TrainConfig, synthetic_tokens

    host = synthetic_tokens(3, args.local_batch, cfg.seq_len, cfg.vocab_size, seed=0, rank=rank)
    seen = {}
    for comm in ("fused", "nccl"):
        tc = TrainConfig(micro_batch=args.micro_batch, local_batch=args.local_batch, warmup_steps=64, seed=0, comm=comm,
                         zero_stage=args.zero_stage)
        tr = PretrainTrainer(cfg, opt, tc, device)
        losses, norms = [], []
        for i in range(3):
            losses.append(tr.train_step(host[i]))
            norms.append(tr.engine.grad_norm())
        torch.cuda.synchronize()
        _lib.check_status(f"check {comm}")
        seen[comm] = (losses, norms)
        del tr
        gc.collect()
        torch.cuda.empty_cache()
    ok = all(abs(a - b) <= 2e-2 * max(abs(b), 1.0) for a, b in zip(seen["fused"][0], seen["nccl"][0]))
    ok &= all(abs(a - b) <= 3e-2 * max(abs(b), 1e-3) for a, b in zip(seen["fused"][1], seen["nccl"][1]))
    flag = torch.tensor([1.0 if ok else 0.0], device=device)
    if world > 1:
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        print(json.dumps({"check": "comm fused vs nccl", "n_gpus": world, "zero_stage": args.zero_stage, "ok": bool(flag.item()),
                          "loss_fused": seen["fused"][0], "loss_nccl": seen["nccl"][0],
                          "grad_norm_fused": seen["fused"][1], "grad_norm_nccl": seen["nccl"][1]}))
        print(f"RESULT ok={bool(flag.item())}", flush=True)
    if world > 1:
        dist.destroy_process_group()
    return 0 if flag.item() == 1.0 else 1


class ClockSampler:
    """Samples SM clock / throttle reasons of this process's GPU with nvidia-smi while running."""

    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, uuid: str | None):
        self.uuid = uuid
        self.proc = None
        self.lines: list[str] = []

    def start(self):
        cmd = ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "200"]
        if self.uuid:
            cmd += ["-i", self.uuid]
        try:
            self.proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        threading.Thread(target=self._read, daemon=True).start()

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons, power = [], [], set(), []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0])); mx.append(float(parts[1])); power.append(float(parts[2]))
            except ValueError:
                continue
            for nm, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(nm)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons)}


def main() -> int:
    args = parse()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "reference is not installable (no setup.py/pyproject.toml; ROCm/HIP-only Primus+Megatron stack pinned by Dockerfiles)"}))
        return 0

    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        print(json.dumps({"error": "no CUDA device"}))
        return 1
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    if args.gpus != world and rank == 0:
        print(f"warning: --gpus {args.gpus} but WORLD_SIZE {world}", file=sys.stderr)

    from mlperf_training_b200.models.gpt import PRESETS
    from mlperf_training_b200.ops import _lib
    from mlperf_training_b200.parallel.engine import OptimConfig
    from mlperf_training_b200.trainer.pretrain import PretrainTrainer, TrainConfig, synthetic_tokens

    cfg = PRESETS[args.model]()
    reduced = False
    if args.layers:
        cfg.n_layers = args.layers; reduced = True
    if args.seq_len:
        cfg.seq_len = args.seq_len; reduced = True
    cfg.precision = args.precision
    opt = OptimConfig(lr=8e-4, beta1=0.9, beta2=0.95, eps=1e-5, weight_decay=0.1, clip_grad=1.0)
    tc = TrainConfig(micro_batch=args.micro_batch, local_batch=args.local_batch, warmup_steps=64, seed=0, comm=args.comm,
                     zero_stage=args.zero_stage)

    if args.check:
        return check_comm_paths(args, cfg, opt, device, world, rank)
    if args.impl == "baseline":
        from baseline.torch_gpt import BaselineTrainer
        cfg.precision = args.precision
        trainer = BaselineTrainer(cfg, opt, tc, device, parallel=args.stock_parallel)
    else:
        trainer = PretrainTrainer(cfg, opt, tc, device)
        trainer.overlap_grad_reduce = not args.no_overlap

    nvls = False
    if args.impl == "b200":
        eng = trainer.engine
        nvls = bool(getattr(eng, "nvls", False)) or any(eng._nvls(getattr(b, "symm_grad", None)) for b in eng.buckets)
        state_gb = round(eng.state_bytes() / 2**30, 2)
        del eng                          # the stock arms below need this arm's memory back: hold no second reference
    K_, W_ = args.steps, args.warmup
    tokens_per_step = args.local_batch * cfg.seq_len * world
    host = synthetic_tokens(W_ + 2 * K_, args.local_batch, cfg.seq_len, cfg.vocab_size, seed=0, rank=rank)
    dev_tokens = host[W_:W_ + K_].to(device)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # warm-up through the public call
    losses = []
    for i in range(W_):
        losses.append(trainer.train_step(host[i]))
    barrier()

    uuid = None
    try:
        uuid = "GPU-" + str(torch.cuda.get_device_properties(device).uuid)
    except Exception:
        uuid = None
    sampler = ClockSampler(uuid)
    sampler.start()

    # (1) device-timed: tokens resident, no host read inside the loop
    launches0 = _lib.launch_count() if args.impl == "b200" else 0
    barrier()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    last = None
    for i in range(K_):
        last = trainer.train_step_device(dev_tokens[i])
    ev1.record()
    barrier()
    dev_ms = ev0.elapsed_time(ev1)
    launches = (_lib.launch_count() - launches0) if args.impl == "b200" else 0
    clocks = sampler.stop()

    # (2) end to end through the public API: H2D of the tokens and D2H of the loss every step
    e2e = None
    if not args.no_e2e:
        barrier()
        t0 = time.perf_counter()
        for i in range(K_):
            losses.append(trainer.train_step(host[W_ + K_ + i]))
        barrier()
        e2e_s = time.perf_counter() - t0
    t = torch.tensor([dev_ms, e2e_s if not args.no_e2e else 0.0], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dev_ms, e2e_s = float(t[0]), float(t[1])

    if args.impl == "b200":
        _lib.check_status("bench")
    stock = {}
    if args.impl == "b200" and args.stock.lower() not in ("", "none"):
        # free this arm's model, optimizer state and peer-mapped buffers before the stock models are built
        del trainer, dev_tokens
        import gc
        gc.collect()
        torch.cuda.synchronize()
        torch.cuda.empty_cache()
        if rank == 0:
            print(f"[bench] own arm freed: {torch.cuda.memory_allocated(device) / 2**30:.1f} GiB still allocated", file=sys.stderr, flush=True)
        for prec in [s.strip() for s in args.stock.split(",") if s.strip()]:
            try:
                stock[prec] = time_stock_arm(args, cfg, opt, tc, device, world, rank, prec)
            except Exception as e:                       # a stock arm that cannot run here must not lose the line
                stock[prec] = {"error": f"{type(e).__name__}: {str(e)[:160]}"}
                gc.collect()
                torch.cuda.empty_cache()
    if rank == 0:
        ms_per_step = dev_ms / K_
        value = tokens_per_step / (ms_per_step / 1e3)
        out = {
            "metric": "train tokens/s", "value": round(value, 1), "unit": "tokens/s", "n_gpus": world, "steps": K_,
            "warmup": W_, "ms_per_step": round(ms_per_step, 2), "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None,
            "dtype": ("mxfp8 linears (e4m3 + e8m0/32 block scales, fp32 accumulate), bf16 attention/norms/residual"
                      if cfg.precision == "mxfp8" else "bf16"), "data": "synthetic uniform token ids (seed 0), random-init weights",
            "impl": args.impl,
            "config": {"model": cfg.name, "layers": cfg.n_layers, "global_batch": args.local_batch * world,
                       "seq_len": cfg.seq_len, "micro_batch": args.micro_batch,
                       "parallelism": f"dp{world} (ZeRO-{args.zero_stage}, {args.comm if world > 1 else 'single GPU'} step"
                                      + (", NVLS multimem" if nvls else "")
                                      + (", reduce-scatter overlapped with backward)" if (world > 1 and not args.no_overlap) else ")"),
                       "l2": "no flush: per-step working set (>48 GB of weights and gradients) exceeds L2",
                       "reduced": reduced},
            "clocks": clocks, "gpu_launches": int(launches), "engine_state_gb_per_gpu": state_gb if args.impl == "b200" else None,
            "model_tflops_per_gpu": round(cfg.flops_per_token() * tokens_per_step / world / (ms_per_step / 1e3) / 1e12, 1),
            "loss_first": round(losses[0], 4) if losses else None, "loss_last": round(losses[-1], 4) if losses else None,
        }
        for prec, rec in stock.items():
            if "value" in rec:
                rec["ratio"] = round(value / rec["value"], 3)
        if stock:
            out["stock"] = stock
            same = stock.get(cfg.precision, {})
            if "ratio" in same:
                out["vs_baseline"] = same["ratio"]
                out["vs_baseline_of"] = f"stock PyTorch arm at {cfg.precision}, same box, same invocation"
        if not args.no_e2e:
            bi = int(host[0].numel() * host[0].element_size())
            out["e2e"] = {"value": round(tokens_per_step * K_ / e2e_s, 1), "unit": "tokens/s",
                          "h2d_bytes_per_step": bi, "d2h_bytes_per_step": 4, "ms_per_step": round(e2e_s * 1e3 / K_, 2)}
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
