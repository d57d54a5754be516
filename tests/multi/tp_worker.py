"""Worker: a tensor+sequence-parallel GPT (optionally with LoRA) must follow the same loss curve as
the unsharded model.  argv: backend [comm] [lora] [fp8]: with ``fp8`` the frozen linears of the fused path run
on per-tensor 8-bit operands and the comparison allows for their rounding."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from mlperf_training_b200.models.gpt import GPT, GPTConfig, shard_of  # noqa: E402
from mlperf_training_b200.models.lora import freeze_base  # noqa: E402
from mlperf_training_b200.parallel.engine import OptimConfig, ZeroEngine  # noqa: E402
from mlperf_training_b200.parallel.tensor import TPContext  # noqa: E402


def main():
    backend = sys.argv[1]
    comm = sys.argv[2] if len(sys.argv) > 2 else "nccl"
    lora = len(sys.argv) > 3 and sys.argv[3] == "lora"
    fp8 = len(sys.argv) > 4 and sys.argv[4] == "fp8"
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    gpu = backend == "nccl"
    if gpu:
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    device = torch.device("cuda", torch.cuda.current_device()) if gpu else torch.device("cpu")
    dist.init_process_group(backend)
    solo = [dist.new_group([r]) for r in range(world)][rank]          # data-parallel group of one
    heads, kv = max(4, world), max(2, world)              # every rank needs at least one query and one kv head
    hd = 64 if gpu else 16
    cfg = GPTConfig(n_layers=2, hidden=heads * hd, n_heads=heads, n_kv_heads=kv, head_dim=hd,
                    ffn_hidden=(512 if gpu else 128) * max(world // 2, 1), vocab_size=512, seq_len=256 * world if gpu else 32,     # 256 rows per rank: the CTA-pair fused kernels
                    dtype="bf16" if gpu else "fp32", lora_rank=8 if lora else 0, lora_dropout=0.0)
    torch.manual_seed(1)
    full = GPT(cfg, device=device, seed=3)
    tp = TPContext(dist.group.WORLD, comm=comm, device=device, precision="fp8" if fp8 else "bf16")
    torch.manual_seed(1)
    model = GPT(cfg, device=device, seed=3, tp=tp)
    if lora:
        with torch.no_grad():
            for bf, bt in zip(full.blocks, model.blocks):
                bf.lora_qkv.b.normal_(0, 0.05)
                bf.lora_proj.b.normal_(0, 0.05)
                dist.broadcast(bf.lora_qkv.b, 0), dist.broadcast(bf.lora_proj.b, 0)
                dist.broadcast(bf.lora_qkv.a, 0), dist.broadcast(bf.lora_proj.a, 0)
                bt.lora_qkv.a.copy_(bf.lora_qkv.a)
                bt.lora_qkv.b.copy_(shard_of(bf.lora_qkv.b, "qkv", world, rank, cfg))
                bt.lora_proj.a.copy_(shard_of(bf.lora_proj.a, "cols", world, rank, cfg))
                bt.lora_proj.b.copy_(bf.lora_proj.b)
        freeze_base(full), freeze_base(model)
    opt = OptimConfig(lr=2e-3, weight_decay=0.0, clip_grad=1.0)
    e_full = ZeroEngine(full, opt, group=solo)
    e_tp = ZeroEngine(model, opt, group=solo, tp_group=dist.group.WORLD)
    ok = True
    B, S = (1, cfg.seq_len) if gpu else (2, cfg.seq_len)
    for step in range(5):
        g = torch.Generator().manual_seed(step)
        tok = torch.randint(0, cfg.vocab_size, (B, S + 1), generator=g).to(device)
        x, y = tok[:, :-1].contiguous(), tok[:, 1:].contiguous()
        l_full = full(x, y)
        l_full.backward()
        e_full.step()
        l_tp = model(x, y)
        l_tp.backward()
        e_tp.step()
        tot = l_tp.detach().float().clone()
        dist.all_reduce(tot)
        n_full, n_tp = e_full.grad_norm(), e_tp.grad_norm()
        tol = (8e-2 if fp8 else 3e-2) if gpu else 2e-4
        good = abs(tot.item() - l_full.item()) < tol * max(1.0, abs(l_full.item())) and abs(n_full - n_tp) < 10 * tol * max(1.0, n_full)
        ok &= good
        if rank == 0:
            print(f"step {step} full {l_full.item():.5f} tp {tot.item():.5f} gnorm {n_full:.4f} {n_tp:.4f}", flush=True)
    if gpu:
        from mlperf_training_b200.ops import _lib
        torch.cuda.synchronize()
        _lib.check_status("tp worker")
    print(f"RESULT rank {rank} ok={ok}", flush=True)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
