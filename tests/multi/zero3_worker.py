"""Worker: the sharded-parameter (ZeRO-3) engine against the replicated-parameter engine on identical
models and data.  gloo ranks on CPU, or NCCL / NVLS transports on GPUs.
  argv: backend [comm] [precision]"""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from mlperf_training_b200.models.gpt import GPTConfig  # noqa: E402
from mlperf_training_b200.parallel.engine import OptimConfig  # noqa: E402
from mlperf_training_b200.trainer.pretrain import PretrainTrainer, TrainConfig, synthetic_tokens  # noqa: E402


def main():
    backend = sys.argv[1]
    comm = sys.argv[2] if len(sys.argv) > 2 else "nccl"
    precision = sys.argv[3] if len(sys.argv) > 3 else "bf16"
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    gpu = backend == "nccl"
    if gpu:
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
        dev = torch.device("cuda", torch.cuda.current_device())
        dist.init_process_group("nccl", device_id=dev)
    else:
        dev = torch.device("cpu")
        dist.init_process_group("gloo")
    if gpu:
        cfg = GPTConfig(n_layers=4, hidden=512, n_heads=4, n_kv_heads=2, head_dim=128, ffn_hidden=1024, vocab_size=2048,
                        seq_len=256, precision=precision)
    else:
        cfg = GPTConfig(n_layers=4, hidden=64, n_heads=4, n_kv_heads=2, head_dim=16, ffn_hidden=128, vocab_size=128,
                        seq_len=32, dtype="fp32")
    opt = OptimConfig(lr=2e-3, clip_grad=1.0)
    t1 = PretrainTrainer(cfg, opt, TrainConfig(micro_batch=1, local_batch=2, warmup_steps=1, seed=3, comm="nccl"), dev)
    t3 = PretrainTrainer(cfg, opt, TrainConfig(micro_batch=1, local_batch=2, warmup_steps=1, seed=3, comm=comm, zero_stage=3), dev)
    e3 = t3.engine
    sharded = [b for b in e3.buckets if b.zero3]
    ok = len(sharded) == cfg.n_layers and all(b.param_buf.numel() * world == b.numel for b in sharded)
    data = synthetic_tokens(4, 2, cfg.seq_len, cfg.vocab_size, seed=1, rank=rank, pin=gpu)
    l1, l3 = [], []
    for s in range(4):
        l1.append(t1.train_step(data[s]))
        l3.append(t3.train_step(data[s]))
    ev1 = float(t1.eval_loss(data[0].to(dev)))
    ev3 = float(t3.eval_loss(data[0].to(dev)))
    if gpu:
        torch.cuda.synchronize()
        from mlperf_training_b200.ops import _lib
        _lib.check_status("zero3 worker")
    tol = 3e-2 if gpu else 2e-5
    ok &= all(abs(a - b) < tol for a, b in zip(l1, l3)) and abs(ev1 - ev3) < tol
    # the shards, gathered, equal the replicated engine's parameter buffers
    by_key = {b.key: b for b in t1.engine.buckets}
    worst = 0.0
    for b in sharded:
        full = e3.gather_full(b)
        mats = torch.cat([p.detach().reshape(-1) for n, p in t1.model.named_parameters()
                          if n.startswith(f"blocks.{b.block_idx}.") and p.dim() >= 2 and p.requires_grad])
        # same parameter order inside the bucket: weight-decayed matrices in registration order
        ref = torch.cat([p.detach().reshape(-1) for (n, p) in [(n, dict(t1.model.named_parameters())[n]) for n, _ in b.params]])
        worst = max(worst, (full[:ref.numel()].float() - ref.float()).abs().max().item())
        del mats
    ok &= worst < (3e-2 if gpu else 2e-5)
    flag = torch.tensor([1.0 if ok else 0.0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        print(f"zero1 {l1} eval {ev1:.5f}\nzero3 {l3} eval {ev3:.5f}\nworst param diff {worst:.3g} nvls={e3.nvls} "
              f"state MB z1 {t1.engine.state_bytes() / 2**20:.1f} z3 {e3.state_bytes() / 2**20:.1f}", flush=True)
    print(f"RESULT rank {rank} ok={bool(flag.item())}", flush=True)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if flag.item() == 1.0 else 1)


if __name__ == "__main__":
    main()
