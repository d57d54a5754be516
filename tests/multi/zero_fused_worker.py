"""Worker of test_gpu_multi.py: the peer-memory ZeRO step against the NCCL step on identical
models and data (run under torchrun, one process per GPU)."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from mlperf_training_b200.models.gpt import GPTConfig  # noqa: E402
from mlperf_training_b200.ops import _lib  # noqa: E402
from mlperf_training_b200.parallel.engine import OptimConfig  # noqa: E402
from mlperf_training_b200.trainer.pretrain import PretrainTrainer, TrainConfig, synthetic_tokens  # noqa: E402


def main():
    rank = int(os.environ["RANK"])
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    cfg = GPTConfig(n_layers=2, hidden=512, n_heads=4, n_kv_heads=2, head_dim=128, ffn_hidden=1024, vocab_size=2048,
                    seq_len=256)
    opt = OptimConfig(lr=2e-3, clip_grad=1.0)
    trainers = {c: PretrainTrainer(cfg, opt, TrainConfig(micro_batch=1, local_batch=2, warmup_steps=1, seed=3, comm=c), dev)
                for c in ("nccl", "fused")}
    data = synthetic_tokens(4, 2, cfg.seq_len, cfg.vocab_size, seed=1, rank=rank)
    losses = {c: [] for c in trainers}
    for s in range(4):
        for c, t in trainers.items():
            losses[c].append(t.train_step(data[s]))
    torch.cuda.synchronize()
    _lib.check_status("fused zero")
    worst = 0.0
    for (n, p), (_, q) in zip(trainers["nccl"].model.named_parameters(), trainers["fused"].model.named_parameters()):
        worst = max(worst, (p.float() - q.float()).abs().max().item())
    ok = worst < 2e-2 and all(abs(a - b) < 2e-2 for a, b in zip(losses["nccl"], losses["fused"]))
    # every rank must hold identical parameters after the in-kernel all-gather
    flat = torch.cat([p.detach().float().reshape(-1) for p in trainers["fused"].model.parameters()])
    ref = flat.clone()
    dist.broadcast(ref, 0)
    same = bool((flat == ref).all())
    flag = torch.tensor([1.0 if (ok and same) else 0.0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        print(f"RESULT ok={bool(flag.item())} worst_param_diff={worst:.4g} losses_nccl={losses['nccl']} losses_fused={losses['fused']}")
    dist.destroy_process_group()
    return 0 if flag.item() == 1.0 else 1


if __name__ == "__main__":
    sys.exit(main())
