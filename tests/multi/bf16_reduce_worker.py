"""Worker (gloo, 2 ranks): gradients reduced in bf16 on the wire (accumulated and applied in fp32) follow the fp32-wire
run closely; the reduced shard holds bf16-representable averages."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from mlperf_training_b200.models.gpt import GPTConfig  # noqa: E402
from mlperf_training_b200.parallel.engine import OptimConfig  # noqa: E402
from mlperf_training_b200.trainer.pretrain import PretrainTrainer, TrainConfig  # noqa: E402


def main():
    rank = int(os.environ["RANK"])
    dist.init_process_group("gloo")
    cfg = dict(n_layers=2, hidden=32, n_heads=4, n_kv_heads=2, head_dim=8, ffn_hidden=64, vocab_size=64, seq_len=32, dtype="fp32")
    tc = TrainConfig(micro_batch=1, local_batch=1, warmup_steps=0, seed=3)
    runs = {}
    for name, wire in (("fp32", None), ("bf16", torch.bfloat16)):
        opt = OptimConfig(lr=3e-3, weight_decay=0.01, clip_grad=1.0, reduce_dtype=wire)
        tr = PretrainTrainer(GPTConfig(**cfg), opt, tc, "cpu", group=dist.group.WORLD)
        losses = []
        for step in range(5):
            g = torch.Generator().manual_seed(100 + 10 * step + rank)
            losses.append(tr.train_step(torch.randint(0, 64, (1, 33), generator=g)))
        runs[name] = (losses, torch.cat([p.detach().reshape(-1) for p in tr.model.parameters()]))
    ok = max(abs(a - b) for a, b in zip(*[runs[k][0] for k in ("fp32", "bf16")])) < 2e-3
    ok &= not torch.equal(runs["fp32"][1], runs["bf16"][1])              # the wire rounding is real ...
    ok &= bool((runs["fp32"][1] - runs["bf16"][1]).abs().max() < 5e-3)    # ... and small
    # replicas stay identical under the rounded reduction
    mine = runs["bf16"][1].clone()
    other = mine.clone()
    dist.broadcast(other, src=0)
    ok &= torch.equal(mine, other)
    print(f"RESULT rank {rank} ok={bool(ok)}", flush=True)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
