"""Worker: interleaved pipeline (v chunks per rank) follows the unsplit model's loss curve."""
import os
import sys

import torch
import torch.distributed as dist
import torch.nn as nn

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from mlperf_training_b200.models.gpt import GPT, GPTConfig  # noqa: E402
from mlperf_training_b200.parallel.engine import OptimConfig, ZeroEngine  # noqa: E402
from mlperf_training_b200.parallel.pipeline import GPTStage, InterleavedRunner  # noqa: E402


def main():
    v, M = int(sys.argv[1]), int(sys.argv[2])
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo")
    solo = [dist.new_group([r]) for r in range(world)][rank]
    cfg = GPTConfig(n_layers=world * v + 1, hidden=32, n_heads=2, n_kv_heads=1, head_dim=16, ffn_hidden=64, vocab_size=128,
                    seq_len=16, dtype="fp32")
    full = GPT(cfg, seed=5)
    chunks = [GPTStage(cfg, c * world + rank, world * v) for c in range(v)]
    for ch in chunks:
        ch.load_from_full(full)
    holder = nn.ModuleList(chunks)
    opt = OptimConfig(lr=2e-3, weight_decay=0.0, clip_grad=0.0)
    e_full = ZeroEngine(full, opt, group=solo)
    e_pp = ZeroEngine(holder, opt, group=solo, bucket_of=lambda n: "c" + n.split(".")[0])
    runner = InterleavedRunner(chunks, rank, world, (rank - 1) % world, (rank + 1) % world)
    ok = True
    for step in range(3):
        g = torch.Generator().manual_seed(step)
        tok = torch.randint(0, cfg.vocab_size, (M, 2, cfg.seq_len + 1), generator=g)
        mbs = [(tok[i, :, :-1].contiguous(), tok[i, :, 1:].contiguous()) for i in range(M)]
        ref = 0.0
        for x, y in mbs:
            l = full(x, y)
            l.backward()
            ref += l.item()
        e_full.step(grad_scale=1.0 / M)
        tot = runner.run(mbs)
        e_pp.step(grad_scale=1.0 / M)
        got = torch.tensor([tot.item() if tot is not None else 0.0])
        dist.all_reduce(got)
        ok &= abs(got.item() - ref) < 2e-4 * max(1.0, abs(ref))
        if rank == 0:
            print(f"step {step} full {ref / M:.5f} vpp {got.item() / M:.5f}", flush=True)
    print(f"RESULT rank {rank} ok={ok}", flush=True)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
