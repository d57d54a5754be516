"""Worker (gloo, world 4): hybrid sharding (shard over 2 ranks x 2 replicas) follows plain
data-parallel sharding over all 4 ranks; replicas keep identical weights."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from mlperf_training_b200.models.gpt import GPT, GPTConfig  # noqa: E402
from mlperf_training_b200.parallel.engine import OptimConfig, ZeroEngine  # noqa: E402
from mlperf_training_b200.parallel.mesh import Mesh, MeshSpec  # noqa: E402


def main():
    rank = int(os.environ["RANK"])
    dist.init_process_group("gloo")
    mesh = Mesh(MeshSpec(dp_replicate=2))
    cfg = GPTConfig(n_layers=2, hidden=32, n_heads=2, n_kv_heads=1, head_dim=16, ffn_hidden=64, vocab_size=128, seq_len=16,
                    dtype="fp32")
    a, b = GPT(cfg, seed=1), GPT(cfg, seed=1)
    opt = OptimConfig(lr=3e-3, weight_decay=0.0, clip_grad=1.0)
    ea = ZeroEngine(a, opt)
    eb = ZeroEngine(b, opt, group=mesh.group("dp_shard"), replicate_group=mesh.group("dp_replicate"))
    ok = True
    for step in range(3):
        g = torch.Generator().manual_seed(10 * step + rank)
        tok = torch.randint(0, cfg.vocab_size, (2, cfg.seq_len + 1), generator=g)
        la = a(tok[:, :-1], tok[:, 1:]); la.backward(); ea.step()
        lb = b(tok[:, :-1], tok[:, 1:]); lb.backward(); eb.step()
        ok &= abs(la.item() - lb.item()) < 1e-5
    for pa, pb in zip(a.parameters(), b.parameters()):
        ok &= bool(torch.allclose(pa, pb, atol=1e-5))
    ok &= ea.replica_checksum_spread() < 1e-6
    print(f"RESULT rank {rank} ok={ok}", flush=True)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
