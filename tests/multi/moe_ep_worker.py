"""Worker (GPUs, NCCL): a small MoE GPT with expert parallelism over the ranks follows the same
loss curve whether tokens move by all-to-all collectives or by the peer-memory kernels."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from mlperf_training_b200.models.gpt import GPT, tiny_moe  # noqa: E402
from mlperf_training_b200.ops import _lib  # noqa: E402
from mlperf_training_b200.parallel.engine import OptimConfig, ZeroEngine  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dev = torch.device("cuda", torch.cuda.current_device())
    dist.init_process_group("nccl")
    curves = {}
    for comm in ("nccl", "fused"):
        cfg = tiny_moe(n_layers=2, hidden=256, n_heads=4, n_kv_heads=2, head_dim=64, moe_ffn_hidden=256, n_experts=4 * world,
                       top_k=2, vocab_size=1024, seq_len=256, dtype="bf16", ep_comm=comm)
        torch.manual_seed(0)
        model = GPT(cfg, dev, seed=0, ep_group=dist.group.WORLD)
        eng = ZeroEngine(model, OptimConfig(lr=1e-3, weight_decay=0.0, clip_grad=1.0))
        losses = []
        for step in range(4):
            g = torch.Generator().manual_seed(100 * step + rank)
            tok = torch.randint(0, cfg.vocab_size, (2, cfg.seq_len + 1), generator=g).to(dev)
            loss = model(tok[:, :-1], tok[:, 1:])
            loss.backward()
            eng.step()
            losses.append(float(loss))
        curves[comm] = losses
    torch.cuda.synchronize()
    _lib.check_status("moe ep")
    ok = all(abs(a - b) < 3e-2 * max(1.0, abs(a)) for a, b in zip(curves["nccl"], curves["fused"]))
    ok &= curves["fused"][-1] < curves["fused"][0]
    if rank == 0:
        print("nccl ", [round(x, 4) for x in curves["nccl"]], flush=True)
        print("fused", [round(x, 4) for x in curves["fused"]], flush=True)
    print(f"RESULT rank {rank} ok={ok}", flush=True)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
