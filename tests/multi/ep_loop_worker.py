"""Worker: the run loop with the experts of an MoE model spread over the ranks (gloo): every rank holds
its share of the experts, and an exit after a checkpoint resumes exactly (expert shards are saved per rank).
  argv: <out_dir>"""
import io
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from mlperf_training_b200.trainer.loop import run  # noqa: E402

MOE = dict(preset="tiny-moe", n_layers=2, hidden=64, n_heads=4, n_kv_heads=2, head_dim=16, moe_ffn_hidden=64, n_experts=4, top_k=2,
           vocab_size=128, seq_len=32, window=16)


def main():
    root = sys.argv[1]
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo")
    base = dict(model=MOE, global_batch=4, micro_batch=1, train_iters=4, lr=3e-3, lr_warmup_iters=1, warmup_train_steps=1)
    rep = run(dict(base, expert_parallel=1), device="cpu", stream=io.StringIO())
    ep = run(dict(base, expert_parallel=world, moe_dispatch="nccl"), device="cpu", stream=io.StringIO())
    n_local = sum(p.numel() for n, p in ep["trainer"].model.named_parameters())
    n_full = sum(p.numel() for n, p in rep["trainer"].model.named_parameters())
    ok = n_local < n_full                                           # the experts really are spread
    # (expert weights are drawn per rank, so the two runs start from different experts: the model-level
    # parity of the sharded layer against the unsharded one is tests/test_dist_moe_parity.py)
    ok &= all(l == l for l in ep["losses"]) and abs(ep["losses"][0] - rep["losses"][0]) < 0.1
    if rank == 0:
        print("replicated", [round(x, 5) for x in rep["losses"]], "ep", [round(x, 5) for x in ep["losses"]], flush=True)
    exp = dict(base, expert_parallel=world, moe_dispatch="nccl", checkpoint_dir=os.path.join(root, "ck"), die_at_step=2)
    try:
        run(dict(exp), device="cpu", stream=io.StringIO())
        ok = False
    except SystemExit as e:
        ok &= int(e.code) == 42
    out = run(dict(exp, die_at_step=0), device="cpu", stream=io.StringIO())
    ok &= out["steps"] == 2 and max(abs(a - b) for a, b in zip(out["losses"], ep["losses"][2:])) < 1e-6
    print(f"RESULT rank {rank} ok={ok}", flush=True)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
