"""Worker (gloo, 2 ranks): an expert-parallel MoE model saves a ``torch_dist`` checkpoint in which every rank wrote its
own experts as a block of the stacked expert dimension; it loads into the same expert sharding and into a model that
holds every expert.  argv: checkpoint directory"""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from mlperf_training_b200.checkpoint import megatron as M  # noqa: E402
from mlperf_training_b200.models.gpt import GPT, tiny_moe  # noqa: E402


def main():
    root = sys.argv[1]
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo")
    cfg = tiny_moe(n_layers=2, hidden=64, n_heads=4, n_kv_heads=2, head_dim=16, ffn_hidden=96, moe_ffn_hidden=48, vocab_size=128,
                   seq_len=32, n_experts=4, top_k=2)
    src = GPT(cfg, device="cpu", seed=11 + rank, ep_group=dist.group.WORLD)      # experts differ per rank
    with torch.no_grad():
        for p in src.parameters():
            if getattr(p, "expert_shard", None) is None:
                dist.broadcast(p, 0)
    M.save_torch_dist(src, root, iteration=1)
    import torch.distributed.checkpoint as dcp
    meta = dcp.FileSystemReader(os.path.join(root, "iter_0000001")).read_metadata().state_dict_metadata
    key = "model.decoder.layers.0.mlp.experts.linear_fc1.weight"
    ok = len(meta[key].chunks) == world and tuple(meta[key].size) == (cfg.n_experts, 2 * cfg.moe_ffn_hidden, cfg.hidden)
    same = GPT(cfg, device="cpu", seed=3, ep_group=dist.group.WORLD)
    M.load_torch_dist(same, root)
    for (n, a), (_, b) in zip(src.named_parameters(), same.named_parameters()):
        ok &= torch.equal(a, b)
    full = GPT(cfg, device="cpu", seed=5)                                       # every expert on every rank
    M.load_torch_dist(full, root)
    want = M.to_megatron_state(src)
    got = M.to_megatron_state(full)
    for k in want:
        ok &= torch.equal(want[k], got[k])
    print(f"RESULT rank {rank} ok={bool(ok)}", flush=True)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
