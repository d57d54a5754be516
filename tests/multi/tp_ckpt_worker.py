"""Worker (gloo, 2 ranks): a tensor-parallel model saves a ``torch_dist`` checkpoint in which every rank wrote only its
slices; the same checkpoint then loads into (a) a model with the same sharding, (b) an unsharded model - the chunk
offsets recorded in the checkpoint carry the layout.  argv: checkpoint directory"""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from mlperf_training_b200.checkpoint import megatron as M  # noqa: E402
from mlperf_training_b200.models.gpt import GPT, GPTConfig  # noqa: E402
from mlperf_training_b200.parallel.tensor import TPContext  # noqa: E402


def main():
    root = sys.argv[1]
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo")
    cfg = GPTConfig(n_layers=2, hidden=64, n_heads=4, n_kv_heads=2, head_dim=16, ffn_hidden=96, vocab_size=128, seq_len=32,
                    dtype="fp32", lora_rank=4)
    tp = TPContext(dist.group.WORLD, comm="nccl", device="cpu")
    src = GPT(cfg, device="cpu", seed=11, tp=tp)
    with torch.no_grad():
        for p in src.parameters():
            p.add_(torch.randn_like(p) * 0.01)                    # LoRA B starts at zero: make every tensor distinctive
        for p in src.parameters():
            if getattr(p, "tensor_parallel", None) is None:
                dist.broadcast(p, 0)                              # replicated parameters are equal on every rank
    M.save_torch_dist(src, root, iteration=3)
    ok = True
    files = sorted(f for f in os.listdir(os.path.join(root, "iter_0000003")) if f.endswith(".distcp"))
    ok &= len(files) == world                                     # every rank wrote its own slices
    import torch.distributed.checkpoint as dcp
    meta = dcp.FileSystemReader(os.path.join(root, "iter_0000003")).read_metadata().state_dict_metadata
    key = "model.decoder.layers.0.mlp.linear_fc1.weight"
    ok &= len(meta[key].chunks) == 2 * world and tuple(meta[key].size) == (2 * cfg.ffn_hidden, cfg.hidden)   # gate and up chunks
    ok &= len(meta["model.decoder.layers.0.self_attention.linear_qkv.weight"].chunks) == world
    # (a) same sharding
    same = GPT(cfg, device="cpu", seed=99, tp=tp)
    M.load_torch_dist(same, root)
    for (n, a), (_, b) in zip(src.named_parameters(), same.named_parameters()):
        ok &= torch.equal(a, b)
    # (b) unsharded model: its full tensors equal the gathered slices
    full = GPT(cfg, device="cpu", seed=5)
    M.load_torch_dist(full, root)
    want = M.to_megatron_state(src, dist.group.WORLD)
    got = M.to_megatron_state(full)
    for k in want:
        ok &= torch.equal(want[k], got[k])
    print(f"RESULT rank {rank} ok={bool(ok)}", flush=True)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
