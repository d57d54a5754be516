"""Worker (gloo, 4 ranks): tensor parallel 2 x data parallel 2 with the experts of the mixture-of-experts blocks spread
over the two data-parallel ranks - every tensor-parallel rank routes its own block of token rows - follows the unsplit
model trained on the same micro-batches; then the run loop on the same mesh."""
import io
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from mlperf_training_b200.models.gpt import GPT, shard_of, tiny_moe  # noqa: E402
from mlperf_training_b200.parallel.engine import OptimConfig, ZeroEngine  # noqa: E402
from mlperf_training_b200.parallel.mesh import Mesh, MeshSpec  # noqa: E402
from mlperf_training_b200.parallel.tensor import TPContext  # noqa: E402
from mlperf_training_b200.trainer.loop import run  # noqa: E402

SMALL = dict(n_layers=2, hidden=64, n_heads=4, n_kv_heads=2, head_dim=16, moe_ffn_hidden=64, n_experts=4, top_k=2,
             vocab_size=128, seq_len=32, window=16)


def main():
    rank = int(os.environ["RANK"])
    dist.init_process_group("gloo")
    solo = [dist.new_group([r]) for r in range(4)][rank]
    cfg = tiny_moe(**SMALL)
    full = GPT(cfg, "cpu", seed=0)
    opt = OptimConfig(lr=2e-3, weight_decay=0.05, clip_grad=1.0)
    e_full = ZeroEngine(full, opt, group=solo)
    mesh = Mesh(MeshSpec(tp=2, ep=2))
    tp = TPContext(mesh.group("tp"), comm="nccl")
    model = GPT(cfg, "cpu", seed=0, ep_group=mesh.group("ep"), tp=tp)
    ep_rank, per = mesh.index("ep"), cfg.n_experts // 2
    with torch.no_grad():          # the unsplit model's weights: this rank's block of the expert stacks, its slices of the attention
        src = dict(full.named_parameters())
        for n, p in model.named_parameters():
            shard = getattr(p, "tensor_parallel", None)
            if getattr(p, "expert_parallel", False):
                p.copy_(src[n][ep_rank * per:(ep_rank + 1) * per])
            elif shard is not None:
                p.copy_(shard_of(src[n], shard[0], shard[1], shard[2], cfg))
            else:
                p.copy_(src[n])
    eng = ZeroEngine(model, opt, group=mesh.group("dp"), tp_group=mesh.group("tp"))
    ok = model.blocks[0].mlp.w1.shape[0] == per and model.blocks[0].w_qkv.shape[0] * 2 == full.blocks[0].w_qkv.shape[0]
    d = mesh.index("dp")
    for step in range(4):
        g = torch.Generator().manual_seed(70 + step)
        tok = torch.randint(0, cfg.vocab_size, (2, cfg.seq_len + 1), generator=g)      # one sequence per data-parallel rank
        ref = 0.0
        for i in range(2):
            l = full(tok[i:i + 1, :-1].contiguous(), tok[i:i + 1, 1:].contiguous())
            l.backward()
            ref += float(l.detach()) / 2
        e_full.step(grad_scale=0.5)
        lt = model(tok[d:d + 1, :-1].contiguous(), tok[d:d + 1, 1:].contiguous())
        lt.backward()
        eng.step()
        tot = lt.detach().float().clone()
        dist.all_reduce(tot)                               # sum over tensor-parallel shares and both replicas
        loss = float(tot) / 2
        n_ref, n_tp = e_full.grad_norm() / 2, eng.grad_norm()
        ok &= abs(loss - ref) < 2e-4 * max(1.0, abs(ref)) and abs(n_ref - n_tp) < 2e-3 * max(1.0, n_ref)
        if rank == 0:
            print(f"step {step} unsplit {ref:.5f} tp x ep {loss:.5f} gnorm {n_ref:.4f} {n_tp:.4f}", flush=True)
    out = run(dict(model=dict(preset="tiny-moe", **SMALL), global_batch=2, micro_batch=1, train_iters=3, lr=3e-3, lr_warmup_iters=1,
                   warmup_train_steps=1, tensor_parallel=2, expert_parallel=2, moe_dispatch="nccl", eval_interval=3, eval_iters=1),
              device="cpu", stream=io.StringIO())
    ok &= out["steps"] == 3 and all(l == l for l in out["losses"])
    print(f"RESULT rank {rank} ok={bool(ok)}", flush=True)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
