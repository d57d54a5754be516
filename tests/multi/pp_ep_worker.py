"""Worker (gloo, 4 ranks): a mixture-of-experts model over pipeline 2 x data 2 with the experts of every stage spread
over its two data-parallel replicas follows the unsplit model trained on the same four micro-batches; then the run
loop drives the same mesh from a configuration and resumes it after an exit.  argv: <checkpoint root>"""
import io
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from mlperf_training_b200.models.gpt import GPT, tiny_moe  # noqa: E402
from mlperf_training_b200.parallel.engine import OptimConfig, ZeroEngine  # noqa: E402
from mlperf_training_b200.parallel.mesh import Mesh, MeshSpec  # noqa: E402
from mlperf_training_b200.trainer.loop import run  # noqa: E402
from mlperf_training_b200.trainer.pipeline_train import PipelineTrainer  # noqa: E402
from mlperf_training_b200.trainer.pretrain import TrainConfig  # noqa: E402

SMALL = dict(n_layers=4, hidden=64, n_heads=4, n_kv_heads=2, head_dim=16, moe_ffn_hidden=64, n_experts=4, top_k=2,
             vocab_size=128, seq_len=32, window=16)


def main():
    root = sys.argv[1]
    rank = int(os.environ["RANK"])
    dist.init_process_group("gloo")
    solo = [dist.new_group([r]) for r in range(4)][rank]
    cfg = tiny_moe(**SMALL)
    full = GPT(cfg, "cpu", seed=0)
    opt = OptimConfig(lr=2e-3, weight_decay=0.05, clip_grad=1.0)
    e_full = ZeroEngine(full, opt, group=solo)
    mesh = Mesh(MeshSpec(pp=2, ep=2))
    ok = mesh.size("dp") == 2 and mesh.size("ep") == 2
    tr = PipelineTrainer(cfg, opt, TrainConfig(micro_batch=1, local_batch=2, seed=0), "cpu", mesh, ep_group=mesh.group("ep"))
    for chunk in tr.chunks:
        chunk.load_from_full(full)
    blk = tr.chunks[0].blocks[0]
    ok &= blk.mlp.w1.shape[0] * 2 == full.blocks[0].mlp.w1.shape[0]                 # half the experts live here
    d = mesh.index("dp")
    for step in range(4):
        g = torch.Generator().manual_seed(50 + step)
        tok = torch.randint(0, cfg.vocab_size, (4, cfg.seq_len + 1), generator=g)   # two micro-batches per replica
        ref = 0.0
        for i in range(4):
            l = full(tok[i:i + 1, :-1].contiguous(), tok[i:i + 1, 1:].contiguous())
            l.backward()
            ref += float(l.detach()) / 4
        e_full.step(tr.lr(), grad_scale=0.25)
        loss = tr.train_step_device(tok[2 * d:2 * d + 2]).clone()
        dist.all_reduce(loss, group=mesh.group("dp"))
        loss = float(loss) / 2
        # (the norm is reported before the 1 / micro-batches scale: four accumulated micro-batches there, two here)
        n_ref, n_pp = e_full.grad_norm() / 4, tr.engine.grad_norm() / 2
        ok &= abs(loss - ref) < 2e-4 * max(1.0, abs(ref)) and abs(n_ref - n_pp) < 2e-3 * max(1.0, n_ref)
        if rank == 0:
            print(f"step {step} unsplit {ref:.5f} pp x ep {loss:.5f} gnorm {n_ref:.4f} {n_pp:.4f}", flush=True)
    ep_rank = mesh.index("ep")
    for chunk in tr.chunks:
        for b, i in zip(chunk.blocks, chunk.layers):
            want = full.blocks[i].mlp.w1[ep_rank * 2:(ep_rank + 1) * 2]
            ok &= bool((b.mlp.w1 - want).abs().max() < 5e-5)

    exp = dict(model=dict(preset="tiny-moe", **SMALL), global_batch=4, micro_batch=1, train_iters=4, lr=3e-3, lr_warmup_iters=1,
               warmup_train_steps=1, pipeline_parallel=2, expert_parallel=2, moe_dispatch="nccl")
    straight = run(dict(exp), device="cpu", stream=io.StringIO())
    ok &= straight["steps"] == 4 and all(l == l for l in straight["losses"])
    ck = dict(exp, checkpoint_dir=os.path.join(root, "ck"), die_at_step=2)
    try:
        run(dict(ck), device="cpu", stream=io.StringIO())
        ok = False
    except SystemExit as e:
        ok &= int(e.code) == 42
    out = run(dict(ck, die_at_step=0), device="cpu", stream=io.StringIO())
    ok &= out["steps"] == 2 and max(abs(a - b) for a, b in zip(out["losses"], straight["losses"][2:])) < 1e-6
    print(f"RESULT rank {rank} ok={bool(ok)}", flush=True)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
