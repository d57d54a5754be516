"""Worker (gloo, 4 ranks): context parallel 2 x data parallel 2 with the experts spread over the two data-parallel ranks
of a chunk - the copies of an expert in the other chunk sum their gradients - follows the unsplit mixture-of-experts
model through the run loop's trainer; then the run loop from a configuration."""
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
from mlperf_training_b200.trainer.pretrain import PretrainTrainer, TrainConfig  # noqa: E402

SMALL = dict(n_layers=2, hidden=64, n_heads=4, n_kv_heads=2, head_dim=16, moe_ffn_hidden=64, n_experts=4, top_k=2,
             vocab_size=128, seq_len=32, window=0, sink=False)


def main():
    rank = int(os.environ["RANK"])
    dist.init_process_group("gloo")
    solo = [dist.new_group([r]) for r in range(4)][rank]
    cfg = tiny_moe(**SMALL)
    full = GPT(cfg, "cpu", seed=0)
    opt = OptimConfig(lr=2e-3, weight_decay=0.05, clip_grad=1.0)
    e_full = ZeroEngine(full, opt, group=solo)
    mesh = Mesh(MeshSpec(cp=2, ep=2))
    ok = mesh.size("ep") == 2 and mesh.size("edp_cp") == 2 and mesh.size("dp_cp") == 4
    tr = PretrainTrainer(tiny_moe(**SMALL), opt, TrainConfig(micro_batch=1, local_batch=1, warmup_steps=0, seed=0), "cpu",
                         group=mesh.group("dp_cp"), ep_group=mesh.group("ep"), cp_group=mesh.group("cp"), cp_mode="ring",
                         expert_dp_group=mesh.group("edp_cp"))
    ep_rank, per = mesh.index("ep"), cfg.n_experts // 2
    with torch.no_grad():
        src = dict(full.named_parameters())
        for n, p in tr.model.named_parameters():
            p.copy_(src[n][ep_rank * per:(ep_rank + 1) * per] if getattr(p, "expert_parallel", False) else src[n])
    d = mesh.index("dp")
    for step in range(4):
        g = torch.Generator().manual_seed(90 + step)
        tok = torch.randint(0, cfg.vocab_size, (2, cfg.seq_len + 1), generator=g)      # one sequence per data-parallel rank
        ref = 0.0
        for i in range(2):
            l = full(tok[i:i + 1, :-1].contiguous(), tok[i:i + 1, 1:].contiguous())
            l.backward()
            ref += float(l.detach()) / 2
        e_full.step(tr.lr(), grad_scale=0.5)
        loss = tr.train_step_device(tok[d:d + 1]).clone()          # already averaged over the two chunks
        dist.all_reduce(loss, group=mesh.group("dp"))
        loss = float(loss) / 2
        n_ref, n_cp = e_full.grad_norm() / 2, tr.engine.grad_norm()
        ok &= abs(loss - ref) < 2e-4 * max(1.0, abs(ref)) and abs(n_ref - n_cp) < 2e-3 * max(1.0, n_ref)
        if rank == 0:
            print(f"step {step} unsplit {ref:.5f} cp x ep {loss:.5f} gnorm {n_ref:.4f} {n_cp:.4f}", flush=True)
    out = run(dict(model=dict(preset="tiny-moe", **SMALL), global_batch=2, micro_batch=1, train_iters=3, lr=3e-3, lr_warmup_iters=1,
                   warmup_train_steps=1, context_parallel=2, context_parallel_mode="ring", expert_parallel=2, moe_dispatch="nccl",
                   eval_interval=3, eval_iters=1), device="cpu", stream=io.StringIO())
    ok &= out["steps"] == 3 and all(l == l for l in out["losses"])
    print(f"RESULT rank {rank} ok={bool(ok)}", flush=True)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
