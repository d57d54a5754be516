"""Worker (gloo, 4 ranks): tensor parallel 2 x context parallel 2 (all-gather and zig-zag ring forms) follows the plain
trainer fed the whole sequences - losses, gradient norms, evaluation loss; then the run loop on the same mesh."""
import io
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from mlperf_training_b200.models.gpt import GPTConfig  # noqa: E402
from mlperf_training_b200.parallel.engine import OptimConfig  # noqa: E402
from mlperf_training_b200.parallel.mesh import Mesh, MeshSpec  # noqa: E402
from mlperf_training_b200.parallel.tensor import TPContext  # noqa: E402
from mlperf_training_b200.trainer.loop import run  # noqa: E402
from mlperf_training_b200.trainer.pretrain import PretrainTrainer, TrainConfig  # noqa: E402


def main():
    rank = int(os.environ["RANK"])
    dist.init_process_group("gloo")
    solo = [dist.new_group([r]) for r in range(4)][rank]
    mesh = Mesh(MeshSpec(tp=2, cp=2))
    cfg = dict(n_layers=2, hidden=32, n_heads=4, n_kv_heads=2, head_dim=8, ffn_hidden=64, vocab_size=64, seq_len=32, dtype="fp32")
    opt = OptimConfig(lr=3e-3, weight_decay=0.01, clip_grad=1.0)
    tp = TPContext(mesh.group("tp"), comm="nccl")
    ok = mesh.ranks["tp"] == [rank - rank % 2, rank - rank % 2 + 1] and mesh.ranks["cp"] == [rank % 2, rank % 2 + 2]
    for mode, masked in (("allgather", False), ("ring", False), ("ring", True)):
        tc = TrainConfig(micro_batch=1, local_batch=2, warmup_steps=0, seed=3)
        plain = PretrainTrainer(GPTConfig(**cfg), opt, tc, "cpu", group=solo)
        both = PretrainTrainer(GPTConfig(**cfg), opt, tc, "cpu", group=mesh.group("dp_cp"), tp=tp, cp_group=mesh.group("cp"),
                               cp_mode=mode)
        for step in range(4):
            g = torch.Generator().manual_seed(100 + step)
            tok = torch.randint(0, 64, (2, 33), generator=g)
            if masked:
                x, y = tok[:, :-1].contiguous(), tok[:, 1:].clone()
                y[:, :19] = -100
                a, b = plain.train_step((x, y)), both.train_step((x, y))
            else:
                a, b = plain.train_step(tok), both.train_step(tok)
            good = abs(a - b) < 3e-5 * max(1.0, abs(a)) and abs(plain.engine.grad_norm() - both.engine.grad_norm()) < 2e-4
            ok &= good
            if rank == 0:
                print(f"{mode} masked={masked} step {step}: plain {a:.6f} tp x cp {b:.6f} gnorm {plain.engine.grad_norm():.5f} "
                      f"{both.engine.grad_norm():.5f}", flush=True)
        tok = torch.randint(0, 64, (2, 33), generator=torch.Generator().manual_seed(7))
        ok &= abs(float(plain.eval_loss(tok)) - float(both.eval_loss(tok))) < 2e-5
    out = run(dict(model=cfg, global_batch=2, micro_batch=1, train_iters=3, warmup_train_steps=1, tensor_parallel=2,
                   context_parallel=2, context_parallel_mode="ring", eval_interval=3, eval_iters=1),
              device="cpu", stream=io.StringIO())
    t = torch.tensor(out["losses"], dtype=torch.float64)
    lo, hi = t.clone(), t.clone()
    dist.all_reduce(lo, op=dist.ReduceOp.MIN)
    dist.all_reduce(hi, op=dist.ReduceOp.MAX)
    ok &= bool((hi - lo).abs().max() < 1e-9) and out["steps"] == 3 and out["eval_loss"] is not None
    print(f"RESULT rank {rank} ok={bool(ok)}", flush=True)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
