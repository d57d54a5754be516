"""Worker: training with the sequence sharded over the ranks (context parallel) follows the plain
trainer fed the whole sequences: losses, gradient norms and final parameters (gloo, fp32)."""
import io
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from mlperf_training_b200.models.gpt import GPTConfig  # noqa: E402
from mlperf_training_b200.parallel.engine import OptimConfig  # noqa: E402
from mlperf_training_b200.trainer.pretrain import PretrainTrainer, TrainConfig  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo")
    solo = [dist.new_group([r]) for r in range(world)][rank]
    cfg = dict(n_layers=2, hidden=32, n_heads=4, n_kv_heads=2, head_dim=8, ffn_hidden=64, vocab_size=64, seq_len=32, dtype="fp32")
    opt = OptimConfig(lr=3e-3, weight_decay=0.01, clip_grad=1.0)
    ok = True
    for mode, masked in (("allgather", False), ("ulysses", False), ("allgather", True), ("ring", False), ("ring", True)):
        tc = TrainConfig(micro_batch=1, local_batch=2, warmup_steps=0, seed=3)
        plain = PretrainTrainer(GPTConfig(**cfg), opt, tc, "cpu", group=solo)
        cp = PretrainTrainer(GPTConfig(**cfg), opt, tc, "cpu", group=dist.group.WORLD, cp_group=dist.group.WORLD, cp_mode=mode)
        for step in range(4):
            g = torch.Generator().manual_seed(100 + step)
            tok = torch.randint(0, 64, (2, 33), generator=g)
            if masked:
                x, y = tok[:, :-1].contiguous(), tok[:, 1:].clone()
                y[:, :19] = -100                       # an uneven split of the labelled positions over the chunks
                a, b = plain.train_step((x, y)), cp.train_step((x, y))
            else:
                a, b = plain.train_step(tok), cp.train_step(tok)
            good = abs(a - b) < 2e-5 * max(1.0, abs(a)) and abs(plain.engine.grad_norm() - cp.engine.grad_norm()) < 1e-4
            ok &= good
            if rank == 0:
                print(f"{mode} masked={masked} step {step}: plain {a:.6f} cp {b:.6f} gnorm {plain.engine.grad_norm():.5f} "
                      f"{cp.engine.grad_norm():.5f}", flush=True)
        for (n, p), (_, q) in zip(plain.model.named_parameters(), cp.model.named_parameters()):
            ok &= (p - q).abs().max().item() < 1e-5
        tok = torch.randint(0, 64, (2, 33), generator=torch.Generator().manual_seed(7))
        ea, eb = plain.eval_loss(tok), cp.eval_loss(tok)
        ok &= abs(float(ea) - float(eb)) < 1e-5
    # the run loop over a context x data mesh
    from mlperf_training_b200.trainer.loop import run
    per_mode = []
    for mode in ("allgather", "ring"):
        out = run(dict(model=cfg, global_batch=2, micro_batch=1, train_iters=3, warmup_train_steps=1, context_parallel=world,
                       context_parallel_mode=mode, eval_interval=3, eval_iters=1), device="cpu", stream=io.StringIO())
        t = torch.tensor(out["losses"], dtype=torch.float64)
        lo, hi = t.clone(), t.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        ok &= bool((hi - lo).abs().max() < 1e-9) and out["steps"] == 3 and out["eval_loss"] is not None
        per_mode.append(t)
    ok &= bool((per_mode[0] - per_mode[1]).abs().max() < 1e-5)          # the two forms train the same model
    print(f"RESULT rank {rank} ok={ok}", flush=True)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
