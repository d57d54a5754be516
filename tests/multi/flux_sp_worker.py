"""Worker: MMDiT training with every sample's tokens sharded over the ranks (Ulysses exchange around the
joint attention) follows the plain trainer: mean loss, gradient norm, parameters (gloo, fp32)."""
import io
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from mlperf_training_b200.models.mmdit import tiny_mmdit  # noqa: E402
from mlperf_training_b200.parallel.engine import OptimConfig  # noqa: E402
from mlperf_training_b200.trainer.flux import FluxTrainer, SyntheticFluxData, run  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo")
    if world == 4:
        # hybrid sharding (2 shards x 2 replicas) follows plain 4-way data parallelism
        base = dict(model=dict(preset="tiny-mmdit"), global_batch=4, train_iters=3, lr=2e-3)
        a = run(dict(base), device="cpu", stream=io.StringIO())
        b = run(dict(base, fsdp=dict(dp_replicate=2)), device="cpu", stream=io.StringIO())
        ok = max(abs(x - y) for x, y in zip(a["losses"], b["losses"])) < 1e-5
        for (n, p), (_, q) in zip(a["trainer"].model.named_parameters(), b["trainer"].model.named_parameters()):
            ok &= (p - q).abs().max().item() < 1e-5
        print(f"RESULT rank {rank} ok={ok}", flush=True)
        dist.barrier()
        dist.destroy_process_group()
        sys.exit(0 if ok else 1)
    solo = [dist.new_group([r]) for r in range(world)][rank]
    cfg = tiny_mmdit()
    opt = OptimConfig(lr=2e-3, weight_decay=0.01, clip_grad=1.0)
    plain = FluxTrainer(cfg, opt, "cpu", 2, prompt_dropout=0.1, seed=3, group=solo)
    sp = FluxTrainer(cfg, opt, "cpu", 2, prompt_dropout=0.1, seed=3, sp_group=dist.group.WORLD, group=dist.group.WORLD)
    data = SyntheticFluxData(cfg, seed=1)
    ok = True
    for step in range(3):
        b = data.batch(step, 0, 2)
        a = plain.train_step(b)
        mine = torch.tensor([sp.train_step(b)], dtype=torch.float64)
        dist.all_reduce(mine)
        mean = float(mine) / world
        good = abs(a - mean) < 1e-5 * max(1.0, abs(a)) and abs(plain.engine.grad_norm() - sp.engine.grad_norm()) < 1e-4
        ok &= good
        if rank == 0:
            print(f"step {step}: plain {a:.6f} sp {mean:.6f} gnorm {plain.engine.grad_norm():.5f} {sp.engine.grad_norm():.5f}", flush=True)
    for (n, p), (_, q) in zip(plain.model.named_parameters(), sp.model.named_parameters()):
        ok &= (p - q).abs().max().item() < 1e-5
    ok &= abs(plain.eval_loss(data.batch(9, 0, 2)) - sp.eval_loss(data.batch(9, 0, 2))) < 1e-5
    out = run(dict(model=dict(preset="tiny-mmdit"), global_batch=2, train_iters=3, sp_size=world, eval_every_samples=4),
              device="cpu", stream=io.StringIO())
    ok &= len(out["losses"]) == 3 and out["eval_loss"] is not None
    print(f"RESULT rank {rank} ok={ok}", flush=True)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
