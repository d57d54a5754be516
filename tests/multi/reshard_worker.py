"""Worker: a checkpoint written by N data-parallel ranks resumes on another number of ranks.
  argv: <dir> <phase: write | read>.  ``write`` trains 3 steps, saves, and dumps the full (gathered)
  optimizer state; ``read`` resumes under the current world size and checks its slices against that dump."""
import io
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from mlperf_training_b200.trainer.loop import run  # noqa: E402

TINY = dict(n_layers=2, hidden=32, n_heads=2, n_kv_heads=1, head_dim=16, ffn_hidden=64, vocab_size=64, seq_len=16, dtype="fp32")


def full_state(engine):
    """{bucket: (m, v, params)} gathered over the ranks, cut to the parameter payload."""
    out = {}
    world = dist.get_world_size()
    for b in engine.buckets:
        n = b.offsets[-1] + b.params[-1][1].numel()
        parts = {}
        for name in ("m", "v"):
            pieces = [torch.empty_like(getattr(b, name)) for _ in range(world)]
            dist.all_gather(pieces, getattr(b, name).contiguous())
            parts[name] = torch.cat(pieces)[:n].clone()
        out[b.key] = (parts["m"], parts["v"], b.param_buf[:n].clone())
    return out


def main():
    root, phase = sys.argv[1], sys.argv[2]
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo")
    exp = dict(model=TINY, global_batch=8, micro_batch=1, lr=5e-3, lr_warmup_iters=2, warmup_train_steps=0,
               checkpoint_dir=os.path.join(root, "ck"))
    ok = True
    if phase == "write":
        out = run(dict(exp, train_iters=3, checkpoint_every=3), device="cpu", stream=io.StringIO())
        state = full_state(out["trainer"].engine)
        if rank == 0:
            torch.save(state, os.path.join(root, "full.pt"))
    else:
        out = run(dict(exp, train_iters=3), device="cpu", stream=io.StringIO())       # already at step 3: loads, runs nothing
        ok &= out["steps"] == 0 and out["trainer"].engine.step_count == 3
        want = torch.load(os.path.join(root, "full.pt"), weights_only=False)
        got = full_state(out["trainer"].engine)
        for k, (m, v, p) in want.items():
            ok &= torch.equal(got[k][0], m) and torch.equal(got[k][1], v) and torch.equal(got[k][2], p)
            ok &= float(m.abs().sum()) > 0
        more = run(dict(exp, train_iters=5), device="cpu", stream=io.StringIO())      # and it trains on from there
        ok &= more["steps"] == 2 and all(l == l for l in more["losses"])
    print(f"RESULT rank {rank} ok={ok}", flush=True)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
