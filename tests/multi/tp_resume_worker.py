"""Worker (gloo, world 2, tensor parallel 2): (1) a Megatron torch_dist checkpoint written by the
sharded model holds the unsharded tensors and loads back into sharded and unsharded models;
(2) the run loop resumes a tensor-parallel run exactly (every rank gets its own slices back);
(3) a resumed LoRA run reloads the frozen base from the pretrained checkpoint.
  argv: <out_dir>"""
import io
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from mlperf_training_b200.checkpoint.megatron import load_torch_dist, save_torch_dist, to_megatron_state  # noqa: E402
from mlperf_training_b200.models.gpt import GPT, GPTConfig  # noqa: E402
from mlperf_training_b200.parallel.tensor import TPContext  # noqa: E402
from mlperf_training_b200.trainer.loop import run  # noqa: E402

MODEL = dict(n_layers=2, hidden=64, n_heads=4, n_kv_heads=2, head_dim=16, ffn_hidden=128, vocab_size=128, seq_len=32,
             dtype="fp32")


def main():
    root = sys.argv[1]
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo")
    ok = True

    # ---- (1) checkpoint round trip across layouts
    cfg = GPTConfig(**MODEL)
    tp = TPContext(dist.group.WORLD, comm="nccl", device=None)
    sharded = GPT(cfg, device="cpu", seed=5, tp=tp)
    plain = GPT(cfg, device="cpu", seed=5)                 # a tensor-parallel model starts from the unsharded model's weights
    base_dir = os.path.join(root, "base")
    save_torch_dist(sharded, base_dir, iteration=0)
    want = to_megatron_state(plain)
    got = to_megatron_state(sharded, dist.group.WORLD)
    ok &= all(torch.equal(want[k], got[k]) for k in want)
    fresh_plain = GPT(cfg, device="cpu", seed=9)
    load_torch_dist(fresh_plain, base_dir)
    ok &= all(torch.equal(a, b) for (_, a), (_, b) in zip(fresh_plain.named_parameters(), plain.named_parameters()))
    fresh_sharded = GPT(cfg, device="cpu", seed=9, tp=tp)
    load_torch_dist(fresh_sharded, base_dir)
    ok &= all(torch.equal(a, b) for (_, a), (_, b) in zip(fresh_sharded.named_parameters(), sharded.named_parameters()))
    if rank == 0:
        print(f"round trip ok={ok}", flush=True)

    # ---- (2) tensor-parallel run: die after step 2, resume, same losses as the uninterrupted run
    base = dict(model=MODEL, global_batch=2, micro_batch=1, train_iters=4, lr=3e-3, lr_warmup_iters=1, warmup_train_steps=1,
                tensor_parallel=2, tp_comm_overlap="nccl")
    whole = run(dict(base), device="cpu", stream=io.StringIO())
    exp = dict(base, checkpoint_dir=os.path.join(root, "ck_tp"), die_at_step=2)
    try:
        run(dict(exp), device="cpu", stream=io.StringIO())
        ok = False
    except SystemExit as e:
        ok &= int(e.code) == 42
    out = run(dict(exp, die_at_step=0), device="cpu", stream=io.StringIO())
    d = max(abs(a - b) for a, b in zip(out["losses"], whole["losses"][2:]))
    ok &= out["steps"] == 2 and d < 1e-6
    if rank == 0:
        print(f"tp resume: max loss diff {d:.2e}", flush=True)

    # ---- (3) LoRA on a pretrained base: the resumed run holds the checkpoint's base weights again
    lora = dict(base, model=dict(MODEL, lora_rank=4, lora_dropout=0.0), pretrained_checkpoint=base_dir)
    whole = run(dict(lora), device="cpu", stream=io.StringIO())
    exp = dict(lora, checkpoint_dir=os.path.join(root, "ck_lora"), die_at_step=2)
    try:
        run(dict(exp), device="cpu", stream=io.StringIO())
        ok = False
    except SystemExit as e:
        ok &= int(e.code) == 42
    out = run(dict(exp, die_at_step=0), device="cpu", stream=io.StringIO())
    d = max(abs(a - b) for a, b in zip(out["losses"], whole["losses"][2:]))
    ok &= out["steps"] == 2 and d < 1e-6
    resumed = dict(out["trainer"].model.named_parameters())
    for name, p in sharded.named_parameters():
        if "lora" not in name:
            ok &= torch.equal(resumed[name].detach(), p.detach())          # frozen base == pretrained checkpoint
    if rank == 0:
        print(f"lora resume: max loss diff {d:.2e}", flush=True)
    print(f"RESULT rank {rank} ok={ok}", flush=True)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
