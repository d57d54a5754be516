"""Worker: the run loop over a pipeline x data mesh (gloo): a straight run and a run that exits after a
checkpoint and resumes must end on the same loss; every rank reports the same losses.
  argv: <out_dir> <pipeline_parallel> <virtual stages> <phase: straight | die | resume> [tensor_parallel]"""
import io
import json
import os
import sys

import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from mlperf_training_b200.trainer.loop import run  # noqa: E402

TINY = dict(n_layers=4, hidden=32, n_heads=2, n_kv_heads=2, head_dim=16, ffn_hidden=64, vocab_size=64, seq_len=16, dtype="fp32")


def main():
    out_dir, pp, v, phase = sys.argv[1], int(sys.argv[2]), int(sys.argv[3]), sys.argv[4]
    tp = int(sys.argv[5]) if len(sys.argv) > 5 else 1
    rank = int(os.environ["RANK"])
    dist.init_process_group("gloo")
    exp = dict(model=TINY, global_batch=8, micro_batch=1, train_iters=6, lr=5e-3, lr_warmup_iters=2, warmup_train_steps=1,
               pipeline_parallel=pp, virtual_pipeline_parallel=v, tensor_parallel=tp, eval_interval=3, eval_iters=1, clip_grad=1.0)
    if phase != "straight":
        exp.update(checkpoint_dir=os.path.join(out_dir, "ck"), die_at_step=3 if phase == "die" else 0)
    try:
        out = run(exp, device="cpu", stream=io.StringIO())
    except SystemExit as e:
        dist.destroy_process_group()
        sys.exit(int(e.code))
    with open(os.path.join(out_dir, f"{phase}_rank{rank}.json"), "w") as f:
        json.dump({"losses": out["losses"], "steps": out["steps"], "eval": out.get("eval_losses")}, f)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
