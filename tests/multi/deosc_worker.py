"""Worker (gloo, 2 ranks): weight de-oscillation under a sharded optimizer - every rank snaps the oscillating weights of
its own shard, the shards are gathered again, and the data-parallel replicas stay bit-identical."""
import io
import os
import sys

import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from mlperf_training_b200.trainer.loop import run  # noqa: E402


def main():
    dist.init_process_group("gloo")
    rank = dist.get_rank()
    tiny = dict(n_layers=2, hidden=128, n_heads=2, n_kv_heads=2, head_dim=64, ffn_hidden=256, vocab_size=256, seq_len=128,
                dtype="fp32", precision="mxfp4")
    spec = {"initial": "mxfp4", "deosc": {"enabled": True, "start_step": 0, "period": 2, "ratio": 0.5}}
    out = run(dict(model=tiny, global_batch=4, micro_batch=2, train_iters=6, lr=5e-3, lr_warmup_iters=1, clip_grad=1.0,
                   precision_schedule=spec, check_replicas_every=1), device="cpu", stream=io.StringIO())
    hist = out["deosc_history"]
    ok = [s for s, _ in hist] == [1, 3, 5] and all(n > 0 for _, n in hist)           # each rank snapped weights of its shard
    ok &= out["trainer"].engine.replica_checksum_spread() == 0.0 and all(l == l for l in out["losses"])
    print(f"RESULT rank {rank} ok={bool(ok)}", flush=True)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
