"""Worker (gloo): a multi-table embedding collection saves its TorchRec-layout sharded state; the checkpoint is read
back (a) under the same plan, (b) under another placement plan (row-wise <-> table-wise <-> column-wise), and the rows every rank then
holds equal the rows of the full tables.  argv: checkpoint directory"""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from mlperf_training_b200.parallel.embedding_collection import EmbeddingCollection, TableConfig  # noqa: E402


def full_table(t, group_world):
    """Every row of table ``t`` (all-gather of the ranks' row blocks, padded to the largest block; of the
    column slices for a column-wise table)."""
    if hasattr(t, "cols"):
        parts = [torch.zeros_like(t.weight) for _ in range(group_world)]
        dist.all_gather(parts, t.weight.clone())
        return torch.cat(parts, 1)
    n = torch.tensor([t.local_rows]); sizes = [torch.zeros(1, dtype=torch.int64) for _ in range(group_world)]
    dist.all_gather(sizes, n)
    m = int(max(s.item() for s in sizes))
    pad = torch.zeros(m, t.dim, dtype=t.weight.dtype); pad[: t.local_rows] = t.weight
    parts = [torch.zeros_like(pad) for _ in range(group_world)]
    dist.all_gather(parts, pad)
    return torch.cat([p[: int(s.item())] for p, s in zip(parts, sizes)], 0)


def main():
    root = sys.argv[1]
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo")
    tables = [TableConfig("item", 1003, 16, ("item_id",), "fp32"), TableConfig("artist", 97, 8, ("artist_id",), "fp32"),
              TableConfig("uid", 55, 8, ("uid",), "fp32")]
    plan_a = {"item": ("row_wise", None), "artist": ("table_wise", 1 % world), "uid": ("table_wise", 0)}
    plan_b = {"item": ("table_wise", 0), "artist": ("row_wise", None), "uid": ("table_wise", 1 % world)}
    src = EmbeddingCollection(tables, group=dist.group.WORLD, device="cpu", seed=4, plan=plan_a)
    for t in src.tables.values():
        t.state.uniform_(0.1, 1.0)
    src.save_sharded(os.path.join(root, "sparse"), prefix="model._embedding_collection.")
    ok = True
    import torch.distributed.checkpoint as dcp
    meta = dcp.FileSystemReader(os.path.join(root, "sparse")).read_metadata().state_dict_metadata
    key = "model._embedding_collection.embeddings.item.weight"
    ok &= tuple(meta[key].size) == (1003, 16) and len(meta[key].chunks) == world
    ok &= len(meta["model._embedding_collection.embeddings.uid.weight"].chunks) == 1          # table-wise: one owner
    want = {n: full_table(t, world) for n, t in src.tables.items()}
    plan_c = {"item": ("column_wise", None), "artist": ("table_wise", 0), "uid": ("row_wise", None)}
    for plan in (plan_a, plan_b, plan_c):
        dst = EmbeddingCollection(tables, group=dist.group.WORLD, device="cpu", seed=77, plan=plan)
        dst.load_sharded(os.path.join(root, "sparse"), prefix="model._embedding_collection.")
        for n, t in dst.tables.items():
            ok &= torch.equal(full_table(t, world), want[n])
        if plan is plan_a:
            for n, t in dst.tables.items():
                ok &= torch.equal(t.state, src.tables[n].state)
    # written column-wise (the last plan above), read back column-wise with its per-shard sums and row-wise without them
    for t in dst.tables.values():
        t.state.uniform_(0.1, 1.0)
    dst.save_sharded(os.path.join(root, "sparse_cw"))
    meta = dcp.FileSystemReader(os.path.join(root, "sparse_cw")).read_metadata().state_dict_metadata
    ok &= [tuple(c.offsets) for c in meta["embeddings.item.weight"].chunks] == [(0, 16 // world * r) for r in range(world)]
    for plan in (plan_c, plan_a):
        back = EmbeddingCollection(tables, group=dist.group.WORLD, device="cpu", seed=5, plan=plan)
        back.load_sharded(os.path.join(root, "sparse_cw"))
        for n, t in back.tables.items():
            ok &= torch.equal(full_table(t, world), want[n])
        if plan is plan_c:
            ok &= torch.equal(back.tables["item"].state, dst.tables["item"].state)
    print(f"RESULT rank {rank} ok={bool(ok)}", flush=True)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
