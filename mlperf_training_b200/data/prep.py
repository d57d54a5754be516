"""Dataset preparation utilities (the reference's ``scripts/`` of each workload):

    python -m mlperf_training_b200.data.prep convert-sft  <in.jsonl|in.parquet> <out.npy> [--seq-len 8192]
    python -m mlperf_training_b200.data.prep convert-events <processed_dir> <store_root> [--metadata-dir <dir>]
    python -m mlperf_training_b200.data.prep metadata     <packed.npy> <packed_metadata.jsonl>
    python -m mlperf_training_b200.data.prep hash         <directory>
    python -m mlperf_training_b200.data.prep verify       <directory> <checksums.md5>
    python -m mlperf_training_b200.data.prep window-index <timestamps.npy> <out.npz> --window-seconds N [--holdout F --salt S]

* ``convert-sft``: tokenised samples (``input_ids`` + optional ``loss_mask`` / ``labels``) are packed
  first-fit into rows of ``seq_len + 1`` tokens with ``seq_start_id`` boundaries - the GovReport
  parquet -> packed ``.npy`` conversion (llama2_sft/primus/scripts/convert_dataset.py) - and
  ``metadata`` writes the per-row ``packed_metadata.jsonl`` (create_metadata.py).
* ``hash`` / ``verify``: a directory MD5 manifest and its check (llama2_sft/primus/scripts/hash.py;
  recommendation_v4/scripts/verify_dataset.sh).
* ``window-index``: offline time-window index for the recommender stream: per window the sample
  ids in time order, with a deterministic salted hold-out split
  (generative_recommenders/dlrm_v4/datasets/offline_ts_indices.py, recommendation_v4/scripts/ts_index_tool.py).

There is no downloader: the reference fetches its data with an external tool from the network.
"""
from __future__ import annotations

import argparse
import hashlib
import json
import sys
from pathlib import Path

import numpy as np


# --------------------------------------------------------------------------- packing
def pack_samples(samples: list[dict], seq_len: int) -> list[dict]:
    """First-fit-decreasing packing of tokenised samples into rows of at most ``seq_len + 1`` tokens."""
    cap = seq_len + 1
    items = []
    for s in samples:
        ids = np.asarray(s["input_ids"], dtype=np.int64)[:cap]
        if "loss_mask" in s:
            mask = np.asarray(s["loss_mask"], dtype=np.int64)[:cap]
        elif "labels" in s:
            mask = (np.asarray(s["labels"], dtype=np.int64)[:cap] != -100).astype(np.int64)
        else:
            mask = np.ones_like(ids)
        items.append((ids, mask))
    items.sort(key=lambda t: -len(t[0]))
    rows: list[dict] = []
    space: list[int] = []
    for ids, mask in items:
        for r, free in enumerate(space):
            if len(ids) <= free:
                row = rows[r]
                row["seq_start_id"].append(len(row["input_ids"]))
                row["input_ids"] = np.concatenate([row["input_ids"], ids])
                row["loss_mask"] = np.concatenate([row["loss_mask"], mask])
                space[r] -= len(ids)
                break
        else:
            rows.append({"input_ids": ids, "loss_mask": mask, "seq_start_id": [0]})
            space.append(cap - len(ids))
    return rows


def read_samples(path: str) -> list[dict]:
    p = Path(path)
    if p.suffix == ".parquet":
        import pandas as pd
        df = pd.read_parquet(p)
        return [{k: row[k] for k in df.columns} for _, row in df.iterrows()]
    if p.suffix == ".npy":
        return list(np.load(p, allow_pickle=True))
    return [json.loads(l) for l in p.read_text().splitlines() if l.strip()]


def convert_sft(src: str, dst: str, seq_len: int) -> int:
    from .indexed import write_packed_sft
    rows = pack_samples(read_samples(src), seq_len)
    write_packed_sft(dst, rows, None)
    return len(rows)


def write_metadata(npy: str, out: str) -> int:
    rows = np.load(npy, allow_pickle=True)
    with open(out, "w") as f:
        for i, r in enumerate(rows):
            n = int(len(r["input_ids"]))
            f.write(json.dumps({"row": i, "tokens": n, "loss_tokens": int(np.asarray(r.get("loss_mask", np.ones(n))).sum()),
                                "sequences": len(r.get("seq_start_id", [0]))}) + "\n")
    return len(rows)


# --------------------------------------------------------------------------- checksums
def md5_file(path: Path, chunk: int = 1 << 22) -> str:
    h = hashlib.md5()
    with open(path, "rb") as f:
        while True:
            b = f.read(chunk)
            if not b:
                break
            h.update(b)
    return h.hexdigest()


def hash_directory(root: str) -> list[tuple[str, str]]:
    base = Path(root)
    return [(md5_file(p), str(p.relative_to(base))) for p in sorted(base.rglob("*")) if p.is_file()]


def verify_directory(root: str, manifest: str) -> list[str]:
    """Names that are missing or whose checksum differs (empty = verified)."""
    want = {}
    for line in Path(manifest).read_text().splitlines():
        if line.strip():
            digest, name = line.split(None, 1)
            want[name.strip().lstrip("*")] = digest
    have = {name: digest for digest, name in hash_directory(root)}
    return sorted(n for n, d in want.items() if have.get(n) != d)


# --------------------------------------------------------------------------- time windows
def build_window_index(timestamps: np.ndarray, window_seconds: int, holdout: float = 0.0, salt: int = 0) -> dict:
    """Samples grouped into consecutive time windows (ids in time order inside a window) and a
    deterministic hold-out mask: sample ``i`` is held out when ``hash(i, salt)`` falls below ``holdout``."""
    ts = np.asarray(timestamps, dtype=np.int64)
    order = np.argsort(ts, kind="stable")
    win = (ts[order] - ts[order][0]) // int(window_seconds)
    starts = np.flatnonzero(np.r_[True, win[1:] != win[:-1]])
    with np.errstate(over="ignore"):                       # splitmix64 finaliser, wrap-around intended
        z = np.arange(len(ts), dtype=np.uint64) + np.uint64(salt) * np.uint64(0x9E3779B97F4A7C15) + np.uint64(1)
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        z = z ^ (z >> np.uint64(31))
    held = ((z >> np.uint64(40)).astype(np.float64) / float(1 << 24)) < holdout
    return {"order": order.astype(np.int64), "window_start": starts.astype(np.int64),
            "window_id": win[starts].astype(np.int64), "holdout": held,
            "contract": np.array([window_seconds, salt, int(holdout * 1e6)], dtype=np.int64)}


# --------------------------------------------------------------------------- downloads
def download_manifest(manifest: str, dest: str, retries: int = 3) -> list[str]:
    """Fetch the files of a manifest (one ``<md5>  <relative path>  <url>`` per line) into ``dest``, skipping
    files whose md5 already matches, verifying each download.  Returns the paths fetched.  The dataset
    scripts of the reference do the same with rclone / wget and md5 lists
    (small_llm_pretraining/primus/README.md:30-60, llama2_sft/primus/README.md:10-64)."""
    import hashlib
    import urllib.request
    got = []
    for line in Path(manifest).read_text().splitlines():
        parts = line.split()
        if len(parts) < 3 or line.lstrip().startswith("#"):
            continue
        digest, rel, url = parts[0], parts[1], parts[2]
        out = Path(dest) / rel
        if out.exists() and hashlib.md5(out.read_bytes()).hexdigest() == digest:
            continue
        out.parent.mkdir(parents=True, exist_ok=True)
        for attempt in range(retries):
            tmp = out.with_suffix(out.suffix + ".part")
            urllib.request.urlretrieve(url, tmp)
            if hashlib.md5(tmp.read_bytes()).hexdigest() == digest:
                tmp.replace(out)
                got.append(str(out))
                break
            tmp.unlink(missing_ok=True)
        else:
            raise OSError(f"{rel}: md5 mismatch after {retries} attempts")
    return got


# --------------------------------------------------------------------------- Hugging Face -> torch_dist
def hf_llama_to_gpt_state(hf: dict, n_layers: int) -> dict:
    """Hugging Face Llama parameter names -> this package's ``GPT`` names (fused q|k|v and gate|up rows;
    both sides use the rotate-half rotary convention, so no permutation of the projection rows)."""
    import torch
    out = {"embed": hf["model.embed_tokens.weight"], "final_norm": hf["model.norm.weight"],
           "lm_head": hf.get("lm_head.weight", hf["model.embed_tokens.weight"])}
    for i in range(n_layers):
        p = f"model.layers.{i}."
        out[f"blocks.{i}.attn_norm"] = hf[p + "input_layernorm.weight"]
        out[f"blocks.{i}.w_qkv"] = torch.cat([hf[p + f"self_attn.{n}_proj.weight"] for n in ("q", "k", "v")], 0)
        out[f"blocks.{i}.w_proj"] = hf[p + "self_attn.o_proj.weight"]
        out[f"blocks.{i}.mlp_norm"] = hf[p + "post_attention_layernorm.weight"]
        out[f"blocks.{i}.mlp.w_gate_up"] = torch.cat([hf[p + "mlp.gate_proj.weight"], hf[p + "mlp.up_proj.weight"]], 0)
        out[f"blocks.{i}.mlp.w_down"] = hf[p + "mlp.down_proj.weight"]
    return out


def convert_hf_llama(hf_dir: str, out_root: str, preset: str = "llama2-70b", dtype: str = "bf16") -> str:
    """A Hugging Face Llama directory (``*.safetensors`` or ``pytorch_model*.bin`` shards + ``config.json``) ->
    a Megatron ``torch_dist`` checkpoint that ``pretrained_checkpoint`` loads (the reference converts with
    Megatron-Bridge: llama2_sft/primus/README.md:53-76)."""
    import json

    import torch

    from ..checkpoint.megatron import save_torch_dist
    from ..models.gpt import GPT, PRESETS
    cfg = PRESETS[preset]()
    hf_cfg = json.loads((Path(hf_dir) / "config.json").read_text()) if (Path(hf_dir) / "config.json").exists() else {}
    for ours, theirs in (("n_layers", "num_hidden_layers"), ("hidden", "hidden_size"), ("n_heads", "num_attention_heads"),
                         ("n_kv_heads", "num_key_value_heads"), ("ffn_hidden", "intermediate_size"), ("vocab_size", "vocab_size")):
        if theirs in hf_cfg:
            setattr(cfg, ours, int(hf_cfg[theirs]))
    cfg.dtype = dtype
    state = {}
    shards = sorted(Path(hf_dir).glob("*.safetensors"))
    if shards:
        from safetensors.torch import load_file
        for f in shards:
            state.update(load_file(str(f)))
    else:
        for f in sorted(Path(hf_dir).glob("pytorch_model*.bin")):
            state.update(torch.load(f, map_location="cpu", weights_only=True))
    if not state:
        raise FileNotFoundError(f"no *.safetensors or pytorch_model*.bin under {hf_dir}")
    model = GPT(cfg, device="cpu", seed=0)
    mine = dict(model.named_parameters())
    with torch.no_grad():
        for name, t in hf_llama_to_gpt_state(state, cfg.n_layers).items():
            if tuple(mine[name].shape) != tuple(t.shape):
                raise ValueError(f"{name}: checkpoint shape {tuple(t.shape)} vs model {tuple(mine[name].shape)}")
            mine[name].copy_(t.to(mine[name].dtype))
    return str(save_torch_dist(model, out_root, iteration=0))


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="b200-data-prep")
    sub = ap.add_subparsers(dest="cmd", required=True)
    c = sub.add_parser("convert-sft"); c.add_argument("src"); c.add_argument("dst"); c.add_argument("--seq-len", type=int, default=8192)
    m = sub.add_parser("metadata"); m.add_argument("npy"); m.add_argument("out")
    h = sub.add_parser("hash"); h.add_argument("root")
    v = sub.add_parser("verify"); v.add_argument("root"); v.add_argument("manifest")
    w = sub.add_parser("window-index"); w.add_argument("timestamps"); w.add_argument("out")
    w.add_argument("--window-seconds", type=int, required=True); w.add_argument("--holdout", type=float, default=0.0)
    w.add_argument("--salt", type=int, default=0)
    e = sub.add_parser("synthetic-events"); e.add_argument("root"); e.add_argument("--users", type=int, default=10_000)
    e.add_argument("--events-per-user", type=int, default=200); e.add_argument("--items", type=int, default=1_000_000)
    e.add_argument("--days", type=int, default=7); e.add_argument("--seed", type=int, default=0)
    q = sub.add_parser("synthetic-sequences"); q.add_argument("path"); q.add_argument("--users", type=int, default=10_000)
    q.add_argument("--items", type=int, default=100_000); q.add_argument("--kind", default="movielens", choices=["movielens", "kuairand"])
    q.add_argument("--min-len", type=int, default=8); q.add_argument("--max-len", type=int, default=200); q.add_argument("--seed", type=int, default=0)
    cv = sub.add_parser("convert-events"); cv.add_argument("processed_dir"); cv.add_argument("root")
    cv.add_argument("--metadata-dir", default=None); cv.add_argument("--listen-plus-threshold", type=float, default=50.0)
    d = sub.add_parser("download"); d.add_argument("manifest"); d.add_argument("dest")
    f = sub.add_parser("hf-to-torch-dist"); f.add_argument("hf_dir"); f.add_argument("out_root")
    f.add_argument("--preset", default="llama2-70b"); f.add_argument("--dtype", default="bf16")
    a = ap.parse_args(argv)
    if a.cmd == "download":
        for path in download_manifest(a.manifest, a.dest):
            print(f"fetched {path}")
    elif a.cmd == "hf-to-torch-dist":
        print(f"torch_dist checkpoint -> {convert_hf_llama(a.hf_dir, a.out_root, a.preset, a.dtype)}")
    elif a.cmd == "synthetic-events":
        from .yambda import write_synthetic_event_store
        n = write_synthetic_event_store(a.root, a.users, a.events_per_user, a.items, days=a.days, seed=a.seed)
        print(f"{n} events of {a.users} users -> {a.root}")
    elif a.cmd == "convert-events":
        from .yambda import convert_sessions
        n = convert_sessions(a.processed_dir, a.metadata_dir, a.root, a.listen_plus_threshold)
        print(f"{n} events -> {a.root}")
    elif a.cmd == "synthetic-sequences":
        from .sequences import write_synthetic_sequences
        write_synthetic_sequences(a.path, a.users, a.items, min_len=a.min_len, max_len=a.max_len, seed=a.seed, kind=a.kind)
        print(f"{a.users} users -> {a.path}")
    elif a.cmd == "convert-sft":
        print(f"{convert_sft(a.src, a.dst, a.seq_len)} packed rows -> {a.dst}")
    elif a.cmd == "metadata":
        print(f"{write_metadata(a.npy, a.out)} rows -> {a.out}")
    elif a.cmd == "hash":
        for digest, name in hash_directory(a.root):
            print(f"{digest}  {name}")
    elif a.cmd == "verify":
        bad = verify_directory(a.root, a.manifest)
        for n in bad:
            print(f"FAILED {n}")
        print("verified" if not bad else f"{len(bad)} file(s) differ")
        return 1 if bad else 0
    else:
        idx = build_window_index(np.load(a.timestamps), a.window_seconds, a.holdout, a.salt)
        np.savez(a.out, **idx)
        print(f"{len(idx['window_start'])} windows -> {a.out}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
