"""Pre-encoded text-to-image samples for the MMDiT run: VAE latents and text-encoder outputs computed
offline, read memory-mapped.

A dataset directory holds ``latents.npy`` ``[N, C, h, w]`` (16-channel VAE latents, e.g. 32 x 32 for
256-pixel images), ``t5.npy`` ``[N, txt_tokens, 4096]``, ``clip.npy`` ``[N, 768]`` (pooled), and
optionally ``empty_t5.npy`` ``[txt_tokens, 4096]`` / ``empty_clip.npy`` ``[768]``: the encodings of the empty
prompt that prompt dropout substitutes.  ``batch(step, rank, local_batch, world)`` returns the
tuple the trainer consumes - latents cut into 2 x 2 patches ``[B, (h/2)(w/2), 4C]``, text states,
pooled vector - for a pass order reshuffled per epoch from the seed, each rank taking its slice of the
step's samples; the evaluation directory is read in file order.  This mirrors what the reference's
diffusion trainer is configured with: a pre-encoded training set, an evaluation set and the
empty-prompt encodings (flux1/primus/conf/flux.1_schnell_t2i-pretrain.yaml:40-44).
"""
from __future__ import annotations

from pathlib import Path

import numpy as np
import torch

from ..models.mmdit import patchify


def write_encoded_dataset(root: str, latents: np.ndarray, t5: np.ndarray, clip: np.ndarray, empty_t5=None, empty_clip=None) -> None:
    d = Path(root)
    d.mkdir(parents=True, exist_ok=True)
    if not (len(latents) == len(t5) == len(clip)):
        raise ValueError("latents, t5 and clip must hold the same number of samples")
    np.save(d / "latents.npy", latents)
    np.save(d / "t5.npy", t5)
    np.save(d / "clip.npy", clip)
    if empty_t5 is not None:
        np.save(d / "empty_t5.npy", empty_t5)
    if empty_clip is not None:
        np.save(d / "empty_clip.npy", empty_clip)


class EncodedFluxData:
    def __init__(self, root: str, cfg, seed: int = 0, shuffle: bool = True, patch: int = 2):
        d = Path(root)
        self.latents = np.load(d / "latents.npy", mmap_mode="r")
        self.t5 = np.load(d / "t5.npy", mmap_mode="r")
        self.clip = np.load(d / "clip.npy", mmap_mode="r")
        self.n, self.seed, self.shuffle, self.patch = len(self.latents), seed, shuffle, patch
        C, h, w = self.latents.shape[1:]
        if (h // patch) * (w // patch) != cfg.img_tokens or C * patch * patch != cfg.in_channels:
            raise ValueError(f"latents {tuple(self.latents.shape[1:])} do not give {cfg.img_tokens} tokens of {cfg.in_channels} channels")
        if tuple(self.t5.shape[1:]) != (cfg.txt_tokens, cfg.txt_dim) or self.clip.shape[1] != cfg.vec_dim:
            raise ValueError(f"text encodings {self.t5.shape[1:]} / {self.clip.shape[1:]} do not match the model "
                             f"({cfg.txt_tokens} x {cfg.txt_dim}, {cfg.vec_dim})")
        self.empty_t5 = torch.from_numpy(np.load(d / "empty_t5.npy").astype(np.float32))[None] if (d / "empty_t5.npy").exists() else None
        self.empty_clip = torch.from_numpy(np.load(d / "empty_clip.npy").astype(np.float32))[None] if (d / "empty_clip.npy").exists() else None

    def steps_per_epoch(self, local_batch: int, world: int = 1) -> int:
        return self.n // (local_batch * world)

    def indices(self, step: int, rank: int, local_batch: int, world: int = 1) -> np.ndarray:
        per = self.steps_per_epoch(local_batch, world)
        if per == 0:
            raise IndexError(f"{self.n} samples do not fill one step of {local_batch} x {world}")
        epoch, k = divmod(step, per)
        order = np.random.default_rng([self.seed, epoch]).permutation(self.n) if self.shuffle else np.arange(self.n)
        lo = (k * world + rank) * local_batch
        return np.sort(order[lo:lo + local_batch])              # ascending: friendlier to the memory map

    def batch(self, step: int, rank: int, local_batch: int, world: int = 1):
        idx = self.indices(step, rank, local_batch, world)
        lat = torch.from_numpy(np.ascontiguousarray(self.latents[idx]).astype(np.float32))
        return (patchify(lat, self.patch), torch.from_numpy(np.ascontiguousarray(self.t5[idx]).astype(np.float32)),
                torch.from_numpy(np.ascontiguousarray(self.clip[idx]).astype(np.float32)))
