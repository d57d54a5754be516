"""Tolerance helpers of the GPU tests: a result is compared tile by tile (relative Frobenius error of
every 128 x 128 tile against the reference tile) and by cosine, so that a wrong tile far away from
the largest element cannot hide behind a max-norm bound."""
import torch


def tile_errors(got: torch.Tensor, ref: torch.Tensor, tile: int = 128) -> torch.Tensor:
    """Relative Frobenius error of every ``tile x tile`` block of 2-D ``got`` against ``ref`` (ragged edges
    padded with zeros on both sides)."""
    g, r = got.float(), ref.float()
    M, N = r.shape
    Mp, Np = (M + tile - 1) // tile * tile, (N + tile - 1) // tile * tile
    if (Mp, Np) != (M, N):
        g = torch.nn.functional.pad(g, (0, Np - N, 0, Mp - M))
        r = torch.nn.functional.pad(r, (0, Np - N, 0, Mp - M))
    e = (g - r).reshape(Mp // tile, tile, Np // tile, tile).norm(dim=(1, 3))
    n = r.reshape(Mp // tile, tile, Np // tile, tile).norm(dim=(1, 3))
    return e / (n + 1e-6 * n.max().clamp_min(1e-30))


def assert_tiles_close(got, ref, rel: float, cos: float = 0.9999, what: str = "", tile: int = 128) -> None:
    g2, r2 = got.reshape(-1, got.shape[-1]), ref.reshape(-1, ref.shape[-1])
    te = tile_errors(g2, r2, tile)
    worst = float(te.max())
    c = float(torch.nn.functional.cosine_similarity(g2.float().reshape(1, -1), r2.float().reshape(1, -1)))
    assert worst <= rel, f"{what}: worst tile relative error {worst:.3e} > {rel:.1e} at tile {divmod(int(te.argmax()), te.shape[1])}"
    assert c >= cos, f"{what}: cosine {c:.6f} < {cos}"
