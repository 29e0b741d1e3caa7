"""Seeded synthetic inputs with the shapes, sizes and value distributions of the data the
reference is run on (Pathfinder-style stroke images, PathTracker-style dot clips, N(0,1)
images).  The real datasets are not used anywhere; nothing here reproduces their items."""
from __future__ import annotations

import numpy as np


def stroke_image(seed: int, size: int = 128) -> np.ndarray:
    """(size, size) float32: background 0, 2-4 dashed polylines of 2-4 px width set to 1.0,
    regenerated until 5-7 % of the pixels are covered."""
    rng = np.random.default_rng(seed)
    for _ in range(200):
        img = np.zeros((size, size), np.float32)
        for _ in range(int(rng.integers(2, 5))):
            nv = int(rng.integers(3, 7))
            pts = rng.uniform(4, size - 4, size=(nv, 2))
            width = int(rng.integers(2, 5))
            on, off = int(rng.integers(6, 11)), int(rng.integers(3, 7))
            travelled = 0.0
            for a, b in zip(pts[:-1], pts[1:]):
                seg = float(np.hypot(*(b - a)))
                n = max(2, int(seg * 2))
                for s in np.linspace(0.0, 1.0, n):
                    d = (travelled + s * seg) % (on + off)
                    if d < on:
                        y, x = a + s * (b - a)
                        y0, x0 = int(round(y)) - width // 2, int(round(x)) - width // 2
                        img[max(0, y0):y0 + width, max(0, x0):x0 + width] = 1.0
                travelled += seg
        cov = float(img.mean())
        if 0.05 <= cov <= 0.07:
            return img
        # steer the next draw toward the coverage window
        rng = np.random.default_rng(rng.integers(1 << 31))
    return img


def stroke_batch(n: int, seed0: int = 1000, size: int = 128) -> np.ndarray:
    """(n, size, size, 1) float32."""
    return np.stack([stroke_image(seed0 + i, size) for i in range(n)])[..., None]


def dot_clips(n: int, T: int = 32, size: int = 32, dots: int = 16, seed0: int = 2000) -> np.ndarray:
    """(n, T, size, size, 3) float32: black frames with `dots` 1-px coloured dots doing a
    random walk of at most 2 px per frame."""
    out = np.zeros((n, T, size, size, 3), np.float32)
    for i in range(n):
        rng = np.random.default_rng(seed0 + i)
        pos = rng.integers(0, size, size=(dots, 2))
        col = rng.uniform(0.3, 1.0, size=(dots, 3)).astype(np.float32)
        for t in range(T):
            out[i, t, pos[:, 0], pos[:, 1]] = col
            pos = np.clip(pos + rng.integers(-2, 3, size=(dots, 2)), 0, size - 1)
    return out


def stem_features(images: np.ndarray, T: int, C: int, layers: int = 1, seed: int = 7):
    """Stand-in for SimpleCSSM's stem on stroke images (conv 3x3 -> softplus -> LayerNorm ->
    2x2 max-pool per layer, then repeat over T), giving a block input (B,T,H',W',C) with a
    realistic value distribution.  Random-init weights; NumPy only (set-up code, untimed)."""
    rng = np.random.default_rng(seed)
    x = images.astype(np.float32)                     # (B,H,W,cin)
    for _ in range(layers):
        cin = x.shape[-1]
        w = (rng.standard_normal((3, 3, cin, C)) / np.sqrt(9 * cin)).astype(np.float32)
        B, H, W, _ = x.shape
        xp = np.pad(x, ((0, 0), (1, 1), (1, 1), (0, 0)))
        y = np.zeros((B, H, W, C), np.float32)
        for i in range(3):
            for j in range(3):
                y += xp[:, i:i + H, j:j + W, :] @ w[i, j]
        y = np.logaddexp(y, 0.0)
        mu = y.mean(-1, keepdims=True)
        var = y.var(-1, keepdims=True)
        y = (y - mu) / np.sqrt(var + 1e-6)
        x = y.reshape(B, H // 2, 2, W // 2, 2, C).max(axis=(2, 4))
    return np.repeat(x[:, None], T, axis=1).astype(np.float32)
