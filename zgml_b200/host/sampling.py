"""Next-token choice from a row of logits (host side; the logits of a step are downloaded anyway)."""
from typing import Optional

import numpy as np


class Sampler:
    """temperature == 0: greedy (lowest index among equal maxima, like np.argmax).  Otherwise softmax sampling at that
    temperature, optionally restricted to the `top_k` largest logits and / or the smallest set of probability `top_p`."""

    def __init__(self, temperature: float = 0.0, top_k: int = 0, top_p: float = 1.0, seed: Optional[int] = None):
        self.temperature, self.top_k, self.top_p = float(temperature), int(top_k), float(top_p)
        self.rng = np.random.default_rng(seed)

    def __call__(self, logits: np.ndarray) -> int:
        z = np.asarray(logits, dtype=np.float64).ravel()
        if self.temperature <= 0.0:
            return int(np.argmax(z))
        z = z / self.temperature
        if 0 < self.top_k < z.size:
            kth = np.partition(z, -self.top_k)[-self.top_k]
            z = np.where(z < kth, -np.inf, z)
        p = np.exp(z - z.max())
        p /= p.sum()
        if self.top_p < 1.0:
            order = np.argsort(-p, kind="stable")
            keep = np.cumsum(p[order]) - p[order] < self.top_p
            mask = np.zeros_like(p)
            mask[order[keep]] = 1.0
            p = p * mask
            p /= p.sum()
        return int(self.rng.choice(z.size, p=p))
