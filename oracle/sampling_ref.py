"""Oracle (test infrastructure): NumPy restatement of the reference's sampling pipeline,
src/sampling/mod.rs:30-113 with src/sampling/penalty.rs:28-52 and
src/sampling/nucleus.rs:7-62:

    penalties -> temperature -> softmax -> top-p nucleus filter -> renormalise -> draw

Everything is float32 as in the reference.  The draw itself (rand's SmallRng +
WeightedIndex, crates that are not in the reference tree) is restated as an inverse-CDF
lookup for a given uniform number u, so that a test can feed the same u to both sides;
the random stream of the reference is parity-unpinned.
"""
from __future__ import annotations

import numpy as np


def count_tokens(output_ids, vocab_size: int) -> np.ndarray:
    """count_tokens (penalty.rs:59-67): ids outside the vocabulary are ignored."""
    counts = np.zeros(vocab_size, dtype=np.uint32)
    for i in output_ids:
        if 0 <= int(i) < vocab_size:
            counts[int(i)] += 1
    return counts


def apply_penalties(logits: np.ndarray, counts: np.ndarray, presence: float, frequency: float) -> np.ndarray:
    """apply_penalties (penalty.rs:28-52): logit[t] -= presence + frequency * count[t] / total
    for every token seen at least once; a no-op when both penalties are below 1e-6."""
    out = np.array(logits, dtype=np.float32, copy=True)
    if abs(presence) < 1e-6 and abs(frequency) < 1e-6:
        return out
    counts = np.asarray(counts, dtype=np.uint32)
    total = np.float32(max(int(counts.sum()), 1))
    seen = counts > 0
    out[seen] = out[seen] - np.float32(presence)
    out[seen] = out[seen] - np.float32(frequency) * (counts[seen].astype(np.float32) / total)
    return out


def softmax(x: np.ndarray) -> np.ndarray:
    """softmax_inplace (nucleus.rs:15-26): exp(x - max), multiplied by 1/sum, in f32."""
    x = np.asarray(x, dtype=np.float32)
    e = np.exp(x - np.max(x)).astype(np.float32)
    return (e * (np.float32(1.0) / np.float32(e.sum(dtype=np.float32)))).astype(np.float32)


def nucleus_filter(probs: np.ndarray, top_p: float) -> np.ndarray:
    """nucleus_filter (nucleus.rs:32-49): indices by descending probability, accumulate in f32
    until the mass reaches top_p, zero the rest.  Ties are ordered by index here (the
    reference's sort is unstable)."""
    p = np.array(probs, dtype=np.float32, copy=True)
    order = np.argsort(-p, kind="stable")
    cum = np.float32(0.0)
    cutoff = len(p)
    for rank, idx in enumerate(order):
        cum = np.float32(cum + p[idx])
        if cum >= np.float32(top_p):
            cutoff = rank + 1
            break
    p[order[cutoff:]] = 0.0
    return p


def renormalize(probs: np.ndarray) -> np.ndarray:
    """renormalize (nucleus.rs:53-61)."""
    p = np.asarray(probs, dtype=np.float32)
    s = np.float32(p.sum(dtype=np.float32))
    return (p * (np.float32(1.0) / s)).astype(np.float32) if s > 0 else p


def logits_to_probs(logits, temperature: float, top_p: float, counts=None, presence: float = 0.0,
                    frequency: float = 0.0) -> np.ndarray:
    """logits_to_probs (mod.rs:78-100) after the penalties of the worker's sampling call:
    temperature below 1e-6 gives the delta distribution on the first maximum."""
    x = np.asarray(logits, dtype=np.float32)
    if counts is not None:
        x = apply_penalties(x, counts, presence, frequency)
    if temperature < 1e-6:
        out = np.zeros_like(x)
        out[int(np.argmax(x))] = 1.0
        return out
    p = softmax(x * (np.float32(1.0) / np.float32(temperature)))
    if top_p < 1.0 - 1e-6:
        p = renormalize(nucleus_filter(p, top_p))
    return p


def draw(probs: np.ndarray, u: float) -> int:
    """Inverse CDF in index order: the first token whose cumulative weight exceeds u * total
    (what WeightedIndex does with its uniform number, mod.rs:109-113)."""
    c = np.cumsum(np.asarray(probs, dtype=np.float64))
    return int(min(np.searchsorted(c, u * c[-1], side="right"), len(c) - 1))


def uniform_from_seed(seed: int) -> float:
    """The uniform number the CUDA sampler derives from a 64-bit seed: one splitmix64 step,
    top 24 bits.  (Not the reference's SmallRng stream, which is unpinned.)"""
    z = (seed + 0x9E3779B97F4A7C15) & 0xFFFFFFFFFFFFFFFF
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & 0xFFFFFFFFFFFFFFFF
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & 0xFFFFFFFFFFFFFFFF
    z ^= z >> 31
    return (z >> 40) / float(1 << 24)
