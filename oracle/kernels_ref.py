"""Oracle (test infrastructure): NumPy restatement of the reference's kernel-level math.

Every function names the reference lines it follows.  ``dtype`` is one of
"f32", "f16", "bf16"; tensors are carried as float32 arrays whose values are exactly
representable in that dtype, and ``rnd`` rounds a float32 array to it.
"""
from __future__ import annotations

import numpy as np


# ------------------------------------------------------------------ dtype rounding
def round_bf16(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even float32 -> bfloat16 -> float32."""
    a = np.ascontiguousarray(x, dtype=np.float32)
    u = a.view(np.uint32).astype(np.uint64)
    lsb = (u >> 16) & 1
    r = ((u + 0x7FFF + lsb) >> 16) << 16
    out = (r & 0xFFFFFFFF).astype(np.uint32).view(np.float32).reshape(a.shape)
    nan = np.isnan(a)
    if nan.any():
        out = out.copy()
        out[nan] = np.nan
    return out


def rnd(x: np.ndarray, dtype: str) -> np.ndarray:
    if dtype == "f32":
        return np.asarray(x, dtype=np.float32)
    if dtype == "f16":
        return np.asarray(x, dtype=np.float32).astype(np.float16).astype(np.float32)
    if dtype == "bf16":
        return round_bf16(np.asarray(x, dtype=np.float32))
    raise ValueError(dtype)


def to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """uint16 bit patterns of round_bf16(x)."""
    return (round_bf16(x).view(np.uint32) >> 16).astype(np.uint16)


def from_bf16_bits(b: np.ndarray) -> np.ndarray:
    return (b.astype(np.uint32) << 16).view(np.float32)


# ------------------------------------------------------------------------- RMSNorm
def rms_norm_kernel(x: np.ndarray, w: np.ndarray, eps: float, dtype: str = "f32") -> np.ndarray:
    """The fused kernel's numerics: fp32 sum of squares, y = x * rsqrt(ss/H + eps) * w,
    one rounding (kernels/rms_norm.cu:74-82 and :99-110)."""
    x = np.asarray(x, dtype=np.float32)
    hidden = x.shape[-1]
    ss = np.sum(x.astype(np.float64) ** 2, axis=-1, keepdims=True)
    scale = (1.0 / np.sqrt(ss / hidden + eps)).astype(np.float32)
    return rnd(x * scale * np.asarray(w, dtype=np.float32), dtype)


def rms_norm_fallback(x: np.ndarray, w: np.ndarray, eps: float, dtype: str = "f32") -> np.ndarray:
    """candle_fallback: (x.sqr().mean_keepdim(-1) + eps).sqrt(); x / rms * w, every op
    materialised in the tensor dtype (src/kernels/rms_norm.rs:128-132)."""
    x = np.asarray(x, dtype=np.float32)
    sq = rnd(x * x, dtype)
    mean = rnd(np.mean(sq.astype(np.float64), axis=-1, keepdims=True).astype(np.float32), dtype)
    rms = rnd(np.sqrt(rnd(mean + np.float32(eps), dtype)), dtype)
    return rnd(rnd(x / rms, dtype) * np.asarray(w, dtype=np.float32), dtype)


# ---------------------------------------------------------------------------- RoPE
def rope_inv_freq(theta: float, head_dim: int) -> np.ndarray:
    """inv_freq[i] = 1 / theta^(2i/d) in f32 (src/engine/arch/llama_tp.rs:119-121)."""
    i = np.arange(head_dim // 2, dtype=np.float32)
    expo = (np.float32(2.0) * i / np.float32(head_dim)).astype(np.float32)
    return (np.float32(1.0) / np.power(np.float32(theta), expo, dtype=np.float32)).astype(np.float32)


def rope_tables(positions: np.ndarray, theta: float, head_dim: int, dtype: str = "f32"):
    """cos/sin [n, d/2]: freqs = pos * inv_freq in f32, cos/sin in f32, then cast to the
    tensor dtype (src/engine/arch/llama_tp.rs:124-133)."""
    pos = np.asarray(positions, dtype=np.float32)
    freqs = (pos[:, None] * rope_inv_freq(theta, head_dim)[None, :]).astype(np.float32)
    return rnd(np.cos(freqs, dtype=np.float32), dtype), rnd(np.sin(freqs, dtype=np.float32), dtype)


def apply_rope(x: np.ndarray, cos: np.ndarray, sin: np.ndarray, dtype: str = "f32",
               per_op_rounding: bool = False) -> np.ndarray:
    """Rotate-half on x [n, heads, d] with cos/sin [n, d/2]:
    out = cat(x1*c - x2*s, x1*s + x2*c) (src/engine/arch/llama_tp.rs:135-149;
    kernels/rope.cu:36-39 computes the same in fp32 with one rounding).
    per_op_rounding=True rounds each product/sum to dtype as the eager path does."""
    x = np.asarray(x, dtype=np.float32)
    half = x.shape[-1] // 2
    x1, x2 = x[..., :half], x[..., half:]
    c, s = cos[:, None, :], sin[:, None, :]
    if per_op_rounding:
        a = rnd(rnd(x1 * c, dtype) - rnd(x2 * s, dtype), dtype)
        b = rnd(rnd(x1 * s, dtype) + rnd(x2 * c, dtype), dtype)
    else:
        a = rnd(x1 * c - x2 * s, dtype)
        b = rnd(x1 * s + x2 * c, dtype)
    return np.concatenate([a, b], axis=-1)


def rope_single(x: np.ndarray, cos_table: np.ndarray, sin_table: np.ndarray, dtype: str = "f32") -> np.ndarray:
    """rope_single_{f32,f16}: x [b, heads, seq, d], tables [seq, d/2], position =
    token % seq_len (kernels/rope.cu:19-63)."""
    x = np.asarray(x, dtype=np.float32)
    b, h, s, d = x.shape
    half = d // 2
    x0, x1 = x[..., :half], x[..., half:]
    c = np.asarray(cos_table, dtype=np.float32)[None, None, :, :]
    sn = np.asarray(sin_table, dtype=np.float32)[None, None, :, :]
    return np.concatenate([rnd(x0 * c - x1 * sn, dtype), rnd(x0 * sn + x1 * c, dtype)], axis=-1)


# ------------------------------------------------------------------------ KV write
def kv_slot_assign(buf: np.ndarray, src: np.ndarray, offset: int) -> np.ndarray:
    """buf[head*max_seq*hd + offset*hd + e] = src[head*hd + e], everything else
    unchanged (kernels/kv_assign.cu:16-28).  buf [nkv, max_seq, hd], src [nkv, hd]."""
    out = np.array(buf, copy=True)
    nkv, max_seq, hd = out.shape
    flat = out.reshape(-1)
    s = np.asarray(src).reshape(-1)
    for tid in range(nkv * hd):
        head, elem = divmod(tid, hd)
        flat[head * max_seq * hd + offset * hd + elem] = s[head * hd + elem]
    return out


def slot_for_position(table, pos: int, block_size: int = 16) -> int:
    """slot(pos) = table[pos / 16] * 16 + pos % 16."""
    return table[pos // block_size] * block_size + pos % block_size


def kv_assign_paged(cache: np.ndarray, rows: np.ndarray, slots, block_size: int = 16) -> np.ndarray:
    """cache [num_blocks, nkv, 16, hd]; rows [n_tokens, nkv, hd]."""
    out = np.array(cache, copy=True)
    for t, slot in enumerate(slots):
        if slot < 0:
            continue
        out[slot // block_size, :, slot % block_size, :] = rows[t]
    return out


# ---------------------------------------------------------------------------- mask
def causal_mask(sq: int, sk: int, seq_pos: int) -> np.ndarray:
    """Additive mask [sq, sk]: 0 where k_abs <= seq_pos + i, -inf otherwise
    (src/engine/arch/llama_tp.rs:160-179)."""
    q_abs = (seq_pos + np.arange(sq))[:, None]
    k_abs = np.arange(sk)[None, :]
    return np.where(k_abs > q_abs, -np.inf, 0.0).astype(np.float32)


def softmax_last(x: np.ndarray) -> np.ndarray:
    m = np.max(x, axis=-1, keepdims=True)
    e = np.exp(x - m)
    return e / np.sum(e, axis=-1, keepdims=True)


def silu(z: np.ndarray) -> np.ndarray:
    return z / (1.0 + np.exp(-z))
