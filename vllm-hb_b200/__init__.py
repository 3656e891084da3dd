"""ctypes binding of libhb.so — the B200 tensor-parallel decode hot path of vllm-hb.

The product is the C ABI declared in ``include/hb.h``; this module is the thin host
mirror that the tests and ``bench.py`` use.  Names follow the reference's modules:

    kernels.rms_norm.apply / kernels.rope.apply / kernels.kv_assign.assign_slot
        (src/kernels/{rms_norm,rope,kv_assign}.rs)
    parallel.TpWorld, parallel.column_shard / row_shard
        (src/parallel/{world,shard}.rs)
    scheduler.BlockManager (src/scheduler/block_manager.rs)
    Engine (src/engine/loader.rs)

There is no CPU fallback: a missing library raises at import, a missing GPU makes the
compute calls fail with ``HbError``.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path
from typing import Optional, Sequence

import numpy as np

_HERE = Path(__file__).resolve().parent
# HB_LIBRARY names another build of the same library (the trace variant, libhb_trace.so)
LIB_PATH = Path(os.environ["HB_LIBRARY"]).resolve() if os.environ.get("HB_LIBRARY") else _HERE / "libhb.so"

if not LIB_PATH.exists():
    raise ImportError(
        f"{LIB_PATH} is missing: build it with `python vllm-hb_b200/build.py` "
        "(there is no fallback path)"
    )

lib = C.CDLL(str(LIB_PATH), mode=C.RTLD_GLOBAL)

F32, F16, BF16 = 0, 1, 2
ALGO_AUTO, ALGO_ONE_SHOT, ALGO_TWO_SHOT, ALGO_NCCL, ALGO_MULTIMEM = 0, 1, 2, 3, 4
BLOCK_SIZE = 16
IPC_HANDLE_BYTES = 64
NCCL_ID_BYTES = 128
MAX_RANKS = 8

ERR_INVALID_ARG, ERR_UNSUPPORTED_DTYPE, ERR_NOT_DIVISIBLE, ERR_CUDA = -1, -2, -3, -4
ERR_NCCL, ERR_TIMEOUT, ERR_OOM_BLOCKS, ERR_IO, ERR_EMPTY = -5, -6, -7, -8, -9


class HbError(RuntimeError):
    def __init__(self, code: int, msg: str):
        super().__init__(f"[{code}] {msg}")
        self.code = code
        self.msg = msg


class ModelConfig(C.Structure):
    """hb_model_config: ModelConfig of src/engine/config.rs:14-26 plus rank-side additions."""
    _fields_ = [
        ("model_path", C.c_char_p),
        ("max_seq_len", C.c_size_t),
        ("gpu_memory_utilization", C.c_double),
        ("bf16", C.c_int),
        ("tensor_parallel_size", C.c_int),
        ("num_kv_blocks", C.c_int64),
        ("max_batch", C.c_int),
        ("force_f32", C.c_int),
    ]


class ModelShape(C.Structure):
    _fields_ = [
        ("hidden_size", C.c_int64),
        ("intermediate_size", C.c_int64),
        ("num_hidden_layers", C.c_int64),
        ("num_attention_heads", C.c_int64),
        ("num_key_value_heads", C.c_int64),
        ("vocab_size", C.c_int64),
        ("rms_norm_eps", C.c_double),
        ("rope_theta", C.c_double),
        ("num_local_experts", C.c_int64),
        ("num_experts_per_tok", C.c_int64),
        ("sliding_window", C.c_int64),
    ]


_vp, _i, _i64, _f, _sz, _u64 = C.c_void_p, C.c_int, C.c_int64, C.c_float, C.c_size_t, C.c_uint64

_SIGS = {
    "hb_last_error": (C.c_char_p, []),
    "hb_version": (C.c_char_p, []),
    "hb_device_count": (_i, []),
    "hb_rms_norm": (_i, [_vp, _vp, _vp, _vp, _i64, _i64, _f, _i]),
    "hb_add_rms_norm": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _f, _i]),
    "hb_rope_inv_freq": (_i, [_f, _i, _vp]),
    "hb_rope": (_i, [_vp, _vp, _vp, _vp, _vp, _i64, _i, _i, _i, _i]),
    "hb_rope_cos_sin": (_i, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i, _i]),
    "hb_kv_assign_contig": (_i, [_vp, _vp, _vp, _i, _i64, _i, _i64, _i]),
    "hb_kv_assign_paged": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i, _i, _i64, _i]),
    "hb_attention_workspace_bytes": (_sz, [_i64, _i, _i, _i]),
    "hb_paged_decode_attention": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i, _i, _i, _i64, _i64, _i, _vp, _i]),
    "hb_paged_decode_attention_window": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i, _i, _i, _i64, _i64, _i, _vp, _i, _i]),
    "hb_moe_route": (_i, [_vp, _vp, _vp, _vp, _i64, _i64, _i, _i, _i]),
    "hb_paged_decode_attention_static_max_bytes": (_sz, []),
    "hb_paged_decode_attention_static": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i, _i, _i, _i64, _i64, _i, _i]),
    "hb_gemm_workspace_bytes": (_sz, [_i64, _i64, _i64, _i]),
    "hb_gemm": (_i, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _i, _vp]),
    "hb_gemm_ex_workspace_bytes": (_sz, [_i64, _i64, _i64, _i, _i]),
    "hb_gemm_ex": (_i, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _i, _i, _i, _vp]),
    "hb_silu_mul": (_i, [_vp, _vp, _vp, _i64, _i64, _i]),
    "hb_embed": (_i, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _i]),
    "hb_argmax": (_i, [_vp, _vp, _vp, _i64, _i64, _i]),
    "hb_world_create_local": (_i, [_i, _vp, _sz, _vp]),
    "hb_world_create_rank": (_i, [_i, _i, _i, _sz, _vp]),
    "hb_world_ipc_handle": (_i, [_vp, _vp]),
    "hb_world_attach": (_i, [_vp, _vp]),
    "hb_world_attach_ptrs": (_i, [_vp, _vp]),
    "hb_nccl_unique_id": (_i, [_vp]),
    "hb_world_init_nccl": (_i, [_vp, _vp]),
    "hb_world_free": (_i, [_vp]),
    "hb_world_size": (_i, [_vp]),
    "hb_world_rank": (_i, [_vp]),
    "hb_world_device": (_i, [_vp]),
    "hb_world_is_single": (_i, [_vp]),
    "hb_world_staging_bytes": (_sz, [_vp]),
    "hb_world_stream": (_vp, [_vp]),
    "hb_world_status": (_i, [_vp]),
    "hb_world_set_wait_limit": (_i, [_vp, C.c_uint32]),
    "hb_world_multicast_bytes": (C.c_size_t, [_i64, _i64]),
    "hb_world_attach_multicast": (_i, [_vp, _vp, _vp, C.c_size_t]),
    "hb_world_detach_multicast": (_i, [_vp]),
    "hb_world_has_multicast": (_i, [_vp]),
    "hb_world_multicast_partial": (_vp, [_vp]),
    "hb_all_reduce": (_i, [_vp, _vp, _vp, _sz, _i, _i]),
    "hb_all_reduce_add_rms_norm": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _f, _i, _i]),
    "hb_fused_rowparallel_workspace_bytes": (_sz, [_i64, _i64, _i64]),
    "hb_fused_rowparallel_form": (_i, [_vp, _i64, _i64, _i64, _i]),
    "hb_fused_rowparallel": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _f, _i, _vp]),
    "hb_column_shard": (_i, [_vp, _vp, _i64, _i64, _sz, _i, _i]),
    "hb_row_shard": (_i, [_vp, _vp, _i64, _i64, _sz, _i, _i]),
    "hb_bm_create": (_i, [_i64, _i64, _vp]),
    "hb_bm_free_manager": (_i, [_vp]),
    "hb_bm_num_free_gpu_blocks": (_i64, [_vp]),
    "hb_bm_num_free_cpu_blocks": (_i64, [_vp]),
    "hb_bm_num_prefix_cached_blocks": (_i64, [_vp]),
    "hb_bm_allocate": (_i, [_vp, _u64, _vp, _i64, _i64, _vp]),
    "hb_bm_can_allocate": (_i, [_vp, _i64]),
    "hb_bm_can_append_slot": (_i, [_vp, _u64, _i64]),
    "hb_bm_append_slot": (_i, [_vp, _u64, _i64, _vp]),
    "hb_bm_free_seq": (_i, [_vp, _u64]),
    "hb_bm_swap_out": (_i, [_vp, _u64, _vp, _vp]),
    "hb_bm_swap_in": (_i, [_vp, _u64, _vp, _vp]),
    "hb_bm_block_table": (_i64, [_vp, _u64, _vp, _i64]),
    "hb_hash_block": (_u64, [_vp, _i64]),
    "hb_num_logical_blocks": (_i64, [_i64, _i64]),
    "hb_last_block_num_filled": (_i64, [_i64, _i64]),
    "hb_slot_for_position": (_i64, [_vp, _i64, _i64]),
    "hb_engine_load": (_i, [_vp, _vp, _vp]),
    "hb_engine_create_random": (_i, [_vp, _vp, _vp, _u64, _f, _i, _vp]),
    "hb_engine_free": (_i, [_vp]),
    "hb_engine_num_layers": (_i64, [_vp]),
    "hb_engine_vocab_size": (_i64, [_vp]),
    "hb_engine_hidden_size": (_i64, [_vp]),
    "hb_engine_param_count": (_i64, [_vp]),
    "hb_engine_num_free_blocks": (_i64, [_vp]),
    "hb_engine_step_bytes": (C.c_double, [_vp, _vp, _i64]),
    "hb_engine_get_tensor": (_i64, [_vp, C.c_char_p, _vp, _i64]),
    "hb_seq_create": (_i, [_vp, _vp]),
    "hb_seq_free": (_i, [_vp, _vp]),
    "hb_seq_len": (_i64, [_vp]),
    "hb_seq_block_table": (_i64, [_vp, _vp, _i64]),
    "hb_forward": (_i, [_vp, _vp, _vp, _sz, _sz, _vp]),
    "hb_decode_batch": (_i, [_vp, _vp, _sz, _vp, _vp, _vp]),
    "hb_engine_profile_step": (_i, [_vp, _vp, _sz, _vp, _vp, _vp]),
    "hb_decode_batch_tables": (_i, [_vp, _sz, _vp, _vp, _vp, _sz, _vp, _sz, _vp, _vp]),
    "hb_forward_tables": (_i, [_vp, _vp, _sz, _sz, _vp, _sz, _vp]),
    "hb_kv_copy_blocks": (_i, [_vp, _vp, _sz]),
    "hb_forward_all_positions": (_i, [_vp, _vp, _vp, _sz, _sz, _vp]),
    "hb_seq_truncate": (_i, [_vp, _vp, _i64]),
    "hb_logits_to_probs": (_i, [_vp, _vp, _vp, _vp, _i64, _i64, _f, _f, _f, _f]),
    "hb_sample": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _f, _f, _f, _f]),
    "hb_engine_reserve_cpu_blocks": (_i, [_vp, _i64]),
    "hb_kv_swap_blocks": (_i, [_vp, _vp, _sz, _i]),
    "hb_engine_gemm_bytes": (C.c_double, [_vp, _i64]),
    "hb_engine_last_step_ms": (_f, [_vp]),
    "hb_engine_last_step_launches": (_i64, [_vp]),
    "hb_engine_stream": (_vp, [_vp]),
}

#: every symbol include/hb.h declares (tests check the library exports all of them)
DECLARED_SYMBOLS = tuple(_SIGS)

for _name, (_res, _args) in _SIGS.items():
    _fn = getattr(lib, _name)
    _fn.restype = _res
    _fn.argtypes = _args


def last_error() -> str:
    return lib.hb_last_error().decode("utf-8", "replace")


def check(rc: int) -> int:
    if rc < 0:
        raise HbError(rc, last_error())
    return rc


def device_count() -> int:
    return lib.hb_device_count()


# --------------------------------------------------------------------------- dtypes
def dtype_code(t) -> int:
    """Map a torch or numpy dtype to hb_dtype."""
    name = str(t).replace("torch.", "")
    try:
        return {"float32": F32, "float16": F16, "bfloat16": BF16}[name]
    except KeyError:
        raise HbError(ERR_UNSUPPORTED_DTYPE, f"unsupported dtype {t}") from None


def _ptr(x) -> Optional[int]:
    """Raw address of a torch tensor / numpy array / int / None."""
    if x is None:
        return None
    if isinstance(x, int):
        return x
    if isinstance(x, np.ndarray):
        return x.ctypes.data
    return x.data_ptr()


def _stream(stream=None) -> Optional[int]:
    if stream is None:
        try:
            import torch

            if torch.cuda.is_available():
                return torch.cuda.current_stream().cuda_stream
        except Exception:
            pass
        return None
    if isinstance(stream, int):
        return stream
    return stream.cuda_stream


# ------------------------------------------------------------------ kernels mirror
class kernels:
    """Mirror of src/kernels: caller-allocated outputs, torch CUDA tensors in."""

    class rms_norm:
        @staticmethod
        def apply(x, weight, eps: float, out=None, stream=None):
            """rms_norm::apply (src/kernels/rms_norm.rs:23)."""
            import torch

            hidden = x.shape[-1]
            rows = x.numel() // hidden if hidden else 0
            out = torch.empty_like(x) if out is None else out
            check(lib.hb_rms_norm(_stream(stream), _ptr(out), _ptr(x), _ptr(weight), rows, hidden,
                                  float(eps), dtype_code(x.dtype)))
            return out

        @staticmethod
        def add_apply(x, resid, weight, eps: float, stream=None):
            """Residual add + norm; returns (normed, new_residual)."""
            import torch

            hidden = x.shape[-1]
            rows = x.numel() // hidden
            normed, res = torch.empty_like(x), torch.empty_like(x)
            check(lib.hb_add_rms_norm(_stream(stream), _ptr(normed), _ptr(res), _ptr(x), _ptr(resid),
                                      _ptr(weight), rows, hidden, float(eps), dtype_code(x.dtype)))
            return normed, res

    class rope:
        @staticmethod
        def inv_freq(theta: float, head_dim: int) -> np.ndarray:
            out = np.empty(head_dim // 2, dtype=np.float32)
            check(lib.hb_rope_inv_freq(float(theta), head_dim, out.ctypes.data))
            return out

        @staticmethod
        def apply(q, k, cos, sin, stream=None):
            """rope::apply (src/kernels/rope.rs:25): q,k [b,h,s,d], cos/sin [s,d/2]."""
            import torch

            outs = []
            for x in (q, k):
                b, h, s, d = x.shape
                o = torch.empty_like(x)
                check(lib.hb_rope_cos_sin(_stream(stream), _ptr(o), _ptr(x), _ptr(cos), _ptr(sin),
                                          b * h, s, d, dtype_code(x.dtype)))
                outs.append(o)
            return outs[0], outs[1]

        @staticmethod
        def apply_positions(q, k, positions, inv_freq, stream=None):
            """In place on q [t,hq,d] and k [t,hkv,d] with per-token positions."""
            t, hq, d = q.shape
            hkv = k.shape[1] if k is not None else 0
            check(lib.hb_rope(_stream(stream), _ptr(q), _ptr(k), _ptr(positions), _ptr(inv_freq), t,
                              hq, hkv, d, dtype_code(q.dtype)))
            return q, k

    class kv_assign:
        @staticmethod
        def assign_slot(buf, src, offset: int, stream=None):
            """kv_assign::assign_slot (src/kernels/kv_assign.rs:34): buf [1,nkv,max_seq,d],
            src [1,nkv,1,d]; written in place and returned."""
            _, nkv, max_seq, d = buf.shape
            check(lib.hb_kv_assign_contig(_stream(stream), _ptr(buf), _ptr(src), nkv, max_seq, d,
                                          int(offset), dtype_code(buf.dtype)))
            return buf

        @staticmethod
        def assign_paged(k_cache, v_cache, k, v, slot_mapping, stream=None):
            num_blocks, nkv, _, d = k_cache.shape
            check(lib.hb_kv_assign_paged(_stream(stream), _ptr(k_cache), _ptr(v_cache), _ptr(k), _ptr(v),
                                         _ptr(slot_mapping), k.shape[0], nkv, d, num_blocks,
                                         dtype_code(k.dtype)))


def paged_decode_attention(q, k_cache, v_cache, block_tables, ctx_lens, n_splits: int = 1, stream=None,
                           sliding_window: int = 0):
    """q [n_seqs,hq,d]; caches [num_blocks,hkv,16,d]; block_tables int32 [n_seqs,max_blocks];
    sliding_window > 0 limits every query to its last `sliding_window` keys."""
    import torch

    n_seqs, hq, d = q.shape
    num_blocks, hkv = k_cache.shape[0], k_cache.shape[1]
    out = torch.empty_like(q)
    ws_bytes = lib.hb_attention_workspace_bytes(n_seqs, hq, d, n_splits)
    ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=q.device)
    if sliding_window:
        check(lib.hb_paged_decode_attention_window(_stream(stream), _ptr(out), _ptr(q), _ptr(k_cache), _ptr(v_cache),
                                                   _ptr(block_tables), _ptr(ctx_lens), n_seqs, hq, hkv, d,
                                                   block_tables.shape[1], num_blocks, n_splits, _ptr(ws),
                                                   sliding_window, dtype_code(q.dtype)))
        return out
    check(lib.hb_paged_decode_attention(_stream(stream), _ptr(out), _ptr(q), _ptr(k_cache), _ptr(v_cache),
                                        _ptr(block_tables), _ptr(ctx_lens), n_seqs, hq, hkv, d,
                                        block_tables.shape[1], num_blocks, n_splits, _ptr(ws),
                                        dtype_code(q.dtype)))
    return out


def moe_route(x, w_gate, top_k: int, stream=None):
    """scale [n_tokens, n_experts] f32: renormalised top-k routing weights, 0 elsewhere."""
    import torch

    n, hidden = x.shape
    n_experts = w_gate.shape[0]
    scale = torch.empty((n, n_experts), dtype=torch.float32, device=x.device)
    check(lib.hb_moe_route(_stream(stream), _ptr(scale), _ptr(x), _ptr(w_gate), n, hidden, n_experts, top_k,
                           dtype_code(x.dtype)))
    return scale


def paged_decode_attention_static(q, k_cache, v_cache, block_tables, ctx_lens, n_splits: int = 2, stream=None):
    """paged_decode_attention without any allocation by the library: the split partials
    use the array built into libhb.so (bounded size; calls must not overlap on the GPU)."""
    import torch

    n_seqs, hq, d = q.shape
    num_blocks, hkv = k_cache.shape[0], k_cache.shape[1]
    out = torch.empty_like(q)
    check(lib.hb_paged_decode_attention_static(_stream(stream), _ptr(out), _ptr(q), _ptr(k_cache), _ptr(v_cache),
                                               _ptr(block_tables), _ptr(ctx_lens), n_seqs, hq, hkv, d,
                                               block_tables.shape[1], num_blocks, n_splits, dtype_code(q.dtype)))
    return out


def gemm(x, w, stream=None):
    """y = x @ w.T with w stored [out, in]."""
    import torch

    M, K = x.shape
    N = w.shape[0]
    y = torch.empty((M, N), dtype=x.dtype, device=x.device)
    code = dtype_code(x.dtype)
    ws_bytes = lib.hb_gemm_workspace_bytes(M, N, K, code)
    ws = torch.zeros(max(ws_bytes, 16), dtype=torch.uint8, device=x.device)
    check(lib.hb_gemm(_stream(stream), _ptr(y), _ptr(x), _ptr(w), M, N, K, code, _ptr(ws)))
    return y


def gemm_ex(x, w, epilogue: int = 0, out_f32: bool = False, force_splits: int = 0, stream=None):
    """tcgen05 GEMM with a fused epilogue: 0 = store (bf16 or fp32), 1 = SwiGLU over
    w = [gate ; up] giving [M, N/2]."""
    import torch

    M, K = x.shape
    N = w.shape[0]
    n_out = N // 2 if epilogue == 1 else N
    y = torch.empty((M, n_out), dtype=torch.float32 if out_f32 else x.dtype, device=x.device)
    ws_bytes = lib.hb_gemm_ex_workspace_bytes(M, N, K, epilogue, force_splits)
    ws = torch.zeros(max(ws_bytes, 16), dtype=torch.uint8, device=x.device)
    check(lib.hb_gemm_ex(_stream(stream), _ptr(y), _ptr(x), _ptr(w), M, N, K, epilogue, int(out_f32),
                         force_splits, _ptr(ws)))
    return y


def logits_to_probs(logits, temperature: float, top_p: float = 1.0, token_counts=None, presence: float = 0.0,
                    frequency: float = 0.0, stream=None):
    """Sampling distribution of every row of `logits` (torch CUDA float32 [n, vocab])."""
    import torch

    n, vocab = logits.shape
    probs = torch.empty_like(logits)
    check(lib.hb_logits_to_probs(_stream(stream), _ptr(probs), _ptr(logits), _ptr(token_counts), n, vocab,
                                 float(temperature), float(top_p), float(presence), float(frequency)))
    return probs


def sample(logits, seeds, temperature: float, top_p: float = 1.0, token_counts=None, presence: float = 0.0,
           frequency: float = 0.0, stream=None):
    """One token per row of `logits`, drawn on the device; seeds: torch CUDA uint64/int64 [n]."""
    import torch

    n, vocab = logits.shape
    probs = torch.empty_like(logits)
    out = torch.empty(n, dtype=torch.int32, device=logits.device)
    check(lib.hb_sample(_stream(stream), _ptr(out), _ptr(probs), _ptr(logits), _ptr(token_counts), _ptr(seeds), n,
                        vocab, float(temperature), float(top_p), float(presence), float(frequency)))
    return out, probs


def silu_mul(gate_up, stream=None):
    import torch

    M, two_i = gate_up.shape
    out = torch.empty((M, two_i // 2), dtype=gate_up.dtype, device=gate_up.device)
    check(lib.hb_silu_mul(_stream(stream), _ptr(out), _ptr(gate_up), M, two_i // 2, dtype_code(gate_up.dtype)))
    return out


def embed(table, ids, stream=None):
    import torch

    out = torch.empty((ids.numel(), table.shape[1]), dtype=table.dtype, device=table.device)
    check(lib.hb_embed(_stream(stream), _ptr(out), _ptr(table), _ptr(ids), ids.numel(), table.shape[1],
                       table.shape[0], dtype_code(table.dtype)))
    return out


def argmax(logits, stream=None):
    import torch

    n, vocab = logits.shape
    out = torch.empty(n, dtype=torch.int32, device=logits.device)
    check(lib.hb_argmax(_stream(stream), _ptr(out), _ptr(logits), n, vocab, dtype_code(logits.dtype)))
    return out


# ----------------------------------------------------------------- parallel mirror
def column_shard(weight: np.ndarray, rank: int, world_size: int) -> np.ndarray:
    """column_shard (src/parallel/shard.rs:46)."""
    w = np.ascontiguousarray(weight)
    rows, cols = w.shape
    out = np.empty((rows // max(world_size, 1), cols), dtype=w.dtype)
    check(lib.hb_column_shard(out.ctypes.data, w.ctypes.data, rows, cols, w.itemsize, rank, world_size))
    return out


def row_shard(weight: np.ndarray, rank: int, world_size: int) -> np.ndarray:
    """row_shard (src/parallel/shard.rs:66)."""
    w = np.ascontiguousarray(weight)
    rows, cols = w.shape
    out = np.empty((rows, cols // max(world_size, 1)), dtype=w.dtype)
    check(lib.hb_row_shard(out.ctypes.data, w.ctypes.data, rows, cols, w.itemsize, rank, world_size))
    return out


class TpWorld:
    """One rank's side of a tensor-parallel group (TpWorld, src/parallel/world.rs)."""

    def __init__(self, handle: int, owner: bool = True):
        self.handle = handle
        self._owner = owner

    # --- constructors
    @classmethod
    def new_local(cls, n: int, device_ids: Optional[Sequence[int]] = None,
                  staging_bytes: int = 64 << 20) -> list["TpWorld"]:
        """Single-process form of TpWorld::new(n): one handle per rank."""
        arr = (C.c_void_p * n)()
        ids = (C.c_int * n)(*device_ids) if device_ids is not None else None
        check(lib.hb_world_create_local(n, ids, staging_bytes, arr))
        return [cls(arr[i]) for i in range(n)]

    @classmethod
    def new_rank(cls, world_size: int, rank: int, device: int, staging_bytes: int = 64 << 20) -> "TpWorld":
        h = C.c_void_p()
        check(lib.hb_world_create_rank(world_size, rank, device, staging_bytes, C.byref(h)))
        return cls(h.value)

    @classmethod
    def from_torch_distributed(cls, device: int, staging_bytes: int = 64 << 20, nccl: bool = False) -> "TpWorld":
        """One process per GPU: exchange the IPC handles over torch.distributed."""
        import torch.distributed as dist

        ws, rank = dist.get_world_size(), dist.get_rank()
        w = cls.new_rank(ws, rank, device, staging_bytes)
        if ws > 1:
            handles: list = [None] * ws
            dist.all_gather_object(handles, w.ipc_handle())
            w.attach(b"".join(handles))
            if nccl:
                box = [w.nccl_unique_id() if rank == 0 else None]
                dist.broadcast_object_list(box, src=0)
                w.init_nccl(box[0])
            dist.barrier()
        return w

    # --- plumbing
    def ipc_handle(self) -> bytes:
        buf = C.create_string_buffer(IPC_HANDLE_BYTES)
        check(lib.hb_world_ipc_handle(self.handle, buf))
        return buf.raw

    def attach(self, all_handles: bytes) -> None:
        check(lib.hb_world_attach(self.handle, all_handles))

    @staticmethod
    def nccl_unique_id() -> bytes:
        buf = C.create_string_buffer(NCCL_ID_BYTES)
        check(lib.hb_nccl_unique_id(buf))
        return buf.raw

    def init_nccl(self, uid: bytes) -> None:
        check(lib.hb_world_init_nccl(self.handle, uid))

    # --- TpWorld surface
    def world_size(self) -> int:
        return lib.hb_world_size(self.handle)

    def rank(self) -> int:
        return lib.hb_world_rank(self.handle)

    def device(self) -> int:
        return lib.hb_world_device(self.handle)

    def is_single(self) -> bool:
        return bool(lib.hb_world_is_single(self.handle))

    def status(self) -> int:
        return lib.hb_world_status(self.handle)

    def set_wait_limit(self, polls: int) -> None:
        """Polls after which a device-side wait on a peer flag gives up (0 = default)."""
        check(lib.hb_world_set_wait_limit(self.handle, polls))

    def enable_multicast(self, max_rows: int, hidden: int, group=None) -> str:
        """Gives the world a window for ALGO_MULTIMEM (the sum formed inside the NVLink switch).
        Collective over `group` (default: all ranks).  The window comes from torch's
        symmetric-memory allocator, which binds the ranks' allocations to one multicast
        object; returns "" on success, else why the switch reduction is unavailable (every
        rank gets the same answer).  Call disable_multicast() on every rank before the
        process group goes away."""
        import torch
        import torch.distributed as dist

        why = ""
        tensor = handle = None
        nbytes = lib.hb_world_multicast_bytes(max_rows, hidden)
        try:
            import torch.distributed._symmetric_memory as symm

            dev = torch.device("cuda", self.device())
            grp = group if group is not None else dist.group.WORLD
            tensor = symm.empty(nbytes, dtype=torch.uint8, device=dev)
            handle = symm.rendezvous(tensor, grp)
            if not int(handle.multicast_ptr):
                why = "the symmetric-memory allocation has no multicast address (no NVLink switch reduction here)"
        except Exception as exc:  # allocator or rendezvous not available in this build / on this fabric
            why = f"symmetric memory unavailable: {type(exc).__name__}: {exc}"
        # every rank must agree before anybody starts to use the window
        flags: list = [None] * dist.get_world_size(group)
        dist.all_gather_object(flags, why, group=group)
        bad = [f for f in flags if f]
        if bad:
            return bad[0]
        check(lib.hb_world_attach_multicast(self.handle, tensor.data_ptr(), int(handle.multicast_ptr), nbytes))
        self._mc = (tensor, handle, group)
        # a rank that leaves on an error still unbinds its memory before the process ends
        import atexit

        atexit.register(self.close)
        dist.barrier(group=group)
        return ""

    def has_multicast(self) -> bool:
        return bool(lib.hb_world_has_multicast(self.handle))

    def multicast_partial(self, rows: int, hidden: int, dtype):
        """The [rows, hidden] view inside the window where a row-parallel GEMM leaves its partial."""
        tensor = self._mc[0]
        off = lib.hb_world_multicast_partial(self.handle) - tensor.data_ptr()
        return tensor[off:off + rows * hidden * 2].view(dtype).view(rows, hidden)

    def disable_multicast(self, collective: bool = True) -> None:
        """Drains the device, forgets the window and releases it.  collective=True (the normal
        path): all ranks do so together, between barriers.  collective=False is for a rank that
        is about to leave on an error: it still unbinds its own memory before the process ends."""
        import torch.distributed as dist

        mc = getattr(self, "_mc", None)
        if mc is None:
            return
        check(lib.hb_world_detach_multicast(self.handle))
        if collective:
            dist.barrier(group=mc[2])
        self._mc = None
        del mc

    def all_reduce(self, buf, algo: int = ALGO_AUTO, stream=None):
        """In-place SUM over ranks of a torch CUDA tensor (TpWorld::all_reduce)."""
        check(lib.hb_all_reduce(self.handle, _stream(stream), _ptr(buf), buf.numel(),
                                dtype_code(buf.dtype), algo))
        return buf

    def all_reduce_add_rms_norm(self, partial, resid, norm_w, eps: float, algo: int = ALGO_AUTO, stream=None):
        """(normed, new_resid) = rms_norm(resid + SUM_ranks partial) in one kernel per rank."""
        import torch

        rows, hidden = partial.shape
        normed, res = torch.empty_like(resid), torch.empty_like(resid)
        check(lib.hb_all_reduce_add_rms_norm(self.handle, _stream(stream), _ptr(normed), _ptr(res), _ptr(partial),
                                             _ptr(resid), _ptr(norm_w), rows, hidden, eps, dtype_code(partial.dtype),
                                             algo))
        return normed, res

    def fused_rowparallel(self, x, w, resid, norm_w, eps: float, algo: int = ALGO_AUTO, stream=None):
        """(normed, new_resid) = fused o_proj/down_proj + all-reduce + residual + RMSNorm."""
        return fused_rowparallel(self, x, w, resid, norm_w, eps, algo, stream)

    def close(self) -> None:
        if self.handle and getattr(self, "_mc", None) is not None:
            self.disable_multicast(collective=False)
        if self.handle and self._owner:
            lib.hb_world_free(self.handle)
        self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def fused_rowparallel_workspace(x, w):
    """A zeroed workspace for fused_rowparallel; may be kept and reused across calls."""
    import torch

    M, Kl = x.shape
    n = lib.hb_fused_rowparallel_workspace_bytes(M, w.shape[0], Kl)
    return torch.zeros(max(n, 16), dtype=torch.uint8, device=x.device)


def fused_rowparallel(world, x, w, resid, norm_w, eps: float, algo: int = ALGO_AUTO, stream=None,
                      workspace=None, out=None):
    """(normed, new_resid) = rms_norm(resid + SUM_ranks x_r @ w_r.T) in one kernel per rank.
    world is a TpWorld or None (single rank)."""
    import torch

    M, Kl = x.shape
    N = w.shape[0]
    if out is None:
        out = (torch.empty((M, N), dtype=x.dtype, device=x.device), torch.empty((M, N), dtype=x.dtype, device=x.device))
    normed, res = out
    ws = workspace if workspace is not None else fused_rowparallel_workspace(x, w)
    check(lib.hb_fused_rowparallel(world.handle if world is not None else None, _stream(stream), _ptr(normed),
                                   _ptr(res), _ptr(x), _ptr(w), _ptr(resid), _ptr(norm_w), M, N, Kl, float(eps),
                                   algo, _ptr(ws)))
    return normed, res


ROWPAR_FORMS = {0: "single", 1: "push", 2: "exchange", 3: "nccl", 4: "multimem"}


def fused_rowparallel_form(world, M: int, N: int, K_local: int, algo: int = ALGO_AUTO) -> str:
    """Which form fused_rowparallel takes for this world, shape and algo."""
    return ROWPAR_FORMS[check(lib.hb_fused_rowparallel_form(world.handle if world is not None else None, M, N,
                                                            K_local, algo))]


# ---------------------------------------------------------------- scheduler mirror
class BlockManager:
    """BlockManager (src/scheduler/block_manager.rs:143-414), one sequence per group."""

    def __init__(self, num_gpu_blocks: int, num_cpu_blocks: int):
        h = C.c_void_p()
        check(lib.hb_bm_create(num_gpu_blocks, num_cpu_blocks, C.byref(h)))
        self.handle = h.value

    def num_free_gpu_blocks(self) -> int:
        return lib.hb_bm_num_free_gpu_blocks(self.handle)

    def num_free_cpu_blocks(self) -> int:
        return lib.hb_bm_num_free_cpu_blocks(self.handle)

    def num_prefix_cached_blocks(self) -> int:
        return lib.hb_bm_num_prefix_cached_blocks(self.handle)

    def can_allocate(self, total_len: int) -> bool:
        return bool(lib.hb_bm_can_allocate(self.handle, total_len))

    def allocate(self, seq_id: int, prompt_ids: Sequence[int], output_len: int = 0) -> int:
        ids = np.ascontiguousarray(np.asarray(prompt_ids, dtype=np.uint32))
        hits = C.c_int64(0)
        check(lib.hb_bm_allocate(self.handle, seq_id, ids.ctypes.data, len(ids), output_len, C.byref(hits)))
        return hits.value

    def free(self, seq_id: int) -> None:
        check(lib.hb_bm_free_seq(self.handle, seq_id))

    def can_append_slot(self, seq_id: int, total_len: int) -> bool:
        return bool(lib.hb_bm_can_append_slot(self.handle, seq_id, total_len))

    def append_slot(self, seq_id: int, total_len: int) -> list[tuple[int, int]]:
        pair = (C.c_int64 * 2)()
        check(lib.hb_bm_append_slot(self.handle, seq_id, total_len, pair))
        return [] if pair[0] < 0 else [(pair[0], pair[1])]

    def _swap(self, fn, seq_id: int) -> list[tuple[int, int]]:
        n_tab = max(lib.hb_bm_block_table(self.handle, seq_id, None, 0), 0)
        buf = (C.c_int64 * (2 * max(n_tab, 1)))()
        n = C.c_int64(0)
        check(fn(self.handle, seq_id, buf, C.byref(n)))
        return [(buf[2 * i], buf[2 * i + 1]) for i in range(n.value)]

    def swap_out(self, seq_id: int) -> list[tuple[int, int]]:
        return self._swap(lib.hb_bm_swap_out, seq_id)

    def swap_in(self, seq_id: int) -> list[tuple[int, int]]:
        return self._swap(lib.hb_bm_swap_in, seq_id)

    def get_block_table(self, seq_id: int) -> Optional[list[int]]:
        n = lib.hb_bm_block_table(self.handle, seq_id, None, 0)
        if n < 0:
            return None
        buf = (C.c_int64 * max(n, 1))()
        lib.hb_bm_block_table(self.handle, seq_id, buf, n)
        return [buf[i] for i in range(n)]

    def close(self) -> None:
        if self.handle:
            lib.hb_bm_free_manager(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def hash_block(tokens: Sequence[int]) -> int:
    ids = np.ascontiguousarray(np.asarray(tokens, dtype=np.uint32))
    return lib.hb_hash_block(ids.ctypes.data, len(ids))


# ------------------------------------------------------------------- engine mirror
class Sequence_:
    def __init__(self, engine: "Engine", handle: int):
        self.engine, self.handle = engine, handle

    def __len__(self) -> int:
        return lib.hb_seq_len(self.handle)

    def block_table(self) -> list[int]:
        n = lib.hb_seq_block_table(self.handle, None, 0)
        buf = (C.c_int64 * max(n, 1))()
        lib.hb_seq_block_table(self.handle, buf, n)
        return [buf[i] for i in range(n)]

    def free(self) -> None:
        if self.handle and self.engine.handle:
            lib.hb_seq_free(self.engine.handle, self.handle)
        self.handle = None


class Engine:
    """Engine (src/engine/loader.rs:66-339) for the TP Llama path."""

    def __init__(self, handle: int, world: Optional[TpWorld]):
        self.handle = handle
        self.world = world

    @staticmethod
    def _config(model_path: Optional[str], max_seq_len: int, bf16: bool, tp: int, num_kv_blocks: int,
                max_batch: int, force_f32: bool) -> ModelConfig:
        return ModelConfig(model_path.encode() if model_path else None, max_seq_len, 0.9, int(bf16), tp,
                           num_kv_blocks, max_batch, int(force_f32))

    @classmethod
    def load(cls, model_path: str, *, max_seq_len: int = 2048, bf16: bool = True,
             tensor_parallel_size: int = 1, world: Optional[TpWorld] = None, num_kv_blocks: int = 0,
             max_batch: int = 64, force_f32: bool = False) -> "Engine":
        cfg = cls._config(model_path, max_seq_len, bf16, tensor_parallel_size, num_kv_blocks, max_batch,
                          force_f32)
        h = C.c_void_p()
        check(lib.hb_engine_load(C.byref(cfg), world.handle if world else None, C.byref(h)))
        return cls(h.value, world)

    @classmethod
    def create_random(cls, shape: dict, *, seed: int = 1, std: float = 0.02, norm_ones: bool = True,
                      max_seq_len: int = 2048, bf16: bool = True, tensor_parallel_size: int = 1,
                      world: Optional[TpWorld] = None, num_kv_blocks: int = 0, max_batch: int = 64,
                      force_f32: bool = False) -> "Engine":
        cfg = cls._config(None, max_seq_len, bf16, tensor_parallel_size, num_kv_blocks, max_batch, force_f32)
        sh = ModelShape(shape["hidden_size"], shape["intermediate_size"], shape["num_hidden_layers"],
                        shape["num_attention_heads"], shape.get("num_key_value_heads", 0),
                        shape["vocab_size"], shape.get("rms_norm_eps", 1e-5), shape.get("rope_theta", 10000.0),
                        shape.get("num_local_experts", 0), shape.get("num_experts_per_tok", 0),
                        shape.get("sliding_window", 0))
        h = C.c_void_p()
        check(lib.hb_engine_create_random(C.byref(sh), C.byref(cfg), world.handle if world else None,
                                          seed, std, int(norm_ones), C.byref(h)))
        return cls(h.value, world)

    def num_layers(self) -> int:
        return lib.hb_engine_num_layers(self.handle)

    def vocab_size(self) -> int:
        return lib.hb_engine_vocab_size(self.handle)

    def hidden_size(self) -> int:
        return lib.hb_engine_hidden_size(self.handle)

    def param_count(self) -> int:
        return lib.hb_engine_param_count(self.handle)

    def num_free_blocks(self) -> int:
        return lib.hb_engine_num_free_blocks(self.handle)

    def step_bytes(self, ctx_lens: Sequence[int]) -> float:
        a = np.ascontiguousarray(np.asarray(ctx_lens, dtype=np.int32))
        return lib.hb_engine_step_bytes(self.handle, a.ctypes.data, len(a))

    def get_tensor(self, name: str) -> np.ndarray:
        n = check(lib.hb_engine_get_tensor(self.handle, name.encode(), None, 0))
        out = np.empty(n, dtype=np.float32)
        check(lib.hb_engine_get_tensor(self.handle, name.encode(), out.ctypes.data, n))
        return out

    def create_kv_cache(self) -> Sequence_:
        h = C.c_void_p()
        check(lib.hb_seq_create(self.handle, C.byref(h)))
        return Sequence_(self, h.value)

    def forward_with_cache(self, token_ids: Sequence[int], seq_pos: int, cache: Sequence_) -> np.ndarray:
        """Last-token logits [vocab] as float32 (Engine::forward_with_cache)."""
        ids = np.ascontiguousarray(np.asarray(token_ids, dtype=np.uint32))
        logits = np.empty(self.vocab_size(), dtype=np.float32)
        check(lib.hb_forward(self.handle, cache.handle, ids.ctypes.data, len(ids), seq_pos, logits.ctypes.data))
        return logits

    def decode_batch(self, seqs: Sequence[Sequence_], last_tokens: np.ndarray,
                     next_tokens: Optional[np.ndarray] = None, logits: Optional[np.ndarray] = None) -> np.ndarray:
        B = len(seqs)
        arr = (C.c_void_p * B)(*[s.handle for s in seqs])
        last = np.ascontiguousarray(np.asarray(last_tokens, dtype=np.uint32))
        if next_tokens is None:
            next_tokens = np.empty(B, dtype=np.uint32)
        check(lib.hb_decode_batch(self.handle, arr, B, last.ctypes.data, next_tokens.ctypes.data,
                                  logits.ctypes.data if logits is not None else None))
        return next_tokens

    # --- the step driven by a scheduler's block tables
    def decode_batch_tables(self, last_tokens, positions, block_tables, copy_pairs=(), logits=None) -> np.ndarray:
        """One decode step for rows whose KV lives in the caller's block tables
        (block_tables: int64 [B, stride], row b covers positions[b]); copy_pairs are the
        scheduler's copy-on-write (src, dst) block pairs, applied first."""
        last = np.ascontiguousarray(np.asarray(last_tokens, dtype=np.uint32))
        pos = np.ascontiguousarray(np.asarray(positions, dtype=np.int64))
        tab = np.ascontiguousarray(np.asarray(block_tables, dtype=np.int64))
        B = len(last)
        assert tab.ndim == 2 and tab.shape[0] == B and len(pos) == B
        pairs = np.ascontiguousarray(np.asarray(list(copy_pairs), dtype=np.int64).reshape(-1, 2))
        nxt = np.empty(B, dtype=np.uint32)
        check(lib.hb_decode_batch_tables(self.handle, B, last.ctypes.data, pos.ctypes.data, tab.ctypes.data, tab.shape[1],
                                         pairs.ctypes.data if len(pairs) else None, len(pairs), nxt.ctypes.data,
                                         logits.ctypes.data if logits is not None else None))
        return nxt

    def forward_tables(self, token_ids, seq_pos: int, block_table) -> np.ndarray:
        """Logits of the last of `token_ids` fed at positions seq_pos.. of the sequence that owns
        `block_table`; positions below seq_pos must already be in the table's blocks."""
        ids = np.ascontiguousarray(np.asarray(token_ids, dtype=np.uint32))
        tab = np.ascontiguousarray(np.asarray(block_table, dtype=np.int64))
        out = np.empty(self.vocab_size(), dtype=np.float32)
        check(lib.hb_forward_tables(self.handle, ids.ctypes.data, len(ids), seq_pos, tab.ctypes.data, len(tab),
                                    out.ctypes.data))
        return out

    def forward_all_positions(self, token_ids, seq_pos: int, cache: "Sequence_") -> np.ndarray:
        """Logits [n, vocab] of every fed position in one forward (speculative verification)."""
        ids = np.ascontiguousarray(np.asarray(token_ids, dtype=np.uint32))
        out = np.empty((len(ids), self.vocab_size()), dtype=np.float32)
        check(lib.hb_forward_all_positions(self.handle, cache.handle, ids.ctypes.data, len(ids), seq_pos, out.ctypes.data))
        return out

    def truncate(self, cache: "Sequence_", new_len: int) -> None:
        check(lib.hb_seq_truncate(self.handle, cache.handle, new_len))

    def kv_copy_blocks(self, pairs) -> None:
        p = np.ascontiguousarray(np.asarray(list(pairs), dtype=np.int64).reshape(-1, 2))
        check(lib.hb_kv_copy_blocks(self.handle, p.ctypes.data if len(p) else None, len(p)))

    def reserve_cpu_blocks(self, n: int) -> None:
        check(lib.hb_engine_reserve_cpu_blocks(self.handle, n))

    def kv_swap_blocks(self, pairs, to_cpu: bool) -> None:
        p = np.ascontiguousarray(np.asarray(list(pairs), dtype=np.int64).reshape(-1, 2))
        check(lib.hb_kv_swap_blocks(self.handle, p.ctypes.data if len(p) else None, len(p), 1 if to_cpu else 0))

    PROFILE_KINDS = ("gemm_qkv", "attention", "rope_kv", "norm", "other", "all_reduce",
                     "gemm_o_proj", "gemm_gate_up", "gemm_down", "gemm_lm_head")

    def profile_step(self, seqs: Sequence[Sequence_], last_tokens: np.ndarray) -> tuple[np.ndarray, dict]:
        """One eager decode step with per-kernel-kind device times (ms)."""
        B = len(seqs)
        arr = (C.c_void_p * B)(*[s.handle for s in seqs])
        last = np.ascontiguousarray(np.asarray(last_tokens, dtype=np.uint32))
        nxt = np.empty(B, dtype=np.uint32)
        ms = np.zeros(len(self.PROFILE_KINDS), dtype=np.float32)
        check(lib.hb_engine_profile_step(self.handle, arr, B, last.ctypes.data, nxt.ctypes.data, ms.ctypes.data))
        by_kind = dict(zip(self.PROFILE_KINDS, ms.tolist()))
        by_kind["gemm"] = sum(v for k, v in by_kind.items() if k.startswith("gemm_"))
        return nxt, by_kind

    def gemm_bytes(self, batch: int) -> float:
        return lib.hb_engine_gemm_bytes(self.handle, batch)

    def last_step_ms(self) -> float:
        return lib.hb_engine_last_step_ms(self.handle)

    def last_step_launches(self) -> int:
        return lib.hb_engine_last_step_launches(self.handle)

    def close(self) -> None:
        if self.handle:
            lib.hb_engine_free(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
