"""hb_paged_decode_attention_static — split-KV decode attention for hosts that may not
allocate GPU memory once they are running (a serving loop with a frozen memory plan, a
runtime that owns the allocator and hands out none of it to libraries).  Its split
partials live in an 8 MiB array inside the library instead of a caller workspace.

The file sorts last on purpose: if it fails under `-x`, every other test has run.
It passes alone in a fresh process and after the rest of the suite (the array keeps
the previous call's bytes; nothing in it needs to start clean).
"""
import numpy as np
import pytest
import torch

from tests.test_gpu_kernels import oracle_attention

pytestmark = pytest.mark.gpu


def make_case(cuda, seed, n_seqs=6, hq=32, hkv=8, hd=128, num_blocks=160, max_blocks=24):
    g = torch.Generator(device="cpu").manual_seed(seed)
    q = torch.randn(n_seqs, hq, hd, generator=g).to(cuda, torch.bfloat16)
    kc = torch.randn(num_blocks, hkv, 16, hd, generator=g).to(cuda, torch.bfloat16)
    vc = torch.randn(num_blocks, hkv, 16, hd, generator=g).to(cuda, torch.bfloat16)
    tables = torch.stack([torch.randperm(num_blocks, generator=g)[:max_blocks] for _ in range(n_seqs)]).to(cuda, torch.int32)
    ctx = torch.tensor([1, 16, 17, 200, 383, 384][:n_seqs], dtype=torch.int32, device=cuda)
    return q, kc, vc, tables, ctx


def test_static_scratch_matches_workspace_entry_point_twice(hb, cuda):
    """Two calls in a row through the C ABI, each checked against the existing entry
    point on the same inputs (same kernels, so within the 2e-2 bf16 tolerance of the
    attention tests — in fact bit-identical)."""
    for call, (seed, n_splits) in enumerate([(11, 4), (12, 3)]):
        q, kc, vc, tables, ctx = make_case(cuda, seed)
        want = hb.paged_decode_attention(q, kc, vc, tables, ctx, n_splits=n_splits)
        got = hb.paged_decode_attention_static(q, kc, vc, tables, ctx, n_splits=n_splits)
        torch.cuda.synchronize()
        w, g_ = want.float().cpu().numpy(), got.float().cpu().numpy()
        assert np.all(np.isfinite(g_)), call
        err = float(np.max(np.abs(g_ - w))) / float(np.max(np.abs(w)))
        assert err <= 2e-2, (call, err)
        assert np.array_equal(g_, w), call
        # ... and against the fp64 oracle of the attention tests, so that the two entry points
        # cannot be wrong together
        truth = oracle_attention(q.float().cpu().numpy(), kc.float().cpu().numpy(), vc.float().cpu().numpy(),
                                 tables.cpu().numpy(), ctx.cpu().numpy(), kc.shape[1])
        assert float(np.max(np.abs(g_ - truth))) / float(np.max(np.abs(truth))) <= 2e-2, call


def test_static_scratch_single_split_and_size_limit(hb, cuda):
    q, kc, vc, tables, ctx = make_case(cuda, 13)
    want = hb.paged_decode_attention(q, kc, vc, tables, ctx, n_splits=1)
    got = hb.paged_decode_attention_static(q, kc, vc, tables, ctx, n_splits=1)
    assert torch.equal(want, got)
    cap = hb.lib.hb_paged_decode_attention_static_max_bytes()
    assert cap == 8 << 20
    # 4096 sequences x 32 heads x 8 splits x 130 floats is far beyond the built-in array
    n_big = 4096
    assert hb.lib.hb_attention_workspace_bytes(n_big, 32, 128, 8) > cap
    with pytest.raises(hb.HbError) as ei:
        hb.check(hb.lib.hb_paged_decode_attention_static(
            None, q.data_ptr(), q.data_ptr(), kc.data_ptr(), vc.data_ptr(), tables.data_ptr(), ctx.data_ptr(),
            n_big, 32, 8, 128, tables.shape[1], kc.shape[0], 8, hb.BF16))
    assert ei.value.code == hb.ERR_INVALID_ARG and "built-in array" in ei.value.msg
