"""Parity of every CUDA kernel behind the C ABI with the CPU oracle on seeded inputs.

Tolerances (relative to the largest |expected| of the tensor): 1e-3 in fp32 and 2e-2 in
bf16/f16 for RMSNorm / RoPE / attention / GEMM; bit-exact for the KV slot writes, the
embedding gather and argmax.
"""
import numpy as np
import pytest
import torch

from oracle import kernels_ref as K

pytestmark = pytest.mark.gpu

TORCH = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}
TOL = {"f32": 1e-3, "f16": 2e-2, "bf16": 2e-2}


def dev(a, dtype, device):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(device=device, dtype=TORCH[dtype])


def host(t):
    return t.detach().float().cpu().numpy()


def rel_err(got, want):
    scale = max(float(np.max(np.abs(want))), 1e-30)
    return float(np.max(np.abs(got.astype(np.float64) - want.astype(np.float64)))) / scale


# ----------------------------------------------------------------------- RMSNorm
@pytest.mark.parametrize("dtype", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("rows,hidden", [(1, 4), (2, 256), (3, 688), (5, 4096), (64, 8192), (2, 20000), (1, 7), (0, 64)])
def test_rms_norm(hb, cuda, dtype, rows, hidden):
    rng = np.random.default_rng(rows * 1000 + hidden)
    x = K.rnd(rng.standard_normal((rows, hidden)).astype(np.float32), dtype)
    w = K.rnd((1 + 0.1 * rng.standard_normal(hidden)).astype(np.float32), dtype)
    out = hb.kernels.rms_norm.apply(dev(x, dtype, cuda), dev(w, dtype, cuda), 1e-5)
    torch.cuda.synchronize()
    if rows == 0:
        return
    want = K.rms_norm_kernel(x, w, 1e-5, dtype)
    assert rel_err(host(out), want) <= TOL[dtype]
    # the eager form the reference uses for bf16 agrees within the same tolerance
    assert rel_err(host(out), K.rms_norm_fallback(x, w, 1e-5, dtype)) <= max(TOL[dtype], 2e-2 if dtype != "f32" else 1e-3)


def test_rms_norm_reference_kats(hb, cuda, kats):
    for case in kats["rms_norm"]:
        x = dev(np.array(case["x"]), "f32", cuda)
        w = dev(np.array(case["w"]), "f32", cuda)
        out = host(hb.kernels.rms_norm.apply(x, w, case["eps"]))
        if "expect_mean_square" in case:
            assert abs(float(np.mean(out ** 2)) - case["expect_mean_square"]) < case["tol"]
        else:
            assert np.all(np.abs(out) < case["expect_all_abs_below"])


@pytest.mark.parametrize("dtype", ["f32", "bf16"])
@pytest.mark.parametrize("rows,hidden", [(1, 256), (64, 4096), (7, 688), (3, 1001)])
def test_add_rms_norm(hb, cuda, dtype, rows, hidden):
    rng = np.random.default_rng(7)
    x = K.rnd(rng.standard_normal((rows, hidden)).astype(np.float32), dtype)
    r = K.rnd(rng.standard_normal((rows, hidden)).astype(np.float32), dtype)
    w = K.rnd((1 + 0.1 * rng.standard_normal(hidden)).astype(np.float32), dtype)
    normed, res = hb.kernels.rms_norm.add_apply(dev(x, dtype, cuda), dev(r, dtype, cuda), dev(w, dtype, cuda), 1e-5)
    want_res = K.rnd(x + r, dtype)
    assert np.array_equal(host(res), want_res)  # a single rounded add: exact
    assert rel_err(host(normed), K.rms_norm_kernel(want_res, w, 1e-5, dtype)) <= TOL[dtype]


# -------------------------------------------------------------------------- RoPE
@pytest.mark.parametrize("dtype", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("n_tok,hq,hkv,hd,theta", [(1, 8, 1, 128, 500000.0), (5, 4, 2, 64, 10000.0),
                                                   (64, 32, 8, 128, 500000.0), (3, 2, 2, 8, 10000.0)])
def test_rope_positions(hb, cuda, dtype, n_tok, hq, hkv, hd, theta):
    rng = np.random.default_rng(n_tok + hd)
    q = K.rnd(rng.standard_normal((n_tok, hq, hd)).astype(np.float32), dtype)
    k = K.rnd(rng.standard_normal((n_tok, hkv, hd)).astype(np.float32), dtype)
    pos = rng.integers(0, 1280, size=n_tok).astype(np.int32)
    inv = hb.kernels.rope.inv_freq(theta, hd)
    assert np.max(np.abs(inv - K.rope_inv_freq(theta, hd)) / K.rope_inv_freq(theta, hd)) < 1e-6
    dq, dk = dev(q, dtype, cuda), dev(k, dtype, cuda)
    hb.kernels.rope.apply_positions(dq, dk, torch.from_numpy(pos).to(cuda), torch.from_numpy(inv).to(cuda))
    cos, sin = K.rope_tables(pos, theta, hd, dtype)
    assert rel_err(host(dq), K.apply_rope(q, cos, sin, dtype)) <= TOL[dtype]
    assert rel_err(host(dk), K.apply_rope(k, cos, sin, dtype)) <= TOL[dtype]


@pytest.mark.parametrize("dtype", ["f32", "f16", "bf16"])
def test_rope_reference_layout(hb, cuda, dtype):
    """rope::apply with q,k [b,h,s,d] and pre-sliced tables [s,d/2] (src/kernels/rope.rs:25)."""
    rng = np.random.default_rng(3)
    b, h, s, d = 2, 4, 3, 64
    q = K.rnd(rng.standard_normal((b, h, s, d)).astype(np.float32), dtype)
    k = K.rnd(rng.standard_normal((b, 2, s, d)).astype(np.float32), dtype)
    cos, sin = K.rope_tables(np.arange(5, 5 + s), 10000.0, d, dtype)
    oq, ok = hb.kernels.rope.apply(dev(q, dtype, cuda), dev(k, dtype, cuda), dev(cos, dtype, cuda), dev(sin, dtype, cuda))
    assert rel_err(host(oq), K.rope_single(q, cos, sin, dtype)) <= TOL[dtype]
    assert rel_err(host(ok), K.rope_single(k, cos, sin, dtype)) <= TOL[dtype]


def test_rope_reference_kats(hb, cuda, kats):
    c = kats["rope"]["pos0_pos1_differ"]
    inv = torch.from_numpy(hb.kernels.rope.inv_freq(c["theta"], c["shape"][2])).to(cuda)
    outs = []
    for p in (0, 1):
        q = torch.full(c["shape"], c["fill"], device=cuda)
        hb.kernels.rope.apply_positions(q, None, torch.tensor([p], dtype=torch.int32, device=cuda), inv)
        assert list(q.shape) == c["shape"]
        outs.append(host(q))
    assert not np.array_equal(outs[0], outs[1])
    assert np.array_equal(outs[0], np.full(c["shape"], c["fill"], dtype=np.float32))


# ---------------------------------------------------------------------- KV writes
@pytest.mark.parametrize("dtype", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("nkv,max_seq,hd,offset", [(8, 2048, 128, 0), (8, 2048, 128, 2047), (2, 64, 64, 17), (3, 10, 6, 4), (1, 1, 2, 0)])
def test_kv_assign_contig_bit_exact(hb, cuda, dtype, nkv, max_seq, hd, offset):
    rng = np.random.default_rng(11)
    buf = K.rnd(rng.standard_normal((nkv, max_seq, hd)).astype(np.float32), dtype)
    src = K.rnd(rng.standard_normal((nkv, hd)).astype(np.float32), dtype)
    dbuf = dev(buf, dtype, cuda).reshape(1, nkv, max_seq, hd)
    out = hb.kernels.kv_assign.assign_slot(dbuf, dev(src, dtype, cuda).reshape(1, nkv, 1, hd), offset)
    assert np.array_equal(host(out).reshape(nkv, max_seq, hd), K.kv_slot_assign(buf, src, offset))


def test_kv_assign_contig_rejects_bad_offset(hb, cuda):
    buf = torch.zeros(1, 2, 8, 16, device=cuda)
    src = torch.zeros(1, 2, 1, 16, device=cuda)
    with pytest.raises(hb.HbError):
        hb.kernels.kv_assign.assign_slot(buf, src, 8)


@pytest.mark.parametrize("dtype", ["f32", "bf16"])
@pytest.mark.parametrize("nkv,hd,n_tok", [(8, 128, 64), (1, 128, 128), (2, 64, 5), (3, 6, 4)])
def test_kv_assign_paged_bit_exact(hb, cuda, dtype, nkv, hd, n_tok):
    rng = np.random.default_rng(5)
    num_blocks = 40
    kc = K.rnd(rng.standard_normal((num_blocks, nkv, 16, hd)).astype(np.float32), dtype)
    vc = K.rnd(rng.standard_normal((num_blocks, nkv, 16, hd)).astype(np.float32), dtype)
    k = K.rnd(rng.standard_normal((n_tok, nkv, hd)).astype(np.float32), dtype)
    v = K.rnd(rng.standard_normal((n_tok, nkv, hd)).astype(np.float32), dtype)
    slots = rng.permutation(num_blocks * 16)[:n_tok].astype(np.int64)
    slots[0] = -1  # skipped token
    dkc, dvc = dev(kc, dtype, cuda), dev(vc, dtype, cuda)
    hb.kernels.kv_assign.assign_paged(dkc, dvc, dev(k, dtype, cuda), dev(v, dtype, cuda), torch.from_numpy(slots).to(cuda))
    assert np.array_equal(host(dkc), K.kv_assign_paged(kc, k, slots))
    assert np.array_equal(host(dvc), K.kv_assign_paged(vc, v, slots))


# --------------------------------------------------------------------- attention
def oracle_attention(q, kc, vc, tables, ctx, hkv):
    """softmax(q k^T / sqrt d) v per sequence over its block table, fp64
    (src/engine/arch/llama_tp.rs:264-324; query head j uses kv head j // n_rep)."""
    n_seqs, hq, d = q.shape
    n_rep = hq // hkv
    out = np.zeros_like(q, dtype=np.float64)
    for s in range(n_seqs):
        n = int(ctx[s])
        if n == 0:
            continue
        blocks = tables[s, :(n + 15) // 16]
        Ks = kc[blocks].transpose(1, 0, 2, 3).reshape(hkv, -1, d)[:, :n].astype(np.float64)
        Vs = vc[blocks].transpose(1, 0, 2, 3).reshape(hkv, -1, d)[:, :n].astype(np.float64)
        for j in range(hq):
            g = j // n_rep
            sc = Ks[g] @ q[s, j].astype(np.float64) / np.sqrt(d)
            p = np.exp(sc - sc.max())
            p /= p.sum()
            out[s, j] = p @ Vs[g]
    return out


@pytest.mark.parametrize("dtype", ["f32", "bf16", "f16"])
@pytest.mark.parametrize("hq,hkv,hd", [(4, 2, 64), (32, 8, 128), (8, 1, 128), (2, 2, 64), (4, 1, 128)])
@pytest.mark.parametrize("n_splits", [1, 3])
def test_paged_decode_attention(hb, cuda, dtype, hq, hkv, hd, n_splits):
    rng = np.random.default_rng(hq * 100 + hd + n_splits)
    n_seqs, num_blocks, max_blocks = 5, 96, 24
    ctx = np.array([1, 16, 17, 300, 383], dtype=np.int32)  # ragged, block edges, > one softmax chunk
    q = K.rnd(rng.standard_normal((n_seqs, hq, hd)).astype(np.float32), dtype)
    kc = K.rnd(rng.standard_normal((num_blocks, hkv, 16, hd)).astype(np.float32), dtype)
    vc = K.rnd(rng.standard_normal((num_blocks, hkv, 16, hd)).astype(np.float32), dtype)
    tables = np.stack([rng.permutation(num_blocks)[:max_blocks] for _ in range(n_seqs)]).astype(np.int32)
    out = hb.paged_decode_attention(dev(q, dtype, cuda), dev(kc, dtype, cuda), dev(vc, dtype, cuda),
                                    torch.from_numpy(tables).to(cuda), torch.from_numpy(ctx).to(cuda), n_splits)
    want = oracle_attention(q, kc, vc, tables, ctx, hkv)
    assert rel_err(host(out), want.astype(np.float32)) <= TOL[dtype]


def test_paged_attention_ignores_garbage_past_context(hb, cuda):
    """Slots beyond ctx_len may hold NaN; they must not reach the output."""
    hq, hkv, hd = 4, 2, 64
    q = torch.randn(1, hq, hd, device=cuda)
    kc = torch.randn(4, hkv, 16, hd, device=cuda)
    vc = torch.randn(4, hkv, 16, hd, device=cuda)
    tables = torch.tensor([[2, 1, 0, 3]], dtype=torch.int32, device=cuda)
    ctx = torch.tensor([20], dtype=torch.int32, device=cuda)
    ref = host(hb.paged_decode_attention(q, kc, vc, tables, ctx))
    kc[1, :, 4:] = float("nan")
    vc[1, :, 4:] = float("nan")
    got = host(hb.paged_decode_attention(q, kc, vc, tables, ctx))
    assert np.array_equal(got, ref) and np.all(np.isfinite(got))


@pytest.mark.parametrize("dtype,hq,hkv,hd", [("bf16", 8, 2, 128), ("f32", 4, 2, 64)])
def test_paged_attention_context_at_table_capacity(hb, cuda, dtype, hq, hkv, hd):
    """A context that fills its table row to the last slot (ctx == max_blocks * 16) is read in
    full; a context CLAIMED longer than the row can describe is cut to the row, so that the
    next sequence's table entries are never taken for this sequence's blocks."""
    rng = np.random.default_rng(3)
    n_seqs, num_blocks, max_blocks = 3, 40, 4
    q = K.rnd(rng.standard_normal((n_seqs, hq, hd)).astype(np.float32), dtype)
    kc = K.rnd(rng.standard_normal((num_blocks, hkv, 16, hd)).astype(np.float32), dtype)
    vc = K.rnd(rng.standard_normal((num_blocks, hkv, 16, hd)).astype(np.float32), dtype)
    tables = np.stack([rng.permutation(num_blocks)[:max_blocks] for _ in range(n_seqs)]).astype(np.int32)
    full = np.array([max_blocks * 16, 5, max_blocks * 16], dtype=np.int32)
    args = (dev(q, dtype, cuda), dev(kc, dtype, cuda), dev(vc, dtype, cuda), torch.from_numpy(tables).to(cuda))
    for n_splits in (1, 2):
        got = host(hb.paged_decode_attention(*args, torch.from_numpy(full).to(cuda), n_splits))
        want = oracle_attention(q, kc, vc, tables, full, hkv)
        assert rel_err(got, want.astype(np.float32)) <= TOL[dtype]
        claimed = np.array([max_blocks * 16 + 40, 5, 10 ** 6], dtype=np.int32)   # host-validated: cut, not followed
        cut = host(hb.paged_decode_attention(*args, torch.from_numpy(claimed).to(cuda), n_splits))
        assert np.array_equal(cut, got)


# -------------------------------------------------------------------------- GEMM
@pytest.mark.parametrize("M,N,K_", [(1, 256, 256), (8, 1024, 512), (64, 4096, 4096), (64, 6144, 4096), (33, 1000, 320),
                                    (128, 8192, 1024), (256, 512, 3584), (1, 128, 64), (17, 8, 64), (300, 256, 128),
                                    # one rank's projections of the 70B shape at TP=4
                                    (128, 2560, 8192), (128, 8192, 2048), (128, 8192, 7168)])
def test_gemm_bf16_tensor_core(hb, cuda, M, N, K_):
    """bf16, K % 64 == 0: the tcgen05 path.  fp32 reference of the same op in torch."""
    g = torch.Generator(device="cpu").manual_seed(M * 7 + N)
    x = torch.randn(M, K_, generator=g).to(cuda, torch.bfloat16)
    w = (torch.randn(N, K_, generator=g) * 0.02).to(cuda, torch.bfloat16)
    y = hb.gemm(x, w)
    torch.cuda.synchronize()
    want = (x.float() @ w.float().T).cpu().numpy()
    assert rel_err(host(y), want) <= 2e-2
    # accumulation is fp32: only the final bf16 rounding separates the two
    assert rel_err(host(y), K.round_bf16(want)) <= 4e-3


@pytest.mark.parametrize("dtype", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("M,N,K_", [(1, 32000, 256), (8, 688, 256), (5, 256, 688), (3, 7, 5)])
def test_gemm_simt_shapes(hb, cuda, dtype, M, N, K_):
    rng = np.random.default_rng(M + N + K_)
    x = K.rnd(rng.standard_normal((M, K_)).astype(np.float32), dtype)
    w = K.rnd((0.02 * rng.standard_normal((N, K_))).astype(np.float32), dtype)
    y = hb.gemm(dev(x, dtype, cuda), dev(w, dtype, cuda))
    want = x.astype(np.float64) @ w.astype(np.float64).T
    assert rel_err(host(y), want.astype(np.float32)) <= TOL[dtype]


def test_gemm_is_deterministic(hb, cuda):
    x = torch.randn(64, 14336, device=cuda).to(torch.bfloat16)
    w = (torch.randn(4096, 14336, device=cuda) * 0.02).to(torch.bfloat16)
    a = host(hb.gemm(x, w))
    b = host(hb.gemm(x, w))
    assert np.array_equal(a, b)  # split-K partials are summed in a fixed order


# ------------------------------------------------------------------ small pieces
@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_silu_mul(hb, cuda, dtype):
    rng = np.random.default_rng(2)
    gu = K.rnd(rng.standard_normal((5, 2 * 688)).astype(np.float32) * 3, dtype)
    out = hb.silu_mul(dev(gu, dtype, cuda))
    want = K.silu(gu[:, :688].astype(np.float64)) * gu[:, 688:]
    assert rel_err(host(out), want.astype(np.float32)) <= TOL[dtype]


def test_embed_bit_exact(hb, cuda):
    rng = np.random.default_rng(4)
    table = K.rnd(rng.standard_normal((1000, 256)).astype(np.float32), "bf16")
    ids = rng.integers(0, 1000, size=17).astype(np.int64)
    out = hb.embed(dev(table, "bf16", cuda), torch.from_numpy(ids.astype(np.int32)).to(cuda))
    assert np.array_equal(host(out), table[ids])


def test_argmax_first_maximum(hb, cuda):
    rng = np.random.default_rng(9)
    x = rng.standard_normal((6, 128256)).astype(np.float32)
    x[0, 5] = x[0, 77777] = 50.0       # tie -> lowest index
    x[1, 128255] = 60.0                # last element
    x[2, :] = -1.0                     # all equal -> 0
    got = hb.argmax(torch.from_numpy(x).to(cuda)).cpu().numpy()
    assert got.tolist() == np.argmax(x, axis=1).tolist()


@pytest.mark.parametrize("M,I,K_", [(16, 1024, 512), (64, 14336, 4096), (128, 3584, 8192), (128, 7168, 8192),
                                    (5, 688, 256)])
@pytest.mark.parametrize("splits", [0, 1, 3])
def test_gemm_swiglu_epilogue(hb, cuda, M, I, K_, splits):
    """gate, up, SiLU and the product in the GEMM epilogue == the unfused sequence
    (src/engine/arch/llama_tp.rs:333-338)."""
    g = torch.Generator(device="cpu").manual_seed(I)
    x = torch.randn(M, K_, generator=g).to(cuda, torch.bfloat16)
    w = (torch.randn(2 * I, K_, generator=g) * 0.05).to(cuda, torch.bfloat16)
    y = hb.gemm_ex(x, w, epilogue=1, force_splits=splits)
    gu = x.float() @ w.float().T
    want = (torch.nn.functional.silu(gu[:, :I]) * gu[:, I:]).cpu().numpy()
    assert rel_err(host(y), want) <= 2e-2


@pytest.mark.parametrize("M,N,K_,splits", [(16, 2048, 512, 0), (64, 128256, 4096, 0), (16, 2048, 512, 2), (1, 384, 1024, 4)])
def test_gemm_fp32_output(hb, cuda, M, N, K_, splits):
    """The logits GEMM keeps the fp32 accumulator (no bf16 rounding of the result)."""
    g = torch.Generator(device="cpu").manual_seed(N)
    x = torch.randn(M, K_, generator=g).to(cuda, torch.bfloat16)
    w = (torch.randn(N, K_, generator=g) * 0.02).to(cuda, torch.bfloat16)
    y = hb.gemm_ex(x, w, epilogue=0, out_f32=True, force_splits=splits)
    assert y.dtype == torch.float32
    want = (x.float() @ w.float().T).cpu().numpy()
    assert rel_err(host(y), want) <= 1e-3


def test_gemm_shared_workspace_between_shapes(hb, cuda):
    """Plans of different shapes may share one zero-initialised workspace back to back
    (the decode step does): counters are left zeroed in a fixed place."""
    shapes = [(16, 768, 512), (16, 2048, 512), (16, 512, 1024), (16, 2048, 512)]
    code = hb.BF16
    need = max(hb.lib.hb_gemm_ex_workspace_bytes(M, N, K_, 0, 2) for M, N, K_ in shapes)
    ws = torch.zeros(need, dtype=torch.uint8, device=cuda)
    for i, (M, N, K_) in enumerate(shapes * 2):
        x = torch.randn(M, K_, device=cuda).to(torch.bfloat16)
        w = (torch.randn(N, K_, device=cuda) * 0.02).to(torch.bfloat16)
        y = torch.empty(M, N, device=cuda, dtype=torch.bfloat16)
        hb.check(hb.lib.hb_gemm_ex(None, y.data_ptr(), x.data_ptr(), w.data_ptr(), M, N, K_, 0, 0, 2, ws.data_ptr()))
        torch.cuda.synchronize()
        assert rel_err(host(y), (x.float() @ w.float().T).cpu().numpy()) <= 2e-2, (i, M, N, K_)
