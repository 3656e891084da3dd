"""hb_fused_rowparallel on one rank (the "single" form: tcgen05 GEMM, then add + RMSNorm)
against the oracle sequence (src/engine/arch/llama_tp.rs:327,533-552):
partial = bf16(x . W^T); h' = bf16(resid + partial); normed = rms_norm(h'; w).
The multi-rank forms are covered on 2+ GPUs and by bench.py at every N > 1."""
import numpy as np
import pytest
import torch

from oracle import kernels_ref as K

pytestmark = pytest.mark.gpu


def host(t):
    return t.detach().float().cpu().numpy()


def rel_err(got, want):
    return float(np.max(np.abs(got.astype(np.float64) - want))) / max(float(np.max(np.abs(want))), 1e-30)


def reference(x, w, resid, nw, eps, n_ranks=1):
    """Oracle in fp64 with the reference's rounding points (bf16 partials, bf16 sum)."""
    parts = [K.round_bf16((xi.astype(np.float64) @ wi.astype(np.float64).T).astype(np.float32)) for xi, wi in zip(x, w)]
    acc = resid.astype(np.float32).copy()
    for p in parts:
        acc = acc + p
    h = K.round_bf16(acc)
    return K.rms_norm_kernel(h, nw, eps, "bf16"), h


def make(M, N, Kl, seed, cuda):
    g = torch.Generator(device="cpu").manual_seed(seed)
    x = torch.randn(M, Kl, generator=g).to(torch.bfloat16)
    w = (torch.randn(N, Kl, generator=g) * 0.02).to(torch.bfloat16)
    resid = torch.randn(M, N, generator=g).to(torch.bfloat16)
    nw = (1 + 0.1 * torch.randn(N, generator=g)).to(torch.bfloat16)
    return [t.to(cuda) for t in (x, w, resid, nw)]


@pytest.mark.parametrize("M,N,Kl", [(1, 256, 256), (8, 1024, 512), (64, 4096, 4096), (64, 4096, 14336),
                                    (128, 8192, 1024), (128, 8192, 3584), (256, 2048, 640), (17, 384, 128)])
def test_fused_single_rank(hb, cuda, M, N, Kl):
    x, w, resid, nw = make(M, N, Kl, M + N, cuda)
    assert hb.fused_rowparallel_form(None, M, N, Kl) == "single"
    normed, res = hb.fused_rowparallel(None, x, w, resid, nw, 1e-5)
    torch.cuda.synchronize()
    want_n, want_h = reference([host(x)], [host(w)], host(resid), host(nw), 1e-5)
    # the residual differs from the oracle only where a bf16 rounding of the partial flips
    assert rel_err(host(res), want_h) <= 1e-2
    assert rel_err(host(normed), want_n) <= 2e-2


def test_fused_equals_unfused_sequence(hb, cuda):
    """Same inputs through hb_gemm -> hb_add_rms_norm called one by one and through the entry
    point: identical rounding points, so the outputs agree to bf16 resolution."""
    M, N, Kl = 64, 4096, 4096
    x, w, resid, nw = make(M, N, Kl, 3, cuda)
    normed, res = hb.fused_rowparallel(None, x, w, resid, nw, 1e-5)
    part = hb.gemm(x, w)
    n2, r2 = hb.kernels.rms_norm.add_apply(part, resid, nw, 1e-5)
    assert rel_err(host(res), host(r2).astype(np.float64)) <= 8e-3
    assert rel_err(host(normed), host(n2).astype(np.float64)) <= 1.6e-2


def test_fused_reuses_workspace_and_is_deterministic(hb, cuda):
    """Back-to-back calls on one workspace give bit-identical results (split-K partials are
    summed in a fixed order)."""
    M, N, Kl = 64, 4096, 14336
    x, w, resid, nw = make(M, N, Kl, 5, cuda)
    ws = hb.fused_rowparallel_workspace(x, w)
    outs = []
    for _ in range(4):
        n, r = hb.fused_rowparallel(None, x, w, resid, nw, 1e-5, workspace=ws)
        torch.cuda.synchronize()
        outs.append((host(n), host(r)))
    for n, r in outs[1:]:
        assert np.array_equal(n, outs[0][0]) and np.array_equal(r, outs[0][1])


def test_fused_rejects_bad_arguments(hb, cuda):
    x, w, resid, nw = make(8, 256, 256, 1, cuda)
    with pytest.raises(hb.HbError):
        hb.check(hb.lib.hb_fused_rowparallel(None, None, None, None, x.data_ptr(), w.data_ptr(), resid.data_ptr(),
                                             nw.data_ptr(), 8, 256, 256, 1e-5, 0, None))
