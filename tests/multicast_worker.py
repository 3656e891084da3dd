"""One rank of the switch-reduction checks (launched by tests/test_gpu_multicast.py through
torch.distributed.run, one process per GPU).  Every rank runs every case; failures are
collected, not raised, so that all ranks reach the orderly teardown (no rank may end while
its memory is bound to the multicast object).  Rank 0 prints one line `RESULT {json}`."""
import json
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, os.environ["HB_ROOT"])
import __graft_entry__ as entry  # noqa: E402
from oracle import kernels_ref as K  # noqa: E402


def host(t):
    return t.detach().float().cpu().numpy()


def time_graph(fn, calls=24, reps=4):
    g = torch.cuda.CUDAGraph()
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        for _ in range(2):
            fn(torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        dist.barrier()
        with torch.cuda.graph(g, stream=s):
            for _ in range(calls):
                fn(torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    dist.barrier()
    g.replay()
    torch.cuda.synchronize()
    dist.barrier()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(reps):
        g.replay()
    b.record()
    torch.cuda.synchronize()
    us = torch.tensor([a.elapsed_time(b) * 1e3 / (reps * calls)], device="cuda")
    dist.all_reduce(us, op=dist.ReduceOp.MAX)
    return float(us.item())


def main():
    hb = entry.load_package()
    dist.init_process_group("nccl")
    rank, ws = dist.get_rank(), dist.get_world_size()
    dev = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(dev)
    cuda = torch.device("cuda", dev)
    world = hb.TpWorld.from_torch_distributed(dev, staging_bytes=64 << 20, nccl=True)
    out = {"ranks": ws, "errors": [], "cases": [], "timing": []}
    why = world.enable_multicast(256, 8192)
    if why:
        out["unavailable"] = why
    else:
        try:
            run_cases(hb, world, rank, ws, cuda, out)
        except Exception as exc:  # keep going to the teardown
            out["errors"].append(f"rank {rank}: {type(exc).__name__}: {exc}")
        torch.cuda.synchronize()
        dist.barrier()
        world.disable_multicast()
    gathered = [None] * ws
    dist.all_gather_object(gathered, out["errors"])
    out["errors"] = [e for errs in gathered for e in errs]
    if rank == 0:
        print("RESULT " + json.dumps(out), flush=True)
    dist.barrier()
    world.close()
    dist.destroy_process_group()


def run_cases(hb, world, rank, ws, cuda, out):
    bf = torch.bfloat16
    for M, N in [(1, 8192), (7, 4096), (64, 8192), (128, 8192), (256, 1024), (33, 8192)]:
        parts = [K.rnd(np.random.default_rng(10 + r).standard_normal((M, N)).astype(np.float32), "bf16") for r in range(ws)]
        resid = K.rnd(np.random.default_rng(4).standard_normal((M, N)).astype(np.float32), "bf16")
        nw = K.rnd((1.0 + 0.1 * np.random.default_rng(5).standard_normal(N)).astype(np.float32), "bf16")
        part = torch.from_numpy(parts[rank]).to(cuda, bf)
        res_in = torch.from_numpy(resid).to(cuda, bf)
        w_t = torch.from_numpy(nw).to(cuda, bf)
        acc = np.zeros((M, N), dtype=np.float32)
        for p_ in parts:
            acc = acc + p_
        want_h = K.rnd(resid + K.rnd(acc, "bf16"), "bf16")
        for rep in range(3):  # repeated calls reuse the window; row counts vary between cases
            normed, h = world.all_reduce_add_rms_norm(part, res_in, w_t, 1e-5, hb.ALGO_MULTIMEM)
            torch.cuda.synchronize()
            err = float(np.max(np.abs(host(h) - want_h))) / float(np.max(np.abs(want_h)))
            # the switch's order of addition is its own: one bf16 rounding step of the sum
            if err > 2e-2:
                out["errors"].append(f"rank {rank} M={M} N={N} rep {rep}: residual off by {err:.4f}")
            # the normalised row is rms_norm of the new residual, bit for bit
            ref = torch.empty_like(h)
            hb.check(hb.lib.hb_rms_norm(None, ref.data_ptr(), h.data_ptr(), w_t.data_ptr(), M, N, 1e-5, hb.BF16))
            torch.cuda.synchronize()
            if not torch.equal(ref, normed):
                out["errors"].append(f"rank {rank} M={M} N={N} rep {rep}: normalised row differs from hb_rms_norm")
            # all ranks hold the same rows
            mine = h.view(torch.int16).to(torch.int64).sum().reshape(1)
            lo, hi = mine.clone(), mine.clone()
            dist.all_reduce(lo, op=dist.ReduceOp.MIN)
            dist.all_reduce(hi, op=dist.ReduceOp.MAX)
            if int(lo) != int(hi):
                out["errors"].append(f"rank {rank} M={M} N={N} rep {rep}: ranks differ")
        # against the peer-memory kernel: same sums up to the order of addition
        normed2, h2 = world.all_reduce_add_rms_norm(part, res_in, w_t, 1e-5, hb.ALGO_AUTO)
        torch.cuda.synchronize()
        d = float((h.float() - h2.float()).abs().max()) / float(h2.float().abs().max())
        out["cases"].append({"M": M, "N": N, "max_rel_vs_oracle": err, "max_rel_vs_peer_kernel": d})
        if world.status() != 0:
            out["errors"].append(f"rank {rank} M={M} N={N}: world status {world.status()}")
    # the fused row-parallel projection through the window against GEMM -> NCCL -> add + norm
    M, N, Kl = 64, 8192, 1024
    g = torch.Generator(device="cpu").manual_seed(100 + rank)
    x = torch.randn(M, Kl, generator=g).to(cuda, bf)
    w = (torch.randn(N, Kl, generator=g) * 0.02).to(cuda, bf)
    g0 = torch.Generator(device="cpu").manual_seed(7)
    res_in = torch.randn(M, N, generator=g0).to(cuda, bf)
    w_t = (1.0 + 0.1 * torch.randn(N, generator=g0)).to(cuda, bf)
    form = hb.fused_rowparallel_form(world, M, N, Kl, hb.ALGO_MULTIMEM)
    n1, h1 = hb.fused_rowparallel(world, x, w, res_in, w_t, 1e-5, hb.ALGO_MULTIMEM)
    n0, h0 = hb.fused_rowparallel(world, x, w, res_in, w_t, 1e-5, hb.ALGO_NCCL)
    torch.cuda.synchronize()
    d = float((h1.float() - h0.float()).abs().max()) / float(h0.float().abs().max())
    out["rowparallel"] = {"form": form, "max_rel_vs_nccl": d}
    if form != "multimem" or d > 2e-2:
        out["errors"].append(f"rank {rank}: fused row-parallel form {form}, off by {d:.4f}")
    # a small tensor-parallel engine on this world (its row-parallel GEMMs write into the window
    # and announce their completion themselves) against the oracle: the checks bench.py makes
    import bench

    par = bench.tp_parity(hb, world, rank, ws, cuda)
    out["tp_parity"] = par
    if rank == 0 and not par.get("ok", False):
        out["errors"].append(f"tensor-parallel engine through the window: {par}")
    # prefill in chunks (row counts 16, 16, 5: the exchange's calls differ in size) followed by
    # decode steps, against the same tokens fed one by one: the two paths must agree
    shape = dict(hidden_size=1024, intermediate_size=2048, num_hidden_layers=2, num_attention_heads=8,
                 num_key_value_heads=8, vocab_size=2048, rms_norm_eps=1e-5, rope_theta=500000.0)
    eng = hb.Engine.create_random(shape, seed=5, std=0.02, norm_ones=True, max_seq_len=64, bf16=True,
                                  tensor_parallel_size=ws, world=world, max_batch=16)
    ids = np.random.default_rng(3).integers(0, shape["vocab_size"], size=40).astype(np.uint32)
    a, b = eng.create_kv_cache(), eng.create_kv_cache()
    la = eng.forward_with_cache(ids[:37], 0, a)
    for t in range(37):
        lb = eng.forward_with_cache(ids[t:t + 1], t, b)
    d0 = float(np.max(np.abs(la - lb))) / float(np.max(np.abs(lb)))
    for t in range(37, 40):
        la = eng.forward_with_cache(ids[t:t + 1], t, a)
        lb = eng.forward_with_cache(ids[t:t + 1], t, b)
    d1 = float(np.max(np.abs(la - lb))) / float(np.max(np.abs(lb)))
    out["prefill_vs_stepwise"] = {"after_prefill": d0, "after_decode": d1}
    if max(d0, d1) > 2e-2 or world.status() != 0:
        out["errors"].append(f"rank {rank}: chunked prefill through the window differs from stepwise by {d0:.4f}/{d1:.4f}, status {world.status()}")
    a.free(); b.free(); eng.close()
    # time of the exchange alone, inside CUDA graphs: switch reduction against the peer-memory kernel
    N = 8192
    for M in (1, 8, 64, 128, 256):
        part = torch.randn(M, N, device=cuda).to(bf)
        res_in = torch.randn(M, N, device=cuda).to(bf)
        w_t = torch.ones(N, device=cuda, dtype=bf)
        normed, h = torch.empty_like(part), torch.empty_like(part)
        win = world.multicast_partial(M, N, bf)
        win.copy_(part)

        def call(algo, src):
            def fn(st):
                hb.check(hb.lib.hb_all_reduce_add_rms_norm(world.handle, st, normed.data_ptr(), h.data_ptr(), src.data_ptr(),
                                                           res_in.data_ptr(), w_t.data_ptr(), M, N, 1e-5, hb.BF16, algo))
            return fn

        out["timing"].append({"M": M, "multimem_us": time_graph(call(hb.ALGO_MULTIMEM, win)),
                              "peer_kernel_us": time_graph(call(hb.ALGO_AUTO, part))})


if __name__ == "__main__":
    main()
