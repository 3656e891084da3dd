"""CPU oracle for the tensor-parallel decode hot path of vllm-hb.

TEST INFRASTRUCTURE ONLY.  These modules restate, in NumPy, the reference's algorithm
for the path (every function cites the reference file:line it follows).  They exist to
check the CUDA library; nothing in the product may import them.  Allowed importers:
``tests/``, ``__graft_entry__.smoke()`` and the ``cpu_baseline`` / ``--impl reference``
legs of ``bench.py``.

Pinning: the reference is Rust on top of the candle crates (candle-core /-nn
/-transformers 0.10.2, Cargo.lock); neither a Rust toolchain nor those crates exist
here, so the reference itself cannot be run.  The restatement is pinned against every
known-answer test the reference's own test modules hold for this path
(tests/golden/reference_kats.json, transcribed from src/parallel/comm.rs:197-284,
src/parallel/shard.rs:114-272, src/engine/arch/llama_tp.rs:613-723,
src/scheduler/block_manager.rs:418-506, src/scheduler/sequence.rs:138-195,
src/scheduler/prefix_cache.rs:141-221).  What those tests do not reach — GEMM,
softmax/attention, SwiGLU, logits, greedy tokens — is "parity unpinned" by the
reference and is cross-checked against an independent torch fp32 implementation of
the same formulas instead.
"""
