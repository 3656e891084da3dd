"""Host-side model of the exchange protocol (tests/protocol_model.cc): C++ threads as ranks,
atomics as the peer flags.  Checks on the CPU what cannot be provoked on a GPU without a
fault: adversarial scheduling of back-to-back collectives over the shared staging area, a
rank that never arrives, a rank whose sequence number lags (the reference has no such
protocol: its NCCL calls either all return or one returns an Err,
src/parallel/comm.rs:113-143)."""
import json
import shutil
import subprocess
from pathlib import Path

import pytest

SRC = Path(__file__).resolve().parent / "protocol_model.cc"
SRC_MULTIMEM = Path(__file__).resolve().parent / "multimem_model.cc"


def compile_model(out_dir: Path, tsan: bool, src: Path = SRC) -> Path | None:
    gxx = shutil.which("g++")
    if gxx is None:
        pytest.skip("no g++")
    exe = out_dir / (src.stem + ("_tsan" if tsan else ""))
    cmd = [gxx, "-std=c++17", "-O1", "-g", "-pthread", str(src), "-o", str(exe)]
    if tsan:
        cmd.insert(1, "-fsanitize=thread")
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        if tsan:
            return None  # the sanitizer runtime is not installed everywhere
        raise AssertionError(res.stderr)
    return exe


@pytest.fixture(scope="module")
def model(tmp_path_factory):
    return compile_model(tmp_path_factory.mktemp("protocol_model"), tsan=False)


def run(exe, *args, timeout=120):
    res = subprocess.run([str(exe), *map(str, args)], capture_output=True, text=True, timeout=timeout)
    line = json.loads(res.stdout.strip().splitlines()[-1]) if res.stdout.strip() else {}
    return res.returncode, line, res.stderr


@pytest.mark.parametrize("ranks,rows,calls", [(2, 4, 50), (4, 8, 30), (8, 16, 12)])
def test_back_to_back_collectives_under_jitter(model, ranks, rows, calls):
    for seed in (1, 2, 3):
        rc, line, err = run(model, "normal", ranks, rows, calls, seed)
        assert rc == 0, (line, err)
        assert line["wrong_words"] == 0 and line["timeouts"] == 0


@pytest.mark.parametrize("ranks", [2, 8])
def test_absent_rank_times_everybody_out(model, ranks):
    rc, line, err = run(model, "absent", ranks, 4)
    assert rc == 0, (line, err)
    assert line["ranks_timed_out"] == ranks - 1      # all who called gave up and reported it


@pytest.mark.parametrize("ranks", [2, 4])
def test_stale_sequence_number_is_reported(model, ranks):
    rc, line, err = run(model, "stale", ranks, 4)
    assert rc == 0, (line, err)
    assert line["ranks_timed_out"] >= ranks - 1


def test_no_data_race_under_thread_sanitizer(tmp_path):
    exe = compile_model(tmp_path, tsan=True)
    if exe is None:
        pytest.skip("g++ has no thread-sanitizer runtime here")
    rc, line, err = run(exe, "normal", 4, 4, 10, 7, timeout=300)
    if "FATAL: ThreadSanitizer" in err or "unexpected memory mapping" in err:
        pytest.skip("thread sanitizer cannot run in this container")
    assert rc == 0 and "WARNING: ThreadSanitizer" not in err, (line, err[-2000:])


# ---- the exchange whose sum is formed inside the NVLink switch (tests/multimem_model.cc): counters
# that only grow, targets derived from them, one partial and one gather area reused call after call
@pytest.fixture(scope="module")
def multimem_model(tmp_path_factory):
    return compile_model(tmp_path_factory.mktemp("multimem_model"), tsan=False, src=SRC_MULTIMEM)


@pytest.mark.parametrize("gemm_signals", [0, 1])
@pytest.mark.parametrize("ranks,max_rows,calls", [(2, 4, 80), (4, 8, 40), (8, 16, 15)])
def test_switch_reduction_protocol_with_varying_row_counts(multimem_model, ranks, max_rows, calls, gemm_signals):
    for seed in (1, 2, 3, 4):
        rc, line, err = run(multimem_model, "normal", ranks, max_rows, calls, seed, gemm_signals)
        assert rc == 0, (line, err)
        assert line["wrong_rows"] == 0 and line["timeouts"] == 0


def test_switch_reduction_absent_rank_times_everybody_out(multimem_model):
    rc, line, err = run(multimem_model, "absent", 4, 4)
    assert rc == 0, (line, err)
    assert line["ranks_timed_out"] == 3 and line["wrong_rows"] == 0


def test_switch_reduction_model_under_thread_sanitizer(tmp_path):
    exe = compile_model(tmp_path, tsan=True, src=SRC_MULTIMEM)
    if exe is None:
        pytest.skip("g++ has no thread-sanitizer runtime here")
    for sig in (0, 1):
        rc, line, err = run(exe, "normal", 4, 4, 10, 7, sig, timeout=300)
        if "FATAL: ThreadSanitizer" in err or "unexpected memory mapping" in err:
            pytest.skip("thread sanitizer cannot run in this container")
        assert rc == 0 and "WARNING: ThreadSanitizer" not in err, (line, err[-2000:])

