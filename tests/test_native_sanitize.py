"""The native plan pipeline (JSON reader, plan loader, validator, lowering, cross-rank protocol check)
built with AddressSanitizer + UndefinedBehaviorSanitizer and fed every template and a set of broken
inputs.  Host code only: no GPU, no torch in the binary."""

import json
import os
import shutil
import subprocess

import pytest

from helpers import build_plans
from pccl_b200.dsl.algorithms import ALGORITHMS

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CSRC = os.path.join(ROOT, "pccl_b200", "csrc")
CUDA_INCLUDE = "/usr/local/cuda/include"


def _build(tmp_path):
    exe = tmp_path / "plan_sanitize"
    cmd = ["g++", "-std=c++17", "-O1", "-g", "-fno-omit-frame-pointer", "-fsanitize=address,undefined",
           "-fno-sanitize-recover=undefined", "-I", CSRC, "-I", CUDA_INCLUDE,
           os.path.join(ROOT, "tests", "native", "plan_sanitize_main.cc"),
           os.path.join(CSRC, "engine", "plan.cc"), os.path.join(CSRC, "common", "json.cc"),
           os.path.join(CSRC, "common", "util.cc"), "-ldl", "-lpthread", "-o", str(exe)]
    done = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    if done.returncode != 0 and ("asan" in done.stderr.lower() or "sanitize" in done.stderr.lower()):
        pytest.skip("this toolchain has no sanitizer runtime")
    assert done.returncode == 0, done.stderr[-3000:]
    return exe


@pytest.mark.skipif(shutil.which("g++") is None or not os.path.isdir(CUDA_INCLUDE), reason="needs g++ and the NVTX headers")
def test_plan_pipeline_under_sanitizers(tmp_path):
    exe = _build(tmp_path)
    good, bad = tmp_path / "cases" / "good", tmp_path / "cases" / "bad"
    bad.mkdir(parents=True)
    cases = 0
    for name, algorithm in sorted(ALGORITHMS.items()):
        for world in (2, 4, 8):
            if name in ("rhd", "tree") and world & (world - 1):
                continue
            for kind in ("allreduce", "allgather", "reduce_scatter", "alltoall"):
                if not hasattr(algorithm(), "build_" + kind):
                    continue
                for numel, channels in ((world * 8, 1), (world * 1000, 2), (world * 4096 + 8 * world, 4)):
                    executor = "multimem" if name in ("nvls", "nvls_twopass", "hybrid") else "sm"
                    try:
                        plans = build_plans(algorithm(), kind, world, numel, "float32", executor, channels)
                    except Exception:
                        continue                  # the template does not offer this collective / shape
                    where = good / f"{name}_{kind}_{world}_{numel}_{channels}"
                    where.mkdir(parents=True)
                    for rank, plan in enumerate(plans):
                        (where / f"{rank}.json").write_text(plan if isinstance(plan, str) else json.dumps(plan))
                    cases += 1
    assert cases > 60
    sample = json.loads(next(iter(sorted(good.iterdir()))).joinpath("0.json").read_text())
    (bad / "truncated.json").write_text(json.dumps(sample)[: len(json.dumps(sample)) // 2])
    (bad / "not_json.json").write_text("{]")
    (bad / "empty.json").write_text("")
    no_ops = dict(sample)
    no_ops.pop("operations", None)
    (bad / "no_operations.json").write_text(json.dumps(no_ops))
    far = json.loads(json.dumps(sample))
    for op in far["operations"]:
        params = op.get("params", op)
        for key in list(params):
            if "offset" in key:
                params[key] = 1 << 40
    (bad / "offset_out_of_range.json").write_text(json.dumps(far))
    peer = json.loads(json.dumps(sample))
    for op in peer["operations"]:
        params = op.get("params", op)
        for key in list(params):
            if key in ("source_rank", "target_rank", "peer"):
                params[key] = 99
    (bad / "peer_out_of_range.json").write_text(json.dumps(peer))
    env = dict(os.environ, ASAN_OPTIONS="detect_leaks=1:abort_on_error=0", UBSAN_OPTIONS="print_stacktrace=1")
    done = subprocess.run([str(exe), str(tmp_path / "cases")], capture_output=True, text=True, timeout=600, env=env)
    assert done.returncode == 0, done.stdout[-2000:] + done.stderr[-4000:]
    assert "ERROR: AddressSanitizer" not in done.stderr and "runtime error" not in done.stderr, done.stderr[-4000:]
    summary = dict(kv.split("=") for kv in done.stdout.strip().split()[1:])
    assert int(summary["good"]) == cases and int(summary["failures"]) == 0 and int(summary["refused"]) >= 4, done.stdout


@pytest.mark.skipif(shutil.which("g++") is None or not os.path.isdir(CUDA_INCLUDE), reason="needs g++ and the NVTX headers")
def test_fd_server_under_thread_sanitizer(tmp_path):
    """The descriptor-passing server (one thread per rank, SCM_RIGHTS over abstract unix sockets) with
    concurrent publishers and fetchers, under ThreadSanitizer."""
    exe = tmp_path / "fd_server_tsan"
    cmd = ["g++", "-std=c++17", "-O1", "-g", "-fno-omit-frame-pointer", "-fsanitize=thread", "-I", CSRC, "-I", CUDA_INCLUDE,
           os.path.join(ROOT, "tests", "native", "fd_server_tsan_main.cc"), os.path.join(CSRC, "common", "fd_socket.cc"),
           os.path.join(CSRC, "common", "util.cc"), "-ldl", "-lpthread", "-o", str(exe)]
    done = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    if done.returncode != 0 and ("tsan" in done.stderr.lower() or "sanitize" in done.stderr.lower()):
        pytest.skip("this toolchain has no ThreadSanitizer runtime")
    assert done.returncode == 0, done.stderr[-3000:]
    env = dict(os.environ, TSAN_OPTIONS="halt_on_error=0:second_deadlock_stack=1")
    run = subprocess.run([str(exe)], capture_output=True, text=True, timeout=300, env=env)
    if "FATAL: ThreadSanitizer" in run.stderr and "unexpected memory mapping" in run.stderr:
        pytest.skip("ThreadSanitizer cannot map its shadow memory in this container")
    assert run.returncode == 0, run.stdout[-1500:] + run.stderr[-4000:]
    assert "WARNING: ThreadSanitizer" not in run.stderr, run.stderr[-4000:]
    assert "FD_SERVER_TSAN failures=0" in run.stdout


@pytest.mark.skipif(shutil.which("g++") is None or not os.path.isdir(CUDA_INCLUDE), reason="needs g++ and the NVTX headers")
def test_rdma_proxy_under_thread_sanitizer(tmp_path):
    """The RDMA proxy's command queue and worker thread over the loopback fabric: concurrent submitters,
    injected errors, dropped requests, shutdown with work queued, under ThreadSanitizer."""
    exe = tmp_path / "rdma_proxy_tsan"
    rdma = os.path.join(CSRC, "executors", "rdma")
    cmd = ["g++", "-std=c++17", "-O1", "-g", "-fno-omit-frame-pointer", "-fsanitize=thread", "-I", CSRC, "-I", CUDA_INCLUDE,
           os.path.join(ROOT, "tests", "native", "rdma_proxy_tsan_main.cc"), os.path.join(rdma, "rdma_proxy.cc"),
           os.path.join(rdma, "verbs_transport.cc"), os.path.join(CSRC, "common", "json.cc"),
           os.path.join(CSRC, "common", "util.cc"), "-ldl", "-lpthread", "-o", str(exe)]
    done = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    if done.returncode != 0 and ("tsan" in done.stderr.lower() or "sanitize" in done.stderr.lower()):
        pytest.skip("this toolchain has no ThreadSanitizer runtime")
    assert done.returncode == 0, done.stderr[-3000:]
    run = subprocess.run([str(exe)], capture_output=True, text=True, timeout=300,
                         env=dict(os.environ, TSAN_OPTIONS="halt_on_error=0"))
    if "FATAL: ThreadSanitizer" in run.stderr and "unexpected memory mapping" in run.stderr:
        pytest.skip("ThreadSanitizer cannot map its shadow memory in this container")
    assert run.returncode == 0, run.stdout[-1500:] + run.stderr[-4000:]
    assert "WARNING: ThreadSanitizer" not in run.stderr, run.stderr[-4000:]
    assert "RDMA_PROXY_TSAN failures=0" in run.stdout
