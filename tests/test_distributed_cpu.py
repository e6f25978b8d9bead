"""Multi-process CPU runs over gloo (world_size 2): the plumbing configuration (compressed
run checked against an uncompressed run), replica equality, and host-injected failures that
must end in exceptions on every surviving rank, never in a hang."""
import json
import os
import socket
import subprocess
import sys
import time

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _run(scenario, tmp_path, world=2, timeout=150):
    port = _free_port()
    procs, outs = [], []
    for r in range(world):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE=str(world), LOCAL_RANK=str(r), MASTER_ADDR="127.0.0.1",
                   MASTER_PORT=str(port), OMP_NUM_THREADS="1", SKML_TEST_TIMEOUT="15", CUDA_VISIBLE_DEVICES="")
        out = tmp_path / f"{scenario}_{r}.json"
        outs.append(out)
        procs.append(subprocess.Popen([sys.executable, os.path.join(HERE, "dist_worker.py"), scenario, str(out)],
                                      env=env, stdout=subprocess.DEVNULL, stderr=subprocess.PIPE))
    deadline = time.time() + timeout
    for p in procs:
        try:
            p.wait(timeout=max(1, deadline - time.time()))
        except subprocess.TimeoutExpired:
            for q in procs:
                q.kill()
            pytest.fail(f"scenario {scenario}: a rank hung")
    res = []
    for o, p in zip(outs, procs):
        assert o.exists(), p.stderr.read().decode()[-2000:]
        res.append(json.loads(o.read_text()))
    return res


def test_plumbing_run_compressed_vs_uncompressed(tmp_path):
    sk = _run("sketch", tmp_path)
    un = _run("none", tmp_path)
    for res in (sk, un):
        assert all(r["ok"] for r in res), res
        assert res[0]["w_sum"] == res[1]["w_sum"] and res[0]["w_abs"] == res[1]["w_abs"]   # replicas identical
        assert res[0]["train_loss"] == res[1]["train_loss"]
        assert res[0]["train_loss"][-1] < res[0]["train_loss"][0]
    gap = abs(sk[0]["valid_loss"][-1] - un[0]["valid_loss"][-1]) / un[0]["valid_loss"][-1]
    assert gap < 0.05
    assert sk[0]["payload"][0] > 256


def test_adam_and_checkpoint_across_ranks(tmp_path):
    res = _run("adam", tmp_path)
    assert all(r["ok"] for r in res) and res[0]["w_abs"] == res[1]["w_abs"]
    res = _run("ckpt", tmp_path)
    assert all(r["ok"] for r in res) and res[0]["ckpt"]


@pytest.mark.parametrize("scenario,errors", [
    ("exit", {"CommFailure", "PeerLost"}), ("stale", {"PayloadError", "PeerLost", "CommFailure"}),
    ("corrupt", {"PayloadError", "PeerLost", "CommFailure"}), ("skip", {"PayloadError", "PeerLost", "CommFailure"})])
def test_host_injected_failures_raise_everywhere(tmp_path, scenario, errors):
    res = _run(scenario, tmp_path)
    if scenario == "exit":
        assert res[1]["error"] == "SystemExit" and res[1]["code"] == 17
        assert not res[0]["ok"] and res[0]["error"] in errors, res
    else:
        assert not any(r["ok"] for r in res), res
        assert all(r["error"] in errors for r in res), res
        assert any(r["error"] == "PayloadError" for r in res), res
