"""Multi-GPU runs (skipped with fewer than 2 GPUs): the fused compress -> peer-store ->
decode exchange against the NCCL baselines, replica equality, and a publish that never
arrives (bounded wait -> StepTimeout, no GPU fault). NVLS is switched off for these runs."""
import json
import os
import socket
import subprocess
import sys
import time

import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def _run(scenario, tmp_path, world, timeout=240):
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    procs, outs = [], []
    for r in range(world):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE=str(world), LOCAL_RANK=str(r), MASTER_ADDR="127.0.0.1",
                   MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0", OMP_NUM_THREADS="2")
        out = tmp_path / f"{scenario}_{r}.json"
        outs.append(out)
        procs.append(subprocess.Popen([sys.executable, os.path.join(HERE, "dist_worker_gpu.py"), scenario, str(out)],
                                      env=env, stdout=subprocess.DEVNULL, stderr=subprocess.PIPE))
    deadline = time.time() + timeout
    for p in procs:
        try:
            p.wait(timeout=max(1, deadline - time.time()))
        except subprocess.TimeoutExpired:
            for q in procs:
                q.kill()
            pytest.fail(f"scenario {scenario}: a rank did not finish")
    res = []
    for o, p in zip(outs, procs):
        assert o.exists(), p.stderr.read().decode()[-3000:]
        res.append(json.loads(o.read_text()))
    return res


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least 2 GPUs")
def test_fused_exchange_matches_nccl_baselines(tmp_path):
    world = 2
    sk, un, kv = _run("sketch", tmp_path, world), _run("none", tmp_path, world), _run("kv", tmp_path, world)
    for res in (sk, un, kv):
        assert all(r["ok"] for r in res), res
        assert len({r["hash"] for r in res}) == 1, "replicas drifted apart"
        assert res[0]["train_loss"][-1] < res[0]["train_loss"][0]
    assert abs(un[0]["valid_loss"][-1] - kv[0]["valid_loss"][-1]) < 1e-4
    gap = abs(sk[0]["valid_loss"][-1] - un[0]["valid_loss"][-1]) / un[0]["valid_loss"][-1]
    assert gap < 0.1, (sk[0], un[0])


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least 2 GPUs")
@pytest.mark.parametrize("scenario", ["sketch_adam", "fixedpoint"])
def test_adam_and_packed_fixed_point_keep_replicas_identical(tmp_path, scenario):
    """Lazy Adam over the fused exchange (plain float sums in rank order inside the owning block) and
    the FixedPoint baseline with its packed codes on the wire: every rank ends with the same bits."""
    res = _run(scenario, tmp_path, 2)
    assert all(r["ok"] for r in res), res
    assert len({r["hash"] for r in res}) == 1, "replicas drifted apart"
    assert res[0]["train_loss"][-1] < res[0]["train_loss"][0]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least 2 GPUs")
def test_missing_publish_times_out_cleanly(tmp_path):
    res = _run("skip", tmp_path, 2)
    assert not any(r["ok"] for r in res), res
    assert any(r["error"] == "StepTimeout" for r in res), res
    assert all(r["error"] in ("StepTimeout", "PeerLost", "CommFailure", "PayloadError") for r in res), res
