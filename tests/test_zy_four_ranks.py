"""Four ranks (skipped with fewer than 4 GPUs): with three or more addends per coordinate the order in
which the ranks' contributions are summed must be the same on every rank: rank order inside the
fused decode kernel, list order in the raw key/value and FixedPoint baselines."""
import pytest
import torch

from test_gpu_multi import _run

pytestmark = pytest.mark.gpu


@pytest.mark.skipif(torch.cuda.device_count() < 4, reason="needs at least 4 GPUs")
@pytest.mark.parametrize("scenario", ["sketch", "sketch_adam", "kv", "fixedpoint"])
def test_four_ranks_keep_replicas_identical(tmp_path, scenario):
    res = _run(scenario, tmp_path, 4)
    assert all(r["ok"] for r in res), res
    assert len({r["hash"] for r in res}) == 1, "replicas drifted apart"
    assert res[0]["train_loss"][-1] < res[0]["train_loss"][0]
