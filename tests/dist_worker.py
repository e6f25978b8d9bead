"""One rank of a multi-process CPU (gloo) test. Usage: dist_worker.py <scenario> <out_json>."""
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402

from sketchml_b200.config import MLConf  # noqa: E402
from sketchml_b200.parallel import FaultInjector, TorchComm  # noqa: E402
from sketchml_b200.trainer import Trainer  # noqa: E402


def main():
    scenario, out = sys.argv[1], sys.argv[2]
    rank = int(os.environ["RANK"])
    torch.set_num_threads(1)
    comm = TorchComm("gloo", timeout_s=float(os.environ.get("SKML_TEST_TIMEOUT", "20")))
    kw = dict(algo="lr", format="synthetic", feature_num=4000, syn_rows=4000, syn_nnz_per_row=12, epoch_num=3,
              learn_rate=0.5, l2_reg=1e-4, valid_ratio=0.1, batch_sample_ratio=0.25, device="cpu", dtype="float64",
              quant_bin_num=128, sketch_row_num=3, sketch_col_ratio=0.2, seed=5,
              extras={"heartbeat_timeout_s": 5.0})
    inj = None
    if scenario == "none":
        kw["compressor"] = "None"
    elif scenario == "adam":
        kw.update(optimizer="adam", learn_rate=0.02)
    elif scenario == "exit" and rank == 1:
        inj = FaultInjector(exit_at_step=3)
    elif scenario == "stale" and rank == 1:
        inj = FaultInjector(stale_steps={2})
    elif scenario == "corrupt" and rank == 0:
        inj = FaultInjector(corrupt_steps={1})
    elif scenario == "skip" and rank == 1:
        inj = FaultInjector(skip_publish_steps={2})
    res = {"rank": rank, "scenario": scenario}
    try:
        t = Trainer(MLConf(**kw), comm=comm, injector=inj)
        t.load_data()
        h = t.train()
        res.update(ok=True, train_loss=h["train_loss"], valid_loss=h["valid_loss"],
                   w_sum=float(t.model.weights.sum()), w_abs=float(t.model.weights.abs().sum()),
                   payload=[r["payload_bytes"] for r in t.metrics.of("exchange")][-1:] or None)
        if scenario == "ckpt":
            p = os.path.join(os.path.dirname(out), "dist.ckpt")
            t.checkpoint(p, 3)
            res["ckpt"] = os.path.exists(p)
    except SystemExit as e:
        res.update(ok=False, error="SystemExit", code=e.code)
    except Exception as e:  # the failure must surface as a Python exception, never as a hang
        res.update(ok=False, error=type(e).__name__, message=str(e)[:300], step=getattr(locals().get("t"), "step", None))
    with open(out, "w") as f:
        json.dump(res, f)
    os._exit(0)   # skip process-group teardown: a peer may be gone


if __name__ == "__main__":
    main()
