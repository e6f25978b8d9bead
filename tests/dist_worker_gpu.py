"""One rank of a multi-GPU test (one process per GPU, NCCL + peer-memory exchange).
Usage: dist_worker_gpu.py <scenario> <out_json>."""
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402

from sketchml_b200.config import MLConf  # noqa: E402
from sketchml_b200.parallel import FaultInjector  # noqa: E402
from sketchml_b200.trainer import Trainer  # noqa: E402
from sketchml_b200.utils import weights_hash  # noqa: E402


def main():
    scenario, out = sys.argv[1], sys.argv[2]
    rank = int(os.environ["RANK"])
    kw = dict(algo="lr", format="synthetic", feature_num=300000, syn_rows=200000, syn_nnz_per_row=30, epoch_num=2,
              learn_rate=0.5, l2_reg=1e-4, valid_ratio=0.1, batch_sample_ratio=0.1, device="cuda", seed=5,
              quant_bin_num=256, sketch_group_num=16, sketch_row_num=3, sketch_col_ratio=0.5, step_timeout_s=1.0,
              extras={"heartbeat_timeout_s": 10.0, "check_status_every_step": scenario == "skip"})
    inj = None
    if scenario == "none":
        kw["compressor"] = "None"
    elif scenario == "kv":
        kw["compressor"] = "Float"
    elif scenario == "sketch_adam":
        kw.update(optimizer="adam", learn_rate=0.01)
    elif scenario.startswith("wire_"):
        # no held-out rows: the shard is a whole number of batches, so the gradient comes from the
        # transposed batch index (no floating-point atomics) and the run is reproducible bit for bit
        kw.update(valid_ratio=0.0)
        if scenario != "wire_plain":
            kw.update(key_encoder="delta_adaptive", cell_bits=0 if scenario == "wire_huffman" else -1)
    elif scenario == "fixedpoint":
        kw.update(compressor="FixedPoint", fixed_point_bit_num=8)
    elif scenario == "zip":
        kw.update(compressor="Zip")
    elif scenario == "skip" and rank == 1:
        inj = FaultInjector(skip_publish_steps={3})
    res = {"rank": rank, "scenario": scenario}
    try:
        t = Trainer(MLConf(**kw), injector=inj)
        t.load_data()
        h = t.train()
        res.update(ok=True, train_loss=h["train_loss"], valid_loss=h["valid_loss"], hash=weights_hash(t.model.weights))
    except Exception as e:
        res.update(ok=False, error=type(e).__name__, message=str(e)[:300])
    with open(out, "w") as f:
        json.dump(res, f)
    torch.cuda.synchronize()
    os._exit(0)


if __name__ == "__main__":
    main()
