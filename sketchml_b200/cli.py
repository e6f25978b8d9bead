"""Command line entry: ``python -m sketchml_b200 {train,demo,export,microbench}``.

``train`` takes the reference's options either as flags (``--algo``, ``--feature-num``,
``--batch-sample-ratio``, ``--quantization-bin-num`` ...) or verbatim as
``--conf spark.sketchml.key=value`` (ml/SketchML.scala:8-26, ml/conf/MLConf.scala:47-66).
Under ``torchrun`` every process is one worker.
"""
from __future__ import annotations

import argparse
import json
import sys

from . import config as C


def _train(ns) -> int:
    from .trainer import Trainer
    conf = C.conf_from_args(ns)
    t = Trainer(conf)
    try:
        t.load_data()
        hist = t.train()
        if t.comm.rank == 0:
            print(json.dumps({"train_loss": hist["train_loss"], "valid_loss": hist["valid_loss"],
                              "time_ms": hist["time_ms"]}))
    finally:
        t.close()
        t.comm.close()
    return 0


def _demo(ns) -> int:
    from .compress import app
    app.main(ns.size, ns.seed)
    return 0


def _export(ns) -> int:
    from .utils import export_model, load_checkpoint
    blob = load_checkpoint(ns.checkpoint)
    n = export_model(ns.out, blob["model"]["weights"], blob["model"].get("model", "model"))
    print(f"wrote {n} non-zero weights to {ns.out}")
    return 0


def _microbench(ns) -> int:
    from benchmarks import microbench  # repo-root package
    return microbench.main(ns.rest)


def main(argv=None) -> int:
    p = argparse.ArgumentParser(prog="sketchml_b200")
    sub = p.add_subparsers(dest="cmd", required=True)
    tr = sub.add_parser("train", help="train a generalized linear model")
    C.add_arguments(tr)
    tr.set_defaults(fn=_train)
    de = sub.add_parser("demo", help="compress/decompress demo of the stand-alone library")
    de.add_argument("--size", type=int, default=1_000_000)
    de.add_argument("--seed", type=int, default=0)
    de.set_defaults(fn=_demo)
    ex = sub.add_parser("export", help="write a checkpoint's weights as index:weight text")
    ex.add_argument("checkpoint")
    ex.add_argument("out")
    ex.set_defaults(fn=_export)
    mb = sub.add_parser("microbench", help="compression / collective microbenchmark")
    mb.add_argument("rest", nargs=argparse.REMAINDER)
    mb.set_defaults(fn=_microbench)
    ns = p.parse_args(argv)
    return ns.fn(ns)


if __name__ == "__main__":
    sys.exit(main())
