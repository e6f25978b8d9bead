"""Checkpoint / resume and model export.

The reference writes neither a checkpoint nor a model (``main`` ends after ``train()``
with a TODO, ml/SketchML.scala:20-23; weights live in an executor-side static,
ml/algorithm/GeneralizedLinearModel.scala:21-26). Both formats here are therefore new:

* checkpoint: one torch file with weights, optimizer state (SGD/Adam counters, Adam
  moments and beta powers), data cursor, step/epoch counters, the configuration and a
  hash of the weights that every rank compares with rank 0's to detect replica drift;
* model export: text ``index:weight`` lines for the non-zero weights (libsvm style) and
  a ``.pt`` tensor beside it.
"""
from __future__ import annotations

import hashlib
import os
from typing import Optional

import torch


def weights_hash(w: torch.Tensor) -> str:
    return hashlib.sha256(w.detach().cpu().contiguous().numpy().tobytes()).hexdigest()


def save_checkpoint(path: str, *, model_state: dict, conf: dict, step: int, epoch: int, cursor: int,
                    extra: Optional[dict] = None) -> str:
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    blob = {"format": "sketchml_b200.checkpoint.v1", "model": model_state, "conf": conf, "step": step,
            "epoch": epoch, "cursor": cursor, "weights_hash": weights_hash(model_state["weights"]),
            "extra": extra or {}}
    tmp = path + ".tmp"
    torch.save(blob, tmp)
    os.replace(tmp, path)
    return blob["weights_hash"]


def load_checkpoint(path: str) -> dict:
    blob = torch.load(path, map_location="cpu", weights_only=False)
    if blob.get("format") != "sketchml_b200.checkpoint.v1":
        raise ValueError(f"{path} is not a sketchml_b200 checkpoint")
    if weights_hash(blob["model"]["weights"]) != blob["weights_hash"]:
        raise ValueError(f"{path}: weights do not match their recorded hash")
    return blob


def export_model(path: str, weights: torch.Tensor, name: str = "model") -> int:
    """Writes ``path`` (text) and ``path + '.pt'``; returns the number of non-zero weights."""
    w = weights.detach().cpu()
    nz = torch.nonzero(w).flatten()
    with open(path, "w") as f:
        f.write(f"# sketchml_b200 model={name} dim={w.numel()} nnz={nz.numel()}\n")
        vals = w[nz].double().tolist()
        for i, v in zip(nz.tolist(), vals):
            f.write(f"{i}:{v!r}\n")
    torch.save({"name": name, "weights": w}, path + ".pt")
    return int(nz.numel())


def import_model(path: str, dtype=torch.float32) -> torch.Tensor:
    if path.endswith(".pt"):
        return torch.load(path, map_location="cpu", weights_only=False)["weights"].to(dtype)
    dim, idx, val = None, [], []
    with open(path) as f:
        for line in f:
            line = line.strip()
            if line.startswith("#"):
                for tok in line.split():
                    if tok.startswith("dim="):
                        dim = int(tok[4:])
                continue
            if line:
                i, v = line.split(":")
                idx.append(int(i))
                val.append(float(v))
    w = torch.zeros(dim if dim is not None else (max(idx) + 1 if idx else 0), dtype=dtype)
    if idx:
        w[torch.tensor(idx)] = torch.tensor(val, dtype=dtype)
    return w
