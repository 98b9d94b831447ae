"""train-gpt's checkpoint format for the step harness's parameters.

The reference writes `pickle.dump({"step", "config", "run_id", "params"})` where `params` is a
plain dict of host NumPy arrays (ml_dtypes bfloat16) with every per-layer tensor STACKED along a
leading layer axis, the layout `lax.scan` consumes (train_modal.py:71-78,393-413; model.py:19-54);
`generate.py:47-76` reads the same file back.  These helpers write and read exactly that, so
reference-trained weights can drive this repository's kernels and the other way round.
"""
from __future__ import annotations

import pickle
from pathlib import Path

import ml_dtypes
import numpy as np
import torch

LAYER_KEYS = ("norm1", "wq", "wk", "wv", "wo", "norm2", "w_up", "w_down")      # model.py:33-42
TOP_KEYS = ("embed", "pos", "final_norm")                                      # model.py:47-52


def _to_numpy(t: torch.Tensor) -> np.ndarray:
    t = t.detach().to("cpu").contiguous()
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().view(ml_dtypes.bfloat16)
    return t.numpy()


def _to_torch(a: np.ndarray, like: torch.Tensor) -> torch.Tensor:
    a = np.ascontiguousarray(a)
    if a.dtype == ml_dtypes.bfloat16:
        t = torch.from_numpy(a.view(np.int16)).view(torch.bfloat16)
    else:
        t = torch.from_numpy(a.astype(np.float32))
    return t.to(device=like.device, dtype=like.dtype)                          # generate.py:70-72 casts to the model dtype


def params_tree(model) -> dict:
    """The reference's parameter pytree (model.py:46-54) from a `step.GPT`."""
    tree = {k: _to_numpy(getattr(model, k)) for k in TOP_KEYS}
    tree["layers"] = {k: np.stack([_to_numpy(lp[k]) for lp in model.layers]) for k in LAYER_KEYS}
    tree["unembed"] = _to_numpy(model.unembed)
    return tree


def save_checkpoint(path, model, step: int, config: str = "custom", run_id: str = "") -> Path:
    """train_modal.py:393-413.  `config` is the reference's config NAME ("small" selects its
    SMALL preset on load, anything else its default Config; generate.py:66)."""
    path = Path(path)
    path.parent.mkdir(parents=True, exist_ok=True)
    payload = {"step": int(step), "config": config, "run_id": run_id, "params": params_tree(model)}
    with open(path, "wb") as f:
        pickle.dump(payload, f, protocol=pickle.HIGHEST_PROTOCOL)
    return path


def load_checkpoint(path):
    """generate.py:47-76 without the JAX part: returns (params tree of NumPy arrays, config name, step)."""
    path = Path(path)
    if not path.exists():
        raise FileNotFoundError(f"checkpoint not found: {path}")
    with open(path, "rb") as f:
        ckpt = pickle.load(f)
    for key in ("params", "config"):
        if key not in ckpt:
            raise ValueError(f"checkpoint {path} is missing '{key}'; expected a dict written "
                             f"by train_modal.py with keys step/config/params")
    return ckpt["params"], ckpt["config"], int(ckpt.get("step", 0))


def load_params(model, tree: dict) -> None:
    """Copy a reference parameter tree into a `step.GPT` of matching shapes (in place).
    A tree without "unembed" (tie_embeddings, model.py:95) fills the head with embed^T."""
    def put(dst: torch.Tensor, src: np.ndarray, name: str):
        if tuple(src.shape) != tuple(dst.shape):
            raise ValueError(f"{name}: checkpoint shape {tuple(src.shape)} does not match the model's {tuple(dst.shape)}")
        with torch.no_grad():
            dst.copy_(_to_torch(src, dst))

    for k in TOP_KEYS:
        put(getattr(model, k), tree[k], k)
    layers = tree["layers"]
    n = len(model.layers)
    for k in LAYER_KEYS:
        if layers[k].shape[0] != n:
            raise ValueError(f"layers/{k}: checkpoint has {layers[k].shape[0]} layers, the model {n}")
        for i, lp in enumerate(model.layers):
            put(lp[k], layers[k][i], f"layers/{k}[{i}]")
    if "unembed" in tree:
        put(model.unembed, tree["unembed"], "unembed")
    else:
        put(model.unembed, np.ascontiguousarray(np.asarray(tree["embed"]).T), "embed^T")
