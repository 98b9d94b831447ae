"""Checkpoint format of train_modal.py:393-413 / generate.py:47-76 (CPU only)."""
import pickle

import ml_dtypes
import numpy as np
import pytest
import torch

from train_gpt_b200 import checkpoint
from train_gpt_b200.step import GPT, SMALL, StepConfig


def _cfg():
    return StepConfig(**SMALL, mm="bf16", norm="torch_reference", loss="torch", optimizer="torch")


def test_round_trip_keeps_every_bit(tmp_path):
    a, b = GPT(_cfg(), "cpu", seed=1), GPT(_cfg(), "cpu", seed=2)
    p = checkpoint.save_checkpoint(tmp_path / "run_x" / "step_7.pkl", a, step=7, config="small", run_id="run_x")
    tree, config, step = checkpoint.load_checkpoint(p)
    assert (config, step) == ("small", 7)
    checkpoint.load_params(b, tree)
    for x, y in zip(a.parameters(), b.parameters()):
        assert torch.equal(x, y)


def test_file_has_the_reference_layout(tmp_path):
    m = GPT(_cfg(), "cpu", seed=0)
    p = checkpoint.save_checkpoint(tmp_path / "c.pkl", m, step=3)
    with open(p, "rb") as f:
        raw = pickle.load(f)
    assert set(raw) == {"step", "config", "run_id", "params"}
    assert set(raw["params"]) == {"embed", "pos", "layers", "final_norm", "unembed"}          # model.py:46-54
    assert set(raw["params"]["layers"]) == set(checkpoint.LAYER_KEYS)
    c = m.cfg
    assert raw["params"]["layers"]["wq"].shape == (c.n_layers, c.d_model, c.n_heads * c.head_dim)   # stacked for lax.scan
    assert raw["params"]["layers"]["w_down"].dtype == ml_dtypes.bfloat16
    assert raw["params"]["embed"].shape == (c.vocab_size, c.d_model)


def test_reads_a_tree_written_by_the_reference_side(tmp_path):
    """A payload built the way `_tree_to_numpy` builds it (float32 here, as a float32-config run
    would write) loads and is cast to the model dtype; tied embeddings fill the head."""
    m = GPT(_cfg(), "cpu", seed=0)
    c = m.cfg
    rng = np.random.default_rng(0)
    h = c.n_heads * c.head_dim
    shapes = {"norm1": (c.d_model,), "wq": (c.d_model, h), "wk": (c.d_model, h), "wv": (c.d_model, h), "wo": (h, c.d_model),
              "norm2": (c.d_model,), "w_up": (c.d_model, c.d_ff), "w_down": (c.d_ff, c.d_model)}
    tree = {"embed": rng.standard_normal((c.vocab_size, c.d_model)).astype(np.float32),
            "pos": rng.standard_normal((c.seq_len, c.d_model)).astype(np.float32),
            "final_norm": np.ones(c.d_model, np.float32),
            "layers": {k: rng.standard_normal((c.n_layers,) + s).astype(np.float32) for k, s in shapes.items()}}
    with open(tmp_path / "ref.pkl", "wb") as f:
        pickle.dump({"step": 11, "config": "small", "params": tree}, f)
    got, config, step = checkpoint.load_checkpoint(tmp_path / "ref.pkl")
    checkpoint.load_params(m, got)
    assert step == 11
    assert torch.equal(m.layers[1]["w_up"], torch.from_numpy(tree["layers"]["w_up"][1]).to(torch.bfloat16))
    assert torch.equal(m.unembed, torch.from_numpy(tree["embed"].T.copy()).to(torch.bfloat16))


def test_errors_are_the_reference_s(tmp_path):
    with pytest.raises(FileNotFoundError, match="checkpoint not found"):
        checkpoint.load_checkpoint(tmp_path / "nope.pkl")
    with open(tmp_path / "bad.pkl", "wb") as f:
        pickle.dump({"step": 1, "params": {}}, f)
    with pytest.raises(ValueError, match="is missing 'config'"):
        checkpoint.load_checkpoint(tmp_path / "bad.pkl")
    m = GPT(_cfg(), "cpu", seed=0)
    tree = checkpoint.params_tree(m)
    tree["pos"] = tree["pos"][:-1]
    with pytest.raises(ValueError, match="pos: checkpoint shape"):
        checkpoint.load_params(m, tree)
