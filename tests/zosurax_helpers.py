"""Small Zosurax configurations with seeded weights, written as model folders, and the helpers that run
them through the engine and through the plain implementation.

The configurations differ from one another in every size and option: 1 to 5 heads per key/value head and
a single head; values wider, narrower and as wide as keys; rotations over a whole head, over a part of it
and none; recurrent layers with and without a feed-forward, attention layers with and without; a loop over
the first layers, over the last one, over one layer run once, and no loop; widths that are multiples of 64
(the shapes the tensor-core kernels take) and widths that no vectorised kernel takes.  Weights are
N(0, 1/inputs) ("loud": every layer changes the stream by as much as it holds).
"""
from __future__ import annotations

import json
from pathlib import Path

import numpy as np
import torch

import plain_zosurax as P


def _hgrn2(heads, dim, vdim, ff=None):
    return {"type": "hgrn2", "mixer": {"heads": heads, "dim": dim, "vdim": vdim},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def _attn(kind, heads, kv_heads, dim, vdim, scale, rot=None, ff=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if rot is not None:
        m["rot"] = {"base": rot[0], "dims": rot[1]}
    return {"type": kind, "mixer": m, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


CONFIGS = {
    # a loop over the first two layers (a recurrence and an attention), three heads on one key/value head, values
    # wider than keys, a rotation over half a head; then mixed heads with two heads per key/value head
    "za": {"architecture": "Zosurax", "vocab": 97, "width": 40, "norm": {"eps": 1e-6},
           "loop": {"start": 0, "stop": 2, "times": 2},
           "layers": [_hgrn2(2, 8, 12, ff=56),
                      _attn("attention", 3, 1, 16, 24, 0.3, rot=(100.0, 8)),
                      _attn("attention_2", 4, 2, 10, 6, 0.35, rot=(50.0, 10), ff=48)]},
    # no loop; mixed heads over ONE key/value head with a partial interleaved rotation; a recurrence without
    # feed-forward; an attention without any rotation
    "zb": {"architecture": "Zosurax", "vocab": 130, "width": 64, "norm": {"eps": 1e-5},
           "layers": [_attn("attention_2", 2, 1, 32, 32, 0.2, rot=(10000.0, 16), ff=72),
                      _hgrn2(4, 16, 16),
                      _attn("attention", 4, 4, 8, 8, 0.4, ff=80)]},
    # sizes in multiples of 64 (what the tensor-core contractions and attention kernels take): head widths 64 and
    # 128, four heads per key/value head, a loop over one layer in the middle
    "zc": {"architecture": "Zosurax", "vocab": 512, "width": 128, "norm": {"eps": 1e-5},
           "loop": {"start": 2, "stop": 3, "times": 2},
           "layers": [_attn("attention", 8, 2, 64, 64, 0.12, rot=(10000.0, 64), ff=256),
                      _hgrn2(2, 64, 64, ff=128),
                      _attn("attention_2", 4, 4, 64, 64, 0.11, rot=(500.0, 32), ff=256),
                      _attn("attention", 2, 2, 128, 128, 0.09, rot=(10000.0, 64))]},
    # the least there can be: one recurrent layer with one head, in a loop that runs once
    "zd": {"architecture": "Zosurax", "vocab": 50, "width": 32, "norm": {"eps": 1e-5},
           "loop": {"start": 0, "stop": 1, "times": 1},
           "layers": [_hgrn2(1, 4, 4)]},
    # sizes no vectorised kernel takes (a width that is no multiple of 4, head widths 10, 7, 5, 9, a prime
    # vocabulary), five heads on five, and a loop of three passes over the LAST layer, a recurrence
    "ze": {"architecture": "Zosurax", "vocab": 71, "width": 38, "norm": {"eps": 1e-4},
           "loop": {"start": 1, "stop": 2, "times": 3},
           "layers": [_attn("attention_2", 5, 5, 10, 7, 0.3, rot=(20.0, 6)),
                      _hgrn2(3, 5, 9, ff=50)]},
}


def bf16_round(a: np.ndarray) -> np.ndarray:
    return torch.from_numpy(np.asarray(a, dtype=np.float32)).to(torch.bfloat16).float().numpy()


def make_weights(cfg: dict, seed: int) -> dict[str, np.ndarray]:
    """Seeded weights that bfloat16 holds exactly, as float32, by tensor name."""
    import zinfer_b200 as z
    from zinfer_b200.config.registry import build_model

    rng = np.random.default_rng(seed)
    model = build_model(z.config_from_dict(cfg))
    W = {}
    for name, spec in model.weight_specs().items():
        shape = spec.shape
        if name.endswith(".talk"):
            W[name] = bf16_round(np.eye(shape[0]) * 0.7 + rng.normal(0, 0.35, shape))
        elif name.endswith(".lower"):
            W[name] = bf16_round(rng.uniform(0.0, 0.9, shape))
        elif name.endswith(".shift"):
            W[name] = bf16_round(rng.uniform(0.05, 0.95, shape))
        elif name.endswith(".f.b"):
            W[name] = bf16_round(rng.normal(0.5, 1.0, shape))
        elif name.endswith(".ls1") or name.endswith(".ls2"):
            W[name] = bf16_round(rng.normal(0.8, 0.3, shape))
        elif "norm" in name:
            W[name] = bf16_round(1.0 + rng.normal(0, 0.2, shape))
        elif name == "loop.step":
            W[name] = bf16_round(rng.normal(0, 0.5, shape))
        elif name == "embed":
            W[name] = bf16_round(rng.normal(0, 1.0, shape))
        else:
            W[name] = bf16_round(rng.normal(0, shape[-1] ** -0.5, shape))
    return W


def write_folder(folder, cfg: dict, W: dict[str, np.ndarray]) -> Path:
    from zinfer_b200.weights import write_safetensors

    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(cfg))
    write_safetensors(folder / "model.safetensors", {n: torch.from_numpy(a).to(torch.bfloat16) for n, a in W.items()})
    return folder


def plain_logits(cfg: dict, W: dict[str, np.ndarray], tokens) -> np.ndarray:
    return P.forward(cfg, {n: a.astype(np.float64) for n, a in W.items()}, list(tokens))


def tokens_for(cfg: dict, seed: int, n: int) -> list[int]:
    return np.random.default_rng(seed).integers(0, cfg["vocab"], size=n).tolist()


TOL = {"float32": 5e-5, "bfloat16": 4e-2}


def rel_err(got, ref) -> float:
    got, ref = np.asarray(got, dtype=np.float64), np.asarray(ref, dtype=np.float64)
    scale = float(np.abs(ref).max())
    assert scale > 0 and got.shape == ref.shape, (got.shape, ref.shape)
    return float(np.abs(got - ref).max()) / scale
