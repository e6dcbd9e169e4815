"""Small Ponusun configurations with hand-made or seeded weights, written as model folders, and the
helpers that run them through the engine and through the plain implementation.

The configurations differ from one another in every size and option: heads per key/value head 1, 2, 3
and 4; value rows wider, narrower and as wide as key rows; 1 to 5 convolution taps or none; windows
shorter and longer than a page, and a reader whose window differs from the owner's; 1, 2 and 3 experts
per token, with and without a shared expert; layers without a feed-forward; with and without a logit cap.
Weights are N(0, 1/width) ("loud": every layer changes the stream by as much as it holds), norm weights
1 + N, distance-bias numbers and depth weights of a size that matters.
"""
from __future__ import annotations

import json
from pathlib import Path

import numpy as np
import torch

import plain_ponusun as P


def _mixer(heads, kv_heads, dim, vdim, scale, window=None, kv_from=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if window:
        m["mask"] = {"size": window}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def _moe(experts, top, ff, shared=None):
    m = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared:
        m["shared"] = {"ff": shared}
    return m


def _layer(mixer, mlp):
    return {"type": "attention", "mixer": mixer, "mlp": mlp}


CONFIGS = {
    # three heads on one key/value head, values wider than keys, a reader with a wider window than its owner,
    # three experts per token, a layer without feed-forward, widths that are no multiple of 16
    "pa": {"architecture": "Ponusun", "vocab": 97, "width": 40, "max_positions": 200, "norm": {"eps": 1e-6},
           "canon": {"taps": 3}, "logit_softcap": 12.0,
           "layers": [_layer(_mixer(3, 1, 16, 24, 0.3, 11), _moe(5, 3, 24, 40)),
                      _layer(_mixer(3, 1, 16, 24, 0.3, 21, kv_from=0), None),
                      _layer(_mixer(3, 1, 16, 24, 0.25, 6), {"kind": "dense", "ff": 56})]},
    # one head per key/value head, narrow heads, windows longer than a page, one expert per token without a
    # shared one, two taps, the last layer reads the FIRST layer's cache with a narrower window
    "pb": {"architecture": "Ponusun", "vocab": 130, "width": 64, "max_positions": 400, "norm": {"eps": 1e-5},
           "canon": {"taps": 2}, "logit_softcap": 50.0,
           "layers": [_layer(_mixer(4, 4, 8, 8, 0.5, 70), {"kind": "dense", "ff": 72}),
                      _layer(_mixer(4, 2, 32, 16, 0.2, 33), _moe(3, 1, 16)),
                      _layer(_mixer(4, 2, 32, 16, 0.2, 33, kv_from=1), _moe(4, 2, 32, 16)),
                      _layer(_mixer(4, 4, 8, 8, 0.4, 40, kv_from=0), {"kind": "dense", "ff": 80})]},
    # sizes in multiples of 16 and 64 (the shapes the tensor-core contractions and fused epilogues take),
    # four heads per key/value head, five taps, a window of exactly one page
    "pc": {"architecture": "Ponusun", "vocab": 512, "width": 128, "max_positions": 512, "norm": {"eps": 1e-5},
           "canon": {"taps": 5}, "logit_softcap": 24.0,
           "layers": [_layer(_mixer(8, 2, 64, 64, 0.12, 64), _moe(8, 2, 64, 64)),
                      _layer(_mixer(8, 2, 64, 64, 0.12, 48, kv_from=0), {"kind": "dense", "ff": 256}),
                      _layer(_mixer(4, 2, 64, 128, 0.1, 100), _moe(6, 2, 32, 96))]},
    # what the file does not mention does not exist: no convolution, no cap, no window, one layer, no feed-forward
    "pd": {"architecture": "Ponusun", "vocab": 50, "width": 32, "max_positions": 128, "norm": {"eps": 1e-5},
           "layers": [_layer(_mixer(2, 1, 16, 8, 0.25), None)]},
    # a single tap (the convolution sees the current token only)
    "pe": {"architecture": "Ponusun", "vocab": 61, "width": 48, "max_positions": 128, "norm": {"eps": 1e-5},
           "canon": {"taps": 1}, "logit_softcap": 5.0,
           "layers": [_layer(_mixer(2, 2, 24, 24, 0.2, 9), _moe(2, 2, 16, 8)),
                      _layer(_mixer(2, 2, 24, 24, 0.2, 9, kv_from=0), _moe(3, 1, 8))]},
    # sizes that no vectorised or tensor-core kernel takes: a width that is no multiple of 4, odd head widths,
    # five heads on five, a vocabulary that is prime, experts of 10 hidden units
    "pf": {"architecture": "Ponusun", "vocab": 71, "width": 38, "max_positions": 150, "norm": {"eps": 1e-4},
           "canon": {"taps": 6}, "logit_softcap": 20.0,
           "layers": [_layer(_mixer(5, 5, 10, 6, 0.3, 14), _moe(3, 2, 10, 14)),
                      _layer(_mixer(5, 5, 10, 6, 0.3, 30, kv_from=0), {"kind": "dense", "ff": 50})]},
}


def bf16_round(a: np.ndarray) -> np.ndarray:
    return torch.from_numpy(np.asarray(a, dtype=np.float32)).to(torch.bfloat16).float().numpy()


def make_weights(cfg: dict, seed: int) -> dict[str, np.ndarray]:
    """Seeded weights that bfloat16 holds exactly, as float32 (tables int32), by tensor name."""
    import zinfer_b200 as z
    from zinfer_b200.config.registry import build_model

    rng = np.random.default_rng(seed)
    model = build_model(z.config_from_dict(cfg))
    width = cfg["width"]
    W = {}
    for name, spec in model.weight_specs().items():
        shape = spec.shape
        if spec.role == "table":
            W[name] = np.stack([rng.permutation(spec.bound)[:shape[1]] for _ in range(shape[0])]).astype(np.int32)
        elif name.endswith(".r1"):
            W[name] = bf16_round(rng.uniform(0.2, 1.5, shape))
        elif name.endswith(".r2"):
            W[name] = bf16_round(rng.uniform(0.05, 2.0, shape))
        elif name.endswith(".dwa"):
            W[name] = bf16_round(rng.normal(0, 0.3, shape) + 1.0 / shape[0] + (np.arange(shape[0]) == shape[0] - 1) * 0.5)
        elif "norm" in name:
            W[name] = bf16_round(1.0 + rng.normal(0, 0.2, shape))
        elif name.endswith("canon1"):
            W[name] = bf16_round(rng.normal(0, 0.4, shape))
        elif name.endswith(".sg"):
            W[name] = bf16_round(rng.normal(0, 0.3, shape))
        elif name in ("embed", "pos"):
            W[name] = bf16_round(rng.normal(0, 1.0, shape))
        else:
            W[name] = bf16_round(rng.normal(0, shape[-1] ** -0.5, shape))
    assert width == W["embed"].shape[1]
    return W


def write_folder(folder, cfg: dict, W: dict[str, np.ndarray]) -> Path:
    from zinfer_b200.weights import write_safetensors

    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(cfg))
    tensors = {n: torch.from_numpy(a) if a.dtype == np.int32 else torch.from_numpy(a).to(torch.bfloat16) for n, a in W.items()}
    write_safetensors(folder / "model.safetensors", tensors)
    return folder


def plain_logits(cfg: dict, W: dict[str, np.ndarray], tokens) -> np.ndarray:
    W64 = {n: (a if a.dtype == np.int32 else a.astype(np.float64)) for n, a in W.items()}
    return P.forward(cfg, W64, list(tokens))


def tokens_for(cfg: dict, seed: int, n: int) -> list[int]:
    return np.random.default_rng(seed).integers(0, cfg["vocab"], size=n).tolist()


TOL = {"float32": 5e-5, "bfloat16": 4e-2}


def rel_err(got, ref) -> float:
    got, ref = np.asarray(got, dtype=np.float64), np.asarray(ref, dtype=np.float64)
    scale = float(np.abs(ref).max())
    assert scale > 0 and got.shape == ref.shape, (got.shape, ref.shape)
    return float(np.abs(got - ref).max()) / scale
