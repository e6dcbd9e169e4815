"""Typed configuration of the Zosurax architecture, read from its own config.json keys.

The file is nested: `vocab`, `width`, `norm.eps`, optionally `loop` {start, stop, times} (layers
start .. stop-1 run `times` times in a row with the same weights) and `layers`, a list with one entry per
layer: `type` (the mixer kind: "hgrn2", "attention" = softmax attention with weighted q/k norms before a
half-split rotation, "attention_2" = interleaved rotation, then unweighted q/k norms, and softmax weights
mixed across the heads), `mixer` (heads, dim, vdim; for the attentions also kv_heads, scale and optionally
rot {base, dims}) and `mlp` (null, or kind "dense" with ff).  Every size and constant comes from here; what
the file does not mention (no `loop`, no `rot`) the model does not have.  The design sets no longest sequence;
`max_positions`, if a file has it, is only the default context of an engine (else DEFAULT_CONTEXT).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Optional

from .base import ConfigError, ModelConfig, as_float, as_int, need

MIXER_TYPES = ("hgrn2", "attention", "attention_2")
DEFAULT_CONTEXT = 8192


@dataclass(frozen=True)
class ZosuraxMixer:
    heads: int
    dim: int
    vdim: int
    kv_heads: int = 0                   # attentions only
    scale: float = 0.0                  # attentions only
    rot_base: float = 0.0               # 0 with rot_dims 0 = no rotation
    rot_dims: int = 0


@dataclass(frozen=True)
class ZosuraxMlp:
    kind: str                           # "dense"
    ff: int


@dataclass(frozen=True)
class ZosuraxLayer:
    type: str
    mixer: ZosuraxMixer
    mlp: Optional[ZosuraxMlp]


@dataclass(frozen=True)
class ZosuraxLoop:
    start: int
    stop: int
    times: int


def _obj(d: dict, key: str, where: str) -> dict:
    v = d.get(key)
    if v is None:
        return {}
    if not isinstance(v, dict):
        raise ConfigError(f"config.json: '{where}{key}' must be an object")
    return v


@dataclass
class ZosuraxConfig(ModelConfig):
    layers: tuple[ZosuraxLayer, ...] = ()
    loop: Optional[ZosuraxLoop] = None
    norm_eps: float = 1e-5

    @classmethod
    def from_json_dict(cls, d: dict[str, Any]) -> "ZosuraxConfig":
        vocab = as_int(d, "vocab", need(d, "vocab"), 1)
        width = as_int(d, "width", need(d, "width"), 1)
        norm = _obj(d, "norm", "")
        raw_layers = need(d, "layers")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, L in enumerate(raw_layers):
            w = f"layers[{i}]."
            if not isinstance(L, dict):
                raise ConfigError(f"config.json: 'layers[{i}]' must be an object")
            kind = str(need(L, "type"))
            if kind not in MIXER_TYPES:
                raise ConfigError(f"config.json: '{w}type' = {kind!r}; known types are {list(MIXER_TYPES)}")
            m = _obj(L, "mixer", w)
            dim = as_int(m, w + "mixer.dim", need(m, "dim"), 1)
            heads = as_int(m, w + "mixer.heads", need(m, "heads"), 1)
            vdim = as_int(m, w + "mixer.vdim", m.get("vdim", dim), 1)
            if kind == "hgrn2":
                mixer = ZosuraxMixer(heads, dim, vdim)
            else:
                rot = _obj(m, "rot", w + "mixer.")
                mixer = ZosuraxMixer(heads, dim, vdim,
                                     kv_heads=as_int(m, w + "mixer.kv_heads", m.get("kv_heads", heads), 1),
                                     scale=as_float(w + "mixer.scale", need(m, "scale")),
                                     rot_base=as_float(w + "mixer.rot.base", need(rot, "base")) if rot else 0.0,
                                     rot_dims=as_int(rot, w + "mixer.rot.dims", need(rot, "dims"), 0) if rot else 0)
            mlp = None
            ml = L.get("mlp")
            if ml is not None:
                if not isinstance(ml, dict):
                    raise ConfigError(f"config.json: '{w}mlp' must be an object or null")
                mk = str(ml.get("kind", "dense"))
                if mk != "dense":
                    raise ConfigError(f"config.json: '{w}mlp.kind' = {mk!r}; known kinds are ['dense']")
                mlp = ZosuraxMlp("dense", as_int(ml, w + "mlp.ff", need(ml, "ff"), 1))
            layers.append(ZosuraxLayer(kind, mixer, mlp))
        loop = None
        lp = _obj(d, "loop", "")
        if lp:
            loop = ZosuraxLoop(as_int(lp, "loop.start", need(lp, "start"), 0), as_int(lp, "loop.stop", need(lp, "stop"), 0),
                               as_int(lp, "loop.times", need(lp, "times"), 1))
        eos = d.get("eos_token_id")
        max_pos = d.get("max_positions")
        cfg = cls(architecture=str(d.get("architecture") or (d.get("architectures") or ["Zosurax"])[0]),
                  vocab_size=vocab, hidden_size=width,
                  max_position_embeddings=DEFAULT_CONTEXT if max_pos is None else as_int(d, "max_positions", max_pos, 1),
                  eos_token_ids=() if eos is None else tuple(int(e) for e in (eos if isinstance(eos, (list, tuple)) else [eos])),
                  raw=dict(d), layers=tuple(layers), loop=loop, norm_eps=as_float("norm.eps", norm.get("eps", 1e-5)))
        cfg.validate()
        return cfg

    def validate(self) -> None:
        if self.norm_eps <= 0:
            raise ConfigError(f"config.json: norm.eps must be positive, found {self.norm_eps}")
        for i, L in enumerate(self.layers):
            m = L.mixer
            if L.type not in MIXER_TYPES:
                raise ConfigError(f"config.json: layers[{i}].type = {L.type!r}; known types are {list(MIXER_TYPES)}")
            if L.type == "hgrn2":
                continue
            if m.heads % m.kv_heads:
                raise ConfigError(f"config.json: layers[{i}]: {m.heads} heads are not a multiple of {m.kv_heads} kv_heads")
            if m.rot_dims % 2 or m.rot_dims > m.dim:
                raise ConfigError(f"config.json: layers[{i}].mixer.rot.dims = {m.rot_dims} must be even and at most dim {m.dim}")
            if m.rot_dims and m.rot_base <= 0:
                raise ConfigError(f"config.json: layers[{i}].mixer.rot.base must be positive, found {m.rot_base}")
        if self.loop is not None:
            lp = self.loop
            if not 0 <= lp.start < lp.stop <= len(self.layers):
                raise ConfigError(f"config.json: loop {lp.start}..{lp.stop} is no stretch of the {len(self.layers)} layers")

    def layer_runs(self) -> list[tuple[int, Optional[int]]]:
        """The order layers run in: (layer, pass number if this run opens a pass of the loop, else None)."""
        n = len(self.layers)
        if self.loop is None:
            return [(i, None) for i in range(n)]
        lp = self.loop
        runs: list[tuple[int, Optional[int]]] = [(i, None) for i in range(lp.start)]
        for t in range(lp.times):
            runs += [(i, t if i == lp.start else None) for i in range(lp.start, lp.stop)]
        return runs + [(i, None) for i in range(lp.stop, n)]

    def to_json_dict(self) -> dict[str, Any]:
        layers = []
        for L in self.layers:
            m = L.mixer
            mixer: dict[str, Any] = {"heads": m.heads, "dim": m.dim, "vdim": m.vdim}
            if L.type != "hgrn2":
                mixer.update(kv_heads=m.kv_heads, scale=m.scale)
                if m.rot_dims:
                    mixer["rot"] = {"base": m.rot_base, "dims": m.rot_dims}
            layers.append({"type": L.type, "mixer": mixer,
                           "mlp": None if L.mlp is None else {"kind": L.mlp.kind, "ff": L.mlp.ff}})
        d: dict[str, Any] = {"architecture": self.architecture, "vocab": self.vocab_size, "width": self.hidden_size,
                             "norm": {"eps": self.norm_eps}, "layers": layers}
        if self.loop is not None:
            d["loop"] = {"start": self.loop.start, "stop": self.loop.stop, "times": self.loop.times}
        if self.max_position_embeddings != DEFAULT_CONTEXT:
            d["max_positions"] = self.max_position_embeddings
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        return d
