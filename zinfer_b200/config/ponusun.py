"""Typed configuration of the Ponusun architecture, read from its own config.json keys.

The file is nested: `vocab`, `width`, `max_positions`, `norm.eps`, `canon.taps`, `logit_softcap`, and
`layers`, a list with one entry per layer: `type` (the mixer kind; "attention" is the one this design
has), `mixer` (heads, kv_heads, dim, vdim, scale, mask.size, optionally kv_from = the layer whose
keys and values it reads) and `mlp` (null, or kind "dense" with ff, or kind "moe" with expert.ff,
router.experts, router.top and optionally shared.ff).  Every size and constant comes from here; what
the file does not mention (no `canon`, no `logit_softcap`, no `mask`, no `shared`) the model does not have.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Optional

from .base import ConfigError, ModelConfig, as_float, as_int, need


@dataclass(frozen=True)
class PonusunMixer:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int = 0                     # mask.size; 0 = every earlier token
    kv_from: Optional[int] = None


@dataclass(frozen=True)
class PonusunMlp:
    kind: str                           # "dense" | "moe"
    ff: int = 0                         # dense: hidden units; moe: hidden units of one expert
    experts: int = 0
    top: int = 0
    shared_ff: int = 0                  # 0 = no shared expert


@dataclass(frozen=True)
class PonusunLayer:
    type: str
    mixer: PonusunMixer
    mlp: Optional[PonusunMlp]


def _section(d: dict, key: str, where: str) -> dict:
    v = d.get(key)
    if v is None:
        return {}
    if not isinstance(v, dict):
        raise ConfigError(f"config.json: '{where}{key}' must be an object")
    return v


@dataclass
class PonusunConfig(ModelConfig):
    layers: tuple[PonusunLayer, ...] = ()
    norm_eps: float = 1e-5
    canon_taps: int = 0                 # 0 = no convolution on the mixers' input
    logit_softcap: Optional[float] = None

    @classmethod
    def from_json_dict(cls, d: dict[str, Any]) -> "PonusunConfig":
        vocab = as_int(d, "vocab", need(d, "vocab"), 1)
        width = as_int(d, "width", need(d, "width"), 1)
        max_pos = as_int(d, "max_positions", need(d, "max_positions"), 1)
        norm = _section(d, "norm", "")
        canon = _section(d, "canon", "")
        raw_layers = need(d, "layers")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, L in enumerate(raw_layers):
            w = f"layers[{i}]."
            if not isinstance(L, dict):
                raise ConfigError(f"config.json: 'layers[{i}]' must be an object")
            m = _section(L, "mixer", w)
            mask = _section(m, "mask", w + "mixer.")
            kv_from = m.get("kv_from")
            dim = as_int(m, w + "mixer.dim", need(m, "dim"), 1)
            mixer = PonusunMixer(
                heads=as_int(m, w + "mixer.heads", need(m, "heads"), 1),
                kv_heads=as_int(m, w + "mixer.kv_heads", need(m, "kv_heads"), 1),
                dim=dim,
                vdim=as_int(m, w + "mixer.vdim", m.get("vdim", dim), 1),
                scale=as_float(w + "mixer.scale", need(m, "scale")),
                window=as_int(mask, w + "mixer.mask.size", mask.get("size") or 0, 0),
                kv_from=None if kv_from is None else as_int(m, w + "mixer.kv_from", kv_from, 0))
            mlp = None
            ml = L.get("mlp")
            if ml is not None:
                if not isinstance(ml, dict):
                    raise ConfigError(f"config.json: '{w}mlp' must be an object or null")
                kind = need(ml, "kind")
                if kind == "dense":
                    mlp = PonusunMlp("dense", ff=as_int(ml, w + "mlp.ff", need(ml, "ff"), 1))
                elif kind == "moe":
                    ex, ro, sh = _section(ml, "expert", w + "mlp."), _section(ml, "router", w + "mlp."), _section(ml, "shared", w + "mlp.")
                    mlp = PonusunMlp("moe", ff=as_int(ex, w + "mlp.expert.ff", need(ex, "ff"), 1),
                                     experts=as_int(ro, w + "mlp.router.experts", need(ro, "experts"), 1),
                                     top=as_int(ro, w + "mlp.router.top", need(ro, "top"), 1),
                                     shared_ff=as_int(sh, w + "mlp.shared.ff", sh.get("ff") or 0, 0))
                else:
                    raise ConfigError(f"config.json: '{w}mlp.kind' = {kind!r}; known kinds are ['dense', 'moe']")
            layers.append(PonusunLayer(str(need(L, "type")), mixer, mlp))
        cap = d.get("logit_softcap")
        eos = d.get("eos_token_id")
        cfg = cls(architecture=str(d.get("architecture") or (d.get("architectures") or ["Ponusun"])[0]),
                  vocab_size=vocab, hidden_size=width, max_position_embeddings=max_pos,
                  eos_token_ids=() if eos is None else tuple(int(e) for e in (eos if isinstance(eos, (list, tuple)) else [eos])),
                  raw=dict(d), layers=tuple(layers),
                  norm_eps=as_float("norm.eps", norm.get("eps", 1e-5)),
                  canon_taps=as_int(canon, "canon.taps", canon.get("taps") or 0, 0),
                  logit_softcap=None if cap is None else as_float("logit_softcap", cap))
        cfg.validate()
        return cfg

    def validate(self) -> None:
        if self.norm_eps <= 0:
            raise ConfigError(f"config.json: norm.eps must be positive, found {self.norm_eps}")
        if self.logit_softcap is not None and self.logit_softcap <= 0:
            raise ConfigError(f"config.json: logit_softcap must be positive, found {self.logit_softcap}")
        for i, L in enumerate(self.layers):
            m = L.mixer
            if L.type != "attention":
                raise ConfigError(f"config.json: layers[{i}].type = {L.type!r}; known types are ['attention']")
            if m.heads % m.kv_heads:
                raise ConfigError(f"config.json: layers[{i}]: {m.heads} heads are not a multiple of {m.kv_heads} kv_heads")
            if m.kv_from is not None:
                if not 0 <= m.kv_from < i:
                    raise ConfigError(f"config.json: layers[{i}].mixer.kv_from = {m.kv_from} is no earlier layer")
                o = self.layers[m.kv_from].mixer
                if o.kv_from is not None:
                    raise ConfigError(f"config.json: layers[{i}] reads the keys of layer {m.kv_from}, which has none of its own")
                if (o.kv_heads, o.dim, o.vdim) != (m.kv_heads, m.dim, m.vdim):
                    raise ConfigError(f"config.json: layers[{i}] and the layer {m.kv_from} whose keys it reads differ in "
                                      "kv_heads, dim or vdim")
            if L.mlp is not None and L.mlp.kind == "moe" and not 0 < L.mlp.top <= L.mlp.experts:
                raise ConfigError(f"config.json: layers[{i}].mlp.router: top {L.mlp.top} of {L.mlp.experts} experts")

    def to_json_dict(self) -> dict[str, Any]:
        layers = []
        for L in self.layers:
            m = L.mixer
            mixer: dict[str, Any] = {"heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "scale": m.scale}
            if m.window:
                mixer["mask"] = {"size": m.window}
            if m.kv_from is not None:
                mixer["kv_from"] = m.kv_from
            mlp: Any = None
            if L.mlp is not None and L.mlp.kind == "dense":
                mlp = {"kind": "dense", "ff": L.mlp.ff}
            elif L.mlp is not None:
                mlp = {"kind": "moe", "expert": {"ff": L.mlp.ff}, "router": {"experts": L.mlp.experts, "top": L.mlp.top}}
                if L.mlp.shared_ff:
                    mlp["shared"] = {"ff": L.mlp.shared_ff}
            layers.append({"type": L.type, "mixer": mixer, "mlp": mlp})
        d: dict[str, Any] = {"architecture": self.architecture, "vocab": self.vocab_size, "width": self.hidden_size,
                             "max_positions": self.max_position_embeddings, "norm": {"eps": self.norm_eps}, "layers": layers}
        if self.canon_taps:
            d["canon"] = {"taps": self.canon_taps}
        if self.logit_softcap is not None:
            d["logit_softcap"] = self.logit_softcap
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        return d
