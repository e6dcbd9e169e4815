"""Zosurax: a pre-norm decoder that mixes three kinds of layers -- an HGRN2 recurrence, softmax attention
with weighted q/k norms before a half-split partial rotation, and softmax attention with an interleaved
rotation, unweighted q/k norms behind it and weights mixed across the heads after the softmax -- each
optionally followed by a dense feed-forward with a squared-relu.  Every mixer reads its normalised input
through a token shift; every sublayer's result is summed through a learned scale per channel; a stretch
of layers may run several times in a row (each pass with a cache and state of its own), and is then given
the embedding's rows again and a learned vector per pass; the head is the embedding table.

Per layer i the tensors are `l<i>.*`.  Every part is a general part of `parts/`; this file only names
tensors and passes the configuration's numbers on."""
from __future__ import annotations

from ..config.registry import register_architecture
from ..config.zosurax import ZosuraxConfig
from ..parts import (ActMlp, GqaAttention, Hgrn2, LMHead, PassInput, PreNormBlock, RMSNorm, RotaryEncoding, TokenEmbedding,
                     TokenShift)
from .model import LayerCall, Model


def build_zosurax(cfg: ZosuraxConfig) -> Model:
    D, eps = cfg.hidden_size, cfg.norm_eps
    embedding = TokenEmbedding(cfg.vocab_size, D, "embed")
    layers = []
    for i, L in enumerate(cfg.layers):
        p, m = f"l{i}.", L.mixer
        a = p + "mix."
        if L.type == "hgrn2":
            mixer = Hgrn2(D, m.heads, m.dim, m.vdim, a + "q", a + "f", a + "f.b", a + "lower", a + "v", a + "norm", a + "o",
                          norm_eps=eps)
        else:
            talking = L.type == "attention_2"
            position = RotaryEncoding(m.dim, m.rot_base, n_rot=m.rot_dims, interleaved=talking) if m.rot_dims else None
            mixer = GqaAttention(D, m.heads, m.kv_heads, m.dim, a + "q", a + "k", a + "v", a + "o",
                                 q_norm_name=None if talking else a + "q.norm",
                                 k_norm_name=None if talking else a + "k.norm", norm_eps=eps, position=position,
                                 scale=m.scale, value_dim=m.vdim, unit_norm_after_rotation=talking,
                                 talk_name=a + "talk" if talking else None)
        ffn = None
        if L.mlp is not None:
            ffn = ActMlp(D, L.mlp.ff, p + "mlp.up", p + "mlp.down", act="relu_squared")
        layers.append(PreNormBlock(RMSNorm(D, eps, p + "norm1"), TokenShift(mixer, D, p + "shift"),
                                   RMSNorm(D, eps, p + "norm2") if ffn is not None else None, ffn,
                                   mixer_scale_name=p + "ls1", ffn_scale_name=p + "ls2" if ffn is not None else None))
    runs = cfg.layer_runs()
    passes = None
    if cfg.loop is not None:
        passes = PassInput("loop.step", cfg.loop.times, D, {c: t for c, (_, t) in enumerate(runs) if t is not None})
    return Model(cfg, embedding, layers, RMSNorm(D, eps, "final.norm"), LMHead(cfg.vocab_size, D, None, embedding),
                 schedule=[LayerCall(layer) for layer, _ in runs], pass_input=passes)


register_architecture("Zosurax", ZosuraxConfig, build_zosurax)
