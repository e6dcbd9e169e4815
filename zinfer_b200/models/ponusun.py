"""Ponusun: a decoder whose layers normalise what a sublayer returns (x += norm(mixer(x)), then
x += norm(ff(x))), whose mixers read x through a short causal convolution over time, and whose
layers hand on a learned mix of all layer results so far instead of their own alone.

Per layer i (tensors `l<i>.*`): windowed grouped-query attention without rotation -- q and k are
RMS-normalised over the whole projection, scores are q.k * scale minus r1_h * ln(1 + r2_h * distance)
-- that may read the keys and values another layer cached (`kv_from`); then no feed-forward, a dense
one (erf gelu), or experts picked by a table over token ids plus a gated shared expert.  Token and
learned position embeddings are summed; the logits are soft-capped.  Every part is a general part of
`parts/`; this file only names tensors and passes the configuration's numbers on."""
from __future__ import annotations

from ..config.ponusun import PonusunConfig
from ..config.registry import register_architecture
from ..parts import (ActMlp, DepthAverage, GqaAttention, InputConv, LMHead, RMSNorm, SublayerNormBlock, SwiGLU, TableMoE,
                     TokenEmbedding)
from .model import LayerCall, Model


def build_ponusun(cfg: PonusunConfig) -> Model:
    D, eps = cfg.hidden_size, cfg.norm_eps
    embedding = TokenEmbedding(cfg.vocab_size, D, "embed", position_name="pos", max_positions=cfg.max_position_embeddings)
    layers, schedule = [], []
    for i, L in enumerate(cfg.layers):
        p, m = f"l{i}.", L.mixer
        a = p + "mix."
        shares = m.kv_from is not None
        mixer = GqaAttention(D, m.heads, m.kv_heads, m.dim, a + "q", a + "k", a + "v", a + "o",
                             q_norm_name=a + "q.norm", k_norm_name=a + "k.norm", norm_eps=eps, window=m.window,
                             scale=m.scale, value_dim=m.vdim, qk_norm_span="all", distance_bias=(a + "r1", a + "r2"),
                             own_kv=not shares)
        if cfg.canon_taps:
            mixer = InputConv(mixer, D, cfg.canon_taps, p + "canon1")
        ffn = None
        if L.mlp is not None and L.mlp.kind == "dense":
            ffn = ActMlp(D, L.mlp.ff, p + "mlp.up", p + "mlp.down", act="gelu_erf")
        elif L.mlp is not None:
            s = p + "mlp.shared."
            shared = SwiGLU(D, L.mlp.shared_ff, s + "gate", s + "up", s + "down") if L.mlp.shared_ff else None
            ffn = TableMoE(D, L.mlp.ff, L.mlp.experts, L.mlp.top, cfg.vocab_size, p + "mlp.table",
                           lambda e, p=p: (f"{p}mlp.e{e}.gate", f"{p}mlp.e{e}.up", f"{p}mlp.e{e}.down"),
                           shared=shared, shared_gate_name=s + "sg" if shared is not None else None)
        layers.append(SublayerNormBlock(mixer, RMSNorm(D, eps, p + "norm1"), ffn,
                                        RMSNorm(D, eps, p + "norm2") if ffn is not None else None))
        schedule.append(LayerCall(i, cache_of=m.kv_from))
    return Model(cfg, embedding, layers, RMSNorm(D, eps, "final.norm"),
                 LMHead(cfg.vocab_size, D, "head", softcap=cfg.logit_softcap), schedule=schedule,
                 depth_mix=DepthAverage([f"l{i}.dwa" for i in range(len(cfg.layers))]))


register_architecture("Ponusun", PonusunConfig, build_ponusun)
