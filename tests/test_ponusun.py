"""Host-side tests of the Ponusun architecture: its configuration reader, the tensors its model asks for,
random model folders, the expert routing of prompt steps, and properties of the plain implementation that
the GPU tests lean on (what a window lets through, that the convolution looks back only)."""
import copy
import json

import numpy as np
import pytest
import torch

import plain_ponusun as P
import ponusun_helpers as H
import zinfer_b200 as z
from zinfer_b200.config import ConfigError, PonusunConfig
from zinfer_b200.config.registry import build_model


def test_configuration_is_read_from_the_nested_keys():
    c = z.config_from_dict(H.CONFIGS["pb"])
    assert isinstance(c, PonusunConfig) and c.architecture == "Ponusun"
    assert (c.vocab_size, c.hidden_size, c.max_position_embeddings, c.canon_taps, c.logit_softcap, c.norm_eps) == (130, 64, 400, 2, 50.0, 1e-5)
    assert [L.mixer.kv_from for L in c.layers] == [None, None, 1, 0]
    assert [L.mixer.window for L in c.layers] == [70, 33, 33, 40]
    assert [(L.mlp.kind, L.mlp.ff, L.mlp.experts, L.mlp.top, L.mlp.shared_ff) for L in c.layers[1:3]] == [("moe", 16, 3, 1, 0), ("moe", 32, 4, 2, 16)]
    d = z.config_from_dict(H.CONFIGS["pd"])       # nothing optional is there
    assert d.canon_taps == 0 and d.logit_softcap is None and d.layers[0].mixer.window == 0 and d.layers[0].mlp is None
    assert d.layers[0].mixer.vdim == 8 and d.layers[0].mixer.dim == 16


@pytest.mark.parametrize("change,text", [
    (lambda c: c.pop("vocab"), "vocab"),
    (lambda c: c["layers"][0]["mixer"].pop("scale"), "scale"),
    (lambda c: c["layers"][1]["mixer"].update(kv_from=1), "no earlier layer"),
    (lambda c: c["layers"][2]["mixer"].update(kv_from=1), "none of its own"),
    (lambda c: c["layers"][1]["mixer"].update(vdim=9), "differ"),
    (lambda c: c["layers"][0]["mlp"].update(kind="sparse"), "known kinds"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=9), "top 9"),
    (lambda c: c["layers"][0].update(type="recurrent"), "known types"),
    (lambda c: c["layers"][0]["mixer"].update(heads=4, kv_heads=3), "multiple"),
    (lambda c: c.update(logit_softcap=-1.0), "positive"),
])
def test_configuration_errors_name_the_key(change, text):
    cfg = copy.deepcopy(H.CONFIGS["pa"])
    change(cfg)
    with pytest.raises(ConfigError, match=text):
        z.config_from_dict(cfg)


def test_model_asks_for_the_tensors_of_its_layers():
    model = build_model(z.config_from_dict(H.CONFIGS["pa"]))
    specs = model.weight_specs()
    assert {"embed", "pos", "head", "final.norm", "l0.canon1", "l0.dwa", "l2.dwa", "l0.mix.q.norm", "l0.mix.k.norm", "l0.mix.r1",
            "l0.mlp.table", "l0.mlp.e4.down", "l0.mlp.shared.sg", "l2.mlp.up"} <= set(specs)
    assert not any(n.startswith(("l1.mix.k", "l1.mix.v", "l1.mlp", "l1.norm2")) for n in specs)      # reads layer 0's cache; no feed-forward
    assert specs["l0.mix.v"].shape == (24, 40) and specs["l0.mix.o"].shape == (40, 72) and specs["l0.mix.q.norm"].shape == (48,)
    assert specs["l2.dwa"].shape == (4,) and specs["l0.mlp.table"].shape == (97, 3) and specs["l0.mlp.table"].role == "table"
    assert specs["pos"].shape == (200, 40) and specs["l0.canon1"].shape == (40, 3) and specs["l0.mlp.shared.sg"].shape == (1, 40)
    assert [(c.layer, c.cache_of) for c in model.schedule] == [(0, None), (1, 0), (2, None)]
    kv = [s.kv for s in model.cache_specs()]
    assert (kv[0].window, kv[1].window, kv[0].v_dim, kv[0].head_dim) == (11, 21, 24, 16)
    assert all(s.state.shape == (2, 40) for s in model.cache_specs())
    none = build_model(z.config_from_dict(H.CONFIGS["pd"]))
    assert "l0.canon1" not in none.weight_specs() and none.cache_specs()[0].state is None


def test_random_model_folder(tmp_path):
    cfg = z.config_from_dict(H.CONFIGS["pe"])
    folder = z.write_random_model(tmp_path / "m", cfg, seed=5, std=0.1)
    assert z.config_from_folder(folder).layers == cfg.layers
    from zinfer_b200.weights import SafetensorsFile
    with SafetensorsFile(folder / "model.safetensors") as f:
        table = f.tensor("l0.mlp.table")
        assert table.dtype == torch.int32 and table.shape == (61, 2)
        assert int(table.min()) >= 0 and int(table.max()) < 2 and all(len(set(r)) == 2 for r in table.tolist())
        one = f.tensor("l1.mlp.table")
        assert one.shape == (61, 1) and int(one.max()) < 3
        assert float(f.tensor("l0.mix.r2").float().min()) >= 0 and f.tensor("embed").dtype == torch.bfloat16
        again = z.write_random_model(tmp_path / "n", cfg, seed=5, std=0.1)
        with SafetensorsFile(again / "model.safetensors") as g:
            assert torch.equal(g.tensor("l0.mlp.table"), table) and torch.equal(g.tensor("head"), f.tensor("head"))


@pytest.mark.parametrize("tile", [1, 4, 128])
def test_expert_rows_of_a_prompt_step(tile):
    from zinfer_b200.parts import TableMoE
    E, top, vocab = 5, 2, 20
    moe = TableMoE(8, 16, E, top, vocab, "t", lambda e: (f"g{e}", f"u{e}", f"d{e}"))
    rng = np.random.default_rng(tile)
    moe.table_host = np.stack([rng.permutation(E)[:top] for _ in range(vocab)]).astype(np.int32)
    moe._set_sort_keys()
    toks = rng.integers(0, vocab, size=37)
    row_token, pair_row, bounds = moe.routing(toks, tile)
    assert bounds[-1] == row_token.size and all((bounds[1:] - bounds[:-1]) % tile == 0)
    assert (row_token >= 0).sum() == 37 * top
    for t in range(37):
        for k in range(top):
            r, e = pair_row[t * top + k], moe.table_host[toks[t]][k]
            assert row_token[r] == t and bounds[e] <= r < bounds[e + 1]
    for e in range(E):      # an expert's rows come first in its stretch, in the order of the tokens; padding behind them
        seg = row_token[bounds[e]:bounds[e + 1]]
        live = seg[seg >= 0]
        assert list(seg[:live.size]) == list(live) == sorted(live)
    # an id outside the vocabulary is the embedding kernel's to flag; here it must only not index outside the table
    moe.routing(np.array([0, 25, -3]), tile)


def test_plain_window_and_convolution_look_where_they_should():
    rng = np.random.default_rng(0)
    D, H_, G, d, vd, W = 24, 2, 1, 8, 6, 5
    Wq, Wk, Wv, Wo = (rng.normal(size=s) for s in ((H_ * d, D), (G * d, D), (G * vd, D), (D, H_ * vd)))
    args = (Wq, Wk, Wv, Wo, np.ones(H_ * d), np.ones(G * d), H_, G, d, vd, 0.4, np.full(H_, 0.5), np.full(H_, 0.7))
    x = rng.normal(size=(12, D))
    y = P.log_distance_attention(x, *args, W, 1e-6)[0]
    moved = x.copy()
    moved[11 - W] += 1.0                                  # distance W from the last query: outside its window
    assert np.allclose(P.log_distance_attention(moved, *args, W, 1e-6)[0][11], y[11])
    moved = x.copy()
    moved[11 - W + 1] += 1.0                              # distance W - 1: the oldest key it sees
    assert not np.allclose(P.log_distance_attention(moved, *args, W, 1e-6)[0][11], y[11])
    assert not np.allclose(P.log_distance_attention(x, *args, 0, 1e-6)[0][11], y[11])      # no window sees more
    # without the bias and with equal keys the weights are uniform: the output is the mean of the values seen
    flat = (np.zeros_like(Wq), Wk, Wv, np.eye(D, H_ * vd), np.ones(H_ * d), np.ones(G * d), H_, G, d, vd, 1.0, np.zeros(H_), np.zeros(H_))
    out = P.log_distance_attention(x, *flat, 3, 1e-6)[0]
    v = x @ Wv.T
    assert np.allclose(out[7][:vd], v[5:8].mean(0))
    c = rng.normal(size=(D, 3))
    h = P.input_conv(x, c)
    assert np.allclose(h[0], x[0] * (1 + c[:, 2])) and np.allclose(h[5], x[5] * (1 + c[:, 2]) + x[4] * c[:, 1] + x[3] * c[:, 0])
    later = x.copy()
    later[6] += 1.0
    assert np.allclose(P.input_conv(later, c)[:6], h[:6])
    assert np.allclose(P.gelu_erf(np.array([0.0, 1.0, -1.0])), [0.0, 0.8413447460685429, -0.15865525393145707])
