"""Zosurax without a GPU: the configuration and its errors, the order of layer runs with a loop, tensor
names and shapes, the cache each run asks for, random model folders, and the plain implementation's
mechanisms against closed forms."""
import dataclasses

import numpy as np
import pytest
import torch

import plain_zosurax as P
import zosurax_helpers as H


def test_configuration_reads_every_key_and_round_trips():
    import zinfer_b200 as z
    for name, d in H.CONFIGS.items():
        c = z.config_from_dict(d)
        assert c.architecture == "Zosurax" and c.vocab_size == d["vocab"] and c.hidden_size == d["width"]
        assert c.norm_eps == d["norm"]["eps"] and len(c.layers) == len(d["layers"])
        assert c.to_json_dict() == d, name
        assert dataclasses.replace(z.config_from_dict(c.to_json_dict()), raw={}) == dataclasses.replace(c, raw={})
    c = z.config_from_dict(H.CONFIGS["zb"])
    assert c.loop is None and c.layers[2].mixer.rot_dims == 0 and c.layers[1].mlp is None
    assert c.layers[0].mixer.rot_dims == 16 and c.layers[0].mixer.scale == 0.2


@pytest.mark.parametrize("change,message", [
    (lambda d: d["layers"][0].update(type="mamba"), "known types"),
    (lambda d: d["layers"][1]["mixer"].update(kv_heads=2), "not a multiple"),
    (lambda d: d["layers"][1]["mixer"]["rot"].update(dims=7), "even"),
    (lambda d: d["layers"][1]["mixer"]["rot"].update(dims=18), "at most dim"),
    (lambda d: d["layers"][1]["mixer"].pop("scale"), "scale"),
    (lambda d: d["loop"].update(stop=4), "stretch"),
    (lambda d: d["loop"].update(times=0), "times"),
    (lambda d: d["layers"][2]["mlp"].update(kind="moe"), "known kinds"),
    (lambda d: d.pop("vocab"), "vocab"),
])
def test_configuration_errors_name_the_key(change, message):
    import copy
    import zinfer_b200 as z
    d = copy.deepcopy(H.CONFIGS["za"])
    change(d)
    with pytest.raises(z.ConfigError, match=message):
        z.config_from_dict(d)


def test_layer_runs_follow_the_loop():
    import zinfer_b200 as z
    runs = {n: z.config_from_dict(d).layer_runs() for n, d in H.CONFIGS.items()}
    assert runs["za"] == [(0, 0), (1, None), (0, 1), (1, None), (2, None)]
    assert runs["zb"] == [(0, None), (1, None), (2, None)]
    assert runs["zc"] == [(0, None), (1, None), (2, 0), (2, 1), (3, None)]
    assert runs["zd"] == [(0, 0)]
    assert runs["ze"] == [(0, None), (1, 0), (1, 1), (1, 2)]
    for n, d in H.CONFIGS.items():
        assert [(i, t) for i, t in P.layer_order(d)] == runs[n]


def test_model_asks_for_the_tensors_of_the_design_and_a_cache_per_run():
    import zinfer_b200 as z
    from zinfer_b200.config.registry import build_model
    model = build_model(z.config_from_dict(H.CONFIGS["za"]))
    specs = model.weight_specs()
    want = {"embed": (97, 40), "final.norm": (40,), "loop.step": (2, 40),
            "l0.norm1": (40,), "l0.norm2": (40,), "l0.shift": (40,), "l0.ls1": (40,), "l0.ls2": (40,),
            "l0.mix.q": (16, 40), "l0.mix.f": (16, 40), "l0.mix.f.b": (16,), "l0.mix.lower": (16,), "l0.mix.v": (24, 40),
            "l0.mix.norm": (12,), "l0.mix.o": (40, 24), "l0.mlp.up": (56, 40), "l0.mlp.down": (40, 56),
            "l1.norm1": (40,), "l1.shift": (40,), "l1.ls1": (40,), "l1.mix.q": (48, 40), "l1.mix.k": (16, 40),
            "l1.mix.v": (24, 40), "l1.mix.q.norm": (16,), "l1.mix.k.norm": (16,), "l1.mix.o": (40, 72),
            "l2.norm1": (40,), "l2.norm2": (40,), "l2.shift": (40,), "l2.ls1": (40,), "l2.ls2": (40,),
            "l2.mix.q": (40, 40), "l2.mix.k": (20, 40), "l2.mix.v": (12, 40), "l2.mix.talk": (4, 4), "l2.mix.o": (40, 24),
            "l2.mlp.up": (48, 40), "l2.mlp.down": (40, 48)}
    assert {n: tuple(s.shape) for n, s in specs.items()} == want
    cache = model.cache_specs()
    assert len(cache) == 5 and [c.kv is None for c in cache] == [True, False, True, False, False]
    # every run keeps the shift's row; the recurrence's runs keep their state [heads * dim * vdim] behind it
    assert [c.state.shape for c in cache] == [(40 + 2 * 8 * 12,), (40,), (40 + 2 * 8 * 12,), (40,), (40,)]
    assert model.pass_input.starts == {0: 0, 2: 1} and model.pass_input.needs_embedding
    from zinfer_b200.cache import CacheManager
    cm = CacheManager(cache, 2, 64, 64, 16, torch.float32, "cpu")
    assert cm.state_view(0).data_ptr() != cm.state_view(2).data_ptr()           # a state per pass
    assert cm.kv_view(1).k.data_ptr() != cm.kv_view(3).k.data_ptr()             # and keys per pass


def test_random_model_folder_holds_what_the_model_asks_for(tmp_path):
    import zinfer_b200 as z
    from zinfer_b200.config.registry import build_model
    from zinfer_b200.weights import SafetensorsFile
    from zinfer_b200.weights.random_init import write_random_model
    cfg = z.config_from_dict(H.CONFIGS["ze"])
    folder = write_random_model(tmp_path / "m", cfg, seed=3, std=0.1)
    assert z.config_from_folder(folder).to_json_dict() == H.CONFIGS["ze"]
    with SafetensorsFile(folder / "model.safetensors") as f:
        lower, mu = f.tensor("l1.mix.lower").float(), f.tensor("l0.shift").float()
        assert set(f.names()) == set(build_model(cfg).weight_specs())
    assert 0 < float(lower.min()) and float(lower.max()) < 1 and 0 < float(mu.min()) and float(mu.max()) < 1


# ------------------------------------------------------------------------------- the plain implementation itself

def test_plain_token_shift():
    h = np.random.default_rng(0).normal(size=(5, 3))
    assert np.allclose(P.token_shift(h, np.zeros(3)), h)
    assert np.allclose(P.token_shift(h, np.ones(3))[1:], h[:-1]) and np.allclose(P.token_shift(h, np.ones(3))[0], 0)


def test_plain_hgrn2_against_its_closed_form():
    """o_t = sum_{s <= t} v_s * sum_i q_t[i] (1 - f_s[i]) prod_{s < r <= t} f_r[i]."""
    rng = np.random.default_rng(1)
    D, H, d, e, T = 6, 2, 3, 4, 7
    p = {"q": rng.normal(size=(H * d, D)), "f": rng.normal(size=(H * d, D)), "f.b": rng.normal(size=H * d),
         "lower": rng.uniform(0, 0.9, H * d), "v": rng.normal(size=(H * e, D)), "norm": np.ones(e), "o": np.eye(H * e)}
    x = rng.normal(size=(T, D))
    got = P.hgrn2(x, p, {"heads": H, "dim": d, "vdim": e}, 1e-6)
    q = P.silu(x @ p["q"].T).reshape(T, H, d)
    f = (p["lower"] + (1 - p["lower"]) * P.sigmoid(x @ p["f"].T + p["f.b"])).reshape(T, H, d)
    v = (x @ p["v"].T).reshape(T, H, e)
    o = np.zeros((T, H, e))
    for t in range(T):
        for s in range(t + 1):
            decay = np.prod(f[s + 1:t + 1], axis=0)                    # [H, d]
            o[t] += np.einsum("hi,he->he", q[t] * (1 - f[s]) * decay, v[s])
    assert np.allclose(got, P.rms(o, 1e-6).reshape(T, H * e))


def test_plain_mixed_heads_reduce_to_plain_attention_with_an_identity_mix():
    rng = np.random.default_rng(2)
    D, H, G, d, e, T = 8, 4, 2, 6, 5, 9
    m = {"heads": H, "kv_heads": G, "dim": d, "vdim": e, "scale": 0.4, "rot": {"base": 30.0, "dims": 4}}
    p = {"q": rng.normal(size=(H * d, D)), "k": rng.normal(size=(G * d, D)), "v": rng.normal(size=(G * e, D)),
         "o": rng.normal(size=(D, H * e)), "talk": np.eye(H), "q.norm": np.ones(d), "k.norm": np.ones(d)}
    x, pos = rng.normal(size=(T, D)), np.arange(T)
    a = P.attention_talking(x, p, m, 1e-6, pos)
    # an unweighted norm commutes with a rotation, so with weights of one the two kinds differ only in the pairing
    q = P.rms(P.rotate((x @ p["q"].T).reshape(T, H, d), pos, 30.0, 4, True), 1e-6)
    k_ = P.rms(P.rotate((x @ p["k"].T).reshape(T, G, d), pos, 30.0, 4, True), 1e-6)
    b = P.apply_weights(P.causal_softmax_weights(q, k_, 0.4), (x @ p["v"].T).reshape(T, G, e)) @ p["o"].T
    assert np.allclose(a, b)
    p["talk"] = np.roll(np.eye(H), 2, axis=1)             # head h takes the weights of head h + 2 (the other group's)
    c = P.attention_talking(x, p, m, 1e-6, pos)
    w = P.causal_softmax_weights(q, k_, 0.4)
    assert np.allclose(c, P.apply_weights(np.roll(w, -2, axis=0), (x @ p["v"].T).reshape(T, G, e)) @ p["o"].T)
    assert not np.allclose(a, c)


def test_plain_rotation_pairs():
    x = np.zeros((1, 1, 6))
    x[0, 0, 0] = 1.0
    pos = np.array([1])
    half = P.rotate(x, pos, 10.0, 4, False)          # pairs (0, 2), (1, 3): the angle of pair 0 is 1 rad
    assert np.allclose(half[0, 0], [np.cos(1), 0, np.sin(1), 0, 0, 0])
    inter = P.rotate(x, pos, 10.0, 4, True)          # pairs (0, 1), (2, 3)
    assert np.allclose(inter[0, 0], [np.cos(1), np.sin(1), 0, 0, 0, 0])
