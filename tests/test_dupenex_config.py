"""Dupenex without a GPU: the configuration reader and its refusals, the run order and caches per run, tensor names
and sizes the file decides, a folder of random weights, and properties of the plain implementation itself."""
import copy

import numpy as np
import pytest

import dupenex_util as du
import plain_dupenex as pd
from cuca_b200.config.dupenex_config import DupenexConfig
from cuca_b200.config.model_config import ConfigError
from cuca_b200.config.registry import architectures, build_spec
from cuca_b200.models.model import Model
from cuca_b200.models.spec import Run
from cuca_b200.weights.loader import WeightsError, check_tensors


def test_registered_and_read():
    assert "Dupenex" in architectures()
    cfg = DupenexConfig.from_json(du.CONFIGS["mix"])
    assert cfg.streams == 3 and cfg.loop.times == 2 and len(cfg.layers) == 4
    assert cfg.layers[0].mixer.kv_heads == 2 and cfg.layers[1].mixer.left.window == 12
    assert cfg.layers[1].mlp.kind == "moe" and cfg.layers[1].mlp.top == 2
    assert cfg.run_order() == [0, 1, 2, 1, 2, 3]
    plain = DupenexConfig.from_json(du.CONFIGS["plain"])
    assert plain.streams is None and plain.loop is None and plain.layers[0].mlp is None
    assert plain.layers[0].mixer.left.window is None and plain.layers[0].mixer.left.rot_dims == 0


@pytest.mark.parametrize("path, value", [
    (("layers", 0, "type"), "conv_only"), (("layers", 0, "mixer", "kv_heads"), 3), (("layers", 0, "mixer", "conv"), 0),
    (("layers", 1, "mixer", "left", "rot", "dims"), 7), (("layers", 1, "mixer", "left", "rot", "dims"), 18),
    (("layers", 1, "mixer", "left", "mask", "size"), 0), (("layers", 1, "mixer", "right", "gate_cap"), 0.0),
    (("layers", 1, "mlp", "router", "top"), 9), (("layers", 1, "mlp", "kind"), "sparse"), (("streams",), 0),
    (("loop", "stop"), 7), (("loop", "times"), 0), (("norm",), None), (("layers", 1, "mixer", "right"), None)])
def test_refusals_name_the_key(path, value):
    cfg = copy.deepcopy(du.CONFIGS["mix"])
    node = cfg
    for k in path[:-1]:
        node = node[k]
    node[path[-1]] = value
    with pytest.raises(ConfigError) as e:
        DupenexConfig.from_json(cfg)
    assert str(path[-1]) in str(e.value) or str(path[-2]) in str(e.value)


def test_run_order_and_a_cache_per_run():
    for name, cfg in du.CONFIGS.items():
        spec = build_spec(cfg)
        runs = spec.runs()
        assert [r.layer for r in runs] == pd.run_order(cfg)
        assert [r.cache for r in runs] == list(range(len(runs))) and all(isinstance(r, Run) and r.owns for r in runs)
        needs = Model(spec, runtime=None).cache_needs()
        for r in runs:
            layer = cfg["layers"][r.layer]
            n = needs[r.cache]
            if layer["type"] == "parallel":
                left = layer["mixer"]["left"]
                assert n.kv.n_kv_heads == left["kv_heads"] and n.kv.head_dim == left["dim"]
                assert (n.kv.v_head_dim or n.kv.head_dim) == left["vdim"]
                assert n.kv.window == (left["mask"]["size"] if "mask" in left else None)
                assert set(n.state) == {"right.mem", "right.norm", "right.max"}
            else:
                m = layer["mixer"]
                assert n.kv is None and n.state["delta"].shape == (m["heads"], m["vdim"], m["dim"])
                assert n.state["conv"].shape == (m["conv"] - 1, 2 * m["kv_heads"] * m["dim"] + m["heads"] * m["vdim"])


def test_tensor_names_and_sizes_the_file_decides():
    cfg = du.CONFIGS["mix"]
    model = Model(build_spec(cfg), runtime=None)
    needs = model.tensor_needs()
    for name in ("embed", "head", "final.norm", "l0.norm1", "l0.hc1.in", "l0.hc2.mix", "l0.mix.q.conv", "l0.mix.a2",
                 "l0.mix.dt_bias", "l1.mix.left.g", "l1.mix.left.out", "l1.mix.right.i.b", "l1.mix.right.norm",
                 "l1.mlp.router", "l1.mlp.e5.down", "l0.mlp.gate"):
        assert name in needs, name
    assert "l1.mlp.e6.up" not in needs and needs["l0.hc1.mix"].shape == (3, 3)
    shapes = {n: tuple(t.shape) for n, t in needs.items()}
    check_tensors(needs, shapes)
    # the two low ranks are whatever the file holds ...
    other = dict(shapes)
    other["l0.mix.a1"], other["l0.mix.a2"] = (11, 64), (shapes["l0.mix.a2"][0], 11)
    check_tensors(needs, other)
    # ... every other size is the configuration's
    other["l0.mix.a1"] = (11, 65)
    with pytest.raises(WeightsError) as e:
        check_tensors(needs, other)
    assert [w[0] for w in e.value.wrong_shape] == ["l0.mix.a1"]
    # a layer without feed-forward does not need what stands around one, and does not mind it
    plain = Model(build_spec(du.CONFIGS["one"]), runtime=None)
    pn = {n: tuple(t.shape) for n, t in plain.tensor_needs().items()}
    assert "l1.hc2.in" not in pn and "l1.norm2" not in pn
    pn["l1.norm2"], pn["l1.hc2.in"] = (40,), (1,)
    plain.check_weights(type("S", (), {"shapes": lambda self: pn, "describe": lambda self: ""})())


def test_a_folder_of_random_weights(tmp_path):
    from cuca_b200.weights.loader import FolderSource, write_model_folder
    cfg = du.CONFIGS["two"]
    model = Model(build_spec(cfg), runtime=None)
    write_model_folder(tmp_path, cfg, model.tensor_needs(), seed=3, norm_std=0.2)
    model.check_weights(FolderSource(tmp_path))


# ------------------------------------------------------------------------------------------ the plain implementation
def _w(cfg, seed):
    return du.plain_weights(du.make_weights(cfg, seed))


@pytest.mark.parametrize("name", list(du.CONFIGS))
def test_plain_is_causal_and_carries_state(name):
    """A position's logits do not change when later tokens do, and do change when the first token does (every
    layer kind carries the first token forward, be it through a window of keys or through its state)."""
    cfg = du.CONFIGS[name]
    w = _w(cfg, 1)
    toks = du.random_tokens(30, cfg["vocab"], 2)
    a = pd.forward(cfg, w, toks)
    b = pd.forward(cfg, w, toks[:20] + du.random_tokens(10, cfg["vocab"], 3))
    assert np.array_equal(a[:20], b[:20]) and not np.allclose(a[20:], b[20:])
    c = pd.forward(cfg, w, [(toks[0] + 1) % cfg["vocab"]] + toks[1:])
    assert not np.allclose(a[-1], c[-1])


def test_plain_window_is_its_size_and_no_more():
    m = du.par(window=5, dims=8)["mixer"]["left"]
    rs = np.random.default_rng(0)
    E = 32
    w = {"q": rs.normal(size=(64, E)), "k": rs.normal(size=(32, E)), "v": rs.normal(size=(48, E)),
         "g": rs.normal(size=(96, E)), "o": rs.normal(size=(E, 96))}
    h = rs.normal(size=(12, E))
    out = pd.window_attention(h, w, "", m)
    h2 = h.copy()
    h2[3] += 1.0  # position 3 is seen by positions 3..7
    out2 = pd.window_attention(h2, w, "", m)
    changed = [t for t in range(12) if not np.allclose(out[t], out2[t])]
    assert changed == [3, 4, 5, 6, 7]


def test_plain_experts_chosen_and_weighted():
    mlp = du.moe(ff=4, experts=5, top=2)
    rs = np.random.default_rng(1)
    E = 6
    w = {"router": rs.normal(size=(5, E))}
    for e in range(5):
        w[f"e{e}.up"], w[f"e{e}.down"] = rs.normal(size=(4, E)), rs.normal(size=(E, 4))
    f = rs.normal(size=(3, E))
    z = f @ w["router"].T
    got = pd.routed_ff(f, w, "", mlp)
    for t in range(3):
        best = np.argsort(-z[t])[:2]
        p = np.exp(z[t, best]) / np.exp(z[t, best]).sum()
        want = sum(p[j] * (w[f"e{e}.down"] @ np.maximum(w[f"e{e}.up"] @ f[t], 0) ** 2) for j, e in enumerate(best))
        assert np.allclose(got[t], want)


def test_plain_matrix_memory_first_token_and_cap():
    """At the first token m = max(f, i) against a start of 0, and the gates never leave (-cap, cap)."""
    m = {"heads": 1, "dim": 3, "vdim": 2, "gate_cap": 2.0}
    E = 4
    rs = np.random.default_rng(2)
    w = {k: rs.normal(size=s) for k, s in (("q", (3, E)), ("k", (3, E)), ("v", (2, E)), ("g", (2, E)), ("o", (E, 2)))}
    w["i"], w["f"] = np.full((1, E), 50.0), np.full((1, E), -50.0)
    w["i.b"], w["f.b"], w["norm"] = np.zeros(1), np.zeros(1), np.ones(2)
    h = np.abs(rs.normal(size=(1, E)))
    out = pd.matrix_memory(h, w, "", m, 1e-5)
    q, k, v = w["q"] @ h[0] * 3 ** -0.5, w["k"] @ h[0], w["v"] @ h[0]
    i = 2.0 * np.tanh(50.0 * h.sum() / 2.0)  # capped at 2
    f = -np.logaddexp(0.0, 2.0)  # logsigmoid(-cap)
    mx = max(f + 0.0, i)
    o = np.exp(i - mx) * v * (k @ q) / (max(abs(np.exp(i - mx) * (k @ q)), np.exp(-mx)) + 1e-6)
    o = o / np.sqrt(np.mean(o * o) + 1e-5) * pd.sigmoid(w["g"] @ h[0])
    assert np.allclose(out[0], w["o"] @ o)
