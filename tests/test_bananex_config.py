"""Bananex without a GPU: the configuration reader, the run order, the tensors a model asks for, random-weight
folders, and properties of the plain implementation that the GPU tests lean on."""
import copy

import numpy as np
import pytest

import bananex_util as bu
import plain_bananex as pb
from cuca_b200.config.bananex_config import BananexConfig
from cuca_b200.config.model_config import ConfigError
from cuca_b200.config.registry import architectures, build_spec
from cuca_b200.models.model import Model
from cuca_b200.models.spec import Between, Run


def test_registered_and_read_from_either_key():
    assert "Bananex" in architectures()
    cfg = copy.deepcopy(bu.CONFIGS["mix"])
    assert build_spec(cfg).architecture == "Bananex"
    cfg["architectures"] = [cfg.pop("architecture")]
    assert build_spec(cfg).architecture == "Bananex"


def test_run_order_and_caches():
    spec = build_spec(bu.CONFIGS["mix"])  # layers 1..2 twice
    runs = [(e.layer, e.cache) if isinstance(e, Run) else ("between", e.arg) for e in spec.schedule]
    assert runs == [(0, 0), ("between", 0), (1, 1), (2, 2), ("between", 1), (1, 3), (2, 4), (3, 5)]
    flat = build_spec(bu.CONFIGS["flat"])
    assert not flat.stream_ops and all(isinstance(e, Run) for e in flat.schedule)
    once = build_spec(bu.CONFIGS["once"])  # a loop of one pass still enters through the remix
    assert isinstance(once.schedule[0], Between) and len(once.schedule) == 3
    empty = copy.deepcopy(bu.CONFIGS["mix"])
    empty["loop"] = {"start": 2, "stop": 2, "times": 3}  # a stretch of no layers: nothing loops, nothing is remixed
    spec = build_spec(empty)
    assert not spec.stream_ops and [e.layer for e in spec.schedule] == [0, 1, 2, 3] and spec.ignorable_tensor("loop.in")
    assert pb.run_order(bu.CONFIGS["mix"]) == [(0, None, False), (1, 0, True), (2, 0, False), (1, 1, True),
                                                (2, 1, False), (3, None, False)]


def test_cache_needs_per_run():
    model = Model(build_spec(bu.CONFIGS["mix"]), runtime=None)
    needs = model.cache_needs()
    assert sorted(needs) == [0, 1, 2, 3, 4, 5]
    assert needs[0].kv.n_kv_heads == 1 and needs[0].kv.head_dim == 40 + 8 and needs[0].kv.window == 12
    assert needs[0].kv.v_head_dim == 0 and set(needs[0].state) == {"shift"}
    assert set(needs[1].state) == {"shift", "mingru"} and needs[1].kv is None
    assert needs[2].state["conv"].shape == (3, 4 * 8 + 2 * 2 * 16) and needs[2].state["ssm"].shape == (4, 8, 16)
    assert needs[5].kv.window == 5
    nomask = Model(build_spec(bu.CONFIGS["loop0"]), runtime=None).cache_needs()
    assert nomask[1].kv.window is None


def test_tensor_names_and_shapes():
    needs = Model(build_spec(bu.CONFIGS["loop0"]), runtime=None).tensor_needs()
    assert needs["loop.in"].shape == (48, 96) and needs["loop.step"].shape == (3, 48)
    assert needs["l0.norm1"].shape == () and needs["final.norm"].shape == ()
    assert needs["l0.mix.in"].shape == (2 * 32 + 2 * 8 + 2, 48) and needs["l0.mix.conv"].shape == (32 + 16, 2)
    assert needs["l1.mix.uk"].shape == (3 * 16, 40) and needs["l1.mix.dkv"].shape == (48, 48)
    assert "l1.mlp.up" not in needs and "l1.norm2" not in needs and "l1.norm1b" in needs  # layer 1 has no feed-forward
    assert needs["l2.mix.z.b"].shape == (40,) and needs["l2.mlp.down.b"].shape == (48,)


@pytest.mark.parametrize("edit, text", [
    (lambda c: c["layers"][0].update(type="lstm"), "type"),
    (lambda c: c["layers"][0]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda c: c["layers"][2]["mixer"].update(groups=3), "groups"),
    (lambda c: c["layers"][2]["mixer"].update(norm_groups=5), "norm groups"),
    (lambda c: c["layers"][0]["mlp"].update(kind="routed"), "kind"),
    (lambda c: c["loop"].update(stop=9), "loop"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), "dims"),
    (lambda c: c.pop("norm"), "eps"),
])
def test_refusals(edit, text):
    cfg = copy.deepcopy(bu.CONFIGS["mix"])
    edit(cfg)
    with pytest.raises(ConfigError, match=text):
        BananexConfig.from_json(cfg)


def test_random_weight_folder(tmp_path):
    from cuca_b200.weights.loader import FolderSource
    from cuca_b200.weights.random_init import write_random_model
    cfg = bu.CONFIGS["once"]
    write_random_model(tmp_path, cfg, seed=3, norm_std=0.2)
    Model(build_spec(cfg), runtime=None).check_weights(FolderSource(tmp_path))


def test_plain_is_causal_and_windows_cut_where_they_should():
    """The plain implementation's own sanity: a later token changes no earlier logits, and with a window of w a
    latent-attention layer alone (no shift, no recurrence) forgets a token exactly w positions later."""
    cfg = bu.CONFIGS["mix"]
    w = bu.plain_weights(bu.make_weights(cfg, 1))
    toks = bu.random_tokens(30, cfg["vocab"], 0)
    a = pb.forward(cfg, w, toks)
    b = pb.forward(cfg, w, toks[:20] + [(t + 1) % cfg["vocab"] for t in toks[20:]])
    assert np.abs(a[:20] - b[:20]).max() == 0 and np.abs(a[20:] - b[20:]).max() > 1e-3
    rs = np.random.default_rng(0)
    layer = bu.latent(window=5)
    m = layer["mixer"]
    ws = {"q": rs.normal(0, .3, (3 * 24, 20)), "dkv": rs.normal(0, .3, (48, 20)), "dkv.norm": np.ones(40),
          "uk": rs.normal(0, .3, (48, 40)), "uv": rs.normal(0, .3, (72, 40)), "g": rs.normal(0, .3, (72, 20)),
          "o": rs.normal(0, .3, (20, 72))}
    h = rs.normal(0, 1, (12, 20))
    h2 = h.copy()
    h2[3] += 1.0
    d = np.abs(pb.latent_attention(h, ws, "", m, 1e-6) - pb.latent_attention(h2, ws, "", m, 1e-6)).max(axis=1)
    assert (d[:3] == 0).all() and (d[3:8] > 0).all() and (d[8:] == 0).all()
    # the candidate of the gated recurrence is continuous where its two branches meet
    assert abs((0.0 + 0.5) - pb.sigmoid(np.array(-1e-12))) < 1e-9
