"""Seeded random Dupenex configurations (any layer order, sizes off the beaten track, every feature on or off) through
the replayer, whole and in mixed batches, against the plain implementation in both dtypes. In bfloat16 the routed
layers become dense ones of the same size: with many experts a token's router logits nearly tie at the cut so often
that most of a run's difference from the plain implementation would be other experts taken, not arithmetic (the routed
layers' own bfloat16 test compares the tokens whose choice is clear)."""
import copy
import numpy as np
import pytest

import dupenex_util as du
import replay_util as ru

pytestmark = pytest.mark.gpu


def random_config(seed: int) -> dict:
    rs = np.random.default_rng(seed)
    pick = lambda xs: xs[int(rs.integers(len(xs)))]  # noqa: E731
    width = pick([40, 64, 72, 96, 128, 136, 200, 256])
    n_layers = int(rs.integers(2, 6))
    layers, mlps = [], []
    for _ in range(n_layers):
        if rs.random() < 0.55:
            heads = pick([1, 2, 3, 4, 6])
            kv = pick([k for k in (1, 2, 3, 4, 6) if heads % k == 0])
            layers.append(du.delta(heads=heads, kv_heads=kv, dim=pick([8, 12, 16, 24, 32, 48, 64, 96, 128]),
                                   vdim=pick([8, 16, 20, 32, 64, 128, 160]), conv=int(rs.integers(1, 6)),
                                   decay_rank=int(rs.integers(4, 25)), gate_rank=int(rs.integers(4, 25))))
        else:
            heads = pick([1, 2, 4, 6, 8])
            kv = pick([k for k in (1, 2, 4, 8) if heads % k == 0 and k <= heads])
            dim = pick([16, 32, 64, 128])
            vdim = pick([dim // 2, dim, 2 * dim, 3 * dim, dim + 8])
            layers.append(du.par(heads=heads, kv_heads=kv, dim=dim, vdim=vdim,
                                 window=pick([None, 1, 7, 16, 33, 64, 136]), dims=pick([0, 2, dim // 2, dim]),
                                 base=pick([10000.0, 250000.0, 500.0]), scale=pick([None, 0.3, dim ** -0.5 * 2]),
                                 r_heads=pick([1, 2, 3]), r_dim=pick([8, 20, 32, 64, 128]),
                                 r_vdim=pick([8, 24, 48, 64, 130]), cap=pick([1.5, 5.0, 15.0, 30.0])))
        kind = rs.random()
        if kind < 0.2:
            mlps.append(None)
        elif kind < 0.55:
            mlps.append(du.dense(int(rs.integers(3, 40)) * 8))
        else:
            experts = pick([1, 2, 4, 8, 16, 33])
            mlps.append(du.moe(ff=pick([8, 24, 36, 64]), experts=experts, top=int(rs.integers(1, min(experts, 6) + 1))))
    loop = None
    if rs.random() < 0.6:
        a = int(rs.integers(0, n_layers))
        b = int(rs.integers(a, n_layers + 1))
        loop = (a, b, int(rs.integers(1, 4)))
    return du.config(layers, mlps, width=width, vocab=int(rs.integers(50, 700)), streams=pick([None, 1, 2, 3, 4, 6, 8]),
                     loop=loop, eps=pick([1e-5, 1e-6]))


@pytest.mark.parametrize("seed", list(range(10)))
def test_random_configuration(tmp_path, seed):
    for dtype in ("float32", "bfloat16"):
        cfg = random_config(seed)
        if dtype == "bfloat16":
            cfg = copy.deepcopy(cfg)
            for layer in cfg["layers"]:
                if layer["mlp"] and layer["mlp"]["kind"] == "moe":
                    layer["mlp"] = du.dense(layer["mlp"]["expert"]["ff"] * layer["mlp"]["router"]["top"])
        weights = du.make_weights(cfg, seed=100 + seed)
        folder = du.write_model(tmp_path / dtype, cfg, weights)
        oracle = du.Oracle(cfg, weights)
        reqs = {f"r{n}": du.random_tokens(n, cfg["vocab"], seed=7 * seed + n) for n in (1, 2, 19, 41, 70, 150)}
        for steps in (ru.trace_whole(reqs), ru.trace_mixed(reqs, max_live=4, seed=seed)):
            got = ru.run_in_process(folder, dtype, steps, ru.peak_tokens(steps), block_size=16)
            # (eight stream copies through a dozen layer runs, or a first token whose gates nearly cancel, leave
            # 32-bit a few times further from 64-bit than the fixed configurations do)
            du.compare(steps, got, reqs, oracle, dtype, tol32=5e-4)
