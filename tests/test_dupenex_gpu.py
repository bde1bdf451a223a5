"""Dupenex on the GPU against the plain implementation (`plain_dupenex.py`): every mechanism alone, whole and cut,
then whole models through the replayer in the four work splits, pages and slots used again, long decoding past
every window, and greedy generation through the entry point and its scheduler."""
import numpy as np
import pytest
import torch

import dupenex_util as du
import plain_dupenex as pd
import replay_util as ru
from test_bananex_gpu import CUTS, _load, _run_cut, _weights_for

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def rt32():
    from cuca_b200.runtime import Runtime
    return Runtime("cuda:0", torch.float32)


def _f32(a, dev):
    return torch.tensor(np.asarray(a), dtype=torch.float32, device=dev)


# ------------------------------------------------------------------------------------------ mechanisms alone
@pytest.mark.parametrize("S, E", [(1, 40), (3, 52), (5, 300), (8, 33), (16, 64), (11, 2052)])
def test_stream_copies_read_and_write(rt32, S, E):
    from cuca_b200.kernels import ops
    dev, eps, rows = rt32.device, 1e-5, 7
    rs = np.random.default_rng(S)
    x = rs.normal(0, 2, (rows, E))
    X = torch.empty(rows, S * E, device=dev)
    ops.spread_streams(_f32(x, dev), X, S)
    assert np.array_equal(X.cpu().numpy().reshape(rows, S, E), np.repeat(x.astype(np.float32)[:, None], S, 1))
    Xn = rs.normal(0, 2, (rows, S, E))
    X = _f32(Xn.reshape(rows, S * E), dev)
    r, o, M = rs.normal(0, 1, S), rs.normal(0, 1, S), rs.normal(0, 1, (S, S))
    w, w2, r2 = 1 + rs.normal(0, 0.3, E), 1 + rs.normal(0, 0.3, E), rs.normal(0, 1, S)
    h = torch.empty(rows, E, device=dev)
    ops.streams_read(X, _f32(r, dev), _f32(w, dev), h, S, eps)
    want = pd.rms(np.einsum("s,rse->re", r, Xn), eps) * w
    assert np.abs(h.cpu().numpy() - want).max() < 1e-5
    gather = torch.tensor([5, 0, 5], dtype=torch.int32, device=dev)
    g = torch.empty(3, E, device=dev)
    ops.streams_read(X, None, _f32(w, dev), g, S, eps, gather)
    assert np.abs(g.cpu().numpy() - (pd.rms(Xn.sum(1), eps) * w)[[5, 0, 5]]).max() < 1e-5
    y = rs.normal(0, 1, (rows, E))
    new = np.einsum("st,rse->rte", M, Xn) + o[None, :, None] * y[:, None, :]
    for nxt in (False, True):
        Xd = X.clone()
        f = torch.empty(rows, E, device=dev) if nxt else None
        ops.streams_write(Xd, _f32(y, dev), _f32(M, dev), _f32(o, dev), S, eps, read2=_f32(r2, dev) if nxt else None,
                          weight2=_f32(w2, dev) if nxt else None, out2=f)
        assert np.abs(Xd.cpu().numpy().reshape(rows, S, E) - new).max() < 2e-5
        if nxt:
            assert np.abs(f.cpu().numpy() - pd.rms(np.einsum("s,rse->re", r2, new), eps) * w2).max() < 2e-5


def test_two_outputs_normed_apart_then_joined(rt32):
    from cuca_b200.kernels import ops
    dev, E, eps = rt32.device, 77, 1e-5
    rs = np.random.default_rng(3)
    x, a, b = (rs.normal(0, s, (9, E)) for s in (1, 3, 0.2))
    wa, wb = 1 + rs.normal(0, 0.3, E), 1 + rs.normal(0, 0.3, E)
    joined = 0.5 * (pd.rms(a, eps) * wa + pd.rms(b, eps) * wb)
    for store in (False, True):
        xd = _f32(x, dev)
        ops.pair_norm_add(xd, _f32(a, dev), _f32(b, dev), _f32(wa, dev), _f32(wb, dev), 0.5, eps, store=store)
        assert np.abs(xd.cpu().numpy() - (joined if store else x + joined)).max() < 1e-5


def _mixer(layer, rt, E, eps):
    from cuca_b200.config.dupenex_config import DupenexConfig
    import cuca_b200.models.model  # noqa: F401  (registers the parts)
    from cuca_b200.models.dupenex import _mixer_spec
    from cuca_b200.parts.base import MIXERS
    cfg = DupenexConfig.from_json(du.config([layer], [None], width=E, eps=eps))
    spec = _mixer_spec(cfg.layers[0], E, eps, "l0.mix.")
    return MIXERS.get(spec.kind)(spec, rt)


def _mixer_weights(part, seed):
    ws = _weights_for(part, seed)
    rs = np.random.default_rng(seed + 1)
    for name in ws:
        if name.endswith(".f.b"):
            ws[name] = rs.normal(2.0, 1.0, ws[name].shape)
        elif name.endswith(".right.i") or name.endswith(".right.f"):
            ws[name] = rs.normal(0.0, 2.0, ws[name].shape) / np.sqrt(ws[name].shape[-1])
    return ws


@pytest.mark.parametrize("layer", [du.delta(), du.delta(heads=3, kv_heads=1, dim=40, vdim=8, conv=1),
                                   du.delta(heads=2, kv_heads=2, dim=128, vdim=96, conv=4, decay_rank=16, gate_rank=8),
                                   du.delta(heads=1, kv_heads=1, dim=7, vdim=150, conv=2),
                                   du.delta(heads=2, kv_heads=1, dim=200, vdim=5, conv=5)])
def test_delta_rule_alone_whole_and_cut(rt32, layer):
    """Three requests in slots 1, 3, 0, whole, one token at a time and in cuts down to two tokens; the state and the
    convolution's kept inputs carry across every cut; slots start from what an earlier run left and are cleared."""
    from cuca_b200.cache.device import CacheView
    dev, E, eps = rt32.device, 44, 1e-5
    part = _mixer(layer, rt32, E, eps)
    ws = _mixer_weights(part, 5)
    _load(part, ws, dev)
    rs = np.random.default_rng(6)
    xs = [rs.normal(0, 1.5, (n, E)) for n in (41, 3, 17)]
    want = [pd.channel_delta(x, ws, "l0.mix.", layer["mixer"], eps) for x in xs]
    needs = part.cache_needs().state
    state = {k: torch.full((4, *v.shape), 7.0, device=dev) for k, v in needs.items()}
    for cuts in ([CUTS[0]] * 3, [CUTS[1], CUTS[2], CUTS[1]], [CUTS[2], CUTS[1], CUTS[2]]):
        for t in state.values():
            t.zero_()  # what the engine does when a slot gets a new request

        def fwd(h, step):
            out = torch.zeros(h.shape[0], E, device=dev)
            part.forward(h, out, step, CacheView(None, None, None, 16, -1, state, step.slots))
            return out
        got = _run_cut(dev, fwd, xs, cuts, [1, 3, 0], E)
        for a, b in zip(got, want):
            assert np.abs(a - b).max() < 3e-5 * max(1.0, np.abs(b).max())


@pytest.mark.parametrize("right", [dict(r_heads=3, r_dim=12, r_vdim=20, cap=6.0), dict(r_heads=1, r_dim=96, r_vdim=40, cap=15.0),
                                   dict(r_heads=2, r_dim=5, r_vdim=130, cap=1.5), dict(r_heads=2, r_dim=260, r_vdim=3, cap=30.0)])
def test_matrix_memory_alone_whole_and_cut(rt32, right):
    from cuca_b200.cache.device import CacheView
    from cuca_b200.parts.recurrent import MatrixLSTM
    dev, E, eps = rt32.device, 36, 1e-5
    layer = du.par(**right)
    whole = _mixer(layer, rt32, E, eps)
    part = whole.sides["right"]
    assert isinstance(part, MatrixLSTM)
    ws = _mixer_weights(part, 9)
    _load(part, ws, dev)
    rs = np.random.default_rng(10)
    xs = [rs.normal(0, 1.5, (n, E)) for n in (50, 2, 19)]
    want = [pd.matrix_memory(x, ws, "l0.mix.right.", layer["mixer"]["right"], eps) for x in xs]
    state = {k: torch.zeros(4, *v.shape, device=dev) for k, v in part.cache_needs().state.items()}
    for cuts in ([CUTS[0]] * 3, [CUTS[1], CUTS[2], CUTS[1]], [CUTS[2], CUTS[1], CUTS[2]]):
        for t in state.values():
            t.zero_()

        def fwd(h, step):
            out = torch.zeros(h.shape[0], E, device=dev)
            part.forward(h, out, step, CacheView(None, None, None, 16, -1, state, step.slots))
            return out
        got = _run_cut(dev, fwd, xs, cuts, [2, 0, 3], E)
        for a, b in zip(got, want):
            assert np.abs(a - b).max() < 3e-5 * max(1.0, np.abs(b).max())


def test_matrix_memory_more_blocks_than_the_gpu_holds(rt32):
    """Forty requests of wide heads in one step: far more blocks than are resident at once, so the last blocks of a
    (head, request) start when its first ones are done. All of them must still start from the same normaliser and
    running maximum, which the step replaces only after every block has read them."""
    from cuca_b200.cache.device import CacheView
    dev, E, eps, R = rt32.device, 24, 1e-5, 40
    layer = du.par(r_heads=4, r_dim=16, r_vdim=520, cap=4.0)
    part = _mixer(layer, rt32, E, eps).sides["right"]
    ws = _mixer_weights(part, 21)
    _load(part, ws, dev)
    rs = np.random.default_rng(22)
    xs = [rs.normal(0, 1.5, (4, E)) for _ in range(R)]
    want = [pd.matrix_memory(x, ws, "l0.mix.right.", layer["mixer"]["right"], eps) for x in xs]
    state = {k: torch.zeros(R, *v.shape, device=dev) for k, v in part.cache_needs().state.items()}

    def fwd(h, step):
        out = torch.zeros(h.shape[0], E, device=dev)
        part.forward(h, out, step, CacheView(None, None, None, 16, -1, state, step.slots))
        return out
    got = _run_cut(dev, fwd, xs, [[1, 1, 2]] * R, list(range(R)), E)
    for a, b in zip(got, want):
        assert np.abs(a - b).max() < 3e-5 * max(1.0, np.abs(b).max())


ATTENTIONS = [du.par(window=12), du.par(window=None, dims=0, heads=3, kv_heads=3),
              du.par(heads=1, kv_heads=1, dim=32, vdim=16, window=1, dims=32),
              du.par(heads=6, kv_heads=2, dim=12, vdim=10, window=16, dims=6, scale=1.2, base=250000.0),
              du.par(heads=2, kv_heads=1, dim=8, vdim=300, window=33, dims=2),
              du.par(heads=2, kv_heads=2, dim=136, vdim=40, window=40, dims=64)]


def _attention(layer, rt, E, eps):
    part = _mixer(layer, rt, E, eps).sides["left"]
    assert part.general
    return part


@pytest.mark.parametrize("layer", ATTENTIONS)
def test_window_attention_alone_whole_and_cut(rt32, layer):
    """Pages of 8 positions handed out in a scrambled order; windows of 1, 12, 16 (two pages exactly), 33 (one past
    four pages), 40 and none; decoding one by one walks every window edge over page borders."""
    from cuca_b200.cache.device import CacheView
    dev, E, eps, bs = rt32.device, 36, 1e-5, 8
    part = _attention(layer, rt32, E, eps)
    m = layer["mixer"]["left"]
    ws = _weights_for(part, 7)
    _load(part, ws, dev)
    part.prepare(128)
    rs = np.random.default_rng(8)
    xs = [rs.normal(0, 1.5, (n, E)) for n in (75, 20)]
    want = [pd.window_attention(x, ws, "l0.mix.left.", m) for x in xs]
    order = rs.permutation(16).tolist()
    for cuts in ([CUTS[0]] * 2, [CUTS[1], CUTS[2]], [CUTS[2], CUTS[1]]):
        kpool = torch.full((16, m["kv_heads"], bs, m["dim"]), float("nan"), device=dev)
        vpool = torch.full((16, m["kv_heads"], bs, m["vdim"]), float("nan"), device=dev)
        tables = torch.full((4, 16), -1, dtype=torch.int32, device=dev)
        tables[2, :10] = torch.tensor(order[:10], dtype=torch.int32)
        tables[0, :3] = torch.tensor(order[10:13], dtype=torch.int32)

        def fwd(h, step):
            out = torch.zeros(h.shape[0], E, device=dev)
            part.forward(h, out, step, CacheView(kpool, vpool, tables, bs, 0, None, step.slots))
            return out
        got = _run_cut(dev, fwd, xs, cuts, [2, 0], E)
        for a, b in zip(got, want):
            assert np.abs(a - b).max() < 2e-5 * max(1.0, np.abs(b).max())
    assert int(rt32.err.item()) == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("dim, vdim", [(16, 24), (64, 128), (32, 96), (128, 128)])
@pytest.mark.parametrize("window, far", [(None, 3), (64, 30), (17, 40), (16, 41)])
def test_one_key_that_matters(dtype, window, far, dim, vdim):
    """A planted key: one unrotated dimension of q reads input column 0 and of k input column 1, both scaled up, and
    only position `far` has column 1 set, so the rows with column 0 set put nearly all their weight on that one key,
    among a hundred others, while they see it. With a window the rows just inside (distance window - 1) and just
    outside (distance window) differ by everything; whole, decoded one by one and in portions that end between them.
    Values as wide as the keys, twice and three times as wide go through the tensor-core kernels in bfloat16 (slab
    by slab), the other sizes and 32-bit through the plain kernel."""
    from cuca_b200.cache.device import CacheView
    from cuca_b200.runtime import Runtime
    rt = Runtime("cuda:0", dtype)
    dev, E, eps, bs, n = rt.device, 40, 1e-5, 8, 120
    layer = du.par(heads=2, kv_heads=1, dim=dim, vdim=vdim, window=window, dims=8, scale=0.25)
    part = _attention(layer, rt, E, eps)
    m = layer["mixer"]["left"]
    ws = {k: du.bf16_round(v) for k, v in _weights_for(part, 13).items()}
    for name in ("l0.mix.left.q", "l0.mix.left.k"):
        ws[name] *= (16.0 / dim) ** 0.5  # the other scores spread by about one whatever the head size
    for head in range(2):
        ws["l0.mix.left.q"][head * dim + dim - 1] = 0.0
        ws["l0.mix.left.q"][head * dim + dim - 1, 0] = 8.0
    ws["l0.mix.left.k"][dim - 1] = 0.0
    ws["l0.mix.left.k"][dim - 1, 1] = 8.0
    needs = part.tensors()
    part.load(lambda name: torch.tensor(ws[name], dtype=torch.float32 if needs[name].keep_fp32 else dtype, device=dev))
    part.prepare(128)
    rs = np.random.default_rng(14)
    x = rs.normal(0, 1.0, (n, E))
    x[:, 0:2] = 0.0
    x[far, 1] = 1.0
    x[far + 1:, 0] = 1.0  # every later row asks for the planted key (score 16 against a spread of about one)
    x = du.bf16_round(x)
    want = pd.window_attention(x, ws, "l0.mix.left.", m)
    edge = far + (window or 1000)  # the first row that no longer sees the key
    if window:
        assert np.abs(want[edge - 1] - want[edge]).max() > 0.3 * np.abs(want[edge - 1]).max()
    tol = 2e-5 if dtype == torch.float32 else 3e-2
    for cuts in ([1000], [far + 2] + [1] * 200, [min(edge, n - 3) - 1, 2, 1000], [min(edge, n - 3), 2, 1, 1, 1000]):
        kpool = torch.zeros((20, 1, bs, dim), dtype=dtype, device=dev)
        vpool = torch.zeros((20, 1, bs, vdim), dtype=dtype, device=dev)
        tables = torch.full((4, 16), -1, dtype=torch.int32, device=dev)
        tables[1, :15] = torch.tensor(rs.permutation(20)[:15].tolist(), dtype=torch.int32)

        def fwd(h, step):
            stream = rt.stream(torch.zeros(h.shape[0], E, device=dev))
            part.forward(h.to(dtype), stream, step, CacheView(kpool, vpool, tables, bs, 0, None, step.slots))
            return stream.data
        got = _run_cut(dev, fwd, [x], [cuts], [1], E)[0]
        assert np.abs(got - want).max() < tol * np.abs(want).max(), cuts


@pytest.mark.parametrize("mlp, E", [(du.moe(ff=24, experts=6, top=2), 48), (du.moe(ff=8, experts=1, top=1), 40),
                                    (du.moe(ff=16, experts=5, top=5), 36), (du.moe(ff=40, experts=37, top=3), 64),
                                    (du.moe(ff=9, experts=130, top=32), 50)])
def test_routed_experts_alone(rt32, mlp, E):
    """Few tokens read only the chosen experts, many tokens run all experts with the unchosen ones weighted 0; both
    against the plain implementation, added to a stream and stored into an unwritten one."""
    from cuca_b200.models.dupenex import _mlp_spec
    from cuca_b200.config.dupenex_config import MlpConfig
    from cuca_b200.parts.mlp import RoutedExperts
    from cuca_b200.runtime import ResidualStream
    dev = rt32.device
    part = RoutedExperts(_mlp_spec(MlpConfig.from_json(mlp, "mlp"), E, "l0.mlp."), rt32)
    rs = np.random.default_rng(E)
    ws = {name: rs.normal(0, 1, need.shape) / np.sqrt(need.shape[-1]) for name, need in part.tensors().items()}
    ws["l0.mlp.router"] *= 4.0
    _load(part, ws, dev)
    for T in (1, 5, part.SPARSE_MAX_TOKENS, part.SPARSE_MAX_TOKENS + 1, 150):
        f = rs.normal(0, 1.5, (T, E))
        want = pd.routed_ff(f, ws, "l0.mlp.", mlp)
        base = rs.normal(0, 1, (T, E))
        x = _f32(base, dev)
        part.forward(_f32(f, dev), x, None)
        assert np.abs(x.cpu().numpy() - (base + want)).max() < 3e-5 * max(1.0, np.abs(want).max())
        y = ResidualStream.unwritten(rt32, T, E)
        part.forward(_f32(f, dev), y, None)
        assert np.abs(y.data.cpu().numpy() - want).max() < 3e-5 * max(1.0, np.abs(want).max())


@pytest.mark.parametrize("mlp, E", [(du.moe(ff=24, experts=6, top=2), 48), (du.moe(ff=64, experts=33, top=5), 64)])
def test_routed_experts_in_bfloat16(mlp, E):
    """Both forms in the serving precision, on the tokens whose choice of experts is clear (the last chosen logit
    well above the first unchosen one): there rounding cannot change the choice."""
    from cuca_b200.config.dupenex_config import MlpConfig
    from cuca_b200.models.dupenex import _mlp_spec
    from cuca_b200.parts.mlp import RoutedExperts
    from cuca_b200.runtime import Runtime
    rt = Runtime("cuda:0", torch.bfloat16)
    dev = rt.device
    part = RoutedExperts(_mlp_spec(MlpConfig.from_json(mlp, "mlp"), E, "l0.mlp."), rt)
    rs = np.random.default_rng(E)
    ws = {name: du.bf16_round(rs.normal(0, 1, need.shape) / np.sqrt(need.shape[-1])) for name, need in part.tensors().items()}
    ws["l0.mlp.router"] = du.bf16_round(ws["l0.mlp.router"] * 4.0)
    part.load(lambda n: torch.tensor(ws[n], dtype=torch.bfloat16, device=dev))
    top = mlp["router"]["top"]
    for T in (7, part.SPARSE_MAX_TOKENS, 200):
        f = du.bf16_round(rs.normal(0, 1.5, (T, E)))
        want = pd.routed_ff(f, ws, "l0.mlp.", mlp)
        z = np.sort(f @ ws["l0.mlp.router"].T, axis=1)[:, ::-1]
        clear = z[:, top - 1] - z[:, top] > 0.1
        assert clear.sum() >= T // 3
        stream = rt.stream(torch.zeros(T, E, device=dev))  # few rows may leave slices pending on it
        part.forward(torch.tensor(f, dtype=torch.bfloat16, device=dev), stream, None)
        got = stream.data.cpu().numpy()
        assert np.abs(got - want)[clear].max() < 3e-2 * np.abs(want).max()


def test_routing_of_rows_that_hold_anything(rt32):
    """A captured step's padding rows hold whatever was in memory: the chosen experts must be experts all the same,
    and distinct ones, since their numbers index the experts' weights."""
    from cuca_b200.kernels import ops
    dev = rt32.device
    z = torch.randn(6, 8, device=dev)
    z[1] = float("nan")
    z[2, 3:] = float("nan")
    z[3] = float("inf")
    z[4] = float("-inf")
    z[5] = 0.0
    for top in (1, 2, 8):
        idx = torch.full((6, top), -7, dtype=torch.int32, device=dev)
        wts = torch.empty(6, top, device=dev)
        ops.moe_route(z, top, idx, wts)
        got = idx.cpu().numpy()
        assert ((got >= 0) & (got < 8)).all()
        assert all(len(set(row)) == top for row in got.tolist())
        assert got[5].tolist() == list(range(top))  # ties go to the lower number
        assert np.isfinite(wts[0].cpu().numpy()).all()


# ------------------------------------------------------------------------------------------ whole models
LENGTHS = {"mix": [1, 2, 5, 16, 33, 64, 97, 130], "plain": [3, 17, 48, 100], "one": [1, 18, 35, 77],
           "wide": [1, 15, 33, 34, 65, 140], "two": [2, 40, 90]}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for i, (name, cfg) in enumerate(du.CONFIGS.items()):
        weights = du.make_weights(cfg, seed=20 + i)
        out[name] = (du.write_model(tmp_path_factory.mktemp(f"dupenex_{name}"), cfg, weights), cfg,
                     du.Oracle(cfg, weights))
    return out


def _requests(name, cfg):
    return {f"r{n}": du.random_tokens(n, cfg["vocab"], seed=300 + n) for n in LENGTHS[name]}


def test_the_stream_after_every_layer_run(models):
    """In 32-bit the sum of the stream's copies after every layer run is the plain implementation's."""
    from cuca_b200.engine.core import EngineCore
    from cuca_b200.engine.step import StepEntry
    for name in ("mix", "plain", "one"):
        folder, cfg, oracle = models[name]
        core = EngineCore.from_folder(folder, dtype="float32", kv_tokens=128, context_length=128, window_pools="full")
        S, E = cfg.get("streams") or 1, cfg["width"]
        seen = []
        core.model.layer_hook = lambda n, stream: seen.append(stream.data.view(-1, S, E).sum(1).cpu().numpy())
        toks = du.random_tokens(29, cfg["vocab"], 4)
        blocks, slot = core.pools.new_seq(), core.slots.alloc()
        core.cache.clear_slot(slot)
        core.pools.reserve(blocks, len(toks))
        core.stepper.step([StepEntry(blocks, slot, toks, [0])])
        want = []
        pd.forward(cfg, oracle.w, toks, want)
        assert len(seen) == len(want) == len(pd.run_order(cfg))
        for a, b in zip(seen, want):
            assert np.abs(a - b).max() < 1e-4 * np.abs(b).max()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(du.CONFIGS))
def test_whole_and_decoded_one_by_one(models, name, dtype):
    folder, cfg, oracle = models[name]
    reqs = _requests(name, cfg)
    for steps in (ru.trace_whole(reqs), ru.trace_tail_one_by_one(reqs, tail=48)):
        got = ru.run_in_process(folder, dtype, steps, ru.peak_tokens(steps), block_size=8)
        du.compare(steps, got, reqs, oracle, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(du.CONFIGS))
def test_portions_down_to_two_tokens(models, name, dtype):
    folder, cfg, oracle = models[name]
    reqs = _requests(name, cfg)
    for sizes in ((5, 2, 17, 3, 2, 32, 7, 2, 64, 11), (2, 2, 3, 1, 1, 8, 9, 40)):
        steps = ru.trace_portions(reqs, sizes=sizes)
        got = ru.run_in_process(folder, dtype, steps, ru.peak_tokens(steps), block_size=16)
        du.compare(steps, got, reqs, oracle, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(du.CONFIGS))
def test_mixed_batches_reuse_pages_and_slots(models, name, dtype):
    """Eight and more requests through four (and three) slots and a pool sized for the peak: every slot and most
    pages serve several requests, whose state must start from zero; windowed groups give pages back as they go."""
    folder, cfg, oracle = models[name]
    reqs = _requests(name, cfg)
    reqs.update({f"s{n}": du.random_tokens(n, cfg["vocab"], seed=900 + n) for n in (4, 9, 23, 31, 58)})
    for live, pools in ((4, "full"), (3, "sized")):
        steps = ru.trace_mixed(reqs, max_live=live, seed=7 + live)
        got = ru.run_in_process(folder, dtype, steps, ru.peak_tokens(steps), block_size=8, window_pools=pools)
        du.compare(steps, got, reqs, oracle, dtype)


def test_32_bit_hardly_depends_on_cuts_or_company(models):
    """In 32-bit a position's logits whole, in portions, decoded and beside other requests differ by rounding alone
    (the routed layers sum a token's experts in another order over few tokens than over many, else they are equal)."""
    folder, cfg, _ = models["mix"]
    reqs = {"a": du.random_tokens(70, cfg["vocab"], 1), "b": du.random_tokens(33, cfg["vocab"], 2)}
    whole = ru.trace_whole(reqs)
    ref = ru.run_in_process(folder, "float32", whole, ru.peak_tokens(whole))
    want = {rid: ref[i] for i, rid in enumerate(reqs)}
    for steps in (ru.trace_portions(reqs, sizes=(3, 2, 9, 1, 1, 30)), ru.trace_mixed(reqs, max_live=2, seed=3)):
        got = ru.run_in_process(folder, "float32", steps, ru.peak_tokens(steps))
        pos = {rid: 0 for rid in reqs}
        for s in steps:
            row = 0
            for e in s["entries"]:
                for w in e["want"]:
                    r = want[e["id"]][pos[e["id"]] + w]
                    assert np.abs(got[s["step"]][row] - r).max() < 2e-5 * np.abs(r).max(), (s["step"], e["id"])
                    row += 1
                pos[e["id"]] += len(e["tokens"])


def test_long_decoding_past_every_window(models):
    folder, cfg, oracle = models["wide"]
    reqs = {"long": du.random_tokens(230, cfg["vocab"], 5)}
    steps = ru.trace_tail_one_by_one(reqs, tail=200)
    for dtype in ("float32", "bfloat16"):
        got = ru.run_in_process(folder, dtype, steps, ru.peak_tokens(steps), block_size=8, window_pools="sized")
        du.compare(steps, got, reqs, oracle, dtype)


def test_long_prompts(models):
    folder, cfg, oracle = models["mix"]
    reqs = {"p": du.random_tokens(610, cfg["vocab"], 8), "q": du.random_tokens(300, cfg["vocab"], 9)}
    for steps in (ru.trace_whole(reqs), ru.trace_portions(reqs, sizes=(7, 300, 2, 280, 1, 64))):
        for dtype in ("bfloat16", "float32"):
            got = ru.run_in_process(folder, dtype, steps, ru.peak_tokens(steps), block_size=16)
            du.compare(steps, got, reqs, oracle, dtype)


def test_trace_run_as_a_program(models):
    folder, cfg, oracle = models["one"]
    reqs = _requests("one", cfg)
    steps = ru.trace_mixed(reqs, max_live=4, seed=1)
    got = ru.run_subprocess(folder, "float32", steps, ru.peak_tokens(steps))
    du.compare(steps, got, reqs, oracle, "float32")


# ------------------------------------------------------------------------------------------ the entry point
def _plain_greedy(cfg, w, prompt, n):
    toks = list(prompt)
    for _ in range(n):
        toks.append(int(np.argmax(pd.forward(cfg, w, toks)[-1])))
    return toks[len(prompt):]


@pytest.mark.parametrize("name", ["mix", "plain"])
def test_greedy_generation_through_the_entry_point(models, name):
    """`LocalModel.generate`: the scheduler admits, cuts prompts into portions, decodes through captured graphs and
    gives slots to later requests; the tokens are the plain implementation's greedy ones."""
    from cuca_b200 import BatchingConfig, LocalModel, LocalModelConfig
    folder, cfg, oracle = models[name]
    prompts = [du.random_tokens(n, cfg["vocab"], seed=40 + n) for n in (3, 50, 21, 9, 70)]
    model = LocalModel.load(LocalModelConfig(source=str(folder), dtype="float32", context_length=256,
                                             batching=BatchingConfig(max_sequences=2, prefill_chunk=16)))
    outs = model.generate(prompts, max_tokens=12, temperature=0.0)
    for prompt, out in zip(prompts, outs):
        assert out.tokens == _plain_greedy(cfg, oracle.w, prompt, 12)


def test_command_line_sampling_and_the_prefix_cache_refusal(models):
    import subprocess
    import sys
    from pathlib import Path

    from cuca_b200 import BatchingConfig, LocalModel, LocalModelConfig
    from cuca_b200.cache.pages import StatefulCacheError
    folder, cfg, oracle = models["two"]
    root = Path(__file__).resolve().parent.parent
    r = subprocess.run([sys.executable, "-m", "cuca_b200", "--model-dir", str(folder), "--prompt", "5 9 20 31",
                        "--max-tokens", "6", "--temperature", "0", "--dtype", "float32"],
                       capture_output=True, text=True, cwd=root, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [int(t) for t in r.stdout.split()] == _plain_greedy(cfg, oracle.w, [5, 9, 20, 31], 6)
    model = LocalModel.load(LocalModelConfig(source=str(folder), dtype="bfloat16", context_length=128))
    prompt = du.random_tokens(20, cfg["vocab"], 77)
    a = model.generate(prompt, max_tokens=16, temperature=1.0, top_k=20, seed=5).tokens
    b = model.generate(prompt, max_tokens=16, temperature=1.0, top_k=20, seed=5).tokens
    c = model.generate(prompt, max_tokens=16, temperature=1.0, top_k=20, seed=6).tokens
    assert a == b and a != c and all(0 <= t < cfg["vocab"] for t in a)
    with pytest.raises(StatefulCacheError):
        LocalModel.load(LocalModelConfig(source=str(folder), dtype="bfloat16", context_length=128,
                                         batching=BatchingConfig(prefix_cache=True)))


def test_bfloat16_generation_through_captured_graphs(models):
    """The serving precision end to end: prompts in portions, decode steps replayed as CUDA graphs. Where two logits
    nearly tie bfloat16 may take the other branch, so every token it takes must be a near-maximum of the plain
    implementation's logits at its place."""
    from cuca_b200 import BatchingConfig, LocalModel, LocalModelConfig
    folder, cfg, oracle = models["two"]
    prompts = [du.random_tokens(n, cfg["vocab"], seed=60 + n) for n in (5, 70, 33)]
    model = LocalModel.load(LocalModelConfig(source=str(folder), dtype="bfloat16", context_length=256,
                                             batching=BatchingConfig(max_sequences=4, prefill_chunk=32)))
    assert model.backend.use_graphs
    outs = model.generate(prompts, max_tokens=40, temperature=0.0)
    assert model.backend.graph_steps > 0
    for prompt, out in zip(prompts, outs):
        ref = pd.forward(cfg, oracle.w, prompt + out.tokens)
        for i, tok in enumerate(out.tokens):
            row = ref[len(prompt) - 1 + i]
            assert float(row.max() - row[tok]) < 0.05 * float(np.abs(row).max()), (i, tok, int(row.argmax()))
