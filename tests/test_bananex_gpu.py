"""Bananex on the GPU against the plain implementation (`plain_bananex.py`): every mechanism alone, whole and cut,
then whole models through the replayer in the four work splits, pages and slots used again, long decoding past
every window, and greedy generation through the entry point and its scheduler."""
import numpy as np
import pytest
import torch

import bananex_util as bu
import plain_bananex as pb
import replay_util as ru

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def rt32():
    from cuca_b200.runtime import Runtime
    return Runtime("cuda:0", torch.float32)


def _step(dev, portions, slots):
    """A hand-made step: request i brings rows `portions[i]` = (first position, count), in slot `slots[i]`."""
    from cuca_b200.engine.step import StepBatch
    pos, sor, row0, cnt, start = [], [], [], [], []
    for (p0, n), s in zip(portions, slots):
        row0.append(len(pos))
        pos += list(range(p0, p0 + n))
        sor += [s] * n
        cnt.append(n)
        start.append(p0)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)  # noqa: E731
    return StepBatch(n_rows=len(pos), n_seqs=len(slots), tokens=None, positions=i32(pos), seq_of_row=i32(sor),
                     slots=i32(slots), logit_rows=None, n_logit_rows=0,
                     host={"counts": cnt, "slots": list(slots), "starts": start},
                     req_row0=i32(row0), req_count=i32(cnt), req_start=i32(start))


def _run_cut(dev, forward, inputs, cuts_per_request, slots, width):
    """Feed every request's rows of `inputs` (a list of [T_i, E] arrays) through `forward(h, step) -> [rows, width]`
    in steps that take the next cut of every request that still has one; returns the outputs per request."""
    done = [0] * len(inputs)
    outs = [[] for _ in inputs]
    k = 0
    while any(d < len(x) for d, x in zip(done, inputs)):
        who, portions, rows = [], [], []
        for i, x in enumerate(inputs):
            cuts = cuts_per_request[i]
            if done[i] < len(x) and k < len(cuts):
                n = min(cuts[k], len(x) - done[i])
                who.append(i)
                portions.append((done[i], n))
                rows.append(x[done[i]:done[i] + n])
        step = _step(dev, portions, [slots[i] for i in who])
        h = torch.tensor(np.concatenate(rows), dtype=torch.float32, device=dev)
        out = forward(h, step).cpu().numpy()
        r = 0
        for i, (_, n) in zip(who, portions):
            outs[i].append(out[r:r + n])
            done[i] += n
            r += n
        k += 1
    return [np.concatenate(o) for o in outs]


CUTS = [[1000], [1, 1, 1, 1, 1, 2, 3, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1000],
        [2, 5, 2, 16, 3, 2, 1, 1, 7, 1000]]


# ------------------------------------------------------------------------------------------ mechanisms alone
def test_norm_and_token_shift_alone(rt32):
    from cuca_b200.kernels import ops
    dev, E, eps = rt32.device, 52, 1e-5
    rs = np.random.default_rng(0)
    mix = rs.uniform(0, 1, E)
    gain = 1.3
    xs = [rs.normal(0, 2, (n, E)) for n in (23, 9)]
    want = [pb.token_shift(pb.rms(x, eps) * gain, mix) for x in xs]
    g = torch.tensor([gain], dtype=torch.float32, device=dev)
    m = torch.tensor(mix, dtype=torch.float32, device=dev)
    for cuts in ([CUTS[0], CUTS[0]], [CUTS[1], CUTS[2]], [CUTS[2], CUTS[1]]):
        kept = torch.zeros(4, E, device=dev)
        kept[0] = 7.0  # another request's row must stay as it is

        def fwd(h, step):
            out = torch.empty_like(h)
            ops.norm_shift(h, g, eps, m, kept, out, step)
            return out
        got = _run_cut(dev, fwd, xs, cuts, [2, 3], E)
        for a, b in zip(got, want):
            assert np.abs(a - b).max() < 1e-5
        assert torch.equal(kept[0].cpu(), torch.full((E,), 7.0))
    # a vector gain through the same kernel
    gv = rs.normal(1, 0.2, E)
    kept = torch.zeros(4, E, device=dev)
    out = torch.empty(23, E, device=dev)
    ops.norm_shift(torch.tensor(xs[0], dtype=torch.float32, device=dev), torch.tensor(gv, dtype=torch.float32, device=dev),
                   eps, m, kept, out, _step(dev, [(0, 23)], [1]))
    assert np.abs(out.cpu().numpy() - pb.token_shift(pb.rms(xs[0], eps) * gv, mix)).max() < 1e-5


def test_post_norm_add_alone(rt32):
    from cuca_b200.kernels import ops
    dev, E, eps = rt32.device, 70, 1e-6
    rs = np.random.default_rng(1)
    x, y = rs.normal(0, 1, (11, E)), rs.normal(0, 3, (11, E))
    xd = torch.tensor(x, dtype=torch.float32, device=dev)
    out = torch.empty(11, E, device=dev)
    g1, g2 = torch.tensor([0.8], device=dev), torch.tensor([1.7], device=dev)
    ops.post_norm_add(xd, torch.tensor(y, dtype=torch.float32, device=dev), g1, eps, gain2=g2, out=out)
    nx = x + pb.rms(y, eps) * 0.8
    assert np.abs(xd.cpu().numpy() - nx).max() < 1e-5
    assert np.abs(out.cpu().numpy() - pb.rms(nx, eps) * 1.7).max() < 1e-5


def _part(kind, cls, layer, rt, E, eps, prefix="l0.mix."):
    from cuca_b200.config.bananex_config import BananexConfig
    from cuca_b200.models.bananex import _mixer_spec
    cfg = BananexConfig.from_json(bu.config([layer], width=E, eps=eps))
    spec = _mixer_spec(cfg.layers[0], E, eps, prefix)
    assert spec.kind == kind
    return cls(spec, rt)


def _weights_for(part, seed):
    rs = np.random.default_rng(seed)
    ws = {}
    for name, need in part.tensors().items():
        shape = tuple(need.shape)
        if name.endswith("A_log"):
            v = rs.uniform(-1.5, 1.0, shape)
        elif name.endswith("dt_bias"):
            v = rs.uniform(-2, 1, shape)
        elif need.init == "ones" or name.endswith(".D"):
            v = 1 + rs.normal(0, 0.3, shape)
        elif len(shape) == 1:
            v = rs.normal(0, 0.3, shape)
        elif name.endswith(".conv"):
            v = rs.normal(0, 0.5, shape)
        else:
            v = rs.normal(0, 1, shape) / np.sqrt(shape[-1])
        ws[name] = np.asarray(v, dtype=np.float32).astype(np.float64)
    return ws


def _load(part, ws, dev):
    part.load(lambda n: torch.tensor(ws[n], dtype=torch.float32, device=dev))


@pytest.mark.parametrize("inner", [48, 130])
def test_mingru_alone_whole_and_cut(rt32, inner):
    from cuca_b200.parts.recurrent import MinGRU
    dev, E = rt32.device, 40
    part = _part("mingru", MinGRU, bu.mingru(inner), rt32, E, 1e-5)
    ws = _weights_for(part, 3)
    _load(part, ws, dev)
    rs = np.random.default_rng(4)
    xs = [rs.normal(0, 1.5, (n, E)) for n in (37, 12, 5)]
    want = [pb.mingru(x, ws, "l0.mix.", {"width": inner}) for x in xs]
    for cuts in ([CUTS[0]] * 3, [CUTS[1], CUTS[2], CUTS[1]], [CUTS[2], CUTS[1], CUTS[0]]):
        state = torch.zeros(4, inner, device=dev)

        def fwd(h, step):
            from cuca_b200.cache.device import CacheView
            out = torch.zeros(h.shape[0], E, device=dev)
            part.forward(h, out, step, CacheView(None, None, None, 16, -1, {"mingru": state}, step.slots))
            return out
        got = _run_cut(dev, fwd, xs, cuts, [3, 0, 2], E)
        for a, b in zip(got, want):
            assert np.abs(a - b).max() < 2e-5 * max(1.0, np.abs(b).max())


def test_mingru_long_portions_in_chunks():
    """In bfloat16 a portion of 256 tokens or more runs as chunks side by side with the state carried across
    them: whole, and cut so that a chunked portion starts from a state that single tokens left."""
    from cuca_b200.cache.device import CacheView
    from cuca_b200.kernels import ops
    from cuca_b200.parts.recurrent import MinGRU
    from cuca_b200.runtime import Runtime
    rt = Runtime("cuda:0", torch.bfloat16)
    dev, E, inner = rt.device, 40, 70
    part = _part("mingru", MinGRU, bu.mingru(inner), rt, E, 1e-5)
    ws = {k: bu.bf16_round(v) for k, v in _weights_for(part, 3).items()}
    part.load(lambda n: torch.tensor(ws[n], dtype=torch.bfloat16, device=dev))
    rs = np.random.default_rng(4)
    xs = [bu.bf16_round(rs.normal(0, 1.5, (n, E))) for n in (700, 300)]
    want = [pb.mingru(x, ws, "l0.mix.", {"width": inner}) for x in xs]
    assert ops.MINGRU_CHUNKED_FROM <= 256
    for cuts in ([CUTS[0]] * 2, [[1, 1, 3, 290, 1, 1, 1000], [260, 1, 1000]]):
        state = torch.zeros(4, inner, device=dev)

        def fwd(h, step):
            stream = rt.stream(torch.zeros(h.shape[0], E, device=dev))
            part.forward(h.to(torch.bfloat16), stream, step, CacheView(None, None, None, 16, -1, {"mingru": state}, step.slots))
            return stream.data
        got = _run_cut(dev, fwd, xs, cuts, [2, 1], E)
        for a, b in zip(got, want):
            assert np.abs(a - b).max() < 3e-2 * np.abs(b).max()


@pytest.mark.parametrize("layer", [bu.mamba2(), bu.mamba2(heads=3, vdim=20, state=40, groups=3, conv=1, norm_groups=3),
                                   bu.mamba2(heads=2, vdim=64, state=128, groups=1, conv=7, norm_groups=1),
                                   bu.mamba2(heads=4, vdim=12, state=6, groups=4, conv=2, norm_groups=4)])
def test_mamba2_alone_whole_and_cut(rt32, layer):
    from cuca_b200.parts.recurrent import Mamba2
    dev, E, eps = rt32.device, 44, 1e-5
    part = _part("mamba2", Mamba2, layer, rt32, E, eps)
    ws = _weights_for(part, 5)
    _load(part, ws, dev)
    rs = np.random.default_rng(6)
    xs = [rs.normal(0, 1.5, (n, E)) for n in (41, 3, 17)]
    want = [pb.mamba2(x, ws, "l0.mix.", layer["mixer"], eps) for x in xs]
    needs = part.cache_needs().state
    for cuts in ([CUTS[0]] * 3, [CUTS[1], CUTS[2], CUTS[1]], [CUTS[2], CUTS[1], CUTS[2]]):
        state = {k: torch.zeros(4, *v.shape, device=dev) for k, v in needs.items()}

        def fwd(h, step):
            from cuca_b200.cache.device import CacheView
            out = torch.zeros(h.shape[0], E, device=dev)
            part.forward(h, out, step, CacheView(None, None, None, 16, -1, state, step.slots))
            return out
        got = _run_cut(dev, fwd, xs, cuts, [1, 3, 0], E)
        for a, b in zip(got, want):
            assert np.abs(a - b).max() < 3e-5 * max(1.0, np.abs(b).max())


@pytest.mark.parametrize("layer", [bu.latent(window=12), bu.latent(window=None, dims=4),
                                   bu.latent(heads=1, dim=32, rot_dim=4, vdim=16, kv_rank=136, window=1),
                                   bu.latent(heads=5, dim=12, rot_dim=6, vdim=10, kv_rank=33, window=16, scale=1.2),
                                   bu.latent(heads=2, dim=8, rot_dim=16, vdim=8, kv_rank=300, window=33)])
def test_latent_attention_alone_whole_and_cut(rt32, layer):
    """Pages of 8 positions handed out in a scrambled order; windows of 1, 12, 16 (two pages exactly), 33 (one past
    four pages) and none; decoding one by one walks every window edge over page borders."""
    from cuca_b200.cache.device import CacheView
    from cuca_b200.parts.latent_attention import LatentAttention
    dev, E, eps, bs = rt32.device, 36, 1e-5, 8
    part = _part("latent_attention", LatentAttention, layer, rt32, E, eps)
    ws = _weights_for(part, 7)
    _load(part, ws, dev)
    part.prepare(128)
    rs = np.random.default_rng(8)
    xs = [rs.normal(0, 1.5, (n, E)) for n in (75, 20)]
    want = [pb.latent_attention(x, ws, "l0.mix.", layer["mixer"], eps) for x in xs]
    order = rs.permutation(16).tolist()
    for cuts in ([CUTS[0]] * 2, [CUTS[1], CUTS[2]], [CUTS[2], CUTS[1]]):
        pool = torch.full((16, 1, bs, part.key_dim), float("nan"), device=dev)
        tables = torch.full((4, 16), -1, dtype=torch.int32, device=dev)
        tables[2, :10] = torch.tensor(order[:10], dtype=torch.int32)
        tables[0, :3] = torch.tensor(order[10:13], dtype=torch.int32)

        def fwd(h, step):
            out = torch.zeros(h.shape[0], E, device=dev)
            part.forward(h, out, step, CacheView(pool, None, tables, bs, 0, None, step.slots))
            return out
        got = _run_cut(dev, fwd, xs, cuts, [2, 0], E)
        for a, b in zip(got, want):
            assert np.abs(a - b).max() < 2e-5 * max(1.0, np.abs(b).max())
    assert int(rt32.err.item()) == 0


@pytest.mark.parametrize("layer", [
    bu.latent(heads=3, dim=16, rot_dim=16, vdim=24, kv_rank=64, window=20, scale=1.0),
    bu.latent(heads=20, dim=8, rot_dim=32, vdim=8, kv_rank=96, window=None, scale=0.8),
    bu.latent(heads=2, dim=24, rot_dim=16, vdim=12, kv_rank=256, window=70, scale=0.9),
    bu.latent(heads=1, dim=8, rot_dim=64, vdim=8, kv_rank=512, window=130, scale=1.0),
    bu.latent(heads=16, dim=16, rot_dim=0, vdim=8, kv_rank=32, window=64, scale=1.0)])
def test_latent_attention_on_tensor_cores(layer):
    """The bfloat16 forms: prompts in groups of 16 tokens per head, single tokens with their heads as the group.
    Scales near one make the softmax pick few keys, so a key that is dropped, seen too early or too late moves
    the result by far more than rounding does. 200 tokens walk windows over several key tiles and page borders."""
    from cuca_b200.cache.device import CacheView
    from cuca_b200.kernels import ops
    from cuca_b200.parts.latent_attention import LatentAttention
    from cuca_b200.runtime import Runtime
    rt = Runtime("cuda:0", torch.bfloat16)
    dev, E, eps, bs = rt.device, 48, 1e-5, 16
    part = _part("latent_attention", LatentAttention, layer, rt, E, eps)
    assert ops.latent_attention_mma_supported(part.rank, part.key_dim)
    ws = {k: bu.bf16_round(v) for k, v in _weights_for(part, 11).items()}
    needs = part.tensors()
    part.load(lambda n: torch.tensor(ws[n], dtype=torch.float32 if needs[n].keep_fp32 else torch.bfloat16, device=dev))
    part.prepare(256)
    rs = np.random.default_rng(12)
    xs = [bu.bf16_round(rs.normal(0, 1.5, (n, E))) for n in (200, 37)]
    want = [pb.latent_attention(x, ws, "l0.mix.", layer["mixer"], eps) for x in xs]
    pb.ROUND = bu.bf16_round
    try:
        rounded = [pb.latent_attention(x, ws, "l0.mix.", layer["mixer"], eps) for x in xs]
    finally:
        pb.ROUND = None
    tol = [max(2e-2 * np.abs(b).max(), 4 * np.abs(a - b).max()) for a, b in zip(rounded, want)]
    order = rs.permutation(20).tolist()
    for cuts in ([CUTS[0]] * 2, [[150] + CUTS[1], CUTS[2]], [[3, 64, 17, 90] + CUTS[1], CUTS[1]]):
        pool = torch.full((20, 1, bs, part.key_dim), float("nan"), dtype=torch.bfloat16, device=dev)
        tables = torch.full((4, 16), -1, dtype=torch.int32, device=dev)
        tables[1, :13] = torch.tensor(order[:13], dtype=torch.int32)
        tables[3, :3] = torch.tensor(order[13:16], dtype=torch.int32)

        def fwd(h, step):
            stream = rt.stream(torch.zeros(h.shape[0], E, device=dev))  # few rows may leave slices pending on it
            part.forward(h.to(torch.bfloat16), stream, step, CacheView(pool, None, tables, bs, 0, None, step.slots))
            return stream.data
        got = _run_cut(dev, fwd, xs, cuts, [1, 3], E)
        for a, b, t in zip(got, want, tol):
            assert np.isfinite(a).all() and np.abs(a - b).max() < t, (np.abs(a - b).max(), t)
    assert int(rt.err.item()) == 0


def test_dense_feed_forward_and_loop_entry_alone(rt32):
    from cuca_b200.parts.base import PartSpec
    from cuca_b200.parts.mlp import DenseActivation
    from cuca_b200.parts.stream_ops import LoopEntry
    dev, E, F = rt32.device, 28, 50
    rs = np.random.default_rng(9)
    ff = DenseActivation(PartSpec("dense_act", {"width": E, "inner": F, "act": "gelu", "bias": True},
                                  {"up": "m.up", "up_bias": "m.up.b", "down": "m.down", "down_bias": "m.down.b"}), rt32)
    ws = {"m.up": rs.normal(0, 0.4, (F, E)), "m.up.b": rs.normal(0, 0.5, F), "m.down": rs.normal(0, 0.3, (E, F)),
          "m.down.b": rs.normal(0, 0.5, E)}
    _load(ff, ws, dev)
    h = rs.normal(0, 1.5, (13, E))
    out = torch.zeros(13, E, device=dev)
    ff.forward(torch.tensor(h, dtype=torch.float32, device=dev), out, None)
    assert np.abs(out.cpu().numpy() - pb.dense_ff(h, ws, "m.")).max() < 2e-5
    op = LoopEntry(PartSpec("loop_entry", {"width": E, "times": 3}, {"mix": "loop.in", "step": "loop.step"}), rt32)
    wl = {"loop.in": rs.normal(0, 0.3, (E, 2 * E)), "loop.step": rs.normal(0, 1, (3, E))}
    _load(op, wl, dev)
    x, e = rs.normal(0, 1, (13, E)), rs.normal(0, 1, (13, E))
    stream = rt32.stream(torch.tensor(x, dtype=torch.float32, device=dev))
    ed = torch.tensor(e, dtype=torch.float32, device=dev)
    op.forward(stream, ed, None, 2)
    assert np.abs(stream.data.cpu().numpy() - (np.concatenate([x, e], 1) @ wl["loop.in"].T + wl["loop.step"][2])).max() < 2e-5
    assert np.array_equal(ed.cpu().numpy(), e.astype(np.float32))  # the embedding output is only read


# ------------------------------------------------------------------------------------------ whole models
LENGTHS = {"wide": [1, 15, 16, 17, 63, 65, 140], "mix": [1, 2, 5, 16, 33, 64, 97, 130], "loop0": [3, 17, 48, 100], "flat": [2, 40, 41, 42, 90, 150],
           "once": [1, 18, 35, 77]}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for i, (name, cfg) in enumerate(bu.CONFIGS.items()):
        weights = bu.make_weights(cfg, seed=20 + i)
        out[name] = (bu.write_model(tmp_path_factory.mktemp(f"bananex_{name}"), cfg, weights), cfg,
                     bu.Oracle(cfg, weights))
    return out


def _requests(name, cfg):
    return {f"r{n}": bu.random_tokens(n, cfg["vocab"], seed=300 + n) for n in LENGTHS[name]}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(bu.CONFIGS))
def test_whole_and_decoded_one_by_one(models, name, dtype):
    folder, cfg, oracle = models[name]
    reqs = _requests(name, cfg)
    for steps in (ru.trace_whole(reqs), ru.trace_tail_one_by_one(reqs, tail=48)):
        got = ru.run_in_process(folder, dtype, steps, ru.peak_tokens(steps), block_size=8)
        ru.compare(steps, got, reqs, oracle, oracle.tolerance(dtype, reqs))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(bu.CONFIGS))
def test_portions_down_to_two_tokens(models, name, dtype):
    folder, cfg, oracle = models[name]
    reqs = _requests(name, cfg)
    for sizes in ((5, 2, 17, 3, 2, 32, 7, 2, 64, 11), (2, 2, 3, 1, 1, 8, 9, 40)):
        steps = ru.trace_portions(reqs, sizes=sizes)
        got = ru.run_in_process(folder, dtype, steps, ru.peak_tokens(steps), block_size=16)
        ru.compare(steps, got, reqs, oracle, oracle.tolerance(dtype, reqs))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(bu.CONFIGS))
def test_mixed_batches_reuse_pages_and_slots(models, name, dtype):
    """Eight and more requests through four (and three) slots and a pool sized for the peak: every slot and most
    pages serve several requests, whose state must start from zero; windowed groups give pages back as they go."""
    folder, cfg, oracle = models[name]
    reqs = _requests(name, cfg)
    reqs.update({f"s{n}": bu.random_tokens(n, cfg["vocab"], seed=900 + n) for n in (4, 9, 23, 31, 58)})
    for live, pools in ((4, "full"), (3, "sized")):
        steps = ru.trace_mixed(reqs, max_live=live, seed=7 + live)
        got = ru.run_in_process(folder, dtype, steps, ru.peak_tokens(steps), block_size=8, window_pools=pools)
        ru.compare(steps, got, reqs, oracle, oracle.tolerance(dtype, reqs))


def test_32_bit_does_not_depend_on_cuts_or_company(models):
    """In 32-bit a position's logits are the same bits whole, in portions, decoded and beside other requests."""
    folder, cfg, _ = models["mix"]
    reqs = {"a": bu.random_tokens(70, cfg["vocab"], 1), "b": bu.random_tokens(33, cfg["vocab"], 2)}
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
                    assert np.array_equal(got[s["step"]][row], want[e["id"]][pos[e["id"]] + w]), (s["step"], e["id"])
                    row += 1
                pos[e["id"]] += len(e["tokens"])


def test_long_decoding_past_every_window(models):
    folder, cfg, oracle = models["flat"]
    reqs = {"long": bu.random_tokens(230, cfg["vocab"], 5)}
    steps = ru.trace_tail_one_by_one(reqs, tail=200)
    for dtype in ("float32", "bfloat16"):
        got = ru.run_in_process(folder, dtype, steps, ru.peak_tokens(steps), block_size=8, window_pools="sized")
        ru.compare(steps, got, reqs, oracle, oracle.tolerance(dtype, reqs))


def test_long_prompts(models):
    """Prompts long enough for the forms that only long portions take (chunks of the gated recurrence side by side,
    many key tiles per group of the tensor-core attention), whole and in portions that start inside a chunk."""
    folder, cfg, oracle = models["wide"]
    reqs = {"p": bu.random_tokens(610, cfg["vocab"], 8), "q": bu.random_tokens(300, cfg["vocab"], 9)}
    for steps in (ru.trace_whole(reqs), ru.trace_portions(reqs, sizes=(7, 300, 2, 280, 1, 64))):
        for dtype in ("bfloat16", "float32"):
            got = ru.run_in_process(folder, dtype, steps, ru.peak_tokens(steps), block_size=16)
            ru.compare(steps, got, reqs, oracle, oracle.tolerance(dtype, reqs))


def test_trace_run_as_a_program(models):
    folder, cfg, oracle = models["loop0"]
    reqs = _requests("loop0", cfg)
    steps = ru.trace_mixed(reqs, max_live=4, seed=1)
    got = ru.run_subprocess(folder, "float32", steps, ru.peak_tokens(steps))
    ru.compare(steps, got, reqs, oracle, oracle.tolerance("float32", reqs))


# ------------------------------------------------------------------------------------------ the entry point
def _plain_greedy(cfg, w, prompt, n):
    toks = list(prompt)
    for _ in range(n):
        toks.append(int(np.argmax(pb.forward(cfg, w, toks)[-1])))
    return toks[len(prompt):]


@pytest.mark.parametrize("name", ["mix", "flat"])
def test_greedy_generation_through_the_entry_point(models, name):
    """`LocalModel.generate`: the scheduler admits, cuts prompts into portions, decodes through captured graphs and
    gives slots to later requests; the tokens are the plain implementation's greedy ones."""
    from cuca_b200 import BatchingConfig, LocalModel, LocalModelConfig
    folder, cfg, oracle = models[name]
    prompts = [bu.random_tokens(n, cfg["vocab"], seed=40 + n) for n in (3, 50, 21, 9, 70)]
    model = LocalModel.load(LocalModelConfig(source=str(folder), dtype="float32", context_length=256,
                                             batching=BatchingConfig(max_sequences=2, prefill_chunk=16)))
    outs = model.generate(prompts, max_tokens=12, temperature=0.0)
    for prompt, out in zip(prompts, outs):
        assert out.tokens == _plain_greedy(cfg, oracle.w, prompt, 12)
    stats = model.serving_stats()
    assert stats is not None


def test_command_line_sampling_and_the_prefix_cache_refusal(models):
    """`python -m cuca_b200` on a Bananex folder; seeded sampling is repeatable and differs from greedy somewhere;
    the prefix cache is refused (the layers keep state that cached pages do not bring back)."""
    import subprocess
    import sys
    from pathlib import Path

    from cuca_b200 import BatchingConfig, LocalModel, LocalModelConfig
    from cuca_b200.cache.pages import StatefulCacheError
    folder, cfg, oracle = models["once"]
    root = Path(__file__).resolve().parent.parent
    r = subprocess.run([sys.executable, "-m", "cuca_b200", "--model-dir", str(folder), "--prompt", "5 9 20 31",
                        "--max-tokens", "6", "--temperature", "0", "--dtype", "float32"],
                       capture_output=True, text=True, cwd=root, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [int(t) for t in r.stdout.split()] == _plain_greedy(cfg, oracle.w, [5, 9, 20, 31], 6)
    model = LocalModel.load(LocalModelConfig(source=str(folder), dtype="bfloat16", context_length=128))
    prompt = bu.random_tokens(20, cfg["vocab"], 77)
    a = model.generate(prompt, max_tokens=16, temperature=1.0, top_k=20, seed=5).tokens
    b = model.generate(prompt, max_tokens=16, temperature=1.0, top_k=20, seed=5).tokens
    c = model.generate(prompt, max_tokens=16, temperature=1.0, top_k=20, seed=6).tokens
    assert a == b and a != c and all(0 <= t < cfg["vocab"] for t in a)
    with pytest.raises(StatefulCacheError):
        LocalModel.load(LocalModelConfig(source=str(folder), dtype="bfloat16", context_length=128,
                                         batching=BatchingConfig(prefix_cache=True)))


def test_bfloat16_generation_through_captured_graphs(models):
    """The serving precision end to end: prompts in portions, decode steps replayed as CUDA graphs (the tensor-core
    attention's single-token form with its key tiles dealt to several CTAs, the few-row contractions). Where two
    logits nearly tie bfloat16 may take the other branch, so every token it takes must be a near-maximum of the
    plain implementation's logits at its place."""
    from cuca_b200 import BatchingConfig, LocalModel, LocalModelConfig
    folder, cfg, oracle = models["wide"]
    prompts = [bu.random_tokens(n, cfg["vocab"], seed=60 + n) for n in (5, 70, 33)]
    model = LocalModel.load(LocalModelConfig(source=str(folder), dtype="bfloat16", context_length=256,
                                             batching=BatchingConfig(max_sequences=4, prefill_chunk=32)))
    assert model.backend.use_graphs
    outs = model.generate(prompts, max_tokens=40, temperature=0.0)
    assert model.backend.graph_steps > 0
    for prompt, out in zip(prompts, outs):
        ref = pb.forward(cfg, oracle.w, prompt + out.tokens)
        for i, tok in enumerate(out.tokens):
            row = ref[len(prompt) - 1 + i]
            assert float(row.max() - row[tok]) < 0.05 * float(np.abs(row).max()), (i, tok, int(row.argmax()))
