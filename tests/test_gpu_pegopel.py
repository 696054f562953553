"""The Pegopel design on the GPU against the plain float64 restatement (tests/plain_pegopel.py): each mechanism alone,
every way of cutting requests into steps, batches against requests alone, pages and state slots that are used again,
keys far back, at page borders and just inside and just outside a window and the kept first tokens, in prompts and in
decoding, the first tokens of a sequence, long decoding, and greedy generation through the engine's own entry point."""
import math
from types import SimpleNamespace

import pytest
import torch

import pegopel_models as pm
import plain_pegopel as plain
import traces

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
F64 = torch.float64


@pytest.fixture(scope="module")
def dirs(tmp_path_factory):
    return {n: pm.write_model(tmp_path_factory.mktemp(f"pegopel_{n}"), raw, seed=7 + i, sigma=pm.SIGMA[n])
            for i, (n, raw) in enumerate(pm.CONFIGS.items())}


def _ops():
    from pih_b200.kernels import get_ops
    return get_ops(torch.device(DEV))


def _check(got, truth, dtype, what):
    """Per position: the error of the logits (mean taken off, root mean square over the vocabulary) relative to the
    logits' spread.  32-bit: every position of every request.  bfloat16, over the positions of all requests together:
    the median within rounding, and at most one position in ten beyond three times that."""
    errs = []
    for rid, ref in truth.items():
        g = got[rid].double()
        assert g.shape == ref.shape, (what, rid)
        d = g - ref
        d = d - d.mean(dim=1, keepdim=True)
        err = d.pow(2).mean(dim=1).sqrt() / ref.std()
        errs.append(err)
        if dtype == "float32":
            worst = int(err.argmax())
            assert float(err.max()) < 5e-5, f"{what} {rid}: error {float(err.max()):.3e} of the logits' spread at position {worst}"
    if dtype != "float32":
        err = torch.cat(errs)
        over = int((err > 0.09).sum())
        assert float(err.median()) < 0.03 and over <= len(err) // 10, \
            f"{what}: median {float(err.median()):.3e}, {over} of {len(err)} positions beyond 0.09, worst {float(err.max()):.3e}"


LENGTHS = {"P1": [70, 45, 131, 33, 64, 50, 1, 2], "P2": [65, 33, 97, 128, 80, 3, 35, 66], "P3": [40, 17, 5, 64, 2, 1]}
FAMILIES = ["whole", "tail_decode", "portions", "mixed"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["P1", "P2", "P3"])
@pytest.mark.parametrize("family", FAMILIES)
def test_cuttings_against_the_plain_implementation(dirs, name, dtype, family):
    """Whole prompts; most of a prompt and then token by token (the windows pass over decoded tokens); portions down to
    two tokens; up to three live requests mixed, with a pool so small and so few state slots that pages and slots are
    used again."""
    from pih_b200.engine.factory import create_runner
    requests = traces.make_requests(pm.CONFIGS[name]["vocab"], LENGTHS[name], seed=21)
    kw = dict(max_live=3) if family == "mixed" else (dict(tail=48) if family == "tail_decode" else {})
    steps = getattr(traces, family)(requests, **kw)
    _, model, cache, runner = create_runner(dirs[name], dtype, page_size=16 if name == "P1" else 8,
                                            max_cache_tokens=traces.peak_tokens(steps, round_to=16), max_requests=3)
    got = traces.replay(runner, steps)
    model.rt.ops.check_errors()
    _check(got, pm.plain_logits(dirs[name], requests), dtype, f"{name} {family} {dtype}")
    cache.check()
    assert all(f == cache.num_pages for f in cache.num_free_pages()) and cache.slots.num_free == 3
    if family == "mixed":
        assert all(g.pool.pages_handed_out > g.pool.num_pages for g in cache.groups)


def test_the_streams_behind_every_layer(dirs):
    """The sum of the residual streams behind every layer that runs (a looped layer each time) against the plain
    implementation, in 32-bit: the blocks one by one through the model's own schedule and caches."""
    from pih_b200.engine import StepEntry
    from pih_b200.engine.factory import create_runner
    name = "P1"
    toks = traces.make_requests(pm.CONFIGS[name]["vocab"], [53], seed=4)["r0"]
    cfg, w = pm.load_plain(dirs[name])
    _, layers = plain.forward(cfg, w, toks, with_layers=True)
    _, model, cache, runner = create_runner(dirs[name], "float32", page_size=16, max_cache_tokens=64, max_requests=1)
    seen = []
    ops = model.rt.ops
    for block in set(model.blocks):
        inner = block.forward

        def spy(x, pending, step, c, inner=inner, block=block):
            x, pending = inner(x, pending, step, c)
            y, mix, spread = pending
            after = x.clone()                                   # the pending output written into a copy of the streams
            ops.hyper_stream(after, y, mix=mix, spread=spread)
            seen.append(after.sum(dim=1).double().cpu())
            return x, pending
        block.forward = spy
    runner.step([StepEntry("a", toks, [len(toks) - 1])])
    ops.check_errors()
    assert len(seen) == layers.shape[0] == 6
    for i, (got, ref) in enumerate(zip(seen, layers)):
        assert float((got - ref).abs().max()) < 2e-5 * float(ref.abs().max()), f"behind layer run {i}"


@pytest.mark.parametrize("kind, changes", [
    ("attention", {}), ("attention_2", {}),
    ("attention", {"conv": 1, "bias_rows": 2, "bias_max": 1.5, "heads": 1, "kv_heads": 1, "mask": {"size": 200}}),
    ("attention", {"conv": 9, "bias_rows": 32, "bias_max": 17.0, "mask": {"size": 33}, "vdim": 8, "dim": 40}),
    ("attention_2", {"rot": None, "softcap": None, "mask": {"size": 4, "keep_first": 30}}),
    ("attention_2", {"rot": {"dims": 12, "base": 9.0}, "heads": 3, "kv_heads": 3, "mask": {"size": 16}}),
    ("attention_2", {"rot": {"dims": 2, "base": 1e6, "scaling": {"factor": 32.0, "original": 8, "fast": 2.0, "slow": 1.5}},
                     "heads": 1, "kv_heads": 1, "softcap": 0.7, "mask": {"size": 1, "keep_first": 1}})])
def test_a_mixer_alone(tmp_path, kind, changes):
    """One layer of one mixer and no feed-forward, whole, token by token and in portions: also a single tap and a table
    of two rows, more taps than a portion has rows, no rotation and no cap, more kept tokens than the window is wide, a
    rotation over the whole head, a window of the row itself."""
    from pih_b200.engine.factory import create_runner
    d = pm.write_model(tmp_path / kind, pm.single_layer(kind, **changes), seed=3, sigma=0.2)
    requests = traces.make_requests(120, [60, 7, 2], seed=2)
    truth = pm.plain_logits(d, requests)
    for family in ("whole", "tail_decode", "portions"):
        _, model, cache, runner = create_runner(d, "float32", page_size=8, max_cache_tokens=96, max_requests=3)
        _check(traces.replay(runner, getattr(traces, family)(requests)), truth, "float32", f"{kind} {family}")
        model.rt.ops.check_errors()


@pytest.mark.parametrize("streams", [0, 1, 2, 5, 8])
def test_a_feed_forward_behind_the_streams(tmp_path, streams):
    """The gated feed-forward with the tanh form of GELU behind a mixer, over one plain stream and over one, two, five
    and eight connected streams."""
    from pih_b200.engine.factory import create_runner
    d = pm.write_model(tmp_path / "ff", pm.single_layer("attention", mlp={"kind": "dense", "ff": 52}, streams=streams),
                       seed=4, sigma=0.25)
    requests = traces.make_requests(120, [50, 9], seed=5)
    _, model, cache, runner = create_runner(d, "float32", page_size=8, max_cache_tokens=64, max_requests=2)
    _check(traces.replay(runner, traces.whole(requests)), pm.plain_logits(d, requests), "float32", "feed-forward")
    model.rt.ops.check_errors()
