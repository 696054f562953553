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


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", range(8))
def test_configurations_drawn_at_random(tmp_path, seed, dtype):
    """Sizes, the order of layers, loops, streams, windows and constants drawn at random (odd sizes that no fast kernel
    takes among them): three live requests mixed over a pool that forces pages and slots to be used again."""
    from pih_b200.engine.factory import create_runner
    raw = pm.random_config(seed)
    d = pm.write_model(tmp_path / "m", raw, seed=50 + seed, sigma=0.2)
    requests = traces.make_requests(raw["vocab"], [70, 33, 129, 18, 2, 64], seed=seed)
    steps = traces.mixed(requests, seed=seed, max_live=3)
    _, model, cache, runner = create_runner(d, dtype, page_size=8, max_cache_tokens=traces.peak_tokens(steps, round_to=8),
                                            max_requests=3)
    _check(traces.replay(runner, steps), pm.plain_logits(d, requests), dtype, f"random configuration {seed} {dtype}")
    model.rt.ops.check_errors()
    cache.check()


@pytest.mark.parametrize("kind, changes", [
    ("attention", {"heads": 4, "kv_heads": 2, "dim": 128, "vdim": 128, "scale": 0.09, "bias_rows": 32, "bias_max": 150.0,
                   "mask": {"size": 200}}),
    ("attention", {"heads": 2, "kv_heads": 1, "dim": 64, "vdim": 128, "scale": 0.12, "mask": {"size": 130}}),
    ("attention_2", {"heads": 4, "kv_heads": 2, "dim": 128, "vdim": 128, "scale": 0.09, "softcap": 20.0,
                     "rot": {"dims": 64, "base": 1e4, "scaling": {"factor": 4.0, "original": 64, "fast": 16.0, "slow": 1.0}},
                     "mask": {"size": 150, "keep_first": 70}}),
    ("attention_2", {"heads": 2, "kv_heads": 2, "dim": 32, "vdim": 32, "scale": 0.18, "rot": {"dims": 32, "base": 100.0},
                     "mask": {"size": 64, "keep_first": 129}})])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_mixer_at_the_sizes_of_the_tensor_core_kernel(tmp_path, kind, changes, dtype):
    """Heads of 128, 64 and 32 numbers and prompts of several row tiles: windows that end inside a key tile and inside a
    row tile, kept first tokens beyond a key tile, whole, in portions and token by token."""
    from pih_b200.engine.factory import create_runner
    raw = pm.single_layer(kind, **changes)
    raw["max_positions"] = 400
    d = pm.write_model(tmp_path / kind, raw, seed=9, sigma=0.15)
    requests = traces.make_requests(120, [300, 129, 40], seed=6)
    truth = pm.plain_logits(d, requests)
    for family in ("whole", "portions", "tail_decode"):
        _, model, cache, runner = create_runner(d, dtype, page_size=16, max_cache_tokens=512, max_requests=3)
        _check(traces.replay(runner, getattr(traces, family)(requests)), truth, dtype, f"{kind} {family} {dtype}")
        model.rt.ops.check_errors()


def _step(positions, request_of_row, cu_q):
    t = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    starts = [positions[c] for c in cu_q[:-1]]
    return SimpleNamespace(positions=t(positions), request_of_row=t(request_of_row), cu_q=t(cu_q), num_requests=len(starts),
                           host_cu_q=list(cu_q), host_q_start=starts, q_start=t(starts), meta=None, attention_plans={})


def _plain_window_rows(q, K, V, positions, scale, window, keep, sink, group):
    """q [rows, heads, dim], K [n, kv_heads, dim], V [n, kv_heads, vdim] (float64): softmax over the seen keys with the
    sink's term in the denominator."""
    rows, heads, _ = q.shape
    out = torch.zeros(rows, heads, V.shape[2], dtype=F64)
    j = torch.arange(K.shape[0])
    for r, p in enumerate(positions):
        seen = (j <= p) & ((p - j < window) | (j < keep))
        for h in range(heads):
            s = (K[seen, h // group] @ q[r, h]) * scale
            m = max(float(s.max()), float(sink[h]))
            w = torch.exp(s - m)
            out[r, h] = (w[:, None] * V[seen, h // group]).sum(0) / (w.sum() + math.exp(float(sink[h]) - m))
    return out


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows_of_step", [260, 5, 1])
def test_keys_that_stand_out_at_the_edges(dtype, rows_of_step):
    """Queries and keys are multiples of unit vectors numbered by position, so that for every row exactly the keys at
    chosen distances score high: on head 0 the key just OUTSIDE the window (and keys 64 and 128 places nearer), on
    head 1 the key just INSIDE it (and one 64 places beyond the edge), on head 2 the last kept key, on head 3 the
    first key that is not kept.  A key seen or lost by mistake moves the output by a third or more.  A prompt of
    several row tiles (the tensor-core kernel in bf16), a short portion and single rows (the cut warp kernel)."""
    ops = _ops()
    heads, kv_heads, dim, vdim, window, keep, page, n = 4, 4, 64, 64, 150, 9, 16, 300
    g = torch.Generator().manual_seed(3)
    unit = torch.eye(dim, dtype=F64)
    K = 0.05 * torch.randn(n, kv_heads, dim, generator=g, dtype=F64)
    V = torch.randn(n, kv_heads, vdim, generator=g, dtype=F64)
    place = torch.arange(n)
    K[:, 0] += 6.0 * unit[(place + window) % dim]             # row p meets key p - window (outside), and 64, 128 nearer
    K[:, 1] += 6.0 * unit[(place + window - 1) % dim]         # row p meets key p - window + 1 (inside), and 64 beyond
    K[keep - 1, 2] += 6.0 * unit[0]                           # the last kept key
    K[keep, 3] += 6.0 * unit[0]                               # the first key that is not kept
    first = n - rows_of_step
    positions = list(range(first, n))
    q = 0.05 * torch.randn(rows_of_step, heads, dim, generator=g, dtype=F64)
    q[:, 0] += 6.0 * unit[torch.tensor(positions) % dim]
    q[:, 1] += 6.0 * unit[torch.tensor(positions) % dim]
    q[:, 2] += 6.0 * unit[0]
    q[:, 3] += 6.0 * unit[0]
    sink = torch.tensor([0.5, -1.0, 2.0, 0.0], dtype=F64)
    qd, Kd, Vd = (x.to(dtype).double() for x in (q, K, V))    # what the kernels are given
    want = _plain_window_rows(qd, Kd, Vd, positions, 0.5, window, keep, sink, heads // kv_heads)
    pages = -(-n // page)
    order = torch.randperm(pages + 3, generator=g)[:pages]     # pages out of order, some unused
    cache = torch.zeros(pages + 3, page, kv_heads * (dim + vdim), dtype=dtype, device=DEV)
    flat = torch.cat([Kd.reshape(n, -1), Vd.reshape(n, -1)], dim=1).to(dtype).to(DEV)
    for i in range(pages):
        rows = flat[i * page:(i + 1) * page]
        cache[order[i], :rows.shape[0]] = rows
    table = order.to(torch.int32).to(DEV).reshape(1, -1).contiguous()
    step = _step(positions, [0] * rows_of_step, [0, rows_of_step])
    got = ops.window_attention(qd.to(dtype).reshape(rows_of_step, -1).contiguous().to(DEV), cache=cache, block_table=table,
                               step=step, scale=0.5, window=window, keep_first=keep, softcap=0.0, bias=None,
                               sink=sink.float().to(DEV), gate=None, heads=heads, kv_heads=kv_heads, key_dim=dim,
                               value_dim=vdim)
    ops.check_errors()
    got = got.double().cpu().reshape(rows_of_step, heads, vdim)
    limit = 1e-5 if dtype == torch.float32 else 2e-2
    for h in range(heads):
        assert float((got[:, h] - want[:, h]).abs().max()) < limit * float(want.abs().max()), f"head {h}"
    # the check would see a fault: one more key at the window's far edge moves head 0
    wider = _plain_window_rows(qd, Kd, Vd, positions, 0.5, window + 1, keep, sink, heads // kv_heads)
    assert float((wider[:, 0] - want[:, 0]).abs().max()) > 0.2 * float(want.abs().max())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_engine(dirs, dtype):
    """Five prompts through ``Engine.complete_batch`` (the scheduler admits three at a time, cuts the prompts into
    portions of at most 24 tokens and has so few pages that finished requests' pages are used again; decode steps
    replay from graphs): every generated token is the plain implementation's most probable one given the tokens
    before it (in bf16: or within a hair of it)."""
    from pih_b200.engine import Engine
    name = "P2"
    cfg, w = pm.load_plain(dirs[name])
    prompts = list(traces.make_requests(pm.CONFIGS[name]["vocab"], [41, 9, 77, 2, 30], seed=12).values())
    engine = Engine(dirs[name], dtype, page_size=8, max_cache_tokens=384, maximum_batch_sequences=3,
                    maximum_batch_tokens=24, capture_decode_after=2)
    results = engine.complete_batch(prompts, max_tokens=40, ignore_eos=True)
    engine.drain()
    engine.rt.ops.check_errors()
    for prompt, res in zip(prompts, results):
        got = res["token_ids"]
        assert len(got) == 40
        ids = list(prompt)
        logits = plain.forward(cfg, w, ids + got)             # causal: row i depends on the tokens up to i only
        for i, tok in enumerate(got):
            row = logits[len(prompt) - 1 + i]
            best = int(torch.argmax(row))
            gap = float(row[best] - row[tok])
            assert tok == best or gap < (1e-4 if dtype == "float32" else 0.03) * float(row.std()), (dtype, i, tok, best, gap)


@pytest.mark.parametrize("rows", [1, 8, 13])
def test_the_few_rows_product_with_gelu_in_its_epilogue(rows):
    """``gelu(x Wg^T) * (x Wu^T)`` from the few-rows product (gate and up rows interleaved in blocks of 8) against the
    formula on the bf16 roundings of the two products."""
    ops = _ops()
    g = torch.Generator().manual_seed(rows)
    hidden, ff = 96, 72
    x = torch.randn(rows, hidden, generator=g).to(torch.bfloat16).to(DEV)
    gate, up = (torch.randn(ff, hidden, generator=g).mul(0.3).to(torch.bfloat16) for _ in range(2))
    stacked = torch.stack([gate.reshape(-1, 8, hidden), up.reshape(-1, 8, hidden)], dim=1).reshape(2 * ff, hidden).to(DEV)
    got = ops.linear_skinny(x, stacked.contiguous(), swiglu=True, activation="gelu_tanh")
    ops.check_errors()
    assert got is not None and got.shape == (rows, ff)
    a = (x.double().cpu() @ gate.double().t()).to(torch.bfloat16).double()
    b = (x.double().cpu() @ up.double().t()).to(torch.bfloat16).double()
    want = 0.5 * a * (1 + torch.tanh(math.sqrt(2 / math.pi) * (a + 0.044715 * a ** 3))) * b
    # the products' roundings may fall on either side of a tie: a bf16 step of the inputs, and the output's own rounding
    assert float((got.double().cpu() - want).abs().max()) < 0.02 * float(want.abs().max())
    silu = ops.linear_skinny(x, stacked.contiguous(), swiglu=True)
    assert float((silu.double().cpu() - a / (1 + torch.exp(-a)) * b).abs().max()) < 0.02 * float(want.abs().max())
