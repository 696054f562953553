"""The Sagelorn design on the GPU against the plain float64 restatement (tests/plain_sagelorn.py): each mechanism
alone, every way of cutting requests into steps, batches against requests alone, pages and state slots that are used
again, keys that must be found far back / at page borders / at a window's edges, in prompts and in decoding, the first
tokens of a sequence, long decoding, configurations drawn at random, and greedy generation through the engine's own
entry point and command lines."""
import math
from types import SimpleNamespace

import pytest
import torch

import plain_sagelorn as plain
import sagelorn_models as sm
import traces

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
F64 = torch.float64


@pytest.fixture(scope="module")
def dirs(tmp_path_factory):
    out = {}
    for i, (n, raw) in enumerate(sm.CONFIGS.items()):
        out[n] = sm.write_model(tmp_path_factory.mktemp(f"sagelorn_{n}"), raw, seed=5 + i, sigma=sm.SIGMA[n])
        out[n + "-all"] = sm.write_model(tmp_path_factory.mktemp(f"sagelorn_{n}_all"), sm.all_chosen(raw), seed=5 + i,
                                         sigma=sm.SIGMA[n])
    return out


def _ops():
    from pih_b200.kernels import get_ops
    return get_ops(torch.device(DEV))


def _errors(got, truth):
    errs = []
    for rid, ref in truth.items():
        d = got[rid].double() - ref
        d = d - d.mean(dim=1, keepdim=True)
        errs.append(d.pow(2).mean(dim=1).sqrt() / ref.std())
    return torch.cat(errs)


def _check(got, truth, dtype, what, rounding=None):
    """Per position: the error of the logits (mean taken off, root mean square over the vocabulary) relative to the
    logits' spread.  32-bit: every position of every request.  bfloat16 (models whose routers choose every expert), over
    the positions of all requests together: the median within rounding, and at most one position in ten beyond three
    times that.  ``rounding``: a function that gives the errors of a plain bfloat16 evaluation of the same steps (torch
    operations with a rounding after each), for a model so deep or so steep that rounding alone exceeds the fixed
    bound: the median may then be one and a half times that evaluation's."""
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
        bound = 0.03
        if rounding is not None and (float(err.median()) >= bound or int((err > 3 * bound).sum()) > len(err) // 10):
            bound = max(bound, 1.5 * float(rounding().median()))
        over = int((err > 3 * bound).sum())
        assert float(err.median()) < bound and over <= len(err) // 10, \
            f"{what}: median {float(err.median()):.3e}, {over} of {len(err)} positions beyond {3 * bound:.3f}, worst {float(err.max()):.3e}"


LENGTHS = {"S1": [70, 45, 131, 33, 64, 50, 1, 2], "S2": [65, 33, 97, 128, 80, 3, 35, 66]}
FAMILIES = ["whole", "tail_decode", "portions", "mixed"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["S1", "S2"])
@pytest.mark.parametrize("family", FAMILIES)
def test_cuttings_against_the_plain_implementation(dirs, name, dtype, family):
    """Whole prompts; most of a prompt and then token by token; portions down to two tokens; up to three live
    requests mixed, with a pool so small and so few state slots that pages and slots are used again.  The requests are
    longer than every window, and one layer reads another's keys through a wider window than the owner's."""
    from pih_b200.engine.factory import create_runner
    requests = traces.make_requests(sm.CONFIGS[name]["vocab"], LENGTHS[name], seed=21)
    kw = dict(max_live=3) if family == "mixed" else {}
    steps = getattr(traces, family)(requests, **kw)
    folder = dirs[name] if dtype == "float32" else dirs[name + "-all"]
    _, model, cache, runner = create_runner(folder, dtype, page_size=16 if name == "S1" else 8,
                                            max_cache_tokens=traces.peak_tokens(steps, round_to=16), max_requests=3)
    got = traces.replay(runner, steps)
    model.rt.ops.check_errors()
    _check(got, sm.plain_logits(folder, requests), dtype, f"{name} {family} {dtype}")
    cache.check()
    assert all(f == cache.num_pages for f in cache.num_free_pages()) and cache.slots.num_free == 3
    if family == "mixed":
        assert all(g.pool.pages_handed_out > g.pool.num_pages for g in cache.groups)


@pytest.mark.parametrize("kind, changes", [
    ("retention", {}), ("attention", {}), ("latent_attention", {}),
    ("retention", {"heads": 1, "decay": [1.0]}),
    ("attention", {"heads": 1, "kv_heads": 1, "dim": 40, "vdim": 8, "rot": {"dims": 40, "base": 3.0}, "mask": {"size": 1}}),
    ("attention", {"mask": {"size": 1000}}),
    ("latent_attention", {"heads": 1, "dim": 8, "vdim": 56, "kv_rank": 64, "rot_dim": 16, "rot": {"dims": 16, "base": 7.0},
                          "mask": {"size": 2}}),
])
def test_a_mixer_alone(tmp_path, kind, changes):
    """One layer of one mixer and no feed-forward, whole and token by token; also with one head, a rotation over the
    whole head, a decay of one, windows of one and two keys and one wider than the requests."""
    from pih_b200.engine.factory import create_runner
    d = sm.write_model(tmp_path / kind, sm.single_layer(kind, **changes), seed=3, sigma=0.2)
    requests = traces.make_requests(120, [40, 7], seed=2)
    truth = sm.plain_logits(d, requests)
    for family in ("whole", "tail_decode"):
        _, model, cache, runner = create_runner(d, "float32", page_size=8, max_cache_tokens=64, max_requests=2)
        _check(traces.replay(runner, getattr(traces, family)(requests)), truth, "float32", f"{kind} {family}")
        model.rt.ops.check_errors()


@pytest.mark.parametrize("mlp", [sm._dense(52), sm._moe(7, 3, 36, shared=28), sm._moe(4, 4, 20), sm._moe(9, 1, 24),
                                 sm._moe(1, 1, 16, shared=8)])
@pytest.mark.parametrize("bigram", [True, False])
def test_a_feed_forward_alone(tmp_path, mlp, bigram):
    """The gated feed-forward, and the routed one with and without a shared expert, choosing some, all and one of its
    experts, behind a mixer; with the bigram embedding and without."""
    from pih_b200.engine.factory import create_runner
    d = sm.write_model(tmp_path / "ff", sm.single_layer("retention", mlp=mlp, bigram=bigram), seed=4, sigma=0.25)
    requests = traces.make_requests(120, [50, 9], seed=5)
    for family in ("whole", "portions"):
        _, model, cache, runner = create_runner(d, "float32", page_size=8, max_cache_tokens=64, max_requests=2)
        _check(traces.replay(runner, getattr(traces, family)(requests)), sm.plain_logits(d, requests), "float32", "feed-forward")
        model.rt.ops.check_errors()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("weigh", ["input", "output"])
def test_sigmoid_routing_with_decided_scores(dtype, weigh):
    """The routed feed-forward as an op with router logits given so that no rounding decides a choice: distinct
    logits, sigmoid scores as weights on what the expert reads (or on what it gives); every row's output against the
    plain sum over its chosen experts, for many rows and for few."""
    ops = _ops()
    g = torch.Generator().manual_seed(6)
    rows, hidden, ff, experts, top = 300, 40, 72, 9, 3
    x = (torch.randn(rows, hidden, generator=g) * 0.8).to(dtype)
    wu = (torch.randn(experts, ff, hidden, generator=g) * 0.2).to(dtype)
    wd = (torch.randn(experts, hidden, ff, generator=g) * 0.2).to(dtype)
    logits = torch.stack([torch.randperm(experts, generator=g).float() * 0.7 - 2.0 for _ in range(rows)])
    f = {"router": {"experts": experts, "top": top}}
    chosen, weights = plain.route(logits.double(), f, {"m.router": torch.eye(experts, dtype=F64)}, "m.")
    assert len(set(chosen.flatten().tolist())) > top
    ref = torch.zeros(rows, hidden, dtype=F64)
    xd = x.double()
    for t in range(rows):
        for e, a in zip(chosen[t].tolist(), weights[t]):
            w = {"up": wu[e].double(), "down": wd[e].double()}
            ref[t] += plain.expert(a * xd[t:t + 1], w, "")[0] if weigh == "input" else a * plain.expert(xd[t:t + 1], w, "")[0]
    routing = dict(outputs=experts, correction=None, groups=1, groups_keep=1, renormalize=False, scoring="sigmoid",
                   gated=False, weigh=weigh)
    tol = 1e-5 if dtype == torch.float32 else 3e-2
    for count in (rows, 5):
        got = ops.moe_experts(x[:count].to(DEV), logits[:count].to(DEV), wu.to(DEV).contiguous(), wd.to(DEV).contiguous(), top,
                              routing=routing)
        ops.check_errors()
        assert float((got.double().cpu() - ref[:count]).abs().max()) < tol * float(ref.abs().max()), count


def _step(positions, request_of_row, cu_q, slots, ids=None):
    t = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    return SimpleNamespace(positions=t(positions), request_of_row=t(request_of_row), cu_q=t(cu_q), state_slots=t(slots),
                           num_requests=len(slots), host_cu_q=list(cu_q), host_q_start=[positions[c] for c in cu_q[:-1]],
                           q_start=t([positions[c] for c in cu_q[:-1]]), meta=None, attention_plans={},
                           token_ids=t(ids) if ids is not None else None)


def test_bigram_embedding_and_the_previous_token():
    """Rows of two requests in one step, then their next tokens: the first token of a sequence takes the last row of the
    bigram table, a row inside a portion pairs with the row before it, a step's first row with the token that the
    request's state slot holds; multipliers far above 32 bits stay exact; another request's slot is left alone."""
    ops = _ops()
    g = torch.Generator().manual_seed(1)
    vocab, width, buckets = 50, 24, 13
    mul_prev, mul_cur = 2 ** 40 + 7, 2 ** 33 + 1
    table = torch.randn(vocab, width, generator=g)
    bigram = torch.randn(buckets + 1, width, generator=g)
    state = torch.full((4, 1), 49, dtype=torch.int32, device=DEV)
    a, b = [3, 49, 49, 0, 17], [8, 8]
    for dtype, out_dtype in ((torch.float32, torch.float32), (torch.bfloat16, torch.float32), (torch.bfloat16, torch.bfloat16)):
        tb, bg = table.to(dtype), bigram.to(dtype)

        def ref(tokens, previous):
            out = []
            for t in tokens:
                r = buckets if previous is None else (previous * mul_prev + t * mul_cur) % buckets
                out.append(tb[t].double() + bg[r].double())
                previous = t
            return torch.stack(out)

        # request a (slot 2) brings 3 tokens from its start, request b (slot 0) one token from its start
        step = _step([0, 1, 2, 0], [0, 0, 0, 1], [0, 3, 4], [2, 0], ids=a[:3] + b[:1])
        got = ops.embed_bigram(tb.to(DEV), bg.to(DEV), step, state=state, mul_prev=mul_prev, mul_cur=mul_cur, buckets=buckets,
                               out_dtype=out_dtype)
        want = torch.cat([ref(a[:3], None), ref(b[:1], None)])
        tol = 1e-6 if out_dtype == torch.float32 else 2e-2
        assert float((got.double().cpu() - want).abs().max()) < tol
        assert state[:, 0].tolist() == [8, 49, 49, 49]
        # then b decodes one token and a brings its last two; the order of the requests in the step is the other one
        step = _step([1, 3, 4], [0, 1, 1], [0, 1, 3], [0, 2], ids=b[1:] + a[3:])
        got = ops.embed_bigram(tb.to(DEV), bg.to(DEV), step, state=state, mul_prev=mul_prev, mul_cur=mul_cur, buckets=buckets,
                               out_dtype=out_dtype)
        want = torch.cat([ref(b[1:], b[0]), ref(a[3:], a[2])])
        assert float((got.double().cpu() - want).abs().max()) < tol
        assert state[:, 0].tolist() == [8, 49, 17, 49]
        state.fill_(49)
    ops.check_errors()


def test_row_wise_kernels():
    """The norm over the columns of a view, the rotation of part of every head in both pairings (also far out), the gates
    a column, the squared ReLU, and the scaling in place."""
    ops = _ops()
    g = torch.Generator().manual_seed(2)
    rows = 9
    wide = torch.randn(rows, 100, generator=g)
    w = torch.randn(37, generator=g)
    for dtype in (torch.float32, torch.bfloat16):
        x = wide.to(dtype)
        got = ops.rmsnorm_rows(x.to(DEV)[:, 5:42], w.to(DEV), 1e-5).double().cpu()
        ref = plain.rms_unit(x[:, 5:42].double(), 1e-5) * w.double()
        assert float((got - ref).abs().max()) < (1e-5 if dtype == torch.float32 else 3e-2)
    positions = [0, 1, 2, 77, 1000, 31000, 5, 6, 7]
    heads, width, offset, rot = 3, 20, 6, 10
    x = torch.randn(rows, 4 + heads * width, generator=g)
    rot_cfg = {"dims": rot, "base": 70.0, "scaling": {"factor": 3.0, "low": 1.0, "high": 2.0, "original": 50}}
    freq = plain.frequencies(rot_cfg).float().to(DEV)
    for neighbours in (False, True):
        got = ops.rotate_heads(x.to(DEV)[:, 4:].view(rows, heads, width), offset=offset, frequencies=freq, interleaved=neighbours,
                               positions=torch.tensor(positions, dtype=torch.int32, device=DEV)).double().cpu()
        v = x[:, 4:].double().view(rows, heads, width)
        ref = torch.cat([v[..., :offset], plain.rotate(v[..., offset:], torch.tensor(positions), rot_cfg, neighbours)], dim=-1)
        tol = torch.tensor([1e-5] * 4 + [2e-4, 6e-3] + [1e-5] * 3, dtype=F64)[:, None, None]   # 32-bit angles far out
        assert bool(((got - ref).abs() < tol).all()), neighbours
    a, gate = torch.randn(rows, 33, generator=g), torch.randn(rows, 50, generator=g) * 3
    got = ops.gate_mul(a.to(DEV), gate.to(DEV)[:, 9:42], "sigmoid").double().cpu()
    assert float((got - a.double() * torch.sigmoid(gate[:, 9:42].double())).abs().max()) < 1e-6
    got = ops.gate_mul(a.to(DEV), gate.to(DEV)[:, 9:42], "silu").double().cpu()
    assert float((got - a.double() * plain.silu(gate[:, 9:42].double())).abs().max()) < 1e-5
    got = ops.activation(gate.to(DEV)[:, 3:20], "relu2").double().cpu()
    assert float((got - torch.relu(gate[:, 3:20].double()) ** 2).abs().max()) < 1e-5 and float(got.min()) == 0.0
    z = torch.randn(7, 19, generator=g).to(DEV)
    keep = z.clone()
    assert ops.scale_(z, 0.3) is z and float((z - keep * 0.3).abs().max()) < 1e-7
    got = ops.add_gated(a.to(DEV), a.to(DEV) * 2, None).double().cpu()
    assert float((got - 3 * a.double()).abs().max()) < 1e-5
    # the squared ReLU in the few-rows product's epilogue: the bits of the product followed by the activation's kernel
    for m, n, k in ((5, 96, 64), (16, 520, 256), (8, 4096, 1024)):
        xb = (torch.randn(m, k, generator=g) * 0.5).bfloat16().to(DEV)
        wb = (torch.randn(n, k, generator=g) * 0.1).bfloat16().to(DEV)
        fused = ops.linear_skinny(xb, wb, activation="relu2")
        assert fused is not None and torch.equal(fused, ops.activation(ops.linear(xb, wb), "relu2"))
        ref = torch.relu((xb.double() @ wb.double().T).bfloat16().double()) ** 2
        assert float((fused.double() - ref).abs().max()) <= 0.02 * float(ref.abs().max())
    ops.check_errors()


@pytest.mark.parametrize("neighbours", [True, False])
def test_the_few_rows_fold_rotates_and_gates_like_the_separate_kernels(neighbours):
    """A batched product of few rows with the rotation of part of every head on its way in and the sigmoid gate a column
    on its way out gives the bits of ``rotate_heads``, the product and ``gate_mul`` one after the other (which is also
    what many rows run); and the values of the plain computation."""
    ops = _ops()
    g = torch.Generator().manual_seed(8)
    T, B, K, N, offset, rot = 7, 3, 40, 24, 16, 16
    x = (torch.randn(T, 5 + B * K, generator=g) * 0.7).bfloat16().to(DEV)[:, 5:].view(T, B, K)     # rows strided
    w = (torch.randn(B, N, K, generator=g) * 0.3).bfloat16().to(DEV)
    gate = torch.randn(T, B * N + 3, generator=g).bfloat16().to(DEV)[:, :B * N]
    rot_cfg = {"dims": rot, "base": 40.0}
    positions = [0, 3, 900, 17, 2, 64, 65]
    rotate = dict(offset=offset, frequencies=plain.frequencies(rot_cfg).float().to(DEV), interleaved=neighbours,
                  positions=torch.tensor(positions, dtype=torch.int32, device=DEV))
    fused = ops.linear_batched(x, w, rotate=rotate, gate=gate)
    apart = ops.gate_mul(ops.linear_batched(ops.rotate_heads(x, **rotate), w).view(T, B * N), gate, "sigmoid").view(T, B, N)
    ops.check_errors()
    assert torch.equal(fused, apart)
    many = ops.linear_batched(x.repeat(30, 1, 1), w, rotate=dict(rotate, positions=rotate["positions"].repeat(30)),
                              gate=gate.repeat(30, 1))
    assert float((many[:T].double() - fused.double()).abs().max()) <= 0.02 * float(fused.double().abs().max())
    xd = x.double().cpu()
    turned = torch.cat([xd[..., :offset], plain.rotate(xd[..., offset:offset + rot], torch.tensor(positions), rot_cfg, neighbours),
                        xd[..., offset + rot:]], dim=-1)
    ref = torch.einsum("tbk,bnk->tbn", turned, w.double().cpu()) * torch.sigmoid(gate.double().cpu()).view(T, B, N)
    assert float((fused.double().cpu() - ref).abs().max()) < 0.03 * float(ref.abs().max())


def test_queries_alone_are_normed_and_rotated_and_nothing_is_written():
    """The kernel in front of the attention for a mixer that reads another's keys: the norm over the WHOLE query
    projection, the rotation in halves by computed angles with stretched slow pairs over part of a head, and a cache that
    stays as it was; with keys and values of its own the same rows also fill their slots."""
    ops = _ops()
    g = torch.Generator().manual_seed(4)
    heads, kv_heads, dim, vdim, rot, page, T = 3, 1, 20, 12, 8, 4, 5
    positions, slots = [0, 1, 5, 1000, 0], [9, 2, 3, 17, -2]
    rot_cfg = {"dims": rot, "base": 50.0, "scaling": {"factor": 4.0, "low": 1.0, "high": 3.0, "original": 20}}
    freq = plain.frequencies(rot_cfg).float().to(DEV)
    nq, nk, nv = heads * dim, kv_heads * dim, kv_heads * vdim
    src = torch.randn(T, nq + nk + nv, generator=g)
    qn, kn = torch.randn(nq, generator=g) + 1, torch.randn(nk, generator=g) + 1
    pos = torch.tensor(positions)
    ref_q = plain.rotate((plain.rms_unit(src[:, :nq].double(), 1e-5) * qn.double()).view(T, heads, dim), pos, rot_cfg, False)
    ref_k = plain.rotate((plain.rms_unit(src[:, nq:nq + nk].double(), 1e-5) * kn.double()).view(T, kv_heads, dim), pos, rot_cfg, False)
    common = dict(eps=1e-5, rope_table=None, rotary_dim=rot, interleaved=False,
                  positions=torch.tensor(positions, dtype=torch.int32, device=DEV),
                  slot_mapping=torch.tensor(slots, dtype=torch.int32, device=DEV), heads=heads, kv_heads=kv_heads, key_dim=dim,
                  value_dim=vdim, values_from_keys=False, frequencies=freq)
    tol = torch.tensor([1e-5, 1e-5, 1e-5, 3e-4, 1e-5], dtype=F64)[:, None]
    cache = torch.full((6, page, nk + nv), 7.0, dtype=torch.float32, device=DEV)
    q = ops.window_qk_prepare(src[:, :nq].contiguous().to(DEV), q_norm=qn.to(DEV), k_norm=None, cache=cache, write_kv=False, **common)
    ops.check_errors()
    assert bool(((q.double().cpu() - ref_q.reshape(T, -1)).abs() < tol).all()) and bool((cache == 7.0).all())
    q = ops.window_qk_prepare(src.to(DEV), q_norm=qn.to(DEV), k_norm=kn.to(DEV), cache=cache, **common)
    ops.check_errors()
    assert bool(((q.double().cpu() - ref_q.reshape(T, -1)).abs() < tol).all())
    flat = cache.view(-1, nk + nv).double().cpu()
    for t, s in enumerate(slots[:-1]):
        assert bool(((flat[s, :nk] - ref_k[t].reshape(-1)).abs() < tol[t]).all())
        assert torch.equal(flat[s, nk:], src[t, nq + nk:].double())
    assert bool((flat[[s for s in range(flat.shape[0]) if s not in slots]] == 7.0).all())


def _paged_rows(rows, page, dtype):
    """The cache tensor [pages, page, width] and block table of one request whose cached vectors are given, its pages in
    descending order."""
    n = rows.shape[0]
    pages = list(range(-(-n // page) + 1))[::-1]
    cache = torch.zeros(max(pages) + 2, page, rows.shape[1], dtype=dtype, device=DEV)
    for j in range(n):
        cache[pages[j // page], j % page] = rows[j].to(dtype).to(DEV)
    return cache, torch.tensor([pages], dtype=torch.int32, device=DEV)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rank, rot, heads", [(40, 8, 3), (96, 32, 4), (18, 6, 1), (112, 16, 5), (520, 56, 2), (800, 32, 1)])
def test_latent_attention_window_edges_with_a_rotated_key_part(dtype, rank, rot, heads):
    """300 cached vectors [latent | rotated key part] of which ONE matches the folded query (its score stands out by
    construction, half of it through the rotated part): as the oldest key of the window, one place beyond it, across a
    page border and far back without a window — as a single decoded row and as the last row of a portion of 70 rows.
    Widths with a tensor-core instance (128), without one, and beyond the widest instance (576, 832: the warp kernels)."""
    ops = _ops()
    n, page, scale, rows, width = 300, 16, 0.4, 70, rank + rot
    last = n - 1
    for needle in (5, 239, 240, 241, 299):
        g = torch.Generator().manual_seed(needle)
        C = torch.randn(n, width, generator=g, dtype=F64) * 0.3
        C[needle] = torch.randn(width, generator=g, dtype=F64)
        q = torch.randn(rows, heads, width, generator=g, dtype=F64) * 0.1
        q[-1] += 8.0 * C[needle] / math.sqrt(width)
        C, q = C.to(dtype).double(), q.to(dtype).double()
        assert float((C[needle, rank:] @ q[-1, 0, rank:]).abs()) > 0.3          # the rotated part carries its share
        cache, table = _paged_rows(C, page, dtype)
        tol = 1e-5 if dtype == torch.float32 else 2e-2
        results = {}
        for window in (0, last - needle + 1, last - needle):
            if window == 0 and needle == last:
                continue
            lo = max(0, last - window + 1) if window else 0
            wts = torch.softmax((C[lo:] @ q[-1].T) * scale, dim=0)                # [keys, heads]
            ref = wts.T @ C[lo:]
            if window != last - needle:
                assert float(wts[needle - lo, 0]) > 0.5                            # the key does stand out
            one = ops.latent_attention(q[-1:].to(dtype).to(DEV).contiguous(), gate=None, sink=None, cache=cache,
                                       block_table=table, step=_step([last], [0], [0, 1], [0]), scale=scale, window=window)[0]
            many = ops.latent_attention(q.to(dtype).to(DEV).contiguous(), gate=None, sink=None, cache=cache, block_table=table,
                                        step=_step(list(range(n - rows, n)), [0] * rows, [0, rows], [0]), scale=scale,
                                        window=window)[-1]
            ops.check_errors()
            for got in (one, many):
                assert float((got.double().cpu() - ref).abs().max()) < tol * float(ref.abs().max()), (needle, window)
            results[window] = one.double().cpu()
        if needle != last:
            assert float((results[last - needle + 1] - results[last - needle]).abs().max()) > 0.1


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_window_attention_with_a_sink_at_the_windows_edges(dtype):
    """Keys and values of unequal sizes, a learned sink, and a key that stands out: just inside the window, just outside,
    across a page border, as a decoded row and as the last row of a portion; and a sink so large that it takes nearly
    all of the weight."""
    ops = _ops()
    g = torch.Generator().manual_seed(1)
    heads, kv_heads, dim, vdim, n, page, rows = 4, 2, 32, 24, 200, 8, 40
    needle, last = 135, n - 1
    K = torch.randn(n, kv_heads, dim, generator=g, dtype=F64) * 0.3
    V = torch.randn(n, kv_heads, vdim, generator=g, dtype=F64)
    q = torch.randn(rows, heads, dim, generator=g, dtype=F64) * 0.1
    q[-1] += 6.0 * K[needle].repeat_interleave(heads // kv_heads, dim=0) / math.sqrt(dim) * 4
    K, V, q = K.to(dtype).double(), V.to(dtype).double(), q.to(dtype).double()
    cache, table = _paged_rows(torch.cat([K.reshape(n, -1), V.reshape(n, -1)], dim=1), page, dtype)
    geometry = dict(heads=heads, kv_heads=kv_heads, key_dim=dim, value_dim=vdim)
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    results = {}
    for sink_value in (0.3, 30.0):
        sink = torch.tensor([sink_value, -1.0, 0.0, sink_value], dtype=torch.float32)
        for window in (last - needle + 1, last - needle):
            lo = last - window + 1
            ref = torch.zeros(heads, vdim, dtype=F64)
            for h in range(heads):
                s = (K[lo:, h // 2] @ q[-1, h]) * 0.5
                e = torch.exp(s - s.max())
                ref[h] = (e / (e.sum() + math.exp(float(sink[h]) - float(s.max())))) @ V[lo:, h // 2]
            kw = dict(cache=cache, block_table=table, scale=0.5, window=window, keep_first=0, softcap=0.0, bias=None,
                      sink=sink.to(DEV), gate=None, **geometry)
            one = ops.window_attention(q[-1:].reshape(1, -1).to(dtype).to(DEV).contiguous(), step=_step([last], [0], [0, 1], [0]),
                                       **kw)[0]
            many = ops.window_attention(q.reshape(rows, -1).to(dtype).to(DEV).contiguous(),
                                        step=_step(list(range(n - rows, n)), [0] * rows, [0, rows], [0]), **kw)[-1]
            ops.check_errors()
            for got in (one, many):
                assert float((got.double().cpu().view(heads, vdim) - ref).abs().max()) < tol * max(float(ref.abs().max()), 0.05)
            results[sink_value, window] = one.double().cpu().view(heads, vdim)
    assert float((results[0.3, last - needle + 1] - results[0.3, last - needle]).abs().max()) > 0.1
    assert float(results[30.0, last - needle + 1][0].abs().max()) < 1e-3 * float(results[0.3, last - needle + 1][0].abs().max())


def test_batches_against_each_request_alone(dirs):
    """Unequal requests side by side in one step — a long portion, a short one, single tokens — give each request
    the bits it gets alone (32-bit: every reduction has an order fixed by the row)."""
    from pih_b200.engine import StepEntry
    from pih_b200.engine.factory import create_runner
    name = "S1"
    requests = traces.make_requests(sm.CONFIGS[name]["vocab"], [61, 18, 40, 9], seed=8)
    alone = {}
    for rid, toks in requests.items():
        _, _, _, runner = create_runner(dirs[name], "float32", page_size=16, max_cache_tokens=128, max_requests=1)
        alone[rid] = traces.replay(runner, traces.whole({rid: toks}))[rid]
    _, model, cache, runner = create_runner(dirs[name], "float32", page_size=16, max_cache_tokens=256, max_requests=4)
    cuts = {"r0": [33, 27, 1], "r1": [1, 16, 1], "r2": [2, 37, 1], "r3": [7, 1, 1]}
    got = {rid: [] for rid in requests}
    at = {rid: 0 for rid in requests}
    for i in range(3):
        entries = []
        for rid, toks in requests.items():
            n = cuts[rid][i]
            entries.append(StepEntry(rid, toks[at[rid]:at[rid] + n], list(range(n))))
            at[rid] += n
        logits = runner.step(entries)
        j = 0
        for e in entries:
            got[e.rid].append(logits[j:j + len(e.tokens)].clone())
            j += len(e.tokens)
    model.rt.ops.check_errors()
    for rid in requests:
        assert float((torch.cat(got[rid]).cpu() - alone[rid]).abs().max()) < 1e-6, rid


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_sizes_that_only_the_plain_kernels_take(tmp_path, dtype):
    """A width, head sizes, ranks and a vocabulary that are multiples of two at most: no 16-byte piece, no tensor-core
    instance, no few-rows product; a mixed schedule against the plain implementation."""
    from pih_b200.engine.factory import create_runner
    raw = sm.S3 if dtype == "float32" else sm.all_chosen(sm.S3)
    d = sm.write_model(tmp_path / "m", raw, seed=11, sigma=0.2)
    requests = traces.make_requests(77, [50, 21, 1, 2, 34], seed=12)
    steps = traces.mixed(requests, seed=3, max_live=3)
    _, model, cache, runner = create_runner(d, dtype, page_size=8, max_cache_tokens=traces.peak_tokens(steps, round_to=8),
                                            max_requests=3)
    got = traces.replay(runner, steps)
    model.rt.ops.check_errors()
    _check(got, sm.plain_logits(d, requests), dtype, f"odd sizes {dtype}")
    cache.check()


@pytest.mark.parametrize("seed", range(8))
def test_configurations_drawn_at_random(tmp_path, seed):
    """Sizes, orders of layers, shared caches with windows of their own and constants drawn at random (odd sizes and
    sizes that only the plain kernels take among them): a mixed schedule in 32-bit against the plain implementation
    position by position, and in bfloat16 (every expert chosen) within rounding."""
    from pih_b200.engine.factory import create_runner
    raw = sm.random_config(seed)
    requests = traces.make_requests(raw["vocab"], [70, 45, 33, 18, 1, 2], seed=seed)
    steps = traces.mixed(requests, seed=seed, max_live=3)
    for dtype, cfg in (("float32", raw), ("bfloat16", sm.all_chosen(raw))):
        d = sm.write_model(tmp_path / dtype, cfg, seed=seed, sigma=0.15)
        _, model, cache, runner = create_runner(d, dtype, page_size=16, max_cache_tokens=traces.peak_tokens(steps, round_to=16),
                                                max_requests=3)
        got = traces.replay(runner, steps)
        model.rt.ops.check_errors()

        def rounding():
            from fake_ops import FakeOps
            _, _, _, plain_runner = create_runner(d, dtype, device="cpu", page_size=16, max_requests=3, ops=FakeOps(),
                                                  max_cache_tokens=traces.peak_tokens(steps, round_to=16))
            return _errors(traces.replay(plain_runner, steps), sm.plain_logits(d, requests))

        _check(got, sm.plain_logits(d, requests), dtype, f"seed {seed} {dtype}", rounding=rounding)
        cache.check()


def test_long_decoding(dirs):
    """A short prompt and 300 tokens one by one (pages fill, follow one another and go back behind the windows; the
    states run on)."""
    from pih_b200.engine.factory import create_runner
    name = "S2"
    requests = traces.make_requests(sm.CONFIGS[name]["vocab"], [310], seed=9)
    steps = traces.tail_decode(requests, tail=300)
    _, model, cache, runner = create_runner(dirs[name], "float32", page_size=8, max_cache_tokens=96, max_requests=1)
    _check(traces.replay(runner, steps), sm.plain_logits(dirs[name], requests), "float32", "long decoding")
    model.rt.ops.check_errors()


@pytest.mark.parametrize("cuda_graphs", [False, True])
@pytest.mark.parametrize("name", ["S1", "S2"])
def test_greedy_generation_through_the_engine(dirs, name, cuda_graphs):
    """Engine.complete (scheduler, cache, sampler, graphs, padded steps, ids fed on the device) against greedy decoding
    with the plain implementation; three requests at once with room for two, so they queue."""
    from pih_b200.engine import Engine
    cfg, w = sm.load_plain(dirs[name])
    prompts = list(traces.make_requests(sm.CONFIGS[name]["vocab"], [9, 21, 5], seed=13).values())
    new = 12
    want = []
    for p in prompts:
        toks = list(p)
        for _ in range(new):
            toks.append(int(plain.model_layers(cfg, w, toks)[1][-1].argmax()))
        want.append(toks[len(p):])
    engine = Engine(dirs[name], "float32", page_size=16, max_cache_tokens=256, maximum_batch_sequences=2,
                    maximum_batch_tokens=64, maximum_context_tokens=64, cuda_graphs=cuda_graphs)
    results = engine.complete_batch(prompts, max_tokens=new, temperature=0.0, ignore_eos=True)
    engine.rt.ops.check_errors()
    for r, expect in zip(results, want):
        assert r["token_ids"] == expect


def test_command_lines(dirs, tmp_path):
    """bin/pih-worker makes a random Sagelorn model from a configuration file and generates from it; bin/trace_run
    replays a trace on it; both agree with the plain implementation."""
    import json
    import os
    import subprocess
    import sys

    import numpy as np
    from conftest import ROOT
    worker = [sys.executable, os.path.join(ROOT, "bin", "pih-worker")]
    cfg_file = tmp_path / "config.json"
    cfg_file.write_text(json.dumps(sm.S2))
    folder = str(tmp_path / "made")
    proc = subprocess.run(worker + ["--random-model", folder, "--config", str(cfg_file), "--seed", "4", "--sigma", "0.15"],
                          capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    prompt = [5, 17, 3, 200, 9]
    proc = subprocess.run(worker + ["--model", folder, "--generate-tokens", ",".join(map(str, prompt)), "--max-tokens", "7",
                                    "--dtype", "float32", "--ignore-eos"], capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    res = json.loads(proc.stdout.strip().splitlines()[-1])
    cfg, w = sm.load_plain(folder)
    toks = list(prompt)
    for _ in range(7):
        toks.append(int(plain.model_layers(cfg, w, toks)[1][-1].argmax()))
    assert res["token_ids"] == toks[len(prompt):]

    requests = traces.make_requests(sm.S2["vocab"], [40, 9, 23], seed=6)
    steps = traces.mixed(requests, seed=1, max_live=3)
    for s_ in steps:
        for e in s_["entries"]:
            e["want"] = e["want"][-1:]                              # the last place of every portion
    out_dir = str(tmp_path / "out")
    cmd = [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", "float32", "--out", out_dir,
           "--max-tokens", str(traces.peak_tokens(steps))]
    proc = subprocess.run(cmd, input="\n".join(json.dumps(s_) for s_ in steps) + "\n", capture_output=True, text=True,
                          timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done ")] == [f"done {s_['step']}" for s_ in steps]
    truth = sm.plain_logits(folder, requests)
    at = {rid: 0 for rid in requests}
    for s_ in steps:
        got = np.fromfile(os.path.join(out_dir, f"{s_['step']}.f32"), dtype="<f4").reshape(-1, sm.S2["vocab"])
        for j, e in enumerate(s_["entries"]):
            at[e["id"]] += len(e["tokens"])
            ref = truth[e["id"]][at[e["id"]] - 1].numpy()
            assert np.abs(got[j] - ref).max() < 1e-4 * max(1.0, np.abs(ref).max()), (s_["step"], e["id"])
