"""Host-side logic of the Sagelorn design without a GPU: configuration, tensor names, the cache a layer shares with
another and how far back it reaches, the previous token as a request's state, and the real parts, cache manager and
step function over stand-in kernels (tests/fake_ops.py) against the plain float64 restatement."""
import copy
import math

import pytest
import torch

import plain_sagelorn as plain
import sagelorn_models as sm
import traces
from fake_ops import FakeOps


def test_configuration_to_parts():
    from pih_b200.config import config_from_dict
    cfg = config_from_dict(copy.deepcopy(sm.S1))
    spec = cfg.model_spec()
    assert cfg.architecture == "Sagelorn" and spec.stream_dtype == "float32" and not spec.tie_embeddings
    assert spec.logit_scale == 0.3 and (spec.bigram.buckets, spec.bigram.mul_prev, spec.bigram.mul_cur) == (53, 31, 5)
    assert [b.arrangement for b in spec.blocks] == ["outnorm"] * 5 and spec.final_norm.offset == 1.0
    assert [b.mixer.kind for b in spec.blocks] == ["window_attention", "latent_attention", "window_attention", "retention",
                                                   "window_attention"]
    assert [e.reads_cache_of for e in spec.schedule] == [None, None, 0, None, None]
    owner, reader = spec.blocks[0].mixer, spec.blocks[2].mixer
    assert owner.own_kv and not reader.own_kv and (owner.window, reader.window) == (20, 37)
    assert owner.cache_window == 37                      # the owner keeps what its reader still looks at
    assert owner.sink == "learned" and owner.position.stretch == (8.0, 1.0, 4.0, 64.0) and not owner.position.interleaved
    lat = spec.blocks[1].mixer
    assert (lat.latent_rank, lat.rotary_dim, lat.query_rank, lat.window, lat.gate_per, lat.sink) == (40, 8, 24, 11, "column", False)
    assert lat.position.interleaved and lat.cached_width == 48 and lat.query_dim == 24
    ret = spec.blocks[3].mixer
    assert ret.position is None and ret.key_scale == 0.25 and ret.decays == (1.0, 0.97, 0.995)
    moe = spec.blocks[1].ffn
    assert (moe.experts, moe.top, moe.scoring, moe.weigh, moe.gated, moe.activation) == (6, 2, "sigmoid", "input", False, "relu2")
    assert moe.shared.kind == "plain_mlp" and moe.shared.intermediate == 56 and not moe.shared_gate and not moe.correction
    assert spec.blocks[2].ffn is None and spec.blocks[2].norm_post is None and spec.blocks[0].ffn.kind == "swiglu"
    assert config_from_dict(cfg.to_dict()) == cfg


def test_a_cache_reaches_as_far_as_its_widest_reader():
    from pih_b200.config import config_from_dict
    spec = config_from_dict(copy.deepcopy(sm.S2)).model_spec()
    assert [e.reads_cache_of for e in spec.schedule] == [None, None, 1, None, 1]
    assert [spec.blocks[i].mixer.window for i in (1, 2, 4)] == [24, 9, 64] and spec.blocks[1].mixer.cache_window == 64
    raw = copy.deepcopy(sm.S2)
    del raw["layers"][4]["mixer"]["mask"]                # a reader that sees every key: the cache keeps every key
    assert config_from_dict(raw).model_spec().blocks[1].mixer.cache_window == 0


def test_tensor_names():
    from pih_b200.config import config_from_dict
    from pih_b200.models import expected_tensors
    names = expected_tensors(config_from_dict(copy.deepcopy(sm.S1)).model_spec())
    assert names["embed"].shape == (311, 96) and names["bigram"].shape == (54, 96) and names["head"].shape == (311, 96)
    assert names["final.norm"].shape == (96,) and names["l2.norm1"].shape == (96,) and "l2.norm2" not in names
    assert names["l0.mix.q"].shape == (64, 96) and names["l0.mix.k"].shape == (32, 96) and names["l0.mix.v"].shape == (48, 96)
    assert names["l0.mix.q.norm"].shape == (64,) and names["l0.mix.k.norm"].shape == (32,) and names["l0.mix.sink"].shape == (4,)
    assert names["l0.mix.o"].shape == (96, 96)
    assert all(n not in names for n in ("l2.mix.k", "l2.mix.v", "l2.mix.k.norm")) and names["l2.mix.q.norm"].shape == (64,)
    assert names["l1.mix.dq"].shape == (24, 96) and names["l1.mix.dq.norm"].shape == (24,) and names["l1.mix.uq"].shape == (72, 24)
    assert names["l1.mix.dkv"].shape == (48, 96) and names["l1.mix.dkv.norm"].shape == (40,)
    assert names["l1.mix.uk"].shape == (48, 40) and names["l1.mix.uv"].shape == (36, 40)
    assert names["l1.mix.g"].shape == (36, 96) and names["l1.mix.o"].shape == (96, 36) and "l1.mix.sink" not in names
    assert names["l3.mix.g"].shape == (72, 96) and names["l3.mix.q"].shape == (48, 96)
    assert names["l1.mlp.router"].shape == (6, 96) and names["l1.mlp.e5.up"].shape == (40, 96) and "l1.mlp.e6.up" not in names
    assert "l1.mlp.e0.gate" not in names and "l1.mlp.correction" not in names
    assert names["l1.mlp.shared.up"].shape == (56, 96) and names["l1.mlp.shared.down"].shape == (96, 56)
    assert names["l0.mlp.gate"].shape == (136, 96)


@pytest.mark.parametrize("change, message", [
    (lambda c: c["layers"][0].update(type="conv"), "type"),
    (lambda c: c["layers"][2]["mixer"].update(kv_from=2), "kv_from"),
    (lambda c: c["layers"][2]["mixer"].update(kv_from=1), "kv_from"),
    (lambda c: c["layers"][2]["mixer"].update(dim=8), "kv_from"),
    (lambda c: c["layers"][4]["mixer"].update(kv_from=2), "kv_from"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=7), "top"),
    (lambda c: c["layers"][3]["mixer"].update(decay=[0.5, 0.5]), "decay"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), "dims"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=4), "rot_dim"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "kv_heads"),
    (lambda c: c["embedding"]["bigram"].update(buckets=0), "buckets"),
    (lambda c: c.pop("norm"), "norm"),
])
def test_configuration_errors(change, message):
    from pih_b200.config import config_from_dict
    raw = copy.deepcopy(sm.S1)
    change(raw)
    with pytest.raises(ValueError, match=message):
        config_from_dict(raw)


def test_stretched_frequencies():
    """The position part's frequencies against the plain restatement, band by band: a pair that turns often keeps its
    frequency, a slow one is divided by the factor, one in between is blended."""
    from pih_b200.config.specs import ComputedRopeSpec
    from pih_b200.parts.rope import ComputedRotary
    rot = {"dims": 16, "base": 300.0, "scaling": {"factor": 5.0, "low": 1.0, "high": 3.0, "original": 40}}
    ref = plain.frequencies(rot)
    got = ComputedRotary.frequencies_of(ComputedRopeSpec(head_dim=16, rotary_dim=16, theta=300.0, stretch=(5.0, 1.0, 3.0, 40)))
    assert float((got - ref).abs().max()) < 1e-15
    base = torch.tensor([300.0 ** (-2.0 * i / 16) for i in range(8)], dtype=torch.float64)
    ratio = ref / base
    assert ratio[0] == 1.0 and abs(float(ratio[-1]) - 0.2) < 1e-15 and bool(((ratio > 0.2) & (ratio < 1.0)).any())


def test_the_plain_implementation_cut_in_two():
    """The oracle itself: a sequence fed in two parts through its state (the previous token, the keys, the retention
    state) gives what it gives whole."""
    cfg = copy.deepcopy(sm.S2)
    g = torch.Generator().manual_seed(0)
    from pih_b200.config import config_from_dict
    from pih_b200.models import expected_tensors
    w = {n: torch.randn(i.shape, generator=g, dtype=torch.float64) * 0.2
         for n, i in expected_tensors(config_from_dict(cfg).model_spec()).items()}
    toks = traces.make_requests(257, [21], seed=1)["r0"]
    _, whole, _ = plain.model_layers(cfg, w, toks)
    _, a, st = plain.model_layers(cfg, w, toks[:13])
    _, b, _ = plain.model_layers(cfg, w, toks[13:], st)
    assert float((torch.cat([a, b]) - whole).abs().max()) < 1e-9


def test_plain_routing_and_weights_by_hand():
    """Sigmoid scores, the two largest chosen (a tie goes to the smaller index), the weight on what the expert reads:
    with the squared ReLU an expert's output grows with the SQUARE of the weight."""
    f = {"router": {"experts": 4, "top": 2}}
    w = {"m.router": torch.eye(4, dtype=torch.float64)}
    for e in range(4):
        w[f"m.e{e}.up"] = torch.full((3, 4), 0.5 + e, dtype=torch.float64)
        w[f"m.e{e}.down"] = torch.ones(4, 3, dtype=torch.float64)
    h = torch.tensor([[1.0, 2.0, 2.0, -1.0]], dtype=torch.float64)
    chosen, weights = plain.route(h, f, w, "m.")
    assert chosen.tolist() == [[1, 2]] and abs(float(weights[0, 0]) - 1 / (1 + math.exp(-2.0))) < 1e-15
    s = float(weights[0, 0])
    ref = sum(3 * (s * 4.0 * (0.5 + e)) ** 2 for e in (1, 2))
    assert float((plain.mixture(h, f, w, "m.") - ref).abs().max()) < 1e-9


def test_bigram_rows_by_hand():
    cfg = {"embedding": {"bigram": {"buckets": 5, "mul_prev": 3, "mul_cur": 4}}}
    w = {"embed": torch.zeros(10, 2, dtype=torch.float64), "bigram": torch.arange(6, dtype=torch.float64)[:, None].repeat(1, 2)}
    got = plain.embed(cfg, w, [7, 2, 9], None)[:, 0].tolist()
    assert got == [5.0, float((7 * 3 + 2 * 4) % 5), float((2 * 3 + 9 * 4) % 5)]
    assert plain.embed(cfg, w, [9], 2)[0, 0] == float((2 * 3 + 9 * 4) % 5)


@pytest.mark.parametrize("name", ["S1", "S2"])
@pytest.mark.parametrize("family", ["whole", "portions", "mixed"])
def test_cut_invariance_with_stand_in_kernels(tmp_path, name, family):
    """Block tables, slot mappings, state slots, the previous token of a request, the cache that one layer reads of
    another (kept as far back as the widest reader looks), and their reuse: the real parts and step function with torch
    stand-ins for the kernels agree with the plain implementation however the requests are cut."""
    from pih_b200.engine.factory import create_runner
    d = sm.write_model(tmp_path / name, sm.CONFIGS[name], seed=1, sigma=sm.SIGMA[name])
    requests = traces.make_requests(sm.CONFIGS[name]["vocab"], [19, 6, 71, 1, 12], seed=3)
    kw = dict(max_live=2, decode_tail=3, max_portion=7) if family == "mixed" else {}
    steps = getattr(traces, family)(requests, **kw)
    _, model, cache, runner = create_runner(d, "float32", device="cpu", page_size=4,
                                            max_cache_tokens=traces.peak_tokens(steps, round_to=4), max_requests=2,
                                            ops=FakeOps())
    # layers that read another's cache keep none: one group tensor entry per layer with a paged cache of its own
    assert sum(len(g.entries) for g in cache.groups) == sum(
        1 for layer in sm.CONFIGS[name]["layers"] if layer["type"] != "retention" and "kv_from" not in layer["mixer"])
    got = traces.replay(runner, steps)
    for rid, ref in sm.plain_logits(d, requests).items():
        assert float((got[rid].double() - ref).abs().max()) < 2e-4 * float(ref.abs().max()), (family, rid)
    cache.check()
    assert cache.slots.num_free == 2 and all(f == cache.num_pages for f in cache.num_free_pages())
    if family != "whole":
        # windows smaller than the longest request: pages went back to the pool while it was still live
        assert any(g.pool.pages_handed_out > 0 and g.need.window for g in cache.groups)


def test_pages_behind_every_window_go_back(tmp_path):
    """A request far longer than the windows holds, at any time, only the pages that some reader can still see."""
    from pih_b200.engine import StepEntry
    from pih_b200.engine.factory import create_runner
    d = sm.write_model(tmp_path / "m", sm.S1, seed=2, sigma=0.12)
    toks = traces.make_requests(311, [150], seed=4)["r0"]
    _, model, cache, runner = create_runner(d, "float32", device="cpu", page_size=4, max_cache_tokens=80, max_requests=1,
                                            ops=FakeOps())
    got = []
    for at in range(0, 150, 6):
        got.append(runner.step([StepEntry("a", toks[at:at + 6], list(range(6)))]).clone())
        held = {g.need.window: g.pool.num_pages - g.pool.num_free for g in cache.groups}
        for window, pages in held.items():               # a window of w keys and a portion of 6 span so many pages of 4
            assert pages <= (window + 6) // 4 + 2, (window, pages)
    assert sorted(held) == [11, 37, 50]                  # (the owner of layer 0's cache keeps 37 keys for its reader)
    ref = sm.plain_logits(d, {"a": toks})["a"]
    assert float((torch.cat(got).double() - ref).abs().max()) < 2e-4 * float(ref.abs().max())


def test_a_failed_step_leaves_the_states_as_they_were(tmp_path):
    """A step that raises after the layers have advanced their states (the retention state, the previous token) is
    rolled back."""
    from pih_b200.engine import StepEntry
    from pih_b200.engine.factory import create_runner
    d = sm.write_model(tmp_path / "m", sm.CONFIGS["S2"], seed=2, sigma=0.15)
    toks = traces.make_requests(257, [14], seed=1)["r0"]
    _, model, cache, runner = create_runner(d, "float32", device="cpu", page_size=4, max_cache_tokens=32, max_requests=1,
                                            ops=FakeOps())
    runner.step([StepEntry("a", toks[:9], [])])
    head = model.head
    model.head = None                                   # the head product fails, after every layer has run
    with pytest.raises(Exception):
        runner.step([StepEntry("a", toks[9:], [4])])
    model.head = head
    again = runner.step([StepEntry("a", toks[9:], [4])])
    ref = sm.plain_logits(d, {"a": toks})["a"][-1]
    assert float((again[0].double() - ref).abs().max()) < 2e-4 * float(ref.abs().max())


@pytest.mark.parametrize("seed", range(6))
def test_configurations_drawn_at_random_with_stand_in_kernels(tmp_path, seed):
    from pih_b200.engine.factory import create_runner
    raw = sm.random_config(seed)
    d = sm.write_model(tmp_path / "m", raw, seed=seed, sigma=0.15)
    requests = traces.make_requests(raw["vocab"], [23, 9, 1, 14], seed=seed)
    steps = traces.mixed(requests, seed=seed, max_live=2, decode_tail=3, max_portion=6)
    _, model, cache, runner = create_runner(d, "float32", device="cpu", page_size=4,
                                            max_cache_tokens=traces.peak_tokens(steps, round_to=4), max_requests=2, ops=FakeOps())
    got = traces.replay(runner, steps)
    for rid, ref in sm.plain_logits(d, requests).items():
        assert float((got[rid].double() - ref).abs().max()) < 3e-4 * max(1.0, float(ref.abs().max())), rid
    cache.check()


def test_the_cached_latent_is_padded_to_a_tensor_core_width_in_bfloat16(tmp_path):
    """In bfloat16 the cache of a latent attention layer is as wide as the next tensor-core instance; the columns of
    padding stay zero and change nothing (here: stand-in kernels that round to bfloat16 after each step)."""
    from pih_b200.engine.factory import create_runner
    d = sm.write_model(tmp_path / "m", sm.single_layer("latent_attention"), seed=1, sigma=0.2)
    requests = traces.make_requests(120, [23, 5], seed=3)
    steps = traces.portions(requests)
    _, model, cache, runner = create_runner(d, "bfloat16", device="cpu", page_size=4, max_cache_tokens=32, max_requests=2,
                                            ops=FakeOps())
    assert [g.need.width for g in cache.groups] == [64] and model.blocks[0].mixer.w_fold_k.shape == (2, 64, 18)
    got = traces.replay(runner, steps)
    assert bool((cache.groups[0].kv[..., 24:] == 0).all()) and bool((cache.groups[0].kv[..., :24] != 0).any())
    for rid, ref in sm.plain_logits(d, requests).items():
        err = (got[rid].double() - ref).pow(2).mean().sqrt() / ref.std()
        assert float(err) < 0.05, (rid, float(err))
    _, _, cache32, _ = create_runner(d, "float32", device="cpu", page_size=4, max_cache_tokens=32, max_requests=2, ops=FakeOps())
    assert [g.need.width for g in cache32.groups] == [24]
