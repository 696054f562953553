"""Host-side logic of the Pegopel design without a GPU: configuration, tensor names, the order of looped layers, the
rows of a bias table taken from the tensor's shape, the pages a window keeps, and the real parts, cache manager and
step function over stand-in kernels (tests/fake_ops.py) against the plain float64 restatement (tests/plain_pegopel.py)."""
import copy
import json
import math
import os

import pytest
import torch

import pegopel_models as pm
import plain_pegopel as plain
import traces
from fake_ops import FakeOps

F64 = torch.float64


def test_configuration_to_parts():
    from pih_b200.config import config_from_dict
    cfg = config_from_dict(copy.deepcopy(pm.P1))
    spec = cfg.model_spec()
    assert cfg.architecture == "Pegopel" and spec.stream_dtype == "float32" and spec.tie_embeddings
    assert spec.streams == 3 and spec.position_name == "pos" and spec.max_positions == 400
    assert [b.arrangement for b in spec.blocks] == ["hyper"] * 4
    assert [e.layer for e in spec.schedule] == [0, 1, 2, 1, 2, 3]
    a, b = spec.blocks[0].mixer, spec.blocks[1].mixer
    assert (a.kind, a.conv_taps, a.bias_rows, a.bias_far, a.sink, a.window, a.keep_first) == ("window_attention", 3, 10, 50, "learned", 23, 0)
    assert (a.heads, a.kv_heads, a.key_dim, a.value_dim, a.scale) == (4, 2, 16, 24, 0.3)
    assert not a.values_from_keys and a.position is None and a.softcap is None and not a.head_gate
    assert (b.values_from_keys, b.sink, b.head_gate, b.softcap, b.keep_first, b.window, b.conv_taps, b.bias_rows) == \
        (True, "zero", True, 5.0, 5, 37, 0, 0)
    assert (b.position.rotary_dim, b.position.theta, b.position.factor, b.position.original, b.position.fast) == (8, 1e4, 4.0, 64, 8.0)
    assert b.position.interleaved and spec.blocks[3].mixer.position.factor is None
    assert spec.blocks[1].ffn is None and spec.blocks[1].norm_post is None
    assert spec.blocks[0].ffn.activation == "gelu_tanh" and spec.blocks[0].ffn.intermediate == 136
    assert config_from_dict(cfg.to_dict()) == cfg
    plainer = config_from_dict(copy.deepcopy(pm.P2)).model_spec()
    assert plainer.streams == 0 and [b.arrangement for b in plainer.blocks] == ["prenorm"] * 3
    assert [e.layer for e in config_from_dict(copy.deepcopy(pm.P3)).model_spec().schedule] == [0, 1] * 3


def test_tensor_names():
    from pih_b200.config import config_from_dict
    from pih_b200.models import expected_tensors
    names = expected_tensors(config_from_dict(copy.deepcopy(pm.P1)).model_spec())
    assert names["embed"].shape == (307, 96) and names["pos"].shape == (400, 96) and names["final.norm"].shape == (96,)
    assert "head" not in names
    assert names["l0.mix.q"].shape == (64, 96) and names["l0.mix.k"].shape == (32, 96) and names["l0.mix.v"].shape == (48, 96)
    assert names["l0.mix.q.norm"].shape == (64,) and names["l0.mix.k.norm"].shape == (32,)
    assert names["l0.mix.q.conv"].shape == (64, 3) and names["l0.mix.v.conv"].shape == (48, 3)
    assert names["l0.mix.rel"].shape == (10, 4) and names["l0.mix.sink"].shape == (4,) and names["l0.mix.o"].shape == (96, 96)
    assert names["l1.mix.g"].shape == (6, 96) and names["l1.mix.o"].shape == (96, 96) and names["l1.mix.k"].shape == (32, 96)
    for absent in ("l1.mix.v", "l1.mix.rel", "l1.mix.sink", "l1.mix.q.conv", "l0.mix.g", "l1.norm2", "l1.hc2.in", "l1.mlp.up"):
        assert absent not in names, absent
    assert names["l0.hc1.in"].shape == (3,) and names["l0.hc2.out"].shape == (3,) and names["l2.hc1.mix"].shape == (3, 3)
    assert names["l2.mlp.gate"].shape == (72, 96) and names["l2.mlp.down"].shape == (96, 72)
    one = expected_tensors(config_from_dict(copy.deepcopy(pm.P2)).model_spec())
    assert not any(".hc" in n for n in one)


@pytest.mark.parametrize("change, message", [
    (lambda c: c["layers"][0].update(type="attention_3"), "type"),
    (lambda c: c["layers"][1]["mixer"].update(vdim=24), "vdim"),
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=4), "kv_heads"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=7), "dims"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=32), "dims"),
    (lambda c: c["layers"][0]["mixer"].pop("mask"), "mask"),
    (lambda c: c["layers"][0]["mlp"].update(kind="routed"), "kind"),
    (lambda c: c["loop"].update(stop=9), "loop"),
    (lambda c: c.update(streams=9), "streams"),
    (lambda c: c.pop("norm"), "norm"),
])
def test_configuration_errors(change, message):
    from pih_b200.config import config_from_dict
    raw = copy.deepcopy(pm.P1)
    change(raw)
    with pytest.raises(ValueError, match=message):
        config_from_dict(raw)


def test_bias_rows_come_from_the_tensor(tmp_path):
    """config.json does not say how many rows a bias table has; the loader reads it off the tensor."""
    from pih_b200.config import load_config
    from pih_b200.weights.loader import tensor_shapes
    d = pm.write_model(tmp_path / "m", pm.P1, seed=1, sigma=0.1)
    with open(os.path.join(d, "config.json")) as f:
        assert "bias_rows" not in json.dumps(json.load(f))
    cfg = load_config(d).with_shapes(tensor_shapes(d))
    spec = cfg.model_spec()
    assert spec.blocks[0].mixer.bias_rows == 10 and spec.blocks[2].mixer.bias_rows == 8


def test_buckets_of_the_distance_bias():
    """One row a distance in the first half of the table; beyond, rows spread by the logarithm up to the far distance,
    the last row from there on; the spread-out table has one column a distance."""
    from pih_b200.parts.window_attention import bias_by_distance, distance_bucket
    rows, far = 12, 96.0
    assert [distance_bucket(n, rows, far) for n in range(6)] == list(range(6))
    assert distance_bucket(6, rows, far) == 6 and distance_bucket(95, rows, far) == 11 and distance_bucket(5000, rows, far) == 11
    # 6 * 16^(k/6) is where row 6 + k begins: 6 * 16^(1/6) = 9.52.., 6 * 16^(1/2) = 24
    assert distance_bucket(9, rows, far) == 6 and distance_bucket(10, rows, far) == 7
    assert distance_bucket(23, rows, far) == 8 and distance_bucket(25, rows, far) == 9
    seen = [distance_bucket(n, rows, far) for n in range(200)]
    assert seen == sorted(seen) and set(seen) == set(range(rows))
    table = torch.arange(rows * 3, dtype=torch.float32).view(rows, 3)
    spread = bias_by_distance(table, far, 120)
    assert spread.shape == (3, 120) and torch.equal(spread[:, 30], table[distance_bucket(30, rows, far)])
    for n in range(150):                               # the oracle's own bucket, written apart, agrees
        assert plain.distance_bucket(n, rows, far) == seen[n]


def test_rotation_table_with_stretched_frequencies():
    """High frequencies stay, low ones are divided by the factor, those between are blended; cosine and sine carry the
    gain; without a factor the table is the plain one."""
    from pih_b200.config.specs import ScaledRopeSpec
    from pih_b200.parts.rope import ScaledRotary
    spec = ScaledRopeSpec(head_dim=32, rotary_dim=16, theta=1e4, max_positions=64, factor=4.0, original=64.0, fast=8.0, slow=1.0)
    f, gain = ScaledRotary.frequencies_and_gain(spec)
    base = torch.tensor([1e4 ** (-2.0 * i / 16) for i in range(8)], dtype=F64)
    turn = lambda t: 16 * math.log(64.0 / (2 * math.pi * t)) / (2 * math.log(1e4))
    lo, hi = max(math.floor(turn(8.0)), 0), min(math.ceil(turn(1.0)), 15)
    assert (lo, hi) == (0, 3)
    assert abs(float(f[0]) - float(base[0])) < 1e-15 and torch.allclose(f[3:], base[3:] / 4.0, rtol=1e-14, atol=0)
    assert abs(float(f[1]) - float(base[1]) * (1 / 3 / 4.0 + 2 / 3)) < 1e-15
    assert abs(gain - (0.1 * math.log(4.0) + 1.0)) < 1e-15
    table = ScaledRotary.table(spec)
    assert table.shape == (64, 8, 2) and abs(float(table[0, 0, 0]) - gain) < 1e-15 and float(table[0, 0, 1]) == 0.0
    assert abs(float(table[37, 5, 1]) - gain * math.sin(37 * float(f[5]))) < 1e-14
    c, s = plain.yarn_rotation(16, 1e4, {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}, torch.arange(64))
    assert float((table[..., 0] - c).abs().max()) < 1e-14 and float((table[..., 1] - s).abs().max()) < 1e-14
    bare = ScaledRotary.frequencies_and_gain(ScaledRopeSpec(head_dim=32, rotary_dim=16, theta=1e4, max_positions=64))
    assert torch.equal(bare[0], base) and bare[1] == 1.0


def test_plain_mechanisms_by_hand():
    """The oracle's own pieces on numbers small enough to do by hand."""
    # the convolution: the LAST tap weighs the current token, zeros before the start
    u = torch.tensor([[1.0], [2.0], [4.0]], dtype=F64)
    w = torch.tensor([[100.0, 10.0, 1.0]], dtype=F64)
    assert plain.short_conv(u, w).flatten().tolist() == [1.0, 12.0, 124.0]
    # the window: itself and size - 1 before it; kept first tokens stay
    m = plain.window_mask(6, 2, keep_first=1)
    assert m[5].tolist() == [True, False, False, False, True, True] and m[1].tolist() == [True, True, False, False, False, False]
    # the sink: one more term in the denominator, no value
    p = plain.sink_softmax(torch.zeros(1, 2, 2, dtype=F64), plain.window_mask(2, 2), torch.tensor([math.log(2.0)], dtype=F64))
    assert torch.allclose(p[0], torch.tensor([[1 / 3, 0.0], [0.25, 0.25]], dtype=F64))
    # the rotation: neighbours, by the position's angle
    x = torch.tensor([[[1.0, 0.0, 5.0, 7.0]]], dtype=F64)
    c, s = torch.tensor([[0.0]], dtype=F64), torch.tensor([[1.0]], dtype=F64)
    assert plain.rotate_pairs(x, c, s, 2)[0, 0].tolist() == [0.0, 1.0, 5.0, 7.0]
    # the streams: mix is indexed [from, to]
    streams = torch.tensor([[[1.0]], [[10.0]]], dtype=F64)
    hc = {"in": torch.tensor([1.0, 0.0], dtype=F64), "out": torch.tensor([0.0, 1.0], dtype=F64),
          "mix": torch.tensor([[0.0, 1.0], [0.0, 0.0]], dtype=F64)}
    out = plain.hyper_sublayer(streams, hc, torch.ones(1, dtype=F64), 0.0, lambda z: 100.0 * z)
    assert out.flatten().tolist() == [0.0, 101.0]


def test_pages_before_the_window_go_back_except_the_kept_first(tmp_path):
    """A layer with a window gives back the pages its window has moved past, but never a page that holds one of the
    first tokens it keeps; a released request gives back everything."""
    from pih_b200.engine import StepEntry
    from pih_b200.engine.factory import create_runner
    raw = pm.single_layer("attention_2", mask={"size": 9, "keep_first": 5})
    d = pm.write_model(tmp_path / "m", raw, seed=1, sigma=0.2)
    _, model, cache, runner = create_runner(d, "float32", device="cpu", page_size=4, max_cache_tokens=64, max_requests=1,
                                            ops=FakeOps())
    toks = traces.make_requests(120, [50], seed=1)["r0"]
    runner.step([StepEntry("a", toks[:40], [])])
    runner.step([StepEntry("a", toks[40:41], [0])])
    # 41 tokens: keys 32 .. 40 are in the window (pages 8 .. 10), keys 0 .. 4 are kept (pages 0, 1)
    assert cache.num_pages - cache.num_free_pages()[0] == 2 + 3
    cache.check()
    runner.finish("a")
    assert cache.num_free_pages()[0] == cache.num_pages


@pytest.mark.parametrize("name", ["P1", "P2", "P3"])
@pytest.mark.parametrize("family", ["whole", "tail_decode", "portions", "mixed"])
def test_cut_invariance_with_stand_in_kernels(tmp_path, name, family):
    """Block tables, slot mappings, the convolutions' state slots, the caches of a looped layer's passes, and the reuse
    of pages and slots: the real parts and step function with torch stand-ins for the kernels agree with the plain
    implementation however the requests are cut."""
    from pih_b200.engine.factory import create_runner
    d = pm.write_model(tmp_path / name, pm.CONFIGS[name], seed=1, sigma=pm.SIGMA[name])
    requests = traces.make_requests(pm.CONFIGS[name]["vocab"], [45, 6, 23, 1, 12, 2], seed=3)
    kw = dict(max_live=2, decode_tail=3, max_portion=7) if family == "mixed" else (dict(tail=20) if family == "tail_decode" else {})
    steps = getattr(traces, family)(requests, **kw)
    _, model, cache, runner = create_runner(d, "float32", device="cpu", page_size=4,
                                            max_cache_tokens=traces.peak_tokens(steps, round_to=4), max_requests=2,
                                            ops=FakeOps())
    # every pass of a looped layer has a cache of its own
    assert sum(len(g.entries) for g in cache.groups) == len(plain.layer_order(pm.CONFIGS[name]))
    got = traces.replay(runner, steps)
    for rid, ref in pm.plain_logits(d, requests).items():
        assert float((got[rid].double() - ref).abs().max()) < 2e-4 * float(ref.abs().max()), (family, rid)
    cache.check()
    assert cache.slots.num_free == 2 and all(f == cache.num_pages for f in cache.num_free_pages())


@pytest.mark.parametrize("seed", range(6))
def test_configurations_drawn_at_random_with_stand_in_kernels(tmp_path, seed):
    from pih_b200.engine.factory import create_runner
    raw = pm.random_config(seed)
    d = pm.write_model(tmp_path / "m", raw, seed=seed, sigma=0.15)
    requests = traces.make_requests(raw["vocab"], [40, 9, 21, 2], seed=seed)
    steps = traces.mixed(requests, seed=seed, max_live=2, decode_tail=4, max_portion=9)
    _, model, cache, runner = create_runner(d, "float32", device="cpu", page_size=8,
                                            max_cache_tokens=traces.peak_tokens(steps, round_to=8), max_requests=2, ops=FakeOps())
    got = traces.replay(runner, steps)
    for rid, ref in pm.plain_logits(d, requests).items():
        assert float((got[rid].double() - ref).abs().max()) < 2e-4 * float(ref.abs().max()), (seed, rid)
    cache.check()


def test_a_failed_step_leaves_the_convolution_state_as_it_was(tmp_path):
    """A step that raises after the layers have advanced their states is rolled back."""
    from pih_b200.engine import StepEntry
    from pih_b200.engine.factory import create_runner
    d = pm.write_model(tmp_path / "m", pm.P1, seed=2, sigma=pm.SIGMA["P1"])
    toks = traces.make_requests(307, [14], seed=1)["r0"]
    _, model, cache, runner = create_runner(d, "float32", device="cpu", page_size=4, max_cache_tokens=32, max_requests=1,
                                            ops=FakeOps())
    runner.step([StepEntry("a", toks[:9], [])])
    head = model.head
    model.head = None                                   # the head product fails, after every layer has run
    with pytest.raises(Exception):
        runner.step([StepEntry("a", toks[9:], [4])])
    model.head = head
    again = runner.step([StepEntry("a", toks[9:], [4])])
    ref = pm.plain_logits(d, {"a": toks})["a"][-1]
    assert float((again[0].double() - ref).abs().max()) < 2e-4 * float(ref.abs().max())
