"""The Pegopel design written out plainly in float64, one function a mechanism, whole sequences at once.

Nothing here is shared with the engine: no cache, no pages, no portions.  A sequence's tokens go in, every position's
logits come out, so that the engine's prefill, decoding, portions and batches can all be held against the same numbers.

Notation: ``T`` tokens, ``W`` width, ``H`` query heads, ``G`` key/value heads, ``d`` key size, ``e`` value size.
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def rms_norm(x, w, eps):
    """``x / sqrt(mean(x^2) + eps) * w`` over the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps) * w


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def short_conv(u, w):
    """Causal convolution per channel: ``u [T, C]``, ``w [C, taps]``; the last tap weighs the current token, tokens
    before the sequence count as zeros."""
    T, C = u.shape
    taps = w.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, C, dtype=u.dtype), u], dim=0)
    out = torch.zeros_like(u)
    for j in range(taps):
        out += w[:, j] * padded[j:j + T]
    return out


def distance_bucket(n: int, rows: int, far: float) -> int:
    """Row of the bias table for the distance ``n >= 0``: the first half of the rows one a distance, the other half
    spread logarithmically up to the distance ``far``."""
    half = rows // 2
    if n < half:
        return n
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))


def distance_bias(table, far, T):
    """``[T, T, H]``: entry (i, j) is the bias of query i on key j (zero where j > i)."""
    rows, H = table.shape
    out = torch.zeros(T, T, H, dtype=F64)
    for i in range(T):
        for j in range(i + 1):
            out[i, j] = table[distance_bucket(i - j, rows, far)]
    return out


def sink_softmax(scores, visible, sink):
    """Softmax over the visible keys of each row with ``exp(sink)`` added to the denominator: ``scores [H, T, T]``,
    ``visible [T, T]`` (bool), ``sink [H]``."""
    s = scores.masked_fill(~visible, -math.inf)
    m = torch.maximum(s.max(dim=-1).values, sink[:, None])
    p = torch.exp(s - m[..., None])
    return p / (p.sum(dim=-1) + torch.exp(sink[:, None] - m))[..., None]


def window_mask(T, size, keep_first=0):
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    return (j <= i) & ((i - j < size) | (j < keep_first))


def yarn_rotation(dims, base, scaling, positions):
    """Cosines and sines ``[T, dims / 2]`` of the rotation with stretched low frequencies; ``scaling`` None: plain."""
    i = torch.arange(dims // 2, dtype=F64)
    f = torch.pow(torch.tensor(base, dtype=F64), -2.0 * i / dims)
    gain = 1.0
    if scaling is not None:
        factor, original = float(scaling["factor"]), float(scaling["original"])

        def turn(t):
            return dims * math.log(original / (2.0 * math.pi * t)) / (2.0 * math.log(base))

        lo = max(math.floor(turn(float(scaling["fast"]))), 0)
        hi = min(math.ceil(turn(float(scaling["slow"]))), dims - 1)
        ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
        f = f / factor * ramp + f * (1.0 - ramp)
        gain = 0.1 * math.log(factor) + 1.0
    a = positions.to(F64)[:, None] * f[None, :]
    return torch.cos(a) * gain, torch.sin(a) * gain


def rotate_pairs(x, cos, sin, dims):
    """Neighbouring pairs (2i, 2i + 1) of the first ``dims`` columns of every head are rotated: ``x [T, heads, d]``."""
    out = x.clone()
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    c, s = cos[:, None, :], sin[:, None, :]
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


def attend(q, k, v, weights_of):
    """``q [T, H, d]``, ``k [T, G, d]``, ``v [T, G, e]``; ``weights_of(scores [H, T, T]) -> [H, T, T]``."""
    T, H, d = q.shape
    G = k.shape[1]
    kk = k.repeat_interleave(H // G, dim=1)
    vv = v.repeat_interleave(H // G, dim=1)
    p = weights_of(torch.einsum("ihd,jhd->hij", q, kk))
    return torch.einsum("hij,jhe->ihe", p, vv)


def conv_bias_attention(h, w, m, eps):
    """The mixer with short convolutions, a distance bias and a learned sink.  ``w``: tensors by their name behind
    ``mix.``; ``m``: the mixer's configuration."""
    T = h.shape[0]
    H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = short_conv(h @ w["q"].T, w["q.conv"])
    k = short_conv(h @ w["k"].T, w["k.conv"])
    v = short_conv(h @ w["v"].T, w["v.conv"])
    q = rms_norm(q, w["q.norm"], eps).reshape(T, H, d)
    k = rms_norm(k, w["k.norm"], eps).reshape(T, G, d)
    bias = distance_bias(w["rel"], m["bias_max"], T).permute(2, 0, 1)
    visible = window_mask(T, m["mask"]["size"])
    o = attend(q, k, v.reshape(T, G, e), lambda s: sink_softmax(s * m["scale"] + bias, visible, w["sink"]))
    return o.reshape(T, H * e) @ w["o"].T


def key_value_attention(h, w, m, eps):
    """The mixer whose values are its keys as projected: rotation, capped scores, kept first tokens, a sink of
    score zero and a gate a head."""
    T = h.shape[0]
    H, G, d = m["heads"], m["kv_heads"], m["dim"]
    q = h @ w["q"].T
    k_raw = h @ w["k"].T
    v = k_raw.reshape(T, G, d)
    q = rms_norm(q, w["q.norm"], eps).reshape(T, H, d)
    k = rms_norm(k_raw, w["k.norm"], eps).reshape(T, G, d)
    rot = m.get("rot")
    if rot is not None:
        cos, sin = yarn_rotation(rot["dims"], rot["base"], rot.get("scaling"), torch.arange(T))
        q, k = rotate_pairs(q, cos, sin, rot["dims"]), rotate_pairs(k, cos, sin, rot["dims"])
    cap = m.get("softcap")
    visible = window_mask(T, m["mask"]["size"], m["mask"].get("keep_first", 0))

    def weights_of(s):
        s = s * m["scale"]
        if cap is not None:
            s = cap * torch.tanh(s / cap)
        return sink_softmax(s, visible, torch.zeros(H, dtype=F64))

    o = attend(q, k, v, weights_of)
    gate = torch.sigmoid(h @ w["g"].T)                                  # [T, H]
    return (o * gate[:, :, None]).reshape(T, H * d) @ w["o"].T


def gated_feed_forward(h, w):
    return (gelu_tanh(h @ w["gate"].T) * (h @ w["up"].T)) @ w["down"].T


def hyper_sublayer(streams, hc, norm_w, eps, sublayer):
    """``streams [S, T, W]``; ``hc``: 'in' [S], 'out' [S], 'mix' [S, S] indexed [from, to]."""
    u = torch.einsum("s,stw->tw", hc["in"], streams)
    y = sublayer(rms_norm(u, norm_w, eps))
    return torch.einsum("sr,stw->rtw", hc["mix"], streams) + hc["out"][:, None, None] * y[None]


def layer_order(config):
    n = len(config["layers"])
    loop = config.get("loop")
    if not loop:
        return list(range(n))
    a, b, times = loop["start"], loop["stop"], loop["times"]
    return list(range(a)) + list(range(a, b)) * times + list(range(b, n))


def _sub(weights, prefix):
    return {k[len(prefix):]: v.to(F64) for k, v in weights.items() if k.startswith(prefix)}


def forward(config, weights, tokens, with_layers=False):
    """Logits ``[T, vocab]`` (float64) of one sequence; with ``with_layers`` also the summed streams behind every
    layer that ran."""
    eps = config["norm"]["eps"]
    T = len(tokens)
    x = weights["embed"].to(F64)[torch.tensor(tokens)] + weights["pos"].to(F64)[:T]
    S = config.get("streams", 0)
    streams = x[None].repeat(max(S, 1), 1, 1)
    seen = []
    for i in layer_order(config):
        layer = config["layers"][i]
        p = f"l{i}."
        mixer = conv_bias_attention if layer["type"] == "attention" else key_value_attention
        mw, m = _sub(weights, p + "mix."), layer["mixer"]
        subs = [("hc1.", p + "norm1", lambda z: mixer(z, mw, m, eps))]
        if layer.get("mlp") is not None:
            fw = _sub(weights, p + "mlp.")
            subs.append(("hc2.", p + "norm2", lambda z: gated_feed_forward(z, fw)))
        for hc_name, norm_name, fn in subs:
            if S:
                streams = hyper_sublayer(streams, _sub(weights, p + hc_name), weights[norm_name].to(F64), eps, fn)
            else:
                streams = streams + fn(rms_norm(streams[0], weights[norm_name].to(F64), eps))[None]
        seen.append(streams.sum(dim=0))
    x = streams.sum(dim=0)
    logits = rms_norm(x, weights["final.norm"].to(F64), eps) @ weights["embed"].to(F64).T
    return (logits, torch.stack(seen)) if with_layers else logits
