"""The Sagelorn design written out plainly: float64, token by token, one function per mechanism.

Nothing here is shared with ``pih_b200``: the tests compare the engine with these functions.  A model is a dict
``config`` (the keys of config.json) and a dict ``w`` of float64 tensors by name (integer tables as they are).
"""
from __future__ import annotations

import math

import torch

F = torch.float64


def rms_unit(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def silu(z):
    return z * torch.sigmoid(z)


# -- embedding ---------------------------------------------------------------------------------------------------------
def embed(config, w, tokens, previous):
    """Rows of the token table plus rows of the bigram table, picked by a hash of the pair (token before, token);
    ``previous`` None (nothing came before): the row behind the hashed ones."""
    b = (config.get("embedding") or {}).get("bigram")
    if b is None:
        return w["embed"][torch.tensor(tokens)]
    rows = []
    for t in tokens:
        r = b["buckets"] if previous is None else (previous * b["mul_prev"] + t * b["mul_cur"]) % b["buckets"]
        rows.append(w["embed"][t] + w["bigram"][r])
        previous = t
    return torch.stack(rows)


# -- rotations -----------------------------------------------------------------------------------------------------------
def frequencies(rot):
    """f_i = base^(-2i/dims); with ``scaling`` the long waves are made longer: a wave shorter than original / high
    positions keeps its frequency, one longer than original / low gets f / factor, one in between a blend of the two."""
    dims = rot["dims"]
    out = []
    for i in range(dims // 2):
        f = rot["base"] ** (-2.0 * i / dims)
        sc = rot.get("scaling")
        if sc:
            wave = 2.0 * math.pi / f
            if wave > sc["original"] / sc["low"]:
                f = f / sc["factor"]
            elif wave >= sc["original"] / sc["high"]:
                s = (sc["original"] / wave - sc["low"]) / (sc["high"] - sc["low"])
                f = (1.0 - s) * f / sc["factor"] + s * f
        out.append(f)
    return torch.tensor(out, dtype=F)


def rotate(x, positions, rot, neighbours):
    """Rotation of the first ``dims`` columns of the last axis of x [T, ..., d] by positions [T]: column i is paired
    with column i + dims/2, or (``neighbours``) column 2i with column 2i + 1."""
    dims = rot["dims"]
    half = dims // 2
    ang = positions.to(F)[:, None] * frequencies(rot)[None, :]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [half]
    c, s = torch.cos(ang).reshape(shape), torch.sin(ang).reshape(shape)
    if neighbours:
        u, v = x[..., 0:dims:2], x[..., 1:dims:2]
        turned = torch.stack([u * c - v * s, v * c + u * s], dim=-1).reshape(x.shape[:-1] + (dims,))
        return torch.cat([turned, x[..., dims:]], dim=-1)
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


# -- mixers --------------------------------------------------------------------------------------------------------------
def attention_keys_values(h, m, w, pre, eps, start):
    """Keys after norm and rotation [T, G, dim] and values [T, G, vdim] of one sequence's rows."""
    T = h.shape[0]
    G, d, dv = m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(start, start + T)
    k = rms_unit(h @ w[pre + "k"].T, eps) * w[pre + "k.norm"]              # over the whole projection
    k = rotate(k.reshape(T, G, d), pos, m["rot"], neighbours=False)
    return k, (h @ w[pre + "v"].T).reshape(T, G, dv)


def attention(h, m, w, pre, eps, keys, values, start):
    """Softmax attention over a sliding window with a sink.  h [T, width]: the rows at positions start..; keys and
    values: ALL of the sequence's, from position 0 up to the last row."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(start, start + T)
    q = rms_unit(h @ w[pre + "q"].T, eps) * w[pre + "q.norm"]
    q = rotate(q.reshape(T, H, d), pos, m["rot"], neighbours=False)
    out = torch.zeros(T, H, dv, dtype=F)
    for t in range(T):
        p = start + t
        lo = max(0, p - m["mask"]["size"] + 1) if m.get("mask") else 0
        for hd in range(H):
            g = hd // (H // G)
            s = (keys[lo:p + 1, g] @ q[t, hd]) * m["scale"]
            e = torch.exp(s - s.max())
            out[t, hd] = (e / (e.sum() + math.exp(float(w[pre + "sink"][hd]) - float(s.max())))) @ values[lo:p + 1, g]
    return out.reshape(T, H * dv) @ w[pre + "o"].T


def latent_rows(h, m, w, pre, eps, start):
    """What latent attention caches per token: the normed latent [T, kv_rank] and the rotated key part [T, rot_dim]."""
    T = h.shape[0]
    R = m["kv_rank"]
    pos = torch.arange(start, start + T)
    down = h @ w[pre + "dkv"].T
    c = rms_unit(down[:, :R], eps) * w[pre + "dkv.norm"]
    return c, rotate(down[:, R:], pos, m["rot"], neighbours=True)


def latent_attention(h, m, w, pre, eps, latents, rotated_keys, start):
    """h [T, width]: the rows at positions start..; latents / rotated_keys: ALL of the sequence's."""
    T = h.shape[0]
    H, d, dr, dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(start, start + T)
    cq = rms_unit(h @ w[pre + "dq"].T, eps) * w[pre + "dq.norm"]
    q = (cq @ w[pre + "uq"].T).reshape(T, H, d + dr)
    q_plain, q_rot = q[..., :d], rotate(q[..., d:], pos, m["rot"], neighbours=True)
    k_plain = (latents @ w[pre + "uk"].T).reshape(-1, H, d)
    v = (latents @ w[pre + "uv"].T).reshape(-1, H, dv)
    out = torch.zeros(T, H, dv, dtype=F)
    for t in range(T):
        p = start + t
        lo = max(0, p - m["mask"]["size"] + 1) if m.get("mask") else 0
        for hd in range(H):
            s = (k_plain[lo:p + 1, hd] @ q_plain[t, hd] + rotated_keys[lo:p + 1] @ q_rot[t, hd]) * m["scale"]
            out[t, hd] = torch.softmax(s, dim=0) @ v[lo:p + 1, hd]
    gated = out.reshape(T, H * dv) * torch.sigmoid(h @ w[pre + "g"].T)
    return gated @ w[pre + "o"].T


def retention(h, m, w, pre, eps, S0=None):
    """One sequence: h [T, width] -> ([T, width], final state [heads, dim, vdim])."""
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    q = (h @ w[pre + "q"].T).reshape(T, H, d)
    k = (h @ w[pre + "k"].T).reshape(T, H, d) * d ** -0.5
    v = (h @ w[pre + "v"].T).reshape(T, H, dv)
    S = torch.zeros(H, d, dv, dtype=F) if S0 is None else S0.clone()
    decay = torch.tensor(m["decay"], dtype=F)
    o = torch.zeros(T, H, dv, dtype=F)
    for t in range(T):
        S = decay[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    o = rms_unit(o, eps).reshape(T, H * dv) * silu(h @ w[pre + "g"].T)
    return o @ w[pre + "o"].T, S


# -- feed-forwards ---------------------------------------------------------------------------------------------------------
def gated_ff(h, w, pre):
    return (silu(h @ w[pre + "gate"].T) * (h @ w[pre + "up"].T)) @ w[pre + "down"].T


def expert(h, w, pre):
    return (torch.relu(h @ w[pre + "up"].T) ** 2) @ w[pre + "down"].T


def route(h, f, w, pre):
    """Per row: the ``top`` outputs with the largest sigmoid scores (ties: the smaller index) and those scores."""
    s = torch.sigmoid(h @ w[pre + "router"].T)
    top = f["router"]["top"]
    chosen = torch.zeros(h.shape[0], top, dtype=torch.long)
    for t in range(h.shape[0]):
        order = sorted(range(s.shape[1]), key=lambda e: (-float(s[t, e]), e))
        chosen[t] = torch.tensor(order[:top])
    return chosen, torch.gather(s, 1, chosen)


def mixture(h, f, w, pre):
    """The chosen experts read the row times its weight; a shared expert reads every row as it is."""
    chosen, weights = route(h, f, w, pre)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, a in zip(chosen[t].tolist(), weights[t]):
            out[t] += expert(a * h[t:t + 1], w, f"{pre}e{e}.")[0]
    if f.get("shared"):
        out = out + expert(h, w, pre + "shared.")
    return out


def feed_forward(h, f, w, pre):
    return gated_ff(h, w, pre) if f["kind"] == "dense" else mixture(h, f, w, pre)


# -- the model ---------------------------------------------------------------------------------------------------------------
def model_layers(config, w, tokens, state=None):
    """One sequence's next ``tokens`` from ``state`` (None: a new sequence).  Returns (the stream after every layer
    [layers, T, width], logits [T, vocab], state)."""
    eps = config["norm"]["eps"]
    if state is None:
        state = {"n": 0, "previous": None, "S": {}, "K": {}, "V": {}}
    start = state["n"]
    x = embed(config, w, tokens, state["previous"])
    streams = []

    def grown(store, i, new):
        store[i] = new if i not in store else torch.cat([store[i], new])
        return store[i]

    for i, layer in enumerate(config["layers"]):
        m, pre = layer["mixer"], f"l{i}.mix."
        if layer["type"] == "retention":
            y, state["S"][i] = retention(x, m, w, pre, eps, state["S"].get(i))
        elif layer["type"] == "latent_attention":
            c, kr = latent_rows(x, m, w, pre, eps, start)
            y = latent_attention(x, m, w, pre, eps, grown(state["K"], i, c), grown(state["V"], i, kr), start)
        else:
            src = m.get("kv_from")
            if src is None:
                k, v = attention_keys_values(x, m, w, pre, eps, start)
                grown(state["K"], i, k)
                grown(state["V"], i, v)
                src = i
            y = attention(x, m, w, pre, eps, state["K"][src], state["V"][src], start)
        x = x + rms_unit(y, eps) * (1.0 + w[f"l{i}.norm1"])
        if layer.get("mlp"):
            x = x + rms_unit(feed_forward(x, layer["mlp"], w, f"l{i}.mlp."), eps) * (1.0 + w[f"l{i}.norm2"])
        streams.append(x)
    state["n"] = start + len(tokens)
    state["previous"] = tokens[-1]
    logits = (rms_unit(x, eps) * (1.0 + w["final.norm"])) @ w["head"].T * config.get("logit_scale", 1.0)
    return torch.stack(streams), logits, state
