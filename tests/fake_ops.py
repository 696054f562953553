"""A torch stand-in for the kernel pack, for tests of HOST-SIDE logic on the CPU.

The product has no CPU path.  This file lets the tests that run without a
GPU drive the real config, loader, parts, cache manager, batch builder,
step function and scheduler, so that faults in block tables, slot mappings
and request bookkeeping show up before a GPU is involved.  It mirrors the
method names of ``pih_b200.kernels.ops.CudaOps`` and nothing else of it.
"""
import torch


class FakeOps:
    launches = 0

    def __init__(self):
        self.error_word = torch.zeros(1, dtype=torch.int32)      # as the kernels' error word: first fault stays

    def _report(self, code):
        if int(self.error_word) == 0:
            self.error_word[0] = code

    def clear_errors(self):
        self.error_word.zero_()

    def check_errors(self):
        code = int(self.error_word)
        if code:
            self.clear_errors()
            raise RuntimeError(f"a kernel reported error code {code}")

    def embedding(self, table, ids, out_dtype=None):
        return table[ids.long()].to(out_dtype or table.dtype).clone()

    def rmsnorm(self, x, weight, eps, delta=None, rows=None):
        if rows is not None:
            v = x[rows.long()].float()
            if delta is not None:
                v = (v + delta[rows.long()].float()).to(x.dtype).float()
        else:
            v = x.float()
            if delta is not None:
                v = (v + delta.float()).to(x.dtype).float()
                x.copy_(v.to(x.dtype))
        scale = torch.rsqrt((v * v).sum(-1, keepdim=True) / v.shape[-1] + eps)
        return ((v * scale) * weight.float()).to(x.dtype)

    def linear(self, x, w, out_dtype=None):
        return (x.float() @ w.float().T).to(out_dtype or x.dtype)

    def qk_norm_rope_kv_write(self, qkv, *, heads, kv_heads, head_dim, q_norm, k_norm, eps, rope_table,
                              rotary_dim, positions, slot_mapping, kv_cache, write_kv):
        T = qkv.shape[0]
        D = head_dim
        page_size = kv_cache.shape[3]

        def norm_rope(x, w):                      # x [T, n, D]
            v = x.float()
            if w is not None:
                scale = torch.rsqrt((v * v).sum(-1, keepdim=True) / D + eps)
                v = ((v * scale) * w.float()).to(x.dtype).float()
            if rope_table is not None:
                cs = rope_table[positions.long()]        # [T, rot/2, 2]
                c, s = cs[..., 0][:, None, :], cs[..., 1][:, None, :]
                half = rotary_dim // 2
                a, b = v[..., :half], v[..., half:rotary_dim]
                v = torch.cat([a * c - b * s, b * c + a * s, v[..., rotary_dim:]], dim=-1)
            return v.to(x.dtype)

        q = qkv[:, :heads * D].reshape(T, heads, D)
        qkv[:, :heads * D] = norm_rope(q, q_norm).reshape(T, heads * D)
        if not write_kv:
            return
        k = qkv[:, heads * D:(heads + kv_heads) * D].reshape(T, kv_heads, D)
        v = qkv[:, (heads + kv_heads) * D:].reshape(T, kv_heads, D)
        k = norm_rope(k, k_norm)
        qkv[:, heads * D:(heads + kv_heads) * D] = k.reshape(T, kv_heads * D)
        sm = slot_mapping.long()
        assert (sm >= 0).all()
        page, off = sm // page_size, sm % page_size
        kv_cache[page, 0, :, off, :] = k
        kv_cache[page, 1, :, off, :] = v

    def paged_attention(self, qkv, *, heads, kv_heads, head_dim, kv_cache, block_table, step, scale, window):
        T, D = qkv.shape[0], head_dim
        page_size = kv_cache.shape[3]
        out = torch.zeros(T, heads, D, dtype=torch.float32)
        group = heads // kv_heads
        for t in range(T):
            r = int(step.request_of_row[t])
            p = int(step.positions[t])
            first = max(0, p - window + 1) if window else 0
            js = torch.arange(first, p + 1)
            pages = block_table[r, (js // page_size).long()].long()
            if not (pages >= 0).all():              # as the kernels: report "a row maps to no cache page", go on
                self._report(2)
                pages = pages.clamp(min=0)
            K = kv_cache[pages, 0, :, (js % page_size).long(), :].float()      # [n, kvh, D]
            V = kv_cache[pages, 1, :, (js % page_size).long(), :].float()
            q = qkv[t, :heads * D].reshape(heads, D).float()
            for h in range(heads):
                s = (K[:, h // group, :] @ q[h]) * scale
                out[t, h] = torch.softmax(s, dim=0) @ V[:, h // group, :]
        return out.reshape(T, heads * D).to(qkv.dtype)

    def silu_mul(self, gate_up, interleave=None):
        inter = gate_up.shape[1] // 2
        il = interleave or inter
        blocks = gate_up.reshape(gate_up.shape[0], inter // il, 2, il).float()
        g, u = blocks[:, :, 0, :].reshape(-1, inter), blocks[:, :, 1, :].reshape(-1, inter)
        return ((g / (1.0 + torch.exp(-g))) * u).to(gate_up.dtype)

    def norm_linear(self, h, delta, norm_weight, eps, w, swiglu_interleave=0):
        xn = self.rmsnorm(h, norm_weight, eps, delta=delta)
        out = self.linear(xn, w)
        if swiglu_interleave:
            out = self.silu_mul(out, swiglu_interleave)
        return h, out

    def argmax(self, logits):
        return torch.argmax(logits, dim=-1).to(torch.int32)

    def selected_logprob(self, logits, tokens, fparams=None, iparams=None):
        out = []
        for i in range(logits.shape[0]):
            t = float(fparams[i, 0]) if fparams is not None else 0.0
            scaled = logits[i].double() / (t if t > 0 else 1.0)
            keep = torch.ones(logits.shape[1], dtype=torch.bool)
            if iparams is not None:
                nsup = int(iparams[i, 5])
                keep[[int(v) for v in iparams[i, 6:6 + nsup].tolist()]] = False
            out.append(float(scaled[int(tokens[i])] - torch.logsumexp(scaled[keep], dim=0)))
        return torch.tensor(out, dtype=torch.float32)

    def top_logprobs(self, logits, count, fparams=None, iparams=None):
        from plain_impl import top_logprobs
        ids, lps = [], []
        for i in range(logits.shape[0]):
            t = float(fparams[i, 0]) if fparams is not None else 0.0
            nsup = int(iparams[i, 5]) if iparams is not None else 0
            sup = [int(v) for v in iparams[i, 6:6 + nsup].tolist()] if nsup else []
            top = top_logprobs(logits[i].tolist(), count, temperature=t, suppressed=sup)
            ids.append([a for a, _ in top])
            lps.append([b for _, b in top])
        return torch.tensor(ids, dtype=torch.int32), torch.tensor(lps, dtype=torch.float32)

    def sample(self, logits, fparams, iparams):
        from plain_impl import sample
        out = []
        for i in range(logits.shape[0]):
            ip = [int(v) & 0xFFFFFFFF for v in iparams[i].tolist()]
            nsup = ip[5]
            tok, _, _ = sample(logits[i].tolist(), temperature=float(fparams[i, 0]), top_p=float(fparams[i, 1]),
                               top_k=ip[0] or None, seed=ip[1] | (ip[2] << 32), ordinal=ip[3] | (ip[4] << 32),
                               suppressed=[int(v) for v in iparams[i, 6:6 + nsup].tolist()])
            out.append(tok)
        return torch.tensor(out, dtype=torch.int32)

    # -- a 32-bit residual stream, mixers with state, attention over a latent, routed experts ---------------------
    def rmsnorm_stream(self, h, weight, eps, delta=None, rows=None, out_dtype=torch.bfloat16):
        assert h.dtype == torch.float32
        if rows is not None:
            v = h[rows.long()]
            if delta is not None:
                v = v + delta[rows.long()].float()
        else:
            if delta is not None:
                h += delta.float()
            v = h
        return (v / torch.sqrt((v * v).mean(-1, keepdim=True) + eps) * weight).to(out_dtype)

    def linear_batched(self, x, w, out_dtype=None, rotate=None, gate=None):
        if rotate is not None:
            x = self.rotate_heads(x, **rotate)
        out = torch.einsum("tbk,bnk->tbn", x.float(), w.float()).to(out_dtype or x.dtype).contiguous()
        if gate is not None:
            T, B, N = out.shape
            out = self.gate_mul(out.view(T, B * N), gate, "sigmoid").view(T, B, N)
        return out

    @staticmethod
    def _requests(step):
        cu, slots = step.cu_q.tolist(), step.state_slots.tolist()
        return [(cu[r], cu[r + 1], slots[r]) for r in range(len(slots)) if cu[r + 1] > cu[r] and slots[r] >= 0]

    def causal_conv(self, x, w, *, step, state, state_offset, in_bias=None, out_bias=None, activation=None):
        T, C = x.shape
        taps = w.shape[1]
        out = torch.zeros(T, C, dtype=x.dtype)
        for lo, hi, slot in self._requests(step):
            hist = (state[slot, state_offset:state_offset + (taps - 1) * C].view(taps - 1, C) if taps > 1
                    else torch.zeros(0, C))                     # a single tap keeps no history
            xin = x[lo:hi].float() + (in_bias if in_bias is not None else 0.0)
            seq = torch.cat([hist, xin], dim=0)
            acc = torch.zeros(hi - lo, C)
            for j in range(taps):
                acc += seq[j:j + hi - lo] * w[:, j].float()[None, :]
            if out_bias is not None:
                acc += out_bias
            if activation == "silu":
                acc = acc * torch.sigmoid(acc)
            out[lo:hi] = acc.to(x.dtype)
            hist.copy_(seq[seq.shape[0] - (taps - 1):])
        return out

    def gated_delta_rule(self, qkv, ba, *, decay_log, decay_bias, state, step, heads, kv_heads, key_dim, value_dim,
                         unit_eps, q_scale):
        T = qkv.shape[0]
        QK = kv_heads * key_dim
        q = qkv[:, :QK].float().view(T, kv_heads, key_dim)
        k = qkv[:, QK:2 * QK].float().view(T, kv_heads, key_dim)
        v = qkv[:, 2 * QK:].float().view(T, heads, value_dim)
        q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + unit_eps) * q_scale
        k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + unit_eps)
        beta = torch.sigmoid(ba[:, :heads].float())
        decay = torch.exp(-torch.exp(decay_log) * torch.nn.functional.softplus(ba[:, heads:].float() + decay_bias))
        out = torch.zeros(T, heads, value_dim)
        per = heads // kv_heads
        for lo, hi, slot in self._requests(step):
            S = state[slot, :heads * key_dim * value_dim].view(heads, key_dim, value_dim)
            for t in range(lo, hi):
                for h in range(heads):
                    kk, qq = k[t, h // per], q[t, h // per]
                    S[h] *= decay[t, h]
                    u = beta[t, h] * (v[t, h] - S[h].T @ kk)
                    S[h] += torch.outer(kk, u)
                    out[t, h] = S[h].T @ qq
        return out

    def gated_rmsnorm(self, o, gate, weight, eps):
        T, heads, vdim = o.shape
        g = gate.float().view(T, heads, vdim)
        y = o / torch.sqrt((o * o).mean(-1, keepdim=True) + eps) * weight * (g * torch.sigmoid(g))
        return y.reshape(T, heads * vdim).to(gate.dtype)

    def rglru_scan(self, u, gates, y_pre, *, y_bias, r_bias, i_bias, lam, decay_scale, state, step, blocks):
        T, W = u.shape
        bw = W // blocks
        r = torch.sigmoid(gates[:, :, :bw].reshape(T, W) + r_bias)
        i = torch.sigmoid(gates[:, :, bw:].reshape(T, W) + i_bias)
        log_a = -decay_scale * r * torch.nn.functional.softplus(lam)
        a = torch.exp(log_a)
        mult = torch.sqrt(-torch.expm1(2 * log_a))
        y = y_pre.float() + y_bias
        y = 0.5 * y * (1 + torch.tanh(0.7978845608028654 * (y + 0.044715 * y ** 3)))
        out = torch.zeros(T, W, dtype=u.dtype)
        for lo, hi, slot in self._requests(step):
            S = state[slot, :W]
            for t in range(lo, hi):
                S.copy_(a[t] * S + mult[t] * i[t] * u[t].float())
                out[t] = (S * y[t]).to(u.dtype)
        return out

    @staticmethod
    def _turn(x, positions, frequencies, interleaved):
        """x [T, ..., rot]: every number of the last axis rotated, rot = 2 len(frequencies)."""
        rot = 2 * frequencies.shape[0]
        ang = positions.float()[:, None] * frequencies[None, :]
        shape = [x.shape[0]] + [1] * (x.dim() - 2) + [rot // 2]
        c, s = torch.cos(ang).reshape(shape), torch.sin(ang).reshape(shape)
        if interleaved:
            a, b = x[..., 0::2], x[..., 1::2]
            return torch.stack([a * c - b * s, b * c + a * s], dim=-1).reshape(x.shape)
        a, b = x[..., :rot // 2], x[..., rot // 2:]
        return torch.cat([a * c - b * s, b * c + a * s], dim=-1)

    def latent_write(self, raw, weight, eps, cache, slot_mapping, frequencies=None, interleaved=False, positions=None,
                     query_latent=None, query_weight=None):
        rot = 2 * frequencies.shape[0] if frequencies is not None else 0
        rank = raw.shape[1] - rot
        v = raw[:, :rank].float()
        c = v / torch.sqrt((v * v).mean(-1, keepdim=True) + eps) * weight
        if rot:
            c = torch.cat([c, self._turn(raw[:, rank:].float(), positions, frequencies, interleaved)], dim=-1)
        if cache.shape[-1] > c.shape[1]:                                     # columns of padding stay zero
            c = torch.cat([c, torch.zeros(c.shape[0], cache.shape[-1] - c.shape[1])], dim=-1)
        flat = cache.view(-1, cache.shape[-1])
        for t, slot in enumerate(slot_mapping.tolist()):
            if slot == -2:
                continue
            assert slot >= 0
            flat[slot] = c[t].to(cache.dtype)
        if query_latent is not None:
            return self.rmsnorm_rows(query_latent, query_weight, eps)

    def latent_attention(self, q, *, gate, sink, cache, block_table, step, scale, window=0):
        T, heads, rank = q.shape
        page_size = cache.shape[1]
        out = torch.zeros(T, heads, rank)
        for t in range(T):
            r = int(step.request_of_row[t])
            if r < 0:
                continue
            p = int(step.positions[t])
            js = torch.arange(max(0, p - window + 1) if window else 0, p + 1)
            pages = block_table[r, (js // page_size).long()].long()
            if not (pages >= 0).all():
                self._report(2)
                pages = pages.clamp(min=0)
            C = cache[pages, (js % page_size).long()].float()                    # [n, rank]
            s = (q[t].float() @ C.T) * scale                                     # [heads, n]
            if sink is not None:
                s = torch.cat([s, sink[:, None]], dim=1)
            w = torch.softmax(s, dim=-1)[:, :C.shape[0]]
            o = w @ C
            if gate is not None:
                o = o * torch.sigmoid(gate[t].float())[:, None]
            out[t] = o
        return out.to(q.dtype)

    @staticmethod
    def _scored_choice(logits, top, routing):
        n = routing["outputs"]
        if routing.get("scoring", "softmax") == "sigmoid":
            s = torch.sigmoid(logits[:, :n].float())
        else:
            s = torch.softmax(logits[:, :n].float(), dim=-1)
        c = s + (routing["correction"] if routing.get("correction") is not None else 0.0)
        groups, keep = routing.get("groups", 1), routing.get("groups_keep", 1)
        if groups > 1:
            best = c.view(-1, groups, n // groups).max(-1).values
            order = torch.argsort(best, dim=-1, descending=True, stable=True)[:, :keep]
            kept = torch.zeros_like(best, dtype=torch.bool).scatter_(1, order, True)
            c = torch.where(kept.repeat_interleave(n // groups, dim=1), c, torch.full_like(c, float("-inf")))
        idx = torch.argsort(c, dim=-1, descending=True, stable=True)[:, :top]
        wt = torch.gather(s, 1, idx)
        return idx, wt / wt.sum(-1, keepdim=True) if routing.get("renormalize") else wt

    def moe_experts(self, x, logits, w_gate_up, w_down, top, routing=None):
        if routing is not None and not routing.get("gated", True):
            # two-matrix experts around the squared ReLU; the weight on what the expert reads or on what it gives
            idx, wt = self._scored_choice(logits, top, routing)
            out = torch.zeros(x.shape, dtype=torch.float32)
            xf = x.float()
            on_input = routing.get("weigh", "output") == "input"
            for t in range(x.shape[0]):
                for j in range(top):
                    e = int(idx[t, j])
                    row = (xf[t] * wt[t, j]).to(x.dtype).float() if on_input else xf[t]
                    a = torch.relu((row @ w_gate_up[e].float().T).to(x.dtype).float()) ** 2
                    y = a.to(x.dtype).float() @ w_down[e].float().T
                    out[t] += y if on_input else wt[t, j] * y
            return out.to(x.dtype)
        ff = w_gate_up.shape[1] // 2
        w_gate, w_up = w_gate_up[:, :ff], w_gate_up[:, ff:]
        if routing is not None:
            idx, wt = self._scored_choice(logits, top, routing)
            out = torch.zeros(x.shape, dtype=torch.float32)
            xf = x.float()
            for t in range(x.shape[0]):
                for j in range(top):
                    e = int(idx[t, j])
                    if e >= w_gate_up.shape[0]:                                  # an identity expert
                        out[t] += wt[t, j] * xf[t]
                        continue
                    a = torch.nn.functional.silu(xf[t] @ w_gate[e].float().T) * (xf[t] @ w_up[e].float().T)
                    out[t] += wt[t, j] * (a @ w_down[e].float().T)
            return out.to(x.dtype)
        val, idx = torch.topk(logits, top, dim=-1)
        wt = torch.softmax(val, dim=-1)
        out = torch.zeros(x.shape, dtype=torch.float32)
        xf = x.float()
        for t in range(x.shape[0]):
            for j in range(top):
                e = int(idx[t, j])
                g, u = (xf[t] @ w_gate[e].float().T).to(x.dtype).float(), (xf[t] @ w_up[e].float().T).to(x.dtype).float()
                a = ((g * torch.sigmoid(g)) * u).to(x.dtype).float()
                out[t] += wt[t, j] * (a @ w_down[e].float().T)
        return out.to(x.dtype)

    # -- norms on the sub-layers' outputs, retention, differential attention, a biased feed-forward ---------------------
    def stream_cast(self, h, dtype):
        return h.to(dtype)

    def stream_norm_add(self, h, y, weight, eps, bias=None, copy_dtype=None):
        v = y.float() + (bias if bias is not None else 0.0)
        h += v / torch.sqrt((v * v).mean(-1, keepdim=True) + eps) * weight.float()
        return h.to(copy_dtype) if copy_dtype is not None else None

    def bias_xielu(self, z, bias, alpha_positive, alpha_negative):
        u = z.float() + (bias if bias is not None else 0.0)
        v = torch.where(u > 0, alpha_positive * u * u + 0.5 * u, alpha_negative * (torch.expm1(u.clamp(max=0.0)) - u) + 0.5 * u)
        return v.to(z.dtype)

    def add_gated(self, a, b, gate):
        if gate is None:
            return (a.float() + b.float()).to(a.dtype)
        return (a.float() + torch.sigmoid(gate)[:, None] * b.float()).to(a.dtype)

    @staticmethod
    def _rotate(x, positions, frequencies):
        """x [T, n, d]: rotate-half over the first 2 * len(frequencies) columns."""
        if frequencies is None:
            return x
        half = frequencies.shape[0]
        ang = positions.float()[:, None] * frequencies[None, :]
        c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
        u, v = x[..., :half], x[..., half:2 * half]
        return torch.cat([u * c - v * s, v * c + u * s, x[..., 2 * half:]], dim=-1)

    def retention(self, qk, v, *, frequencies, decay_minus_one, key_scale, state, step, heads, key_dim, value_dim):
        T = qk.shape[0]
        QK = heads * key_dim
        q = self._rotate(qk[:, :QK].float().view(T, heads, key_dim), step.positions, frequencies)
        k = self._rotate(qk[:, QK:].float().view(T, heads, key_dim), step.positions, frequencies) * key_scale
        vv = v.float().view(T, heads, value_dim)
        out = torch.zeros(T, heads, value_dim)
        for lo, hi, slot in self._requests(step):
            S = state[slot].view(heads, key_dim, value_dim)
            for t in range(lo, hi):
                S += decay_minus_one[:, None, None] * S + k[t][:, :, None] * vv[t][:, None, :]
                out[t] = torch.einsum("hdv,hd->hv", S, q[t])
        return out

    def diff_qk_prepare(self, qkv, *, q_norm, k_norm, eps, frequencies, positions, slot_mapping, cache, write_kv, heads,
                        kv_heads, key_dim, value_dim):
        T = qkv.shape[0]
        nq, nk = heads * 2 * key_dim, kv_heads * 2 * key_dim

        def prepared(x, w):
            x = x.float().view(T, -1, key_dim)
            if w is not None:
                x = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w
            return self._rotate(x, positions, frequencies).reshape(T, -1)

        qkv[:, :nq] = prepared(qkv[:, :nq], q_norm).to(qkv.dtype)
        if write_kv:
            k = prepared(qkv[:, nq:nq + nk], k_norm)
            flat = cache.view(-1, cache.shape[-1])
            for t, slot in enumerate(slot_mapping.tolist()):
                if slot == -2:
                    continue
                assert slot >= 0
                flat[slot, :nk] = k[t].to(cache.dtype)
                flat[slot, nk:] = qkv[t, nq + nk:]

    def diff_attention(self, qkv, *, cache, block_table, step, scale, lam, out_scale, norm_eps, window, heads, kv_heads,
                       key_dim, value_dim):
        T = qkv.shape[0]
        page_size = cache.shape[1]
        nk = kv_heads * 2 * key_dim
        out = torch.zeros(T, heads, value_dim)
        for t in range(T):
            r = int(step.request_of_row[t])
            if r < 0:
                continue
            p = int(step.positions[t])
            js = torch.arange(max(0, p - window + 1) if window else 0, p + 1)
            pages = block_table[r, (js // page_size).long()].long()
            if not (pages >= 0).all():
                self._report(2)
                pages = pages.clamp(min=0)
            C = cache[pages, (js % page_size).long()].float()
            K = C[:, :nk].view(-1, kv_heads, 2, key_dim)
            V = C[:, nk:].view(-1, kv_heads, value_dim)
            q = qkv[t, :heads * 2 * key_dim].float().view(heads, 2, key_dim)
            for h in range(heads):
                g = h // (heads // kv_heads)
                a = [torch.softmax((K[:, g, j] @ q[h, j]) * scale, dim=0) @ V[:, g] for j in range(2)]
                out[t, h] = a[0] - lam * a[1]
        out = out / torch.sqrt((out * out).mean(-1, keepdim=True) + norm_eps) * out_scale
        return out.reshape(T, heads * value_dim).to(qkv.dtype)

    # -- several residual streams, attention over a window with a sink ----------------------------------------------
    def act_mul(self, gate_up, interleave=None, activation="silu"):
        if activation == "silu":
            return self.silu_mul(gate_up, interleave)
        assert activation == "gelu_tanh"
        inter = gate_up.shape[1] // 2
        il = interleave or inter
        blocks = gate_up.reshape(gate_up.shape[0], inter // il, 2, il).float()
        g, u = blocks[:, :, 0, :].reshape(-1, inter), blocks[:, :, 1, :].reshape(-1, inter)
        return (0.5 * g * (1.0 + torch.tanh(0.7978845608028654 * (g + 0.044715 * g ** 3))) * u).to(gate_up.dtype)

    def embed_positions(self, table, places, ids, positions, streams=1, out_dtype=torch.float32):
        x = table[ids.long()].float()
        if places is not None:
            x = x + places[positions.long()].float()
        return x[:, None, :].repeat(1, streams, 1).to(out_dtype).contiguous()

    def hyper_stream(self, x, y, *, mix=None, spread=None, collect=None, weight=None, eps=0.0, rows=None, out_dtype=None):
        assert x.dtype == torch.float32
        v = x if rows is None else x[rows.long()]
        if y is not None:
            yy = (y if rows is None else y[rows.long()]).float()
            v = torch.einsum("st,nsw->ntw", mix, v) + spread[None, :, None] * yy[:, None, :]
            if rows is None:
                x.copy_(v)
        if collect is None:
            return None
        u = torch.einsum("t,ntw->nw", collect, v)
        if weight is not None:
            u = u / torch.sqrt((u * u).mean(-1, keepdim=True) + eps) * weight
        return u.to(out_dtype or torch.float32)

    def window_qk_prepare(self, src, *, q_norm, k_norm, eps, rope_table, rotary_dim, interleaved, positions, slot_mapping,
                          cache, heads, kv_heads, key_dim, value_dim, values_from_keys, frequencies=None, write_kv=True):
        T = src.shape[0]
        nq, nk, nv = heads * key_dim, kv_heads * key_dim, kv_heads * value_dim

        def prepared(x, w):
            x = x.float()
            if w is not None:
                x = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w
            x = x.view(T, -1, key_dim).clone()
            if rope_table is not None:
                cs = rope_table[positions.long()]                       # [T, rot / 2, 2]
                c, s = cs[..., 0][:, None, :], cs[..., 1][:, None, :]
                if interleaved:
                    a, b = x[..., 0:rotary_dim:2].clone(), x[..., 1:rotary_dim:2].clone()
                    x[..., 0:rotary_dim:2], x[..., 1:rotary_dim:2] = a * c - b * s, b * c + a * s
                else:
                    half = rotary_dim // 2
                    a, b = x[..., :half].clone(), x[..., half:rotary_dim].clone()
                    x[..., :half], x[..., half:rotary_dim] = a * c - b * s, b * c + a * s
            elif frequencies is not None:
                x[..., :rotary_dim] = self._turn(x[..., :rotary_dim].clone(), positions, frequencies, interleaved)
            return x.reshape(T, -1)

        q = prepared(src[:, :nq], q_norm).to(src.dtype)
        if not write_kv:
            return q
        k = prepared(src[:, nq:nq + nk], k_norm).to(src.dtype)
        v = src[:, nq:nq + nk] if values_from_keys else src[:, nq + nk:nq + nk + nv]
        flat = cache.view(-1, cache.shape[-1])
        for t, slot in enumerate(slot_mapping.tolist()):
            if slot == -2:
                continue
            assert slot >= 0
            flat[slot, :nk] = k[t]
            flat[slot, nk:] = v[t]
        return q

    def window_attention(self, q, *, cache, block_table, step, scale, window, keep_first, softcap, bias, sink, gate, heads,
                         kv_heads, key_dim, value_dim):
        T = q.shape[0]
        page_size = cache.shape[1]
        nk = kv_heads * key_dim
        out = torch.zeros(T, heads, value_dim)
        for t in range(T):
            r = int(step.request_of_row[t])
            if r < 0:
                continue
            p = int(step.positions[t])
            js = torch.arange(0, p + 1)
            if window:
                js = js[(p - js < window) | (js < keep_first)]
            pages = block_table[r, (js // page_size).long()].long()
            if not (pages >= 0).all():
                self._report(2)
                pages = pages.clamp(min=0)
            C = cache[pages, (js % page_size).long()].float()
            K = C[:, :nk].view(-1, kv_heads, key_dim)
            V = C[:, nk:].view(-1, kv_heads, value_dim)
            qq = q[t].float().view(heads, key_dim)
            for h in range(heads):
                g = h // (heads // kv_heads)
                s = (K[:, g] @ qq[h]) * scale
                if softcap:
                    s = softcap * torch.tanh(s / softcap)
                if bias is not None:
                    s = s + bias[h, (p - js).clamp(max=bias.shape[1] - 1)]
                m = s.max() if sink is None else torch.maximum(s.max(), sink[h])
                e = torch.exp(s - m)
                den = e.sum() + (torch.exp(sink[h] - m) if sink is not None else 0.0)
                o = (e / den) @ V[:, g]
                if gate is not None:
                    o = o * torch.sigmoid(gate[t, h].float())
                out[t, h] = o
        return out.reshape(T, heads * value_dim).to(q.dtype)

    # -- a bigram embedding, rotations by computed angles, gates a column, two-matrix experts -----------------------------
    def embed_bigram(self, table, bigram, step, *, state, mul_prev, mul_cur, buckets, out_dtype=None):
        ids, pos = step.token_ids.tolist(), step.positions.tolist()
        req, cu, slots = step.request_of_row.tolist(), step.cu_q.tolist(), step.state_slots.tolist()
        rows = []
        for t, tok in enumerate(ids):
            prev = None
            if req[t] >= 0 and pos[t] > 0:
                prev = int(state[slots[req[t]], 0]) if t == cu[req[t]] else ids[t - 1]
            rows.append(buckets if prev is None else (prev * mul_prev + tok * mul_cur) % buckets)
        for r in range(len(slots)):
            if slots[r] >= 0 and cu[r + 1] > cu[r]:
                state[slots[r], 0] = ids[cu[r + 1] - 1]
        out = table[step.token_ids.long()].float() + bigram[torch.tensor(rows)].float()
        return out.to(out_dtype or table.dtype)

    def rmsnorm_rows(self, x, weight, eps):
        v = x.float()
        return (v / torch.sqrt((v * v).mean(-1, keepdim=True) + eps) * weight).to(x.dtype)

    def rotate_heads(self, x, *, offset, frequencies, interleaved, positions):
        out = x.float().clone()
        rot = 2 * frequencies.shape[0]
        out[..., offset:offset + rot] = self._turn(out[..., offset:offset + rot].clone(), positions, frequencies, interleaved)
        return out.to(x.dtype).contiguous()

    def gate_mul(self, a, gate, kind="sigmoid"):
        g = gate.float()
        return (a.float() * (torch.sigmoid(g) if kind == "sigmoid" else g * torch.sigmoid(g))).to(a.dtype)

    def activation(self, z, kind):
        assert kind == "relu2"
        return (torch.relu(z.float()) ** 2).to(z.dtype)

    def scale_(self, x, scale):
        return x.mul_(scale)
