"""A stand-in for ullm_b200.csrc.ops.Kernels written in plain torch, so that the
host-side logic of the engine (block tables, slot mappings, batching, windows,
scheduling) can be exercised without a GPU.  It is a test double: nothing in
the package imports it, and on a GPU the real kernels run.  It follows the
kernels' contracts (in-place updates, -1 slots skipped, padding rows zero)."""

from __future__ import annotations

import math

import torch


class CpuKernels:
    def __init__(self):
        self.status = torch.zeros(4, dtype=torch.int32)
        self.timer = None
        self.calls = {}

    def _count(self, name):
        self.calls[name] = self.calls.get(name, 0) + 1

    def raise_on_status(self):
        pass

    def linear(self, x, weight, out, bias=None):
        self._count("linear")
        y = x.float() @ weight.float().t()
        if bias is not None:
            y = y + bias.float()
        out.copy_(y.to(out.dtype))
        return out

    def linear_act_mul(self, x, weight, out, gate_up, act=0):
        self.linear(x, weight, gate_up)
        self.act_mul(gate_up, out, act)
        return out

    def linear_f32_out(self, x, weight, out):
        self._count("linear")
        out.copy_(x.float() @ weight.float().t())
        return out

    def embedding(self, ids, table, out, last_tokens=None, token_req=None, req_slots=None):
        self._count("embedding")
        idx = ids[: out.shape[0]].long().clone()
        if last_tokens is not None:
            for t in (idx < 0).nonzero().flatten().tolist():
                b = int(token_req[t])
                idx[t] = int(last_tokens[int(req_slots[b])]) if b >= 0 else 0
        out.copy_(table[idx])

    def gather_rows(self, src, rows, out):
        self._count("gather_rows")
        out.copy_(src[rows[: out.shape[0]].long()])

    def add_rmsnorm(self, x, residual, weight, eps, out):
        self._count("add_rmsnorm")
        s = x.float()
        if residual is not None:
            s = s + residual.float()
            residual.copy_(s.to(residual.dtype))
        y = s * torch.rsqrt(s.pow(2).mean(-1, keepdim=True) + eps) * weight
        out.copy_(y.to(out.dtype))

    def act_mul(self, gate_up, out, act=0):
        self._count("act_mul")
        I = out.shape[1]
        g, u = gate_up[:, :I].float(), gate_up[:, I:].float()
        a = g * torch.sigmoid(g) if act == 0 else torch.nn.functional.gelu(g, approximate="tanh")
        out.copy_((a * u).to(out.dtype))

    def layer_tail_applies(self, *args, **kwargs):
        return False

    def stream_chain_applies(self, *args, **kwargs):
        return False

    def decode_fusion_applies(self, *args, **kwargs):
        return False  # the stand-in always prepares q and k in a step of their own

    def qk_norm_rope_store(self, qkv, num_q, num_kv, D, q_w, k_w, eps, cos, sin, rotary_dim, positions,
                           slot_mapping, k_pages, v_pages, v_dim=None, kv_in_row=True):
        self._count("qk_norm_rope_store")
        T = qkv.shape[0]
        Dv = D if v_dim is None else v_dim
        x = qkv.float().clone()
        q = x[:, :num_q * D].reshape(T, num_q, D)
        if kv_in_row:
            k = x[:, num_q * D:(num_q + num_kv) * D].reshape(T, num_kv, D)
            v = x[:, (num_q + num_kv) * D:].reshape(T, num_kv, Dv)
        else:
            k, v, slot_mapping = q[:, :0], None, None

        def norm(t, w):
            if w is None:
                return t
            return t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + eps) * w

        def rope(t):
            if rotary_dim == 0:
                return t
            half = rotary_dim // 2
            c = cos[positions[:T].long()][:, None, :]
            s = sin[positions[:T].long()][:, None, :]
            x1, x2, rest = t[..., :half], t[..., half:rotary_dim], t[..., rotary_dim:]
            return torch.cat((x1 * c - x2 * s, x2 * c + x1 * s, rest), -1)

        q = rope(norm(q, q_w))
        k = rope(norm(k, k_w))
        qkv[:, : num_q * D] = q.reshape(T, num_q * D).to(qkv.dtype)
        if slot_mapping is not None:
            kf = k_pages.view(-1, num_kv, D)
            vf = v_pages.view(-1, num_kv, Dv)
            sm = slot_mapping[:T].long()
            ok = sm >= 0
            kf[sm[ok]] = k[ok].to(kf.dtype)
            vf[sm[ok]] = v[ok].to(vf.dtype)

    def qk_norm_in_place(self, qkv, num_q, num_kv, D, q_w, k_w, eps):
        T = qkv.shape[0]
        x = qkv.float().clone().view(T, num_q + 2 * num_kv, D)
        for lo, hi, w in ((0, num_q, q_w), (num_q, num_q + num_kv, k_w)):
            if w is not None:
                t = x[:, lo:hi]
                x[:, lo:hi] = t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + eps) * w
        qkv.copy_(x.view(T, -1).to(qkv.dtype))

    def paged_attention(self, qkv, out, k_pages, v_pages, block_table, req_slots, cu_q, kv_len, token_req,
                        num_q, num_kv, D, page_size, window, scale, ctx=None, ragged=False, v_dim=None, keep_first=0,
                        softcap=0.0, parts=None, general=False):
        self._count("paged_attention")
        T = out.shape[0]
        Dv = D if v_dim is None else v_dim
        kf = k_pages.view(-1, num_kv, D).float()
        vf = v_pages.view(-1, num_kv, Dv).float()
        q = qkv[:T, : num_q * D].float().reshape(T, num_q, D)
        group = num_q // num_kv
        o = torch.zeros(T, num_q, Dv)
        if parts is not None:
            parts.zero_()
        for t in range(T):
            r = int(token_req[t])
            if r < 0:
                continue
            qlen = int(cu_q[r + 1] - cu_q[r])
            kvl = int(kv_len[r])
            pos = kvl - qlen + (t - int(cu_q[r]))
            if qlen <= 0 or kvl <= 0 or pos < 0:
                continue
            lo = max(0, pos - window + 1) if window > 0 else 0
            keys = torch.cat((torch.arange(0, min(keep_first, lo)), torch.arange(lo, pos + 1)))
            pages = block_table[int(req_slots[r])][(keys // page_size).long()].long()
            assert (pages >= 0).all(), "attention touched a page that was given back"
            slots = pages * page_size + keys % page_size
            for h in range(num_q):
                kh = h // group
                s = (kf[slots, kh] @ q[t, h]) * scale
                if softcap > 0:
                    s = softcap * torch.tanh(s / softcap)
                p = torch.softmax(s, 0)
                o[t, h] = p @ vf[slots, kh]
                if parts is not None:
                    parts.view(T, num_q, num_kv, Dv)[t, h] = torch.einsum("j,jcd->cd", p, vf[slots])
        if parts is None:
            out.copy_(o.reshape(T, num_q * Dv).to(out.dtype))

    def mix_heads(self, parts, mix, out, num_q, num_kv, v_dim):
        T = out.shape[0]
        p = parts.view(T, num_q, num_kv, v_dim)
        own = p[:, :, torch.arange(num_q) // (num_q // num_kv)]  # [T, g, h, dv]: head g's weights on head h's values
        out.copy_(torch.einsum("hg,tghd->thd", mix.float(), own).reshape(T, -1).to(out.dtype))

    def qkv_prepare(self, qkv, q_out, num_q, num_kv, head_dim, v_dim, positions, slot_mapping, k_pages, v_pages, *,
                    conv_w=None, taps=0, conv_state=None, cu_q=None, token_req=None, req_slots=None, inv_freq=None,
                    rotary_dim=0, q_w=None, k_w=None, norm_first=False, norm_last=False, eps=0.0, vmix_mode=0,
                    vmix_lambda=None, v_first=None):
        self._count("qkv_prepare")
        T, W = qkv.shape
        x = qkv.float().clone()
        if conv_w is not None:
            y = torch.zeros_like(x)
            for t in range(T):
                r = int(token_req[t])
                if r < 0:
                    y[t] = x[t]
                    continue
                t0 = int(cu_q[r])
                for j in range(taps):
                    row = t - (taps - 1 - j)
                    if row >= t0:
                        u = x[row]
                    else:
                        u = conv_state[int(req_slots[r])].view(-1, W)[taps - 1 - (t0 - row)]
                    y[t] += conv_w[:, j].float() * u
            x = y
        qs, ks = num_q * head_dim, num_kv * head_dim
        q, k, v = x[:, :qs].reshape(T, num_q, head_dim), x[:, qs:qs + ks].reshape(T, num_kv, head_dim), x[:, qs + ks:]

        def unit(u, w):
            u = u / torch.sqrt(u.pow(2).mean(-1, keepdim=True) + eps)
            return u * w if w is not None else u

        if norm_first:
            q, k = unit(q, q_w), unit(k, k_w)
        if rotary_dim > 0:
            half = rotary_dim // 2
            ang = positions[:T].float()[:, None] * inv_freq[None, :half]
            cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]

            def rot(u):
                a, b = u[..., :half], u[..., half:rotary_dim]
                return torch.cat((a * cos - b * sin, b * cos + a * sin, u[..., rotary_dim:]), -1)

            q, k = rot(q), rot(k)
        if norm_last:
            q, k = unit(q, None), unit(k, None)
        if vmix_mode == 2:
            lam = float(vmix_lambda)
            v = (1.0 - lam) * v + lam * v_first.float()
        v = v.to(qkv.dtype)
        if vmix_mode == 1:
            v_first.copy_(v)
        q_out.copy_(q.reshape(T, -1).to(q_out.dtype))
        if slot_mapping is not None:
            kf, vf = k_pages.view(-1, num_kv, head_dim), v_pages.view(-1, num_kv, v_dim)
            for t in range(T):
                s = int(slot_mapping[t])
                if s >= 0:
                    kf[s] = k[t].to(kf.dtype)
                    vf[s] = v[t].view(num_kv, v_dim)

    def conv_state_update(self, qkv, taps, conv_state, cu_q, token_req, req_slots, requests):
        W = qkv.shape[1]
        for r in range(requests):
            t0, t1 = int(cu_q[r]), int(cu_q[r + 1])
            if t1 <= t0 or int(token_req[t0]) < 0:
                continue
            st = conv_state[int(req_slots[r])].view(-1, W)[: taps - 1]
            rows = torch.cat((st, qkv[t0:t1].float()))[-(taps - 1):]
            st.copy_(rows)

    def gla_recurrence(self, qkv, q_off, k_off, v_off, z, z_bias, inv_tau, q_scale, state, cu_q, req_slots, token_req,
                       out, requests, heads, dim, vdim):
        self._count("gla")
        x = qkv.float()
        for r in range(requests):
            t0, t1 = int(cu_q[r]), int(cu_q[r + 1])
            if t1 <= t0:
                continue
            if int(token_req[t0]) < 0:
                out[t0:t1] = 0
                continue
            S = state[int(req_slots[r])][: heads * vdim * dim].view(heads, vdim, dim)
            for t in range(t0, t1):
                q = x[t, q_off:q_off + heads * dim].view(heads, dim) * q_scale
                k = x[t, k_off:k_off + heads * dim].view(heads, dim)
                v = x[t, v_off:v_off + heads * vdim].view(heads, vdim)
                zz = z[t] + (z_bias if z_bias is not None else 0)
                a = torch.exp(torch.nn.functional.logsigmoid(zz) * inv_tau).view(heads, dim)
                S.mul_(a[:, None, :]).add_(v[:, :, None] * k[:, None, :])
                out[t] = torch.einsum("hvd,hd->hv", S, q).reshape(-1)

    def head_norm_gate(self, o, g, weight, eps, out, heads, vdim, silu=False):
        T = o.shape[0]
        x = o.view(T, heads, vdim)
        x = x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)
        w = weight.view(heads, vdim) if weight.numel() == heads * vdim else weight.view(1, vdim)
        gf = g.float()
        gate = torch.nn.functional.silu(gf) if silu else torch.sigmoid(gf)
        out.copy_(((x * w).reshape(T, -1) * gate).to(out.dtype))

    def gated_add_f32(self, a, f, gates, b1, b2, stream, copy=None):
        self._count("add_rmsnorm")
        W = a.shape[1]
        stream += torch.sigmoid(gates[:, :W] + b1) * a.float()
        if f is not None:
            stream += torch.sigmoid(gates[:, W:] + b2) * f.float()
        if copy is not None:
            copy.copy_(stream.to(copy.dtype))

    def side_gate_mul(self, s, ids, table, offset, out, last_tokens=None, token_req=None, req_slots=None):
        T, C = s.shape
        idx = ids[:T].long().clone()
        if last_tokens is not None:
            for t in (idx < 0).nonzero().flatten().tolist():
                b = int(token_req[t])
                idx[t] = int(last_tokens[int(req_slots[b])]) if b >= 0 else 0
        e = table[idx][:, offset:offset + C].float()
        out.copy_((torch.nn.functional.gelu(s.float(), approximate="tanh") * e).to(out.dtype))

    def softcap_f32(self, x, cap):
        x.copy_(cap * torch.tanh(x / cap))

    # -- a 32-bit residual stream, matrix memory, routed experts -----------------------------
    def embed_scaled(self, ids, table, stream, copy=None, scale=1.0, inv_freq=None, positions=None, last_tokens=None,
                     token_req=None, req_slots=None):
        self._count("embedding")
        T, H = stream.shape
        idx = ids[:T].long().clone()
        if last_tokens is not None:
            for t in (idx < 0).nonzero().flatten().tolist():
                b = int(token_req[t])
                idx[t] = int(last_tokens[int(req_slots[b])]) if b >= 0 else 0
        v = table[idx].float() * scale
        if inv_freq is not None:
            ang = positions[:T].float()[:, None] * inv_freq[None, :]
            pe = torch.stack((torch.sin(ang), torch.cos(ang)), -1).reshape(T, -1)[:, :H]
            v = v + pe
        stream.copy_(v)
        if copy is not None:
            copy.copy_(v.to(copy.dtype))

    def norm_scale_add(self, a, stream, weight, eps, mult, copy=None, next_norm=None):
        self._count("add_rmsnorm")
        x = a.float()
        stream += mult * (x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps) * weight)
        if copy is not None:
            copy.copy_(stream.to(copy.dtype))
        if next_norm is not None:
            w2, eps2, out = next_norm
            out.copy_((stream / torch.sqrt(stream.pow(2).mean(-1, keepdim=True) + eps2) * w2).to(out.dtype))
            return True

    def rmsnorm_rows_f32(self, stream, rows, weight, eps, out):
        self._count("add_rmsnorm")
        s = stream[: out.shape[0]] if rows is None else stream[rows[: out.shape[0]].long()]
        out.copy_((s / torch.sqrt(s.pow(2).mean(-1, keepdim=True) + eps) * weight).to(out.dtype))

    def cast_rows_f32(self, src, out):
        out.copy_(src.to(out.dtype))

    def act_mul_clamped(self, gate_up, out, limit, alpha):
        self._count("act_mul")
        I = out.shape[1]
        g = gate_up[:, :I].float().clamp(max=limit)
        u = gate_up[:, I:].float().clamp(-limit, limit)
        out.copy_((g * torch.sigmoid(alpha * g) * (u + 1)).to(out.dtype))

    def mlstm_recurrence(self, qkv, q_off, k_off, v_off, gates, bias_i, bias_f, state, cu_q, req_slots, token_req, out,
                         requests, heads, dim, vdim, q_scale, cap):
        self._count("mlstm")
        x = qkv.float()
        for r in range(requests):
            t0, t1 = int(cu_q[r]), int(cu_q[r + 1])
            if t1 <= t0:
                continue
            if int(token_req[t0]) < 0:
                out[t0:t1] = 0
                continue
            row = state[int(req_slots[r])]
            S = row[: heads * vdim * dim].view(heads, vdim, dim)
            n = row[heads * vdim * dim: heads * vdim * dim + heads * dim].view(heads, dim)
            m = row[heads * vdim * dim + heads * dim: heads * vdim * dim + heads * dim + heads]
            for t in range(t0, t1):
                q = x[t, q_off:q_off + heads * dim].view(heads, dim) * q_scale
                k = x[t, k_off:k_off + heads * dim].view(heads, dim)
                v = x[t, v_off:v_off + heads * vdim].view(heads, vdim)
                ig = cap * torch.tanh((gates[t, :heads] + bias_i) / cap)
                fg = torch.nn.functional.logsigmoid(cap * torch.tanh((gates[t, heads:] + bias_f) / cap))
                m_new = torch.maximum(fg + m, ig)
                keep, take = torch.exp(fg + m - m_new), torch.exp(ig - m_new)
                S.mul_(keep[:, None, None]).add_(take[:, None, None] * v[:, :, None] * k[:, None, :])
                n.mul_(keep[:, None]).add_(take[:, None] * k)
                m.copy_(m_new)
                den = torch.maximum((n * q).sum(-1).abs(), torch.exp(-m)) + 1e-6
                out[t] = (torch.einsum("hvd,hd->hv", S, q) / den[:, None]).reshape(-1)

    def mlstm_out_gate(self, o, g, weight, eps, out, heads, vdim):
        T = o.shape[0]
        x = o.view(T, heads, vdim)
        x = (x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)).reshape(T, -1)
        out.copy_((x * weight * torch.sigmoid(g.float())).to(out.dtype))

    def moe_route(self, logits, choice, weight, top, softmax_scores=False, renormalize=False, correction=None,
                  experts=None):
        self._count("moe")
        if experts is not None:
            logits = logits[:, :experts]
        s = torch.softmax(logits, -1) if softmax_scores else torch.sigmoid(logits)
        c = torch.topk(s if correction is None else s + correction, top, dim=-1).indices
        w = torch.gather(s, 1, c)
        if renormalize:
            w = w / w.sum(-1, keepdim=True)
        choice.copy_(c.to(torch.int32))
        weight.copy_(w)

    def moe_arrange(self, choice, pairs, experts, offsets, sorted_pairs, place):
        c = choice.reshape(-1)[:pairs].long()
        order = torch.argsort(c, stable=True)  # (choices at or beyond `experts` come last and get no expert's rows)
        sorted_pairs.view(-1)[:pairs] = order.to(torch.int32)
        place.view(-1)[order] = torch.arange(pairs, dtype=torch.int32)
        counts = torch.bincount(c[c < experts], minlength=experts)
        offsets.view(-1)[0] = 0
        offsets.view(-1)[1:experts + 1] = torch.cumsum(counts, 0).to(torch.int32)

    def moe_grouped_linear(self, x, weights, offsets, sorted_pairs, pair_weight, out, top, rows_from_pairs, gated, act=0,
                           limit=0.0, alpha=1.0):
        self._count("moe")
        off = offsets.view(-1).tolist()
        sp = sorted_pairs.view(-1)
        pw = pair_weight.view(-1) if pair_weight is not None else None
        n_out = out.shape[1]
        for e in range(weights.shape[0]):
            for p in range(off[e], off[e + 1]):
                pair = int(sp[p])
                row = x[pair // top if rows_from_pairs else p].float()
                y = weights[e].float() @ row
                if pw is not None:
                    y = y * pw[pair]
                if gated:
                    g, u = y[:n_out], y[n_out:]
                    if act == 2:
                        g, u = g.clamp(max=limit), u.clamp(-limit, limit)
                        y = g * torch.sigmoid(alpha * g) * (u + 1)
                    else:
                        y = (g * torch.sigmoid(g) if act == 0 else torch.nn.functional.gelu(g, approximate="tanh")) * u
                out[p] = y.to(out.dtype)

    def moe_combine(self, rows, place, pair_weight, y, top, passing=None, shared=None):
        T = y.shape[0]
        pl = place.view(-1)[: T * top].long()
        v = rows[pl.clamp(0, rows.shape[0] - 1)].float()
        if passing is not None:
            choice, experts, x = passing
            passes = choice.view(-1)[: T * top] >= experts
            v = torch.where(passes[:, None], x.float().repeat_interleave(top, 0), v)
        if pair_weight is not None:
            v = v * pair_weight.view(-1)[: T * top, None]
        out = v.view(T, top, -1).sum(1)
        if shared is not None:
            s_rows, gate = shared
            out = out + s_rows.float() * (torch.sigmoid(gate[:, :1]) if gate is not None else 1.0)
        y.copy_(out.to(y.dtype))

    def argmax(self, logits, out):
        out[: logits.shape[0]] = torch.argmax(logits, -1).to(torch.int32)

    def sample(self, logits, temperature, top_k, top_p, min_p, uniform, out, probs_out=None, row_slots=None,
               last_tokens=None):
        import plain_model as pm

        for r in range(logits.shape[0]):
            t = float(temperature[r])
            if t <= 0:
                out[r] = int(torch.argmax(logits[r]))
            else:
                probs = pm.filtered_distribution(logits[r], t, int(top_k[r]), float(top_p[r]), float(min_p[r]))
                out[r] = pm.inverse_cdf_draw(probs, float(uniform[r]))
                if probs_out is not None:
                    probs_out[r] = probs
            if row_slots is not None and last_tokens is not None and int(row_slots[r]) >= 0:
                last_tokens[int(row_slots[r])] = out[r]
