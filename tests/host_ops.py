"""A stand-in for the kernel table, for tests of the host side only (engine loop, scheduler, sampler
plumbing, error handling) where no GPU is: the same calls as ``csrc/ops.py`` answered with slow torch
code on the CPU.  It is test material: nothing of the package imports it, and the package has no CPU
path of its own.  The math follows the plain implementation (plain_llama.py), read from the same step
metadata and pages that the kernels read.
"""
from __future__ import annotations

import torch

import plain_bumolix as PB
import plain_dosovik as PD
import plain_kulivik as PK
import plain_tutezen as PT
import plain_llama as P
from atoma_infer_b200.csrc.ops import (META_BT_OFFSET, META_BT_STRIDE, META_NUM_ROWS, META_NUM_TOKENS, STATUS_WORDS,
                                       CudaOps)


class HostOps:
    describe_status = staticmethod(CudaOps.describe_status)

    def __init__(self):
        self.device = torch.device("cpu")
        self.launches = 0
        self.status = torch.zeros(STATUS_WORDS, dtype=torch.int32)
        self.last_tokens = torch.zeros(1 << 10, dtype=torch.int32)
        self.fused_rope = False
        self.fail_at_launch = None  # (launch number, status word, value): raise a status word there, as a kernel would

    def _count(self):
        self.launches += 1
        if self.fail_at_launch and self.launches >= self.fail_at_launch[0]:
            _, word, value = self.fail_at_launch
            self.status[word] = value
            self.fail_at_launch = None

    def clear_status(self):
        self.status.zero_()

    def check_status(self):
        what = self.describe_status(self.status.tolist())
        if what:
            self.clear_status()
            raise RuntimeError("device status: " + what)

    def fast_attention(self, *a):
        return False

    def embed(self, tokens, table, resid, meta, T, scale=1.0):
        self._count()
        n = int(meta[META_NUM_TOKENS])
        tok = tokens[:n].long()
        neg = tok < 0
        tok = torch.where(neg, self.last_tokens[(-tok - 1).clamp(min=0)].long(), tok)
        resid[:n] = scale * table[tok].float()

    def add_rmsnorm(self, resid, delta, w, eps, out, meta, n, rows=None):
        self._count()
        if rows is None:
            n = int(meta[META_NUM_TOKENS])
            if delta is not None:
                resid[:n] += delta[:n].float()
            x = resid[:n]
        else:
            n = int(meta[META_NUM_ROWS])
            r = rows[:n].long()
            x = resid[r] + (delta[r].float() if delta is not None else 0)
        out[:n] = P.rms_norm(x, w, eps).to(out.dtype)

    def linear(self, x, w, *, out_dtype=None, silu_mul=False, meta=None, use_rows=False):
        self._count()
        y = x.float() @ w.float().T
        if silu_mul:
            inter = w.shape[0] // 2
            g, u = y[:, :inter], y[:, inter:]
            y = g * torch.sigmoid(g) * u
        return y.to(out_dtype or x.dtype)

    def rope_kv_store(self, qkv, positions, token_entry, meta, group, inv_freq, cache, num_pages, T, nq, nkv, d, rot,
                      page_size, store_kv):
        self._count()
        n = int(meta[META_NUM_TOKENS])
        off, stride = int(meta[META_BT_OFFSET + group]), int(meta[META_BT_STRIDE + group])
        rows = qkv[:n].view(n, nq + 2 * nkv, d).float()
        pos = positions[:n]
        qk = rows[:, :nq + nkv].clone()
        qk[..., :rot] = P.rope(qk[..., :rot], pos, inv_freq)
        qkv[:n].view(n, nq + 2 * nkv, d)[:, :nq] = qk[:, :nq].to(qkv.dtype)
        if store_kv:
            for t in range(n):
                p = int(pos[t])
                page = int(meta[off + int(token_entry[t]) * stride + p // page_size])
                if not 0 < page < num_pages:
                    self.status[1] = t + 1
                    continue
                cache[page, 0, :, p % page_size] = qk[t, nq:].to(cache.dtype)
                cache[page, 1, :, p % page_size] = rows[t, nq + nkv:].to(cache.dtype)

    # -- layers other than the plain pre-norm block (rings: the row of position p at place p mod (taps - 1))
    def _entries(self, ctx):
        n, S = int(ctx.meta[META_NUM_TOKENS]), int(ctx.meta[1])
        cu = [int(ctx.cu_tokens[k]) for k in range(S)] + [n]
        return [(k, cu[k], cu[k + 1], int(ctx.state_slots[k])) for k in range(S)]

    def short_conv(self, x, w, state, ctx, out, *, add_input=True):
        self._count()
        taps, w = w.shape[0], w.t()  # the kernels take [taps, channels]
        for _, a, b, slot in self._entries(ctx):
            p0 = int(ctx.positions[a])
            past = [state[slot, p % (taps - 1)] if p >= 0 else torch.zeros_like(x[0]) for p in range(p0 - taps + 1, p0)]
            rows = torch.stack(past + list(x[a:b])) if past else x[a:b]
            y = PD.short_conv(rows.float(), w.float())[len(past):]
            out[a:b] = ((x[a:b] + y) if add_input else y).to(out.dtype)

    def short_conv_save(self, x, state, ctx, taps):
        self._count()
        for _, a, b, slot in self._entries(ctx):
            for t in range(max(a, b - (taps - 1)), b):
                state[slot, int(ctx.positions[t]) % (taps - 1)] = x[t]

    def scaled_add_rmsnorm(self, resid, delta, alpha, w, eps, ctx, *, keep=None, conv=None):
        n = int(ctx.meta[META_NUM_TOKENS])
        if keep is not None and keep[0] is not None:
            self.short_conv_save(resid, keep[0], ctx, keep[1])
        self._count()
        v = alpha * resid[:n] + (delta[:n].float() if delta is not None else 0)
        resid[:n] = PD.rms_divide(v, eps) * w
        if conv is not None:
            self.short_conv(resid, conv[0], conv[1], ctx, conv[2], add_input=True)

    def qkv_prepare(self, qkv, ctx, cache, group, q_out, *, nq, nkv, d, dv, dp, page_size, num_pages, store_kv, bias=None,
                    q_norm=None, k_norm=None, eps=0.0, inv_freq=None, rot=0, v_first=None, v_lambda=None, v_out=None,
                    head_norm=False, interleaved=False, q_temp=None):
        self._count()
        meta = ctx.meta
        n = int(meta[META_NUM_TOKENS])
        off, stride = int(meta[META_BT_OFFSET + group]), int(meta[META_BT_STRIDE + group])
        NQ, NK = nq * d, nkv * d
        bias, q_norm, k_norm = (t.float() if t is not None else None for t in (bias, q_norm, k_norm))
        rows = qkv[:n].float() + (bias if bias is not None else 0)
        q, k, v = rows[:, :NQ], rows[:, NQ:NQ + NK], rows[:, NQ + NK:]
        if q_norm is not None and not head_norm:
            q = PD.rms_divide(q, eps) * q_norm
        if k_norm is not None and not head_norm:
            k = PD.rms_divide(k, eps) * k_norm
        q, k = q.reshape(n, nq, d).clone(), k.reshape(n, nkv, d).clone()
        weighted = head_norm and q_norm is not None
        if weighted:  # the norm per head with a shared weight comes before the rotation
            q, k = PB.rms_divide(q, eps) * q_norm, PB.rms_divide(k, eps) * k_norm
        if inv_freq is not None and rot:
            pos = ctx.positions[:n]
            if interleaved:
                ang = pos.double()[:, None, None] * inv_freq.double()
                for x in (q, k):
                    a, b = x[..., 0:rot:2].double(), x[..., 1:rot:2].double()
                    x[..., 0:rot:2] = (a * torch.cos(ang) - b * torch.sin(ang)).float()
                    x[..., 1:rot:2] = (b * torch.cos(ang) + a * torch.sin(ang)).float()
            else:
                q[..., :rot] = P.rope(q[..., :rot], pos, inv_freq)
                k[..., :rot] = P.rope(k[..., :rot], pos, inv_freq)
        if head_norm and not weighted:
            q, k = PB.rms_divide(q, eps), PB.rms_divide(k, eps)
        if q_temp:
            p = ctx.positions[:n].double()
            q = q * (1.0 + q_temp[0] * torch.log(torch.floor((p + 1) / q_temp[1]) + 1.0)).float()[:, None, None]
        if v_out is not None:
            v_out[:n] = v.to(v_out.dtype)
        if v_first is not None:
            v = (1 - v_lambda) * v + v_lambda * v_first[:n].float()
        q_out[:n] = 0
        q_out[:n].view(n, nq, dp)[..., :d] = q.to(q_out.dtype)
        if store_kv:
            for t in range(n):
                p = int(ctx.positions[t])
                page = int(meta[off + int(ctx.token_entry[t]) * stride + p // page_size])
                if not 0 < page < num_pages:
                    self.status[1] = t + 1
                    continue
                cache[page, :, :, p % page_size] = 0
                cache[page, 0, :, p % page_size, :d] = k[t].to(cache.dtype)
                cache[page, 1, :, p % page_size, :dv] = v[t].reshape(nkv, dv).to(cache.dtype)

    def narrow(self, x, dtype):
        self._count()
        return x.to(dtype)

    def polynorm(self, z, coef, eps, out, meta):
        self._count()
        n = int(meta[META_NUM_TOKENS])
        out[:n] = PD.poly_norm(z[:n].float(), coef, eps).to(out.dtype)

    def attention(self, q, q_stride, cache, ctx, group, out, nq, nkv, d, page_size, num_pages, window, scale, rope=None,
                  chunk=0, sink=False, keep_first=0, softcap=0.0, slopes=None):
        self._count()
        meta = ctx.meta
        n = int(meta[META_NUM_TOKENS])
        off, stride = int(meta[META_BT_OFFSET + group]), int(meta[META_BT_STRIDE + group])
        for t in range(n):
            pos, e = int(ctx.positions[t]), int(ctx.token_entry[t])
            first = max(0, pos - window + 1) if window else 0
            if chunk:
                first = max(first, pos - pos % chunk)
            idx = list(range(min(keep_first, first) if window else 0)) + list(range(first, pos + 1)) if keep_first else range(first, pos + 1)
            dist = torch.tensor([float(pos - j) for j in idx])
            pages = [int(meta[off + e * stride + j // page_size]) for j in idx]
            k = torch.stack([cache[p, 0, :, j % page_size] for p, j in zip(pages, idx)]).float()  # [keys, nkv, d]
            v = torch.stack([cache[p, 1, :, j % page_size] for p, j in zip(pages, idx)]).float()
            qq = q[t].view(-1, d)[:nq].float()
            g = nq // nkv
            for h in range(nq):
                sc = (k[:, h // g] @ qq[h]) * scale
                if softcap:
                    sc = softcap * torch.tanh(sc / softcap)
                if slopes is not None:
                    sc = sc - slopes[h] * dist
                if torch.is_tensor(sink):  # a learned sink per head: exp(sink_h) in the denominator
                    w = torch.softmax(torch.cat([sc, sink[h].float().reshape(1)]), 0)[:-1]
                else:
                    w = torch.softmax(torch.cat([sc, sc.new_zeros(1)]), 0)[:-1] if sink else torch.softmax(sc, 0)
                out[t, h * d:(h + 1) * d] = (w @ v[:, h // g]).to(out.dtype)

    # -- parallel blocks, state-space mixers, latent attention, routed experts
    def sum_rmsnorm(self, resid, pending, w, eps, out, meta, n, rows=None, second=None):
        self._count()
        if rows is None:
            n = int(meta[META_NUM_TOKENS])
            idx = torch.arange(n)
        else:
            n = int(meta[META_NUM_ROWS])
            idx = rows[:n].long()
        x = resid[idx]
        if pending is not None:
            add = torch.zeros_like(x)
            for t, f in zip(pending.terms, pending.weights()):
                add = add + f * t[idx].float()
            x = x + pending.mult * add
            if pending.rows is not None:
                x = x + pending.rows[idx]
            if pending.vector is not None:
                x = x + pending.vector
        if rows is None:
            resid[:n] = x
        if out is not None:
            out[:n] = P.rms_norm(x, w, eps).to(out.dtype)
        if second is not None:
            second[2][:n] = P.rms_norm(x, second[0], second[1]).to(second[2].dtype)

    def sigmoid_gate(self, y, gate, meta):
        self._count()
        n = int(meta[META_NUM_TOKENS])
        y[:n] = (y[:n].float() * torch.sigmoid(gate[:n].float())).to(y.dtype)

    def gla_scan(self, q, k, v, z, z_bias, tau, q_scale, state, ctx, o, *, heads, dim, vdim, head_decay=None, silu=False):
        self._count()
        act = PK.silu if silu else (lambda x: x)
        for _, a, b, slot in self._entries(ctx):
            for t in range(a, b):
                qt, kt = act(q[t].float()).view(heads, dim) * q_scale, act(k[t].float()).view(heads, dim)
                vt = act(v[t].float()).view(heads, vdim)
                if head_decay is not None:
                    decay = head_decay[:, None].expand(heads, dim)
                else:
                    decay = torch.exp(torch.nn.functional.logsigmoid(z[t] + z_bias) / tau).view(heads, dim)  # no underflow below the power
                for h in range(heads):
                    S = decay[h][:, None] * state[slot, h] + torch.outer(kt[h], vt[h])
                    state[slot, h] = S
                    o[t, h * vdim:(h + 1) * vdim] = S.T @ qt[h]

    def head_norm_gate(self, o, gate, w, eps, out, meta, heads):
        self._count()
        n = int(meta[META_NUM_TOKENS])
        y = PB.rms_divide(o[:n].view(n, heads, -1), eps) * w
        out[:n] = (y.reshape(n, -1) * PB.silu(gate[:n].float())).to(out.dtype)

    def selective_scan(self, u, dt_raw, dt_bias, bc, zg, a_log, d_skip, state, ctx, out, *, inner, nstate):
        self._count()
        A = -torch.exp(a_log)
        for _, a, b, slot in self._entries(ctx):
            for t in range(a, b):
                ut, dt = u[t].float(), PB.softplus(dt_raw[t] + dt_bias)
                B, C = bc[t, :nstate].float(), bc[t, nstate:].float()
                S = torch.exp(dt[:, None] * A) * state[slot] + (dt * ut)[:, None] * B[None, :]
                state[slot] = S
                out[t] = ((S @ C + d_skip * ut) * PB.silu(zg[t].float())).to(out.dtype)

    def causal_conv_act(self, u, w, bias, state, ctx, out, *, act="silu"):
        self._count()
        taps, wt = w.shape[0], w.t()  # the kernels take [taps, channels]
        for _, a, b, slot in self._entries(ctx):
            p0 = int(ctx.positions[a])
            past = [state[slot, p % (taps - 1)] if p >= 0 else torch.zeros_like(state[slot, 0]) for p in range(p0 - taps + 1, p0)]
            rows = torch.cat([torch.stack(past), u[a:b].float()]) if past else u[a:b].float()
            y = PT.causal_conv(rows, wt.float(), bias if bias is not None else torch.zeros(wt.shape[0]))[len(past):]
            out[a:b] = (PT.silu(y) if act == "silu" else y).to(out.dtype)
        return taps == 1  # the state is left to causal_conv_save

    def causal_conv_save(self, u, state, ctx, taps):
        self._count()
        for _, a, b, slot in self._entries(ctx):
            for t in range(max(a, b - (taps - 1)), b):
                state[slot, int(ctx.positions[t]) % (taps - 1)] = u[t].float()

    def ssm_scan(self, xbc, dt, dt_bias, a_log, d_skip, state, ctx, y, *, heads, head_dim, nstate, groups):
        self._count()
        inner, per = heads * head_dim, heads // groups
        for _, a, b, slot in self._entries(ctx):
            for t in range(a, b):
                row = xbc[t].float()
                x = row[:inner].view(heads, head_dim)
                B = row[inner:inner + groups * nstate].view(groups, nstate)
                C = row[inner + groups * nstate:].view(groups, nstate)
                step = PT.softplus(dt[t].float() + dt_bias)
                for h in range(heads):
                    S = torch.exp(-torch.exp(a_log[h]) * step[h]) * state[slot, h] + step[h] * torch.outer(B[h // per], x[h])
                    state[slot, h] = S
                    y[t, h * head_dim:(h + 1) * head_dim] = S.T @ C[h // per] + d_skip[h] * x[h]

    def gated_group_norm(self, y, z, w, groups, eps, out, meta):
        self._count()
        n = int(meta[META_NUM_TOKENS])
        out[:n] = (PT.grouped_rms(y[:n] * PT.silu(z[:n].float()), groups, eps) * w).to(out.dtype)

    def rms_rows(self, x, w, eps, out, meta):
        self._count()
        n = int(meta[META_NUM_TOKENS])
        out[:n] = (PT.rms_divide(x[:n].float(), eps) * w).to(out.dtype)

    def head_linear(self, x, w, out, meta, gate=None):
        self._count()
        n = int(meta[META_NUM_TOKENS])
        y = torch.einsum("thk,hnk->thn", x[:n].float(), w.float())
        if gate is not None:
            y = y * torch.sigmoid(gate[:n].float())
        out[:n] = y.to(out.dtype)

    def latent_rows(self, q_rot, q_abs, dkv, norm_w, eps, ctx, cache, group, q_out, *, heads, kv_rank, rot_dim, padded,
                    page_size, num_pages, store, inv_freq=None, rotary_dims=0):
        self._count()
        meta = ctx.meta
        n = int(meta[META_NUM_TOKENS])
        off, stride = int(meta[META_BT_OFFSET + group]), int(meta[META_BT_STRIDE + group])
        pos = ctx.positions[:n]

        def turn(v):  # pairs (2i, 2i+1) of the first rotary_dims dimensions
            if not rotary_dims:
                return v
            ang = pos.float()[:, None] * inv_freq
            while ang.dim() < v.dim():
                ang = ang.unsqueeze(1)
            cs, sn = torch.cos(ang), torch.sin(ang)
            o = v.clone()
            a, b = v[..., 0:rotary_dims:2], v[..., 1:rotary_dims:2]
            o[..., 0:rotary_dims:2] = a * cs - b * sn
            o[..., 1:rotary_dims:2] = b * cs + a * sn
            return o

        c = PT.rms_divide(dkv[:n, :kv_rank].float(), eps) * norm_w
        key = torch.cat([c, turn(dkv[:n, kv_rank:].float())], -1)
        q_out[:n] = 0
        qv = q_out[:n].view(n, heads, padded)
        qv[..., :kv_rank] = q_abs[:n].to(q_out.dtype)
        qv[..., kv_rank:kv_rank + rot_dim] = turn(q_rot[:n].float()).to(q_out.dtype)
        if store:
            for t in range(n):
                p = int(pos[t])
                page = int(meta[off + int(ctx.token_entry[t]) * stride + p // page_size])
                if not 0 < page < num_pages:
                    self.status[1] = t + 1
                    continue
                cache[page, :, 0, p % page_size] = 0
                cache[page, :, 0, p % page_size, :kv_rank + rot_dim] = key[t].to(cache.dtype)

    def activation(self, z, out, kind, meta):
        self._count()
        n = int(meta[META_NUM_TOKENS])
        out[:n] = {"gelu_tanh": PT.gelu_tanh, "relu2": PB.relu_squared}[kind](z[:n].float()).to(out.dtype)

    def moe_route(self, h, w_router, ids, wts, meta, bias=None, over_chosen=False):
        self._count()
        n = int(meta[META_NUM_TOKENS])
        if bias is not None or over_chosen:
            z = h[:n].float() @ w_router.T + (bias if bias is not None else 0)
            if over_chosen:
                idx, wt = PK.route(z, ids.shape[1])
            else:
                sc = torch.softmax(z, -1)
                wt, idx = torch.topk(sc, ids.shape[1], dim=-1)
                wt = wt / wt.sum(-1, keepdim=True)
            ids[:n], wts[:n] = idx.to(torch.int32), wt.float()
            return
        idx, wt = PT.route(h[:n].float(), w_router, ids.shape[1])
        ids[:n], wts[:n] = idx.to(torch.int32), wt

    def moe_experts(self, h, ids, wts, w_gate_up, w_down, shared, out, meta):
        self._count()
        n = int(meta[META_NUM_TOKENS])
        f = w_gate_up.shape[1] // 2
        for t in range(n):
            acc = torch.zeros(w_down.shape[1])
            for k in range(ids.shape[1]):
                e = int(ids[t, k])
                gu = w_gate_up[e].float() @ h[t].float()
                act = (PT.silu(gu[:f]) * gu[f:]).to(h.dtype).float()
                acc = acc + wts[t, k] * (w_down[e].float() @ act)
            if shared is not None:
                acc = acc + shared[t].float()
            out[t] = acc.to(out.dtype)

    # -- blocks that norm and gate a sublayer's result, with the mixer's input shifted toward the token before
    def norm_shift(self, resid, w, eps, ctx, *, shift=None, state=None, h=None, hs=None, last=None):
        self._count()
        for k, a, b, slot in self._entries(ctx):
            if a == b:
                continue
            hv = P.rms_norm(resid[a:b], w, eps).float()
            if h is not None:
                h[a:b] = hv.to(h.dtype)
            if last is not None:
                last[k] = hv[-1]
            if hs is not None:
                if shift is None:
                    hs[a:b] = hv.to(hs.dtype)
                    continue
                first = state[slot].clone() if (state is not None and int(ctx.positions[a]) > 0) else torch.zeros_like(hv[0])
                before = torch.cat([first[None], hv[:-1]], 0)
                hs[a:b] = (hv + (before - hv) * shift).to(hs.dtype)

    def gated_norm_add(self, resid, pending, gate, gate_bias, w, eps, ctx, *, next_norm=None, keep=None):
        self._count()
        n = int(ctx.meta[META_NUM_TOKENS])
        y = torch.zeros_like(resid[:n])
        for t, f in zip(pending.terms, pending.weights()):
            y = y + f * t[:n].float()
        y = y * pending.mult
        if pending.vector is not None:
            y = y + pending.vector
        y = y * torch.sigmoid(gate[:n].float() + (gate_bias if gate_bias is not None else 0))
        resid[:n] += P.rms_norm(y, w, eps).float()
        if next_norm is not None:
            next_norm[2][:n] = P.rms_norm(resid[:n], next_norm[0], next_norm[1]).to(next_norm[2].dtype)
        if keep is not None:
            for k, a, b, slot in self._entries(ctx):
                if b > a:
                    keep[1][slot] = keep[0][k]

    def clamped_glu(self, gu, out, limit, alpha, meta):
        self._count()
        n, f = int(meta[META_NUM_TOKENS]), out.shape[1]
        g = gu[:n, :f].float().clamp(max=limit)
        u = gu[:n, f:].float().clamp(-limit, limit)
        out[:n] = (g * torch.sigmoid(alpha * g) * (u + 1.0)).to(out.dtype)

    def head_gate(self, y, gate, meta):
        self._count()
        n = int(meta[META_NUM_TOKENS])
        y[:n] = (y[:n].float() * torch.sigmoid(gate[:n].float())[:, :, None]).to(y.dtype)

    def row_norm_gate(self, o, gate, w, eps, out, meta, kind="sigmoid"):
        self._count()
        n = int(meta[META_NUM_TOKENS])
        g = gate[:n].float()
        out[:n] = (PB.rms_divide(o[:n], eps) * w * (torch.sigmoid(g) if kind == "sigmoid" else PB.silu(g))).to(out.dtype)

    def scale_softcap(self, logits, scale, cap, meta):
        self._count()
        n = int(meta[META_NUM_ROWS])
        z = logits[:n] * scale
        logits[:n] = cap * torch.tanh(z / cap) if cap else z

    def sample(self, logits, temperature, top_k, top_p, seed, step, out, num_rows=None, slots=None):
        self._count()
        import numpy as np

        seeds = seed.numpy().view(np.uint64)
        steps = step.numpy().view(np.uint64)
        for r in range(logits.shape[0]):
            t = float(temperature[r])
            if t == 0.0:
                tok = P.greedy(logits[r])
            else:
                tok = P.sample(logits[r], temperature=t, seed=int(seeds[r]), step=int(steps[r]), top_k=int(top_k[r]),
                               top_p=float(top_p[r]))
            out[r] = tok
            if slots is not None:
                self.last_tokens[int(slots[r])] = tok

    def repeat_penalty(self, row, penalty, context):
        self._count()
        row.copy_(P.apply_repeat_penalty(row, penalty, context.tolist()))
