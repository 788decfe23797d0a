"""Plain PyTorch twins of the CUDA kernels, one function per kernel, with the same call
signature as ``turingserve_b200.kernels.CudaOps``.

Two uses: (1) the ``-m gpu`` tests compare each kernel alone with its twin; (2) the CPU tests
install ``TwinOps()`` behind ``kernels.ops()`` to drive the engine's HOST logic (cache manager,
batch builder, step function, scheduler, replay) without a GPU.  The product never uses this file.

Formulas: turingserve/ops/reference.py (rmsnorm :13-23, silu_mul :26-28, rope :31-42,
linear :45-47, kv_write :50-57, attention :60-77,94-111), sampling as
turingserve/sampling/sampler.py:45-107.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F

from tests import plain_qwen2 as plain


class TwinOps:
    def embedding(self, out, table, ids):
        out.copy_(table[ids.long()])

    def gather_rows(self, out, x, rows):
        out.copy_(x[rows.long()])

    def rmsnorm(self, out, x, weight, eps, residual=None):
        if residual is not None:
            residual.copy_(x + residual)
            x = residual
        x32 = x.float()
        y = (x32 * torch.rsqrt(x32.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype)
        out.copy_((weight.float() * y.float()).to(x.dtype))

    def silu_mul(self, out, gu, group=0):
        i = gu.shape[-1] // 2
        if group:
            blocks = gu.reshape(gu.shape[0], i // group, 2, group)
            g, u = blocks[:, :, 0].reshape(-1, i), blocks[:, :, 1].reshape(-1, i)
        else:
            g, u = gu[..., :i], gu[..., i:]
        out.copy_(F.silu(g) * u)

    def gated_linear(self, out, x, w, bias, group):
        gu = torch.empty((x.shape[0], w.shape[0]), dtype=x.dtype)
        self.linear(gu, x, w, bias)
        self.silu_mul(out, gu, group)

    def qkv_rope(self, out, x, w, bias, positions, cos, sin, H, KVH, D, rotary_dim, k_cache, v_cache, slots,
                 page_size):
        self.linear(out, x, w, bias)
        return self.rope_kv_write(out, positions, cos, sin, H, KVH, D, rotary_dim, k_cache, v_cache, slots, page_size)

    def rope_kv_write(self, qkv, positions, cos, sin, H, KVH, D, rotary_dim, k_cache, v_cache, slots,
                      page_size):
        T = qkv.shape[0]
        pos = positions.long()
        qk = qkv[:, : (H + KVH) * D].view(T, H + KVH, D)
        if rotary_dim:
            half = rotary_dim // 2
            c = cos[pos].to(qkv.dtype).float()[:, None, :]
            s = sin[pos].to(qkv.dtype).float()[:, None, :]
            x1, x2 = qk[..., :half].float(), qk[..., half:rotary_dim].float()
            o1, o2 = x1 * c - x2 * s, x2 * c + x1 * s
            qk[..., :half] = o1.to(qkv.dtype)
            qk[..., half:rotary_dim] = o2.to(qkv.dtype)
        if k_cache is None:
            return qkv
        k = qkv[:, H * D:(H + KVH) * D].view(T, KVH, D)
        v = qkv[:, (H + KVH) * D:].view(T, KVH, D)
        m = slots >= 0
        sl = slots[m].long()
        k_cache[sl // page_size, :, sl % page_size, :] = k[m]
        v_cache[sl // page_size, :, sl % page_size, :] = v[m]
        return qkv

    def attention(self, out, qkv, k_cache, v_cache, block_tables, step, H, KVH, D, page_size, scale,
                  window):
        paged_attention(out, qkv, k_cache, v_cache, block_tables, step.q_start, step.seq_lens,
                        H, KVH, D, page_size, scale, window)

    def linear(self, out, x, w, bias=None, rows=None, may_defer=False, lazy=True):
        if rows is not None:
            x = x[rows.long()]
        y = F.linear(x.float(), w.float(), None if bias is None else bias.float())
        out.copy_(y.to(out.dtype))
        return out

    def materialize(self, x):
        return x

    def sample(self, out, logits, fparams, iparams):
        S = logits.shape[0]
        for r in range(S):
            row = logits[r].float().cpu()
            if not torch.isfinite(row).all():
                out[0, r], out[1, r] = 0, 1
                continue
            tok, _ = plain.sample(row, float(fparams[r, 0]), int(iparams[r, 0]), float(fparams[r, 1]),
                                  int(iparams[r, 1]), int(iparams[r, 2]))
            out[0, r], out[1, r] = tok, 0

    def penalize(self, logits, ids, meta, pen):
        ids = ids.tolist()
        for r in range(logits.shape[0]):
            a, b, c, d = (int(x) for x in meta[r, :4])
            if c > a:
                logits[r] = plain.penalize(logits[r].cpu(), ids[a:b], ids[b:c], float(pen[r, 0]),
                                           float(pen[r, 1]), float(pen[r, 2])).to(logits.device)
            for t in ids[c:d]:
                logits[r, t] = float("-inf")

    # -- the kernels of the stream norm, the linear-attention mixer, the two-map attention and the routed
    # feed-forward (formulas restated from the kernels' own headers) ------------------------------------------
    def rmsnorm_stream(self, out, stream, add1, add2, weight, eps, first=False, alpha=1.0, row=None, norm_bias=None):
        total = torch.zeros_like(stream) if first else stream.clone()
        for a in (add1, add2):
            if a is not None:
                total = total + alpha * a.float()
        if row is not None:
            total = total + row.float()
        stream.copy_(total)
        if out is None:
            return
        if norm_bias is not None:
            dev = total - total.mean(-1, keepdim=True)
            y = dev / torch.sqrt(dev.pow(2).mean(-1, keepdim=True) + eps) * weight.float() + norm_bias.float()
        else:
            y = total / torch.sqrt(total.pow(2).mean(-1, keepdim=True) + eps) * weight.float()
        out.copy_(y.to(out.dtype))

    def gated_rmsnorm(self, out, x, gate, weight, eps):
        y = x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps) * weight.float()
        out.copy_((y * torch.sigmoid(gate.float())).to(out.dtype))

    def activation(self, out, x, kind):
        z = x.float()
        if kind == "gelu_tanh":
            y = 0.5 * z * (1.0 + torch.tanh(0.7978845608028654 * (z + 0.044715 * z ** 3)))
        elif kind == "relu2":
            y = torch.relu(z) ** 2
        elif kind == "gelu":
            y = 0.5 * z * (1.0 + torch.erf(z * 0.7071067811865476))
        else:
            y = F.silu(z)
        out.copy_(y.to(out.dtype))

    def lightning(self, out, proj, state, decay, step, H, D, V):
        qs = step.q_start.tolist()
        slots = step.state_slots.tolist()
        act = lambda t: F.silu(t.float()).to(proj.dtype).float()
        q = act(proj[:, : H * D]).view(-1, H, D)
        k = act(proj[:, H * D: 2 * H * D]).view(-1, H, D)
        v = act(proj[:, 2 * H * D: 2 * H * D + H * V]).view(-1, H, V)
        for b in range(step.num_requests):
            S = state[slots[b]]
            for t in range(qs[b], qs[b + 1]):
                S.mul_(decay[:, None, None]).add_(k[t, :, :, None] * v[t, :, None, :])
                out[t] = torch.einsum("hdv,hd->hv", S, q[t]).reshape(-1)

    def kv_write_pair(self, proj, k_off, v_off, k_cache, v_cache, slots, KVH, DK, DV, page_size):
        m = slots >= 0
        sl = slots[m].long()
        k_cache[sl // page_size, :, sl % page_size, :] = proj[m, k_off:k_off + KVH * DK].view(-1, KVH, DK)
        v_cache[sl // page_size, :, sl % page_size, :] = proj[m, v_off:v_off + KVH * DV].view(-1, KVH, DV)

    def attention_diff(self, out, proj, k_cache, v_cache, block_tables, step, H, KVH, D, V, page_size, scale, lam,
                       eps, out_scale):
        qsl = step.q_start.tolist()
        G = H // KVH
        out.zero_()
        for b, seq_len in enumerate(step.seq_lens.tolist()):
            qs, qe = qsl[b], qsl[b + 1]
            if seq_len == 0 or qe == qs:
                continue
            Tq = qe - qs
            nb = -(-seq_len // page_size)
            blocks = block_tables[b, :nb].long()
            kk = k_cache[blocks].permute(0, 2, 1, 3).reshape(nb * page_size, KVH, 2, D)[:seq_len].float()
            vv = v_cache[blocks].permute(0, 2, 1, 3).reshape(nb * page_size, KVH, V)[:seq_len].float()
            q = proj[qs:qe, : H * 2 * D].view(Tq, H, 2, D).float()
            i = torch.arange(Tq)[:, None] + (seq_len - Tq)
            ok = torch.arange(seq_len)[None, :] <= i
            for h in range(H):
                maps = []
                for c in range(2):
                    s = (q[:, h, c] @ kk[:, h // G, c].t()) * scale
                    maps.append(torch.softmax(s.masked_fill(~ok, float("-inf")), -1) @ vv[:, h // G])
                o = maps[0] - lam * maps[1]
                o = o / torch.sqrt(o.pow(2).mean(-1, keepdim=True) + eps) * out_scale
                out[qs:qe, h * V:(h + 1) * V] = o.to(out.dtype)

    def router_topk(self, idx, weights, x, w_router, softmax, renormalize, correction=None):
        z = F.linear(x.float(), w_router.float())
        scores = torch.softmax(z, -1) if softmax else torch.sigmoid(z)
        best = (z if correction is None else scores + correction.float()).topk(idx.shape[1], dim=-1)
        idx.copy_(best.indices.to(torch.int32))
        w = scores.gather(1, best.indices)
        weights.copy_(w / w.sum(-1, keepdim=True) if renormalize else w)

    def moe_align(self, idx, E, with_tiles=None):
        flat = idx.reshape(-1).long()
        order = torch.sort(flat, stable=True).indices.to(torch.int32)
        place = torch.empty_like(order)
        place[order.long()] = torch.arange(order.numel(), dtype=torch.int32)
        counts = torch.bincount(flat, minlength=E)
        offsets = torch.cat([torch.zeros(1, dtype=torch.long), counts.cumsum(0)]).to(torch.int32)
        return offsets, order, place, None

    def grouped_linear(self, out, x, w, order, row_scale, offsets, tiles, top, act="none"):
        off = offsets.tolist()
        for e in range(w.shape[0]):
            a, b = off[e], off[e + 1]
            if a == b:
                continue
            if order is None:
                rows = x[a:b].float()
            else:
                pairs = order[a:b].long()
                rows = x[pairs // top].float()
                if row_scale is not None:
                    rows = (rows * row_scale.reshape(-1)[pairs][:, None]).to(x.dtype).float()
            y = F.linear(rows, w[e].float())
            tmp = torch.empty_like(y)
            if act == "none":
                tmp = y
            else:
                self.activation(tmp, y, act)
            out[a:b] = tmp.to(out.dtype)

    def moe_gather(self, xs, x, order, row_scale, top):
        pairs = order[: xs.shape[0]].long()
        rows = x[pairs // top].float()
        if row_scale is not None:
            rows = rows * row_scale.reshape(-1)[pairs][:, None]
        xs.copy_(rows.to(xs.dtype))

    def moe_combine(self, out, y, place, pair_weights, top, x=None, pass_from=None, add=None):
        rows = y[place.long()].view(out.shape[0], top, -1)
        if x is not None:
            own = (place.long() >= int(pass_from)).view(out.shape[0], top, 1)
            rows = torch.where(own, x.float()[:, None, :], rows)
        if pair_weights is not None:
            rows = rows * pair_weights.view(out.shape[0], top, 1)
        acc = torch.zeros(out.shape, dtype=torch.float32)
        for r in range(top):
            acc += rows[:, r]
        if add is not None:
            acc += add.float()
        out.copy_(acc.to(out.dtype))


def paged_attention(out, qkv, k_cache, v_cache, block_tables, q_start, seq_lens, H, KVH, D, page_size,
                    scale, window):
    """Attention from the paged cache for a flat batch (turingserve/ops/reference.py:94-111 with the
    bottom-right mask of :60-77, plus the window)."""
    qsl = q_start.tolist()
    G = H // KVH
    out.zero_()
    for b, seq_len in enumerate(seq_lens.tolist()):
        qs, qe = qsl[b], qsl[b + 1]
        if seq_len == 0 or qe == qs:
            continue
        Tq = qe - qs
        nb = -(-seq_len // page_size)
        blocks = block_tables[b, :nb].long()
        kk = k_cache[blocks].permute(0, 2, 1, 3).reshape(nb * page_size, KVH, D)[:seq_len].float()
        vv = v_cache[blocks].permute(0, 2, 1, 3).reshape(nb * page_size, KVH, D)[:seq_len].float()
        q = qkv[qs:qe, : H * D].view(Tq, H, D).float().permute(1, 0, 2)
        kf = kk.repeat_interleave(G, dim=1).permute(1, 0, 2)
        vf = vv.repeat_interleave(G, dim=1).permute(1, 0, 2)
        scores = torch.matmul(q, kf.transpose(1, 2)) * scale
        i = torch.arange(Tq, device=qkv.device)[:, None] + (seq_len - Tq)
        j = torch.arange(seq_len, device=qkv.device)[None, :]
        ok = j <= i
        if window:
            ok = ok & (j > i - window)
        scores = scores.masked_fill(~ok, float("-inf"))
        p = torch.softmax(scores, dim=-1)
        # keys of pages a window gave back may hold anything: they carry zero weight, keep them out
        vf = torch.where(ok.any(0)[None, :, None], vf, torch.zeros_like(vf))
        o = torch.matmul(p, vf).permute(1, 0, 2).reshape(Tq, H * D)
        out[qs:qe] = o.to(out.dtype)


# ------------------------------------------------------------------------------------------------------------
# Twins of the kernels of the delta rule, the biased attention and the latent attention.  They are methods of
# TwinOps (attached below) and follow the kernels' call signatures.

def _delta_prepare(self, ready, proj, conv_w, a_log, dt_bias, state, step, H, G, D, V, taps, unit_eps):
    qk, hv = G * D, H * V
    C = 2 * qk + hv
    tail0 = H * D * V
    qs = step.q_start.tolist()
    for b, slot in enumerate(step.state_slots.tolist()):
        a, e = qs[b], qs[b + 1]
        if e == a:
            continue
        tail = state[slot, tail0:tail0 + (taps - 1) * C].view(taps - 1, C)
        x = torch.cat([tail, proj[a:e, :C].float()], 0)
        n = e - a
        y = torch.zeros(n, C)
        for u in range(taps):
            y += x[u:u + n] * conv_w[:, u]
        y = F.silu(y)
        q = y[:, :qk].view(n, G, D)
        k = y[:, qk:2 * qk].view(n, G, D)
        q = q / torch.sqrt(q.pow(2).sum(-1, keepdim=True) + unit_eps) * D ** -0.5
        k = k / torch.sqrt(k.pow(2).sum(-1, keepdim=True) + unit_eps)
        bb = proj[a:e, C + hv:C + hv + H].float()
        aa = proj[a:e, C + hv + H:C + hv + 2 * H].float()
        ready[a:e, :qk] = q.reshape(n, qk)
        ready[a:e, qk:2 * qk] = k.reshape(n, qk)
        ready[a:e, 2 * qk:C] = y[:, 2 * qk:]
        ready[a:e, C:C + H] = torch.exp(-torch.exp(a_log) * F.softplus(aa + dt_bias))
        ready[a:e, C + H:C + 2 * H] = torch.sigmoid(bb)
        ready[a:e, C + 2 * H:] = (q * k).sum(-1)


def _delta_scan(self, out, ready, proj, state, step, H, G, D, V, taps):
    qk, hv = G * D, H * V
    C = 2 * qk + hv
    tail0 = H * D * V
    qs = step.q_start.tolist()
    per = H // G
    for b, slot in enumerate(step.state_slots.tolist()):
        a, e = qs[b], qs[b + 1]
        if e == a:
            continue
        S = state[slot, :tail0].view(H, D, V)
        for t in range(a, e):
            q = ready[t, :qk].view(G, D).repeat_interleave(per, 0)
            k = ready[t, qk:2 * qk].view(G, D).repeat_interleave(per, 0)
            v = ready[t, 2 * qk:C].view(H, V)
            g, beta = ready[t, C:C + H], ready[t, C + H:C + 2 * H]
            S.mul_(g[:, None, None])
            u = beta[:, None] * (v - torch.einsum("hdv,hd->hv", S, k))
            S.add_(k[:, :, None] * u[:, None, :])
            out[t] = torch.einsum("hdv,hd->hv", S, q).reshape(-1)
        if taps > 1:
            tail = state[slot, tail0:tail0 + (taps - 1) * C].view(taps - 1, C)
            tail.copy_(torch.cat([tail, proj[a:e, :C].float()], 0)[-(taps - 1):].clone())


def _head_gated_rmsnorm(self, out, x, gate, weight, eps, H, V):
    T = x.shape[0]
    o = x.float().view(T, H, V)
    o = o / torch.sqrt(o.pow(2).mean(-1, keepdim=True) + eps) * weight.float() * F.silu(gate.float()).view(T, H, V)
    out.copy_(o.reshape(T, H * V).to(out.dtype))


def _rms_rows(self, out, x, col0, weight, eps):
    n = out.shape[1]
    r = x[:, col0:col0 + n].float()
    out.copy_((r / torch.sqrt(r.pow(2).mean(-1, keepdim=True) + eps) * weight.float()).to(out.dtype))


def _qk_rownorm_write(self, proj, q_w, k_w, eps, positions, coef, every, k_cache, v_cache, slots, H, G, D, page_size):
    hd, gd = H * D, G * D
    q, k = proj[:, :hd].float(), proj[:, hd:hd + gd].float()
    heat = 1.0 + coef * torch.log(torch.floor((positions.float() + 1.0) / every) + 1.0)
    qn = q / torch.sqrt(q.pow(2).mean(-1, keepdim=True) + eps) * q_w.float() * heat[:, None]
    kn = k / torch.sqrt(k.pow(2).mean(-1, keepdim=True) + eps) * k_w.float()
    if slots is not None:
        m = slots >= 0
        sl = slots[m].long()
        k_cache[sl // page_size, :, sl % page_size, :] = kn[m].view(-1, G, D).to(k_cache.dtype)
        v_cache[sl // page_size, :, sl % page_size, :] = proj[m, hd:hd + gd].view(-1, G, D)
    proj[:, :hd] = qn.to(proj.dtype)


def _pair_angles(positions, freq, magnitude):
    a = positions.float()[:, None] * freq.float()[None, :]              # 32-bit angles, as the kernels take them
    return torch.cos(a) * magnitude, torch.sin(a) * magnitude


def _rotate(x, cos, sin):
    """x [T, ..., R] float: the first 2 n dims in neighbouring pairs; cos, sin [T, n]."""
    n = cos.shape[1]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [n]
    c, s = cos.view(shape), sin.view(shape)
    a, b = x[..., 0:2 * n:2], x[..., 1:2 * n:2]
    out = x.clone()
    out[..., 0:2 * n:2] = a * c - b * s
    out[..., 1:2 * n:2] = b * c + a * s
    return out


def _latent_kv_write(self, proj, col0, weight, eps, positions, freq, magnitude, rot_dims, k_cache, slots, rank, R, page_size):
    c = proj[:, col0:col0 + rank].float()
    c = c / torch.sqrt(c.pow(2).mean(-1, keepdim=True) + eps) * weight.float()
    cos, sin = _pair_angles(positions, freq, magnitude)
    kr = _rotate(proj[:, col0 + rank:col0 + rank + R].float(), cos[:, :rot_dims // 2], sin[:, :rot_dims // 2])
    m = slots >= 0
    sl = slots[m].long()
    k_cache[sl // page_size, 0, sl % page_size, :] = torch.cat([c, kr], -1)[m].to(k_cache.dtype)


def _rotate_pairs(self, dst, src, positions, freq, magnitude, rot_dims):
    cos, sin = _pair_angles(positions, freq, magnitude)
    dst.copy_(_rotate(src.float(), cos[:, :rot_dims // 2], sin[:, :rot_dims // 2]).to(dst.dtype))


def _batched_linear(self, out, x, w):
    out.copy_(torch.einsum("thk,hnk->thn", x.float(), w.float()).to(out.dtype))


def _rope_headnorm_write(self, proj, k_off, v_off, positions, freq, rot_dims, norm_eps, k_cache, v_cache, slots, H, G, D, V,
                         page_size):
    T = proj.shape[0]
    q = proj[:, :H * D].float().reshape(T, H, D).clone()
    k = proj[:, k_off:k_off + G * D].float().reshape(T, G, D).clone()

    def turn(x):
        if rot_dims:
            half = rot_dims // 2
            a = positions.float()[:, None] * freq.float()[None, :]
            c, s = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
            u, v = x[..., :half], x[..., half:rot_dims]
            x = torch.cat([u * c - v * s, v * c + u * s, x[..., rot_dims:]], -1)
        if norm_eps is not None:
            x = x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + norm_eps)
        return x

    proj[:, :H * D] = turn(q).reshape(T, H * D).to(proj.dtype)
    if slots is None:
        return proj
    k = turn(k).to(proj.dtype)
    v = proj[:, v_off:v_off + G * V].view(T, G, V)
    for t, slot in enumerate(slots.tolist()):
        if slot >= 0:
            k_cache[slot // page_size, :, slot % page_size] = k[t]
            v_cache[slot // page_size, :, slot % page_size] = v[t]
    return proj


def _attention_biased(self, out, q, k_cache, v_cache, block_tables, step, KVH, page_size, scale, softcap, slopes, window,
                      chunk=None, sinks=None):
    T, H, Dk = q.shape
    Dv = out.shape[2]
    G = H // KVH
    qsl = step.q_start.tolist()
    out.zero_()
    for b, seq_len in enumerate(step.seq_lens.tolist()):
        qs, qe = qsl[b], qsl[b + 1]
        if seq_len == 0 or qe == qs:
            continue
        Tq = qe - qs
        nb = -(-seq_len // page_size)
        blocks = block_tables[b, :nb].long()
        kk = k_cache[blocks].permute(0, 2, 1, 3).reshape(nb * page_size, KVH, Dk)[:seq_len].float()
        if v_cache is None:
            vv = kk[:, :, :Dv]
        else:
            vv = v_cache[blocks].permute(0, 2, 1, 3).reshape(nb * page_size, KVH, Dv)[:seq_len].float()
        i = torch.arange(Tq)[:, None] + (seq_len - Tq)
        j = torch.arange(seq_len)[None, :]
        ok = j <= i
        if window:
            ok = ok & (j > i - window)
        if chunk:
            ok = ok & (j >= i // chunk * chunk)
        vv = torch.where(ok.any(0)[:, None, None], vv, torch.zeros_like(vv))      # pages a window gave back
        kk = torch.where(ok.any(0)[:, None, None], kk, torch.zeros_like(kk))
        for h in range(H):
            s = (q[qs:qe, h].float() @ kk[:, h // G].t()) * scale
            if softcap:
                s = softcap * torch.tanh(s / softcap)
            if slopes is not None:
                s = s - float(slopes[h]) * (i - j).float()
            s = s.masked_fill(~ok, float("-inf"))
            if sinks is not None:
                s = torch.cat([s, sinks[h].float().expand(Tq, 1)], -1)
            p = torch.softmax(s, -1)[:, :seq_len]
            out[qs:qe, h] = (p @ vv[:, h // G]).to(out.dtype)


# -- a residual stream in several copies, the state-space mixer, gates -----------------------------------------------
def _hyper_norm(self, out, streams, y, mix, out_w, in_w, weight, eps, first=False, alpha=1.0):
    T, S, h = streams.shape
    y = self.materialize(y)
    if first:
        streams.copy_((alpha * y.float())[:, None, :].expand(T, S, h))
    elif y is not None:
        m = torch.eye(S) if mix is None else mix.float()
        o = torch.ones(S) if out_w is None else out_w.float()
        streams.copy_(torch.einsum("st,bsh->bth", m, streams) + o[None, :, None] * y.float()[:, None, :])
    if out is None:
        return
    w_in = torch.ones(S) if in_w is None else in_w.float()
    u = torch.einsum("s,bsh->bh", w_in, streams)
    out.copy_((u / torch.sqrt(u.pow(2).mean(-1, keepdim=True) + eps) * weight.float()).to(out.dtype))


def _ssm_prepare(self, ready, proj, xbc_off, dt_off, conv_w, conv_b, a_log, dt_bias, state, tail_off, step, H, channels, taps):
    qs, slots = step.q_start.tolist(), step.state_slots.tolist()
    for b in range(step.num_requests):
        lo, hi = qs[b], qs[b + 1]
        if hi <= lo:
            continue
        tail = state[slots[b]][tail_off:tail_off + (taps - 1) * channels].view(taps - 1, channels)
        x = torch.cat([tail, proj[lo:hi, xbc_off:xbc_off + channels].float()], 0)
        acc = conv_b.float().expand(hi - lo, channels).clone() if conv_b is not None else torch.zeros(hi - lo, channels)
        for u in range(taps):
            acc = acc + x[u:u + hi - lo] * conv_w.float()[:, u]
        ready[lo:hi, :channels] = F.silu(acc)
        dt = F.softplus(proj[lo:hi, dt_off:dt_off + H].float() + dt_bias.float())
        ready[lo:hi, channels:channels + H] = dt
        ready[lo:hi, channels + H:] = torch.exp(-torch.exp(a_log.float()) * dt)


def _ssm_scan(self, out, ready, proj, xbc_off, state, skip, step, H, G, N, P, taps):
    qs, slots = step.q_start.tolist(), step.state_slots.tolist()
    inner, channels = H * P, H * P + 2 * G * N
    for b in range(step.num_requests):
        lo, hi = qs[b], qs[b + 1]
        if hi <= lo:
            continue
        row = state[slots[b]]
        S = row[:H * N * P].view(H, N, P)
        for t in range(lo, hi):
            x = ready[t, :inner].view(H, P)
            Bm = ready[t, inner:inner + G * N].view(G, N).repeat_interleave(H // G, 0)
            Cm = ready[t, inner + G * N:channels].view(G, N).repeat_interleave(H // G, 0)
            dt, a = ready[t, channels:channels + H], ready[t, channels + H:]
            S.mul_(a[:, None, None]).add_(dt[:, None, None] * Bm[:, :, None] * x[:, None, :])
            y = torch.einsum("hnp,hn->hp", S, Cm)
            if skip is not None:
                y = y + skip.float()[:, None] * x
            out[t] = y.reshape(-1)
        if taps > 1:
            tail = row[H * N * P:].view(taps - 1, channels)
            tail.copy_(torch.cat([tail, proj[lo:hi, xbc_off:xbc_off + channels].float()], 0)[-(taps - 1):].clone())


def _gate(g, kind):
    return F.silu(g.float()) if kind == "silu" else torch.sigmoid(g.float())


def _gated_group_rmsnorm(self, out, x, gate, weight, eps, groups=1, gate_kind="sigmoid", gate_first=False, scale=1.0):
    T, n = x.shape
    g = _gate(gate, gate_kind)
    v = x.float() * g if gate_first else x.float()
    v = v.view(T, groups, n // groups)
    v = (v / torch.sqrt(v.pow(2).mean(-1, keepdim=True) + eps)).reshape(T, n) * weight.float()
    if not gate_first:
        v = v * g
    out.copy_((v * scale).to(out.dtype))


def _gate_mul(self, out, a, gate, gate_kind="sigmoid", scale=1.0):
    out.copy_((a.float() * _gate(gate, gate_kind) * scale).to(out.dtype))


def _act_mul(self, out, gu, act, group=0):
    i = gu.shape[-1] // 2
    if group:
        blocks = gu.reshape(gu.shape[0], i // group, 2, group)
        g, u = blocks[:, :, 0].reshape(-1, i), blocks[:, :, 1].reshape(-1, i)
    else:
        g, u = gu[..., :i], gu[..., i:]
    a = torch.empty_like(g)
    self.activation(a, g, act)
    out.copy_((a.float() * u.float()).to(out.dtype))


def _rope_pairs_write(self, proj, k_off, v_off, positions, freq, magnitude, rot_dims, k_cache, v_cache, slots, H, G, D, V,
                      page_size):
    T = proj.shape[0]

    def turn(x):
        if not rot_dims:
            return x.clone()
        a = positions.float()[:, None] * freq.float()[None, :rot_dims // 2]
        c, s = (torch.cos(a) * magnitude)[:, None, :], (torch.sin(a) * magnitude)[:, None, :]
        y = x.clone()
        u, v = x[..., 0:rot_dims:2], x[..., 1:rot_dims:2]
        y[..., 0:rot_dims:2] = u * c - v * s
        y[..., 1:rot_dims:2] = v * c + u * s
        return y

    q = turn(proj[:, :H * D].float().reshape(T, H, D))
    k = turn(proj[:, k_off:k_off + G * D].float().reshape(T, G, D)).to(proj.dtype)
    proj[:, :H * D] = q.reshape(T, H * D).to(proj.dtype)
    if slots is None:
        return
    v = proj[:, v_off:v_off + G * V].reshape(T, G, V)
    for t, slot in enumerate(slots.tolist()):
        if slot >= 0:
            k_cache[slot // page_size, :, slot % page_size] = k[t]
            v_cache[slot // page_size, :, slot % page_size] = v[t]


for _name, _fn in (("hyper_norm", _hyper_norm), ("ssm_prepare", _ssm_prepare), ("ssm_scan", _ssm_scan),
                   ("gated_group_rmsnorm", _gated_group_rmsnorm), ("gate_mul", _gate_mul), ("act_mul", _act_mul),
                   ("rope_pairs_write", _rope_pairs_write)):
    setattr(TwinOps, _name, _fn)

for _name, _fn in (("delta_prepare", _delta_prepare), ("delta_scan", _delta_scan),
                   ("head_gated_rmsnorm", _head_gated_rmsnorm), ("rms_rows", _rms_rows),
                   ("qk_rownorm_write", _qk_rownorm_write), ("latent_kv_write", _latent_kv_write),
                   ("rotate_pairs", _rotate_pairs), ("batched_linear", _batched_linear),
                   ("attention_biased", _attention_biased), ("rope_headnorm_write", _rope_headnorm_write)):
    setattr(TwinOps, _name, _fn)
