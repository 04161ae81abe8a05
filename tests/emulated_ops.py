"""Plain torch statements of what each CUDA kernel of the engine computes.

Two uses, both in tests only: (1) the per-kernel GPU tests compare every kernel with
the function of the same name here; (2) the CPU tests put this table in place of the
kernel table so that the engine's host logic (batching, cache, scheduler, replay) can
be exercised without a GPU.  Loops are deliberately simple; nothing here is fast.
"""

from __future__ import annotations


import torch


class TorchOps:
    name = "torch-emulation"

    def prepare(self, groups):
        pass

    # ---- norms ----------------------------------------------------------------------
    def fused_norm(self, out, weight, eps, *, resid=None, pending=None, ids=None, table=None, rows=None,
                   write_resid=True, num_rows=None, post_weight=None, post_eps=0.0, add_ids=None, add_table=None,
                   add_vector=None, center=False, post_center=False):
        n = out.shape[0] if num_rows is None else num_rows
        src = rows[:n].long() if rows is not None else torch.arange(n, device=out.device)
        if ids is not None:
            v = table[ids.long()[src]].float()
        else:
            v = resid[src].float()
        if pending is not None and pending.dim() == 3:  # fp32 partial sums [parts, rows, H], added in order
            total = pending[0][src]
            for p in range(1, pending.shape[0]):
                total = total + pending[p][src]
        elif pending is not None:
            total = pending[src].float()
        if pending is not None:
            if post_weight is not None:  # what is pending is normalised before it is added
                if post_center:
                    total = total - total.mean(-1, keepdim=True)
                total = (total * torch.rsqrt(total.pow(2).mean(-1, keepdim=True) + post_eps)) * post_weight.float()
            v = v + total
        if add_ids is not None:
            v = v + add_table[add_ids.long()[src]].float()
        if add_vector is not None:
            v = v + add_vector.float()
        if write_resid:
            resid[src] = v
        if weight is None:  # the sum itself, rounded
            out[:n] = v.to(out.dtype)
            return out
        if center:
            v = v - v.mean(-1, keepdim=True)
        var = v.pow(2).mean(-1, keepdim=True)
        out[:n] = ((v * torch.rsqrt(var + eps)) * weight.float()).to(out.dtype)
        return out

    def sigmoid_mul(self, x, gate):
        x.copy_((x.float() * torch.sigmoid(gate.float())).to(x.dtype))
        return x

    def grouped_norm(self, out, weight, eps, groups, *, resid, pending=None, pending_more=None, rows=None,
                     write_resid=True, num_rows=None, out2=None, weight2=None):
        n = out.shape[0] if num_rows is None else num_rows
        src = rows[:n].long() if rows is not None else torch.arange(n, device=out.device)
        H = resid.shape[1]
        add = None
        if pending is not None and pending.dim() == 3:
            add = pending[0][src]
            for p in range(1, pending.shape[0]):
                add = add + pending[p][src]
        elif pending is not None:
            add = pending[src].float()
        if pending_more is not None:
            add = pending_more[src].float() if add is None else add + pending_more[src].float()
        v = resid[src].float()
        if add is not None:
            v = v + add
        if write_resid:
            resid[src] = v
        if weight is None:
            out[:n] = v.to(out.dtype)
            return out
        parts = v.reshape(n, groups, H // groups)
        unit = (parts * torch.rsqrt(parts.pow(2).mean(-1, keepdim=True) + eps)).reshape(n, H)
        out[:n] = (unit * weight.float()).to(out.dtype)
        if out2 is not None:
            out2[:n] = (unit * weight2.float()).to(out2.dtype)
        return out

    def bigram_embed(self, ids, *, embed, scale, bigram, buckets, mul_prev, mul_cur, prev_state, positions,
                     token_seq, cu_seqlens, state_slots, num_seqs, out, copy=None):
        T = out.shape[0]
        tok = ids[:T].long()
        x = embed[tok].float() * scale
        if buckets:
            for b in range(num_seqs):
                t0, t1 = int(cu_seqlens[b]), int(cu_seqlens[b + 1])
                slot = int(state_slots[b])
                for t in range(t0, t1):
                    if int(positions[t]) == 0:
                        row = buckets
                    else:
                        prev = int(tok[t - 1]) if t > t0 else int(prev_state[slot, 0])
                        row = (prev * mul_prev + int(tok[t]) * mul_cur) % buckets
                    x[t] = x[t] + bigram[row].float()
                if t1 > t0:
                    prev_state[slot, 0] = int(tok[t1 - 1])
        out.copy_(x)
        if copy is not None:
            copy.copy_(x.to(copy.dtype))
        return out

    def token_shift_mix(self, h, mu, *, state, positions, token_seq, cu_seqlens, state_slots, num_seqs):
        T, W = h.shape
        prev = torch.zeros((T, W), dtype=torch.float32, device=h.device)
        for b in range(num_seqs):
            t0, t1 = int(cu_seqlens[b]), int(cu_seqlens[b + 1])
            slot = int(state_slots[b])
            for t in range(t0, t1):
                if int(positions[t]) > 0:
                    prev[t] = h[t - 1].float() if t > t0 else state[slot]
            if t1 > t0:
                state[slot] = h[t1 - 1].float()
        hf = h.float()
        return (hf[None] + (prev - hf)[None] * mu.float()[:, None, :]).to(h.dtype)

    def tanh_rows(self, x):
        x.copy_(torch.tanh(x.float()).to(x.dtype))
        return x

    def stabilised_gates(self, zi, zf, *, i_bias, f_bias, cap, m_state, cu_seqlens, state_slots, num_seqs):
        T, H = zi.shape
        li = cap * torch.tanh((zi.float() + i_bias.float()) / cap)
        lf = torch.nn.functional.logsigmoid(cap * torch.tanh((zf.float() + f_bias.float()) / cap))
        decay = torch.empty((T, H), dtype=torch.float32, device=zi.device)
        k_scale, m_run = torch.empty_like(decay), torch.empty_like(decay)
        for b in range(num_seqs):
            slot = int(state_slots[b])
            m = m_state[slot].clone()
            for t in range(int(cu_seqlens[b]), int(cu_seqlens[b + 1])):
                m_new = torch.maximum(lf[t] + m, li[t])
                decay[t] = torch.exp(lf[t] + m - m_new)
                k_scale[t] = torch.exp(li[t] - m_new)
                m_run[t] = m = m_new
            m_state[slot] = m
        return decay, k_scale, m_run

    def qk_norm_store(self, proj, *, num_heads, num_kv_heads, head_dim, value_dim, k_start, v_start, q_weight, k_weight,
                      eps, positions, token_seq, block_table, k_pages, v_pages, page_size, write_kv, maps=1,
                      num_value_heads=None, inv_freq=None, pairing="half", magnitude=1.0):
        T = proj.shape[0]
        H, G, D, Dv = num_heads, num_kv_heads, head_dim, value_dim
        Gv = int(num_value_heads or G)
        Dm = D // maps

        def unit(x, w):  # x [T, n, D] float: every map normalised by itself, then turned
            x = x.reshape(T, -1, maps, Dm)
            if w is not None:
                x = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w.float()
            if inv_freq is not None:
                x = self._turn_pairs(x, positions.long(), inv_freq, pairing, magnitude)
            return x.reshape(T, -1, D)

        raw_k = proj[:, k_start:k_start + G * D].reshape(T, G, D).float()
        raw_v = proj[:, v_start:v_start + Gv * Dv].reshape(T, Gv, Dv).clone()
        q = unit(proj[:, : H * D].reshape(T, H, D).float(), q_weight)
        proj[:, : H * D] = q.reshape(T, H * D).to(proj.dtype)
        if not write_kv:
            return
        k = unit(raw_k, k_weight).to(proj.dtype)
        for t in range(T):
            p = int(positions[t])
            page = int(block_table[int(token_seq[t]), p // page_size])
            if page < 0:
                continue
            k_pages[page, :, p % page_size, :] = k[t]
            v_pages[page, :, p % page_size, :] = raw_v[t]

    @staticmethod
    def _turn_pairs(x, pos, inv_freq, pairing, magnitude=1.0):
        """x [T, ..., n] float: the leading 2 * len(inv_freq) elements of the last axis turn by position * inv_freq[i];
        pair i is (2i, 2i + 1) ("interleaved") or (i, i + pairs) ("half"); cos and sin times ``magnitude``."""
        if inv_freq is None:
            return x
        pairs = inv_freq.numel()
        ang = pos.float()[:, None] * inv_freq.float()[None, :]
        shape = [x.shape[0]] + [1] * (x.dim() - 2) + [pairs]
        c, s = (ang.cos() * magnitude).reshape(shape), (ang.sin() * magnitude).reshape(shape)
        out = x.clone()
        if pairing == "interleaved":
            u, v = x[..., 0:2 * pairs:2], x[..., 1:2 * pairs:2]
            out[..., 0:2 * pairs:2] = u * c - v * s
            out[..., 1:2 * pairs:2] = v * c + u * s
        else:
            u, v = x[..., :pairs], x[..., pairs:2 * pairs]
            out[..., :pairs] = u * c - v * s
            out[..., pairs:2 * pairs] = v * c + u * s
        return out

    def silu_mul(self, gate_up, out):
        I = out.shape[-1]
        g, u = gate_up[:, :I].float(), gate_up[:, I:].float()
        out.copy_(((g / (1 + torch.exp(-g))) * u).to(out.dtype))
        return out

    def relu_squared(self, x, out):
        out.copy_((torch.relu(x[:, : out.shape[1]].float()) ** 2).to(out.dtype))
        return out

    def gelu_gate_rows(self, gate, ids, table, offset, out):
        z = gate.float()
        g = 0.5 * z * (1.0 + torch.tanh(0.7978845608028654 * (z + 0.044715 * z ** 3)))
        out.copy_((g * table[ids.long(), offset:offset + gate.shape[1]].float()).to(out.dtype))
        return out

    # ---- decayed matrix state and short convolution ----------------------------------------
    @staticmethod
    def _turn_halves(x, pos, inv_freq):
        """Pairs (i, i + pairs) of the leading 2 * len(inv_freq) elements of the last axis; x [T, H, n] float."""
        if inv_freq is None:
            return x
        pairs = inv_freq.numel()
        ang = pos.float()[:, None] * inv_freq.float()[None, :]
        c, s = ang.cos()[:, None, :], ang.sin()[:, None, :]
        u, v = x[..., :pairs], x[..., pairs:2 * pairs]
        return torch.cat([u * c - v * s, v * c + u * s, x[..., 2 * pairs:]], dim=-1)

    def decayed_state_scan(self, q, k, v, *, state, cu_seqlens, state_slots, num_seqs, decay_logits=None,
                           decay_bias=None, tau=1.0, head_decay=None, inv_freq=None, positions=None, q_scale=1.0,
                           k_scale=1.0, decay_mode="sigmoid_pow", token_decay=None, token_k_scale=None, bonus=None,
                           ones_column=False):
        T, H, D = q.shape
        Dv = v.shape[2] + int(ones_column)
        vf = v.float()
        if ones_column:
            vf = torch.cat([vf, torch.ones((T, H, 1), dtype=torch.float32, device=v.device)], dim=-1)
        qf, kf = q.float(), k.float()
        if inv_freq is not None:
            qf, kf = self._turn_halves(qf, positions.long(), inv_freq), self._turn_halves(kf, positions.long(), inv_freq)
        qf, kf = qf * q_scale, kf * k_scale
        if decay_logits is not None:
            z = decay_logits.float()
            if decay_bias is not None:
                z = z + decay_bias.float().reshape(1, H, D)
            a = torch.exp(-torch.exp(z)) if decay_mode == "exp_neg_exp" else torch.exp(torch.nn.functional.logsigmoid(z) / tau)
        elif token_decay is not None:
            a = token_decay.float().reshape(T, H, 1).expand(T, H, D)
        else:
            a = head_decay.float().reshape(1, H, 1).expand(T, H, D)
        if token_k_scale is not None:
            kf = kf * token_k_scale.float().reshape(T, H, 1)
        u = bonus.float().reshape(H, D) if bonus is not None else None
        out = torch.empty((T, H, Dv), dtype=torch.float32, device=q.device)
        for b in range(num_seqs):
            slot = int(state_slots[b])
            S = state[slot].clone()
            for t in range(int(cu_seqlens[b]), int(cu_seqlens[b + 1])):
                kv = kf[t][:, :, None] * vf[t][:, None, :]
                if u is not None:  # the present token counts with the bonus, the state is read before its update
                    out[t] = torch.einsum("hdv,hd->hv", S + u[:, :, None] * kv, qf[t])
                S = a[t][:, :, None] * S + kv
                if u is None:
                    out[t] = torch.einsum("hdv,hd->hv", S, qf[t])
            state[slot] = S
        return out

    def head_norm_gate(self, o, gate, out, *, weight, eps, out_scale=1.0, gate_act="silu", per_head_weight=False,
                       denominator=None):
        T, H, Dv = out.shape
        if denominator is not None:  # o's last column is n . q; the value columns are divided first
            den = torch.maximum(o[:, :, Dv].abs(), torch.exp(-denominator.float())) + 1e-6
            o = o[:, :, :Dv] / den[:, :, None]
        x = o * torch.rsqrt(o.pow(2).mean(-1, keepdim=True) + eps)
        if weight is not None:
            x = x * (weight.float().reshape(H, Dv) if per_head_weight else weight.float())
        g = gate.float()
        act = torch.sigmoid(g) if gate_act == "sigmoid" else g / (1 + torch.exp(-g))
        out.copy_((x * act * out_scale).to(out.dtype))
        return out

    def conv_rope_store(self, x, *, num_heads, num_kv_heads, head_dim, value_dim, conv_weight, conv_state, inv_freq,
                        positions, token_seq, cu_seqlens, state_slots, num_seqs, block_table, k_pages, v_pages,
                        page_size, q_out, value_scale=1.0, write_kv=True):
        T, C = x.shape
        nq, nkv, D, Dv = num_heads, num_kv_heads, head_dim, value_dim
        u = x.float()
        y = u.clone()
        taps = conv_weight.shape[0] if conv_weight is not None else 0  # [taps, C]
        if taps:
            for b in range(num_seqs):
                t0, t1 = int(cu_seqlens[b]), int(cu_seqlens[b + 1])
                slot = int(state_slots[b])
                old = conv_state[slot].float() if taps > 1 else u.new_zeros((0, C))
                rows = torch.cat([old, u[t0:t1]])  # row m + n is the portion's token n
                for n in range(t1 - t0):
                    acc = u.new_zeros(C)
                    for j in range(taps):
                        acc = acc + conv_weight[j].float() * rows[n + j]
                    y[t0 + n] = acc
                if taps > 1:
                    conv_state[slot] = rows[rows.shape[0] - (taps - 1):]
        pos = positions.long()
        q = self._turn_halves(y[:, : nq * D].reshape(T, nq, D), pos, inv_freq)
        q_out.copy_(q.reshape(T, nq * D).to(q_out.dtype))
        if not write_kv:
            return
        k = self._turn_halves(y[:, nq * D:(nq + nkv) * D].reshape(T, nkv, D), pos, inv_freq).to(k_pages.dtype)
        v = (y[:, (nq + nkv) * D:].reshape(T, nkv, Dv) * value_scale).to(v_pages.dtype)
        for t in range(T):
            p = int(pos[t])
            page = int(block_table[int(token_seq[t]), p // page_size])
            k_pages[page, :, p % page_size, :] = k[t]
            v_pages[page, :, p % page_size, :] = v[t]

    # ---- position encoding + cache write -----------------------------------------------
    def rope_table(self, inv_freq, max_positions):
        ang = torch.arange(max_positions, dtype=torch.float32, device=inv_freq.device)[:, None] * inv_freq[None, :]
        return ang.cos(), ang.sin()

    def qk_norm_rope_store(self, qkv, *, num_heads, num_kv_heads, head_dim, q_weight, k_weight, eps, cos, sin,
                           positions, token_seq, block_table, k_pages, v_pages, page_size, write_kv,
                           pairing="half"):
        T = qkv.shape[0]
        D = head_dim
        pos = positions.long()

        def norm_rope(x, w):  # x [T, n, D] float
            if w is not None:
                x = (x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps)) * w.float()
            if cos is not None:
                half = cos.shape[1]
                c, s = cos[pos][:, None, :], sin[pos][:, None, :]
                rest = x[..., 2 * half:]
                if pairing == "interleaved":  # pair i = elements (2i, 2i + 1)
                    x1, x2 = x[..., 0:2 * half:2], x[..., 1:2 * half:2]
                    rot = torch.stack((x1 * c - x2 * s, x2 * c + x1 * s), dim=-1).flatten(-2)
                    x = torch.cat((rot, rest), dim=-1)
                else:  # pair i = elements (i, i + half)
                    x1, x2 = x[..., :half], x[..., half:2 * half]
                    x = torch.cat((x1 * c - x2 * s, x2 * c + x1 * s, rest), dim=-1)
            return x

        nq, nkv = num_heads, num_kv_heads
        q = qkv[:, : nq * D].reshape(T, nq, D).float()
        qkv[:, : nq * D] = norm_rope(q, q_weight).reshape(T, nq * D).to(qkv.dtype)
        if not write_kv:
            return
        k = norm_rope(qkv[:, nq * D:(nq + nkv) * D].reshape(T, nkv, D).float(), k_weight).to(qkv.dtype)
        v = qkv[:, (nq + nkv) * D:(nq + 2 * nkv) * D].reshape(T, nkv, D)
        for t in range(T):
            p = int(pos[t])
            page = int(block_table[int(token_seq[t]), p // page_size])
            k_pages[page, :, p % page_size, :] = k[t]
            v_pages[page, :, p % page_size, :] = v[t]

    # ---- attention --------------------------------------------------------------------
    def paged_attention(self, q, q_stride, *, num_heads, num_kv_heads, head_dim, k_pages, v_pages, block_table,
                        token_seq, positions, out, page_size, scale, window, step=None, decode_slices=None,
                        value_dim=None, keep_first=0, sink=None, gate=None, chunk=None, softcap=None):
        T = out.shape[0]
        D = head_dim
        group = num_heads // num_kv_heads
        for t in range(T):
            p = int(positions[t])
            lo = max(0, p - window + 1) if window else 0
            if chunk:
                lo = max(lo, p // chunk * chunk)
            table = block_table[int(token_seq[t])]
            js = torch.cat([torch.arange(0, min(keep_first, lo)), torch.arange(lo, p + 1)])
            pages = table[(js // page_size).to(table.device)].long()
            offs = (js % page_size).to(pages.device)
            keys = k_pages[pages, :, offs, :].float()  # [n, nkv, D]
            vals = v_pages[pages, :, offs, :].float()
            qt = q[t, : num_heads * D].reshape(num_heads, D).float()
            kh = keys.repeat_interleave(group, dim=1)  # [n, nq, D]
            vh = vals.repeat_interleave(group, dim=1)
            scores = torch.einsum("hd,nhd->hn", qt, kh) * scale
            if softcap:
                scores = softcap * torch.tanh(scores / softcap)
            if sink is not None:  # one more score that has no value
                scores = torch.cat([scores, torch.full((num_heads, 1), float(sink), device=scores.device)], dim=-1)
                probs = torch.softmax(scores, dim=-1)[:, :-1]
            else:
                probs = torch.softmax(scores, dim=-1)
            res = torch.einsum("hn,nhd->hd", probs, vh).reshape(-1)
            if gate is not None:
                res = res * torch.sigmoid(gate[t].float())
            out[t] = res.to(out.dtype)
        return out

    def differential_attention(self, q, q_stride, *, num_heads, num_kv_heads, map_dim, value_dim, k_pages, v_pages,
                               block_table, token_seq, positions, out, page_size, scale, lam, eps, out_scale,
                               window=None, chunk=None, step=None):
        T = out.shape[0]
        D = map_dim
        group = num_heads // num_kv_heads
        for t in range(T):
            p = int(positions[t])
            lo = max(0, p - window + 1) if window else 0
            if chunk:
                lo = max(lo, p // chunk * chunk)
            table = block_table[int(token_seq[t])]
            js = torch.arange(lo, p + 1)
            pages = table[(js // page_size).to(table.device)].long()
            offs = (js % page_size).to(pages.device)
            keys = k_pages[pages, :, offs, :].float().repeat_interleave(group, dim=1)  # [n, nq, 2D]
            vals = v_pages[pages, :, offs, :].float().repeat_interleave(group, dim=1)  # [n, nq, Dv]
            qt = q[t, : num_heads * 2 * D].reshape(num_heads, 2, D).float()
            kk = keys.reshape(-1, num_heads, 2, D)
            probs = torch.softmax(torch.einsum("hmd,nhmd->hmn", qt, kk) * scale, dim=-1)
            a = torch.einsum("hmn,nhd->hmd", probs, vals)
            o = a[:, 0] - lam * a[:, 1]
            o = o * torch.rsqrt(o.pow(2).mean(-1, keepdim=True) + eps) * out_scale
            out[t] = o.reshape(-1).to(out.dtype)
        return out

    # ---- attention through a latent ------------------------------------------------------
    @staticmethod
    def _turn(x, pos, inv_freq):
        """Interleaved pairs of the leading 2 * len(inv_freq) elements of the last axis; x [T, ..., n] float."""
        if inv_freq is None:
            return x
        pairs = inv_freq.numel()
        ang = pos.float()[:, None] * inv_freq.float()[None, :]
        shape = [x.shape[0]] + [1] * (x.dim() - 2) + [pairs]
        c, s = ang.cos().reshape(shape), ang.sin().reshape(shape)
        u, v = x[..., 0:2 * pairs:2], x[..., 1:2 * pairs:2]
        out = x.clone()
        out[..., 0:2 * pairs:2] = u * c - v * s
        out[..., 1:2 * pairs:2] = v * c + u * s
        return out

    def latent_norm_rope_store(self, down, *, q_rank, kv_rank, rot_dim, q_weight, kv_weight, eps, inv_freq, positions,
                               token_seq, block_table, pages, page_size, write, q_out, pairing="interleaved",
                               magnitude=1.0):
        x = down.float()
        if q_rank:
            a = x[:, :q_rank]
            q_out.copy_(((a * torch.rsqrt(a.pow(2).mean(-1, keepdim=True) + eps)) * q_weight.float()).to(q_out.dtype))
        if not write:
            return
        c = x[:, q_rank:q_rank + kv_rank]
        c = (c * torch.rsqrt(c.pow(2).mean(-1, keepdim=True) + eps)) * kv_weight.float()
        k = self._turn_pairs(x[:, q_rank + kv_rank:q_rank + kv_rank + rot_dim], positions.long(), inv_freq, pairing,
                             magnitude)
        row = torch.cat([c, k], dim=-1).to(pages.dtype)
        for t in range(down.shape[0]):
            p = int(positions[t])
            page = int(block_table[int(token_seq[t]), p // page_size])
            pages[page, p % page_size] = row[t]

    def head_linear(self, x, weight, out):
        """out[t, h] = weight[h] @ x[t, h]; x [T, H, K], weight [H, N, K], out [T, H, N] (views allowed)."""
        out.copy_(torch.einsum("thk,hnk->thn", x.float(), weight.float()).to(out.dtype))
        return out

    def rotate_heads(self, x, out, *, positions, inv_freq, pairing="interleaved", magnitude=1.0):
        out.copy_(self._turn_pairs(x.float(), positions.long(), inv_freq, pairing, magnitude).to(out.dtype))
        return out

    def latent_attention(self, q, *, pages, value_dim, block_table, token_seq, positions, sink, out, page_size, scale,
                         window, step=None):
        T = q.shape[0]
        for t in range(T):
            p = int(positions[t])
            lo = max(0, p - window + 1) if window else 0
            table = block_table[int(token_seq[t])]
            js = torch.arange(lo, p + 1)
            rows = pages[table[js // page_size].long(), js % page_size].float()  # [n, width]
            scores = (q[t].float() @ rows.t()) * scale  # [H, n]
            if sink is not None:
                scores = torch.cat([scores, sink.float()[:, None]], dim=-1)
            probs = torch.softmax(scores, dim=-1)[:, : js.numel()]
            out[t] = (probs @ rows[:, :value_dim]).to(out.dtype)
        return out

    # ---- routed experts ----------------------------------------------------------------
    def route_top(self, h, router, top, renormalize=False, score="sigmoid", correction=None, groups=None):
        if score == "softmax_all":
            s_all = torch.softmax(h.float() @ router.float().t(), dim=-1)
            choice = s_all + correction.float() if correction is not None else s_all.clone()
            if groups and groups[0] > 1:
                count, keep = groups
                E = choice.shape[1]
                best = choice.reshape(-1, count, E // count).max(-1).values
                kept = torch.zeros_like(best, dtype=torch.bool)
                kept.scatter_(1, best.topk(keep, dim=-1).indices, True)
                choice = choice.masked_fill(~kept.repeat_interleave(E // count, dim=1), float("-inf"))
            chosen = choice.topk(top, dim=-1).indices
            w = s_all.gather(1, chosen)
            if renormalize:
                w = w / (w.sum(-1, keepdim=True) + 1e-20)
            return chosen.to(torch.int32), w.float()
        best = torch.topk(h.float() @ router.float().t(), top, dim=-1)  # on the logits: no saturated ties
        if score == "softmax_chosen":
            return best.indices.to(torch.int32), torch.softmax(best.values, dim=-1).float()
        w = torch.sigmoid(best.values)
        if renormalize:
            w = w / w.sum(-1, keepdim=True)
        return best.indices.to(torch.int32), w.float()

    def clamped_glu(self, gate_up, out, *, limit, alpha, up_offset):
        F = out.shape[-1]
        g = gate_up[:, :F].float().clamp(max=limit)
        u = gate_up[:, F:].float().clamp(-limit, limit)
        out.copy_((g * torch.sigmoid(alpha * g) * (u + up_offset)).to(out.dtype))
        return out

    def routed_experts(self, h, chosen, weights, gate_up, down, *, limit=0.0, alpha=1.0, up_offset=0.0,
                       weight_on="input", shared=None, activation="clamped_glu", shared_gate=None, num_identity=0):
        T, W = h.shape
        gated = activation == "clamped_glu"
        F = gate_up.shape[1] // 2 if gated else gate_up.shape[1]
        total = torch.zeros((T, W), dtype=torch.float32, device=h.device)
        for t in range(T):
            for e, w in zip(chosen[t].tolist(), weights[t].tolist()):
                if e >= gate_up.shape[0]:  # an identity expert: the input itself, times the weight
                    total[t] += h[t].float() * w
                    continue
                x = (h[t].float() * w).to(h.dtype) if weight_on == "input" else h[t]
                gu = (gate_up[e].float() @ x.float()).to(h.dtype)
                mid = torch.empty((1, F), dtype=h.dtype, device=h.device)
                if gated:
                    self.clamped_glu(gu[None], mid, limit=limit, alpha=alpha, up_offset=up_offset)
                else:
                    self.relu_squared(gu[None], mid)
                y = (down[e].float() @ mid[0].float()).to(h.dtype).float()
                total[t] += y if weight_on == "input" else y * w
        if shared is not None and shared_gate is not None:
            total += shared.float() * torch.sigmoid(shared_gate.float())[:, None]
        elif shared is not None:
            total += shared.float()
        return total.to(h.dtype)

    # ---- matrix products ----------------------------------------------------------------
    partial_parts = 0  # > 1: linear(partial_sums=True) answers with that many planes

    def add_bias(self, out, bias):
        out.copy_((out.float() + bias.float()).to(out.dtype))
        return out

    def logit_scale_cap(self, logits, scale=1.0, cap=0.0):
        v = logits * scale
        logits.copy_(cap * torch.tanh(v / cap) if cap > 0 else v)
        return logits

    def linear(self, x, weight, out=None, out_dtype=None, partial_sums=False, bias=None):
        if bias is not None:
            return self.add_bias(self.linear(x, weight, out, out_dtype), bias)
        if partial_sums and self.partial_parts > 1 and out is None and out_dtype is None:
            cuts = torch.linspace(0, x.shape[1], self.partial_parts + 1).long().tolist()
            return torch.stack([x[:, a:b].float() @ weight[:, a:b].float().t() for a, b in zip(cuts, cuts[1:])])
        res = x.float() @ weight.float().t()
        res = res.to(out_dtype or x.dtype)
        if out is not None:
            out.copy_(res)
            return out
        return res

    def gated_linear(self, x, gate_up_weight, out):
        return self.silu_mul(self.linear(x, gate_up_weight), out)

    # ---- sampling ---------------------------------------------------------------------
    def argmax(self, logits, want_logprob=False):
        tok = logits.argmax(-1).to(torch.int32)
        lp = None
        if want_logprob:
            lp = torch.log_softmax(logits.float(), -1).gather(1, tok.long()[:, None])[:, 0]
        return tok, lp

    def sample(self, logits, temperature, uniform, want_logprob=False):
        probs = torch.softmax(logits.float() / temperature[:, None], -1)
        cdf = probs.cumsum(-1)
        idx = torch.searchsorted(cdf, uniform[:, None].contiguous(), right=True)[:, 0].clamp(0, logits.shape[1] - 1)
        lp = None
        if want_logprob:
            lp = torch.log(probs.gather(1, idx[:, None])[:, 0].clamp_min(1e-30))
        return idx.to(torch.int32), lp

    def bias_penalty_row(self, row, *, logit_bias, seen_ids, repetition_penalty, presence_penalty,
                         frequency_penalty):
        for tok, val in (logit_bias or {}).items():
            row[int(tok)] += float(val)
        if seen_ids and not (repetition_penalty == 1.0 and presence_penalty == 0.0 and frequency_penalty == 0.0):
            V = row.numel()
            counts = torch.bincount(torch.tensor([t for t in seen_ids if 0 <= t < V], dtype=torch.long), minlength=V)
            counts = counts.to(row.device)
            seen = counts > 0
            rep = torch.where(row > 0, row / repetition_penalty, row * repetition_penalty)
            row.copy_(torch.where(seen, rep, row) - presence_penalty * seen.float() - frequency_penalty * counts.float())
        return row

    def bias_penalty_rows(self, logits, rows, *, logit_bias, seen_ids, repetition_penalty, presence_penalty,
                          frequency_penalty):
        for i, b, s, rp, pp, fp in zip(rows, logit_bias, seen_ids, repetition_penalty, presence_penalty,
                                       frequency_penalty):
            self.bias_penalty_row(logits[i], logit_bias=b, seen_ids=list(s), repetition_penalty=rp,
                                  presence_penalty=pp, frequency_penalty=fp)
        return logits

    def filter_rows(self, logits, temperature, min_p, top_k, top_p):
        lowest = torch.finfo(torch.float32).min
        for r in range(logits.shape[0]):
            x = logits[r] / temperature[r]
            if float(min_p[r]) > 0:
                p = torch.softmax(x, -1)
                x = torch.where(p < float(min_p[r]) * p.max(), torch.full_like(x, float("-inf")), x)
            k = int(top_k[r])
            if 0 < k < x.numel():
                kth = torch.topk(x, k).values[-1]
                x = torch.where(x < kth, torch.full_like(x, lowest), x)
            tp = float(top_p[r])
            if 0 < tp < 1:
                p = torch.softmax(x, -1)
                order = torch.argsort(x, descending=True, stable=True)
                before = p[order].cumsum(0) - p[order]  # mass ranked before each token
                keep = torch.zeros_like(x, dtype=torch.bool)
                keep[order] = before <= tp
                # tokens tied with a kept one are kept as well (the kernel cuts by value)
                keep |= x >= x[keep].min()
                x = torch.where(keep, x, torch.full_like(x, lowest))
            logits[r] = x
        return logits
