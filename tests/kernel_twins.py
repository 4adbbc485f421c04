"""Plain PyTorch twins of the CUDA kernels, one per kernel, with the same signatures.

They have two uses: each kernel's GPU test compares the kernel with its twin, and the CPU
tests build a runner on top of `TorchOps` to exercise the step function, the cache manager,
the scheduler and the replay program without a GPU. The product never imports this file:
its only kernel set is the CUDA one.

Arithmetic is float32 throughout (float64 with `exact=True`), whatever the storage dtype.
"""

from __future__ import annotations

import torch


class TorchOps:
    def __init__(self, exact: bool = False):
        self.acc = torch.float64 if exact else torch.float32

    # ---------------------------------------------------------------- embedding and norms

    def embed(self, token_ids, table, out, positions=None, position_table=None):
        rows = table[token_ids.long()].to(self.acc)
        if position_table is not None:
            rows = rows + position_table[positions[:out.shape[0]].long()].to(self.acc)
        out.copy_(rows.to(out.dtype))

    def rmsnorm_add(self, h, delta, weight, eps, next_weight, next_eps, out):
        d = delta.to(self.acc)
        normed = d * torch.rsqrt(d.pow(2).mean(-1, keepdim=True) + eps) * weight.to(self.acc)
        h.add_(normed.to(h.dtype))
        if next_weight is not None:
            x = h.to(self.acc)
            out.copy_((x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + next_eps)
                       * next_weight.to(self.acc)).to(out.dtype))

    def patch_tokens(self, token_ids, token_from, sampled):
        late = token_from >= 0
        token_ids[late] = sampled[token_from[late].long()]

    def add_rmsnorm(self, h, delta, weight, eps, out, rows=None):
        if rows is None:
            if delta is not None:
                h.add_(delta.to(h.dtype))
            x = h.to(self.acc)
        else:
            index = rows.long()
            x = h[index].to(self.acc)
            if delta is not None:
                x = x + delta[index].to(self.acc)
        rstd = torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps)
        out.copy_((x * rstd * weight.to(self.acc)).to(out.dtype))

    # ---------------------------------------------------------------- products

    # inputs may be an unevaluated norm (PendingNorm); the twin simply evaluates it

    def can_fuse_norm(self, rows, hidden, weight):
        return rows <= 16

    @staticmethod
    def _x(x):
        return x.materialize() if hasattr(x, "materialize") else x

    def linear_residual(self, x, weight, bias, h, ctx, name, then_norm=None):
        y = self._x(x).to(self.acc) @ weight.to(self.acc).T
        if bias is not None:
            y = y + bias.to(self.acc)
        h.add_(y.to(h.dtype))
        return None

    def linear(self, x, weight, bias, out):
        x = self._x(x)
        y = x.to(self.acc) @ weight.to(self.acc).T
        if bias is not None:
            y = y + bias.to(self.acc)
        out.copy_(y.to(out.dtype))

    def linear_swiglu(self, x, weight, out, ctx=None, ahead=None):
        x = self._x(x)
        gate_up = torch.empty((x.shape[0], weight.shape[0]), dtype=x.dtype, device=x.device)
        self.linear(x, weight, None, gate_up)
        self.swiglu(gate_up, out)

    def linear_gated(self, x, weight, out, ctx, activation):
        x = self._x(x)
        width = out.shape[-1]
        both = x.to(self.acc) @ weight.to(self.acc).T
        both = both.to(x.dtype).to(self.acc)          # the product lands in the activation type
        gate, up = both[:, :width], both[:, width:]
        if activation == "silu":
            act = gate * torch.sigmoid(gate)
        elif activation == "gelu_tanh":
            act = 0.5 * gate * (1.0 + torch.tanh(0.7978845608028654 * (gate + 0.044715 * gate ** 3)))
        else:
            raise ValueError(activation)
        out.copy_((act * up).to(out.dtype))

    # ---------------------------------------------------------------- recurrences

    @staticmethod
    def _sequences(batch):
        starts, slots = batch.q_start.tolist(), batch.slots.tolist()
        for s in range(batch.num_seqs):
            if starts[s + 1] > starts[s]:
                yield starts[s], starts[s + 1], slots[s]

    def mingru_scan(self, pre, state, batch, out):
        width = out.shape[1]
        for begin, end, slot in self._sequences(batch):
            rows = pre[begin:end].to(self.acc)
            z = torch.sigmoid(rows[:, :width])
            u = rows[:, width:2 * width]
            cand = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
            g = rows[:, 2 * width:]
            g = g * torch.sigmoid(g)
            s = state[slot].to(self.acc)
            for t in range(end - begin):
                s = (1.0 - z[t]) * s + z[t] * cand[t]
                out[begin + t] = (s * g[t]).to(out.dtype)
            state[slot] = s.to(state.dtype)

    def causal_conv(self, pre, offset, width, conv, conv_bias, state, batch, u):
        """u[t] = sum_k conv[:, k] * x[t - (taps - 1 - k)] + bias with x = pre[:, offset:
        offset + width]; inputs before the step come from rows 1.. of the state (row j: j
        tokens back), zeros before the sequence's start. The state is left as it was."""
        taps = conv.shape[1]
        for begin, end, slot in self._sequences(batch):
            x = pre[begin:end, offset:offset + width].to(self.acc)
            past = state[slot, 1:taps].to(self.acc).flip(0)          # oldest first
            padded = torch.cat([past, x])
            acc = torch.zeros_like(x)
            for k in range(taps):
                acc = acc + padded[k:k + x.shape[0]] * conv[:, k].to(self.acc)
            u[begin:end] = (acc + conv_bias.to(self.acc)).to(u.dtype)

    def block_gates(self, u, weight, bias, gates):
        """weight [kinds][blocks][in][out], bias [kinds][blocks][out]; gates [tokens][kinds *
        width] = sigmoid of the block-diagonal products."""
        kinds, blocks, size, _ = weight.shape
        ub = u.to(self.acc).view(u.shape[0], blocks, size)
        for kind in range(kinds):
            pre = torch.einsum("bio,tbi->tbo", weight[kind].to(self.acc), ub) + bias[kind].to(self.acc)
            gates[:, kind * blocks * size:(kind + 1) * blocks * size] = \
                torch.sigmoid(pre).reshape(u.shape[0], -1).to(gates.dtype)

    def gated_recurrence_scan(self, pre, u, gates, softplus_lam, decay_scale, state, batch, out):
        width = out.shape[1]
        taps = state.shape[1]
        for begin, end, slot in self._sequences(batch):
            y = pre[begin:end, :width].to(self.acc)
            y = 0.5 * y * (1.0 + torch.tanh(0.7978845608028654 * (y + 0.044715 * y ** 3)))
            uu = u[begin:end].to(self.acc)
            r, i = gates[begin:end, :width].to(self.acc), gates[begin:end, width:].to(self.acc)
            a = torch.exp(-decay_scale * r * softplus_lam.to(self.acc))
            b = torch.sqrt(1.0 - a * a) * i * uu
            s = state[slot, 0].to(self.acc)
            for t in range(end - begin):
                s = a[t] * s + b[t]
                out[begin + t] = (s * y[t]).to(out.dtype)
            state[slot, 0] = s.to(state.dtype)
            if taps > 1:
                x = pre[begin:end, width:2 * width].to(state.dtype)
                history = torch.cat([state[slot, 1:taps].flip(0), x])[-(taps - 1):]
                state[slot, 1:taps] = history.flip(0)

    def qkv_rope_store(self, x, weight, bias, qkv, num_heads, num_kv_heads, head_dim, tables,
                       batch, cache):
        x = self._x(x)
        self.linear(x, weight, bias, qkv)
        self.rope_cache_write(qkv, num_heads, num_kv_heads, head_dim, tables, batch, cache)

    def swiglu(self, gate_up, out):
        width = out.shape[-1]
        gate = gate_up[:, :width].to(self.acc)
        up = gate_up[:, width:].to(self.acc)
        out.copy_((gate * torch.sigmoid(gate) * up).to(out.dtype))

    # ---------------------------------------------------------------- attention

    def rope_cache_write(self, qkv, num_heads, num_kv_heads, head_dim, tables, batch, cache):
        tokens = qkv.shape[0]
        q_size, kv_size = num_heads * head_dim, num_kv_heads * head_dim
        live = batch.seq_of_token[:tokens] >= 0
        pos = batch.positions[:tokens].long()
        if tables is not None:
            cos_t, sin_t = tables
            half = cos_t.shape[1]
            cos = cos_t[pos].to(self.acc).unsqueeze(1)
            sin = sin_t[pos].to(self.acc).unsqueeze(1)
            for start, heads in ((0, num_heads), (q_size, num_kv_heads)):
                x = qkv[:, start:start + heads * head_dim].view(tokens, heads, head_dim)
                a = x[..., :half].to(self.acc)
                b = x[..., half:2 * half].to(self.acc)
                first = (a * cos - b * sin).to(qkv.dtype)
                second = (b * cos + a * sin).to(qkv.dtype)
                x[..., :half] = first
                x[..., half:2 * half] = second
        if cache is None or not cache.write:
            return
        seq = batch.seq_of_token[:tokens].long().clamp(min=0)
        page = cache.table[seq, pos // cache.page_size].long()
        offset = pos % cache.page_size
        k = qkv[:, q_size:q_size + kv_size].view(tokens, num_kv_heads, head_dim)
        v = qkv[:, q_size + kv_size:].view(tokens, num_kv_heads, head_dim)
        keep = live & (page >= 0)
        cache.k[page[keep], :, offset[keep], :] = k[keep].to(cache.k.dtype)
        cache.v[page[keep], :, offset[keep], :] = v[keep].to(cache.v.dtype)

    def qkv_attention(self, x, weight, bias, qkv, num_heads, num_kv_heads, head_dim, tables, batch,
                      cache, scale, window, out):
        self.qkv_rope_store(x, weight, bias, qkv, num_heads, num_kv_heads, head_dim, tables, batch,
                            cache)
        self.paged_attention(qkv, num_heads, num_kv_heads, head_dim, batch, cache, scale, window, out)

    def paged_attention(self, qkv, num_heads, num_kv_heads, head_dim, batch, cache, scale,
                        window, out):
        group = num_heads // num_kv_heads
        q_start = batch.q_start.tolist()
        kv_lens = batch.kv_len.tolist()
        ps = cache.page_size
        for s in range(batch.num_seqs):
            begin, end = q_start[s], q_start[s + 1]
            q_len, kv_len = end - begin, kv_lens[s]
            if q_len == 0:
                continue
            first_pos = kv_len - q_len
            low = max(0, first_pos - window + 1) if window > 0 else 0
            low_page = low // ps
            pages = cache.table[s, low_page:-(-kv_len // ps)].long()
            keys = cache.k[pages].permute(1, 0, 2, 3).reshape(num_kv_heads, -1, head_dim)
            vals = cache.v[pages].permute(1, 0, 2, 3).reshape(num_kv_heads, -1, head_dim)
            key_pos = torch.arange(low_page * ps, low_page * ps + keys.shape[1], device=qkv.device)
            q = qkv[begin:end, :num_heads * head_dim].view(q_len, num_heads, head_dim).to(self.acc)
            q_pos = torch.arange(first_pos, kv_len, device=qkv.device)
            hidden = (key_pos[None, :] > q_pos[:, None]) | (key_pos[None, :] >= kv_len)
            if window > 0:
                hidden = hidden | (key_pos[None, :] <= q_pos[:, None] - window)
            keys = keys.to(self.acc).repeat_interleave(group, dim=0)
            vals = vals.to(self.acc).repeat_interleave(group, dim=0)
            scores = torch.einsum("qhd,hkd->hqk", q, keys) * scale
            scores = scores.masked_fill(hidden[None], float("-inf"))
            weights = torch.softmax(scores, dim=-1)
            weights = torch.nan_to_num(weights)  # a hidden key's value may be non-finite
            vals = torch.where(hidden.all(0)[None, :, None], torch.zeros_like(vals), vals)
            o = torch.einsum("hqk,hkd->qhd", weights, vals)
            out[begin:end] = o.reshape(q_len, num_heads * head_dim).to(out.dtype)

    def rope_blend_store(self, qkv, layout, tables, batch, cache, blend_from, blend, keep):
        """Packed rows [q heads of `dim` | k heads of `dim` | v heads of `vdim`]: q and k are
        rotated over their leading features in place; v is copied to `keep` (if given), then
        blended v <- (1 - c) v + c blend_from (if given); k and v go into the pages."""
        heads, kv_heads, dim, vdim = layout
        tokens = qkv.shape[0]
        q_size, k_size = heads * dim, kv_heads * dim
        live = batch.seq_of_token[:tokens] >= 0
        pos = batch.positions[:tokens].long()
        if tables is not None:
            cos_t, sin_t = tables
            half = cos_t.shape[1]
            cos = cos_t[pos].to(self.acc).unsqueeze(1)
            sin = sin_t[pos].to(self.acc).unsqueeze(1)
            for start, count in ((0, heads), (q_size, kv_heads)):
                x = qkv[:, start:start + count * dim].view(tokens, count, dim)
                a = x[..., :half].to(self.acc)
                b = x[..., half:2 * half].to(self.acc)
                first = (a * cos - b * sin).to(qkv.dtype)
                second = (b * cos + a * sin).to(qkv.dtype)
                x[..., :half] = first
                x[..., half:2 * half] = second
        v = qkv[:, q_size + k_size:]
        if keep is not None:
            keep.copy_(v)
        if blend_from is not None:
            c = blend.to(self.acc)
            v.copy_(((1.0 - c) * v.to(self.acc) + c * blend_from.to(self.acc)).to(qkv.dtype))
        if cache is None or not cache.write:
            return
        seq = batch.seq_of_token[:tokens].long().clamp(min=0)
        page = cache.table[seq, pos // cache.page_size].long()
        offset = pos % cache.page_size
        keep_rows = live & (page >= 0)
        k = qkv[:, q_size:q_size + k_size].view(tokens, kv_heads, dim)
        cache.k[page[keep_rows], :, offset[keep_rows], :] = k[keep_rows].to(cache.k.dtype)
        cache.v[page[keep_rows], :, offset[keep_rows], :] = \
            v.view(tokens, kv_heads, vdim)[keep_rows].to(cache.v.dtype)

    def mixed_head_attention(self, qkv, layout, batch, cache, scale, window, mix, out):
        heads, kv_heads, dim, vdim = layout
        group = heads // kv_heads
        q_start = batch.q_start.tolist()
        kv_lens = batch.kv_len.tolist()
        ps = cache.page_size
        for s in range(batch.num_seqs):
            begin, end = q_start[s], q_start[s + 1]
            q_len, kv_len = end - begin, kv_lens[s]
            if q_len == 0:
                continue
            first_pos = kv_len - q_len
            low = max(0, first_pos - window + 1) if window > 0 else 0
            low_page = low // ps
            pages = cache.table[s, low_page:-(-kv_len // ps)].long()
            keys = cache.k[pages].permute(1, 0, 2, 3).reshape(kv_heads, -1, dim)
            vals = cache.v[pages].permute(1, 0, 2, 3).reshape(kv_heads, -1, vdim)
            key_pos = torch.arange(low_page * ps, low_page * ps + keys.shape[1], device=qkv.device)
            q = qkv[begin:end, :heads * dim].view(q_len, heads, dim).to(self.acc)
            q_pos = torch.arange(first_pos, kv_len, device=qkv.device)
            hidden = (key_pos[None, :] > q_pos[:, None]) | (key_pos[None, :] >= kv_len)
            if window > 0:
                hidden = hidden | (key_pos[None, :] <= q_pos[:, None] - window)
            keys = keys.to(self.acc).repeat_interleave(group, dim=0)
            vals = vals.to(self.acc).repeat_interleave(group, dim=0)
            scores = torch.einsum("qhd,hkd->hqk", q, keys) * scale
            scores = scores.masked_fill(hidden[None], float("-inf"))
            weights = torch.nan_to_num(torch.softmax(scores, dim=-1))
            if mix is not None:
                weights = torch.einsum("hg,gqk->hqk", mix.to(self.acc), weights)
            vals = torch.where(hidden.all(0)[None, :, None], torch.zeros_like(vals), vals)
            o = torch.einsum("hqk,hkd->qhd", weights, vals)
            out[begin:end] = o.reshape(q_len, heads * vdim).to(out.dtype)

    # ---------------------------------------------------------------- sampling

    def argmax(self, logits, out):
        out.copy_(torch.argmax(logits, dim=-1).to(out.dtype))

    def sample(self, logits, temperature, top_p, u, out):
        """Row by row: greedy where temperature <= 0 (lowest index on ties); otherwise
        softmax(logits / max(T, 1e-5)), keep the tokens whose strictly-more-probable
        predecessors hold at most top_p, renormalise, and take the first index whose
        cumulative probability exceeds u."""
        for row in range(logits.shape[0]):
            t = float(temperature[row])
            if t <= 0.0:
                out[row] = int(torch.argmax(logits[row]))
                continue
            probs = torch.softmax(logits[row].double() / max(t, 1e-5), dim=-1)
            p = float(top_p[row])
            if p < 1.0:
                ordered, index = probs.sort(descending=True)
                before = ordered.cumsum(-1) - ordered
                # ties are kept or dropped together: mass of strictly larger values
                first_of_value = torch.searchsorted(-ordered, -ordered, right=False)
                before = before[first_of_value]
                probs = torch.zeros_like(probs).scatter_(0, index, ordered.masked_fill(before > p, 0.0))
            cdf = probs.cumsum(-1)
            target = float(u[row]) * float(cdf[-1])
            choice = int(torch.searchsorted(cdf, torch.tensor(target, dtype=cdf.dtype), right=True))
            out[row] = min(choice, logits.shape[1] - 1)
