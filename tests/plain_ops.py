"""Plain torch restatements of every kernel, with the kernels' own signatures.

Two uses: the ``-m gpu`` tests compare each CUDA kernel with the function of the same name
here, and the CPU tests put this class in the place of the CUDA kernel set so that the
engine's bookkeeping (batches, block tables, slots, the scheduler) can be run without a GPU.
It is test code: the engine itself never falls back to it.
"""

from __future__ import annotations

import torch


class PlainOps:
    name = "plain"

    def __init__(self, device="cpu"):
        self.device = torch.device(device)
        self.launches = 0
        # stands in for the kernels' device flag: a test sets it to see the engine react
        self.error_flag = torch.zeros(1, dtype=torch.int32, device=self.device)

    def describe_error(self, code):
        return RuntimeError(f"a kernel reported code {code}")

    def check_errors(self):
        code = int(self.error_flag.item())
        if code:
            self.error_flag.zero_()
            raise self.describe_error(code)

    def check_attention_sizes(self, heads, kv_heads, head_dim):
        assert heads % kv_heads == 0

    def embedding(self, ids, table):
        return table[ids.long()].float()

    def add_rmsnorm(self, residual, delta, weight, eps, dtype, delta_scale=1.0):
        if delta is not None:
            residual += delta.float() * delta_scale
        inv = torch.rsqrt(residual.pow(2).mean(dim=-1, keepdim=True) + eps)
        return (residual * inv * weight).to(dtype)

    def gather_rows(self, residual, delta, rows):
        index = rows.long()
        return residual[index].clone(), None if delta is None else delta[index].clone()

    def linear(self, a, w, bias=None, out_dtype=None):
        out = a.float() @ w.float().T
        if out_dtype != torch.float32:
            out = out.to(a.dtype).float()
        if bias is not None:
            out = out + bias
        return out.to(out_dtype or a.dtype)

    def linear_swiglu(self, a, gate_up):
        return self.swiglu(self.linear(a, gate_up))

    def linear_add(self, a, w, bias, residual, scale=1.0):
        return self.linear(a, w, bias)      # (the caller adds it, with its factor)

    def linear_gated(self, a, gate_up, kind):
        both = self.linear(a, gate_up)
        width = both.shape[1] // 2
        return (self.activation(both[:, :width], kind).float() * both[:, width:].float()).to(a.dtype)

    def swiglu(self, gate_up):
        width = gate_up.shape[1] // 2
        gate, up = gate_up[:, :width].float(), gate_up[:, width:].float()
        return (gate / (1 + torch.exp(-gate)) * up).to(gate_up.dtype)

    def short_conv(self, bcx, *, kernel, bias, taps, ctx, view, write):
        hidden = bcx.shape[1] // 3
        dtype = bcx.dtype
        gate_b, gate_c, x = bcx[:, :hidden].float(), bcx[:, hidden:2 * hidden].float(), \
            bcx[:, 2 * hidden:].float()
        g = (gate_b * x).to(dtype).float()
        out = torch.empty_like(g)
        starts = ctx.request_start.tolist()
        history = ctx.history.tolist()
        slots = view.slots.tolist()
        for r in range(ctx.requests):
            first, last = starts[r], starts[r + 1]
            n = last - first
            state = view.state[slots[r]].float()                    # [taps-1, hidden]
            if taps > 1:
                valid = torch.arange(taps - 1) + history[r] - (taps - 1) >= 0
                state = state * valid[:, None].to(state.dtype)
                padded = torch.cat((state[:taps - 1], g[first:last]), dim=0)
            else:
                padded = g[first:last]
            y = torch.zeros(n, hidden)
            for k in range(taps):
                y = y + padded[k:k + n] * kernel[:, k]
            if bias is not None:
                y = y + bias
            out[first:last] = gate_c[first:last] * y
            if write and taps > 1:
                view.state[slots[r]][:taps - 1] = padded[n:n + taps - 1].to(view.state.dtype)
        return out.to(dtype)

    def linear_short_conv(self, a, w, w_bias, *, kernel, bias, taps, ctx, view, write):
        return self.short_conv(self.linear(a, w, w_bias), kernel=kernel, bias=bias, taps=taps,
                               ctx=ctx, view=view, write=write)

    def qk_norm_rope_store(self, qkv, *, heads, kv_heads, head_dim, q_weight, k_weight, eps,
                           rotary, ctx, view, write, value_dim=None, amplitude=1.0,
                           norm_after=False):
        tokens = qkv.shape[0]
        dtype = qkv.dtype
        value_dim = value_dim or head_dim
        row_dim = view.kv.shape[-1]
        flat = qkv.float()
        q = flat[:, :heads * head_dim].view(tokens, heads, head_dim)
        k = flat[:, heads * head_dim:(heads + kv_heads) * head_dim].view(tokens, kv_heads, head_dim)
        v = flat[:, (heads + kv_heads) * head_dim:].view(tokens, kv_heads, value_dim)

        def norm(x, weight):
            if weight is None and not norm_after:
                return x
            x = x * torch.rsqrt(x.pow(2).mean(dim=-1, keepdim=True) + eps)
            return x if weight is None else x * weight

        def rotate(x):
            if rotary is None:
                return x
            inv_freq, rotary_dim = rotary
            half = rotary_dim // 2
            angles = ctx.positions.float()[:, None] * inv_freq[None, :]
            cos = (torch.cos(angles) * amplitude)[:, None, :]
            sin = (torch.sin(angles) * amplitude)[:, None, :]
            a, b = x[..., :half], x[..., half:rotary_dim]
            return torch.cat((a * cos - b * sin, b * cos + a * sin, x[..., rotary_dim:]), dim=-1)

        pad = lambda x: torch.nn.functional.pad(x, (0, row_dim - x.shape[-1]))
        if norm_after:
            q, k = norm(rotate(q), None), norm(rotate(k), None)
        else:
            q, k = rotate(norm(q, q_weight)), rotate(norm(k, k_weight))
        q, k, v = pad(q).to(dtype), pad(k).to(dtype), pad(v).to(dtype)
        if write:
            positions = ctx.positions.tolist()
            requests = ctx.token_request.tolist()
            table = view.block_table.tolist()
            for t in range(tokens):
                page = table[requests[t]][positions[t] // view.page_size]
                assert page >= 0, "a key is written to a position without a page"
                offset = positions[t] % view.page_size
                view.kv[0, page, :, offset] = k[t]
                view.kv[1, page, :, offset] = v[t]
        return q.contiguous()

    def qkv_attention(self, qkv, *, heads, kv_heads, head_dim, q_weight, k_weight, eps, rotary,
                      scale, window, ctx, view, write, sinks=None, chunk=None, keep_first=0,
                      **extra):
        q = self.qk_norm_rope_store(qkv, heads=heads, kv_heads=kv_heads, head_dim=head_dim,
                                    q_weight=q_weight, k_weight=k_weight, eps=eps, rotary=rotary,
                                    ctx=ctx, view=view, write=write, **extra)
        return self.paged_attention(q, heads=heads, kv_heads=kv_heads, head_dim=view.kv.shape[-1],
                                    scale=scale, window=window, ctx=ctx, view=view, sinks=sinks,
                                    chunk=chunk, keep_first=keep_first)

    def concat_stream(self, residual, delta, token_ids, table, dtype, delta_scale=1.0):
        stream = residual if delta is None else residual + delta.float() * delta_scale
        return torch.cat([stream.to(dtype), table[token_ids.long()].to(dtype)], dim=1)

    def softcap(self, logits, cap):
        logits.copy_(cap * torch.tanh(logits / cap))

    def route_experts(self, x, router, *, experts, top, groups, keep, group_score):
        scores = torch.sigmoid(x.float() @ router.T)
        tokens, per = scores.shape[0], experts // groups
        weights = torch.zeros_like(scores)
        for t in range(tokens):
            row = scores[t]
            best = sorted(range(groups), key=lambda g: (
                -float(row[g * per:(g + 1) * per].topk(min(group_score, per)).values.sum()), g))[:keep]
            allowed = [e for e in range(experts) if e // per in best]
            chosen = sorted(allowed, key=lambda e: (-float(row[e]), e))[:top]
            total = sum(float(row[e]) for e in chosen) + 1e-20
            for e in chosen:
                weights[t, e] = float(row[e]) / total
        return weights

    def scale_expert_columns(self, gated, weights, width, tail=None):
        experts = weights.shape[1]
        scaled = gated[:, :experts * width].float().view(-1, experts, width) * weights[:, :, None]
        gated[:, :experts * width] = scaled.view(-1, experts * width).to(gated.dtype)
        if tail is not None:
            rest = gated[:, experts * width:].float() * tail[:, None]
            gated[:, experts * width:] = rest.to(gated.dtype)

    def lightning_attention(self, projected, *, decay, norm_weight, eps, ctx, view, write, heads,
                            key_dim, value_dim):
        tokens = projected.shape[0]
        qk, inner = heads * key_dim, heads * value_dim
        flat = projected.float()
        silu = lambda z: z / (1 + torch.exp(-z))
        q = silu(flat[:, :qk]).view(tokens, heads, key_dim)
        k = silu(flat[:, qk:2 * qk]).view(tokens, heads, key_dim)
        v = silu(flat[:, 2 * qk:2 * qk + inner]).view(tokens, heads, value_dim)
        gate = torch.sigmoid(flat[:, 2 * qk + inner:])
        out = torch.empty(tokens, heads, value_dim)
        starts, slots = ctx.request_start.tolist(), view.slots.tolist()
        for r in range(ctx.requests):
            state = view.state[slots[r]].view(heads, key_dim, value_dim).clone()
            for t in range(starts[r], starts[r + 1]):
                state = decay[:, None, None] * state + k[t][:, :, None] * v[t][:, None, :]
                out[t] = torch.einsum("hdv,hd->hv", state, q[t])
            if write:
                view.state[slots[r]] = state.reshape(-1)
        out = out.reshape(tokens, inner)
        out = out * torch.rsqrt(out.pow(2).mean(dim=-1, keepdim=True) + eps) * norm_weight * gate
        return out.to(projected.dtype)

    def add_vectors(self, residual, delta, token_ids, table, vector, delta_scale=1.0):
        if delta is not None:
            residual += delta.float() * delta_scale
        if table is not None:
            residual += table[token_ids.long()].float()
        if vector is not None:
            residual += vector

    def activation(self, x, kind, params=None):
        z = x.float()
        if kind == "xielu":
            above, below = params
            out = torch.where(z > 0, above * z * z + 0.5 * z,
                              below * (torch.expm1(torch.clamp(z, max=0.0)) - z) + 0.5 * z)
        elif kind == "relu2":
            out = torch.relu(z) ** 2
        elif kind == "relu":
            out = torch.relu(z)
        elif kind == "silu":
            out = z / (1 + torch.exp(-z))
        elif kind == "gelu_tanh":
            out = 0.5 * z * (1 + torch.tanh(0.7978845608028654 * (z + 0.044715 * z ** 3)))
        else:
            raise ValueError(kind)
        return out.to(x.dtype)

    def linear_act(self, a, w, kind, params=None):
        return self.activation(self.linear(a, w), kind, params)

    # ---- the stream's first value, the streams kept over the layers, convolutions over time

    def embedding_pairs(self, ids, table, scale, pairs, *, rule, ctx, view, out=None):
        x = table[ids.long()].float() * scale
        if pairs is not None:
            buckets, mul_prev, mul_cur = rule
            tokens = ids.tolist()
            starts, slots = ctx.request_start.tolist(), view.slots.tolist()
            rows = []
            for r in range(ctx.requests):
                before = int(view.state[slots[r], 0]) - 1          # -1: the sequence starts here
                for t in range(starts[r], starts[r + 1]):
                    rows.append(buckets if before < 0
                                else (before * mul_prev + tokens[t] * mul_cur) % buckets)
                    before = tokens[t]
                view.state[slots[r], 0] = before + 1
            x = x + pairs[torch.tensor(rows, dtype=torch.long)].float()
        if out is None:
            return x
        out.copy_(x)
        return out

    def stream_average(self, kept, weights, count, out):
        if weights is None:
            out.copy_(kept[0])
        else:
            out.copy_((kept[:count] * weights[:count, None, None]).sum(dim=0))
        return out

    def stream_conv(self, residual, kernel, *, taps, ctx, view, sublayer, write, dtype):
        if kernel is None or taps < 1:
            return residual.to(dtype)
        out = torch.empty_like(residual)
        starts = ctx.request_start.tolist()
        slots = view.slots.tolist() if view is not None else None
        for r in range(ctx.requests):
            first, last = starts[r], starts[r + 1]
            n = last - first
            rows = residual[first:last]
            if taps > 1:
                state = view.state[slots[r], sublayer]                 # [taps - 1, hidden]
                padded = torch.cat((state, rows), dim=0)
            else:
                padded = rows
            y = rows.clone()
            for j in range(taps):
                y = y + padded[j:j + n] * kernel[:, j]
            out[first:last] = y
            if write and taps > 1:
                view.state[slots[r], sublayer] = padded[n:n + taps - 1]
        return out.to(dtype)

    # ---- attention over one latent row per token

    def latent_prepare(self, projected, queries, *, heads, head_dim, rot_dim, latent, norm_weight,
                       eps, rotary, neighbours, ctx, view, write):
        tokens = projected.shape[0]
        flat = projected.float()
        per_head = head_dim + rot_dim
        q_rot = flat[:, :heads * per_head].view(tokens, heads, per_head)[:, :, head_dim:]
        down = flat[:, heads * per_head:heads * per_head + latent + rot_dim]
        c = down[:, :latent]
        c = c * torch.rsqrt(c.pow(2).mean(dim=-1, keepdim=True) + eps) * norm_weight
        shared = down[:, latent:]

        def rotate(x):
            if rotary is None:
                return x
            inv_freq, dims = rotary
            angles = ctx.positions.float()[:, None] * inv_freq[None, :]
            cos, sin = torch.cos(angles), torch.sin(angles)
            if x.dim() == 3:
                cos, sin = cos[:, None, :], sin[:, None, :]
            out = x.clone()
            if neighbours:
                a, b = x[..., 0:dims:2], x[..., 1:dims:2]
                out[..., 0:dims:2] = a * cos - b * sin
                out[..., 1:dims:2] = b * cos + a * sin
            else:
                half = dims // 2
                a, b = x[..., :half], x[..., half:dims]
                out[..., :half] = a * cos - b * sin
                out[..., half:dims] = b * cos + a * sin
            return out

        queries[:, :, latent:] = rotate(q_rot).to(queries.dtype)
        row = torch.cat((c, rotate(shared)), dim=1).to(view.kv.dtype)
        if write:
            positions, requests = ctx.positions.tolist(), ctx.token_request.tolist()
            table = view.block_table.tolist()
            for t in range(tokens):
                page = table[requests[t]][positions[t] // view.page_size]
                assert page >= 0, "a row is written to a position without a page"
                view.kv[0, page, 0, positions[t] % view.page_size] = row[t]

    def linear_heads(self, a, w, out=None):
        """a [tokens, heads, K] (rows may be slices) with w [heads, N, K] -> [tokens, heads, N]."""
        result = torch.einsum("thk,hnk->thn", a.float(), w.float()).to(a.dtype).contiguous()
        if out is None:
            return result
        out.copy_(result)
        return out

    def latent_attention(self, queries, *, heads, latent, scale, ctx, view):
        tokens, _, row = queries.shape
        flat = self.paged_attention(queries, heads=heads, kv_heads=1, head_dim=row, scale=scale,
                                    window=None, ctx=ctx, view=view)
        return flat.view(tokens, heads, row)

    def sigmoid_gate(self, values, gate):
        return (values.float() * torch.sigmoid(gate.float())).to(values.dtype)

    def differential_combine(self, maps, *, heads, row_dim, value_dim, mix, eps, factor):
        tokens = maps.shape[0]
        both = maps.float().view(tokens, 2, heads, row_dim)[..., :value_dim]
        o = both[:, 0] - torch.tensor(mix, dtype=torch.float32) * both[:, 1]
        o = o * torch.rsqrt(o.pow(2).mean(dim=-1, keepdim=True) + eps) * factor
        return o.reshape(tokens, heads * value_dim).to(maps.dtype)

    def normed_mean_add(self, residual, outputs, weights, eps):
        total = torch.zeros_like(residual)
        for out, weight in zip(outputs, weights):
            x = out.float()
            total += x * torch.rsqrt(x.pow(2).mean(dim=-1, keepdim=True) + eps) * weight
        residual += total / len(outputs)

    def gated_delta_rule(self, projected, *, conv, a_log, dt_bias, norm_weight, eps, unit_eps, ctx,
                         view, write, heads, kv_heads, key_dim, value_dim, taps):
        tokens = projected.shape[0]
        qk, inner = kv_heads * key_dim, heads * value_dim
        channels = 2 * qk + inner
        matrices = heads * key_dim * value_dim
        flat = projected.float()
        gate = flat[:, channels:channels + inner].view(tokens, heads, value_dim)
        beta = torch.sigmoid(flat[:, channels + inner:channels + inner + heads])
        step = torch.nn.functional.softplus(flat[:, channels + inner + heads:] + dt_bias)
        decay = torch.exp(-torch.exp(a_log) * step)
        out = torch.empty(tokens, heads, value_dim)
        starts, history, slots = ctx.request_start.tolist(), ctx.history.tolist(), view.slots.tolist()
        silu = lambda z: z / (1 + torch.exp(-z))
        unit = lambda x: x / torch.sqrt(x.pow(2).sum(dim=-1, keepdim=True) + unit_eps)
        for r in range(ctx.requests):
            first, last = starts[r], starts[r + 1]
            n = last - first
            slot = view.state[slots[r]]
            state = slot[:matrices].view(heads, key_dim, value_dim).clone()
            ring = slot[matrices:].view(taps, channels)        # row p % taps: input at position p
            before = [history[r] - (taps - 1) + s for s in range(taps - 1)]
            tail = torch.stack([ring[p % taps] if p >= 0 else torch.zeros(channels) for p in before]) \
                if taps > 1 else torch.zeros(0, channels)
            padded = torch.cat((tail, flat[first:last, :channels]), dim=0)
            mixed = sum(padded[j:j + n] * conv[:, j] for j in range(taps))
            mixed = silu(mixed)
            q = unit(mixed[:, :qk].view(n, kv_heads, key_dim)) * key_dim ** -0.5
            k = unit(mixed[:, qk:2 * qk].view(n, kv_heads, key_dim))
            v = mixed[:, 2 * qk:].view(n, heads, value_dim)
            for h in range(heads):
                shared = h // (heads // kv_heads)
                s = state[h]
                for t in range(n):
                    s = decay[first + t, h] * s
                    u = beta[first + t, h] * (v[t, h] - s.T @ k[t, shared])
                    s = s + torch.outer(k[t, shared], u)
                    out[first + t, h] = s.T @ q[t, shared]
                state[h] = s
            if write:
                slot[:matrices] = state.reshape(-1)
                for index in range(max(n - taps, 0), n):
                    ring[(history[r] + index) % taps] = flat[first + index, :channels]
        out = out * torch.rsqrt(out.pow(2).mean(dim=-1, keepdim=True) + eps) * norm_weight
        out = out * silu(gate)
        return out.reshape(tokens, inner).to(projected.dtype)

    def paged_attention(self, q, *, heads, kv_heads, head_dim, scale, window, ctx, view,
                        sinks=None, chunk=None, keep_first=0):
        tokens = q.shape[0]
        out = torch.empty(tokens, heads, head_dim)
        positions = ctx.positions.tolist()
        requests = ctx.token_request.tolist()
        table = view.block_table.tolist()
        group = heads // kv_heads
        for t in range(tokens):
            p = positions[t]
            lowest = max(p - window + 1, 0) if window else 0
            if chunk:
                lowest = max(lowest, p - p % chunk)
            keys = list(range(min(keep_first, lowest))) + list(range(lowest, p + 1))
            pages = [table[requests[t]][key // view.page_size] for key in keys]
            assert min(pages) >= 0, "a key is read from a position without a page"
            offsets = [key % view.page_size for key in keys]
            k = view.kv[0, pages, :, offsets].float()            # [keys, kv_heads, head_dim]
            v = view.kv[view.kv.shape[0] - 1, pages, :, offsets].float()
            k = k.repeat_interleave(group, dim=1)
            v = v.repeat_interleave(group, dim=1)
            scores = torch.einsum("hd,khd->hk", q[t].float(), k) * scale
            if sinks is not None:
                # a column without a key or a value: it only takes its share of the weights
                scores = torch.cat([scores, sinks.float()[:, None]], dim=1)
                v = torch.cat([v, torch.zeros_like(v[:1])], dim=0)
            out[t] = torch.einsum("hk,khd->hd", torch.softmax(scores, dim=-1), v)
        return out.reshape(tokens, heads * head_dim).to(q.dtype)

    def channel_conv(self, rows, kernel, bias, *, taps, activation, ctx, view, write):
        tokens, channels = rows.shape
        dtype = rows.dtype
        flat = rows.float()
        out = torch.empty(tokens, channels)
        starts = ctx.request_start.tolist()
        history = ctx.history.tolist()
        for r in range(ctx.requests):
            first, last = starts[r], starts[r + 1]
            n = last - first
            if taps > 1:
                state = view.state[int(view.slots[r])]                  # [taps - 1, channels]
                valid = torch.arange(taps - 1) + history[r] - (taps - 1) >= 0
                padded = torch.cat((state.float() * valid[:, None], flat[first:last]), dim=0)
            else:
                padded = flat[first:last]
            y = torch.zeros(n, channels)
            for j in range(taps):
                y = y + padded[j:j + n] * kernel[:, j]
            if bias is not None:
                y = y + bias
            out[first:last] = y
            if write and taps > 1:
                state[:] = padded[n:n + taps - 1].to(state.dtype)
        if activation == "silu":
            out = out / (1 + torch.exp(-out))
        elif activation is not None:
            raise ValueError(activation)
        return out.to(dtype)

    def gate_heads(self, mixed, gate, *, heads, row_dim, value_dim, per_head):
        tokens = mixed.shape[0]
        values = mixed.float().view(tokens, heads, row_dim)[:, :, :value_dim]
        g = torch.sigmoid(gate.float())
        g = g.view(tokens, heads, 1) if per_head else g.view(tokens, heads, value_dim)
        return (values * g).reshape(tokens, heads * value_dim).to(mixed.dtype)

    def state_space_scan(self, mixed, steps, *, a_log, dt_bias, skip, ctx, view, write, heads,
                         value_dim, state_dim, groups):
        tokens = mixed.shape[0]
        inner, wide = heads * value_dim, groups * state_dim
        flat = mixed.float()
        x = flat[:, :inner].view(tokens, heads, value_dim)
        b = flat[:, inner:inner + wide].view(tokens, groups, state_dim)
        c = flat[:, inner + wide:].view(tokens, groups, state_dim)
        dt = torch.nn.functional.softplus(steps.float() + dt_bias, threshold=30.0)
        decay = torch.exp(-torch.exp(a_log) * dt)
        out = torch.empty(tokens, heads, value_dim)
        starts, slots = ctx.request_start.tolist(), view.slots.tolist()
        per = heads // groups
        for r in range(ctx.requests):
            state = view.state[slots[r]].view(heads, state_dim, value_dim).clone()
            for t in range(starts[r], starts[r + 1]):
                bt = b[t].repeat_interleave(per, dim=0)              # [heads, state]
                ct = c[t].repeat_interleave(per, dim=0)
                state = decay[t][:, None, None] * state + \
                    (dt[t][:, None] * bt)[:, :, None] * x[t][:, None, :]
                out[t] = torch.einsum("hnp,hn->hp", state, ct) + skip[:, None] * x[t]
            if write:
                view.state[slots[r]] = state.reshape(-1)
        return out.reshape(tokens, inner)

    def gated_group_norm(self, y, gate, weight, *, groups, eps, dtype):
        tokens, inner = y.shape
        z = gate.float()
        v = (y * (z / (1 + torch.exp(-z)))).view(tokens, groups, inner // groups)
        v = v * torch.rsqrt(v.pow(2).mean(dim=-1, keepdim=True) + eps)
        return (v.reshape(tokens, inner) * weight).to(dtype)

    def route_general(self, x, router, correction, *, experts, identity, top, scores, normalize,
                      shared_gate):
        logits = x.float() @ router.T
        outputs = experts + identity
        z = logits[:, :outputs]
        s = torch.softmax(z, dim=-1) if scores == "softmax" else torch.sigmoid(z)
        choice = s if correction is None else s + correction
        tokens = s.shape[0]
        weights = torch.zeros(tokens, outputs)
        for t in range(tokens):
            chosen = sorted(range(outputs), key=lambda e: (-float(choice[t, e]), e))[:top]
            total = sum(float(s[t, e]) for e in chosen) + 1e-20 if normalize else 1.0
            for e in chosen:
                weights[t, e] = float(s[t, e]) / total
        others = torch.zeros(2, tokens)
        others[0] = weights[:, experts:].sum(dim=-1)
        if shared_gate:
            others[1] = torch.sigmoid(logits[:, outputs])
        return weights[:, :experts].contiguous(), others

    def add_scaled_rows(self, out, x, factors):
        out.copy_((out.float() + x.float() * factors[:, None]).to(out.dtype))

    def scale_values(self, values, factor):
        values.mul_(factor)

    def argmax(self, logits):
        return torch.argmax(logits, dim=-1).to(torch.int32)

    def decode_advance(self, chosen, token_ids, positions, history, record, counter):
        token_ids.copy_(chosen)
        positions += 1
        history += 1
        step = int(counter)
        if step < record.shape[0]:
            record[step] = chosen
        counter += 1

    def publish_tokens(self, chosen, index, published):
        published[index.long()] = chosen
        return torch.cat([chosen.to(torch.int32), self.error_flag.to(torch.int32)])

    def resolve_tokens(self, token_ids, source, published):
        taken = source >= 0
        token_ids[taken] = published[source[taken].long()]

    def reserve_sample_scratch(self, rows, vocab):
        pass

    def sample(self, logits, temperature, top_k, top_p, seed, step):
        """Token-order draw over the reference's kept set, in float64."""
        rows, vocab = logits.shape
        out = torch.empty(rows, dtype=torch.int32)
        probabilities = torch.empty(rows, vocab, dtype=torch.float32)
        for r in range(rows):
            if float(temperature[r]) <= 0:                   # greedy row
                out[r] = int(torch.argmax(logits[r]))
                probabilities[r] = 0
                probabilities[r, int(out[r])] = 1
                continue
            scaled = (logits[r] - logits[r].max()) * (1.0 / temperature[r])
            p = torch.exp(scaled.float())
            probabilities[r] = p
            kept = kept_set(p, int(top_k[r]), float(top_p[r]))
            weights = torch.zeros(vocab, dtype=torch.float64)
            weights[kept] = p[kept].double()
            running = torch.cumsum(weights, dim=0)
            target = uniform(int(seed[r]), int(step[r])) * float(weights.sum())
            hit = torch.nonzero((running >= target) & (weights > 0))
            out[r] = int(hit[0]) if len(hit) else int(kept.max())
        return out, probabilities


def kept_set(p, top_k, top_p):
    """Indices that the reference's rule keeps (src/mlx_one/text/sampling.py:56-81): stable
    descending order, first top_k, then the shortest prefix reaching top_p of their mass."""
    order = torch.sort(p.double(), descending=True, stable=True).indices
    if top_k > 0:
        order = order[:top_k]
    ranked = p.double()[order]
    if top_p < 1.0:
        running = torch.cumsum(ranked, dim=0)
        cutoff = top_p * float(ranked.sum())
        count = min(int(torch.searchsorted(running, torch.tensor(cutoff, dtype=torch.float64))) + 1,
                    len(order))
        order = order[:count]
    return order


def uniform(seed, step):
    mask = (1 << 64) - 1
    z = (seed * 0x9E3779B97F4A7C15 + (step + 1) * 0xBF58476D1CE4E5B9) & mask
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & mask
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & mask
    z = z ^ (z >> 31)
    return (z >> 40) / float(1 << 24)
