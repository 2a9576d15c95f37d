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

    def embed(self, token_ids, table, out):
        out.copy_(table[token_ids.long()].to(out.dtype))

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
