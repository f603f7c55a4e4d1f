"""Plain PyTorch statement of every kernel's contract, on any device.

Two uses: the GPU tests compare each CUDA kernel with the function of the same name
here, and the CPU tests hand this table to the engine in place of the CUDA one so
that the cache manager, the batch packing and the step function can be checked
without a GPU.  It is test code: the engine itself has no such path.  All math is
done in float32 (float64 where `wide` is set) and rounded once to the output dtype.
"""
from __future__ import annotations

import math

import torch


class PlainKernels:
    name = "plain-torch"

    def __init__(self, wide: bool = False):
        self.acc = torch.float64 if wide else torch.float32
        self.launches = 0

    # ------------------------------------------------------------- elementwise
    def embed(self, table, token_ids, vocab):
        return table[token_ids.long()].to(torch.float32)

    def rmsnorm(self, x, w, eps, out_dtype):
        xa = x.to(self.acc)
        y = xa * torch.rsqrt((xa * xa).mean(-1, keepdim=True) + eps) * w.to(self.acc)
        return y.to(out_dtype)

    def add_rmsnorm(self, x, delta, w, eps, out_dtype):
        x += delta.to(torch.float32)
        return self.rmsnorm(x, w, eps, out_dtype)

    def residual_add(self, x, delta):
        x += delta.to(torch.float32)

    def silu_mul(self, gate_up):
        inter = gate_up.shape[1] // 2
        g, u = gate_up[:, :inter].to(self.acc), gate_up[:, inter:].to(self.acc)
        return (g / (1.0 + torch.exp(-g)) * u).to(gate_up.dtype)

    def gather_rows(self, x, rows):
        return x[rows.long()].clone()

    def scatter_i32(self, table, index, value):
        if index.numel():
            table.view(-1)[index.long()] = value

    def relay_i32(self, dst, dst_index, src, src_index):
        if dst_index.numel():
            dst[dst_index.long()] = src[src_index.long()]

    # ------------------------------------------------------------------ linear
    def linear(self, a, w, bias=None, out_dtype=None, allow_partial=False):
        y = a.to(self.acc) @ w.to(self.acc).t()
        if bias is not None:
            y = y + bias.to(self.acc)
        return y.to(out_dtype or a.dtype)

    linear_generic = linear

    def linear_swiglu(self, a, w_gate_up):
        return self.silu_mul(self.linear(a, w_gate_up))

    def materialize(self, value, bias=None):
        return value if bias is None else value + bias.to(value.dtype)

    # --------------------------------------------------------------- attention
    def rope_append(self, qkv, bias, rotary, nq, nkv, d, ctx, cache):
        T = qkv.shape[0]
        x = qkv.to(self.acc)
        if bias is not None:
            x = x + bias.to(self.acc)
        x = x.view(T, nq + 2 * nkv, d)
        pos = ctx.positions.long()
        if rotary is not None:
            rot = rotary.rotary_dim
            ang = pos.to(torch.float32)[:, None] * rotary.inv_freq[None, :].to(torch.float32)
            cos, sin = torch.cos(ang).to(self.acc)[:, None, :], torch.sin(ang).to(self.acc)[:, None, :]
            qk = x[:, :nq + nkv, :rot]
            if rotary.interleaved:
                a, b = qk[..., 0::2], qk[..., 1::2]
                turned = torch.stack([a * cos - b * sin, a * sin + b * cos], dim=-1).flatten(-2)
            else:
                a, b = qk[..., :rot // 2], qk[..., rot // 2:]
                turned = torch.cat([a * cos - b * sin, a * sin + b * cos], dim=-1)
            x = x.clone()
            x[:, :nq + nkv, :rot] = turned
        x = x.to(qkv.dtype)
        if cache.writes and cache.kv is not None:
            P = cache.page_size
            slot = ctx.req_slot.long()[ctx.token_req.long()]
            page = cache.block_table[slot, pos // P].long()
            off = pos % P
            cache.kv[page, 0, :, off, :] = x[:, nq:nq + nkv, :].to(cache.kv.dtype)
            cache.kv[page, 1, :, off, :] = x[:, nq + nkv:, :].to(cache.kv.dtype)
        return x[:, :nq, :].reshape(T, nq * d).contiguous()

    def attention(self, q, nq, nkv, d, window, scale, ctx, cache):
        T = q.shape[0]
        P = cache.page_size
        out = torch.empty((T, nq, d), dtype=q.dtype, device=q.device)
        qv = q.view(T, nq, d).to(self.acc)
        pos_all = ctx.positions.tolist()
        req_all = ctx.token_req.tolist()
        slots = ctx.req_slot.tolist()
        group = nq // nkv
        for t in range(T):
            pos, slot = pos_all[t], slots[req_all[t]]
            first = max(0, pos - window + 1) if window else 0
            keys = torch.arange(first, pos + 1, device=q.device)
            pages = cache.block_table[slot, keys // P].long()
            K = cache.kv[pages, 0, :, keys % P, :].to(self.acc)          # [n, nkv, d]
            V = cache.kv[pages, 1, :, keys % P, :].to(self.acc)
            for h in range(nq):
                g = h // group
                s = (K[:, g, :] @ qv[t, h]) * scale
                p = torch.softmax(s, dim=0)
                out[t, h] = (p @ V[:, g, :]).to(q.dtype)
        return out.reshape(T, nq * d)

    # ---------------------------------------------------------------- sampling
    def argmax(self, logits):
        return torch.argmax(logits, dim=-1).to(torch.int32)

    def penalties(self, logits, tokens, counts, rep, freq, pres):
        R = logits.shape[0]
        for r in range(R):
            for tok, cnt in zip(tokens[r].tolist(), counts[r].tolist()):
                if tok < 0 or cnt <= 0:
                    continue
                v = logits[r, tok]
                v = v / rep[r] if v > 0 else v * rep[r]
                logits[r, tok] = v - freq[r] * cnt - pres[r]

    def logit_bias(self, logits, rows, tokens, bias):
        for r, t, b in zip(rows.tolist(), tokens.tolist(), bias.tolist()):
            logits[r, t] += b

    def sample(self, logits, temperature, top_k, top_p, min_p, seed_lo, seed_hi, step, features=3):
        R, V = logits.shape
        out = torch.empty((R,), dtype=torch.int32, device=logits.device)
        for r in range(R):
            t = float(temperature[r])
            if not t > 0:
                out[r] = int(torch.argmax(logits[r]))
                continue
            p = torch.softmax(logits[r].to(torch.float32) / t, dim=-1)
            keep = kept_mask(p, int(top_k[r]), float(top_p[r]), float(min_p[r]))
            u = philox_uniform(int(seed_lo[r]), int(seed_hi[r]), int(step[r]))
            kept = torch.where(keep, p, torch.zeros_like(p)).to(torch.float64)
            c = torch.cumsum(kept, 0)
            target = u * float(c[-1])
            idx = int(torch.searchsorted(c, torch.tensor(target, dtype=torch.float64), right=True))
            idx = min(idx, V - 1)
            while not bool(keep[idx]):
                idx -= 1
            out[r] = idx
        return out


def kept_mask(p, top_k, top_p, min_p):
    """Which probabilities survive top-k, then min-p, then the nucleus (ties at a
    threshold are kept)."""
    V = p.numel()
    thr = 0.0
    if 0 < top_k < V:
        thr = float(torch.topk(p, top_k).values[-1])
    if min_p > 0:
        thr = max(thr, min_p * float(p.max()))
    keep = p >= thr
    if 0 < top_p < 1:
        kept = torch.where(keep, p, torch.zeros_like(p))
        need = top_p * float(kept.sum())
        vals, _ = torch.sort(kept, descending=True)
        c = torch.cumsum(vals, 0)
        n = int(torch.searchsorted(c, torch.tensor(need, dtype=c.dtype))) + 1
        n = min(n, V)
        thr = max(thr, float(vals[n - 1]))
        keep = p >= thr
    return keep


def philox_uniform(key0, key1, c0, c1=0, c2=0, c3=0):
    """First word of Philox4x32-10 as a float in [0, 1) with 24 bits."""
    M0, M1, W0, W1 = 0xD2511F53, 0xCD9E8D57, 0x9E3779B9, 0xBB67AE85
    mask = 0xFFFFFFFF
    key0, key1, c0, c1, c2, c3 = (v & mask for v in (key0, key1, c0, c1, c2, c3))
    for _ in range(10):
        p0, p1 = M0 * c0, M1 * c2
        hi0, lo0, hi1, lo1 = p0 >> 32, p0 & mask, p1 >> 32, p1 & mask
        c0, c1, c2, c3 = (hi1 ^ c1 ^ key0) & mask, lo1, (hi0 ^ c3 ^ key1) & mask, lo0
        key0, key1 = (key0 + W0) & mask, (key1 + W1) & mask
    return (c0 >> 8) / 16777216.0
