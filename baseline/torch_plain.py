"""The dense decoder in plain PyTorch (matmul + scaled_dot_product_attention): a timed
baseline on the same GPU and the yardstick `bench.py` checks the engine's logits with.

Not part of the engine: nothing under inferflux_b200/ imports it.  It borrows the
engine's loaded weight tensors (stacked q/k/v and gate/up as the parts keep them) so that
no second copy of a 15 GB model is made, and runs them with library kernels only.
Formulas as in runtime/backends/cuda/native/transformer_forward.cu:1677-2700 of the
reference (pre-norm blocks, bias before the split-half rotation, SwiGLU).
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F


class TorchPlain:
    def __init__(self, model, compute_dtype=torch.bfloat16):
        """`model`: a loaded inferflux_b200 Model whose layers are attention + SwiGLU blocks."""
        self.model = model
        self.dt = compute_dtype
        a = model.layers[0].mixer
        self.nq, self.nkv, self.d = a.nq, a.nkv, a.d
        self.eps = model.final_norm.eps
        self.inv_freq = a.position.rotary(model.device).inv_freq.float()
        self.k_cache = self.v_cache = None

    # ------------------------------------------------------------------ parts
    def _w(self, t):
        return t if t.dtype == self.dt else t.to(self.dt)

    def _norm(self, x, w):
        xf = x.float()
        return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.eps) * w.float()).to(self.dt)

    def _rope(self, x, pos):
        """x [..., T, heads, d]; pos [..., T]."""
        ang = pos.float()[..., None] * self.inv_freq                      # [..., T, d/2]
        cos, sin = ang.cos()[..., None, :], ang.sin()[..., None, :]
        a, b = x.float()[..., : self.d // 2], x.float()[..., self.d // 2:]
        return torch.cat([a * cos - b * sin, a * sin + b * cos], -1).to(self.dt)

    def _layer(self, x, layer, pos, attend):
        """x float32 [B, T, H]; `attend(q, k, v)` with q [B, T, nq, d], k/v [B, T, nkv, d] -> [B, T, nq d]."""
        m, f = layer.mixer, layer.ffn
        B, T, _ = x.shape
        h = self._norm(x, layer.norm_mixer.weight)
        qkv = h @ self._w(m.w_qkv).t()
        if m.b_qkv is not None:
            qkv = (qkv.float() + m.b_qkv).to(self.dt)
        q, k, v = qkv.split([self.nq * self.d, self.nkv * self.d, self.nkv * self.d], -1)
        q = self._rope(q.view(B, T, self.nq, self.d), pos)
        k = self._rope(k.view(B, T, self.nkv, self.d), pos)
        a = attend(q, k, v.reshape(B, T, self.nkv, self.d))
        x = x + (a @ self._w(m.w_o).t()).float()
        h = self._norm(x, layer.norm_ffn.weight)
        gu = h @ self._w(f.w_gate_up).t()
        g, u = gu.split(f.inter, -1)
        act = (F.silu(g.float()) * u.float()).to(self.dt)
        return x + (act @ self._w(f.w_down).t()).float()

    def _head(self, x):
        h = self._norm(x, self.model.final_norm.weight)
        return (h @ self._w(self.model.lm_head.weight).t()).float()

    # -------------------------------------------------------- whole sequences
    @torch.no_grad()
    def logits_last(self, tokens, last=1):
        """float32 logits [last, vocab] of the final `last` positions of one whole sequence."""
        ids = torch.as_tensor(tokens, dtype=torch.long, device=self.model.device)[None]
        pos = torch.arange(ids.shape[1], device=ids.device)[None]
        x = self.model.embedding.table[ids].float()

        def attend(q, k, v):
            o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2),
                                               is_causal=True, enable_gqa=True)
            return o.transpose(1, 2).reshape(q.shape[0], q.shape[1], -1)

        for e in self.model.plan.schedule:
            x = self._layer(x, self.model.layers[e.layer], pos, attend)
        return self._head(x[0, -last:])

    # ------------------------------------------------------------ with a cache
    def make_cache(self, batch, max_len):
        L = len(self.model.plan.schedule)
        shape = (L, batch, self.nkv, max_len, self.d)
        self.k_cache = torch.zeros(shape, dtype=self.dt, device=self.model.device)
        self.v_cache = torch.zeros(shape, dtype=self.dt, device=self.model.device)

    @torch.no_grad()
    def step(self, ids, start):
        """ids [B, T] at positions start..start+T-1 of every sequence (all at the same length):
        stores their keys and values and returns float32 logits [B, vocab] of the last position."""
        B, T = ids.shape
        pos = (start + torch.arange(T, device=ids.device))[None].expand(B, T)
        x = self.model.embedding.table[ids].float()
        end = start + T
        for li, e in enumerate(self.model.plan.schedule):
            def attend(q, k, v, li=li):
                self.k_cache[li, :, :, start:end] = k.transpose(1, 2)
                self.v_cache[li, :, :, start:end] = v.transpose(1, 2)
                kk, vv = self.k_cache[li, :, :, :end], self.v_cache[li, :, :, :end]
                if T == 1:
                    o = F.scaled_dot_product_attention(q.transpose(1, 2), kk, vv, enable_gqa=True)
                else:
                    mask = torch.ones(T, end, dtype=torch.bool, device=q.device).tril(start)
                    o = F.scaled_dot_product_attention(q.transpose(1, 2), kk, vv, attn_mask=mask, enable_gqa=True)
                return o.transpose(1, 2).reshape(B, T, -1)
            x = self._layer(x, self.model.layers[e.layer], pos, attend)
        return self._head(x[:, -1])


def time_torch_plain(model, vocab, batch, context, prefill_tokens, steps=10, warmup=3):
    """(decode ms per step at `batch` x `context`, prefill ms for `prefill_tokens`) of the plain PyTorch model."""
    tp = TorchPlain(model)
    dev = model.device
    g = torch.Generator(device="cpu").manual_seed(5)
    tp.make_cache(1, prefill_tokens)
    ids = torch.randint(0, vocab, (1, prefill_tokens), generator=g).to(dev)
    times = []
    for i in range(2 + 3):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        s.record()
        tp.step(ids, 0)
        e.record()
        torch.cuda.synchronize()
        if i >= 2:
            times.append(s.elapsed_time(e))
    prefill_ms = sorted(times)[len(times) // 2]
    tp.make_cache(batch, context)
    tp.k_cache.normal_(0, 1)
    tp.v_cache.normal_(0, 1)
    start = context - (steps + warmup)
    feed = torch.randint(0, vocab, (steps + warmup, batch, 1), generator=g).to(dev)
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for i in range(steps + warmup):
        if i == warmup:
            torch.cuda.synchronize()
            s.record()
        tp.step(feed[i], start + i).argmax(-1)
    e.record()
    torch.cuda.synchronize()
    tp.k_cache = tp.v_cache = None
    return s.elapsed_time(e) / steps, prefill_ms
