"""Plain whole-sequence implementation of the Qwen2.5 dense decoder (the oracle).

It restates the reference's formulas, each function citing the lines it restates, and
is held to the reference's own results: tests/test_golden.py compares every function
here, and the whole forward, with outputs of the unmodified reference code (its leaf
host wrappers and its LlamaForwardTyped<T> model path, run once on a GPU by
tests/golden/make_goldens.py and kept under tests/golden/).  The reference has no CPU
model code, so it cannot be imported here.

Whole sequences only: no cache, no batching, no paging.  One function per part.
Weights are a dict name -> torch tensor with HF tensor names; the config is the
dict read from config.json.  Everything is computed in `dtype` (float32 by
default, float64 for a tighter oracle).
"""
from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import torch

# --------------------------------------------------------------------------- IO


_ST_DTYPES = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16,
    "BF16": torch.bfloat16, "I64": torch.int64, "I32": torch.int32,
    "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8, "BOOL": torch.bool,
}


def read_safetensors(path):
    """Own reader of the safetensors layout: 8-byte little-endian header length N,
    N bytes of JSON {name: {dtype, shape, data_offsets}}, then the data section
    (runtime/backends/cuda/native/safetensors_parser.cpp:144-246)."""
    raw = Path(path).read_bytes()
    (n,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + n].decode("utf-8"))
    data = memoryview(raw)[8 + n:]
    out = {}
    for name, info in header.items():
        if name.startswith("__"):
            continue
        b, e = info["data_offsets"]
        dt = _ST_DTYPES[info["dtype"]]
        t = torch.frombuffer(bytearray(data[b:e]), dtype=dt) if e > b else torch.empty(0, dtype=dt)
        out[name] = t.reshape(info["shape"]).clone()
    return out


def load_model_dir(model_dir):
    """(config dict, weights dict) of a folder with config.json + model.safetensors."""
    model_dir = Path(model_dir)
    cfg = json.loads((model_dir / "config.json").read_text())
    return cfg, read_safetensors(model_dir / "model.safetensors")


# ------------------------------------------------------------------------ parts


def head_dim_of(cfg):
    """head_dim if present, else hidden_size / num_attention_heads
    (runtime/backends/cuda/inferflux_cuda_executor.cpp:549-559)."""
    hd = cfg.get("head_dim")
    return int(hd) if hd else cfg["hidden_size"] // cfg["num_attention_heads"]


def layer_window(cfg, layer):
    """Key window of a layer, or None for all keys.  The reference reads none of
    use_sliding_window / sliding_window / max_window_layers (it always attends to
    every key, runtime/backends/cuda/kernels/flash_attention.cu:86); the keys'
    meaning is Qwen2's own: with use_sliding_window the layers from index
    max_window_layers on see only the last `sliding_window` keys."""
    if not cfg.get("use_sliding_window", False):
        return None
    w = cfg.get("sliding_window")
    if w is None:
        return None
    return int(w) if layer >= int(cfg.get("max_window_layers", 0)) else None


def embedding(table, tokens):
    """x0[t,:] = E[token[t],:], no scaling
    (runtime/backends/cuda/native/cuda_kernels.cu:256-270)."""
    return table[tokens.long().to(table.device)]


def rmsnorm(x, w, eps):
    """y = x * rsqrt(mean(x^2) + eps) * w, no "1 + w"
    (runtime/backends/cuda/native/cuda_kernels.cu:26-47)."""
    ms = (x * x).mean(dim=-1, keepdim=True)
    return x * torch.rsqrt(ms + eps) * w


def linear(x, w, b=None):
    """y = x . W^T (+ b); W is [out, in] row-major
    (runtime/backends/cuda/native/cublas_gemm.cpp:104-106; bias
    runtime/backends/cuda/native/cuda_kernels.cu:789-803)."""
    y = x @ w.t()
    return y if b is None else y + b


def rope_neox(x, positions, theta):
    """Split-half rotation of every head of x [T, heads, d]: pair i is
    (x[i], x[i + d/2]), inv_freq_i = 1 / theta^(2i/d), angle = pos * inv_freq_i,
    (a, b) -> (a cos - b sin, a sin + b cos)
    (runtime/backends/cuda/native/cuda_kernels.cu:93-116, rope_type 2)."""
    d = x.shape[-1]
    half = d // 2
    inv_freq = 1.0 / (theta ** (torch.arange(0, d, 2, dtype=torch.float32) / d))
    ang = (positions.to(torch.float32)[:, None] * inv_freq[None, :]).to(x.device)   # fp32 angles, made on the CPU
    cos = torch.cos(ang).to(x.dtype)[:, None, :]
    sin = torch.sin(ang).to(x.dtype)[:, None, :]
    a, b = x[..., :half], x[..., half:]
    return torch.cat([a * cos - b * sin, a * sin + b * cos], dim=-1)


def attention_gqa_causal(q, k, v, window=None):
    """q [T, nq, d], k/v [T, nkv, d] of one whole sequence.  Query head h uses KV
    head h // (nq/nkv); score = q.k / sqrt(d); query t sees keys j <= t (and
    j > t - window when a window is given); softmax over the seen keys
    (runtime/backends/cuda/kernels/flash_attention.cu:71-86, 152-172)."""
    T, nq, d = q.shape
    nkv = k.shape[1]
    group = nq // nkv
    scale = 1.0 / math.sqrt(d)
    out = torch.zeros_like(q)
    idx = torch.arange(T, device=q.device)
    seen = idx[None, :] <= idx[:, None]
    if window is not None:
        seen &= idx[None, :] > (idx[:, None] - window)
    for h in range(nq):
        g = h // group
        s = (q[:, h, :] @ k[:, g, :].t()) * scale
        s = s.masked_fill(~seen, float("-inf"))
        p = torch.softmax(s, dim=-1)
        out[:, h, :] = p @ v[:, g, :]
    return out


def silu(g):
    """silu(g) = g / (1 + exp(-g)) (runtime/backends/cuda/native/cuda_kernels.cu:147-150)."""
    return g / (1.0 + torch.exp(-g))


def swiglu_mlp(x, wg, wu, wd):
    """(silu(x Wg^T) * (x Wu^T)) Wd^T, no biases
    (runtime/backends/cuda/native/transformer_forward.cu:2384-2535)."""
    return linear(silu(linear(x, wg)) * linear(x, wu), wd)


def attention_block(x, W, cfg, layer, positions):
    """Projections with optional q/k/v bias, rotation of q and k after the bias,
    attention, output projection (transformer_forward.cu:1945-2185)."""
    p = f"model.layers.{layer}.self_attn."
    nq, nkv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], head_dim_of(cfg)
    T = x.shape[0]
    q = linear(x, W[p + "q_proj.weight"], W.get(p + "q_proj.bias")).view(T, nq, d)
    k = linear(x, W[p + "k_proj.weight"], W.get(p + "k_proj.bias")).view(T, nkv, d)
    v = linear(x, W[p + "v_proj.weight"], W.get(p + "v_proj.bias")).view(T, nkv, d)
    theta = float(cfg.get("rope_theta", 10000.0))
    q = rope_neox(q, positions, theta)
    k = rope_neox(k, positions, theta)
    a = attention_gqa_causal(q, k, v, layer_window(cfg, layer))
    return linear(a.reshape(T, nq * d), W[p + "o_proj.weight"])


def decoder_layer(x, W, cfg, layer, positions):
    """Pre-norm block: x += attn(norm_in(x)); x += mlp(norm_post(x))
    (runtime/backends/cuda/native/llama_forward.h:88-90)."""
    p = f"model.layers.{layer}."
    eps = float(cfg.get("rms_norm_eps", 1e-6))
    x = x + attention_block(rmsnorm(x, W[p + "input_layernorm.weight"], eps), W, cfg, layer, positions)
    m = rmsnorm(x, W[p + "post_attention_layernorm.weight"], eps)
    x = x + swiglu_mlp(m, W[p + "mlp.gate_proj.weight"], W[p + "mlp.up_proj.weight"],
                       W[p + "mlp.down_proj.weight"])
    return x


def lm_head(x, W, cfg):
    """logits = norm_f(x) . W_lm^T; W_lm is lm_head.weight unless the embeddings
    are tied (runtime/backends/cuda/native/weight_map.cpp:33-37; final norm
    transformer_forward.cu:2617-2693)."""
    eps = float(cfg.get("rms_norm_eps", 1e-6))
    n = rmsnorm(x, W["model.norm.weight"], eps)
    if cfg.get("tie_word_embeddings", False) or "lm_head.weight" not in W:
        return linear(n, W["model.embed_tokens.weight"])
    return linear(n, W["lm_head.weight"])


def forward(cfg, weights, tokens, dtype=torch.float32):
    """Logits [T, vocab] of one whole sequence of token ids."""
    W = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in weights.items()}
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    positions = torch.arange(tokens.numel())
    x = embedding(W["model.embed_tokens.weight"], tokens)
    for layer in range(cfg["num_hidden_layers"]):
        x = decoder_layer(x, W, cfg, layer, positions)
    return lm_head(x, W, cfg)


def greedy_generate(cfg, weights, prompt, n_new, dtype=torch.float32):
    """Greedy continuation by recomputing the whole sequence each step; ties go to
    the lowest index (runtime/backends/cuda/native/gpu_sampler.cu:124-156)."""
    seq = list(prompt)
    for _ in range(n_new):
        logits = forward(cfg, weights, seq, dtype)[-1]
        seq.append(int(torch.argmax(logits)))
    return seq[len(prompt):]
