#!/usr/bin/env python3
"""Makes the golden files of this folder by RUNNING the reference's own code.

`baseline/_ref/ref_harness` (built by baseline/build_ref.py from the unmodified
reference sources) is called on small inputs made here:

  reference_leaf.npz    inputs and outputs of single host wrappers
                        (RmsNorm, ResidualAddRmsNormMixed, RoPE with rope_type 2,
                        BatchedRoPE with the bias fold, SiluMul, BiasAddTriple,
                        FlashAttention2Typed, FlashDecodeMultiSeqStrided), in
                        float16 and bfloat16
  reference_model.npz   weights, token ids and the logits that the reference's
                        LlamaForwardTyped<T> (Forward and BatchForward) gives for
                        two tiny random models, in float16 and bfloat16

    python tests/golden/make_goldens.py          (needs a GPU; run from the repository root)

tests/test_golden.py (no GPU) checks that tests/plain/plain_qwen2.py reproduces
them.  16-bit tensors are stored as uint16 bit patterns with the dtype in the key
(`.../f16` or `.../bf16`); everything else as is.
"""
from __future__ import annotations

import subprocess
import sys
import tempfile
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
HARNESS = ROOT / "baseline" / "_ref" / "ref_harness"
DT = {"f16": torch.float16, "bf16": torch.bfloat16}


def bits(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy().view(np.uint16).copy()


def from_bits(a: np.ndarray, dtype: str) -> torch.Tensor:
    return torch.from_numpy(a.view(np.int16).copy()).view(DT[dtype])


def run(mode, **kw):
    cmd = [str(HARNESS), mode] + [f"{k}={v}" for k, v in kw.items()]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"{' '.join(cmd)} failed:\n{proc.stdout[-2000:]}\n{proc.stderr[-4000:]}")


def put(d: Path, name: str, t: torch.Tensor):
    if t.dtype in (torch.float16, torch.bfloat16):
        bits(t).tofile(d / f"{name}.bin")
    else:
        t.contiguous().numpy().tofile(d / f"{name}.bin")


def get16(d: Path, name: str, shape, dtype: str) -> torch.Tensor:
    return from_bits(np.fromfile(d / f"{name}.bin", dtype=np.uint16), dtype).reshape(shape)


def leaf_cases(g: torch.Generator):
    """(case name, op, scalar arguments, inputs {name: float32 tensor or int tensor}, outputs {name: shape})."""
    def rn(*shape, scale=1.0):
        return torch.randn(*shape, generator=g) * scale

    cases = []
    for eps, rows, H in ((1e-6, 5, 96), (1e-5, 3, 200)):
        cases.append((f"rmsnorm_eps{eps:g}", "rmsnorm", dict(rows=rows, hidden=H, eps=eps),
                      {"x": rn(rows, H, scale=2.0), "w": 1.0 + rn(H, scale=0.2)}, {"y": (rows, H)}))
    cases.append(("add_rmsnorm_mixed", "add_rmsnorm_mixed", dict(rows=4, hidden=160, eps=1e-6),
                  {"residual": rn(4, 160, scale=3.0), "x": rn(4, 160), "w": 1.0 + rn(160, scale=0.2)},
                  {"y": (4, 160), "residual_out": (4, 160)}))
    for name, n_past, theta, nh, nkv, d, T in (("rope_start", 0, 10000.0, 4, 2, 64, 7),
                                                ("rope_far", 32000, 1000000.0, 6, 2, 128, 5),
                                                ("rope_mid", 1234, 1000000.0, 3, 1, 32, 4)):
        cases.append((name, "rope", dict(seq_len=T, heads=nh, kv_heads=nkv, head_dim=d, n_past=n_past, theta=theta,
                                         rope_type=2),
                      {"q": rn(T, nh * d), "k": rn(T, nkv * d)}, {"q_out": (T, nh * d), "k_out": (T, nkv * d)}))
    past = torch.tensor([0, 17, 4095, 31999], dtype=torch.int32)
    cases.append(("batched_rope_bias", "batched_rope", dict(batch=4, heads=4, kv_heads=2, head_dim=64, theta=1000000.0,
                                                             rope_type=2, bias=1),
                  {"q": rn(4, 256), "k": rn(4, 128), "q_bias": rn(256, scale=0.5), "k_bias": rn(128, scale=0.5),
                   "n_past": past}, {"q_out": (4, 256), "k_out": (4, 128)}))
    cases.append(("silu_mul", "silu_mul", dict(count=600), {"gate": rn(600, scale=4.0), "up": rn(600)}, {"y": (600,)}))
    cases.append(("bias_triple", "bias_triple", dict(rows=3, q_dim=96, k_dim=32),
                  {"q": rn(3, 96), "k": rn(3, 32), "v": rn(3, 32), "q_bias": rn(96), "k_bias": rn(32), "v_bias": rn(32)},
                  {"q_out": (3, 96), "k_out": (3, 32), "v_out": (3, 32)}))
    # causal attention with a cached prefix (kv_len > query_len), group sizes 2 (grouped kernel), 7, 6 and 5
    for name, ql, kl, nh, nkv, d in (("attn_prefill_g2", 24, 40, 4, 2, 64), ("attn_prefill_g7", 9, 30, 7, 1, 128),
                                     ("attn_prefill_g6", 5, 5, 12, 2, 64), ("attn_prefill_g5", 6, 21, 5, 1, 128),
                                     ("attn_prefill_g1", 3, 11, 2, 2, 32)):
        cases.append((name, "attn_prefill", dict(query_len=ql, kv_len=kl, heads=nh, kv_heads=nkv, head_dim=d),
                      {"q": rn(ql, nh * d, scale=1.5), "k": rn(kl, nkv * d, scale=1.5), "v": rn(kl, nkv * d)},
                      {"o": (ql, nh * d)}))
    for name, nh, nkv, d, lens in (("attn_decode_g7", 7, 1, 128, [1, 33, 50]), ("attn_decode_g2", 4, 2, 64, [48, 7, 20]),
                                   ("attn_decode_g5", 5, 1, 128, [19, 2, 64])):
        slots, max_seq = 4, 64
        cache = rn(slots, 1, 2, max_seq, nkv * d)
        cases.append((name, "attn_decode", dict(batch=3, heads=nh, kv_heads=nkv, head_dim=d, max_seq=max_seq, slots=slots),
                      {"q": rn(3, nh * d, scale=1.5), "cache": cache, "seq_ids": torch.tensor([2, 0, 3], dtype=torch.int32),
                       "kv_lens": torch.tensor(lens, dtype=torch.int32)}, {"o": (3, nh * d)}))
    return cases


def make_leaf():
    out = {}
    g = torch.Generator().manual_seed(20)
    for name, op, scalars, inputs, outputs in leaf_cases(g):
        for dtype in ("f16", "bf16"):
            with tempfile.TemporaryDirectory() as tmp:
                d = Path(tmp)
                for k, t in inputs.items():
                    keep32 = (op == "add_rmsnorm_mixed" and k == "residual") or not t.is_floating_point()
                    v = t if keep32 else t.to(DT[dtype])
                    put(d, k, v)
                    key = f"{name}/{dtype}/in/{k}"
                    out[key] = v.numpy() if keep32 else bits(v)
                run("leaf", op=op, dtype=dtype, dir=d, **scalars)
                for k, shape in outputs.items():
                    if k == "residual_out":
                        out[f"{name}/{dtype}/out/{k}"] = np.fromfile(d / f"{k}.bin", dtype=np.float32).reshape(shape)
                    else:
                        out[f"{name}/{dtype}/out/{k}"] = bits(get16(d, k, shape, dtype))
            for k, v in scalars.items():
                out[f"{name}/{dtype}/arg/{k}"] = np.asarray(v)
            out[f"{name}/{dtype}/op"] = np.asarray(op)
    np.savez_compressed(HERE / "reference_leaf.npz", **out)
    print(f"reference_leaf.npz: {len(out)} arrays")


MODELS = {
    "m1": dict(hidden=64, layers=2, heads=4, kv_heads=2, head_dim=64, inter=160, vocab=200, theta=10000.0, eps=1e-6,
               tied=0, bias=1),
    "m2": dict(hidden=96, layers=3, heads=6, kv_heads=2, head_dim=32, inter=136, vocab=250, theta=1000000.0, eps=1e-5,
               tied=1, bias=1),
}


def model_tensors(s, g):
    H, Q, KV, I, V = s["hidden"], s["heads"] * s["head_dim"], s["kv_heads"] * s["head_dim"], s["inter"], s["vocab"]

    def w(*shape, std=0.08):
        return torch.randn(*shape, generator=g) * std

    t = {"model.embed_tokens.weight": w(V, H, std=0.5), "model.norm.weight": 1.0 + w(H, std=0.1)}
    if not s["tied"]:
        t["lm_head.weight"] = w(V, H, std=0.1)
    for l in range(s["layers"]):
        p = f"model.layers.{l}."
        t[p + "input_layernorm.weight"] = 1.0 + w(H, std=0.1)
        t[p + "post_attention_layernorm.weight"] = 1.0 + w(H, std=0.1)
        t[p + "self_attn.q_proj.weight"] = w(Q, H, std=0.12)
        t[p + "self_attn.k_proj.weight"] = w(KV, H, std=0.12)
        t[p + "self_attn.v_proj.weight"] = w(KV, H)
        t[p + "self_attn.o_proj.weight"] = w(H, Q)
        t[p + "self_attn.q_proj.bias"] = w(Q, std=0.3)
        t[p + "self_attn.k_proj.bias"] = w(KV, std=0.3)
        t[p + "self_attn.v_proj.bias"] = w(KV, std=0.1)
        t[p + "mlp.gate_proj.weight"] = w(I, H)
        t[p + "mlp.up_proj.weight"] = w(I, H)
        t[p + "mlp.down_proj.weight"] = w(H, I)
    return t


def make_model():
    out = {}
    for mi, (name, s) in enumerate(MODELS.items()):
        g = torch.Generator().manual_seed(40 + mi)
        tensors = model_tensors(s, g)
        seq0 = torch.randint(0, s["vocab"], (34,), generator=g).tolist()
        seq1 = torch.randint(0, s["vocab"], (8,), generator=g).tolist()
        # sequence 0: 21 tokens, then 9 more on top of the cache, then two decode steps beside sequence 1
        script = [
            f"forward seq=0 n_past=0 tokens={','.join(map(str, seq0[:21]))} out=a.bin",
            f"forward seq=0 n_past=21 tokens={','.join(map(str, seq0[21:30]))} out=b.bin",
            f"forward seq=1 n_past=0 tokens={','.join(map(str, seq1[:5]))} out=c.bin",
            f"batch tokens={seq0[30]},{seq1[5]} n_past=30,5 seqs=0,1 out=d.bin",
            f"batch tokens={seq1[6]},{seq0[31]} n_past=6,31 seqs=1,0 out=e.bin",
        ]
        for dtype in ("f16", "bf16"):
            with tempfile.TemporaryDirectory() as tmp:
                d = Path(tmp)
                for k, t in tensors.items():
                    put(d, k, t.to(DT[dtype]))
                (d / "script.txt").write_text("\n".join(script) + "\n")
                run("model", dtype=dtype, weights=d, script=d / "script.txt", out=d, max_seq=64, max_batch=2, chunk=32,
                    max_pos=64, **s)
                V = s["vocab"]
                for f, rows in (("a", 1), ("b", 1), ("c", 1), ("d", 2), ("e", 2)):
                    out[f"{name}/{dtype}/logits/{f}"] = np.fromfile(d / f"{f}.bin", dtype=np.float32).reshape(rows, V)
        for k, t in tensors.items():
            out[f"{name}/weights/{k}"] = t.numpy()          # float32; each run rounds them to its dtype
        for k, v in s.items():
            out[f"{name}/config/{k}"] = np.asarray(v)
        out[f"{name}/seq0"] = np.asarray(seq0)
        out[f"{name}/seq1"] = np.asarray(seq1)
    np.savez_compressed(HERE / "reference_model.npz", **out)
    print(f"reference_model.npz: {len(out)} arrays")


if __name__ == "__main__":
    if not HARNESS.is_file():
        sys.exit(f"{HARNESS} is missing: run python baseline/build_ref.py first")
    make_leaf()
    make_model()
