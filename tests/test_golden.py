"""The plain implementation against outputs of the reference's own code.

tests/golden/reference_leaf.npz and reference_model.npz were written by
tests/golden/make_goldens.py, which runs the unmodified reference (its leaf host
wrappers and its LlamaForwardTyped<T> model path, built by baseline/build_ref.py) on
a GPU.  Here, without a GPU, every function of tests/plain/plain_qwen2.py is given
the same inputs in float64 and must reproduce the reference's 16-bit results within
the rounding of that dtype; the bounds are at or below the reference's own
(tests/unit/test_native_forward.cpp:1837 margin 6e-2 for attention, :1897 margin 2e-3
for the rotation, both in float16).
"""
import math
from pathlib import Path

import numpy as np
import pytest
import torch

from plain import plain_qwen2 as P

GOLDEN = Path(__file__).resolve().parent / "golden"
DT = {"f16": torch.float16, "bf16": torch.bfloat16}
# relative rounding step of the dtype: results are compared in units of it
ULP = {"f16": 2.0 ** -10, "bf16": 2.0 ** -7}


def _load(name):
    path = GOLDEN / name
    if not path.is_file():
        pytest.fail(f"{path} is missing: run tests/golden/make_goldens.py on a GPU")
    return np.load(path)


def _t16(a, dtype):
    return torch.from_numpy(a.view(np.int16).copy()).view(DT[dtype]).double()


class Case:
    def __init__(self, z, name, dtype):
        self.z, self.name, self.dtype = z, name, dtype

    def arg(self, k):
        return self.z[f"{self.name}/{self.dtype}/arg/{k}"].item()

    def inp(self, k):
        a = self.z[f"{self.name}/{self.dtype}/in/{k}"]
        return _t16(a, self.dtype) if a.dtype == np.uint16 else torch.from_numpy(a)

    def out(self, k):
        a = self.z[f"{self.name}/{self.dtype}/out/{k}"]
        return _t16(a, self.dtype) if a.dtype == np.uint16 else torch.from_numpy(a).double()


def _cases(op):
    z = _load("reference_leaf.npz")
    names = sorted({k.split("/")[0] for k in z.files if k.endswith("/op") and str(z[k]) == op})
    assert names, f"no golden case of {op}"
    return [Case(z, n, dt) for n in names for dt in ("f16", "bf16")]


def _close(got, want, dtype, ulps, floor=0.0, what=""):
    """|got - want| <= ulps roundings of the dtype at the size of the value (plus `floor`)."""
    tol = ulps * ULP[dtype] * want.abs().clamp_min(floor)
    bad = (got - want).abs() > tol
    assert not bad.any(), (f"{what}: {int(bad.sum())} of {bad.numel()} values differ, worst "
                           f"{float(((got - want).abs() / tol).max()):.2f} x the bound")


def test_rmsnorm_matches_the_reference():
    for c in _cases("rmsnorm"):
        y = P.rmsnorm(c.inp("x"), c.inp("w"), c.arg("eps"))
        _close(y, c.out("y"), c.dtype, 1.01, what=f"{c.name} {c.dtype}")


def test_residual_add_and_norm_matches_the_reference():
    # cuda_kernels.cu:618-655: the float32 residual takes the 16-bit delta, then the norm of the sum
    for c in _cases("add_rmsnorm_mixed"):
        res = c.inp("residual").double() + c.inp("x")
        assert torch.allclose(res, c.out("residual_out"), rtol=2e-7, atol=0), c.name
        y = P.rmsnorm(res, c.inp("w"), c.arg("eps"))
        _close(y, c.out("y"), c.dtype, 1.01, what=f"{c.name} {c.dtype}")


def _rope_check(c, q, k, positions, what):
    nh, nkv, d, theta = c.arg("heads"), c.arg("kv_heads"), c.arg("head_dim"), c.arg("theta")
    T = q.shape[0]
    q_want, k_want = c.out("q_out"), c.out("k_out")
    q_got = P.rope_neox(q.view(T, nh, d), positions, theta).reshape(T, nh * d)
    k_got = P.rope_neox(k.view(T, nkv, d), positions, theta).reshape(T, nkv * d)
    # The angle pos * inv_freq is a float32 product of up to 32,000 rad: its own rounding (2^-24
    # relative, so up to 2e-3 rad) moves the result by that much times the vector's size.  On top,
    # one rounding of the dtype.  The reference's own test allows 2e-3 at small positions in float16.
    big = float(positions.max())
    slack = 2.5 * 2.0 ** -24 * max(big, 1.0)
    for got, want, src in ((q_got, q_want, q), (k_got, k_want, k)):
        size = src.abs().max()
        tol = 1.01 * ULP[c.dtype] * want.abs() + slack * size + 1e-30
        bad = (got - want).abs() > tol
        assert not bad.any(), f"{what}: {int(bad.sum())} values differ, worst {float(((got - want).abs() / tol).max()):.2f}"
        assert float((got - want).abs().max()) < 2e-3 * max(1.0, float(size)) + ULP[c.dtype] * float(size)


def test_rotation_matches_the_reference():
    for c in _cases("rope"):
        T = c.arg("seq_len")
        positions = torch.arange(c.arg("n_past"), c.arg("n_past") + T)
        _rope_check(c, c.inp("q"), c.inp("k"), positions, f"{c.name} {c.dtype}")


def test_bias_then_rotation_matches_the_reference():
    # cuda_kernels.cu:895-958: the bias is added to the loaded value in float32, then the pair is rotated
    for c in _cases("batched_rope"):
        q = c.inp("q") + c.inp("q_bias")[None, :]
        k = c.inp("k") + c.inp("k_bias")[None, :]
        _rope_check(c, q, k, c.inp("n_past").long(), f"{c.name} {c.dtype}")


def test_silu_mul_matches_the_reference():
    for c in _cases("silu_mul"):
        y = P.silu(c.inp("gate")) * c.inp("up")
        _close(y, c.out("y"), c.dtype, 1.01, floor=1e-6, what=f"{c.name} {c.dtype}")


def test_bias_add_matches_the_reference():
    for c in _cases("bias_triple"):
        for n in ("q", "k", "v"):
            y = c.inp(n) + c.inp(f"{n}_bias")[None, :]
            _close(y, c.out(f"{n}_out"), c.dtype, 1.01, floor=1e-3, what=f"{c.name} {n} {c.dtype}")


def _attention_with_prefix(q, k, v, nh, nkv, d):
    """The plain whole-sequence attention, asked for the last len(q) positions of a sequence of
    len(k) keys: queries for the prefix are made up and their rows dropped."""
    ql, kl = q.shape[0], k.shape[0]
    full_q = torch.zeros(kl, nh, d, dtype=q.dtype)
    full_q[kl - ql:] = q.view(ql, nh, d)
    out = P.attention_gqa_causal(full_q, k.view(kl, nkv, d), v.view(kl, nkv, d))
    return out[kl - ql:].reshape(ql, nh * d)


def test_prompt_attention_matches_the_reference():
    for c in _cases("attn_prefill"):
        nh, nkv, d = c.arg("heads"), c.arg("kv_heads"), c.arg("head_dim")
        got = _attention_with_prefix(c.inp("q"), c.inp("k"), c.inp("v"), nh, nkv, d)
        want = c.out("o")
        # outputs are sums of values of size ~1 weighted by probabilities: a few roundings of the dtype
        # at the size of the values (the tensor-core variant keeps probabilities in 16 bits)
        err = float((got - want).abs().max())
        bound = 4 * ULP[c.dtype] * float(c.inp("v").abs().max())
        assert err <= bound, f"{c.name} {c.dtype}: max error {err:.3e} > {bound:.3e}"
        assert err < 6e-2


def test_decode_attention_matches_the_reference():
    for c in _cases("attn_decode"):
        nh, nkv, d, max_seq, slots = (c.arg(k) for k in ("heads", "kv_heads", "head_dim", "max_seq", "slots"))
        cache = c.inp("cache").view(slots, 1, 2, max_seq, nkv * d)
        q, want = c.inp("q"), c.out("o")
        for b, (slot, n) in enumerate(zip(c.inp("seq_ids").tolist(), c.inp("kv_lens").tolist())):
            got = _attention_with_prefix(q[b:b + 1], cache[slot, 0, 0, :n], cache[slot, 0, 1, :n], nh, nkv, d)
            err = float((got[0] - want[b]).abs().max())
            bound = 4 * ULP[c.dtype] * float(cache[slot, 0, 1, :n].abs().max())
            assert err <= bound, f"{c.name} {c.dtype} row {b}: max error {err:.3e} > {bound:.3e}"


# ------------------------------------------------------------------ whole model

def _model(z, name, dtype):
    cfg_raw = {k.split("/")[-1]: z[k].item() for k in z.files if k.startswith(f"{name}/config/")}
    cfg = {"hidden_size": cfg_raw["hidden"], "num_hidden_layers": cfg_raw["layers"], "num_attention_heads": cfg_raw["heads"],
           "num_key_value_heads": cfg_raw["kv_heads"], "head_dim": cfg_raw["head_dim"], "intermediate_size": cfg_raw["inter"],
           "vocab_size": cfg_raw["vocab"], "rope_theta": cfg_raw["theta"], "rms_norm_eps": cfg_raw["eps"],
           "tie_word_embeddings": bool(cfg_raw["tied"])}
    prefix = f"{name}/weights/"
    # the run rounded the float32 weights to its dtype
    W = {k[len(prefix):]: torch.from_numpy(z[k]).to(DT[dtype]).double() for k in z.files if k.startswith(prefix)}
    return cfg, W


@pytest.mark.parametrize("name", ["m1", "m2"])
@pytest.mark.parametrize("dtype", ["f16", "bf16"])
def test_whole_model_logits_match_the_reference(name, dtype):
    """Forward of 21 tokens, 9 more on top of the cache, a second sequence, and two batched
    decode steps of both: the reference's logits against the plain implementation's (float64
    on the same rounded weights).  The reference rounds every activation to 16 bits, so the
    bound is a few roundings of the dtype at the size of the logits."""
    z = _load("reference_model.npz")
    cfg, W = _model(z, name, dtype)
    seq0, seq1 = z[f"{name}/seq0"].tolist(), z[f"{name}/seq1"].tolist()
    want = {
        "a": [(seq0, 21)], "b": [(seq0, 30)], "c": [(seq1, 5)],
        "d": [(seq0, 31), (seq1, 6)], "e": [(seq1, 7), (seq0, 32)],
    }
    worst = 0.0
    for key, rows in want.items():
        ref = torch.from_numpy(z[f"{name}/{dtype}/logits/{key}"]).double()
        for r, (seq, n) in enumerate(rows):
            mine = P.forward(cfg, W, seq[:n], dtype=torch.float64)[-1]
            scale = float(mine.abs().max())
            err = float((mine - ref[r]).abs().max())
            worst = max(worst, err / scale)
            assert int(mine.argmax()) == int(ref[r].argmax()) or err < 2 * ULP[dtype] * scale, (name, dtype, key, r)
            assert err <= 12 * ULP[dtype] * scale, f"{name} {dtype} {key}[{r}]: {err:.3e} against logits of size {scale:.2f}"
    assert worst > 0          # the files hold a 16-bit run, not a copy of the plain implementation
