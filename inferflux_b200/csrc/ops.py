"""The kernel table of the product path: every operation of a step as a call into
the hand-written sm_100a library (plus cuBLAS for the bfloat16 matrix products,
where the reference uses it too).

There is no CPU path and no library model code here: making a `CudaKernels`
without a CUDA device, or without being able to build or load the library, raises.
Tensors are passed as raw device pointers on torch's current stream.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from .build import BuildError, load_library

_DT = {torch.float32: 0, torch.bfloat16: 1}

_ERRORS = {-1: "a size or option the kernel does not take", -2: "unknown dtype",
           -3: "a pointer or stride breaks an alignment rule", -4: "a size beyond the kernel's stated maximum"}


class KernelError(RuntimeError):
    pass


class ScaledRows:
    """Rows of a norm without its row scale: `pre` = x * w in the run's dtype and `sumsq`
    [rows, chunks] float32, the chunks' sums of x^2.  The true rows are
    pre * rsqrt(sum(sumsq[row]) / hidden + eps); a matrix product that takes them applies that
    per-row factor to its accumulator.  `CudaKernels.materialize_rows` gives the plain tensor."""

    def __init__(self, pre: torch.Tensor, sumsq: torch.Tensor, eps: float):
        self.pre, self.sumsq, self.eps = pre, sumsq, float(eps)

    @property
    def shape(self):
        return self.pre.shape

    @property
    def dtype(self):
        return self.pre.dtype


class PartialSum:
    """The result of a matrix product whose K range was split over thread blocks:
    float32 partial sums [splits, rows, cols] that the consuming kernel adds, in split
    order, in the same pass in which it does its own work (residual add and norm, bias
    and rotation).  `CudaKernels.materialize` gives the plain tensor."""

    def __init__(self, parts: torch.Tensor, dtype: torch.dtype):
        self.parts = parts
        self.dtype = dtype                       # the dtype the sum stands for

    @property
    def shape(self):
        return self.parts.shape[1:]

    @property
    def splits(self) -> int:
        return self.parts.shape[0]


def _ptr(t: Optional[torch.Tensor]):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


# The current stream's handle of the current device, asked for at every launch: torch's own accessors
# when they are there (plain integers, a fraction of a microsecond), else through the Stream object
# (several microseconds).
_RAW_STREAM = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_RAW_DEVICE = getattr(torch._C, "_cuda_getDevice", None)


def _stream():
    if _RAW_STREAM is not None and _RAW_DEVICE is not None:
        return ctypes.c_void_p(_RAW_STREAM(_RAW_DEVICE()))
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _check(rc: int, what: str) -> None:
    if rc == 0:
        return
    if rc < 0:
        raise KernelError(f"{what}: refused ({_ERRORS.get(rc, rc)})")
    if rc >= 1000:
        raise KernelError(f"{what}: cuBLAS status {rc - 1000}")
    raise KernelError(f"{what}: CUDA error {rc}")


def _need(cond: bool, msg: str) -> None:
    if not cond:
        raise KernelError(msg)


_I, _F, _P, _LL = ctypes.c_int, ctypes.c_float, ctypes.c_void_p, ctypes.c_longlong


class _StepArgs(ctypes.Structure):
    """IfxStepArgs of csrc/layer_forward.cu: one step's batch, the same for every layer."""
    _fields_ = ([(n, _I) for n in ("T", "num_decode", "num_tiles", "max_kv_len")]
                + [(n, _P) for n in ("positions", "token_req", "req_slot", "decode_rows", "decode_meta", "prefill_tiles",
                                     "norm_sumsq", "norm_tickets", "error_flag")]
                + [(n, _I) for n in ("skinny_max_rows", "swiglu_tiles", "swiglu_tiles_max_k", "tensor_core_prefill",
                                     "overlap_attention", "pad0")])


class _LayerArgs(ctypes.Structure):
    """IfxLayerArgs: one layer's sizes, constants, weights and cache."""
    _fields_ = ([(n, _I) for n in ("hidden", "inter", "nq", "nkv", "d", "window", "rot", "interleaved")]
                + [(n, _F) for n in ("scale", "eps_in", "eps_post")] + [("write_cache", _I)]
                + [(n, _P) for n in ("norm_in_w", "norm_post_w", "b_qkv", "inv_freq", "w_qkv", "w_o", "w_gate_up", "w_down",
                                     "kv_pool", "block_table")]
                + [(n, _I) for n in ("max_blocks", "page_size", "num_pages", "pad0")])


class _LayerIO(ctypes.Structure):
    """IfxLayerIO: what changes from call to call, and what comes back."""
    _fields_ = [("x", _P), ("pending_tensor", _P), ("pending_parts", _P), ("pending_splits", _I), ("parity", _I),
                ("ws", _P), ("ws_bytes", _LL), ("out_tensor", _P), ("out_parts", _P), ("out_splits", _I),
                ("launches", _I), ("library_calls", _I), ("pad0", _I)]


class CudaKernels:
    """Kernel table on one CUDA device."""

    name = "cuda-sm100a"

    def __init__(self, device="cuda"):
        if not torch.cuda.is_available():
            raise BuildError("no CUDA device: the engine has no CPU path")
        self.device = torch.device(device)
        self.lib = load_library()
        for fn in ("ifx_embed", "ifx_rmsnorm", "ifx_silu_mul", "ifx_residual_add", "ifx_gather_rows",
                   "ifx_scatter_i32", "ifx_rope_append", "ifx_attention_generic", "ifx_gemm_generic",
                   "ifx_gemm_cublas_bf16", "ifx_cublas_init", "ifx_argmax", "ifx_penalties", "ifx_logit_bias",
                   "ifx_sample", "ifx_sample_blocks", "ifx_attention_mma_supports", "ifx_attention_prefill_bf16",
                   "ifx_attention_prefill_tcgen05", "ifx_attention_prefill_tcgen05_supports", "ifx_attention_decode_max_splits",
                   "ifx_attention_decode_bf16", "ifx_gemm_skinny", "ifx_residual_add_partial",
                   "ifx_reduce_partial", "ifx_reduce_add_rmsnorm", "ifx_argmax_chunks", "ifx_relay_i32", "ifx_prenorm", "ifx_scale_rows",
                   "ifx_gemm_tcgen05"):
            getattr(self.lib, fn).restype = ctypes.c_int
        self.lib.ifx_sample_scratch_bytes.restype = ctypes.c_longlong
        with torch.cuda.device(self.device):
            _check(self.lib.ifx_cublas_init(), "cublas init")
        if os.environ.get("INFERFLUX_B200_CARVEOUT", "") != "":    # for measurements: -1 leaves the split to the driver
            self.lib.ifx_set_shared_carveout(int(os.environ["INFERFLUX_B200_CARVEOUT"]))
        if os.environ.get("INFERFLUX_B200_PDL", "1") == "0":      # for measurements: no overlap of consecutive kernels
            self.lib.ifx_set_pdl(0)
        # prompt portions on the tcgen05 attention kernel (0: the mma.sync kernel, for comparisons)
        self.tensor_core_prefill = os.environ.get("INFERFLUX_B200_TCGEN05_ATTENTION", "1") != "0"
        # gate/up of prompt portions on the own tcgen05 tiles with the activation fused (0: cuBLAS + silu kernel)
        self.swiglu_tiles = os.environ.get("INFERFLUX_B200_SWIGLU_TILES", "1") != "0"
        self.launches = 0            # kernels of this library launched so far
        self.library_calls = 0       # cuBLAS products called so far
        # scratch of the many-block reduce + norm: sums of squares per (row, chunk), a ticket per row
        self._norm_sumsq = torch.zeros(128 * 64, dtype=torch.float32, device=self.device)
        self._norm_tickets = torch.zeros(128, dtype=torch.int32, device=self.device)
        self._sample_scratch, self._sample_capacity = None, 0   # zeroed once; the sampling kernels leave it zero
        self._argmax_val = torch.zeros(256 * 32, dtype=torch.float32, device=self.device)
        self._argmax_idx = torch.zeros(256 * 32, dtype=torch.int32, device=self.device)
        self._argmax_tickets = torch.zeros(256, dtype=torch.int32, device=self.device)
        self.error_flag = torch.zeros(1, dtype=torch.int32, device=self.device)   # set by a kernel whose bounded wait ran out
        # whole layers from native code (0: every part launches its kernels from Python, the general way)
        self.native_layers = os.environ.get("INFERFLUX_B200_NATIVE_LAYER", "1") != "0"
        # in a natively run layer of a mixed step, the two attention kernels side by side on two streams
        self.overlap_attention = os.environ.get("INFERFLUX_B200_ATTENTION_OVERLAP", "1") != "0"
        self.lib.ifx_layer_forward.restype = ctypes.c_int
        self.lib.ifx_layer_workspace_bytes.restype = ctypes.c_longlong
        self._layer_ws, self._layer_ws_all, self._layer_views = None, [], {}
        self._layer_io = _LayerIO()
        self._layer_io_ref = ctypes.byref(self._layer_io)
        self._layer_parity = 0
        self.native_layer_calls = 0

    # ------------------------------------------------------------- elementwise
    def embed(self, table, token_ids, vocab):
        T, H = token_ids.numel(), table.shape[1]
        out = torch.empty((T, H), dtype=torch.float32, device=table.device)
        _check(self.lib.ifx_embed(_ptr(table), _ptr(token_ids), _ptr(out), T, H, int(vocab), _DT[table.dtype],
                                  _stream()), "embed")
        self.launches += 1
        return out

    def rmsnorm(self, x, w, eps, out_dtype):
        _need(x.dtype == torch.float32 and w.dtype == torch.float32, "rmsnorm: x and w must be float32")
        T, H = x.shape
        out = torch.empty((T, H), dtype=out_dtype, device=x.device)
        _check(self.lib.ifx_rmsnorm(_ptr(x), _ptr(None), _ptr(w), _ptr(out), T, H, ctypes.c_float(eps), 0,
                                    _DT[out_dtype], _stream()), "rmsnorm")
        self.launches += 1
        return out

    def add_rmsnorm(self, x, delta, w, eps, out_dtype):
        """x += delta (in place), then the norm of the sum.  `delta` is a tensor in the run's
        dtype or a PartialSum, whose slices are added in the same pass."""
        _need(x.dtype == torch.float32 and w.dtype == torch.float32, "add_rmsnorm: x and w must be float32")
        T, H = x.shape
        out = torch.empty((T, H), dtype=out_dtype, device=x.device)
        if isinstance(delta, PartialSum):
            _need(tuple(delta.shape) == (T, H), "add_rmsnorm: partial sums do not match x")
            chunks = -(-H // 512)
            if T <= self._norm_tickets.numel() and T * chunks <= self._norm_sumsq.numel():
                _check(self.lib.ifx_reduce_add_rmsnorm(
                    _ptr(x), _ptr(delta.parts), _ptr(w), _ptr(out), T, H, ctypes.c_float(eps), delta.splits,
                    _ptr(self._norm_sumsq), _ptr(self._norm_tickets), _DT[out_dtype], _stream()), "reduce_add_rmsnorm")
                self.launches += 1
                return out
            src, splits = delta.parts, delta.splits
        else:
            _need(delta.dtype == out_dtype and delta.shape == x.shape, "add_rmsnorm: delta must match x and the dtype")
            src, splits = delta, 0
        _check(self.lib.ifx_rmsnorm(_ptr(x), _ptr(src), _ptr(w), _ptr(out), T, H, ctypes.c_float(eps), splits,
                                    _DT[out_dtype], _stream()), "add_rmsnorm")
        self.launches += 1
        return out

    def prenorm(self, x, delta, w, eps, out_dtype):
        """The norm for a consumer that takes ScaledRows (x += delta first, as add_rmsnorm).
        Few bfloat16 rows: one pass that leaves x * w and per-chunk sums of squares, the row scale
        being applied by the matrix product that follows.  Otherwise the plain normed tensor."""
        T, H = x.shape
        if out_dtype != torch.bfloat16 or T > self.SKINNY_MAX_ROWS or H % 8:
            return self.rmsnorm(x, w, eps, out_dtype) if delta is None else self.add_rmsnorm(x, delta, w, eps, out_dtype)
        pre = torch.empty((T, H), dtype=out_dtype, device=x.device)
        sumsq = torch.empty((T, -(-H // 512)), dtype=torch.float32, device=x.device)
        if isinstance(delta, PartialSum):
            _need(tuple(delta.shape) == (T, H), "prenorm: partial sums do not match x")
            src, splits = delta.parts, delta.splits
        else:
            _need(delta is None or (delta.dtype == out_dtype and delta.shape == x.shape), "prenorm: delta must match x")
            src, splits = delta, 0
        _check(self.lib.ifx_prenorm(_ptr(x), _ptr(src), _ptr(w), _ptr(pre), _ptr(sumsq), T, H, splits, _DT[out_dtype],
                                    _stream()), "prenorm")
        self.launches += 1
        return ScaledRows(pre, sumsq, eps)

    def materialize_rows(self, h):
        """A plain tensor from what `prenorm` returned."""
        if not isinstance(h, ScaledRows):
            return h
        T, H = h.shape
        out = torch.empty((T, H), dtype=h.dtype, device=h.pre.device)
        _check(self.lib.ifx_scale_rows(_ptr(h.pre), _ptr(h.sumsq), _ptr(out), T, H, ctypes.c_float(h.eps),
                                       _DT[h.dtype], _stream()), "scale_rows")
        self.launches += 1
        return out

    def residual_add(self, x, delta):
        T, H = x.shape
        if isinstance(delta, PartialSum):
            _check(self.lib.ifx_residual_add_partial(_ptr(x), _ptr(delta.parts), T, H, delta.splits, _stream()),
                   "residual_add")
        else:
            _check(self.lib.ifx_residual_add(_ptr(x), _ptr(delta), T, H, _DT[delta.dtype], _stream()), "residual_add")
        self.launches += 1

    def materialize(self, value, bias=None):
        """A plain tensor from what `linear(..., allow_partial=True)` returned."""
        if not isinstance(value, PartialSum):
            return value if bias is None else value + bias.to(value.dtype)
        T, N = value.shape
        out = torch.empty((T, N), dtype=value.dtype, device=value.parts.device)
        _check(self.lib.ifx_reduce_partial(_ptr(value.parts), _ptr(bias), _ptr(out), T, N, value.splits,
                                           _DT[value.dtype], _stream()), "reduce_partial")
        self.launches += 1
        return out

    def silu_mul(self, gate_up):
        T, two_i = gate_up.shape
        out = torch.empty((T, two_i // 2), dtype=gate_up.dtype, device=gate_up.device)
        _check(self.lib.ifx_silu_mul(_ptr(gate_up), _ptr(out), T, two_i // 2, _DT[gate_up.dtype], _stream()),
               "silu_mul")
        self.launches += 1
        return out

    def gather_rows(self, x, rows):
        R, H = rows.numel(), x.shape[1]
        out = torch.empty((R, H), dtype=torch.float32, device=x.device)
        _check(self.lib.ifx_gather_rows(_ptr(x), _ptr(rows), _ptr(out), R, H, x.shape[0], _stream()), "gather_rows")
        self.launches += 1
        return out

    def scatter_i32(self, table, index, value):
        n = index.numel()
        if n:
            _check(self.lib.ifx_scatter_i32(_ptr(table), _ptr(index), _ptr(value), n, table.numel(), _stream()),
                   "scatter_i32")
            self.launches += 1

    def relay_i32(self, dst, dst_index, src, src_index):
        n = dst_index.numel()
        if n:
            _check(self.lib.ifx_relay_i32(_ptr(dst), _ptr(dst_index), _ptr(src), _ptr(src_index), n, dst.numel(),
                                          src.numel(), _stream()), "relay_i32")
            self.launches += 1

    # ------------------------------------------------------------------ linear
    # The weight-streaming kernel takes up to 256 rows; in a whole step it beats cuBLAS up to about 160
    # (measured at the 7B shape: 4.5 against 4.9 ms at 129 rows, 5.2 against 5.0 ms at 192).
    SKINNY_MAX_ROWS = 160

    def linear(self, a, w, bias=None, out_dtype=None, allow_partial=False):
        """out[T, N] = a[T, K] . w[N, K]^T (+ bias), float32 accumulation.  float32 runs use
        the CUDA-core product.  bfloat16 runs with up to 256 rows use the tcgen05 weight-streaming
        kernel; with `allow_partial` a narrow product is split over K and comes back as a
        PartialSum for a consumer that adds the slices itself.  More rows go to cuBLAS."""
        rows = a if isinstance(a, ScaledRows) else None
        if rows is not None:
            a = rows.pre
        _need(a.dtype == w.dtype, f"linear: activations are {a.dtype}, weights {w.dtype}")
        _need(a.is_contiguous() and w.is_contiguous(), "linear: operands must be contiguous")
        T, K = a.shape
        N = w.shape[0]
        _need(w.shape[1] == K, f"linear: inner sizes differ ({K} vs {w.shape[1]})")
        out_dtype = out_dtype or a.dtype
        if T == 0:
            return torch.empty((T, N), dtype=out_dtype, device=a.device)
        if rows is not None and not (T <= self.SKINNY_MAX_ROWS and K % 8 == 0 and w.data_ptr() % 16 == 0):
            a, rows = self.materialize_rows(rows), None
        if a.dtype == torch.float32:
            _need(out_dtype == torch.float32, "linear: a float32 product gives float32")
            out = torch.empty((T, N), dtype=out_dtype, device=a.device)
            _check(self.lib.ifx_gemm_generic(_ptr(a), _ptr(w), _ptr(bias), _ptr(out), T, N, K, 0, 0, _stream()),
                   "gemm (float32)")
            self.launches += 1
            return out
        if T <= self.SKINNY_MAX_ROWS and K % 8 == 0 and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0:
            tiles = -(-N // 128)
            kblocks = -(-K // 64)
            # up to 128 rows: two blocks a SM and up to 10 K slices; above, a block owns its SM (32 KB of
            # activations a stage) and every slice costs a [T, N] float32 round trip: at most 5
            slots, most = (296, 10) if T <= 128 else (148, 5)
            splits = max(1, min(slots // tiles, most, kblocks // 4)) if allow_partial and bias is None else 1
            if splits > 1:
                parts = self.linear_skinny(a, w, None, splits=splits, mode=1, rows=rows)
                return PartialSum(parts, out_dtype)
            if tiles >= 74 or allow_partial or rows is not None:
                return self.linear_skinny(a, w, bias, out_dtype=out_dtype, splits=1, mode=0, rows=rows)
        out = torch.empty((T, N), dtype=out_dtype, device=a.device)
        _check(self.lib.ifx_gemm_cublas_bf16(_ptr(a), _ptr(w), _ptr(out), T, N, K, _DT[out_dtype], _stream()),
               "gemm (bfloat16)")
        self.library_calls += 1
        if bias is not None:
            out += bias.to(out.dtype)
        return out

    # The many-rows tcgen05 product with SiLU(gate)*up in its epilogue against cuBLAS followed by the activation
    # kernel, measured on a B200 (us a layer, 256 / 512 / 2,048 rows): Qwen2.5-1.5B sizes 21 vs 27, 31 vs 37, 94 vs 110;
    # 7B sizes 63 vs 79, 107 vs 107, 373 vs 381; 32B sizes (inner size 5120) 126 vs 136, 217 vs 212, 851 vs 779.
    # So it is used up to an inner size of 4096.
    SWIGLU_TILES_MAX_K = 4096

    def linear_swiglu(self, a, w_gate_up):
        """silu(a . Wg^T) * (a . Wu^T) with Wg and Wu stacked in w_gate_up [2 I, K]: one kernel
        with both accumulators for few rows, else the product followed by the activation kernel."""
        rows = a if isinstance(a, ScaledRows) else None
        if rows is not None:
            a = rows.pre
        T, K = a.shape
        inter = w_gate_up.shape[0] // 2
        if (a.dtype == torch.bfloat16 and 0 < T <= self.SKINNY_MAX_ROWS and K % 8 == 0 and a.data_ptr() % 16 == 0
                and w_gate_up.data_ptr() % 16 == 0):
            return self.linear_skinny(a, w_gate_up, None, splits=1, mode=2, n_out=inter, up_row_offset=inter, rows=rows)
        if rows is not None:
            a = self.materialize_rows(rows)
        if (self.swiglu_tiles and a.dtype == torch.bfloat16 and K % 8 == 0 and K <= self.SWIGLU_TILES_MAX_K
                and a.data_ptr() % 16 == 0 and w_gate_up.data_ptr() % 16 == 0 and a.is_contiguous()):
            return self.linear_tiles(a, w_gate_up, swiglu=True)        # many rows: own tcgen05 tiles, activation fused
        return self.silu_mul(self.linear(a, w_gate_up))

    def check_errors(self):
        """Raise if a kernel reported that one of its bounded waits ran out (reads the device flag)."""
        code = int(self.error_flag.item())
        if code:
            self.error_flag.zero_()
            raise KernelError(f"a kernel gave up waiting on a barrier (code {code}); its output is not valid")

    def linear_skinny(self, a, w, bias=None, out_dtype=None, splits=1, mode=0, n_out=None, up_row_offset=0, rows=None):
        """The tcgen05 weight-streaming product for up to 256 token rows.
        mode 0: out[T, N] (+bias); mode 1: float32 partial sums [splits, T, N]; mode 2: silu(gate) * up.
        `rows`: the ScaledRows whose `pre` is `a`; the product then applies their row scale."""
        T, K = a.shape
        N = n_out if n_out is not None else w.shape[0]
        _need(a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16, "linear_skinny: bfloat16 only")
        _need(a.is_contiguous() and w.is_contiguous() and w.shape[1] == K, "linear_skinny: bad operands")
        out_dtype = out_dtype or torch.bfloat16
        out = partials = None
        if mode == 1:
            partials = torch.empty((splits, T, N), dtype=torch.float32, device=a.device)
        else:
            out = torch.empty((T, N), dtype=out_dtype, device=a.device)
        _check(self.lib.ifx_gemm_skinny(_ptr(a), _ptr(w), _ptr(bias), _ptr(out), _ptr(partials), T, N, K, w.shape[0],
                                        splits, mode, up_row_offset, int(out_dtype == torch.float32),
                                        _ptr(None if rows is None else rows.sumsq),
                                        0 if rows is None else rows.sumsq.shape[1],
                                        ctypes.c_float(0.0 if rows is None else rows.eps),
                                        _ptr(self.error_flag), _stream()), "gemm_skinny")
        self.launches += 1
        return partials if mode == 1 else out

    def linear_tiles(self, a, w, swiglu=False):
        """The many-rows tcgen05 product (csrc/gemm_tcgen05.cu): a . w^T in bfloat16, or, with `swiglu`,
        silu(a . Wg^T) * (a . Wu^T) for w = [Wg; Wu] stacked, without the [T, 2 I] round trip."""
        T, K = a.shape
        _need(a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16, "linear_tiles: bfloat16 only")
        _need(a.is_contiguous() and w.is_contiguous() and w.shape[1] == K and K % 8 == 0, "linear_tiles: bad operands")
        N = w.shape[0] // 2 if swiglu else w.shape[0]
        out = torch.empty((T, N), dtype=torch.bfloat16, device=a.device)
        _check(self.lib.ifx_gemm_tcgen05(_ptr(a), _ptr(w), _ptr(out), T, N, K, w.shape[0], int(bool(swiglu)),
                                         N if swiglu else 0, _ptr(self.error_flag), _stream()), "gemm_tcgen05")
        self.launches += 1
        return out

    def linear_generic(self, a, w, bias=None, out_dtype=None):
        """The CUDA-core product for any dtype (used by tests and as the refusal-free path)."""
        T, K = a.shape
        N = w.shape[0]
        out_dtype = out_dtype or a.dtype
        out = torch.empty((T, N), dtype=out_dtype, device=a.device)
        _check(self.lib.ifx_gemm_generic(_ptr(a), _ptr(w), _ptr(bias), _ptr(out), T, N, K, _DT[a.dtype],
                                         _DT[out_dtype], _stream()), "gemm_generic")
        self.launches += 1
        return out

    # ------------------------------------------------------------ whole layers
    def _native_parts(self, block):
        """The block's (mixer, ffn, norm before the mixer, norm before the ffn) if it is exactly the arrangement
        and the parts that csrc/layer_forward.cu runs (no subclass: one may have changed a forward), else None."""
        known = getattr(block, "_native_parts", False)
        if known is not False:
            return known
        from ..parts.attention import Attention
        from ..parts.block import PreNormBlock
        from ..parts.mlp import SwiGLU
        from ..parts.norm import RMSNorm
        parts = None
        if type(block) is PreNormBlock:
            m, f, n1, n2 = block.mixer, block.ffn, block.norm_mixer, block.norm_ffn
            if (type(m) is Attention and type(f) is SwiGLU and type(n1) is RMSNorm and type(n2) is RMSNorm
                    and m.hidden == f.hidden == n1.size == n2.size):
                parts = (m, f, n1, n2)
        block._native_parts = parts
        block._native_layers = {}
        return parts

    def _native_workspace(self, T, parts):
        m, f = parts[0], parts[1]
        need = int(self.lib.ifx_layer_workspace_bytes(T, m.hidden, m.nq * m.d, m.nkv * m.d, f.inter, self.SKINNY_MAX_ROWS))
        ws = self._layer_ws
        if ws is None or ws.numel() < need:
            if torch.cuda.is_current_stream_capturing():
                return None                              # no allocation inside a graph: the parts run one by one
            # graphs captured earlier hold the old one's address: it stays alive
            ws = torch.empty(max(need, 2 * (0 if ws is None else ws.numel())), dtype=torch.uint8, device=self.device)
            self._layer_ws_all.append(ws)
            self._layer_ws = ws
            self._layer_views = {}
        return ws

    def _native_layer_args(self, block, parts, ctx, cache):
        """The C structure of one layer with one cache (sizes, constants, weight and cache addresses), made when
        the pair first runs and kept on the block; None if the cache or the weights are not bfloat16."""
        m, f, n1, n2 = parts
        tensors = (m.w_qkv, m.w_o, m.b_qkv, f.w_gate_up, f.w_down, n1.weight, n2.weight)
        kv, table = cache.kv, cache.block_table
        kv_ptr = kv.data_ptr()
        # everything of the cache that the structure holds: another runner may get the same addresses
        key = (kv_ptr, table.data_ptr(), cache.writes, cache.page_size, table.shape[1], kv.shape[0])
        entry = block._native_layers.get(key)
        if entry is None or any(a is not b for a, b in zip(entry[1], tensors)):
            if kv.dtype is not torch.bfloat16 or m.w_qkv.dtype is not torch.bfloat16:
                return None
            rotary = m.position.rotary(ctx.device) if m.position is not None else None
            la = _LayerArgs(
                hidden=m.hidden, inter=f.inter, nq=m.nq, nkv=m.nkv, d=m.d, window=int(m.window or 0),
                rot=0 if rotary is None else int(rotary.rotary_dim),
                interleaved=int(bool(rotary.interleaved)) if rotary is not None else 0,
                scale=m.scale, eps_in=n1.eps, eps_post=n2.eps, write_cache=int(bool(cache.writes)),
                norm_in_w=n1.weight.data_ptr(), norm_post_w=n2.weight.data_ptr(),
                b_qkv=0 if m.b_qkv is None else m.b_qkv.data_ptr(),
                inv_freq=0 if rotary is None else rotary.inv_freq.data_ptr(),
                w_qkv=m.w_qkv.data_ptr(), w_o=m.w_o.data_ptr(), w_gate_up=f.w_gate_up.data_ptr(),
                w_down=f.w_down.data_ptr(), kv_pool=kv_ptr, block_table=table.data_ptr(),
                max_blocks=table.shape[1], page_size=cache.page_size, num_pages=kv.shape[0])
            entry = (la, tensors, rotary, table, ctypes.byref(la))      # the tensors stay alive with the addresses
            if len(block._native_layers) >= 8:           # caches come and go with their runners
                block._native_layers.clear()
            block._native_layers[key] = entry
        return entry[4]

    def _native_step_args(self, ctx, device):
        """The C structure of the step's batch (metadata addresses, counts, this table's knobs), made at the
        step's first layer and kept on the context."""
        step = getattr(ctx, "_native_step", None)
        if step is None or step[1] is not ctx.positions or step[0].max_kv_len != ctx.max_kv_len:
            if "attn.prefill_tiles" not in ctx.extra:      # a step context built without the mixer as a provider
                for name, vals in self.attention_sections(ctx).items():
                    ctx.extra[name] = torch.tensor(vals, dtype=torch.int32, device=device)
                    ctx.extra_len[name] = len(vals)
            sa = _StepArgs(
                T=ctx.num_tokens, num_decode=ctx.extra_len["attn.decode_rows"],
                num_tiles=ctx.extra_len["attn.prefill_tiles"] // 4,
                max_kv_len=int(ctx.max_kv_len), positions=ctx.positions.data_ptr(), token_req=ctx.token_req.data_ptr(),
                req_slot=ctx.req_slot.data_ptr(), decode_rows=ctx.extra["attn.decode_rows"].data_ptr(),
                decode_meta=ctx.extra["attn.decode_meta"].data_ptr(),
                prefill_tiles=ctx.extra["attn.prefill_tiles"].data_ptr(), norm_sumsq=self._norm_sumsq.data_ptr(),
                norm_tickets=self._norm_tickets.data_ptr(), error_flag=self.error_flag.data_ptr(),
                skinny_max_rows=self.SKINNY_MAX_ROWS, swiglu_tiles=int(self.swiglu_tiles),
                swiglu_tiles_max_k=self.SWIGLU_TILES_MAX_K, tensor_core_prefill=int(self.tensor_core_prefill),
                overlap_attention=int(self.overlap_attention))
            step = ctx._native_step = (sa, ctx.positions, ctypes.byref(sa))
        return step[2]

    def fused_prenorm_layer(self, block, x, pending, ctx, cache):
        """One native call for a pre-norm layer of attention and SwiGLU in bfloat16: the kernels that the parts
        would launch one by one, chosen by the same rules, launched from csrc/layer_forward.cu.  Returns
        (x, the layer's last delta, unadded) or None if this block, dtype or cache is not what that code runs."""
        if not self.native_layers or ctx.dtype is not torch.bfloat16 or cache.kv is None or cache.block_table is None:
            return None
        parts = self._native_parts(block)
        if parts is None or x.dtype is not torch.float32:
            return None
        m, f, n1, n2 = parts
        if block.mixer is not m or block.ffn is not f or block.norm_mixer is not n1 or block.norm_ffn is not n2:
            block._native_parts = False                  # a part was exchanged: look again
            return self.fused_prenorm_layer(block, x, pending, ctx, cache)
        T = ctx.num_tokens
        ws = self._native_workspace(T, parts)
        if ws is None:
            return None
        layer = self._native_layer_args(block, parts, ctx, cache)
        if layer is None:
            return None
        step = self._native_step_args(ctx, x.device)
        io = self._layer_io
        io.x = x.data_ptr()
        if pending is None:
            io.pending_tensor, io.pending_parts, io.pending_splits = 0, 0, 0
        elif isinstance(pending, PartialSum):
            if tuple(pending.shape) != tuple(x.shape):
                return None
            io.pending_tensor, io.pending_parts, io.pending_splits = 0, pending.parts.data_ptr(), pending.splits
        else:
            if pending.dtype is not torch.bfloat16 or pending.shape != x.shape or not pending.is_contiguous():
                return None
            io.pending_tensor, io.pending_parts, io.pending_splits = pending.data_ptr(), 0, 0
        parity = self._layer_parity = 1 - self._layer_parity
        io.parity = parity
        io.ws, io.ws_bytes = ws.data_ptr(), ws.numel()
        rc = self.lib.ifx_layer_forward(step, layer, self._layer_io_ref, _stream())
        self.launches += io.launches
        self.library_calls += io.library_calls
        self.native_layer_calls += 1
        _check(rc, "layer (native)")
        view = (T, m.hidden, parity, io.out_splits)
        out = self._layer_views.get(view)
        if out is None:
            at = (io.out_parts or io.out_tensor) - ws.data_ptr()
            if io.out_splits:
                n = io.out_splits * T * m.hidden * 4
                out = PartialSum(ws[at:at + n].view(torch.float32).view(io.out_splits, T, m.hidden), torch.bfloat16)
            else:
                out = ws[at:at + T * m.hidden * 2].view(torch.bfloat16).view(T, m.hidden)
            self._layer_views[view] = out
        return x, out

    # --------------------------------------------------------------- attention
    PREFILL_TILE = 256         # query rows per work item of the prompt-portion attention kernels

    def attention_sections(self, ctx):
        """Work lists of the attention kernels for one step, from the step's spans:
        attn.decode_rows[D] (flat indices of spans of one token), attn.decode_meta[D,4] (flat index,
        position, slot, 0: what the decode kernel needs of a token, in one 16-byte load),
        attn.prefill_tiles[P,4] (request, first flat row, rows, first position) for longer spans."""
        rows, meta, tiles, base = [], [], [], 0
        for r, ((start, n), slot) in enumerate(zip(ctx.spans, ctx.slots_host)):
            if n == 1:
                rows.append(base)
                meta.extend((base, start, int(slot), 0))
            else:
                for off in range(0, n, self.PREFILL_TILE):
                    tiles.extend((r, base + off, min(self.PREFILL_TILE, n - off), start + off))
            base += n
        return {"attn.decode_rows": rows, "attn.decode_meta": meta, "attn.prefill_tiles": tiles}

    @staticmethod
    def small_attention_grid(ctx, nkv):
        """1 if the step is decoded tokens only and their attention grid (tokens x kv heads x up to 8 key slices)
        leaves SMs free: the rotation kernel then lets it in early."""
        extra_len = getattr(ctx, "extra_len", None) or {}
        if "attn.decode_rows" not in extra_len:
            return 0
        return int(extra_len.get("attn.prefill_tiles", 0) == 0 and extra_len["attn.decode_rows"] * nkv * 8 <= 148)

    def rope_append(self, qkv, bias, rotary, nq, nkv, d, ctx, cache):
        """`qkv`: the stacked projections [T, (nq + 2 nkv) d] as a tensor or a PartialSum."""
        partial, splits = None, 0
        if isinstance(qkv, PartialSum):
            partial, splits, dtype, device = qkv.parts, qkv.splits, qkv.dtype, qkv.parts.device
            T, width = qkv.shape
            qkv = None
        else:
            dtype, device = qkv.dtype, qkv.device
            T, width = qkv.shape
        _need(width == (nq + 2 * nkv) * d, "rope_append: qkv width does not fit the head counts")
        q_out = torch.empty((T, nq * d), dtype=dtype, device=device)
        write = bool(cache.writes and cache.kv is not None)
        kv, table = cache.kv, cache.block_table
        if write:
            _need(kv.dtype == dtype, f"rope_append: cache is {kv.dtype}, activations {dtype}")
        rot = 0 if rotary is None else int(rotary.rotary_dim)
        _need(rot <= d, "rope_append: rotary_dim exceeds the head size")
        _check(self.lib.ifx_rope_append(
            _ptr(qkv), _ptr(partial), splits, _ptr(bias), _ptr(None if rotary is None else rotary.inv_freq), rot,
            int(bool(rotary.interleaved)) if rotary is not None else 0,
            _ptr(ctx.positions), _ptr(ctx.token_req), _ptr(ctx.req_slot), _ptr(table),
            0 if table is None else table.shape[1], cache.page_size, 0 if kv is None else kv.shape[0],
            _ptr(kv), _ptr(q_out), T, nq, nkv, d, int(write), self.small_attention_grid(ctx, nkv), _DT[dtype],
            _stream()), "rope_append")
        self.launches += 1
        return q_out

    def attention(self, q, nq, nkv, d, window, scale, ctx, cache):
        """Every token attends its request's keys up to its own position (or the last
        `window` of them) through the block table.  float32: the per-token kernel
        whose additions depend on the position only.  bfloat16: the tiled kernels,
        one launch for the prompt portions and one for the single decoded tokens."""
        T = q.shape[0]
        kv, table = cache.kv, cache.block_table
        _need(kv is not None and table is not None, "attention: the mixer has no key/value cache")
        _need(kv.dtype == q.dtype, f"attention: cache is {kv.dtype}, queries {q.dtype}")
        _need(d % 8 == 0 and d <= 256, f"attention: head size {d} is not a multiple of 8 up to 256")
        _need(q.is_contiguous() and q.shape[1] == nq * d, "attention: queries must be one [tokens, heads * size] block")
        out = torch.empty((T, nq * d), dtype=q.dtype, device=q.device)
        win = 0 if window is None else int(window)
        common = (cache.page_size, table.shape[1], kv.shape[0], win, ctypes.c_float(scale))
        tiled = q.dtype == torch.bfloat16 and bool(self.lib.ifx_attention_mma_supports(d))
        if "attn.prefill_tiles" not in ctx.extra:          # a step context built without the mixer as a provider
            for name, vals in self.attention_sections(ctx).items():
                ctx.extra[name] = torch.tensor(vals, dtype=torch.int32, device=q.device)
                ctx.extra_len[name] = len(vals)
        tiles, num_tiles = ctx.extra["attn.prefill_tiles"], ctx.extra_len["attn.prefill_tiles"] // 4
        decode_rows, decode_meta = ctx.extra["attn.decode_rows"], ctx.extra["attn.decode_meta"]
        if not tiled:
            self._attention_generic(q, kv, table, ctx, None, T, out, nq, nkv, d, common)
            return out
        if num_tiles and self.tensor_core_prefill and self.lib.ifx_attention_prefill_tcgen05_supports(
                d, cache.page_size):
            _check(self.lib.ifx_attention_prefill_tcgen05(
                _ptr(q), T, _ptr(kv), _ptr(table), _ptr(tiles), _ptr(ctx.req_slot), _ptr(out),
                num_tiles, nq, nkv, d, *common, _ptr(self.error_flag), _stream()),
                "attention (prompt portions, tcgen05)")
            self.launches += 1
        elif num_tiles:
            _check(self.lib.ifx_attention_prefill_bf16(
                _ptr(q), _ptr(kv), _ptr(table), _ptr(tiles), _ptr(ctx.req_slot), _ptr(out),
                num_tiles, nq, nkv, d, *common, int(ctx.max_kv_len), _ptr(self.error_flag), _stream()),
                "attention (prompt portions)")
            self.launches += 1
        n = ctx.extra_len["attn.decode_rows"]
        if n:
            if nq // nkv > 16:
                self._attention_generic(q, kv, table, ctx, decode_rows, n, out, nq, nkv, d, common)
                return out
            max_keys = int(ctx.max_kv_len if not win else min(win, ctx.max_kv_len))
            splits = self.decode_splits(n, nkv, max_keys, int(self.lib.ifx_attention_decode_max_splits(d, cache.page_size)))
            _check(self.lib.ifx_attention_decode_bf16(
                _ptr(q), _ptr(kv), _ptr(table), _ptr(decode_meta), _ptr(out), n, nq, nkv, d, *common, splits,
                max_keys, _ptr(self.error_flag), _stream()), "attention (decoded tokens)")
            self.launches += 1
        return out

    @staticmethod
    def decode_splits(num_tokens, nkv, max_keys, max_splits=8):
        """Into how many thread blocks (one cluster: 1, 2, 4, 8, or 16 where the kernel takes it) the
        key range of a decoded token is cut: as many blocks as the 148 SMs hold at once (two each), but
        at least 128 keys per block.  Clusters of 16 only while all of them fit on the SMs at once (measured:
        8.3 against 11.0 us for one token of the 7B shape at 4,096 keys, but 20 against 14 us for 16 clusters)."""
        want = max(1, 296 // max(1, num_tokens * nkv))           # all blocks resident at once: two a SM
        limit = max(1, min(want, max_keys // 128, max_splits))
        splits = 1
        while splits * 2 <= limit:
            splits *= 2
        if splits > 8 and num_tokens * nkv * splits > 148:
            splits = 8
        return splits

    def _attention_generic(self, q, kv, table, ctx, rows, count, out, nq, nkv, d, common):
        _check(self.lib.ifx_attention_generic(
            _ptr(q), _ptr(kv), _ptr(table), _ptr(ctx.positions), _ptr(ctx.token_req), _ptr(ctx.req_slot),
            _ptr(rows), _ptr(out), count, nq, nkv, d, *common, _DT[q.dtype], _stream()), "attention")
        self.launches += 1

    # ---------------------------------------------------------------- sampling
    def argmax(self, logits):
        R, V = logits.shape
        out = torch.empty((R,), dtype=torch.int32, device=logits.device)
        if V >= 16384 and R <= 256:                      # long rows, few of them: many blocks per row
            _check(self.lib.ifx_argmax_chunks(_ptr(logits), _ptr(out), R, V, 32, _ptr(self._argmax_val),
                                              _ptr(self._argmax_idx), _ptr(self._argmax_tickets), _stream()), "argmax")
            self.launches += 1
            return out
        _check(self.lib.ifx_argmax(_ptr(logits), _ptr(out), R, V, _stream()), "argmax")
        self.launches += 1
        return out

    def penalties(self, logits, tokens, counts, rep, freq, pres):
        R, V = logits.shape
        _check(self.lib.ifx_penalties(_ptr(logits), _ptr(tokens), _ptr(counts), _ptr(rep), _ptr(freq), _ptr(pres),
                                      R, tokens.shape[1], V, _stream()), "penalties")
        self.launches += 1

    def logit_bias(self, logits, rows, tokens, bias):
        R, V = logits.shape
        _check(self.lib.ifx_logit_bias(_ptr(logits), _ptr(rows), _ptr(tokens), _ptr(bias), rows.numel(), R, V,
                                       _stream()), "logit_bias")
        self.launches += 1

    def sample(self, logits, temperature, top_k, top_p, min_p, seed_lo, seed_hi, step, features=3):
        """One draw per row (see sampling.cu).  Rows are spread over many blocks; `features` says which
        filters any row uses (bit 0: top-k, bit 1: top-p) so that the passes of the others are not launched."""
        R, V = logits.shape
        out = torch.empty((R,), dtype=torch.int32, device=logits.device)
        if R > self._sample_capacity:                    # the scratch's layout goes with its capacity
            self._sample_capacity = max(64, 1 << (R - 1).bit_length())
            self._sample_scratch = torch.zeros(int(self.lib.ifx_sample_scratch_bytes(self._sample_capacity)),
                                               dtype=torch.uint8, device=logits.device)
        passes = 3 + (1 if features & 3 else 0) + (2 if features & 1 else 0) + (3 if features & 2 else 0)
        _check(self.lib.ifx_sample_blocks(_ptr(logits), _ptr(temperature), _ptr(top_k), _ptr(top_p), _ptr(min_p),
                                          _ptr(seed_lo), _ptr(seed_hi), _ptr(step), _ptr(out), R, V, int(features),
                                          _ptr(self._sample_scratch), self._sample_capacity, _stream()), "sample")
        self.launches += passes
        return out

    def sample_one_block(self, logits, temperature, top_k, top_p, min_p, seed_lo, seed_hi, step):
        """The same draw with one block per row and thresholds by bisection (kept for comparison)."""
        R, V = logits.shape
        probs = torch.empty((R, V), dtype=torch.float32, device=logits.device)
        out = torch.empty((R,), dtype=torch.int32, device=logits.device)
        _check(self.lib.ifx_sample(_ptr(logits), _ptr(probs), _ptr(temperature), _ptr(top_k), _ptr(top_p),
                                   _ptr(min_p), _ptr(seed_lo), _ptr(seed_hi), _ptr(step), _ptr(out), R, V,
                                   _stream()), "sample")
        self.launches += 1
        return out
