"""Python faces of the CUDA kernels.

Each function checks shapes and dtypes, then calls one launcher of the kernel
library through its C symbol on torch's current stream.  Nothing here computes:
there is no CPU or library fallback, and a missing or unloadable library is an
error at first use.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from . import build as _build

ACT_NONE, ACT_GELU_TANH, ACT_GELU_ERF, ACT_RELU_SQ, ACT_SILU, ACT_SWIGLU_CAPPED = 0, 1, 2, 3, 4, 5
#: (the products' epilogues take all but "silu", which the element-wise and expert kernels apply, and
#: "swiglu_capped", a rule for a gated unit's gate and value together that the expert kernels apply)
ACT_CODES = {None: ACT_NONE, "none": ACT_NONE, "tanh": ACT_GELU_TANH, "erf": ACT_GELU_ERF, "relu2": ACT_RELU_SQ,
             "silu": ACT_SILU, "swiglu_capped": ACT_SWIGLU_CAPPED}
UNARY_TANH, UNARY_XIELU, UNARY_SOFTCAP, UNARY_SCALE = 1, 2, 3, 4

STATUS_OK, STATUS_BAD_PAGE, STATUS_WAIT_TIMEOUT = 0, 1, 2
_ERR_NAMES = {-1: "bad argument", -2: "unsupported size", -3: "CUDA driver call failed"}


class KernelError(RuntimeError):
    pass


_lib = None

_c_int, _c_float, _c_ptr = ctypes.c_int, ctypes.c_float, ctypes.c_void_p

_SIGNATURES = {
    "nib_embed": [_c_int, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_int, _c_float, _c_ptr],
    "nib_layernorm": [_c_int, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_int, _c_float, _c_ptr],
    "nib_kv_append": [_c_int, _c_ptr, _c_int, _c_int, _c_int, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_ptr,
                      _c_int, _c_int, _c_int, _c_int, _c_int, _c_ptr, _c_ptr],
    "nib_linear_simt": [_c_int, _c_int, _c_ptr, _c_int, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_int,
                        _c_int, _c_int, _c_int, _c_int, _c_int, _c_ptr],
    "nib_linear_tc_supported": [_c_ptr, _c_int, _c_ptr, _c_int, _c_int],
    "nib_linear_tc": [_c_int, _c_ptr, _c_int, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_int,
                      _c_int, _c_int, _c_ptr, _c_ptr],
    "nib_linear_tc_small": [_c_int, _c_ptr, _c_int, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_int,
                            _c_int, _c_int, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_float, _c_ptr, _c_ptr, _c_ptr,
                            _c_int, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_ptr,
                            ctypes.c_longlong, _c_ptr, _c_int, _c_ptr, _c_ptr],
    "nib_linear_tc_pair_supported": [_c_int, _c_ptr, _c_int, _c_ptr, _c_int, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_int],
    "nib_linear_tc_pair": [_c_int, _c_ptr, _c_int, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_int,
                           _c_int, _c_int, _c_int, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_int, _c_int, _c_int,
                           _c_int, _c_int, _c_ptr, _c_ptr],
    "nib_linear_skinny_supported": [_c_int, _c_int, _c_int, _c_int, _c_ptr],
    "nib_linear_skinny": [_c_int, _c_ptr, _c_int, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_int,
                          _c_int, _c_int, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_float, _c_ptr, _c_ptr, _c_ptr,
                          _c_int, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_ptr, _c_ptr],
    "nib_attention_prefill_tc_supported": [_c_int, _c_int],
    "nib_attention_prefill_tc": [_c_ptr, _c_int, _c_int, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_int, _c_ptr, _c_int, _c_ptr,
                                 _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_int, _c_int, _c_float, _c_int,
                                 _c_ptr, _c_ptr, _c_int, _c_float, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_ptr],
    "nib_attention_simt": [_c_int, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_ptr,
                           _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_int, _c_int, _c_float, _c_int,
                           _c_ptr, _c_ptr, _c_int, _c_float, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_ptr],
    "nib_attention_decode": [_c_int, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_int, _c_ptr, _c_ptr,
                             _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_int, _c_int, _c_float,
                             _c_int, _c_ptr, _c_ptr, _c_int, _c_float, _c_int, _c_ptr, _c_ptr, _c_int, _c_int, _c_ptr, _c_ptr,
                             _c_ptr],
    "nib_attention_decode_mma_supported": [_c_int, _c_int],
    "nib_attention_decode_mma_clusters": [_c_int, _c_int],
    "nib_attention_decode_mma": [_c_ptr, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_ptr,
                                 _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_int, _c_int, _c_int, _c_int,
                                 _c_ptr, _c_ptr, _c_int, _c_int, _c_ptr],
    "nib_attention_prefill_supported": [_c_int],
    "nib_attention_prefill": [_c_ptr, _c_int, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_int, _c_ptr, _c_int, _c_ptr, _c_ptr,
                              _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_int, _c_int, _c_float, _c_int,
                              _c_ptr, _c_ptr, _c_int, _c_float, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_ptr],
    "nib_convert": [_c_int, _c_ptr, _c_int, _c_int, _c_int, _c_ptr, ctypes.c_longlong, ctypes.c_longlong, _c_int, _c_ptr],
    "nib_argmax": [_c_ptr, _c_int, _c_int, _c_int, _c_ptr, _c_ptr],
    "nib_sample": [_c_ptr, _c_int, _c_int, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int,
                   _c_ptr],
    "nib_rmsnorm": [_c_int, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_int, _c_float, _c_ptr],
    "nib_stream_enter": [_c_int, _c_ptr, _c_ptr, _c_ptr, _c_float, _c_int, _c_int, _c_ptr],
    "nib_post_norm": [_c_int, _c_ptr, _c_ptr, _c_float, _c_ptr, ctypes.c_longlong, _c_int, _c_ptr, _c_ptr, _c_float,
                      _c_int, _c_int, _c_ptr],
    "nib_unary": [_c_int, _c_int, _c_ptr, _c_int, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_ptr, _c_ptr],
    "nib_latent_prep": [_c_int, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_float,
                        _c_ptr, _c_int, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_int,
                        _c_ptr, _c_ptr],
    "nib_rope_heads": [_c_int, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_int,
                       _c_int, _c_int, _c_ptr],
    "nib_latent_attention": [_c_int, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_int,
                             _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_int, _c_ptr, _c_int, _c_ptr, _c_ptr],
    "nib_linear_heads": [_c_int, _c_int, _c_ptr, _c_int, _c_int, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_int,
                         _c_int, _c_int, _c_ptr],
    "nib_delta_rule": [_c_int, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_ptr, _c_int, _c_ptr,
                       _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_float, _c_ptr, _c_int,
                       _c_ptr, _c_ptr],
    "nib_moe_route": [_c_int, _c_ptr, _c_int, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_ptr, _c_int,
                      _c_ptr, _c_ptr, _c_ptr, _c_ptr],
    "nib_moe_up": [_c_int, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float,
                   _c_int, _c_ptr, _c_ptr],
    "nib_moe_gate_scale": [_c_int, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_int,
                           _c_float, _c_int, _c_ptr],
    "nib_add_norm": [_c_int, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_float, _c_ptr, _c_int, _c_int, _c_ptr],
    "nib_glu": [_c_int, _c_int, _c_ptr, _c_int, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_ptr],
    "nib_rope_append": [_c_int, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int,
                        _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_ptr,
                        _c_ptr],
    "nib_mlstm": [_c_int, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_ptr, _c_ptr, _c_float,
                  _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_ptr, _c_ptr,
                  _c_int, _c_ptr, _c_ptr, _c_int, _c_ptr],
    "nib_add_sinusoid": [_c_ptr, _c_ptr, _c_ptr, _c_int, _c_int, _c_ptr],
    "nib_gate_by_table": [_c_int, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_ptr, _c_int,
                          _c_int, _c_ptr],
    "nib_norm_rope_append": [_c_int, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_ptr,
                             _c_ptr, _c_float, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_int,
                             _c_int, _c_int, _c_int, _c_ptr, _c_ptr],
    "nib_short_conv": [_c_ptr, _c_int, _c_int, _c_int, _c_int, _c_ptr, _c_ptr, _c_ptr, ctypes.c_longlong, _c_ptr, _c_ptr,
                       _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_ptr, _c_int, _c_ptr],
    "nib_scan_prepare": [_c_ptr, _c_int, _c_int, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_int,
                         _c_int, _c_int, _c_ptr, _c_int, _c_ptr],
    "nib_gated_scan_padded": [_c_int],
    "nib_gated_scan": [_c_int, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_ptr, _c_ptr,
                       _c_ptr, ctypes.c_longlong, ctypes.c_longlong, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_int, _c_ptr],
    "nib_gated_norm": [_c_int, _c_ptr, _c_int, _c_ptr, _c_int, _c_ptr, _c_int, _c_int, _c_int, _c_float, _c_int, _c_float,
                       _c_ptr, _c_int, _c_int, _c_ptr],
    "nib_moe_down": [_c_int, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_ptr],
    "nib_moe_scale": [_c_int, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_ptr],
    "nib_moe_grouped": [_c_int, _c_int, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_int, _c_int,
                        _c_int, _c_int, _c_int, _c_float, _c_ptr],
    "nib_wide_norm_rope_append": [_c_int, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int,
                                  _c_ptr, _c_ptr, _c_float, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_ptr,
                                  _c_int, _c_int, _c_int, _c_int, _c_ptr, _c_ptr],
    "nib_rope_halves": [_c_ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_ptr, _c_ptr, _c_float, _c_ptr, _c_ptr,
                        _c_int, _c_ptr],
    "nib_hyper_enter": [_c_int, _c_ptr, _c_ptr, ctypes.c_longlong, _c_int, _c_ptr, _c_ptr, _c_float, _c_ptr, _c_int, _c_int,
                        _c_ptr],
    "nib_hyper_update": [_c_int, _c_ptr, ctypes.c_longlong, _c_int, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_ptr, _c_ptr,
                         _c_float, _c_ptr, _c_ptr, _c_int, _c_int, _c_ptr],
    "nib_selective_scan": [_c_int, _c_ptr, _c_int, _c_ptr, _c_int, _c_ptr, _c_int, _c_int, _c_int, _c_ptr, _c_int, _c_ptr,
                           _c_ptr, _c_ptr, ctypes.c_longlong, ctypes.c_longlong, _c_ptr, _c_ptr, _c_int, _c_int, _c_int,
                           _c_ptr, _c_int, _c_ptr],
}


#: the active trace recorder (``trace.start`` puts it here), or None
_rec = None


def _recorder():
    return _rec


#: the analytic description of the launch about to be made (set by the faces while a recorder is active)
_pending_op = None


def _note(kind: str, name: str, dims, flops: float, nbytes: float) -> None:
    global _pending_op
    from ..trace import Op
    _pending_op = Op(kind, name, tuple(int(d) for d in dims), float(flops), float(nbytes))


def tracing() -> bool:
    """Whether a trace recorder is active (the faces then describe every launch to it)."""
    return _rec is not None


def trace_scope(layer: int = -1, name: str = "") -> None:
    """Tell the active recorder which layer, and which named product, the next launches belong to."""
    if _rec is not None:
        _rec.layer, _rec.name = layer, name


class _Library:
    """The launchers of the kernel library; with a trace recorder active each call is bracketed by events."""

    def __init__(self, lib: ctypes.CDLL):
        for name, argtypes in _SIGNATURES.items():
            fn = getattr(lib, name)
            fn.argtypes = argtypes
            fn.restype = _c_int
            setattr(self, name, self._wrap(name, fn))
        self.raw = lib

    @staticmethod
    def _wrap(name, fn):
        counted = name not in ("nib_linear_tc_supported", "nib_linear_tc_pair_supported", "nib_linear_skinny_supported",
                               "nib_attention_prefill_tc_supported", "nib_attention_prefill_supported",
                               "nib_attention_decode_mma_supported", "nib_attention_decode_mma_clusters",
                               "nib_gated_scan_padded")

        def call(*args):
            global _pending_op
            rec = _recorder() if counted else None
            if rec is None:
                return fn(*args)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            code = fn(*args)
            e1.record()
            op, _pending_op = _pending_op, None
            if code == 0:
                if op is None:
                    from ..trace import Op
                    op = Op("other", name[4:], (0, 0, 0), 0.0, 0.0)
                rec.add(op, name, e0, e1)
            return code
        return call


def library() -> _Library:
    """The loaded kernel library; compiled on first use if the built file is missing."""
    global _lib
    if _lib is None:
        if not torch.cuda.is_available():
            raise KernelError("nanoinfer_b200 needs a CUDA device: there is no CPU path")
        path = _build.library_path(build=True)
        _lib = _Library(ctypes.CDLL(path))
    return _lib


_bound_stream: Optional[int] = None


def _stream() -> int:
    """The stream that kernels are enqueued on: torch's current stream, looked up once per step when
    the step function has bound it (the look-up costs more than a launch does)."""
    return _bound_stream if _bound_stream is not None else torch.cuda.current_stream().cuda_stream


class bound_stream:
    """``with bound_stream():`` every launch inside goes to the stream that is current on entry."""

    def __enter__(self):
        global _bound_stream
        self._before = _bound_stream
        _bound_stream = torch.cuda.current_stream().cuda_stream
        return self

    def __exit__(self, *exc):
        global _bound_stream
        _bound_stream = self._before
        return False


_launches = 0


def launch_count() -> int:
    """How many kernels this process has enqueued through this interface (captured launches count once)."""
    return _launches


def _check(code: int, what: str, kernels: int = 1) -> None:
    global _launches
    if code == 0:
        _launches += kernels
        return
    if code < 0:
        raise KernelError(f"{what}: {_ERR_NAMES.get(code, code)}")
    raise KernelError(f"{what}: CUDA error {code}")


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return 0
    if t.dtype == torch.bfloat16:
        return 1
    raise KernelError(f"dtype {t.dtype} is not supported by the kernels")


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _i32(t: torch.Tensor, name: str) -> None:
    if t.dtype != torch.int32 or not t.is_contiguous():
        raise KernelError(f"{name} must be a contiguous int32 tensor")


# ------------------------------------------------------------------------------ ops
def embed(tokens: torch.Tensor, table: torch.Tensor, out: torch.Tensor,
          pos_table: Optional[torch.Tensor] = None, positions: Optional[torch.Tensor] = None,
          feedback: Optional[torch.Tensor] = None, scale: float = 1.0) -> None:
    """out[t] = table[tokens[t]] * scale (+ pos_table[positions[t]]), written as 32-bit floats.  A negative
    token -(s + 1) stands for ``feedback[s]``, the token that the step before left on the device for
    slot s."""
    T, C = tokens.shape[0], table.shape[1]
    _i32(tokens, "tokens")
    if out.dtype != torch.float32 or out.shape[0] < T or out.shape[1] != C or not out.is_contiguous():
        raise KernelError("embed: out must be contiguous float32 [T, C]")
    if pos_table is not None:
        if positions is None or pos_table.dtype != table.dtype or pos_table.shape[1] != C:
            raise KernelError("embed: pos_table needs positions, the table's dtype and its width")
        _i32(positions, "positions")
    if feedback is not None:
        _i32(feedback, "feedback")
    if tracing():
        _note("embed", "embed", (T, C, 0), T * C, T * C * ((2 if pos_table is not None else 1) * table.element_size() + 4))
    _check(library().nib_embed(_dt(table), _ptr(tokens), _ptr(positions), _ptr(table), _ptr(pos_table),
                               _ptr(feedback), _ptr(out), T, C, float(scale), _stream()), "embed")


def layernorm(x: torch.Tensor, gamma: torch.Tensor, beta: torch.Tensor, eps: float, out: torch.Tensor,
              n_rows: int, rows: Optional[torch.Tensor] = None) -> None:
    """out[r] = LayerNorm(x[rows[r]] if rows is given else x[r]); x is the 32-bit residual stream."""
    C = x.shape[1]
    if x.dtype != torch.float32 or not x.is_contiguous():
        raise KernelError("layernorm: x must be contiguous float32")
    if gamma.dtype != torch.float32 or beta.dtype != torch.float32 or gamma.numel() != C or beta.numel() != C:
        raise KernelError("layernorm: gamma and beta must be float32 [C]")
    if out.shape[1] != C or out.shape[0] < n_rows or not out.is_contiguous():
        raise KernelError("layernorm: out must be contiguous [n_rows, C]")
    if rows is not None:
        _i32(rows, "rows")
    if tracing():
        _note("ln", "ln", (n_rows, C, 0), 8.0 * n_rows * C, n_rows * C * (4 + out.element_size()) + 8 * C)
    _check(library().nib_layernorm(_dt(out), _ptr(x), _ptr(rows), _ptr(gamma), _ptr(beta), _ptr(out),
                                   n_rows, C, float(eps), _stream()), "layernorm")


def linear_simt(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor, M: int,
                act: int = ACT_NONE, residual: bool = False) -> None:
    """out[:M] = act(a[:M] . w^T + bias) on the CUDA cores; with residual, added to the 32-bit out."""
    N, K = w.shape
    if a.shape[1] != K or a.dtype != w.dtype or a.stride(1) != 1 or w.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("linear: a [M, K] and w [N, K] must share K and dtype, rows contiguous")
    if out.shape[1] != N or out.shape[0] < M or a.shape[0] < M:
        raise KernelError("linear: out must be [M, N]")
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != N):
        raise KernelError("linear: bias must be float32 [N]")
    _check(library().nib_linear_simt(_dt(a), _dt(out), _ptr(a), a.stride(0), _ptr(w), w.stride(0), _ptr(bias),
                                     _ptr(out), out.stride(0), M, N, K, act, int(residual), _stream()),
           "linear_simt")


_status: Optional[torch.Tensor] = None


def status_word() -> torch.Tensor:
    """The device status word (int32 [1]) that kernels write when they meet a fault they can
    name (a page index outside its pool, a wait that ran out).  0 means fine."""
    global _status
    if _status is None:
        _status = torch.zeros(1, dtype=torch.int32, device="cuda")
    return _status


def linear_tc(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor, M: int,
              act: int = ACT_NONE, residual: bool = False) -> None:
    """out[:M] = act(a[:M] . w^T + bias) for bfloat16 a and w on the tensor cores (tcgen05, TMA)."""
    N, K = w.shape
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or a.shape[1] != K:
        raise KernelError("linear_tc: a [M, K] and w [N, K] must be bfloat16 and share K")
    if a.stride(1) != 1 or w.stride(1) != 1 or out.stride(1) != 1 or out.shape[1] != N or out.shape[0] < M:
        raise KernelError("linear_tc: rows must be contiguous and out [M, N]")
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != N):
        raise KernelError("linear_tc: bias must be float32 [N]")
    _check(library().nib_linear_tc(_dt(out), _ptr(a), a.stride(0), _ptr(w), w.stride(0), _ptr(bias), _ptr(out),
                                   out.stride(0), M, N, K, act, int(residual), _ptr(status_word()), _stream()),
           "linear_tc")


_capability: dict = {}


def _can(name: str, *args) -> bool:
    """A capability query of the library, remembered: the answers depend on sizes and alignments
    only, and a foreign-function call costs about as much as a launch."""
    key = (name,) + args
    got = _capability.get(key)
    if got is None:
        got = _capability[key] = bool(getattr(library(), name)(*args))
    return got


def linear_tc_supported(a: torch.Tensor, w: torch.Tensor) -> bool:
    return bool(a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and a.stride(1) == 1 and w.stride(1) == 1
                and _can("nib_linear_tc_supported", 16 + (_ptr(a) & 15), a.stride(0), 16 + (_ptr(w) & 15), w.stride(0),
                         w.shape[1]))   # (only the alignment of the pointers matters: 16 + the low bits)


def linear_tc_pair(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor, M: int,
                   act: int = ACT_NONE, residual: bool = False, bq: int = 0, splits: int = 0, kv=None) -> bool:
    """The tcgen05 product for many rows by pairs of blocks (one 256-row MMA over two SMs, each block
    loading half of the weight tile).  ``kv``: (cache layer, block table, row_entry, positions, q_dim)
    sends keys and values straight to the cache.  False if the shape or an alignment is not taken."""
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or a.stride(1) != 1 or w.stride(1) != 1 \
            or out.stride(1) != 1 or out.dtype not in (torch.bfloat16, torch.float32):
        return False
    N, K = w.shape
    if not _can("nib_linear_tc_pair_supported", _dt(out), 16 + (_ptr(a) & 15), a.stride(0), 16 + (_ptr(w) & 15),
                w.stride(0), 16 + (_ptr(out) & 15), out.stride(0), M, N, K, int(residual)):
        return False
    _, kv_args = _option_args(None, kv)
    if kv is not None and (kv[4] % 64 or kv[0].shape[4] % 16 or out.dtype != torch.bfloat16 or residual):
        return False
    if tracing():
        _note_linear(a, None, w, bias, out, M, residual)
    _check(library().nib_linear_tc_pair(_dt(out), _ptr(a), a.stride(0), _ptr(w), w.stride(0), _ptr(bias), _ptr(out),
                                        out.stride(0), M, N, K, act, int(residual), int(bq), int(splits), *kv_args,
                                        _ptr(status_word()), _stream()), "linear_tc_pair")
    return True


def _note_linear(a, norm, w, bias, out, M, residual) -> None:
    """[M, K, N]: 2 M K N + M N FLOPs; weights, bias, input and output once (the residual stream is read
    and written where the product adds into it)."""
    N, K = w.shape
    in_bytes = M * K * (4 if norm is not None else a.element_size())
    out_bytes = M * N * out.element_size() * (2 if residual else 1)
    _note("matmul", "matmul", (M, K, N), 2.0 * M * K * N + M * N,
          N * K * w.element_size() + (4 * N if bias is not None else 0) + in_bytes + out_bytes)


class NormInput:
    """Activations given as the 32-bit residual stream plus the parameters of the LayerNorm that
    stands before the product: ``linear`` normalises ``x[rows[m]]`` (or ``x[m]``) itself, inside the
    tensor-core kernel where the step is small enough, else with the LayerNorm kernel into scratch
    taken from ``workspace``."""

    def __init__(self, x: torch.Tensor, gamma: torch.Tensor, beta: torch.Tensor, eps: float, workspace,
                 dtype: torch.dtype, rows: Optional[torch.Tensor] = None, max_rows: int = 0):
        self.x, self.gamma, self.beta, self.eps = x, gamma, beta, float(eps)
        self.workspace, self.dtype, self.rows, self.max_rows = workspace, dtype, rows, max_rows

    def materialise(self, M: int) -> torch.Tensor:
        out = self.workspace.get("norm.fallback", (max(M, self.max_rows), self.x.shape[1]), self.dtype)
        layernorm(self.x, self.gamma, self.beta, self.eps, out, M, self.rows)
        return out


SMALL_STEP_MAX_ROWS = 128
_split_scratch: Optional[torch.Tensor] = None
_split_counters: Optional[torch.Tensor] = None


def _split_buffers(device):
    """Scratch for the K splits of small steps: 4 M floats of partial tiles and 4096 tile counters
    (found zero and left zero by the kernel), allocated once."""
    global _split_scratch, _split_counters
    if _split_scratch is None:
        _split_scratch = torch.empty(4 << 20, dtype=torch.float32, device=device)
        _split_counters = torch.zeros(4096, dtype=torch.int32, device=device)
    return _split_scratch, _split_counters


def _option_args(norm, kv):
    if kv is not None:
        cache, block_table, row_entry, positions, q_dim = kv
        n_pages, _, n_kv_head, page_size, head_dim = cache.shape
        kv_args = (_ptr(cache), _ptr(block_table), block_table.shape[1], _ptr(row_entry), _ptr(positions), q_dim,
                   n_kv_head, head_dim, page_size, n_pages)
    else:
        kv_args = (None, None, 0, None, None, 0, 0, 0, 0, 0)
    if norm is not None:
        ln_args = (_ptr(norm.x), norm.x.stride(0), _ptr(norm.gamma), _ptr(norm.beta), norm.eps, _ptr(norm.rows))
    else:
        ln_args = (None, 0, None, None, 0.0, None)
    return ln_args, kv_args


def _small_inputs_ok(a, norm, w, out) -> bool:
    if w.dtype != torch.bfloat16 or w.stride(1) != 1 or out.stride(1) != 1:
        return False
    if a is not None and (a.dtype != torch.bfloat16 or a.stride(1) != 1):
        return False
    if norm is not None and (norm.x.dtype != torch.float32 or norm.x.stride(1) != 1):
        return False
    return a is not None or norm is not None


SKINNY_MAX_ROWS = 128
#: most rows of a step for which the dispatcher lets the few-row kernel normalise the rows itself (every
#: row block of 16 its own rows: 24 launches fewer than with the norm as a kernel of its own)
SKINNY_LN_MAX_ROWS = 128
#: widest row that the few-row kernel normalises in a lane's registers
SKINNY_LN_REGISTER_WIDTH = 1024
PAIR_MIN_ROWS = 256      # the pair kernel's smallest step


def pair_pays(M: int, N: int, K: int) -> bool:
    """Whether a product runs faster by pairs of blocks (one 256-row MMA over two SMs) than on the
    single-block kernel: always from 1536 rows on (measured in whole prefill steps of 2048 rows at
    three model sizes); below that from about one wave of tiles on, or with enough work per output
    (measured alone at widths 768, 1024 and 1600 for the four products of a layer at 256 to 1280 rows)."""
    return M >= 1536 or (M >= PAIR_MIN_ROWS and (M * N >= 3_000_000 or M * N * K >= 3_500_000_000))


def linear_skinny(a, norm, w, bias, out, M, act=ACT_NONE, residual=False, kv=None, split=0) -> bool:
    """The warp-level MMA kernel for steps of at most 128 rows (bfloat16): every SM streams weight
    rows, a few multiply-adds per weight.  ``norm``: the LayerNorm before the product, folded in; ``kv``: (cache layer, block table, row_entry, positions, q_dim) sends keys and
    values straight to the cache; ``split``: blocks of a cluster that split K (0: chosen by the
    library).  False if the kernel does not apply."""
    if M > SKINNY_MAX_ROWS or not _small_inputs_ok(a, norm, w, out):
        return False
    N, K = w.shape
    lib = library()
    if not _can("nib_linear_skinny_supported", M, K, w.stride(0), int(norm is not None), 16 + (_ptr(w) & 15)):
        return False
    ln_args, kv_args = _option_args(norm, kv)
    if tracing():
        _note_linear(a, norm, w, bias, out, M, residual)
    code = lib.nib_linear_skinny(_dt(out), _ptr(a), a.stride(0) if a is not None else 0, _ptr(w), w.stride(0),
                                 _ptr(bias), _ptr(out), out.stride(0), M, N, K, act, int(residual), *ln_args,
                                 *kv_args, int(split), _ptr(status_word()), _stream())
    if code == -2:   # alignment or size not taken
        return False
    _check(code, "linear_skinny")
    return True


def linear_small_tc(a, norm, w, bias, out, M, act=ACT_NONE, residual=False, kv=None, split=True) -> bool:
    """The tensor-core kernel for steps of at most 128 rows with its options: ``norm`` folds the
    LayerNorm before the product into the kernel, ``kv`` sends keys and values straight to the
    cache, ``split`` lets K be split over blocks through scratch.  False if it does not apply."""
    if M > SMALL_STEP_MAX_ROWS or not _small_inputs_ok(a, norm, w, out):
        return False
    N, K = w.shape
    lib = library()
    if not lib.nib_linear_tc_supported(_ptr(a), a.stride(0) if a is not None else 0, _ptr(w), w.stride(0), K):
        return False
    parts, counters = _split_buffers(w.device) if split else (None, None)
    ln_args, kv_args = _option_args(norm, kv)
    if tracing():
        _note_linear(a, norm, w, bias, out, M, residual)
    code = lib.nib_linear_tc_small(_dt(out), _ptr(a), a.stride(0) if a is not None else 0, _ptr(w), w.stride(0),
                                   _ptr(bias), _ptr(out), out.stride(0), M, N, K, act, int(residual), *ln_args,
                                   *kv_args, _ptr(parts), parts.numel() if split else 0, _ptr(counters),
                                   counters.numel() if split else 0, _ptr(status_word()), _stream())
    if code == -2:   # the shape is not taken by the small-step kernel
        return False
    _check(code, "linear_tc_small")
    return True


#: most rows for which the tcgen05 kernel writes keys and values from its epilogue (its swapped orientation)
TC_KV_EPILOGUE_MAX_ROWS = 16


def skinny_pays(M: int, N: int, K: int) -> bool:
    """Whether a product of at most 128 rows goes to the warp-level MMA kernel rather than to tcgen05.
    Measured in whole decode steps at widths 768, 1024 and 1600 (batch 16 to 64): up to 16 rows the MMA
    kernel wins everywhere; up to 32 rows everywhere but the longest rows (K of 4096 and more, split over a
    cluster: GPT-2 medium's second MLP product at 32 rows is 4 % of a step slower here, XL's 20 %) and the
    widest outputs (the head), where its 16-feature tiles read the rows too often; beyond 32 rows while a row
    block holds its rows unsplit.  Flipping one product's choice at a time at 24 to 128 rows and three widths
    moves a step by less than 5 % where the other choice is better and by up to 97 % where it is worse."""
    if M <= 16:
        return True
    if N > 8192 or M > SKINNY_MAX_ROWS:
        return False
    # (33 to 128 rows: while a row block holds its rows unsplit, K up to about a thousand.  The MLP's second
    # product at GPT-2 medium's sizes, K = 4096, on tcgen05 instead: a decode step of 64 rows 1.17 against 1.37 ms)
    return K <= (3072 if M <= 32 else 1088)


def _linear_small(a, norm, w, bias, out, M, act, residual, kv=None) -> bool:
    """Steps of at most 128 rows: the warp-level MMA kernel (with the LayerNorm folded in) where
    ``skinny_pays``, else tcgen05.  Folding the norm into the tcgen05 kernel, or splitting
    K through scratch, costs more round trips than it saves at these sizes, so that kernel is given
    normed rows and is not split here."""
    N, K = w.shape
    mma = skinny_pays(M, N, K)
    if mma:
        # (rows wider than SKINNY_LN_REGISTER_WIDTH are normalised through a buffer per warp in shared memory, which
        # leaves room for one block an SM from 9 rows on: GPT-2 XL at batch 12 to 32 is 2 to 7 % faster with the
        # norm as a kernel of its own there)
        if norm is not None and (M > SKINNY_LN_MAX_ROWS or (K > SKINNY_LN_REGISTER_WIDTH and M > 8)):
            a, norm = norm.materialise(M), None
        if linear_skinny(a, norm, w, bias, out, M, act, residual, kv):
            return True
        if norm is not None:   # too wide or too many rows to be normalised inside the kernel: normalise first
            a, norm = norm.materialise(M), None
            if linear_skinny(a, None, w, bias, out, M, act, residual, kv):
                return True
    if M > TC_KV_EPILOGUE_MAX_ROWS or kv is None:
        return False          # the plain tensor-core call does as well
    if norm is not None:
        a, norm = norm.materialise(M), None
    return linear_small_tc(a, norm, w, bias, out, M, act, residual, kv, split=False)


def linear(a: Optional[torch.Tensor], w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor, M: int,
           act: int = ACT_NONE, residual: bool = False, norm: Optional[NormInput] = None) -> None:
    """The matrix product of the model: out[:M] = act(a[:M] . w^T + bias), added to the 32-bit
    ``out`` with ``residual``.  With ``norm`` the activations are LayerNorm of the residual stream
    (``a`` is then None).  bfloat16 runs on the tensor cores where shape and alignment allow (rows
    of 16-byte multiples), else on the CUDA cores; float32 always runs on the CUDA cores in true
    32-bit arithmetic."""
    if _linear_small(a, norm, w, bias, out, M, act, residual):
        return
    if norm is not None:
        a = norm.materialise(M)   # (scratch: a second call for the same rows rewrites the same values)
    if tracing():
        _note_linear(a, None, w, bias, out, M, residual)
    # pairs of blocks on one 256-row MMA (half of the weight tile per SM) beat the single-block kernel
    # by 5 to 40 per cent where there is enough work
    if pair_pays(M, w.shape[0], w.shape[1]) and linear_tc_pair(a, w, bias, out, M, act, residual):
        return
    if linear_tc_supported(a, w):
        linear_tc(a, w, bias, out, M, act, residual)
    else:
        linear_simt(a, w, bias, out, M, act, residual)


def linear_qkv(a: Optional[torch.Tensor], w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor, M: int,
               q_dim: int, cache: torch.Tensor, block_table: torch.Tensor, row_entry: torch.Tensor,
               positions: torch.Tensor, status: torch.Tensor, norm: Optional[NormInput] = None) -> bool:
    """The fused q/k/v projection with the cache append in its epilogue: queries to out[:M, :q_dim],
    keys and values to their slots of ``cache``.  Returns False (and does nothing) where no fused
    kernel applies: between 129 rows and the pair kernel's minimum (256), float32, or a shape the
    tensor cores refuse."""
    if cache.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        return False
    kv = (cache, block_table, row_entry, positions, q_dim)
    # from the pair kernel's smallest step on: it writes the cache from its epilogue, which beats the
    # single-block kernel and a separate append from about 400 rows on and is one launch less
    if M >= PAIR_MIN_ROWS:
        if norm is not None:
            a, norm = norm.materialise(M), None
        return linear_tc_pair(a, w, bias, out, M, kv=kv)
    return _linear_small(a, norm, w, bias, out, M, ACT_NONE, False, kv=kv)


def kv_append(src: torch.Tensor, k_off: int, v_off: int, cache: torch.Tensor, block_table: torch.Tensor,
              row_entry: torch.Tensor, positions: torch.Tensor, T: int, status: torch.Tensor) -> None:
    """Copy the key and value columns of src[:T] to their slots in one cache layer
    [n_pages, 2, n_kv_head, page_size, head_dim]."""
    n_pages, two, n_kv_head, page_size, head_dim = cache.shape
    if two != 2 or not cache.is_contiguous() or cache.dtype != src.dtype or src.stride(1) != 1:
        raise KernelError("kv_append: cache must be contiguous [pages, 2, kv_heads, page, head_dim] of src's dtype")
    _i32(block_table, "block_table")
    if tracing():
        _note("kv_write", "kv_write", (T, 2 * n_kv_head * head_dim, 0), 0.0, 2.0 * T * 2 * n_kv_head * head_dim * src.element_size())
    _check(library().nib_kv_append(_dt(src), _ptr(src), src.stride(0), k_off, v_off, _ptr(cache),
                                   _ptr(block_table), block_table.shape[1], _ptr(row_entry), _ptr(positions),
                                   T, n_kv_head, head_dim, page_size, n_pages, _ptr(status), _stream()),
           "kv_append")


class AttnExtras:
    """Options of the attention kernels on the scores and on the output:
    ``softcap`` > 0: s <- softcap tanh(s / softcap) after the scale; ``slopes`` (float32 [n_head]): s <- s -
    slopes[h] (query position - key position); ``keep_first``: with a window, the keys 0 .. keep_first - 1 stay
    visible behind it; ``gate`` (float32 [rows, >= n_head], any row stride): head h's output of row t times
    sigmoid(gate[t, h]); ``out_scale``: and times this constant; ``span`` > 0: position i sees key j only if
    i // span == j // span (spans count from position 0 of the sequence); ``head_scale`` (float32 [n_head]): the
    scale times head_scale[h]; ``sinks`` (float32 [n_head]): with a sink, its term of the denominator is
    exp(sinks[h]) instead of exp(0)."""

    __slots__ = ("softcap", "keep_first", "slopes", "gate", "out_scale", "span", "head_scale", "sinks")

    def __init__(self, softcap: float = 0.0, keep_first: int = 0, slopes: Optional[torch.Tensor] = None,
                 gate: Optional[torch.Tensor] = None, out_scale: float = 1.0, span: int = 0,
                 head_scale: Optional[torch.Tensor] = None, sinks: Optional[torch.Tensor] = None):
        self.softcap, self.keep_first, self.slopes = float(softcap), int(keep_first), slopes
        self.gate, self.out_scale = gate, float(out_scale)
        self.span, self.head_scale, self.sinks = int(span), head_scale, sinks

    @property
    def plain(self) -> bool:
        return not (self.softcap > 0.0 or self.keep_first > 0 or self.slopes is not None or self.gate is not None
                    or self.out_scale != 1.0 or self.span > 0 or self.head_scale is not None or self.sinks is not None)

    def args(self) -> tuple:
        g = self.gate
        if g is not None and (g.dtype != torch.float32 or g.stride(1) != 1):
            raise KernelError("attention: the output gate must be float32 with contiguous rows")
        for t in (self.slopes, self.head_scale, self.sinks):
            if t is not None and (t.dtype != torch.float32 or not t.is_contiguous()):
                raise KernelError("attention: the slopes, the heads' scales and the sinks must be contiguous float32")
        if self.span < 0:
            raise KernelError("attention: span must not be negative")
        return (self.softcap, self.keep_first, _ptr(self.slopes), _ptr(g), g.stride(0) if g is not None else 0,
                self.out_scale, self.span, _ptr(self.head_scale), _ptr(self.sinks))


_NO_EXTRAS = AttnExtras()


def attention_simt(q: torch.Tensor, cache: torch.Tensor, out: torch.Tensor, block_table: torch.Tensor,
                   row_entry: torch.Tensor, positions: torch.Tensor, T: int, n_head: int, scale: float,
                   window: int, status: torch.Tensor, rows: Optional[torch.Tensor] = None, sink: bool = False,
                   extras: Optional[AttnExtras] = None) -> None:
    """Causal attention of T rows of q ([*, n_head * head_dim], any row stride) over one cache layer, with
    the general kernel (any head size up to 256, any page size).  ``rows`` lists the rows to process."""
    n_pages, _, n_kv_head, page_size, head_dim = cache.shape
    if q.dtype != cache.dtype or out.dtype != cache.dtype or q.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("attention: q, out and cache must share a dtype, rows contiguous")
    _check(library().nib_attention_simt(_dt(q), _ptr(q), q.stride(0), _ptr(cache), _ptr(out), out.stride(0),
                                        _ptr(block_table), block_table.shape[1], _ptr(rows), _ptr(row_entry),
                                        _ptr(positions), T, n_head, n_kv_head, head_dim, page_size, n_pages,
                                        float(scale), int(window), int(sink), *(extras or _NO_EXTRAS).args(),
                                        _ptr(status), _stream()),
           "attention_simt")


#: blocks of the decode attention that the device holds at once (six an SM): the keys are split so
#: that (rows x heads x splits) stays within it, which also bounds the scratch of the partial results
DECODE_RESIDENT_BLOCKS = 888


_cluster_room: dict = {}


def decode_cluster_room(head_dim: int, cluster: int) -> int:
    """How many clusters of ``cluster`` blocks of the MMA decode attention the device holds at once, asked
    of the runtime once per shape (a cluster's blocks share a GPC: 284 clusters of three, not 296; 142 of
    six).  The splits of a (row, head) are one cluster, and a launch with a cluster too many waits for a
    wave to end: 24 rows of 12 heads took 0.68 ms a step in 3 splits and 0.62 ms in 2."""
    key = (head_dim, cluster)
    got = _cluster_room.get(key)
    if got is None:
        got = int(library().nib_attention_decode_mma_clusters(head_dim, cluster))
        if got < 0:
            raise KernelError(f"attention_decode_mma: the occupancy query failed with CUDA error {-got}")
        _cluster_room[key] = got
    return got


#: numbers of splits that the MMA decode attention runs as one cluster, merging through distributed shared
#: memory instead of global scratch (beyond 8 blocks the cluster size is "non-portable": the kernel is marked
#: as taking it; a lone row at 4,096 keys: 0.331 -> 0.308 ms a step with 16 splits of 256 keys, at 1,024 keys
#: 0.250 -> 0.245 with 16 of 64, one tile a warp)
DECODE_CLUSTER_SPLITS = tuple(range(2, 17))

#: keys per split from which the MMA decode attention gives up the merge inside a cluster for more splits
#: than a cluster holds, merged through scratch (measured at 2 K to 16 K keys, batch 1 to 8: four rows at
#: 16 K keys take 0.67 ms a step in 18 splits through scratch and 0.90 ms in a cluster of 14) ...
DECODE_DEEP_KEYS = 512
#: ... and the fewest such splits: one more than the largest cluster
DECODE_DEEP_SPLITS = 17

def decode_ring_stages(n_blocks: int, n_splits: int, head_dim: int) -> int:
    """How many shared-memory stages per warp the MMA decode attention passes its keys and values through
    (that many tiles in flight per warp beside the one being multiplied; 0: none, the tiles go through
    registers).  The ring pays where the launch fills the device with unsplit rows (measured: -7 to -10 %
    a step at batch 40 to 64, +3 to +7 % at batch 1 to 32, where the keys are split and a block's shared
    memory keeps it from starting beside the kernel ahead).  It is the deepest of two to four stages that
    needs no more waves of blocks than two stages do (shared memory sets how many blocks an SM holds: 40 to 48
    rows of 12 heads take 8 to 9 % less a step with three stages, which still hold them all at once, and
    so do 64 rows of 16 heads, two full waves of four blocks an SM instead of a full and a thin one of six)."""
    if n_splits != 1 or n_blocks < 440:
        return 0
    stage_bytes = 4 * 2 * 16 * head_dim * 2          # four warps, keys and values of a 16-key tile
    by_registers = 6 if head_dim <= 64 else 3

    def waves(stages: int) -> int:
        per_sm = max(1, min(by_registers, (200 * 1024) // (stages * stage_bytes)))
        return -(-n_blocks // (148 * per_sm))

    return max(st for st in (2, 3, 4) if waves(st) <= waves(2))


#: the bfloat16 decode attention on warp-level MMAs where the shape allows (False: always the streaming kernel)
USE_DECODE_MMA = True


def decode_split(n_rows: int, n_head: int, max_keys: int, resident: int = DECODE_RESIDENT_BLOCKS,
                 at_most: int = 0) -> tuple:
    """(chunk, n_splits): keys per split (a multiple of 64) so that the blocks fill the GPU once: six
    blocks an SM are resident, and a block that comes after the first wave runs nearly alone.
    ``at_most``: an upper bound on the number of splits (0: none)."""
    want = max(1, resident // max(1, n_rows * n_head))
    if at_most:
        want = min(want, at_most)
    chunk = max(64, -(-(-(-max_keys // want)) // 64) * 64)
    return chunk, max(1, -(-max_keys // chunk))


def _note_attention(n_q: int, keys_seen: float, kv_rows: float, n_head: int, n_kv_head: int, head_dim: int,
                    itemsize: int) -> None:
    """[queries, keys seen by them in all, width]: per key and head the score (2 hd), the softmax (~5)
    and the weighted sum (2 hd); the queries and outputs, and ``kv_rows`` key and value rows read once."""
    width = n_head * head_dim
    _note("attn", "attn", (n_q, int(keys_seen), width), keys_seen * (4.0 * width + 5.0 * n_head),
          itemsize * (2.0 * n_q * width + 2.0 * kv_rows * n_kv_head * head_dim))


def attention_decode_reserve(workspace, n_head: int, head_dim: int) -> None:
    """Size the decode attention's scratch for good: keys are split only while rows x heads x splits
    fits the resident blocks, so that many partial results (head_dim values, a maximum and a sum
    each) and that many arrival counters are the most any step needs."""
    workspace.reserve("attention.partials", DECODE_RESIDENT_BLOCKS * (head_dim + 2), torch.float32)
    workspace.reserve("attention.arrivals", DECODE_RESIDENT_BLOCKS, torch.int32, zeroed=True)


def attention_decode(q: torch.Tensor, cache: torch.Tensor, out: torch.Tensor, block_table: torch.Tensor,
                     row_entry: torch.Tensor, positions: torch.Tensor, n_rows: int, n_head: int, scale: float,
                     window: int, status: torch.Tensor, max_keys: int, workspace,
                     rows: Optional[torch.Tensor] = None, sink: bool = False,
                     extras: Optional[AttnExtras] = None) -> None:
    """Split-KV attention for rows that are single decoded tokens.  ``max_keys``: the longest key
    range among them; partial results go through ``workspace``.  bfloat16 with a head size of 32, 64,
    96 or 128 runs on the warp-level MMA kernel, everything else (and float32, in true 32-bit
    arithmetic) on the streaming kernel."""
    n_pages, _, n_kv_head, page_size, head_dim = cache.shape
    if q.dtype != cache.dtype or out.dtype != cache.dtype or q.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("attention: q, out and cache must share a dtype, rows contiguous")
    plain = extras is None or extras.plain     # (the MMA kernel takes no options on the scores or the output)
    mma = USE_DECODE_MMA and plain and q.dtype == torch.bfloat16 and _can("nib_attention_decode_mma_supported", head_dim, page_size) \
        and q.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0 and cache.data_ptr() % 16 == 0
    # (the MMA kernel holds a tile's keys and values in registers: six blocks an SM up to head size 64, three beyond)
    resident = DECODE_RESIDENT_BLOCKS if not mma or head_dim <= 64 else DECODE_RESIDENT_BLOCKS // 2
    # (the MMA kernel merges up to sixteen splits inside a cluster, which costs two trips to memory less
    # than the merge through scratch, until a split has DECODE_DEEP_KEYS keys to walk and the device has
    # room for more splits than a cluster holds: a lone row at 16 K keys takes 0.44 ms a step in 64 splits
    # against 0.72 ms in 8)
    at_most = 0
    if mma:
        at_most = max([c for c in DECODE_CLUSTER_SPLITS if n_rows * n_head <= decode_cluster_room(head_dim, c)], default=1)
        deep = min(resident // max(1, n_rows * n_head), max_keys // (DECODE_DEEP_KEYS // 2))
        if deep >= DECODE_DEEP_SPLITS:
            at_most = deep
    chunk, n_splits = decode_split(n_rows, n_head, max_keys, resident, at_most)
    scratch = counters = None
    if n_splits > 1:
        # (never more than the resident blocks: the same size every step, so that the buffers stay put)
        assert n_rows * n_head * n_splits <= DECODE_RESIDENT_BLOCKS
        scratch = workspace.get("attention.partials", (DECODE_RESIDENT_BLOCKS * (head_dim + 2),), torch.float32)
        counters = workspace.get_zeroed("attention.arrivals", (DECODE_RESIDENT_BLOCKS,), torch.int32)
    if mma:
        _check(library().nib_attention_decode_mma(_ptr(q), q.stride(0), _ptr(cache), _ptr(scratch), _ptr(out),
                                                  out.stride(0), _ptr(block_table), block_table.shape[1], _ptr(rows),
                                                  _ptr(row_entry), _ptr(positions), n_rows, n_head, n_kv_head,
                                                  head_dim, page_size, n_pages, float(scale), int(window), int(sink),
                                                  chunk, n_splits, _ptr(counters), _ptr(status),
                                                  int(n_splits in DECODE_CLUSTER_SPLITS),
                                                  decode_ring_stages(n_rows * n_head, n_splits, head_dim), _stream()),
               "attention_decode_mma")
        return
    _check(library().nib_attention_decode(_dt(q), _ptr(q), q.stride(0), _ptr(cache), _ptr(scratch), _ptr(out),
                                          out.stride(0), _ptr(block_table), block_table.shape[1], _ptr(rows),
                                          _ptr(row_entry), _ptr(positions), n_rows, n_head, n_kv_head, head_dim,
                                          page_size, n_pages, float(scale), int(window), int(sink),
                                          *(extras or _NO_EXTRAS).args(), chunk, n_splits,
                                          _ptr(counters), _ptr(status), _stream()), "attention_decode")


def attention_prefill_tc(q: torch.Tensor, cache: torch.Tensor, out: torch.Tensor, block_table: torch.Tensor,
                         tiles: torch.Tensor, n_tiles: int, entry_start: torch.Tensor, entry_pos0: torch.Tensor,
                         n_rows: int, n_head: int, scale: float, window: int, status: torch.Tensor,
                         sink: bool = False, extras: Optional[AttnExtras] = None) -> None:
    """tcgen05 attention for prompt portions (bfloat16, head size 64): ``tiles`` holds (entry, first
    row within the entry) pairs of 128 rows each; ``q`` holds the step's ``n_rows`` rows."""
    n_pages, _, n_kv_head, page_size, head_dim = cache.shape
    if q.dtype != torch.bfloat16 or cache.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise KernelError("attention_prefill_tc: bfloat16 only")
    if not cache.is_contiguous() or q.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("attention_prefill_tc: contiguous cache layer and rows")
    _check(library().nib_attention_prefill_tc(_ptr(q), q.stride(0), n_rows, _ptr(cache), _ptr(out), out.stride(0),
                                              _ptr(block_table), block_table.shape[1], _ptr(tiles), n_tiles,
                                              _ptr(entry_start), _ptr(entry_pos0), n_head, n_kv_head, head_dim,
                                              page_size, n_pages, float(scale), int(window), int(sink),
                                              *(extras or _NO_EXTRAS).args(), _ptr(status), _stream()),
           "attention_prefill_tc")


def attention_prefill(q: torch.Tensor, cache: torch.Tensor, out: torch.Tensor, block_table: torch.Tensor,
                      tiles: torch.Tensor, n_tiles: int, entry_start: torch.Tensor, entry_pos0: torch.Tensor,
                      n_head: int, scale: float, window: int, status: torch.Tensor, sink: bool = False,
                      extras: Optional[AttnExtras] = None) -> None:
    """Tiled tensor-core attention for prompt portions: ``tiles`` holds (entry, first row within the
    entry) pairs of 64 rows each."""
    n_pages, _, n_kv_head, page_size, head_dim = cache.shape
    if q.dtype != torch.bfloat16 or cache.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise KernelError("attention_prefill: bfloat16 only")
    _check(library().nib_attention_prefill(_ptr(q), q.stride(0), _ptr(cache), _ptr(out), out.stride(0),
                                           _ptr(block_table), block_table.shape[1], _ptr(tiles), n_tiles,
                                           _ptr(entry_start), _ptr(entry_pos0), n_head, n_kv_head, head_dim,
                                           page_size, n_pages, float(scale), int(window), int(sink),
                                           *(extras or _NO_EXTRAS).args(), _ptr(status), _stream()), "attention_prefill")


def attention(q: torch.Tensor, cache: torch.Tensor, out: torch.Tensor, block_table: torch.Tensor, ctx,
              n_head: int, scale: float, window: int, plan, sink: bool = False,
              extras: Optional[AttnExtras] = None) -> None:
    """Causal attention of the step's rows over one cache layer.  ``extras``: options on the scores and the output
    (``AttnExtras``); the kernels that take them are the general one, the two of prompt portions and the streaming split-KV one.  ``sink``: the softmax's denominator has
    one more term, exp(0) (a key of score 0 that has no value; every kernel adds it where it divides).
    ``ctx`` is the step's StepContext, ``plan`` says which rows are single decoded tokens and how the
    prompt portions are cut into tiles (``parts.attention.AttentionPlan``).  Single decoded tokens go to the split-KV kernel;
    prompt portions go to the tiled tensor-core kernels in bfloat16 (head sizes 16..128 in steps of
    16) and to the general kernel otherwise."""
    n_pages, _, n_kv_head, page_size, head_dim = cache.shape
    fast_pages = page_size % 16 == 0 and head_dim % 8 == 0 and head_dim <= 128
    plain = extras is None or extras.plain
    traced = tracing()   # (the counts leave a window out: they are those of attention over all keys)
    if not fast_pages:
        if traced:
            _note_attention(ctx.n_rows, plan.decode_keys + plan.prefill_keys, plan.decode_keys + plan.prefill_kv_rows,
                            n_head, n_kv_head, head_dim, q.element_size())
        attention_simt(q, cache, out, block_table, ctx.row_entry, ctx.positions, ctx.n_rows, n_head, scale,
                       window, ctx.status, sink=sink, extras=extras)
        return
    if plan.n_decode:
        keys = plan.max_decode_keys if window <= 0 else min(plan.max_decode_keys, window)
        if extras is not None and extras.span > 0:
            keys = min(keys, extras.span)
        if traced:
            _note_attention(plan.n_decode, plan.decode_keys, plan.decode_keys, n_head, n_kv_head, head_dim,
                            q.element_size())
        attention_decode(q, cache, out, block_table, ctx.row_entry, ctx.positions, plan.n_decode, n_head, scale,
                         window, ctx.status, keys, ctx.workspace, plan.decode_rows, sink=sink, extras=extras)
    if plan.n_prefill_rows:
        if traced:
            _note_attention(plan.n_prefill_rows, plan.prefill_keys, plan.prefill_kv_rows, n_head, n_kv_head, head_dim,
                            q.element_size())
        if q.dtype == torch.bfloat16 and scale > 0 and _can("nib_attention_prefill_tc_supported", head_dim, page_size) \
                and q.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0 and out.stride(0) % 8 == 0 \
                and out.data_ptr() % 16 == 0:
            attention_prefill_tc(q, cache, out, block_table, plan.wide_tiles, plan.n_wide_tiles, ctx.entry_start,
                                 ctx.entry_pos0, ctx.n_rows, n_head, scale, window, ctx.status, sink=sink, extras=extras)
        elif q.dtype == torch.bfloat16 and scale > 0 and _can("nib_attention_prefill_supported", head_dim) \
                and q.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0:
            attention_prefill(q, cache, out, block_table, plan.tiles, plan.n_tiles, ctx.entry_start, ctx.entry_pos0,
                              n_head, scale, window, ctx.status, sink=sink, extras=extras)
        else:
            # (portions alone: all of the step's rows, those of no request among them, which the kernel leaves out;
            # the launch then depends on the step's shape only, as a graph needs it)
            attention_simt(q, cache, out, block_table, ctx.row_entry, ctx.positions,
                           plan.n_prefill_rows if plan.n_decode else ctx.n_rows, n_head, scale, window, ctx.status,
                           plan.prefill_rows, sink=sink, extras=extras)


_SRC_CODES = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}


def convert_rows(src: torch.Tensor, src_dtype: torch.dtype, rows: int, cols: int, dst: torch.Tensor, r0: int,
                 transpose: bool) -> None:
    """Loading: ``src`` holds the raw bytes of ``rows`` x ``cols`` values as a checkpoint stores them;
    they are converted to ``dst``'s dtype and written to dst[r0:r0 + rows, :] or, transposed, to
    dst[:, r0:r0 + rows]."""
    if src_dtype not in _SRC_CODES or not dst.is_contiguous() or dst.dim() != 2:
        raise KernelError("convert: 16- or 32-bit floats into a contiguous matrix")
    _check(library().nib_convert(_SRC_CODES[src_dtype], _ptr(src), rows, cols, _dt(dst), _ptr(dst), dst.stride(0),
                                 int(r0), int(bool(transpose)), _stream()), "convert")


def argmax(logits: torch.Tensor, out: torch.Tensor, n_rows: int) -> None:
    if logits.dtype != torch.float32 or logits.stride(1) != 1:
        raise KernelError("argmax: logits must be float32 with contiguous rows")
    _i32(out, "out")
    if tracing():
        _note("sample", "sample", (n_rows, logits.shape[1], 0), n_rows * logits.shape[1], 4.0 * n_rows * logits.shape[1])
    _check(library().nib_argmax(_ptr(logits), logits.stride(0), n_rows, logits.shape[1], _ptr(out), _stream()),
           "argmax")


def sample(logits: torch.Tensor, n_rows: int, row_slot: torch.Tensor, temperature: torch.Tensor,
           top_k: torch.Tensor, rng_state: torch.Tensor, out: torch.Tensor, scratch: torch.Tensor,
           last_token: Optional[torch.Tensor] = None, teams: bool = True) -> None:
    """One token per row.  ``temperature``, ``top_k`` and ``rng_state`` are per-slot arrays and
    ``row_slot`` names each row's slot: greedy where the slot's temperature <= 0, else
    temperature / top-k sampling that advances the slot's xorshift64* word.  ``last_token``: a
    per-slot array that also receives the tokens (for the next step's embedding).  ``teams``: launch
    clusters of blocks that share a sampled row's passes over the vocabulary (False when every row
    is known to be greedy; the tokens are the same either way).  ``scratch``: two int64 words per
    row that the kernel finds zero and leaves zero (the caller owns them, so that they stay where
    they are for as long as a captured launch may use them)."""
    if logits.dtype != torch.float32 or logits.stride(1) != 1:
        raise KernelError("sample: logits must be float32 with contiguous rows")
    if rng_state.dtype != torch.int64 or temperature.dtype != torch.float32:
        raise KernelError("sample: rng_state must be int64 words, temperature float32")
    _i32(row_slot, "row_slot"); _i32(top_k, "top_k"); _i32(out, "out")
    if scratch.dtype != torch.int64 or scratch.numel() < 2 * n_rows or out.numel() < n_rows:
        raise KernelError("sample: scratch must hold two int64 words per row, out one int32")
    if tracing():
        _note("sample", "sample", (n_rows, logits.shape[1], 0), n_rows * logits.shape[1], 4.0 * n_rows * logits.shape[1])
    _check(library().nib_sample(_ptr(logits), logits.stride(0), n_rows, logits.shape[1], _ptr(row_slot),
                                _ptr(temperature), _ptr(top_k), _ptr(rng_state), _ptr(out),
                                _ptr(last_token), _ptr(scratch), int(bool(teams)), _stream()), "sample")


# ------------------------------------------------------------------------------ post-norm streams
def _f32(t: torch.Tensor, name: str) -> None:
    if t.dtype != torch.float32 or not t.is_contiguous():
        raise KernelError(f"{name} must be a contiguous float32 tensor")


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor, n_rows: int,
            rows: Optional[torch.Tensor] = None) -> None:
    """out[r] = x[rows[r]] / sqrt(mean(x^2) + eps) * weight (rows None: x[r]); x is the 32-bit stream."""
    C = x.shape[1]
    _f32(x, "rmsnorm: x"); _f32(weight, "rmsnorm: weight")
    if weight.numel() != C or out.shape[1] != C or out.shape[0] < n_rows or not out.is_contiguous():
        raise KernelError("rmsnorm: weight [C], out contiguous [n_rows, C]")
    if rows is not None:
        _i32(rows, "rows")
    if tracing():
        _note("ln", "ln", (n_rows, C, 0), 4.0 * n_rows * C, n_rows * C * (4 + out.element_size()) + 4 * C)
    _check(library().nib_rmsnorm(_dt(out), _ptr(x), _ptr(rows), _ptr(weight), _ptr(out), n_rows, C, float(eps),
                                 _stream()), "rmsnorm")


def stream_enter(x: torch.Tensor, xn: torch.Tensor, alpha: float, n_rows: int,
                 level0: Optional[torch.Tensor] = None) -> None:
    """xn = x in the engine's dtype, level0 = x (optional), x = alpha * x: the entry of a layer whose
    sublayers read the stream itself and add into alpha times it."""
    C = x.shape[1]
    _f32(x, "stream_enter: x")
    if xn.shape[1] != C or not xn.is_contiguous() or (level0 is not None and (level0.dtype != torch.float32
                                                                               or not level0.is_contiguous())):
        raise KernelError("stream_enter: xn contiguous [rows, C], level0 contiguous float32")
    if tracing():
        _note("other", "stream", (n_rows, C, 0), n_rows * C, n_rows * C * (8 + xn.element_size()))
    _check(library().nib_stream_enter(_dt(xn), _ptr(x), _ptr(xn), _ptr(level0), float(alpha), n_rows, C, _stream()),
           "stream_enter")


def post_norm(x: torch.Tensor, weight: torch.Tensor, eps: float, n_rows: int, xn: Optional[torch.Tensor] = None,
              alpha_next: float = 1.0, levels: Optional[torch.Tensor] = None, n_levels: int = 0,
              mix: Optional[torch.Tensor] = None) -> None:
    """y = rmsnorm(x) * weight in place on the 32-bit stream.  With ``levels`` ([depth, max_rows, C], float32):
    y becomes level ``n_levels - 1`` and the stream goes on as z = sum_j mix[j] * levels[j] over the first
    ``n_levels``; else z = y.  ``xn`` (optional) receives z in its own dtype; x = alpha_next * z."""
    C = x.shape[1]
    _f32(x, "post_norm: x"); _f32(weight, "post_norm: weight")
    stride = 0
    if levels is not None:
        _f32(levels, "post_norm: levels")
        if mix is None or mix.dtype != torch.float32 or mix.numel() < n_levels or not 1 <= n_levels <= levels.shape[0] \
                or levels.shape[2] != C or levels.shape[1] != x.shape[0]:
            raise KernelError("post_norm: levels [depth, rows of x, C] with n_levels weights")
        stride = levels.stride(0)
    if xn is not None and (xn.shape[1] != C or not xn.is_contiguous()):
        raise KernelError("post_norm: xn contiguous [rows, C]")
    if tracing():
        _note("ln", "ln", (n_rows, C, 0), (4.0 + 2 * n_levels) * n_rows * C,
              n_rows * C * (8 + 4 * n_levels + (xn.element_size() if xn is not None else 0)))
    _check(library().nib_post_norm(_dt(xn) if xn is not None else 0, _ptr(x), _ptr(weight), float(eps), _ptr(levels),
                                   int(stride), int(n_levels), _ptr(mix), _ptr(xn), float(alpha_next), n_rows, C,
                                   _stream()), "post_norm")


def unary(src: torch.Tensor, out: torch.Tensor, n_rows: int, kind: int, prm: Optional[torch.Tensor] = None) -> None:
    """out[:n_rows] = f(src[:n_rows]) element by element (``UNARY_TANH``; ``UNARY_XIELU`` with its two numbers in
    ``prm`` on the device); src and out may be views with their own row strides, or the same buffer."""
    if src.shape[1] != out.shape[1] or src.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("unary: src and out must have the same columns, rows contiguous")
    if tracing():
        _note("other", "act", (n_rows, src.shape[1], 0), 8.0 * n_rows * src.shape[1],
              n_rows * src.shape[1] * (src.element_size() + out.element_size()))
    _check(library().nib_unary(_dt(src), _dt(out), _ptr(src), src.stride(0), _ptr(out), out.stride(0), n_rows,
                               src.shape[1], int(kind), _ptr(prm), _stream()), "unary")


# ------------------------------------------------------------------------------ latent attention
def latent_prep(proj: torch.Tensor, q_rank: int, kv_rank: int, rot_dim: int, rot_dims: int, freqs: torch.Tensor,
                wq: torch.Tensor, wkv: Optional[torch.Tensor], eps: float, cq: torch.Tensor,
                cache: Optional[torch.Tensor], block_table: Optional[torch.Tensor], row_entry: torch.Tensor,
                positions: torch.Tensor, T: int, status: torch.Tensor) -> None:
    """From the down-projections' output ``proj`` (float32 [T, q_rank (+ kv_rank + rot_dim)]): the normed query
    latent into ``cq``, and (with ``cache``, one layer [pages, 1, 1, page_size, kv_rank + rot_dim]) the normed
    key/value latent and the rotated shared key part into the rows' cache slots."""
    _f32(proj, "latent_prep: proj")
    if freqs.dtype != torch.float64 or cq.stride(1) != 1:
        raise KernelError("latent_prep: freqs must be float64, cq rows contiguous")
    has_kv = cache is not None
    if has_kv:
        n_pages, planes, heads, page_size, D = cache.shape
        if planes != 1 or heads != 1 or D != kv_rank + rot_dim or not cache.is_contiguous() or cache.dtype != cq.dtype:
            raise KernelError("latent_prep: cache must be contiguous [pages, 1, 1, page, kv_rank + rot_dim] of cq's dtype")
        _i32(block_table, "block_table")
    else:
        n_pages = page_size = 0
    if tracing():
        _note("other", "latent_prep", (T, proj.shape[1], 0), 6.0 * T * proj.shape[1],
              T * proj.shape[1] * (4 + cq.element_size()))
    _check(library().nib_latent_prep(_dt(cq), _ptr(proj), proj.stride(0), q_rank, kv_rank, rot_dim, rot_dims,
                                     _ptr(freqs), _ptr(wq), _ptr(wkv), float(eps), _ptr(cq), cq.stride(0),
                                     _ptr(cache), _ptr(block_table), block_table.shape[1] if has_kv else 0,
                                     _ptr(row_entry), _ptr(positions), T, page_size, n_pages, int(has_kv),
                                     _ptr(status), _stream()), "latent_prep")


def rope_heads(q: torch.Tensor, nope: int, rot_dim: int, rot_dims: int, freqs: torch.Tensor,
               positions: torch.Tensor, out: torch.Tensor, out_off: int, n_head: int, T: int) -> None:
    """Rotates the last ``rot_dim`` values of every head of q ([T, n_head * (nope + rot_dim)]) by the rows'
    positions (interleaved pairs over the first ``rot_dims``) into out[t, h, out_off:], float32 [T, n_head, D]."""
    _f32(out, "rope_heads: out")
    if q.stride(1) != 1 or freqs.dtype != torch.float64:
        raise KernelError("rope_heads: q rows contiguous, freqs float64")
    if tracing():
        _note("other", "rope", (T, n_head * rot_dim, 0), 6.0 * T * n_head * rot_dim,
              T * n_head * rot_dim * (q.element_size() + 4))
    _check(library().nib_rope_heads(_dt(q), _ptr(q), q.stride(0), nope, rot_dim, rot_dims, _ptr(freqs),
                                    _ptr(positions), _ptr(out), out.shape[2], out_off, n_head, T, _stream()),
           "rope_heads")


#: blocks of the latent attention that fill the device about twice: a step of few rows cuts every row's keys
#: into pieces until it has that many blocks (at most LATENT_MAX_SPLITS pieces a row)
LATENT_BLOCKS, LATENT_MAX_SPLITS, LATENT_HEADS_PER_BLOCK = 296, 16, 8


def latent_splits(n_rows: int, n_head: int) -> int:
    """Into how many pieces the latent attention cuts each row's keys: a function of the step's shape alone
    (a captured step bakes it in); the pieces' sizes follow from each row's own key range on the device."""
    groups = -(-n_head // LATENT_HEADS_PER_BLOCK)
    return max(1, min(LATENT_MAX_SPLITS, LATENT_BLOCKS // max(1, n_rows * groups)))


def latent_attention_reserve(workspace, n_head: int, kv_rank: int) -> None:
    """Scratch of the pieces' partial results: keys are cut only while rows x head groups x pieces stays within
    LATENT_BLOCKS, which bounds it whatever the step."""
    workspace.reserve("latent.partials", LATENT_BLOCKS * LATENT_HEADS_PER_BLOCK * (kv_rank + 2), torch.float32)


def latent_attention(q: torch.Tensor, cache: torch.Tensor, out: torch.Tensor, block_table: torch.Tensor, ctx,
                     n_head: int, kv_rank: int, scale: float, window: int, n_splits: Optional[int] = None) -> None:
    """Causal softmax attention of the step's rows over one latent cache layer: q float32 [T, n_head, D] (the
    absorbed query, then the rotated part), out [T, n_head * kv_rank] the weighted sums of latents.  A step of
    few rows (decoded tokens) cuts every row's keys into ``n_splits`` pieces, merged by a second kernel."""
    n_pages, _, _, page_size, D = cache.shape
    if n_splits is None:
        n_splits = latent_splits(ctx.n_rows, n_head)
    partials = None
    if n_splits > 1:
        need = ctx.n_rows * n_head * n_splits * (kv_rank + 2)
        partials = ctx.workspace.get("latent.partials", (need,), torch.float32)
    _f32(q, "latent_attention: q")
    if out.dtype != cache.dtype or out.stride(1) != 1 or q.shape[2] != D:
        raise KernelError("latent_attention: out in the cache's dtype, q [T, heads, D]")
    if tracing():
        keys = sum(min(p + 1, window) if window > 0 else p + 1
                   for e, p0 in enumerate(ctx.host_entry_pos0)
                   for p in range(p0, p0 + ctx.host_entry_start[e + 1] - ctx.host_entry_start[e]))
        _note("attn", "attn", (ctx.n_rows, keys, n_head * D), keys * n_head * 2.0 * (D + kv_rank),
              4.0 * ctx.n_rows * n_head * D + out.element_size() * (ctx.n_rows * n_head * kv_rank + keys * D))
    _check(library().nib_latent_attention(_dt(cache), _ptr(q), _ptr(cache), _ptr(out), out.stride(0), _ptr(block_table),
                                          block_table.shape[1], None, _ptr(ctx.row_entry), _ptr(ctx.positions),
                                          ctx.n_rows, n_head, kv_rank, D, page_size, n_pages, float(scale),
                                          int(window), _ptr(ctx.status), int(n_splits), _ptr(partials), _stream()),
           "latent_attention", 2 if n_splits > 1 else 1)


def linear_heads(a: torch.Tensor, a_head_stride: int, w: torch.Tensor, out: torch.Tensor, out_head_stride: int,
                 M: int) -> None:
    """out[t, h * out_head_stride + n] = sum_k a[t, h * a_head_stride + k] * w[h, n, k] for w [heads, N, K]."""
    H, N, K = w.shape
    if a.dtype != w.dtype or not w.is_contiguous() or a.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("linear_heads: a and w share a dtype, w contiguous [heads, N, K]")
    if tracing():
        _note("matmul", "matmul_heads", (M, K, H * N), 2.0 * M * H * N * K,
              w.numel() * w.element_size() + M * H * (K * a.element_size() + N * out.element_size()))
    _check(library().nib_linear_heads(_dt(a), _dt(out), _ptr(a), a.stride(0), a_head_stride, _ptr(w), _ptr(out),
                                      out.stride(0), out_head_stride, M, H, N, K, _stream()), "linear_heads")


# ------------------------------------------------------------------------------ delta rule
def delta_rule(proj: torch.Tensor, offsets, wl: torch.Tensor, w0: torch.Tensor, a_bias: torch.Tensor,
               norm_w: torch.Tensor, state: torch.Tensor, ctx, n_head: int, dim: int, eps: float,
               out: torch.Tensor, unit: Optional[torch.Tensor] = None) -> None:
    """The generalised delta rule over the step's entries (csrc/delta_rule.cu).  ``proj`` float32 [T, *] holds
    r, k, v, gate and removal logits at the column ``offsets`` (five), ``wl`` float32 the decay logits; ``state``
    float32 [slots, n_head, dim, dim] is read and written at the entries' slots.  ``wl`` and the removal logits of
    ``proj`` are scratch afterwards; ``unit`` (float32 [rows, n_head * dim], optional) is scratch for the rows' unit
    keys: with it a step that carries prompt portions makes all rows' gates in one pass before the recurrence.
    ``ctx.n_rows`` counts the rows of the entries only where rows of no request follow them."""
    _f32(proj, "delta_rule: proj"); _f32(state, "delta_rule: state")
    if wl.dtype != torch.float32 or wl.stride(1) != 1 or out.stride(1) != 1 or tuple(state.shape[1:]) != (n_head, dim, dim):
        raise KernelError("delta_rule: wl float32, state [slots, heads, dim, dim]")
    r_off, k_off, v_off, g_off, a_off = (int(o) for o in offsets)
    if unit is not None and (unit.dtype != torch.float32 or not unit.is_contiguous() or unit.shape[1] != n_head * dim
                             or unit.shape[0] < ctx.n_rows):
        raise KernelError("delta_rule: unit must be contiguous float32 [rows, heads * dim]")
    if tracing():
        T = ctx.n_rows
        _note("other", "delta_rule", (T, n_head * dim, dim), 8.0 * T * n_head * dim * dim,
              T * n_head * dim * (6 * 4 + out.element_size()) + 8.0 * ctx.n_entries * n_head * dim * dim)
    _check(library().nib_delta_rule(_dt(out), _ptr(proj), proj.stride(0), r_off, k_off, v_off, g_off, a_off, _ptr(wl),
                                    wl.stride(0), _ptr(w0), _ptr(a_bias), _ptr(norm_w), _ptr(state),
                                    _ptr(ctx.entry_start), _ptr(ctx.entry_slot), ctx.n_entries, ctx.n_rows, n_head,
                                    dim, float(eps), _ptr(out), out.stride(0), _ptr(unit), _stream()), "delta_rule")


# ------------------------------------------------------------------------------ routed experts
def moe_route(h: torch.Tensor, w_router: torch.Tensor, T: int, top: int, renorm: bool, ids: torch.Tensor,
              weights: torch.Tensor, score: str = "softmax", choice_bias: Optional[torch.Tensor] = None,
              n_real: Optional[int] = None, x: Optional[torch.Tensor] = None) -> None:
    """Router logits in 32-bit, scores = softmax over all experts (or, ``score`` "sigmoid", each logit's sigmoid),
    the ``top`` largest (ties to the lower index) into ``ids`` int32 [T, top] with their scores in ``weights``
    float32 [T, top] (divided by their sum with ``renorm``).  ``choice_bias`` (float32 [experts]) is added to the
    scores for the choice only.  The experts from ``n_real`` on have no matrices: a row that chooses one gets
    score * h[t] added to ``x`` (float32 [T, C]) right here, and the id -1, which the expert kernels skip."""
    if score not in ("softmax", "sigmoid"):
        raise KernelError("moe_route: score is 'softmax' or 'sigmoid'")
    E, C = w_router.shape
    if h.dtype != w_router.dtype or h.stride(1) != 1 or not w_router.is_contiguous():
        raise KernelError("moe_route: h and the router share a dtype")
    _i32(ids, "ids"); _f32(weights, "moe_route: weights")
    n_real = E if n_real is None else int(n_real)
    if choice_bias is not None and (choice_bias.dtype != torch.float32 or choice_bias.numel() != E
                                    or not choice_bias.is_contiguous()):
        raise KernelError("moe_route: choice_bias must be contiguous float32 [experts]")
    if n_real < E and (x is None or x.dtype != torch.float32 or not x.is_contiguous() or x.shape[1] != C):
        raise KernelError("moe_route: experts without matrices need the 32-bit x [T, C] to add into")
    if tracing():
        _note("matmul", "router", (T, C, E), 2.0 * T * C * E, (E + T) * C * h.element_size() + 8.0 * T * top)
    _check(library().nib_moe_route(_dt(h), _ptr(h), h.stride(0), _ptr(w_router), T, C, E, top, int(renorm),
                                   int(score == "sigmoid"), _ptr(choice_bias), n_real, _ptr(x) if n_real < E else None, _ptr(ids),
                                   _ptr(weights), _stream()), "moe_route")


def moe_up(h: torch.Tensor, w_up: torch.Tensor, ids: torch.Tensor, inner: torch.Tensor, T: int, top: int,
           act: int, gated: bool = False, in_weights: Optional[torch.Tensor] = None, act_prm: float = 0.0) -> None:
    """inner[t * top + k] = act(w_up[ids[t, k]] . h[t]) for w_up [experts, F, C].  ``gated``: w_up is
    [experts, 2F, C] with rows 2f and 2f + 1 the gate and the value of output f, and inner = act(s g) * (s u) with
    s = in_weights[t, k] (None: 1)."""
    E, F, C = w_up.shape
    if gated:
        F //= 2
    if h.dtype != w_up.dtype or inner.dtype != h.dtype or not w_up.is_contiguous() or not inner.is_contiguous() \
            or inner.shape[1] != F:
        raise KernelError("moe_up: h, w_up and inner share a dtype; inner contiguous [T * top, F]")
    if tracing():
        _note("moe", "experts_up", (T * top, C, F), 2.0 * T * top * C * F,
              h.element_size() * (min(E, T * top) * F * C + T * C + T * top * F))
    _check(library().nib_moe_up(_dt(h), _ptr(h), h.stride(0), _ptr(w_up), _ptr(ids), _ptr(inner), T, C, F, top,
                                int(act), float(act_prm), int(gated), _ptr(in_weights), _stream()), "moe_up")


def moe_down(inner: torch.Tensor, w_down: torch.Tensor, ids: torch.Tensor, weights: Optional[torch.Tensor],
             x: torch.Tensor, T: int, top: int) -> None:
    """x[t] += sum_k weights[t, k] * w_down[ids[t, k]] . inner[t * top + k] for w_down [experts, C, F] (weights
    None: all 1)."""
    E, C, F = w_down.shape
    _f32(x, "moe_down: x")
    if inner.dtype != w_down.dtype or not w_down.is_contiguous() or not inner.is_contiguous() or x.shape[1] != C:
        raise KernelError("moe_down: inner and w_down share a dtype; x [T, C]")
    if tracing():
        _note("moe", "experts_down", (T * top, F, C), 2.0 * T * top * C * F,
              inner.element_size() * (min(E, T * top) * F * C + T * top * F) + 8.0 * T * C)
    _check(library().nib_moe_down(_dt(inner), _ptr(inner), _ptr(w_down), _ptr(ids), _ptr(weights), _ptr(x), T, C, F,
                                  top, _stream()), "moe_down")


#: rows per expert (on average) from which the routed feed-forward leaves the row-by-row kernels
MOE_GROUPED_MIN_ROWS_PER_EXPERT = 8
#: the most experts per chosen expert for which a step of many rows runs ALL experts as two products on the tensor
#: cores (n_expert / top times the arithmetic of the chosen ones) rather than expert by expert on the CUDA cores
MOE_DENSE_MAX_RATIO = 8
MOE_GROUPED = True
MOE_DENSE = True


def moe_dense_pays(T: int, top: int, n_expert: int) -> bool:
    return MOE_DENSE and T * top >= MOE_GROUPED_MIN_ROWS_PER_EXPERT * n_expert and n_expert <= MOE_DENSE_MAX_RATIO * top


def moe_scale(inner_all: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor, T: int, n_expert: int, F: int,
              top: int) -> None:
    """inner_all [T, n_expert * F] in place: expert e's part of row t times weights[t, k] where ids[t, k] == e,
    times 0 where the row did not choose e."""
    if not inner_all.is_contiguous() or inner_all.shape[1] != n_expert * F:
        raise KernelError("moe_scale: inner_all contiguous [T, experts * F]")
    if tracing():
        _note("other", "experts_mask", (T, n_expert * F, 0), T * n_expert * F, 2.0 * T * n_expert * F * inner_all.element_size())
    _check(library().nib_moe_scale(_dt(inner_all), _ptr(inner_all), _ptr(ids), _ptr(weights), T, n_expert, F, top,
                                   _stream()), "moe_scale")


def moe_gate_scale(pre: torch.Tensor, inner_all: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor, T: int,
                   n_expert: int, F: int, top: int, act: int, on_input: bool, act_prm: float = 0.0) -> None:
    """pre [T, n_expert * 2F] holds every expert's (gate, value) pairs; inner_all [T, n_expert * F] = act(s g) * (s u)
    (``on_input``) or s * act(g) * u, s the row's weight for the expert, 0 where the row did not choose it."""
    if not pre.is_contiguous() or not inner_all.is_contiguous() or pre.shape[1] != 2 * n_expert * F \
            or inner_all.shape[1] != n_expert * F:
        raise KernelError("moe_gate_scale: pre contiguous [T, experts * 2F], inner_all contiguous [T, experts * F]")
    if tracing():
        _note("other", "experts_gate", (T, n_expert * F, 0), 4.0 * T * n_expert * F,
              T * n_expert * F * (2.0 * pre.element_size() + inner_all.element_size()))
    _check(library().nib_moe_gate_scale(_dt(pre), _dt(inner_all), _ptr(pre), _ptr(inner_all), _ptr(ids), _ptr(weights),
                                        T, n_expert, F, top, int(act), float(act_prm), int(on_input), _stream()), "moe_gate_scale")


def moe_experts(h: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor,
                inner: torch.Tensor, x: torch.Tensor, T: int, top: int, act: int, workspace, gated: bool = False,
                weight_on_input: bool = False, act_prm: float = 0.0) -> None:
    """x[t] += sum_k weights[t, k] * W_down[ids[t, k]] . act(W_up[ids[t, k]] . h[t]) with w_up [experts, F, C] and
    w_down [experts, C, F].  Steps of few rows: row by row.  Steps of many rows: all experts through the engine's
    own products with the unchosen ones scaled to zero in between (``moe_dense_pays``: the first matrices as one
    product, the second ones a product an expert, all adding into the stream), else expert by expert (weights
    staged in shared memory, a fixed order of additions)."""
    E, F, C = w_up.shape
    if gated:
        # w_up [experts, 2F, C]: rows 2f, 2f + 1 the gate and the value of output f.  With ``weight_on_input`` the
        # score scales both products' results before the activation (the first product is linear) and the
        # second product runs unweighted.
        F //= 2
    elif weight_on_input:
        raise KernelError("moe_experts: weight_on_input is built for gated experts")
    if tuple(w_down.shape) != (E, C, F):
        raise KernelError("moe_experts: w_down must be [experts, C, F]")
    in_w = weights if weight_on_input else None
    out_w = None if weight_on_input else weights
    if moe_dense_pays(T, top, E):
        inner_all = workspace.get("moe.inner_all", (x.shape[0], E * F), h.dtype)
        trace_scope(_rec.layer if _rec is not None else -1, "experts_up")
        if gated:
            pre = workspace.get("moe.pre_all", (x.shape[0], E * 2 * F), torch.float32)
            linear(h, w_up.view(E * 2 * F, C), None, pre, T)
            moe_gate_scale(pre, inner_all, ids, weights, T, E, F, top, act, weight_on_input, act_prm)
        else:
            linear(h, w_up.view(E * F, C), None, inner_all, T, act=act)
            moe_scale(inner_all, ids, weights, T, E, F, top)
        trace_scope(_rec.layer if _rec is not None else -1, "experts_down")
        for e in range(E):
            linear(inner_all[:, e * F:(e + 1) * F], w_down[e], None, x, T, residual=True)
        return
    es = h.element_size()
    fits = all(32 * (K + 2) * es + 4 * K * 16 <= 200 * 1024 for K in (C, F))   # a tile of 32 outputs, four rows a warp
    grouped = MOE_GROUPED and T * top >= MOE_GROUPED_MIN_ROWS_PER_EXPERT * E and fits
    if not grouped:
        moe_up(h, w_up, ids, inner, T, top, act, gated, in_w, act_prm)
        moe_down(inner, w_down, ids, out_w, x, T, top)
        return
    _f32(x, "moe_experts: x")
    if h.dtype != w_up.dtype or inner.dtype != h.dtype or not w_up.is_contiguous() or not w_down.is_contiguous() \
            or not inner.is_contiguous() or h.stride(1) != 1:
        raise KernelError("moe_experts: h, the experts and inner share a dtype, contiguous")
    lib, dt = library(), _dt(h)
    if tracing():
        _note("moe", "experts_up", (T * top, C, F), 2.0 * T * top * C * F,
              h.element_size() * (min(E, T * top) * F * C + T * C + T * top * F))
    if gated:
        _check(lib.nib_moe_grouped(dt, 3, _ptr(h), h.stride(0), _ptr(w_up), _ptr(ids), _ptr(in_w), _ptr(inner), None, T,
                                   top, E, 2 * F, C, int(act), float(act_prm), _stream()), "moe_grouped gated up")
    else:
        _check(lib.nib_moe_grouped(dt, 0, _ptr(h), h.stride(0), _ptr(w_up), _ptr(ids), None, _ptr(inner), None, T, top,
                                   E, F, C, int(act), 0.0, _stream()), "moe_grouped up")
    parts = workspace.get("moe.parts", (T * top, C), torch.float32)
    if tracing():
        _note("moe", "experts_down", (T * top, F, C), 2.0 * T * top * C * F,
              h.element_size() * (min(E, T * top) * F * C + T * top * F) + 4.0 * T * top * C)
    _check(lib.nib_moe_grouped(dt, 1, _ptr(inner), inner.stride(0), _ptr(w_down), _ptr(ids), _ptr(out_w), _ptr(parts),
                               None, T, top, E, C, F, 0, 0.0, _stream()), "moe_grouped down")
    if tracing():
        _note("other", "experts_sum", (T, C, top), T * C * top, 4.0 * T * C * (top + 2))
    _check(lib.nib_moe_grouped(dt, 2, _ptr(parts), 0, None, _ptr(ids), None, None, _ptr(x), T, top, E, C, F, 0, 0.0, _stream()),
           "moe_grouped sum")


# ----------------------------------------------------------------------------- sublayers normed on both sides
def add_norm(x: torch.Tensor, y: torch.Tensor, w_out: torch.Tensor, eps: float, n_rows: int,
             w_next: Optional[torch.Tensor] = None, xn: Optional[torch.Tensor] = None) -> None:
    """x[:n] += y / sqrt(mean(y^2) + eps) * w_out and y[:n] = 0, all in 32-bit; with ``xn`` also the next sublayer's
    input in xn's dtype: xn[:n] = x / sqrt(mean(x^2) + eps) * w_next, or the new x itself where ``w_next`` is None."""
    _f32(x, "add_norm: x"); _f32(y, "add_norm: y"); _f32(w_out, "add_norm: w_out")
    C = x.shape[1]
    if not x.is_contiguous() or not y.is_contiguous() or y.shape[1] != C or w_out.numel() != C:
        raise KernelError("add_norm: x and y contiguous [rows, C], the weights [C]")
    if w_next is not None:
        _f32(w_next, "add_norm: w_next")
        if xn is None or w_next.numel() != C:
            raise KernelError("add_norm: w_next [C] needs xn")
    if xn is not None and (not xn.is_contiguous() or xn.shape[1] != C):
        raise KernelError("add_norm: xn contiguous [rows, C]")
    if tracing():
        _note("ln", "add_norm", (n_rows, C, 0), 10.0 * n_rows * C,
              n_rows * C * (16.0 + (xn.element_size() if xn is not None else 0)))
    _check(library().nib_add_norm(_dt(xn) if xn is not None else 0, _ptr(x), _ptr(y), _ptr(w_out), _ptr(w_next),
                                  float(eps), _ptr(xn), n_rows, C, _stream()), "add_norm")


def glu(pre: torch.Tensor, out: torch.Tensor, n_rows: int, F: int, act: int, row_gate: int = -1) -> None:
    """out[t, f] = act(pre[t, 2f]) * pre[t, 2f + 1], times sigmoid(pre[t, row_gate]) where ``row_gate`` >= 0."""
    if pre.stride(1) != 1 or out.stride(1) != 1 or pre.shape[1] < 2 * F or out.shape[1] < F or row_gate >= pre.shape[1]:
        raise KernelError("glu: pre [rows, >= 2F] and out [rows, >= F], rows contiguous")
    if tracing():
        _note("other", "glu", (n_rows, F, 0), 8.0 * n_rows * F, n_rows * F * (2.0 * pre.element_size() + out.element_size()))
    _check(library().nib_glu(_dt(pre), _dt(out), _ptr(pre), pre.stride(0), _ptr(out), out.stride(0), n_rows, F, int(act),
                             int(row_gate), _stream()), "glu")


def rope_append(proj: torch.Tensor, offsets, n_head: int, n_kv_head: int, dim: int, vdim: int, rot_dims: int,
                freqs: Optional[torch.Tensor], ctx, q_out: torch.Tensor, cache: Optional[torch.Tensor],
                block_table: Optional[torch.Tensor]) -> None:
    """From the 32-bit q/k/v projection ``proj`` (q, k, v at the three column ``offsets``; heads of ``dim``,
    ``dim`` and ``vdim`` values): rotary positions on the first ``rot_dims`` values of every query and key head
    (interleaved pairs, angle = position * freqs[i], in double precision), the cast, and the padding of every head
    to the cache's head size; queries to ``q_out`` [rows, n_head * head size], keys and values to the rows' slots of
    the cache layer [pages, 2, kv heads, page, head size] (None: queries only)."""
    _f32(proj, "rope_append: proj")
    hd = q_out.shape[1] // n_head
    if cache is not None:
        n_pages, two, g, page_size, chd = cache.shape
        if two != 2 or g != n_kv_head or chd != hd or not cache.is_contiguous() or cache.dtype != q_out.dtype:
            raise KernelError("rope_append: cache must be contiguous [pages, 2, kv heads, page, head size] of q_out's dtype")
        _i32(block_table, "block_table")
    else:
        n_pages, page_size = 0, 1
    if freqs is not None and freqs.dtype != torch.float64:
        raise KernelError("rope_append: freqs must be float64")
    if tracing():
        n = (n_head + 2 * n_kv_head) * hd
        _note("kv_write", "rope_kv_write", (ctx.n_rows, n, 0), 6.0 * ctx.n_rows * n, ctx.n_rows * n * (4.0 + q_out.element_size()))
    _check(library().nib_rope_append(_dt(q_out), _ptr(proj), proj.stride(0), offsets[0], offsets[1], offsets[2], n_head,
                                     n_kv_head, dim, vdim, hd, rot_dims, _ptr(freqs), _ptr(ctx.positions),
                                     _ptr(ctx.row_entry), _ptr(q_out), q_out.stride(0), _ptr(cache), _ptr(block_table),
                                     block_table.shape[1] if block_table is not None else 0, page_size, n_pages,
                                     ctx.n_rows, _ptr(ctx.status), _stream()), "rope_append")


def mlstm_state_floats(dim: int, vdim: int) -> int:
    """Floats of state per head of the matrix memory: [vdim + 1 columns][dim rounded up to 16], then the running
    maximum and three unused floats."""
    return (vdim + 1) * (-(-dim // 16) * 16) + 4


def mlstm(proj: torch.Tensor, offsets, bias_i: torch.Tensor, bias_f: torch.Tensor, cap: float, norm_w: torch.Tensor,
          state: torch.Tensor, ctx, n_head: int, dim: int, vdim: int, eps: float, out: torch.Tensor, workspace) -> None:
    """The matrix memory over the step's rows, entry by entry in row order, from the 32-bit projections ``proj``
    (q, k, v, g, input gate, forget gate at the six column ``offsets``); state [slots, n_head *
    mlstm_state_floats] float32 from and to each entry's slot; out[:, :n_head * vdim] in out's dtype."""
    _f32(proj, "mlstm: proj"); _f32(state, "mlstm: state"); _f32(norm_w, "mlstm: norm_w")
    if not state.is_contiguous() or state[0].numel() != n_head * mlstm_state_floats(dim, vdim):
        raise KernelError("mlstm: state must be contiguous [slots, n_head * mlstm_state_floats(dim, vdim)]")
    n = proj.shape[0]
    gates = workspace.get("mlstm.gates", (n, n_head, 4), torch.float32)
    num = workspace.get("mlstm.num", (n, n_head * vdim), torch.float32)
    den = workspace.get("mlstm.den", (n, n_head), torch.float32)
    if tracing():
        T = ctx.n_rows
        _note("scan", "mlstm", (T, n_head * dim, n_head * vdim), 6.0 * T * n_head * dim * vdim,
              4.0 * T * n_head * (2 * dim + 3 * vdim) + 8.0 * ctx.n_entries * n_head * dim * vdim)
    _check(library().nib_mlstm(_dt(out), _ptr(proj), proj.stride(0), *[int(o) for o in offsets], _ptr(bias_i), _ptr(bias_f),
                               float(cap), _ptr(norm_w), _ptr(state), _ptr(ctx.entry_start), _ptr(ctx.entry_slot),
                               ctx.n_entries, ctx.n_rows, n_head, dim, vdim, float(eps), _ptr(gates), _ptr(num),
                               num.stride(0), _ptr(den), _ptr(out), out.stride(0), _stream()), "mlstm", 3)


# ----------------------------------------------------------------------------- sinusoidal positions, a per-token gate
def add_sinusoid(x: torch.Tensor, positions: torch.Tensor, freqs: torch.Tensor, n_rows: int) -> None:
    """x[t, 2i] += sin(positions[t] * freqs[i]), x[t, 2i + 1] += cos of the same angle (angles, sines and cosines in
    double precision); x is the 32-bit stream, freqs float64 [ceil(C / 2)]."""
    _f32(x, "add_sinusoid: x")
    _i32(positions, "positions")
    C = x.shape[1]
    if not x.is_contiguous() or freqs.dtype != torch.float64 or freqs.numel() < (C + 1) // 2:
        raise KernelError("add_sinusoid: x contiguous [rows, C], freqs float64 [ceil(C / 2)]")
    if tracing():
        _note("embed", "sinusoid", (n_rows, C, 0), 20.0 * n_rows * C, 8.0 * n_rows * C)
    _check(library().nib_add_sinusoid(_ptr(x), _ptr(positions), _ptr(freqs), n_rows, C, _stream()), "add_sinusoid")


def gate_by_table(pre: torch.Tensor, tokens: torch.Tensor, feedback: Optional[torch.Tensor], table: torch.Tensor,
                  off: int, D: int, act: int, out: torch.Tensor, n_rows: int) -> None:
    """out[t, d] = act(pre[t, d]) * table[tokens[t], off + d] for d < D; pre is 32-bit, table and out share a dtype.
    A negative token -(s + 1) stands for ``feedback[s]``, as in ``embed``."""
    _f32(pre, "gate_by_table: pre")
    _i32(tokens, "tokens")
    if table.dtype != out.dtype or table.stride(1) != 1 or out.stride(1) != 1 or pre.stride(1) != 1 \
            or off < 0 or off + D > table.shape[1] or pre.shape[1] < D or out.shape[1] < D:
        raise KernelError("gate_by_table: table and out of one dtype, rows contiguous, off + D within the table")
    if tracing():
        _note("other", "token_gate", (n_rows, D, 0), 10.0 * n_rows * D, n_rows * D * (4.0 + 2 * out.element_size()))
    _check(library().nib_gate_by_table(_dt(out), _ptr(pre), pre.stride(0), _ptr(tokens), _ptr(feedback), _ptr(table),
                                       table.stride(0), int(off), int(D), int(act), _ptr(out), out.stride(0), n_rows,
                                       _stream()), "gate_by_table")


def norm_rope_append(proj: torch.Tensor, offsets, n_head: int, n_kv_head: int, dim: int, vdim: int,
                     wq: Optional[torch.Tensor], wk: Optional[torch.Tensor], eps: float, rot_dims: int,
                     freqs: Optional[torch.Tensor], ctx, q_out: torch.Tensor, cache: Optional[torch.Tensor],
                     block_table: Optional[torch.Tensor]) -> None:
    """``rope_append`` with an RMS norm of every query and key head ahead of the rotation: x / sqrt(mean(x^2) + eps)
    times a weight of ``dim`` values that the heads share (``wq`` for queries, ``wk`` for keys; None: no norm)."""
    _f32(proj, "norm_rope_append: proj")
    hd = q_out.shape[1] // n_head
    if cache is not None:
        n_pages, two, g, page_size, chd = cache.shape
        if two != 2 or g != n_kv_head or chd != hd or not cache.is_contiguous() or cache.dtype != q_out.dtype:
            raise KernelError("norm_rope_append: cache must be contiguous [pages, 2, kv heads, page, head size] of "
                              "q_out's dtype")
        _i32(block_table, "block_table")
    else:
        n_pages, page_size = 0, 1
    for w in (wq, wk):
        if w is not None and (w.dtype != torch.float32 or w.numel() != dim):
            raise KernelError("norm_rope_append: a norm weight must be float32 [dim]")
    if freqs is not None and freqs.dtype != torch.float64:
        raise KernelError("norm_rope_append: freqs must be float64")
    if tracing():
        n = (n_head + 2 * n_kv_head) * hd
        _note("kv_write", "norm_kv_write", (ctx.n_rows, n, 0), 8.0 * ctx.n_rows * n, ctx.n_rows * n * (4.0 + q_out.element_size()))
    _check(library().nib_norm_rope_append(
        _dt(q_out), _ptr(proj), proj.stride(0), offsets[0], offsets[1], offsets[2], n_head, n_kv_head, dim, vdim, hd,
        _ptr(wq), _ptr(wk), float(eps), rot_dims, _ptr(freqs), _ptr(ctx.positions), _ptr(ctx.row_entry), _ptr(q_out),
        q_out.stride(0), _ptr(cache), _ptr(block_table), block_table.shape[1] if block_table is not None else 0,
        page_size, n_pages, ctx.n_rows, _ptr(ctx.status), _stream()), "norm_rope_append")


# ----------------------------------------------------------------------------- recurrences with one decay per head
def gated_scan_padded(n: int) -> int:
    """The key size ``n`` rounded up to what a variant of the recurrence kernel holds (0: too large)."""
    return int(library().nib_gated_scan_padded(int(n)))


def gated_scan_state_floats(taps: int, channels: int, n_head: int, n: int, v: int) -> int:
    """Floats of state per request: the convolution's last ``taps - 1`` inputs of ``channels`` values each (rounded up
    to a multiple of 4), then a matrix [v][n padded] per head."""
    return -(-(max(taps - 1, 0) * channels) // 4) * 4 + n_head * v * _scan_padded_host(n)


def _scan_padded_host(n: int) -> int:
    for s in (16, 32, 48, 64, 96, 128, 192, 256):
        if n <= s:
            return s
    return 0


def short_conv(proj: torch.Tensor, c_off: int, channels: int, taps: int, w: torch.Tensor, bias: Optional[torch.Tensor],
               state: torch.Tensor, ctx, out: torch.Tensor, act: int, out16: Optional[torch.Tensor] = None) -> None:
    """out[t, c] = act(bias[c] + sum_j w[c, j] x[t - (taps - 1 - j), c]) over the columns c_off .. of the 32-bit
    ``proj``, per batch entry in row order; what lies before an entry's first row comes from the first
    (taps - 1) * channels floats of the request's row of ``state`` (oldest first), which then moves on by the
    entry's rows.  A step in which every entry is one row does both in one launch.  ``out16`` (bfloat16, optional)
    receives the same values once more, for a matrix product that reads them."""
    _f32(proj, "short_conv: proj"); _f32(out, "short_conv: out"); _f32(w, "short_conv: w")
    if state is None and taps > 1:
        raise KernelError("short_conv: more than one tap needs the requests' state")
    if state is not None and state.dtype != torch.float32:       # (a view of some columns of the slots' rows will do)
        raise KernelError("short_conv: state must be float32")
    if w.shape != (channels, taps) or not w.is_contiguous() or proj.stride(1) != 1 or out.stride(1) != 1 \
            or (state is not None and state.stride(1) != 1) or out.shape[1] < channels:
        raise KernelError("short_conv: w contiguous [channels, taps], rows of proj, out and state contiguous")
    T, E = ctx.n_rows, ctx.n_entries
    if out16 is not None and (out16.dtype != torch.bfloat16 or out16.stride(1) != 1 or out16.shape[1] < channels):
        raise KernelError("short_conv: out16 must be bfloat16 [rows, >= channels], rows contiguous")
    fused = int(T == E)      # (every entry has a row, so as many rows as entries means one each)
    if tracing():
        _note("other", "short_conv", (T, channels, taps), 2.0 * T * channels * taps, 8.0 * T * channels)
    _check(library().nib_short_conv(_ptr(proj), proj.stride(0), int(c_off), int(channels), int(taps), _ptr(w),
                                    _ptr(bias), _ptr(state), state.stride(0) if state is not None else 0, _ptr(ctx.row_entry),
                                    _ptr(ctx.entry_start),
                                    _ptr(ctx.entry_slot), _ptr(out), out.stride(0), T, E, int(act), fused, _ptr(out16),
                                    out16.stride(0) if out16 is not None else 0, _stream()),
           "short_conv", 1 if fused or taps <= 1 else 2)


def scan_prepare(proj: torch.Tensor, a_off: int, w_off: int, A_log: torch.Tensor, dt_bias: torch.Tensor,
                 cv: torch.Tensor, q_off: int, k_off: int, n: int, n_head: int, n_kq: int, delta: bool,
                 coef: torch.Tensor, n_rows: int) -> None:
    """coef[t, h] = (decay, strength) of every row and head, from the 32-bit projections; for the delta rule also
    the query and key heads of ``cv`` made unit vectors in place (queries times n^-1/2)."""
    _f32(proj, "scan_prepare: proj"); _f32(cv, "scan_prepare: cv"); _f32(coef, "scan_prepare: coef")
    _f32(A_log, "scan_prepare: A_log"); _f32(dt_bias, "scan_prepare: dt_bias")
    if tracing():
        _note("other", "scan_prepare", (n_rows, n_head, 0), 40.0 * n_rows * n_head, 16.0 * n_rows * n_head)
    _check(library().nib_scan_prepare(_ptr(proj), proj.stride(0), int(a_off), int(w_off), _ptr(A_log), _ptr(dt_bias),
                                      _ptr(cv), cv.stride(0), int(q_off), int(k_off), int(n), int(n_head), int(n_kq),
                                      int(bool(delta)), _ptr(coef), n_rows, _stream()), "scan_prepare")


def gated_scan(delta: bool, cv: torch.Tensor, q_off: int, k_off: int, v_off: int, n: int, v: int, n_head: int,
               kq_ratio: int, coef: torch.Tensor, skip: Optional[torch.Tensor], state: torch.Tensor, s_off: int, ctx,
               out: torch.Tensor) -> None:
    """The recurrence over the step's rows, entry by entry in row order, per head with S [n x v], decay a and
    strength w of the row:  delta rule: S <- a S; u = w (v - S^T k); S <- S + k u^T; o = S^T q;
    state space: S <- a S + k (w v)^T; o = S^T q + skip[h] v.  ``cv`` holds the rows' vectors (q of key/query head g
    at q_off + g n, k at k_off + g n, v of head h at v_off + h v; head h reads key/query head h // kq_ratio);
    the matrices live at ``s_off`` floats into each request's row of ``state``; out [rows, n_head * v] float32."""
    _f32(cv, "gated_scan: cv"); _f32(coef, "gated_scan: coef"); _f32(out, "gated_scan: out")
    if state.dtype != torch.float32 or state.data_ptr() % 16:       # (a view of some columns of the slots' rows will do)
        raise KernelError("gated_scan: state must be float32, 16-byte aligned")
    if state.stride(1) != 1 or cv.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("gated_scan: rows of cv, state and out must be contiguous")
    if tracing():
        T = ctx.n_rows
        _note("scan", "gated_scan", (T, n_head * n, n_head * v), (8.0 if delta else 6.0) * T * n_head * n * v,
              4.0 * T * n_head * (2 * n + 2 * v) + 8.0 * ctx.n_entries * n_head * n * v)
    _check(library().nib_gated_scan(int(bool(delta)), _ptr(cv), cv.stride(0), int(q_off), int(k_off), int(v_off), int(n),
                                    int(v), int(n_head), int(kq_ratio), _ptr(coef), _ptr(skip), _ptr(state),
                                    state.stride(0), int(s_off), _ptr(ctx.entry_start), _ptr(ctx.entry_slot),
                                    ctx.n_entries, _ptr(out), out.stride(0), _stream()), "gated_scan")


def gated_norm(o: torch.Tensor, gate: Optional[torch.Tensor], weight: torch.Tensor, n_groups: int, group_size: int,
               eps: float, gate_first: bool, out_scale: float, out: torch.Tensor, n_rows: int) -> None:
    """Per row and group of ``group_size`` values: y = o (times silu(gate) first where ``gate_first``), over its root
    mean square, times weight[(index in the row) mod len(weight)] (times silu(gate) afterwards otherwise), times
    ``out_scale``, in out's dtype.  o and gate are 32-bit."""
    _f32(o, "gated_norm: o"); _f32(weight, "gated_norm: weight")
    if gate is not None and gate.dtype != torch.float32:
        raise KernelError("gated_norm: gate must be float32")
    if o.stride(1) != 1 or out.stride(1) != 1 or (gate is not None and gate.stride(1) != 1):
        raise KernelError("gated_norm: rows must be contiguous")
    if tracing():
        n = n_groups * group_size
        _note("ln", "gated_norm", (n_rows, n, 0), 12.0 * n_rows * n, n_rows * n * (8.0 + out.element_size()))
    _check(library().nib_gated_norm(_dt(out), _ptr(o), o.stride(0), _ptr(gate), gate.stride(0) if gate is not None else 0,
                                    _ptr(weight), weight.numel(), int(n_groups), int(group_size), float(eps),
                                    int(bool(gate_first)), float(out_scale), _ptr(out), out.stride(0), n_rows, _stream()),
           "gated_norm")


# ----------------------------------------------------------------------------- rotary positions in the halves layout
def wide_norm_rope_append(src: torch.Tensor, offsets, n_head: int, n_kv_head: int, dim: int, vdim: int,
                          wq: Optional[torch.Tensor], wk: Optional[torch.Tensor], eps: float, rot_dims: int,
                          freqs: Optional[torch.Tensor], ctx, q_out: torch.Tensor, cache: Optional[torch.Tensor],
                          block_table: Optional[torch.Tensor]) -> None:
    """From 32-bit rows ``src`` (q, k, v at the three column ``offsets``): queries and keys divided by the root mean
    square of the WHOLE projection (all heads at once, ``eps`` inside the root) and multiplied by a weight of the
    projection's size (``wq`` [n_head * dim], ``wk`` [n_kv_head * dim]; None: no norm), then turned by the rows'
    positions in the halves layout (value i of a head's first ``rot_dims`` pairs with value i + rot_dims / 2), cast,
    padded to the cache's head size and written: queries to ``q_out``, keys and values to the rows' cache slots.
    The values are read as they stand; their offset may be the keys' own."""
    _f32(src, "wide_norm_rope_append: src")
    hd = q_out.shape[1] // n_head
    if cache is not None:
        n_pages, two, g, page_size, chd = cache.shape
        if two != 2 or g != n_kv_head or chd != hd or not cache.is_contiguous() or cache.dtype != q_out.dtype:
            raise KernelError("wide_norm_rope_append: cache must be contiguous [pages, 2, kv heads, page, head size] of "
                              "q_out's dtype")
        _i32(block_table, "block_table")
    else:
        n_pages, page_size = 0, 1
    if (wq is not None and (wq.dtype != torch.float32 or wq.numel() != n_head * dim)) or \
            (wk is not None and (wk.dtype != torch.float32 or wk.numel() != n_kv_head * dim)):
        raise KernelError("wide_norm_rope_append: a norm weight must be float32 of the projection's size")
    if freqs is not None and freqs.dtype != torch.float64:
        raise KernelError("wide_norm_rope_append: freqs must be float64")
    if tracing():
        n = (n_head + 2 * n_kv_head) * hd
        _note("kv_write", "norm_kv_write", (ctx.n_rows, n, 0), 8.0 * ctx.n_rows * n, ctx.n_rows * n * (4.0 + q_out.element_size()))
    _check(library().nib_wide_norm_rope_append(
        _dt(q_out), _ptr(src), src.stride(0), offsets[0], offsets[1], offsets[2], n_head, n_kv_head, dim, vdim, hd,
        _ptr(wq), _ptr(wk), float(eps), rot_dims, _ptr(freqs), _ptr(ctx.positions), _ptr(ctx.row_entry), _ptr(q_out),
        q_out.stride(0), _ptr(cache), _ptr(block_table), block_table.shape[1] if block_table is not None else 0,
        page_size, n_pages, ctx.n_rows, _ptr(ctx.status), _stream()), "wide_norm_rope_append")


def rope_halves(rows: torch.Tensor, q_off: int, k_off: int, n_head: int, dim: int, rot_dims: int,
                freqs: Optional[torch.Tensor], positions: torch.Tensor, k_mul: float, n_rows: int,
                decay: Optional[torch.Tensor] = None, coef: Optional[torch.Tensor] = None) -> None:
    """In place on the 32-bit ``rows``: ``n_head`` query heads at ``q_off`` and as many key heads at ``k_off`` turned
    by the rows' positions in the halves layout, the keys then times ``k_mul``.  With ``coef`` (float32
    [rows, n_head, 2]): coef[t, h] = (decay[h], 1), the decays and strengths of a recurrence whose decay is fixed."""
    _f32(rows, "rope_halves: rows")
    _i32(positions, "positions")
    if freqs is not None and freqs.dtype != torch.float64:
        raise KernelError("rope_halves: freqs must be float64")
    if coef is not None:
        _f32(coef, "rope_halves: coef"); _f32(decay, "rope_halves: decay")
        if decay.numel() != n_head:
            raise KernelError("rope_halves: one decay per head")
    if tracing():
        _note("other", "rope", (n_rows, 2 * n_head * dim, 0), 6.0 * n_rows * n_head * dim, 16.0 * n_rows * n_head * dim)
    _check(library().nib_rope_halves(_ptr(rows), rows.stride(0), int(q_off), int(k_off), int(n_head), int(dim),
                                     int(rot_dims), _ptr(freqs), _ptr(positions), float(k_mul), _ptr(decay), _ptr(coef),
                                     n_rows, _stream()), "rope_halves")


# ----------------------------------------------------------------------------- hyper-connections
def hyper_enter(x: torch.Tensor, streams: torch.Tensor, in_w: torch.Tensor, w_next: torch.Tensor, eps: float,
                xn: torch.Tensor, n_rows: int) -> None:
    """streams[s][:n] = x[:n] for every copy s, and the first sublayer's input xn = u / sqrt(mean(u^2) + eps) * w_next
    with u = sum_s in_w[s] * streams[s]; x [rows, C] and streams [S, rows, C] are 32-bit."""
    _f32(x, "hyper_enter: x"); _f32(streams, "hyper_enter: streams"); _f32(in_w, "hyper_enter: in_w"); _f32(w_next, "hyper_enter: w_next")
    S, C = streams.shape[0], x.shape[1]
    if streams.shape[2] != C or in_w.numel() != S or w_next.numel() != C or not xn.is_contiguous() or xn.shape[1] != C:
        raise KernelError("hyper_enter: streams [S, rows, C], in_w [S], w_next [C], xn contiguous [rows, C]")
    if tracing():
        _note("ln", "hyper", (n_rows, C, S), 4.0 * n_rows * C, n_rows * C * (4.0 + 4.0 * S + xn.element_size()))
    _check(library().nib_hyper_enter(_dt(xn), _ptr(x), _ptr(streams), streams.stride(0), S, _ptr(in_w), _ptr(w_next),
                                     float(eps), _ptr(xn), n_rows, C, _stream()), "hyper_enter")


def hyper_update(streams: torch.Tensor, y: torch.Tensor, gate: Optional[torch.Tensor], mix: torch.Tensor,
                 out_w: torch.Tensor, eps: float, n_rows: int, in_next: Optional[torch.Tensor] = None,
                 w_next: Optional[torch.Tensor] = None, xn: Optional[torch.Tensor] = None,
                 total: Optional[torch.Tensor] = None) -> None:
    """A sublayer's result ``y`` (32-bit [rows, C], zeroed here for the next one) goes back into the S copies of the
    stream: r = y * sigmoid(gate) (``gate`` None: r = y); streams[t] <- sum_s mix[s, t] streams[s] + out_w[t] r, all
    copies at once from the old ones.  With ``xn``: the next sublayer's input, the norm (weight ``w_next``) of
    sum_s in_next[s] streams[s], in xn's dtype.  ``total`` (32-bit [rows, C], optional) receives the copies' sum."""
    _f32(streams, "hyper_update: streams"); _f32(y, "hyper_update: y"); _f32(mix, "hyper_update: mix"); _f32(out_w, "hyper_update: out_w")
    S, C = streams.shape[0], y.shape[1]
    if streams.shape[2] != C or mix.numel() != S * S or out_w.numel() != S:
        raise KernelError("hyper_update: streams [S, rows, C], mix [S, S], out_w [S]")
    if gate is not None and (gate.dtype != torch.float32 or gate.stride(1) != 1 or gate.shape[1] < C):
        raise KernelError("hyper_update: gate must be float32 [rows, >= C], rows contiguous")
    if xn is not None:
        _f32(in_next, "hyper_update: in_next"); _f32(w_next, "hyper_update: w_next")
        if in_next.numel() != S or w_next.numel() != C or not xn.is_contiguous() or xn.shape[1] != C:
            raise KernelError("hyper_update: in_next [S], w_next [C], xn contiguous [rows, C]")
    if total is not None:
        _f32(total, "hyper_update: total")
    if tracing():
        _note("ln", "hyper", (n_rows, C, S), (6.0 + 2.0 * S * S) * n_rows * C,
              n_rows * C * (8.0 + 8.0 * S + (4.0 if gate is not None else 0.0) + (xn.element_size() if xn is not None else 0)))
    _check(library().nib_hyper_update(_dt(xn) if xn is not None else 0, _ptr(streams), streams.stride(0), S, _ptr(y),
                                      _ptr(gate), gate.stride(0) if gate is not None else 0, _ptr(mix), _ptr(out_w),
                                      _ptr(in_next) if xn is not None else None, _ptr(w_next) if xn is not None else None,
                                      float(eps), _ptr(xn), _ptr(total), n_rows, C, _stream()), "hyper_update")


# ----------------------------------------------------------------------------- the selective scan
def selective_scan_padded(n: int) -> int:
    """The state size ``n`` rounded up to lanes x states a lane of the kernel (0: too large): two states a lane while
    the lanes of a warp suffice, then 4 or 8."""
    if n <= 0 or n > 256:
        return 0
    lanes = 1
    while lanes < 32 and -(-n // lanes) > 2:
        lanes *= 2
    per = 1
    while per * lanes < n:
        per *= 2
    return lanes * per


def selective_scan(dtp: torch.Tensor, x: torch.Tensor, bc: torch.Tensor, b_off: int, c_off: int, z: torch.Tensor,
                   A_log: torch.Tensor, D: torch.Tensor, state: torch.Tensor, s_off: int, ctx, inner: int, n: int,
                   out: torch.Tensor) -> None:
    """Mamba's recurrence over the step's rows, entry by entry in row order (csrc/selective_scan.cu): per channel c and
    state index j, with dt = softplus(dtp):  S[c, j] <- exp(-dt_c exp(A_log[c, j])) S[c, j] + dt_c x_c B_j;
    out_c = (sum_j S[c, j] C_j + D_c x_c) * silu(z_c).  ``dtp``, ``x``, ``z`` [rows, >= inner] and ``bc`` (B at
    ``b_off``, C at ``c_off``) are 32-bit; the matrices [inner][selective_scan_padded(n)] live ``s_off`` floats into
    each request's row of ``state``."""
    for t, name in ((dtp, "dtp"), (x, "x"), (bc, "bc"), (z, "z"), (state, "state")):
        if t.dtype != torch.float32 or t.stride(1) != 1:
            raise KernelError(f"selective_scan: {name} must be float32 with contiguous rows")
    _f32(A_log, "selective_scan: A_log"); _f32(D, "selective_scan: D")
    if A_log.numel() != inner * n or D.numel() != inner or out.stride(1) != 1 or selective_scan_padded(n) == 0:
        raise KernelError("selective_scan: A_log [inner, n], D [inner], n at most 256")
    if tracing():
        T = ctx.n_rows
        _note("scan", "selective_scan", (T, inner, n), 9.0 * T * inner * n,
              T * (inner * (12.0 + out.element_size()) + 8.0 * n) + 8.0 * ctx.n_entries * inner * n)
    _check(library().nib_selective_scan(_dt(out), _ptr(dtp), dtp.stride(0), _ptr(x), x.stride(0), _ptr(bc), bc.stride(0),
                                        int(b_off), int(c_off), _ptr(z), z.stride(0), _ptr(A_log), _ptr(D), _ptr(state),
                                        state.stride(0), int(s_off), _ptr(ctx.entry_start), _ptr(ctx.entry_slot),
                                        ctx.n_entries, int(inner), int(n), _ptr(out), out.stride(0), _stream()),
           "selective_scan")
