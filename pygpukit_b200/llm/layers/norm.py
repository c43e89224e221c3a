"""Norm layer (mirror of pygpukit/llm/layers/norm.py:19-44)."""
from __future__ import annotations

from typing import Literal

from ...core.array import GPUArray
from ...ops.nn import layernorm, rmsnorm


class Norm:
    """Unified RMSNorm / LayerNorm."""

    def __init__(self, weight: GPUArray, bias: GPUArray | None = None,
                 norm_type: Literal["rmsnorm", "layernorm"] = "rmsnorm", eps: float = 1e-5):
        self.weight = weight
        self.bias = bias
        self.norm_type = norm_type
        self.eps = eps

    def __call__(self, x: GPUArray, *, out: GPUArray | None = None) -> GPUArray:
        if self.norm_type == "rmsnorm":
            return rmsnorm(x, self.weight, self.eps, out=out)
        if self.bias is None:
            raise ValueError("LayerNorm requires bias")
        return layernorm(x, self.weight, self.bias, self.eps, out=out)


class RowNorm:
    """Norm of float32 rows in the token-major models: "layernorm" (weight, bias; "layernorm_nobias": weight alone), an RMS norm whose weight enters as
    (offset + weight) -- offset 1 for weights stored around zero, 0 for plain ones -- or "dyt", tanh(alpha x) * weight + bias
    with a scalar alpha, a pointwise squashing that takes no statistic of the row and has no eps.  `forward` can gather its rows
    (final norm of the wanted rows), add a second summand first and write the sum back (the start of a loop pass), or
    accumulate into the output (a normalised branch added to the residual stream)."""

    def __init__(self, kind: str, weight: GPUArray, bias: GPUArray | None = None, eps: float = 1e-5, offset: float = 0.0,
                 alpha: float = 1.0):
        if kind not in ("layernorm", "layernorm_nobias", "rmsnorm", "dyt"):
            raise ValueError(f"RowNorm: unknown kind {kind!r}")
        self.alpha = float(alpha)
        if kind == "layernorm" and bias is None:
            raise ValueError("RowNorm: LayerNorm requires a bias")
        if kind == "layernorm_nobias":
            kind, bias = "layernorm", None
        self.kind, self.weight, self.bias, self.eps, self.offset = kind, weight, bias, float(eps), float(offset)

    @property
    def nbytes(self) -> int:
        return self.weight.nbytes + (self.bias.nbytes if self.bias is not None else 0)

    def forward(self, x_ptr: int, out_ptr: int, rows: int, width: int, *, src_rows: int | None = None,
                add_ptr: int | None = None, sum_out_ptr: int | None = None, accumulate: bool = False) -> None:
        from ..._lib import api
        from ...core.stream import current_stream_handle as _st
        if self.kind == "dyt":
            if add_ptr is not None or sum_out_ptr is not None:
                raise ValueError("RowNorm: a dynamic-tanh row takes no second summand")
            api.dyt_rows_f32(x_ptr, src_rows, self.alpha, self.weight.device_ptr,
                             self.bias.device_ptr if self.bias is not None else None, out_ptr, rows, width, 1 if accumulate else 0,
                             _st())
            return
        if self.kind == "rmsnorm":
            api.rms_norm_rows_f32(x_ptr, src_rows, add_ptr, sum_out_ptr, self.weight.device_ptr, self.offset, self.eps,
                                  out_ptr, rows, width, 1 if accumulate else 0, _st())
            return
        if add_ptr is not None or sum_out_ptr is not None:
            raise ValueError("RowNorm: a LayerNorm row takes no second summand")
        api.combine_layernorm_f32(x_ptr, src_rows, None, None, None, 0, self.weight.device_ptr,
                                  self.bias.device_ptr if self.bias is not None else None, self.eps, out_ptr, rows, width,
                                  1 if accumulate else 0, _st())


    def forward_seam(self, y_ptr: int, x_ptr: int, nxt: "RowNorm", h_ptr: int, rows: int, width: int,
                     add_ptr: int | None = None) -> None:
        """One launch for the seam between two pre-norm blocks: x += self(y); x += add (when given); h = nxt(x).  Both
        norms must be RMS norms with the same eps."""
        from ..._lib import api
        from ...core.stream import current_stream_handle as _st
        api.rms_norm_seam_f32(y_ptr, self.weight.device_ptr, self.offset, x_ptr, add_ptr, nxt.weight.device_ptr, nxt.offset,
                              self.eps, h_ptr, rows, width, _st())

    def fuses_with(self, nxt: "RowNorm | None") -> bool:
        return nxt is not None and self.kind == "rmsnorm" and nxt.kind == "rmsnorm" and self.eps == nxt.eps


class CausalConvRows:
    """Short causal convolution over time in front of a sublayer of the token-major models: u_t = h_t + sum_j w[:, j]
    h_(t - taps + 1 + j), channel by channel, zeros before the sequence's start.  The last taps - 1 inputs of every sequence
    are state: a ring of taps - 1 rows per slot in the cache manager (`state_size` float32 elements per slot).  With
    `double_ring` (the default) the ring is kept twice per slot, a step reads one copy and writes the other (the step
    context's parity), and rows and ring update are ONE launch; without it the ring update is a second launch (rows of the
    first still read the old ring)."""

    def __init__(self, weight: GPUArray, double_ring: bool = True):
        self.weight = weight                                  # [width, taps] float32
        self.width, self.taps = weight.shape
        self.double_ring = bool(double_ring)

    @property
    def state_size(self) -> int:
        return max(0, self.taps - 1) * self.width * (2 if self.double_ring else 1)

    @property
    def nbytes(self) -> int:
        return self.weight.nbytes

    def forward(self, ctx, h_ptr: int, u_ptr: int, state: "GPUArray | None") -> None:
        from ..._lib import api
        from ...core.stream import current_stream_handle as _st
        sp = state.device_ptr if state is not None else None
        api.causal_conv_rows_f32(h_ptr, u_ptr, self.weight.device_ptr, sp, ctx.slot_ptr, ctx.pos_ptr,
                                 ctx.parity_ptr if self.double_ring else None, ctx.T, self.width, self.taps, _st())
        if self.taps > 1 and not self.double_ring:
            seqs_ptr, n_seqs = ctx.seqs()
            api.causal_conv_state_f32(h_ptr, sp, seqs_ptr, n_seqs, self.width, self.taps, _st())


__all__ = ["Norm", "RowNorm", "CausalConvRows"]
