"""Gated dense feed-forward of the token-major models (net-new; beside `MLP`, which serves bfloat16 rows one sequence at
a time, and `GroupedRouterMoE`).  Two launches: the fused gate/up product whose epilogue applies the activation to
interleaved (gate_j, up_j) pairs, and the down projection.

  activation "silu":           silu(g) * u
  activation "clamped_swish":  g <- min(g, limit), u <- clamp(u, -limit, limit), g * sigmoid(alpha g) * (u + 1)

`SquaredReluRows` is the feed-forward without a gate, W_down max(W_up h, 0)^2, the activation again in the first product's
epilogue.

`forward(..., out_scale=ptr)` adds `out_scale * result` to `out` in the down projection's epilogue (layer scale and
residual add of a parallel block); without it the result is stored.
"""
from __future__ import annotations

from ..config import DenseSpec
from .linear import LinearRows


class GatedDenseRows:
    def __init__(self, spec: DenseSpec, gate_up: LinearRows, down: LinearRows):
        if spec.activation not in ("silu", "clamped_swish"):
            raise ValueError(f"GatedDenseRows: unknown activation {spec.activation!r}")
        if gate_up.out_features != 2 * spec.ff or down.in_features != spec.ff:
            raise ValueError("GatedDenseRows: matrices do not match the feed-forward size")
        self.spec, self.gate_up, self.down = spec, gate_up, down

    @property
    def weight_bytes(self) -> int:
        return self.gate_up.nbytes + self.down.nbytes

    def forward(self, ctx, h_ptr: int, out_ptr: int, out_scale: int | None = None) -> None:
        sp, T = self.spec, ctx.T
        W, act = self.gate_up.in_features, ctx.buf.shared_act
        if sp.activation == "silu":
            self.gate_up.forward_seq(h_ptr, W, T, act.device_ptr, sp.ff, epilogue=1)
        else:
            self.gate_up.forward_seq(h_ptr, W, T, act.device_ptr, sp.ff, epilogue=3, p0=sp.alpha, p1=sp.limit)
        if out_scale is None:
            self.down.forward_seq(act.device_ptr, sp.ff, T, out_ptr, self.down.out_features, epilogue=0)
        else:
            self.down.forward_seq(act.device_ptr, sp.ff, T, out_ptr, self.down.out_features, epilogue=4, col_scale=out_scale)


class SquaredReluRows:
    def __init__(self, spec: DenseSpec, up: LinearRows, down: LinearRows):
        if spec.activation != "relu2":
            raise ValueError(f"SquaredReluRows: activation {spec.activation!r}")
        if up.out_features != spec.ff or down.in_features != spec.ff:
            raise ValueError("SquaredReluRows: matrices do not match the feed-forward size")
        self.spec, self.up, self.down = spec, up, down

    @property
    def weight_bytes(self) -> int:
        return self.up.nbytes + self.down.nbytes

    def forward(self, ctx, h_ptr: int, out_ptr: int, out_scale: int | None = None) -> None:
        sp, T = self.spec, ctx.T
        W, act = self.up.in_features, ctx.buf.shared_act
        self.up.forward_seq(h_ptr, W, T, act.device_ptr, sp.ff, epilogue=6)
        if out_scale is None:
            self.down.forward_seq(act.device_ptr, sp.ff, T, out_ptr, self.down.out_features, epilogue=0)
        else:
            self.down.forward_seq(act.device_ptr, sp.ff, T, out_ptr, self.down.out_features, epilogue=4, col_scale=out_scale)


class PolyNormRows:
    """Feed-forward without a gate whose activation is a polynomial of normalised powers: with z = W_up h,
    act = c0 z / rms(z) + c1 z^2 / rms(z^2) + c2 z^3 / rms(z^3) + c3 (powers element by element, each root mean square over
    the ff values of the token), then W_down.  The activation needs whole rows, so it is a launch of its own between the two
    products (pgk_polynorm_rows_f32, in place)."""

    def __init__(self, spec: DenseSpec, up: LinearRows, down: LinearRows, coef, eps: float):
        """coef: device array of the four numbers"""
        if spec.activation != "polynorm":
            raise ValueError(f"PolyNormRows: activation {spec.activation!r}")
        if up.out_features != spec.ff or down.in_features != spec.ff or coef.size != 4:
            raise ValueError("PolyNormRows: matrices or coefficients do not match the feed-forward size")
        self.spec, self.up, self.down, self.coef, self.eps = spec, up, down, coef, float(eps)

    @property
    def weight_bytes(self) -> int:
        return self.up.nbytes + self.down.nbytes

    def forward(self, ctx, h_ptr: int, out_ptr: int, out_scale: int | None = None) -> None:
        from ..._lib import api
        from ...core.stream import current_stream_handle as _st
        sp, T = self.spec, ctx.T
        W, act = self.up.in_features, ctx.buf.shared_act
        self.up.forward_seq(h_ptr, W, T, act.device_ptr, sp.ff, epilogue=0)
        api.polynorm_rows_f32(act.device_ptr, sp.ff, self.coef.device_ptr, self.eps, T, sp.ff, _st())
        if out_scale is None:
            self.down.forward_seq(act.device_ptr, sp.ff, T, out_ptr, self.down.out_features, epilogue=0)
        else:
            self.down.forward_seq(act.device_ptr, sp.ff, T, out_ptr, self.down.out_features, epilogue=4, col_scale=out_scale)

    def forward_rows(self, ctx, x, out) -> None:
        self.forward(ctx, x.device_ptr, out.device_ptr)


__all__ = ["GatedDenseRows", "SquaredReluRows", "PolyNormRows"]
