"""Mixers whose recurrence is gated by the data, with a float32 state per sequence in the cache manager (net-new; beside
`LinearAttentionMixer`, whose decay is a constant per head).

`GatedLinearMixer`: S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T, o_t = S_t^T q_t per head, the forget gate f_t per head and
channel.  One fused projection [q | f | v], then

  pgk_seq_gated_prep         q <- silu(q), f <- low + (1 - low) sigmoid(f + bias)
  pgk_seq_gated_recurrence   the walk over the step's tokens, state read and written once
  pgk_seq_linear_finish      every head's output divided by its root mean square, times the shared weight vector

and the output projection.  `attend` is the mixer without its two matrix products, on a block of columns of a wider
projection (one side of a `ParallelMixer`).

`DeltaRuleMixer`: the gated delta rule, S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q.  One fused projection
[q | k | v | gate | beta | a], then

  pgk_causal_conv_rows_ex    the short causal convolution of the q / k / v columns with SiLU, its last inputs kept per
                             sequence (ring kept twice, read one copy and write the other)
  pgk_seq_delta_prep         q and k heads to unit length, q times dim^-1/2; beta and g from their projections
  pgk_seq_gated_recurrence   the walk (delta form)
  pgk_seq_linear_finish      root mean square per head, the shared weight vector, silu of the gate columns

and the output projection.  Every size comes from the spec.
"""
from __future__ import annotations

from ..._lib import api
from ...core.array import GPUArray
from ...core.stream import current_stream_handle as _st
from ..config import DeltaMixerSpec, GatedLinearMixerSpec
from .linear import LinearRows


class GatedLinearMixer:
    queries_per_tile = None              # no attention tiles

    def __init__(self, spec: GatedLinearMixerSpec, layer: int, proj: "LinearRows | None", o_proj: "LinearRows | None",
                 f_bias: GPUArray, lower: GPUArray, norm_weight: GPUArray, eps: float, out_mult: float = 1.0):
        """norm_weight: [heads x vdim], the shared vector repeated per head; proj / o_proj None: one side of a wider mixer
        that owns the products."""
        s = spec
        self.spec, self.layer, self.proj, self.o_proj = spec, layer, proj, o_proj
        self.f_bias, self.lower, self.norm_weight = f_bias, lower, norm_weight
        self.eps, self.out_mult = float(eps), float(out_mult)
        self.q_cols = s.heads * s.dim
        self.v_cols = s.heads * s.vdim
        self.proj_cols = s.proj_cols
        if f_bias.size != self.q_cols or lower.size != self.q_cols or norm_weight.size != self.v_cols:
            raise ValueError(f"layer {layer}: gate bias, lower bound or output norm weight do not match {s}")
        if proj is not None and proj.out_features != self.proj_cols:
            raise ValueError(f"layer {layer}: fused projection has {proj.out_features} rows, the mixer needs {self.proj_cols}")

    @property
    def weight_bytes(self) -> int:
        return (self.proj.nbytes if self.proj is not None else 0) + (self.o_proj.nbytes if self.o_proj is not None else 0)

    def key_slices(self, ctx) -> int:
        return 1

    def forward(self, ctx, x: GPUArray, out: GPUArray, cache_index: int | None = None, out_scale: int | None = None,
                state=None) -> None:
        T, W = ctx.T, self.proj.in_features
        proj, attn = ctx.buf.proj, ctx.buf.attn
        self.proj.forward(x.device_ptr, W, T, proj.device_ptr, self.proj_cols)
        self.attend(ctx, proj.device_ptr, self.proj_cols, attn.device_ptr, self.v_cols, state)
        if out_scale is None:
            self.o_proj.forward(attn.device_ptr, self.v_cols, T, out.device_ptr, self.o_proj.out_features)
        else:
            self.o_proj.forward_seq(attn.device_ptr, self.v_cols, T, out.device_ptr, self.o_proj.out_features, epilogue=4,
                                    col_scale=out_scale)

    def attend(self, ctx, proj_ptr: int, ld: int, attn_ptr: int, ldo: int, state) -> None:
        s, T = self.spec, ctx.T
        if not state:
            raise ValueError(f"layer {self.layer}: the gated linear mixer needs its state array")
        f_off, v_off = self.q_cols, 2 * self.q_cols
        api.seq_gated_prep(proj_ptr, ld, T, s.heads, s.dim, 0, f_off, self.f_bias.device_ptr, self.lower.device_ptr, _st())
        seqs_ptr, n_seqs = ctx.seqs()
        api.seq_gated_recurrence(0, proj_ptr, ld, 0, None, 0, 0, proj_ptr, ld, f_off, None, 0, 0, proj_ptr, ld, v_off, attn_ptr, ldo,
                                 state[0].device_ptr, seqs_ptr, n_seqs, s.heads, s.heads, s.dim, s.vdim, _st())
        api.seq_linear_finish(attn_ptr, ldo, None, 0, 0, self.norm_weight.device_ptr, T, s.heads, s.vdim, 1, 0, self.eps,
                              self.out_mult, _st())


class DeltaRuleMixer:
    queries_per_tile = None

    def __init__(self, spec: DeltaMixerSpec, layer: int, proj: LinearRows, o_proj: LinearRows, conv_weight: GPUArray,
                 A_log: GPUArray, dt_bias: GPUArray, norm_weight: GPUArray, eps: float):
        """conv_weight: [q | k | v channels, taps]; norm_weight: [heads x vdim], the shared vector repeated per head."""
        s = spec
        self.spec, self.layer, self.proj, self.o_proj = spec, layer, proj, o_proj
        self.conv_weight, self.A_log, self.dt_bias, self.norm_weight, self.eps = conv_weight, A_log, dt_bias, norm_weight, float(eps)
        self.qk_cols, self.v_cols = s.qk_heads * s.dim, s.heads * s.vdim
        self.proj_cols = s.proj_cols
        if proj.out_features != self.proj_cols or o_proj.in_features != self.v_cols:
            raise ValueError(f"layer {layer}: the products do not match {s}")
        if tuple(conv_weight.shape) != (s.conv_cols, s.conv_taps):
            raise ValueError(f"layer {layer}: convolution weights {tuple(conv_weight.shape)}, not {(s.conv_cols, s.conv_taps)}")
        if A_log.size != s.heads or dt_bias.size != s.heads or norm_weight.size != self.v_cols:
            raise ValueError(f"layer {layer}: per-head vectors do not match {s}")

    @property
    def weight_bytes(self) -> int:
        return self.proj.nbytes + self.o_proj.nbytes + self.conv_weight.nbytes

    def key_slices(self, ctx) -> int:
        return 1

    def forward(self, ctx, x: GPUArray, out: GPUArray, cache_index: int | None = None, out_scale: int | None = None,
                state=None) -> None:
        s, T = self.spec, ctx.T
        if not state or len(state) < 2:
            raise ValueError(f"layer {self.layer}: the delta-rule mixer needs its state and its convolution ring")
        W = self.proj.in_features
        proj, conv, attn = ctx.buf.proj, ctx.buf.conv, ctx.buf.attn
        ld, lc, ldo = self.proj_cols, s.conv_cols, self.v_cols
        self.proj.forward(x.device_ptr, W, T, proj.device_ptr, ld)
        api.causal_conv_rows_ex_f32(proj.device_ptr, ld, conv.device_ptr, lc, self.conv_weight.device_ptr,
                                    state[1].device_ptr if s.conv_taps > 1 else None, ctx.slot_ptr, ctx.pos_ptr, ctx.parity_ptr,
                                    T, lc, s.conv_taps, 0, 1, _st())
        g_off = lc                                   # gate columns, then beta, then a
        b_off, a_off = g_off + self.v_cols, g_off + self.v_cols + s.heads
        api.seq_delta_prep(conv.device_ptr, lc, 0, self.qk_cols, proj.device_ptr, ld, b_off, a_off, self.A_log.device_ptr,
                           self.dt_bias.device_ptr, T, s.heads, s.qk_heads, s.dim, float(s.dim) ** -0.5, _st())
        seqs_ptr, n_seqs = ctx.seqs()
        api.seq_gated_recurrence(1, conv.device_ptr, lc, 0, conv.device_ptr, lc, self.qk_cols, proj.device_ptr, ld, a_off,
                                 proj.device_ptr, ld, b_off, conv.device_ptr, lc, 2 * self.qk_cols, attn.device_ptr, ldo,
                                 state[0].device_ptr, seqs_ptr, n_seqs, s.heads, s.qk_heads, s.dim, s.vdim, _st())
        api.seq_linear_finish(attn.device_ptr, ldo, proj.device_ptr, ld, g_off, self.norm_weight.device_ptr, T, s.heads, s.vdim,
                              1, 2, self.eps, 1.0, _st())
        if out_scale is None:
            self.o_proj.forward(attn.device_ptr, ldo, T, out.device_ptr, self.o_proj.out_features)
        else:
            self.o_proj.forward_seq(attn.device_ptr, ldo, T, out.device_ptr, self.o_proj.out_features, epilogue=4,
                                    col_scale=out_scale)


__all__ = ["GatedLinearMixer", "DeltaRuleMixer"]
