"""Mixers with a recurrent state per sequence in the token-major models (net-new; beside `PagedAttentionMixer` and
`LatentAttentionMixer`, which keep cache pages).

`LinearAttentionMixer`: linear attention with a fixed decay per head, S_t = a_h S_(t-1) + k_t v_t^T, o_t = S_t^T q_t, the
state S [heads, dim, vdim] in float32 in a per-slot array of the cache manager (`PagedKVCache.state`).  One fused projection
[q | k | v | gate], then three launches

  pgk_seq_linear_prep        activation of q / k / v, rotary positions on q and k, the key scale
  pgk_seq_linear_attention   the recurrence over the step's tokens, chunk by chunk, state read and written once
                             (steps with long portions: pgk_seq_linear_attention_chunks, all chunks at once in three passes)
  pgk_seq_linear_finish      output norm (all heads together with a weight, or head by head without), gate, constant factor

and the output projection.  Every constant comes from the `LinearMixerSpec`.  `attend` is the mixer without its two matrix
products, on a block of columns of a wider projection.

`ParallelMixer`: an attention mixer and a linear-attention mixer side by side on the same input,
left_scale * left + right_scale * right.  Both sides' projections are ONE product, both sides' output projections are ONE
product over the concatenated head outputs (the two factors ride on the head outputs, where the kernels multiply anyway).
"""
from __future__ import annotations

import numpy as np

from ..._lib import api
from ...core.array import GPUArray
from ...core.factory import from_numpy
from ...core.stream import current_stream_handle as _st
from ..config import LinearMixerSpec, ParallelMixerSpec
from .linear import LinearRows
from .paged_attention import PagedAttentionMixer


class LinearAttentionMixer:
    queries_per_tile = None              # no attention tiles
    SEQUENTIAL_CHUNKS = 2                # steps whose longest portion has more chunks take the three-pass form
    WORKSPACE_FLOATS = 1 << 26           # 256 MB of chunk states at most per segment

    def __init__(self, spec: LinearMixerSpec, layer: int, qkvg: "LinearRows | None", o_proj: "LinearRows | None",
                 norm_weight: "GPUArray | None", eps: float, out_mult: float = 1.0):
        s = spec
        if s.activation not in ("none", "silu") or s.out_norm not in ("all", "head") or s.gate not in ("none", "sigmoid", "silu"):
            raise ValueError(f"layer {layer}: unknown activation / output norm / gate in {s}")
        if len(s.decay) != s.heads:
            raise ValueError(f"layer {layer}: {len(s.decay)} decays for {s.heads} heads")
        self.spec, self.layer, self.qkvg, self.o_proj = spec, layer, qkvg, o_proj
        self.norm_weight, self.eps, self.out_mult = norm_weight, float(eps), float(out_mult)
        self.q_cols = self.k_cols = s.heads * s.dim
        self.v_cols = s.heads * s.vdim
        self.proj_cols = s.proj_cols if s.gate != "none" else self.q_cols + self.k_cols + self.v_cols
        if qkvg is not None and qkvg.out_features != self.proj_cols:
            raise ValueError(f"layer {layer}: fused projection has {qkvg.out_features} rows, the mixer needs {self.proj_cols}")
        if norm_weight is not None and norm_weight.size != self.v_cols:
            raise ValueError(f"layer {layer}: the output norm's weight has {norm_weight.size} elements, not {self.v_cols}")
        self.decay = from_numpy(np.asarray(s.decay, np.float32))
        self.chunk_tokens = int(api.seq_linear_chunk_tokens())
        self.inv_freq = from_numpy(np.asarray(s.rot.inv_freq(), np.float64)) if s.rot is not None else None

    @property
    def weight_bytes(self) -> int:
        return (self.qkvg.nbytes if self.qkvg is not None else 0) + (self.o_proj.nbytes if self.o_proj is not None else 0)

    def key_slices(self, ctx) -> int:
        return 1

    def forward(self, ctx, x: GPUArray, out: GPUArray, cache_index: int | None = None, out_scale: int | None = None,
                state=None) -> None:
        """x [T, W] -> out; with out_scale (device pointer of [W] floats) out += out_scale * result.  state: this mixer's
        per-slot arrays in the cache manager ([S])."""
        s, T = self.spec, ctx.T
        W = self.qkvg.in_features
        proj, attn = ctx.buf.proj, ctx.buf.attn
        ld, ldo = self.proj_cols, self.v_cols
        self.qkvg.forward(x.device_ptr, W, T, proj.device_ptr, ld)
        self.attend(ctx, proj.device_ptr, ld, attn.device_ptr, ldo, state)
        if out_scale is None:
            self.o_proj.forward(attn.device_ptr, ldo, T, out.device_ptr, self.o_proj.out_features)
        else:
            self.o_proj.forward_seq(attn.device_ptr, ldo, T, out.device_ptr, self.o_proj.out_features, epilogue=4,
                                    col_scale=out_scale)

    def attend(self, ctx, proj_ptr: int, ld: int, attn_ptr: int, ldo: int, state) -> None:
        s, T = self.spec, ctx.T
        if not state:
            raise ValueError(f"layer {self.layer}: the linear-attention mixer needs its state array")
        k_off, v_off = self.q_cols, self.q_cols + self.k_cols
        api.seq_linear_prep(proj_ptr, ld, T, s.heads, s.dim, s.vdim, 0, k_off, v_off, 1 if s.activation == "silu" else 0,
                            s.rot.dims if s.rot is not None else 0,
                            self.inv_freq.device_ptr if self.inv_freq is not None else None, float(s.k_scale), ctx.pos_ptr, _st())
        seqs_ptr, n_seqs = ctx.seqs()
        chunk = self.chunk_tokens
        n_chunks = -(-ctx.max_rows // chunk)
        if n_chunks > self.SEQUENTIAL_CHUNKS:
            # long prompts: every chunk at once (three launches), in segments that bound the workspace
            per = n_seqs * s.heads * s.dim * s.vdim
            seg = max(1, min(n_chunks, self.WORKSPACE_FLOATS // per))
            ws = ctx.workspace(seg * per).device_ptr
            for c0 in range(0, n_chunks, seg):
                api.seq_linear_attention_chunks(proj_ptr, ld, 0, k_off, v_off, attn_ptr, ldo, state[0].device_ptr,
                                                self.decay.device_ptr, seqs_ptr, n_seqs, s.heads, s.dim, s.vdim, c0,
                                                min(seg, n_chunks - c0), ws, _st())
        else:
            ds = int(api.seq_linear_value_slice(s.heads, s.dim, s.vdim, n_seqs))
            api.seq_linear_attention(proj_ptr, ld, 0, k_off, v_off, attn_ptr, ldo, state[0].device_ptr, self.decay.device_ptr,
                                     seqs_ptr, n_seqs, s.heads, s.dim, s.vdim, ds, _st())
        gate_act = {"none": 0, "sigmoid": 1, "silu": 2}[s.gate]
        api.seq_linear_finish(attn_ptr, ldo, proj_ptr if gate_act else None, ld, v_off + self.v_cols,
                              self.norm_weight.device_ptr if self.norm_weight is not None else None, T, s.heads, s.vdim,
                              1 if s.out_norm == "head" else 0, gate_act, self.eps, self.out_mult, _st())


class ParallelMixer:
    def __init__(self, spec: ParallelMixerSpec, layer: int, proj: LinearRows, o_proj: "LinearRows | None", left: PagedAttentionMixer,
                 right, o_left: "LinearRows | None" = None, o_right: "LinearRows | None" = None,
                 out_weights: "tuple[GPUArray, GPUArray] | None" = None, eps: float = 1e-6):
        """proj: rows [left q | k | v | right's columns]; join "sum": o_proj with columns [left heads | right heads], left /
        right carry the two factors as their `out_mult`; join "rms_mean": o_left and o_right, one output projection per side,
        and out_weights, the weight vectors of the RMS norm over the width that each side's result passes.  `right` is any
        mixer with a state and an `attend` on a block of columns."""
        self.spec, self.layer, self.proj, self.o_proj, self.left, self.right = spec, layer, proj, o_proj, left, right
        self.o_left, self.o_right, self.out_weights, self.eps = o_left, o_right, out_weights, float(eps)
        self.proj_cols = left.proj_cols + right.proj_cols
        self.attn_cols = spec.attn_cols
        if spec.join not in ("sum", "rms_mean"):
            raise ValueError(f"layer {layer}: unknown join {spec.join!r}")
        if proj.out_features != self.proj_cols:
            raise ValueError(f"layer {layer}: the fused projection does not match the two mixers")
        if spec.join == "sum" and (o_proj is None or o_proj.in_features != self.attn_cols):
            raise ValueError(f"layer {layer}: the fused output projection does not match the two mixers")
        if spec.join == "rms_mean":
            if o_left is None or o_right is None or out_weights is None:
                raise ValueError(f"layer {layer}: the RMS-normed join needs both output projections and both weight vectors")
            if o_left.in_features != spec.left.attn_cols or o_right.in_features != spec.right.attn_cols:
                raise ValueError(f"layer {layer}: the output projections do not match the two mixers")
            if spec.left_scale != spec.right_scale:
                raise ValueError(f"layer {layer}: the RMS-normed join weighs both sides alike")
        self.queries_per_tile = left.queries_per_tile

    @property
    def weight_bytes(self) -> int:
        return self.proj.nbytes + sum(o.nbytes for o in (self.o_proj, self.o_left, self.o_right) if o is not None)

    def key_slices(self, ctx) -> int:
        return self.left.key_slices(ctx)

    def forward_pending(self, ctx, x: GPUArray, out: GPUArray, cache_index: int | None = None, state=None) -> dict:
        """`forward` without its last launch, for a block that folds the join into its own seam launch: the description of
        what is still to be done ("pair": the two sides' projected rows and the weights of their RMS norms; "rows": nothing)."""
        if self.spec.join != "rms_mean":
            self.forward(ctx, x, out, cache_index, state=state)
            return {"mode": "rows", "y": out.device_ptr}
        T = ctx.T
        attn, y2 = ctx.buf.attn, ctx.buf.y2
        ldo, la, Wo = self.attn_cols, self.spec.left.attn_cols, self.o_left.out_features
        self._attend(ctx, x, cache_index, state)
        self.o_left.forward(attn.device_ptr, ldo, T, out.device_ptr, Wo)
        self.o_right.forward(attn.device_ptr + 4 * la, ldo, T, y2.device_ptr, Wo)
        return {"mode": "pair", "y": out.device_ptr, "y2": y2.device_ptr, "wa": self.out_weights[0].device_ptr,
                "wb": self.out_weights[1].device_ptr, "mult": self.spec.left_scale, "eps": self.eps}

    def _attend(self, ctx, x: GPUArray, cache_index, state) -> None:
        T, W = ctx.T, self.proj.in_features
        proj, attn = ctx.buf.proj, ctx.buf.attn
        ld, ldo = self.proj_cols, self.attn_cols
        self.proj.forward(x.device_ptr, W, T, proj.device_ptr, ld)
        self.left.attend(ctx, proj.device_ptr, ld, attn.device_ptr, ldo, cache_index)
        self.right.attend(ctx, proj.device_ptr + 4 * self.left.proj_cols, ld, attn.device_ptr + 4 * self.spec.left.attn_cols,
                          ldo, state)

    def forward(self, ctx, x: GPUArray, out: GPUArray, cache_index: int | None = None, out_scale: int | None = None,
                state=None) -> None:
        T = ctx.T
        attn, ldo = ctx.buf.attn, self.attn_cols
        if self.spec.join == "rms_mean":
            if out_scale is not None:
                raise ValueError(f"layer {self.layer}: the RMS-normed join stores its result")
            p = self.forward_pending(ctx, x, out, cache_index, state)
            api.rms_pair_rows_f32(p["y"], p["wa"], p["y2"], p["wb"], p["eps"], p["mult"], out.device_ptr, T,
                                  self.o_left.out_features, _st())
            return
        self._attend(ctx, x, cache_index, state)
        if out_scale is None:
            self.o_proj.forward(attn.device_ptr, ldo, T, out.device_ptr, self.o_proj.out_features)
        else:
            self.o_proj.forward_seq(attn.device_ptr, ldo, T, out.device_ptr, self.o_proj.out_features, epilogue=4,
                                    col_scale=out_scale)


__all__ = ["LinearAttentionMixer", "ParallelMixer"]
