"""Mixture of experts of the token-major models (net-new; beside `MoELayer`, whose router is top-k then softmax over
the chosen logits and whose experts are FP8 / NVF4 GEMVs on bfloat16 rows).

Router: float32 logits from the router GEMM (the router matrix is kept in float32 in both modes, so the logits are
FMAs on the unrounded residual stream), then pgk_moe_route_grouped:
softmax over ALL experts, optional group limit (only members of the best
`group_keep` of `group_count` groups of neighbours), the `top` largest scores, renormalised.  Experts: stacked
[E, 2 ff, W] gate/up pairs (SiLU * up in the GEMM epilogue) and [E, W, ff] down matrices.

  many tokens   rows (token, slot) are sorted by expert on the device (pgk_moe_row_lists) and the two grouped GEMMs
                gather their input rows through the permutation -- tokens are never copied;
  <= 8 tokens   rows stay in slot order and every row streams its own expert's matrices (few-row kernel).

The weighted sum of the expert outputs, the shared expert's output, the block's LayerNorm and the residual add are
ONE launch (pgk_combine_layernorm_f32), issued by the block with what `forward` returns.
"""
from __future__ import annotations

from ..._lib import api
from ...core.array import GPUArray
from ...core.stream import current_stream_handle as _st
from ..config import MoESpec
from .linear import LinearRows


class GroupedRouterMoE:
    def __init__(self, spec: MoESpec, router: GPUArray, gate_up: LinearRows, down: LinearRows,
                 shared_gate_up: LinearRows | None = None, shared_down: LinearRows | None = None):
        self.spec, self.router = spec, LinearRows(router)
        self.gate_up, self.down = gate_up, down
        self.shared_gate_up, self.shared_down = shared_gate_up, shared_down
        if gate_up.groups != spec.experts or down.groups != spec.experts:
            raise ValueError("GroupedRouterMoE: expert stacks do not match the router")

    @property
    def weight_bytes(self) -> int:
        n = self.router.nbytes + self.gate_up.nbytes + self.down.nbytes
        if self.shared_gate_up is not None:
            n += self.shared_gate_up.nbytes + self.shared_down.nbytes
        return n

    def forward(self, ctx, x: GPUArray, shared_out: GPUArray):
        """Returns (base, parts, inv, weights, top) for the combine + norm launch: base = the shared expert's output
        rows (or None), parts [T * top, W] the routed experts' outputs, inv [T, top] their rows."""
        sp, T, b = self.spec, ctx.T, ctx.buf
        W, top, ff = self.gate_up.in_features, sp.top, sp.ff
        few = T <= LinearRows.FEW
        self.router.forward(x.device_ptr, W, T, b.moe_z.device_ptr, sp.experts)       # float32 logits [T, E]
        api.moe_route_grouped(b.moe_z.device_ptr, sp.experts, T, sp.experts, top,
                              sp.group_count, sp.group_keep, b.moe_idx.device_ptr, b.moe_w.device_ptr,
                              None if few else b.moe_rank.device_ptr, None if few else b.moe_counts.device_ptr, _st())
        if few:
            slot_tok, iota = ctx.slot_rows(top)
            self.gate_up.forward_per_row(x.device_ptr, W, T * top, b.moe_act.device_ptr, ff, slot_tok, b.moe_idx.device_ptr)
            self.down.forward_per_row(b.moe_act.device_ptr, ff, T * top, b.moe_parts.device_ptr, W, None, b.moe_idx.device_ptr)
            inv = iota
        else:
            api.moe_row_lists(b.moe_counts.device_ptr, b.moe_off.device_ptr, b.moe_idx.device_ptr, b.moe_rank.device_ptr,
                              b.moe_perm.device_ptr, b.moe_inv.device_ptr, sp.experts, T, top, _st())
            self.gate_up.forward_grouped(x.device_ptr, W, b.moe_act.device_ptr, ff, b.moe_perm.device_ptr,
                                         b.moe_off.device_ptr, T)
            self.down.forward_grouped(b.moe_act.device_ptr, ff, b.moe_parts.device_ptr, W, None, b.moe_off.device_ptr, T)
            inv = b.moe_inv.device_ptr
        base = None
        if self.shared_gate_up is not None:
            fs = self.shared_gate_up.out_cols
            self.shared_gate_up.forward(x.device_ptr, W, T, b.shared_act.device_ptr, fs)
            self.shared_down.forward(b.shared_act.device_ptr, fs, T, shared_out.device_ptr, W)
            base = shared_out.device_ptr
        return base, b.moe_parts.device_ptr, inv, b.moe_w.device_ptr, top


class BiasedRouterMoE:
    """Mixture of experts whose router adds a stored correction to the scores when it CHOOSES (the weights are the scores
    themselves, renormalised or not), whose last `identity` router outputs stand for experts that return their input, and
    whose shared expert is multiplied by sigmoid of one more projection (a number per token).  The router matrix, float32 in
    both modes, carries the shared expert's gate as its last row, so that one product gives both.  Experts and row lists as in
    `GroupedRouterMoE` (rows of experts without matrices sort behind the others and no product touches them; among few rows
    they are skipped by their matrix number -1).  `forward_rows` leaves the layer's result in `out`:

      pgk_moe_route_biased      scores, choice, weights, row lists
      pgk_moe_combine_rows_f32  weighted sum of the chosen experts' rows (or the token's own row) + gated shared expert
    """

    def __init__(self, spec: MoESpec, router: GPUArray, correction: "GPUArray | None", gate_up: "LinearRows | None",
                 down: "LinearRows | None", shared_gate_up: LinearRows | None = None, shared_down: LinearRows | None = None):
        """router: [routes (+ 1 with a gated shared expert), W] float32."""
        self.spec, self.router, self.correction = spec, LinearRows(router), correction
        self.gate_up, self.down = gate_up, down
        self.shared_gate_up, self.shared_down = shared_gate_up, shared_down
        self.z_cols = spec.routes + (1 if spec.shared_gate else 0)
        if self.router.out_features != self.z_cols:
            raise ValueError(f"BiasedRouterMoE: the router has {self.router.out_features} rows, the spec needs {self.z_cols}")
        if spec.experts > 0 and (gate_up is None or gate_up.groups != spec.experts or down.groups != spec.experts):
            raise ValueError("BiasedRouterMoE: expert stacks do not match the router")
        if bool(spec.shared_ff) != (shared_gate_up is not None) or (spec.shared_gate and not spec.shared_ff):
            raise ValueError("BiasedRouterMoE: the shared expert and the spec do not agree")

    @property
    def weight_bytes(self) -> int:
        n = self.router.nbytes
        for m in (self.gate_up, self.down, self.shared_gate_up, self.shared_down):
            if m is not None:
                n += m.nbytes
        return n

    def forward_rows(self, ctx, x: GPUArray, out: GPUArray) -> None:
        """x [T, W] (the normed rows) -> out [T, W]; out must not be x."""
        p = self.forward_pending(ctx, x)
        api.moe_combine_rows_f32(p["parts"], p["inv"], p["mat"], p["w"], p["top"], p["self_rows"], p["shared"], p["gate"], p["ldg"],
                                 p["gate_off"], out.device_ptr, ctx.T, self.router.in_features, _st())

    def forward_pending(self, ctx, x: GPUArray, out: "GPUArray | None" = None) -> dict:
        """Everything but the weighted sum, for a block that folds the sum into its own seam launch: the description of the
        rows to be summed ("experts")."""
        sp, T, b = self.spec, ctx.T, ctx.buf
        W, top, ff, R = self.router.in_features, sp.top, sp.ff, sp.routes
        few = T <= LinearRows.FEW
        self.router.forward(x.device_ptr, W, T, b.moe_z.device_ptr, self.z_cols)          # float32 logits [T, routes (+ 1)]
        api.moe_route_biased(b.moe_z.device_ptr, self.z_cols, T, R, sp.experts, top,
                             self.correction.device_ptr if self.correction is not None else None, 1 if sp.renorm else 0,
                             b.moe_idx.device_ptr, b.moe_mat.device_ptr, b.moe_w.device_ptr,
                             None if few else b.moe_rank.device_ptr, None if few else b.moe_counts.device_ptr, _st())
        if few:
            slot_tok, inv = ctx.slot_rows(top)
            if sp.experts > 0:
                self.gate_up.forward_per_row(x.device_ptr, W, T * top, b.moe_act.device_ptr, ff, slot_tok, b.moe_mat.device_ptr)
                self.down.forward_per_row(b.moe_act.device_ptr, ff, T * top, b.moe_parts.device_ptr, W, None, b.moe_mat.device_ptr)
        else:
            api.moe_row_lists(b.moe_counts.device_ptr, b.moe_off.device_ptr, b.moe_idx.device_ptr, b.moe_rank.device_ptr,
                              b.moe_perm.device_ptr, b.moe_inv.device_ptr, R, T, top, _st())
            if sp.experts > 0:
                self.gate_up.forward_grouped(x.device_ptr, W, b.moe_act.device_ptr, ff, b.moe_perm.device_ptr,
                                             b.moe_off.device_ptr, T)
                self.down.forward_grouped(b.moe_act.device_ptr, ff, b.moe_parts.device_ptr, W, None, b.moe_off.device_ptr, T)
            inv = b.moe_inv.device_ptr
        shared = None
        if self.shared_gate_up is not None:
            fs = self.shared_gate_up.out_cols
            self.shared_gate_up.forward(x.device_ptr, W, T, b.shared_act.device_ptr, fs)
            self.shared_down.forward(b.shared_act.device_ptr, fs, T, b.y2.device_ptr, W)
            shared = b.y2.device_ptr
        return {"mode": "experts", "parts": b.moe_parts.device_ptr, "inv": inv, "mat": b.moe_mat.device_ptr, "w": b.moe_w.device_ptr,
                "top": top, "self_rows": x.device_ptr, "shared": shared, "gate": b.moe_z.device_ptr if sp.shared_gate else None,
                "ldg": self.z_cols, "gate_off": R}


__all__ = ["GroupedRouterMoE", "BiasedRouterMoE"]
