"""Transformer block (mirror of pygpukit/llm/layers/block.py:18-62): Norm -> Attention -> residual,
Norm -> MLP/MoE -> residual.  Residual adds ride in the o_proj / down_proj GEMV epilogues with the
fixed-cache path's rounding (bf16 + bf16 -> one rounding, elementwise_kernels.cuh:381-390).  Under
tensor parallelism the row-parallel partial sums are all-reduced BEFORE the residual is added."""
from __future__ import annotations

from ...core.array import GPUArray
from .attention import Attention
from .linear import can_fuse_norm
from .mlp import MLP
from .moe import MoELayer
from .norm import Norm


class TransformerBlock:
    def __init__(self, attn_norm: Norm, attn: Attention, mlp_norm: Norm, mlp: "MLP | MoELayer", comm=None):
        self.attn_norm = attn_norm
        self.attn = attn
        self.mlp_norm = mlp_norm
        self.mlp = mlp
        self.comm = comm   # TensorParallel communicator or None

    def decode(self, hidden: GPUArray, position: int, context_len: int, bufs=None, pos_buf=None, ctx_buf=None,
               multi: bool = False) -> GPUArray:
        """hidden [M, H] -> hidden [M, H], updated IN PLACE (M consecutive tokens of one sequence; multi = True: the
        new tokens of M independent sequences, pos_buf / ctx_buf are then arrays of M)."""
        M = hidden.shape[0]

        def buf(name):
            b = getattr(bufs, name, None) if bufs is not None else None
            return b if (b is None or b.shape[0] == M) else b.slice_rows(M)

        tp = self.comm is not None and self.comm.world > 1
        # pre-norms ride inside the qkv / gate-up GEMV launches when the formats allow it
        if multi:
            fuse = can_fuse_norm(self.attn_norm, hidden.shape[1])
            x = hidden if fuse else self.attn_norm(hidden, out=buf("norm_out"))
            a = self.attn.attend_multi(x, pos_buf, ctx_buf, qkv_buf=buf("qkv_proj_out"), attn_buf=buf("attn_flat"),
                                       norm=self.attn_norm if fuse else None)
        elif can_fuse_norm(self.attn_norm, hidden.shape[1]):
            a = self.attn.attend(hidden, position, context_len, qkv_buf=buf("qkv_proj_out"), attn_buf=buf("attn_flat"),
                                 pos_buf=pos_buf, ctx_buf=ctx_buf, norm=self.attn_norm)
        else:
            x = self.attn_norm(hidden, out=buf("norm_out"))
            a = self.attn.attend(x, position, context_len, qkv_buf=buf("qkv_proj_out"), attn_buf=buf("attn_flat"),
                                 pos_buf=pos_buf, ctx_buf=ctx_buf)
        if tp and self.comm.fuses_allreduce(self.attn.o_proj, M):
            self.attn.o_proj.forward_allreduce(a, hidden)          # GEMV + all-reduce + residual: one launch
        elif tp:
            part = self.attn.o_proj.forward(a, out=buf("partial"))
            self.comm.allreduce_add(part, hidden)
        else:
            self.attn.o_proj.forward(a, out=hidden, residual=hidden)
        fuse_mlp = isinstance(self.mlp, MLP) and self.mlp.fuses_norm(self.mlp_norm)
        x, nrm = (hidden, self.mlp_norm) if fuse_mlp else (self.mlp_norm(hidden, out=buf("norm_out")), None)
        kw = {"norm": nrm} if fuse_mlp else {}
        if tp and isinstance(self.mlp, MoELayer):
            # expert parallel: the exchange happens inside the layer, on the un-combined rows (bit-identical to 1 GPU)
            self.mlp.forward(x, out=hidden, residual=hidden, act_buf=buf("mlp_act"), comm=self.comm)
        elif tp and isinstance(self.mlp, MLP) and self.mlp.activation != "gelu" and self.comm.fuses_allreduce(self.mlp.down_proj, M):
            self.mlp.forward_allreduce(x, hidden, act_buf=buf("mlp_act"), **kw)
        elif tp:
            part = self.mlp.forward(x, out=buf("partial"), act_buf=buf("mlp_act"), **kw)
            self.comm.allreduce_add(part, hidden)
        else:
            self.mlp.forward(x, out=hidden, residual=hidden, act_buf=buf("mlp_act"), **kw)
        return hidden

    def __call__(self, x: GPUArray, position_ids: list[int] | None = None, past_kv=None, use_cache: bool = False):
        start = position_ids[0] if position_ids else (past_kv or 0)
        h = x.clone()
        self.decode(h, start, start + x.shape[0])
        return h, (start + x.shape[0] if use_cache else None)

    @property
    def weight_bytes(self) -> int:
        return (self.attn.weight_bytes + self.mlp.weight_bytes + self.attn_norm.weight.nbytes
                + self.mlp_norm.weight.nbytes)


class PostNormBlock:
    """Block of the token-major models with the norm on the sublayer's OUTPUT: x += LN1(mixer(x)), then
    x += LN2(ff(x)); both sublayers read the float32 residual stream itself.  Each "norm + add" is one launch that
    also folds the feed-forward's weighted expert sum and shared expert (pgk_combine_layernorm_f32)."""

    def __init__(self, mixer, norm1: tuple[GPUArray, GPUArray], mlp, norm2: "tuple[GPUArray, GPUArray] | None", eps: float):
        self.mixer, self.mlp = mixer, mlp
        self.norm1, self.norm2, self.eps = norm1, norm2, float(eps)

    norm = None                          # no norm in front of the block: nothing for the block before to fuse with

    def forward(self, ctx, x: GPUArray, cache_index: int | None = None, add_ptr: int | None = None, normed: bool = False,
                next_norm=None, next_add_ptr: int | None = None) -> bool:
        from ..._lib import api
        from ...core.stream import current_stream_handle as _st
        if add_ptr is not None:
            raise ValueError("PostNormBlock: no loop passes in this block form")
        T, W = ctx.T, x.shape[1]
        y = ctx.buf.y
        self.mixer.forward(ctx, x, y, cache_index)
        api.combine_layernorm_f32(y.device_ptr, None, None, None, None, 0, self.norm1[0].device_ptr,
                                  self.norm1[1].device_ptr, self.eps, x.device_ptr, T, W, 1, _st())
        if self.mlp is not None:
            base, parts, inv, wts, top = self.mlp.forward(ctx, x, y)
            api.combine_layernorm_f32(base, None, parts, inv, wts, top, self.norm2[0].device_ptr,
                                      self.norm2[1].device_ptr, self.eps, x.device_ptr, T, W, 1, _st())
        return False

    @property
    def weight_bytes(self) -> int:
        n = self.mixer.weight_bytes + 2 * self.norm1[0].nbytes
        if self.mlp is not None:
            n += self.mlp.weight_bytes + 2 * self.norm2[0].nbytes
        return n


class ParallelBlock:
    """Block of the token-major models with ONE norm in front of both sublayers: h = norm(x), then
    x += s1 * mixer(h) + s2 * ff(h) with per-channel factors s1, s2 (layer scales; ones without them), then the optional
    per-layer token input.  The two scaled adds ride in the epilogues of the output projection and of the down projection
    (C += s * product), so the block adds no launch of its own beyond the norm.  `add_ptr`: rows added to x before the norm
    and written back (the embedding output at the start of a loop pass) -- same launch.  When the block ends with a token
    input and another parallel block follows, that block's norm (and its add) ride in the token input's last launch."""

    def __init__(self, norm, mixer, mixer_scale: GPUArray, mlp, mlp_scale: "GPUArray | None", side=None):
        self.norm, self.mixer, self.mlp, self.side = norm, mixer, mlp, side
        self.mixer_scale, self.mlp_scale = mixer_scale, mlp_scale
        if mlp is not None and mlp_scale is None:
            raise ValueError("ParallelBlock: the feed-forward needs its scale vector")

    def forward(self, ctx, x: GPUArray, cache_index: int | None = None, add_ptr: int | None = None, normed: bool = False,
                next_norm=None, next_add_ptr: int | None = None) -> bool:
        """normed: ctx.buf.h already holds norm(x) (the block before wrote it, with `add_ptr` applied).  next_norm /
        next_add_ptr: the norm (and the rows to add first) of the block that runs next; returns True when this block
        has written that block's normed rows (only the token input's last launch can)."""
        T, W = ctx.T, x.shape[1]
        h = ctx.buf.h
        if not normed:
            self.norm.forward(x.device_ptr, h.device_ptr, T, W, add_ptr=add_ptr,
                              sum_out_ptr=x.device_ptr if add_ptr is not None else None)
        self.mixer.forward(ctx, h, x, cache_index, out_scale=self.mixer_scale.device_ptr)
        if self.mlp is not None:
            self.mlp.forward(ctx, h.device_ptr, x.device_ptr, out_scale=self.mlp_scale.device_ptr)
        if self.side is not None:
            return self.side.forward(ctx, x, next_norm, next_add_ptr)
        return False

    @property
    def weight_bytes(self) -> int:
        n = self.mixer.weight_bytes + self.norm.nbytes + self.mixer_scale.nbytes
        if self.mlp is not None:
            n += self.mlp.weight_bytes + self.mlp_scale.nbytes
        if self.side is not None:
            n += self.side.weight_bytes
        return n


class PreNormBlock:
    """Block of the token-major models with a norm in front of EACH sublayer: x += m * mixer(c1(norm1(x))), then
    x += m * ff(c2(norm2(x))); c1 / c2 are optional short causal convolutions over time on the normed rows
    (`CausalConvRows`), m one factor for both sublayers.  The two scaled adds ride in the epilogues of the output projection
    and of the down projection (C += m * product).  Per-sequence state of the block, in this order in the cache manager:
    the rings of c1 and c2, then whatever the mixer keeps."""

    def __init__(self, norm1, conv1, mixer, norm2, conv2, mlp, mult: GPUArray):
        """mult: [width] floats, every element the residual factor m (the epilogue takes a factor per column)."""
        self.norm1, self.conv1, self.mixer, self.norm2, self.conv2, self.mlp, self.mult = norm1, conv1, mixer, norm2, conv2, mlp, mult
        if mlp is None and (norm2 is not None or conv2 is not None):
            raise ValueError("PreNormBlock: a second norm or convolution without a feed-forward")
        self._convs = [c for c in (conv1, conv2) if c is not None and c.taps > 1]

    norm = None                          # the block's norms are not fused with the block before

    @property
    def state_shapes(self) -> tuple:
        return tuple(c.state_size for c in self._convs) + tuple(self.mixer.spec.state_shapes)

    def forward(self, ctx, x: GPUArray, cache_index: int | None = None, add_ptr: int | None = None, normed: bool = False,
                next_norm=None, next_add_ptr: int | None = None) -> bool:
        if add_ptr is not None:
            raise ValueError("PreNormBlock: no loop passes in this block form")
        T, W = ctx.T, x.shape[1]
        h, u = ctx.buf.h, ctx.buf.y
        state = list(ctx.cache.state[cache_index]) if cache_index is not None else []
        rings = {id(c): state.pop(0) for c in self._convs}
        src = self._normed(ctx, self.norm1, self.conv1, rings, x, h, u)
        self.mixer.forward(ctx, src, x, cache_index, out_scale=self.mult.device_ptr, state=state)
        if self.mlp is not None:
            src = self._normed(ctx, self.norm2, self.conv2, rings, x, h, u)
            self.mlp.forward(ctx, src.device_ptr, x.device_ptr, out_scale=self.mult.device_ptr)
        return False

    @staticmethod
    def _normed(ctx, norm, conv, rings, x: GPUArray, h: GPUArray, u: GPUArray) -> GPUArray:
        """the sublayer's input: norm(x), or conv(norm(x))"""
        T, W = ctx.T, x.shape[1]
        norm.forward(x.device_ptr, h.device_ptr, T, W)
        if conv is None:
            return h
        conv.forward(ctx, h.device_ptr, u.device_ptr, rings.get(id(conv)))
        return u

    @property
    def weight_bytes(self) -> int:
        n = self.mixer.weight_bytes + self.norm1.nbytes + (self.conv1.nbytes if self.conv1 is not None else 0)
        if self.mlp is not None:
            n += self.mlp.weight_bytes + self.norm2.nbytes + (self.conv2.nbytes if self.conv2 is not None else 0)
        return n


class SandwichBlock:
    """Block of the token-major models with a norm before AND after each sublayer: x += norm1b(mixer(norm1(x))), then
    x += norm2b(ff(norm2(x))).  The norms are `RowNorm`s of any kind.  With dynamic-tanh norms the seam behind a sublayer is
    ONE launch (pgk_dyt_seam_f32): the sublayer's last step -- the join of a parallel mixer's two RMS-normed sides, or the
    weighted sum of the chosen experts with the gated shared expert -- the norm behind it, the residual add, and the norm in
    front of the next sublayer (the feed-forward's, or the next block's first one).  Other norms take a launch each.  The
    feed-forward is any layer with `forward_rows(ctx, rows, out)`.  Per-sequence state of the block in the cache manager:
    whatever the mixer keeps."""

    def __init__(self, norm1, mixer, norm1b, norm2=None, mlp=None, norm2b=None):
        self.norm1, self.mixer, self.norm1b, self.norm2, self.mlp, self.norm2b = norm1, mixer, norm1b, norm2, mlp, norm2b
        if (mlp is None) != (norm2 is None) or (mlp is None) != (norm2b is None):
            raise ValueError("SandwichBlock: a feed-forward comes with both of its norms")

    @property
    def norm(self):
        """the norm in front of the block: the block before may write its rows (dynamic-tanh norms only)"""
        return self.norm1 if self.norm1.kind == "dyt" else None

    @property
    def state_shapes(self) -> tuple:
        return tuple(self.mixer.spec.state_shapes)

    def forward(self, ctx, x: GPUArray, cache_index: int | None = None, add_ptr: int | None = None, normed: bool = False,
                next_norm=None, next_add_ptr: int | None = None) -> bool:
        """normed: ctx.buf.h already holds norm1(x) (the block before wrote it).  next_norm: the first norm of the block that
        runs next; returns True when this block has written that block's normed rows."""
        if add_ptr is not None:
            raise ValueError("SandwichBlock: no loop passes in this block form")
        T, W = ctx.T, x.shape[1]
        h, y = ctx.buf.h, ctx.buf.y
        state = list(ctx.cache.state[cache_index]) if cache_index is not None else []
        if next_add_ptr is not None:
            next_norm = None
        if not normed:
            self.norm1.forward(x.device_ptr, h.device_ptr, T, W)
        if hasattr(self.mixer, "forward_pending"):
            pend = self.mixer.forward_pending(ctx, h, y, cache_index, state=state)
        else:
            self.mixer.forward(ctx, h, y, cache_index, state=state)
            pend = {"mode": "rows", "y": y.device_ptr}
        wrote = self._seam(ctx, pend, self.norm1b, x, self.norm2 if self.mlp is not None else next_norm)
        if self.mlp is None:
            return wrote
        if not wrote:
            self.norm2.forward(x.device_ptr, h.device_ptr, T, W)
        if hasattr(self.mlp, "forward_pending"):
            pend = self.mlp.forward_pending(ctx, h, y)
        else:
            self.mlp.forward_rows(ctx, h, y)
            pend = {"mode": "rows", "y": y.device_ptr}
        return self._seam(ctx, pend, self.norm2b, x, next_norm)

    @staticmethod
    def _seam(ctx, p: dict, post, x: GPUArray, nxt) -> bool:
        """x += post(the pending result); h = nxt(x) when the launch can take it along (returns whether it did)."""
        from ..._lib import api
        from ...core.stream import current_stream_handle as _st
        T, W = ctx.T, x.shape[1]
        h, y = ctx.buf.h, ctx.buf.y
        if post.kind != "dyt":                       # finish the pending step into y, then the norm's own launch
            if p["mode"] == "pair":
                api.rms_pair_rows_f32(p["y"], p["wa"], p["y2"], p["wb"], p["eps"], p["mult"], y.device_ptr, T, W, _st())
            elif p["mode"] == "experts":
                api.moe_combine_rows_f32(p["parts"], p["inv"], p["mat"], p["w"], p["top"], p["self_rows"], p["shared"], p["gate"],
                                         p["ldg"], p["gate_off"], y.device_ptr, T, W, _st())
            post.forward(y.device_ptr if p["mode"] != "rows" else p["y"], x.device_ptr, T, W, accumulate=True)
            return False
        take = nxt is not None and nxt.kind == "dyt"
        mode = {"rows": 0, "pair": 1, "experts": 2}[p["mode"]]
        api.dyt_seam_f32(mode, p.get("y"), p.get("y2"), p.get("wa"), p.get("wb"), p.get("mult", 1.0), p.get("eps", 0.0),
                         p.get("parts"), p.get("inv"), p.get("mat"), p.get("w"), p.get("top", 0), p.get("self_rows"), p.get("shared"),
                         p.get("gate"), p.get("ldg", 0), p.get("gate_off", 0), post.alpha, post.weight.device_ptr,
                         post.bias.device_ptr if post.bias is not None else None, x.device_ptr,
                         nxt.alpha if take else 1.0, nxt.weight.device_ptr if take else None,
                         nxt.bias.device_ptr if take and nxt.bias is not None else None, h.device_ptr if take else None, T, W, _st())
        return take

    @property
    def weight_bytes(self) -> int:
        n = self.mixer.weight_bytes + self.norm1.nbytes + self.norm1b.nbytes
        if self.mlp is not None:
            n += self.mlp.weight_bytes + self.norm2.nbytes + self.norm2b.nbytes
        return n


__all__ = ["TransformerBlock", "PostNormBlock", "ParallelBlock", "PreNormBlock", "SandwichBlock"]
