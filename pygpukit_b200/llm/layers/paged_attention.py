"""Attention mixer of the token-major models on the paged cache (net-new; beside `Attention`, which serves one
sequence on a fixed cache).  One fused projection [q | k | v | gate], then two launches:

  pgk_seq_mixer_prep   RMS norm of q and k per head, value mixing, K / V rows into the cache pages
  pgk_seq_attention    scores with scale, tanh cap and per-head distance slopes, chunk mask, softmax, P.V, output gate

and the output projection.  Every constant comes from the `AttentionMixerSpec`; `v_role` says what the layer does
with its values: 0 nothing, 1 record them as the step's v_first, 2 mix them with the recorded ones.

Specs with `norm_scope == "all"` take the other preparation launch, pgk_seq_mixer_prep_all: projection biases, RMS norm of
q and of k over the whole projection, and (`values == "keys"`) the keys as projected written as the values.  A sliding
window, a sink (fixed at zero or learned per head) and a per-head gate are arguments of the attention launch.

Specs with rotary positions, with a q / k norm that has no weights, or with no q / k norm at all take the third preparation
launch, pgk_seq_mixer_prep_rot.  Kept first positions under a window, the logarithmic distance term (two learned numbers per
head) and sigmoid weights without normalisation (a learned number per head added to the score) are arguments of the
attention launch as well.  `attend` is the mixer without its two matrix products: it runs on a block of columns of a wider
fused projection, which is how a mixer that runs beside another one shares their products.
"""
from __future__ import annotations

import numpy as np

from ..._lib import api
from ...core.array import GPUArray
from ...core.factory import from_numpy
from ...core.stream import current_stream_handle as _st
from ..config import AttentionMixerSpec
from .linear import LinearRows


def key_slices(ctx, heads: int, kv_heads: int, chunk: int, window: int, queries_per_tile: int, heads_per_block: int,
               decode_heads_per_block: int, keep_first: int = 0) -> int:
    """Few long tiles (decoding over a long context): the key range of every tile is cut into this many slices so that the
    whole GPU reads the cache.  A power of two, so that a decode step's launch shapes change rarely."""
    n_tiles = ctx.tiles(queries_per_tile)[1]
    rep = heads // kv_heads
    keys = ctx.max_keys(chunk, window, keep_first)
    if ctx.decode_only:          # the decoding kernel: eight warps take 32 keys each per round
        blocks = n_tiles * kv_heads * -(-rep // decode_heads_per_block)
        want = max(1, min(64, -(-keys // 256), 592 // max(1, blocks)))
    else:
        blocks = n_tiles * kv_heads * -(-rep // heads_per_block)
        if blocks >= 148 or keys < 256:
            return 1
        want = max(1, min(64, -(-keys // 32), 592 // blocks))
    if n_tiles * kv_heads * rep > 4096:          # one arrival counter per (tile, head block)
        return 1
    return min(64, 1 << (want - 1).bit_length())


class PagedAttentionMixer:
    def __init__(self, spec: AttentionMixerSpec, layer: int, qkvg: "LinearRows | None", o_proj: "LinearRows | None",
                 q_norm: "GPUArray | None", k_norm: "GPUArray | None", eps: float, v_role: int = 0, v_lambda: float = 0.0,
                 q_bias: GPUArray | None = None, k_bias: GPUArray | None = None, sinks: GPUArray | None = None,
                 norm_offset: float = 0.0, distance: "tuple[GPUArray, GPUArray] | None" = None,
                 weight_bias: GPUArray | None = None, out_mult: float = 1.0, v_bias: GPUArray | None = None,
                 head_temp: GPUArray | None = None):
        """qkvg / o_proj None: the mixer is one side of a wider one that owns the products (only `attend` is used).
        distance: the (r1, r2) vectors of the logarithmic distance term; weight_bias: the per-head number of sigmoid weights;
        out_mult: a constant factor on the heads' outputs; q_bias / k_bias / v_bias with `qkv_bias` specs: the projections'
        biases; head_temp: the per-head factor on the score (it multiplies the query)."""
        self.spec, self.layer = spec, layer
        self.qkvg, self.o_proj = qkvg, o_proj
        self.q_norm, self.k_norm, self.eps = q_norm, k_norm, float(eps)
        self.v_role, self.v_lambda = int(v_role), float(v_lambda)
        self.q_bias, self.k_bias, self.sinks, self.norm_offset = q_bias, k_bias, sinks, float(norm_offset)
        s = spec
        if s.norm_scope not in ("head", "all") or s.values not in ("own", "keys") or s.sink not in ("none", "zero", "learned"):
            raise ValueError(f"layer {layer}: unknown norm scope / value source / sink in {s}")
        if s.values == "keys" and (s.norm_scope != "all" or s.vdim != s.dim or v_role):
            raise ValueError(f"layer {layer}: values that are the keys need the whole-projection form and vdim == dim")
        if s.norm_scope == "all" and (s.values != "keys" or not s.qk_norm):
            raise ValueError(f"layer {layer}: the whole-projection norm is built for values that are the keys")
        if (s.sink == "learned") != (sinks is not None):
            raise ValueError(f"layer {layer}: sink {s.sink!r} and the sink vector do not agree")
        if s.sink == "zero":
            self.sinks = from_numpy(np.zeros((s.heads,), np.float32))
        if s.weights not in ("softmax", "sigmoid") or (s.weights == "sigmoid" and s.sink != "none"):
            raise ValueError(f"layer {layer}: key weights {s.weights!r} with sink {s.sink!r}")
        if (s.distance_bias == "log") != (distance is not None):
            raise ValueError(f"layer {layer}: the logarithmic distance term and its two vectors do not agree")
        if s.keep_first and (s.window <= 0 or s.chunk):
            raise ValueError(f"layer {layer}: kept first positions need a window and no chunks")
        # the preparation launch with rotation / unweighted norm / no norm
        self.rot_prep = s.rot is not None or not s.qk_norm or not s.norm_weight
        if s.qkv_bias != (q_bias is not None and k_bias is not None and v_bias is not None) and not s.qk_bias:
            raise ValueError(f"layer {layer}: q / k / v biases and the spec do not agree")
        if s.head_temp != (head_temp is not None):
            raise ValueError(f"layer {layer}: the per-head temperature and the spec do not agree")
        if (s.qkv_bias or s.head_temp) and not self.rot_prep:
            raise ValueError(f"layer {layer}: q / k / v biases and a per-head temperature ride in the rotary preparation launch")
        self.v_bias, self.head_temp = v_bias, head_temp
        if self.rot_prep and (s.norm_scope != "head" or s.values != "own" or v_role or s.qk_bias):
            raise ValueError(f"layer {layer}: rotary / unweighted-norm mixers keep their own values, per-head norms and no biases")
        if not self.rot_prep and (q_norm is None or k_norm is None):
            raise ValueError(f"layer {layer}: the q / k norm needs its weights")
        self.norm_mode = 0 if not s.qk_norm else (2 if s.norm_weight else 1)
        self.inv_freq = from_numpy(np.asarray(s.rot.inv_freq(), np.float64)) if s.rot is not None else None
        self.distance, self.weight_bias, self.out_mult = distance, weight_bias, float(out_mult)
        self.q_cols, self.k_cols = s.heads * s.dim, s.kv_heads * s.dim
        self.v_cols = s.kv_heads * s.vdim if s.values == "own" else 0
        self.g_cols = s.gate_cols
        self.proj_cols = self.q_cols + self.k_cols + self.v_cols + self.g_cols
        if qkvg is not None and qkvg.out_features != self.proj_cols:
            raise ValueError(f"layer {layer}: fused projection has {qkvg.out_features} rows, the mixer needs {self.proj_cols}")
        sl = spec.slopes()
        self.slopes = from_numpy(np.asarray(sl, np.float32)) if sl else None
        self.slopes2 = None
        if distance is not None:
            self.slopes, self.slopes2 = distance
        self.queries_per_tile = int(api.seq_queries_per_tile(s.heads, s.kv_heads))
        self.heads_per_block = int(api.seq_heads_per_block(s.heads, s.kv_heads))
        self.decode_heads_per_block = int(api.seq_decode_heads_per_block())

    @property
    def weight_bytes(self) -> int:
        return self.qkvg.nbytes + self.o_proj.nbytes

    def key_slices(self, ctx) -> int:
        s = self.spec
        return key_slices(ctx, s.heads, s.kv_heads, s.chunk, s.window, self.queries_per_tile, self.heads_per_block,
                          self.decode_heads_per_block, s.keep_first)

    def forward(self, ctx, x: GPUArray, out: GPUArray, cache_index: int | None = None, out_scale: int | None = None,
                state=None) -> None:
        """x [T, W] -> out [T, W] (the mixer's output before the block's norm); K / V of the T tokens enter the cache
        `cache_index` (default: the layer's own).  With out_scale (device pointer of [W] floats) the output projection
        adds out_scale * result to `out` instead of storing it."""
        s, T = self.spec, ctx.T
        W = self.qkvg.in_features
        proj, attn = ctx.buf.proj, ctx.buf.attn
        ld = self.proj_cols
        self.qkvg.forward(x.device_ptr, W, T, proj.device_ptr, ld)
        ldo = s.heads * s.vdim
        self.attend(ctx, proj.device_ptr, ld, attn.device_ptr, ldo, cache_index)
        if out_scale is None:
            self.o_proj.forward(attn.device_ptr, ldo, T, out.device_ptr, self.o_proj.out_features)
        else:
            self.o_proj.forward_seq(attn.device_ptr, ldo, T, out.device_ptr, self.o_proj.out_features, epilogue=4,
                                    col_scale=out_scale)

    def attend(self, ctx, proj_ptr: int, ld: int, attn_ptr: int, ldo: int, cache_index: int | None = None) -> None:
        """Everything between the two matrix products: proj_ptr points at this mixer's [q | k | v | gate] columns inside
        rows of stride ld; the heads' outputs go to attn_ptr (row stride ldo)."""
        s, T = self.spec, ctx.T
        cache = ctx.cache
        ci = self.layer if cache_index is None else cache_index
        kc, vc = cache.k[ci], cache.v[ci]
        if self.rot_prep:
            bias = [b.device_ptr if (s.qkv_bias and b is not None) else None for b in (self.q_bias, self.k_bias, self.v_bias)]
            api.seq_mixer_prep_rot_ex(proj_ptr, ld, T, s.heads, s.kv_heads, s.dim, s.vdim, 0, self.q_cols, self.q_cols + self.k_cols,
                                      s.rot.dims if s.rot is not None else 0,
                                      self.inv_freq.device_ptr if self.inv_freq is not None else None, self.norm_mode,
                                      self.q_norm.device_ptr if self.q_norm is not None else None,
                                      self.k_norm.device_ptr if self.k_norm is not None else None, self.eps, bias[0], bias[1],
                                      bias[2], self.head_temp.device_ptr if self.head_temp is not None else None, kc.device_ptr,
                                      vc.device_ptr, cache.dtype_code, cache.table_dev.device_ptr, cache.pool.max_pages,
                                      cache.page_size, ctx.slot_ptr, ctx.pos_ptr, _st())
        elif s.norm_scope == "all":
            api.seq_mixer_prep_all(proj_ptr, ld, T, s.heads, s.kv_heads, s.dim, self.q_cols,
                                   self.q_bias.device_ptr if self.q_bias is not None else None,
                                   self.k_bias.device_ptr if self.k_bias is not None else None, self.q_norm.device_ptr,
                                   self.k_norm.device_ptr, self.norm_offset, self.eps, kc.device_ptr, vc.device_ptr,
                                   cache.dtype_code, cache.table_dev.device_ptr, cache.pool.max_pages, cache.page_size,
                                   ctx.slot_ptr, ctx.pos_ptr, _st())
        else:
            api.seq_mixer_prep(proj_ptr, ld, T, s.heads, s.kv_heads, s.dim, s.vdim, self.q_norm.device_ptr,
                               self.k_norm.device_ptr, self.eps, self.v_role, self.v_lambda,
                               ctx.buf.v_first.device_ptr if self.v_role else None, kc.device_ptr, vc.device_ptr,
                               cache.dtype_code, cache.table_dev.device_ptr, cache.pool.max_pages, cache.page_size,
                               ctx.slot_ptr, ctx.pos_ptr, _st())
        tiles_ptr, n_tiles = ctx.tiles(self.queries_per_tile)
        splits, ws, tickets = self.key_slices(ctx), None, None
        if splits > 1:
            ws = ctx.workspace(T * s.heads * splits * (s.vdim + 2)).device_ptr
            tickets = ctx.buf.tickets.device_ptr
        gate_mode = 0 if not s.out_gate else (2 if s.gate_per_head else 1)
        api.seq_attention_ex2(proj_ptr, ld, 0, proj_ptr, ld, self.q_cols + self.k_cols + self.v_cols, gate_mode,
                              attn_ptr, ldo, kc.device_ptr, vc.device_ptr, s.dim, s.vdim, cache.dtype_code,
                              cache.table_dev.device_ptr, cache.pool.max_pages, cache.page_size, tiles_ptr, n_tiles,
                              self.slopes.device_ptr if self.slopes is not None else None,
                              self.slopes2.device_ptr if self.slopes2 is not None else None,
                              self.sinks.device_ptr if self.sinks is not None else None, s.heads, s.kv_heads, s.dim, s.vdim,
                              s.chunk, s.window, s.keep_first, s.scale, s.softcap, 1 if s.weights == "sigmoid" else 0,
                              self.weight_bias.device_ptr if self.weight_bias is not None else None, self.out_mult, splits, ws,
                              tickets, 1 if ctx.decode_only else 0, _st())


__all__ = ["PagedAttentionMixer", "key_slices"]
