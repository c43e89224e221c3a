"""Pre-allocated decode buffers (mirror of pygpukit/llm/buffers.py:26-466, reduced to what the
fused B200 step touches).  `allocate(config, dtype, use_qk_norm, vocab_size, max_batch_size)` keeps
the reference's signature; rows = max(1, max_batch_size).  Extra (net-new) members carry the
device-side step state for graph replay: token_buf / position_buf / context_buf (int32)."""
from __future__ import annotations

from dataclasses import dataclass

from ..core.array import GPUArray
from ..core.dtypes import bfloat16, int32
from ..core.factory import zeros
from .config import TransformerConfig


@dataclass
class DecodeBuffers:
    hidden: GPUArray          # [M, H]   residual stream, updated in place
    norm_out: GPUArray        # [M, H]
    qkv_proj_out: GPUArray    # [M, (Hq + 2 Hkv) * hd]  (local heads under TP)
    attn_flat: GPUArray       # [M, Hq * hd]
    mlp_act: GPUArray         # [M, I_local]
    partial: GPUArray         # [M, H]   row-parallel partial sums (TP only)
    logits: GPUArray | None   # [M, V_local]
    token_buf: GPUArray       # int32 [M]  current token ids
    position_buf: GPUArray    # int32 [1]
    context_buf: GPUArray     # int32 [1]
    next_token: GPUArray      # int32 [M]  greedy result
    max_batch_size: int = 1
    num_sequences: int = 1
    state_buf: GPUArray | None = None   # int32 [2 S + M] = [positions, contexts, tokens...]: ONE H2D copy per step

    # aliases with the reference's member names (buffers.py:26-188)
    @property
    def residual(self) -> GPUArray:
        return self.partial

    @property
    def attn_out(self) -> GPUArray:
        return self.attn_flat

    @property
    def mlp_gate(self) -> GPUArray:
        return self.mlp_act

    @classmethod
    def allocate(cls, config: TransformerConfig, dtype: str = "bfloat16", use_qk_norm: bool = False,
                 vocab_size: int | None = None, max_batch_size: int = 0, moe_config: dict | None = None,
                 num_sequences: int = 1) -> "DecodeBuffers":
        if dtype != "bfloat16":
            raise ValueError("the B200 decode path runs in bfloat16")
        M = max(1, max_batch_size)
        tp = max(1, config.tp_size)
        H, hd = config.hidden_size, config.head_dim
        # tp > num_kv_heads: ranks replicate a whole KV head (same rule as Attention.__init__)
        hq, hkv = config.num_heads // tp, max(1, config.num_kv_heads // tp)
        inter = (config.moe_intermediate_size if config.is_moe else config.intermediate_size) // (1 if config.is_moe else tp)
        V = vocab_size if vocab_size is not None else config.vocab_size
        S = max(1, num_sequences)
        # decode state, ONE host-to-device copy per step: [position x S | context x S | token x M]
        state = zeros((2 * S + M,), int32)
        return cls(
            state_buf=state,
            hidden=zeros((M, H), bfloat16), norm_out=zeros((M, H), bfloat16),
            qkv_proj_out=zeros((M, (hq + 2 * hkv) * hd), bfloat16), attn_flat=zeros((M, hq * hd), bfloat16),
            mlp_act=zeros((M, inter), bfloat16), partial=zeros((M, H), bfloat16),
            logits=zeros((M, V), bfloat16) if V else None,
            token_buf=state.narrow(2 * S, M), position_buf=state.narrow(0, S), context_buf=state.narrow(S, S),
            next_token=zeros((M,), int32), max_batch_size=M, num_sequences=S)


@dataclass
class PrefillBuffers:
    """Kept for API parity (buffers.py:467-621); prefill reuses DecodeBuffers in slabs of rows."""
    max_seq_len: int = 0

    @classmethod
    def allocate(cls, config: TransformerConfig, max_seq_len: int, dtype: str = "bfloat16", use_qk_norm: bool = False):
        return cls(max_seq_len=max_seq_len)


__all__ = ["DecodeBuffers", "PrefillBuffers"]


class RowBuffers:
    """Work arrays of the token-major models (llm/models/layered.py), float32 unless noted, sized for `rows` tokens
    of the widest layer and regrown (never shrunk) when a step brings more."""

    def __init__(self, config, rows: int):
        from ..core.dtypes import float32
        W = config.hidden_size
        proj = attn = gv = top = ff = sff = experts = 1
        q_up = q_abs = lat = hout = 1
        conv, second = 0, False
        for L in config.layers:
            m = L.mixer
            proj = max(proj, m.proj_cols)
            conv = max(conv, getattr(m, "conv_cols", 0))
            second = second or getattr(m, "join", "sum") == "rms_mean" or bool(getattr(L.mlp, "shared_gate", False))
            if m.kind == "latent_attention":
                q_up = max(q_up, m.heads * (m.dim + m.rot_dim))
                q_abs = max(q_abs, m.heads * (m.kv_rank + m.rot_dim))
                lat = max(lat, m.heads * m.kv_rank)
                hout = max(hout, m.heads * m.vdim)
            else:
                attn = max(attn, m.attn_cols)
                gv = max(gv, m.kv_heads * getattr(m, "vdim", 0))
            if L.mlp is not None and L.mlp.kind == "dense":
                sff = max(sff, L.mlp.ff)
            elif L.mlp is not None:
                top, ff, sff = max(top, L.mlp.top), max(ff, L.mlp.ff), max(sff, L.mlp.shared_ff)
                experts = max(experts, getattr(L.mlp, "routes", L.mlp.experts) + 1)
        R = self.rows = max(8, int(rows))
        self.x = GPUArray((R, W), float32)
        self.y = GPUArray((R, W), float32)
        normed = getattr(config, "block", "post_norm") in ("parallel", "pre_norm", "sandwich")
        self.y2 = GPUArray((R, W), float32) if second else None             # a second branch's rows
        self.conv = GPUArray((R, conv), float32) if conv else None          # a mixer's convolved columns
        self.moe_mat = GPUArray((R * top,), int32)                          # matrix of every (token, slot) row, -1: none
        self.h = GPUArray((R, W), float32) if normed else None                          # the block's normed rows
        self.x0 = GPUArray((R, W), float32) if getattr(config, "loop_times", 1) > 1 else None   # embedding output
        self.side = GPUArray((R, max(1, getattr(config, "side_dim", 0))), float32)
        self.proj = GPUArray((R, proj), float32)
        self.attn = GPUArray((R, attn), float32)
        self.q_up = GPUArray((R, q_up), float32)            # latent attention: queries, absorbed queries + rotated
        self.q_abs = GPUArray((R, q_abs), float32)          # tails, latent-space outputs, per-head values
        self.latent_out = GPUArray((R, lat), float32)
        self.head_out = GPUArray((R, hout), float32)
        self.v_first = GPUArray((R, gv), float32)
        self.moe_idx = GPUArray((R * top,), int32)
        self.moe_rank = GPUArray((R * top,), int32)
        self.moe_perm = GPUArray((R * top,), int32)
        self.moe_inv = GPUArray((R * top,), int32)
        self.moe_w = GPUArray((R * top,), float32)
        self.moe_z = GPUArray((R, experts), float32)         # router logits
        self.tickets = zeros((4096,), int32)                # arrival counters of the key-sliced attention (self-clearing)
        self.moe_counts = zeros((experts,), int32)          # zero between uses (pgk_moe_row_lists clears it)
        self.moe_off = GPUArray((experts + 1,), int32)
        self.moe_act = GPUArray((R * top, ff), float32)
        self.moe_parts = GPUArray((R * top, W), float32)
        self.shared_act = GPUArray((R, sff), float32)       # shared expert / dense feed-forward activations


__all__.append("RowBuffers")
