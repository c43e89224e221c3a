"""Checkpoint loading for the layered models (net-new; `loader.py` covers the uniform Hugging Face families).

`load_layered_model(path, dtype)` reads `config.json` (its "architecture" picks the family, llm/config.py) and
`model.safetensors` next to it; `build_layered_model(config, tensors, dtype)` takes the tensors as a
{name: float32 ndarray} dictionary (tests, random initialisation).  dtype "bfloat16": matrices go to the device as
bfloat16 (rounded to nearest even when the file holds wider floats), cache in bfloat16; "float32": matrices and
cache in float32.  Norm weights, biases, other small vectors and the router matrices are float32 on the device in both
modes (the router's logits are formed from the unrounded float32 residual stream).

Dolurax tensor names: embed, head, final.norm(.b); per layer l<i>.norm1(.b), l<i>.norm2(.b), l<i>.mix.{q,k,v,g,o},
l<i>.mix.{q,k}.norm, l<i>.mix.vmix (scalar), l<i>.mlp.router, l<i>.mlp.e<j>.{gate,up,down},
l<i>.mlp.shared.{gate,up,down}; linear weights [out, in].  q, k, v and the gate are fused row-wise into one
projection, gate/up pairs are interleaved row by row for the SiLU-multiply epilogue, experts are stacked.

Turutar tensor names: embed, embed.norm, side.embed [vocab, layers x side dim], final.norm, head; per layer l<i>.norm1,
l<i>.ls1, l<i>.ls2, l<i>.mlp.{gate,up,down}, l<i>.side.{gate,proj,norm}; windowed attention l<i>.mix.{q,k} with biases
.q.b / .k.b and whole-projection norm weights .q.norm / .k.norm, l<i>.mix.g [heads, width], l<i>.mix.o; latent attention
l<i>.mix.{dq,uq,dkv,uk,uv,g,o}, .dq.norm, .dkv.norm, .sink.  The projections that read the block's normed rows are fused
row-wise ([q | k | g] and [dq | dkv | g]); uk is stored per head transposed ([heads, kv_rank, dim]) so that the query
absorbs it, uv as the stack [heads, vdim, kv_rank].

Rezulorn tensor names: embed, final.norm, head; per layer l<i>.norm1, l<i>.norm2, l<i>.canon1, l<i>.canon2 [width, taps],
l<i>.mlp.{up,down}; "lightning" l<i>.mix.{q,k,v,g,o,norm}; "attention" l<i>.mix.{q,k,v,o,r1,r2}; "parallel"
l<i>.mix.left.{q,k,v,o,pb} and l<i>.mix.right.{q,k,v,g,o}.  The projections of a mixer are fused row-wise ([q | k | v | g],
both sides of a parallel mixer in one matrix) and the two output projections of a parallel mixer column-wise.

Sumitar tensor names: embed (also the head), final.norm(.b, .alpha); per layer l<i>.norm1, norm1b, norm2, norm2b, each with .b
and the scalar .alpha; "parallel" l<i>.mix.left.{q,k,v} with biases .q.b / .k.b / .v.b, .left.temp [heads], .left.o, .left.out,
l<i>.mix.right.{q,f,v,o}, .right.f.b, .right.lower, .right.norm [vdim], .right.out; "delta" l<i>.mix.{q,k,v} with .conv
[channels, taps] each, l<i>.mix.{b,a} [heads, width], .A_log, .dt_bias, .norm [vdim], .g, .o; dense feed-forward
l<i>.mlp.{up,down,act}; experts l<i>.mlp.e<j>.{gate,up,down}, .router [experts + identity, width], .correction,
.shared.{gate,up,down,sg}.  Both sides' projections of a parallel mixer are one matrix ([left q | k | v | right q | f | v]), a
delta mixer's are [q | k | v | g | b | a]; the router matrix carries the shared expert's gate row as its last row.
"""
from __future__ import annotations

import json
import os

import numpy as np

from ..core.array import GPUArray
from ..core.dtypes import bf16_bits_to_f32, f32_to_bf16_bits
from ..core.factory import from_numpy
from .config import LayeredConfig, layered_config_from_json
from .layers.block import ParallelBlock, PostNormBlock, PreNormBlock, SandwichBlock
from .layers.dense_rows import GatedDenseRows, PolyNormRows, SquaredReluRows
from .layers.gated_recurrent import DeltaRuleMixer, GatedLinearMixer
from .layers.linear_attention import LinearAttentionMixer, ParallelMixer
from .layers.latent_attention import LatentAttentionMixer
from .layers.linear import LinearRows, interleave_gate_up
from .layers.moe_rows import BiasedRouterMoE, GroupedRouterMoE
from .layers.norm import CausalConvRows, RowNorm
from .layers.paged_attention import PagedAttentionMixer
from .layers.token_side import TokenSideInput
from .models.layered import LayeredCausalModel
from .safetensors import load_safetensors


class _Tensors:
    """name -> float32 ndarray, from a dictionary or a safetensors file."""

    def __init__(self, src):
        self.src = src
        self.is_file = not isinstance(src, dict)

    def has(self, name: str) -> bool:
        return name in self.src

    def f32(self, name: str, shape: tuple | None = None) -> np.ndarray:
        if not self.has(name):
            raise KeyError(f"checkpoint has no tensor {name!r}")
        if self.is_file:
            info = self.src.tensor_info(name)
            a = self.src.tensor(name)
            a = bf16_bits_to_f32(a).reshape(info.shape) if info.dtype == "BF16" else np.asarray(a, np.float32).reshape(info.shape)
        else:
            a = np.asarray(self.src[name], np.float32)
        if shape is not None and tuple(a.shape) != tuple(shape):
            raise ValueError(f"tensor {name!r} has shape {tuple(a.shape)}, the config needs {tuple(shape)}")
        return a


def _matrix(a: np.ndarray, dtype: str) -> GPUArray:
    a = np.ascontiguousarray(a, np.float32)
    return from_numpy(f32_to_bf16_bits(a).reshape(a.shape) if dtype == "bfloat16" else a)


def _vector(a: np.ndarray) -> GPUArray:
    return from_numpy(np.ascontiguousarray(a, np.float32))


def build_layered_model(config: LayeredConfig, tensors, dtype: str = "bfloat16") -> LayeredCausalModel:
    if dtype not in ("bfloat16", "float32"):
        raise ValueError("layered models run in 'bfloat16' or 'float32'")
    t = tensors if isinstance(tensors, _Tensors) else _Tensors(tensors)
    builder = _BUILDERS.get(config.architecture.lower())
    if builder is None:
        raise ValueError(f"no weight layout known for architecture {config.architecture!r}")
    return builder(config, t, dtype)


def _build_turutar(config: LayeredConfig, t: _Tensors, dtype: str) -> LayeredCausalModel:
    W, V, eps, sd = config.hidden_size, config.vocab_size, config.norm_eps, config.side_dim
    n_layers = len(config.layers)

    def norm1p(name):                      # the model's norm: weights stored around zero
        return RowNorm("rmsnorm", _vector(t.f32(name, (W,))), None, eps, offset=1.0)

    side_table = _matrix(t.f32("side.embed", (V, n_layers * sd)), dtype) if sd else None
    blocks = []
    for i, L in enumerate(config.layers):
        p, m = f"l{i}.", L.mixer
        mp = p + "mix."
        if m.kind == "attention":
            qd, kd = m.heads * m.dim, m.kv_heads * m.dim
            fused = np.concatenate([t.f32(mp + "q", (qd, W)), t.f32(mp + "k", (kd, W)), t.f32(mp + "g", (m.heads, W))])
            mixer = PagedAttentionMixer(m, i, LinearRows(_matrix(fused, dtype)),
                                        LinearRows(_matrix(t.f32(mp + "o", (W, m.heads * m.vdim)), dtype)),
                                        _vector(t.f32(mp + "q.norm", (qd,))), _vector(t.f32(mp + "k.norm", (kd,))), eps,
                                        q_bias=_vector(t.f32(mp + "q.b", (qd,))), k_bias=_vector(t.f32(mp + "k.b", (kd,))))
        else:
            hd = m.dim + m.rot_dim
            fused = np.concatenate([t.f32(mp + "dq", (m.q_rank, W)), t.f32(mp + "dkv", (m.kv_rank + m.rot_dim, W)),
                                    t.f32(mp + "g", (m.heads, W))])
            uk = t.f32(mp + "uk", (m.heads * m.dim, m.kv_rank)).reshape(m.heads, m.dim, m.kv_rank).transpose(0, 2, 1)
            uv = t.f32(mp + "uv", (m.heads * m.vdim, m.kv_rank)).reshape(m.heads, m.vdim, m.kv_rank)
            mixer = LatentAttentionMixer(m, i, LinearRows(_matrix(fused, dtype)),
                                         LinearRows(_matrix(t.f32(mp + "uq", (m.heads * hd, m.q_rank)), dtype)),
                                         LinearRows(_matrix(uk, dtype)), LinearRows(_matrix(uv, dtype)),
                                         LinearRows(_matrix(t.f32(mp + "o", (W, m.heads * m.vdim)), dtype)),
                                         _vector(t.f32(mp + "dq.norm", (m.q_rank,))), _vector(t.f32(mp + "dkv.norm", (m.kv_rank,))),
                                         eps, sinks=_vector(t.f32(mp + "sink", (m.heads,))))
        mlp = ls2 = None
        if L.mlp is not None:
            f, q = L.mlp, p + "mlp."
            gu = interleave_gate_up(t.f32(q + "gate", (f.ff, W)), t.f32(q + "up", (f.ff, W)))
            mlp = GatedDenseRows(f, LinearRows(_matrix(gu, dtype)), LinearRows(_matrix(t.f32(q + "down", (W, f.ff)), dtype)))
            ls2 = _vector(t.f32(p + "ls2", (W,)))
        side = None
        if sd:
            side = TokenSideInput(side_table, i, sd, LinearRows(_matrix(t.f32(p + "side.gate", (sd, W)), dtype)),
                                  LinearRows(_matrix(t.f32(p + "side.proj", (W, sd)), dtype)),
                                  RowNorm("rmsnorm", _vector(t.f32(p + "side.norm", (W,))), None, eps, offset=0.0))
        blocks.append(ParallelBlock(norm1p(p + "norm1"), mixer, _vector(t.f32(p + "ls1", (W,))), mlp, ls2, side))
    head = LinearRows(_matrix(t.f32("head", (V, W)), dtype))
    return LayeredCausalModel(config, _matrix(t.f32("embed", (V, W)), dtype), blocks, norm1p("final.norm"), head, dtype,
                              embed_norm=norm1p("embed.norm"))


def _build_dolurax(config: LayeredConfig, t: _Tensors, dtype: str) -> LayeredCausalModel:
    W, V, eps = config.hidden_size, config.vocab_size, config.norm_eps
    blocks = []
    first_mix = None          # index and value width of the first value-mixing layer
    for i, L in enumerate(config.layers):
        p, m = f"l{i}.", L.mixer
        mp = p + "mix."
        parts = [t.f32(mp + "q", (m.heads * m.dim, W)), t.f32(mp + "k", (m.kv_heads * m.dim, W)),
                 t.f32(mp + "v", (m.kv_heads * m.vdim, W))]
        if m.out_gate:
            parts.append(t.f32(mp + "g", (m.heads * m.vdim, W)))
        qkvg = LinearRows(_matrix(np.concatenate(parts), dtype))
        o_proj = LinearRows(_matrix(t.f32(mp + "o", (W, m.heads * m.vdim)), dtype))
        role, lam = 0, 0.0
        if m.v_mix:
            if first_mix is None:
                first_mix, role = (i, m.kv_heads * m.vdim), 1
            else:
                if m.kv_heads * m.vdim != first_mix[1]:
                    raise ValueError(f"layer {i} mixes values of width {m.kv_heads * m.vdim} with layer {first_mix[0]}'s {first_mix[1]}")
                role, lam = 2, float(t.f32(mp + "vmix").reshape(-1)[0])
        mixer = PagedAttentionMixer(m, i, qkvg, o_proj, _vector(t.f32(mp + "q.norm", (m.dim,))),
                                    _vector(t.f32(mp + "k.norm", (m.dim,))), eps, role, lam)
        norm1 = (_vector(t.f32(p + "norm1", (W,))), _vector(t.f32(p + "norm1.b", (W,))))
        mlp = norm2 = None
        if L.mlp is not None:
            f, q = L.mlp, p + "mlp."
            gu = np.stack([interleave_gate_up(t.f32(f"{q}e{e}.gate", (f.ff, W)), t.f32(f"{q}e{e}.up", (f.ff, W)))
                           for e in range(f.experts)])
            dn = np.stack([t.f32(f"{q}e{e}.down", (W, f.ff)) for e in range(f.experts)])
            sgu = sdn = None
            if f.shared_ff:
                s = q + "shared."
                sgu = LinearRows(_matrix(interleave_gate_up(t.f32(s + "gate", (f.shared_ff, W)), t.f32(s + "up", (f.shared_ff, W))),
                                         dtype), epilogue=1)
                sdn = LinearRows(_matrix(t.f32(s + "down", (W, f.shared_ff)), dtype))
            # the router stays float32 in both modes: its logits come from the unrounded residual stream
            mlp = GroupedRouterMoE(f, _matrix(t.f32(q + "router", (f.experts, W)), "float32"),
                                   LinearRows(_matrix(gu, dtype), epilogue=1), LinearRows(_matrix(dn, dtype)), sgu, sdn)
            norm2 = (_vector(t.f32(p + "norm2", (W,))), _vector(t.f32(p + "norm2.b", (W,))))
        blocks.append(PostNormBlock(mixer, norm1, mlp, norm2, eps))
    head = LinearRows(_matrix(t.f32("head", (V, W)), dtype), epilogue=2, scale=config.logit_scale, cap=config.logit_softcap)
    final = (_vector(t.f32("final.norm", (W,))), _vector(t.f32("final.norm.b", (W,))))
    return LayeredCausalModel(config, _matrix(t.f32("embed", (V, W)), dtype), blocks, final, head, dtype)


def _build_rezulorn(config: LayeredConfig, t: _Tensors, dtype: str) -> LayeredCausalModel:
    W, V, eps, taps = config.hidden_size, config.vocab_size, config.norm_eps, config.conv_taps
    mult = _vector(np.full((W,), config.residual_mult, np.float32))

    def norm(name):
        return RowNorm("layernorm_nobias", _vector(t.f32(name, (W,))), None, eps)

    def conv(name):
        return CausalConvRows(_vector(t.f32(name, (W, taps)))) if taps > 0 else None

    def attention(m, mp, layer, fused: bool, out_mult: float = 1.0):
        parts = [t.f32(mp + "q", (m.heads * m.dim, W)), t.f32(mp + "k", (m.kv_heads * m.dim, W)),
                 t.f32(mp + "v", (m.kv_heads * m.vdim, W))]
        o = t.f32(mp + "o", (W, m.heads * m.vdim))
        dist = (_vector(t.f32(mp + "r1", (m.heads,))), _vector(t.f32(mp + "r2", (m.heads,)))) if m.distance_bias == "log" else None
        pb = _vector(t.f32(mp + "pb", (m.heads,))) if m.weights == "sigmoid" else None
        mixer = PagedAttentionMixer(m, layer, None if fused else LinearRows(_matrix(np.concatenate(parts), dtype)),
                                    None if fused else LinearRows(_matrix(o, dtype)), None, None, eps, distance=dist,
                                    weight_bias=pb, out_mult=out_mult)
        return mixer, parts, o

    def linear(m, mp, layer, fused: bool, out_mult: float = 1.0):
        parts = [t.f32(mp + "q", (m.heads * m.dim, W)), t.f32(mp + "k", (m.heads * m.dim, W)),
                 t.f32(mp + "v", (m.heads * m.vdim, W)), t.f32(mp + "g", (m.heads * m.vdim, W))]
        o = t.f32(mp + "o", (W, m.heads * m.vdim))
        nw = _vector(t.f32(mp + "norm", (m.heads * m.vdim,))) if m.out_norm == "all" else None
        mixer = LinearAttentionMixer(m, layer, None if fused else LinearRows(_matrix(np.concatenate(parts), dtype)),
                                     None if fused else LinearRows(_matrix(o, dtype)), nw, eps, out_mult=out_mult)
        return mixer, parts, o

    blocks = []
    for i, L in enumerate(config.layers):
        p, m = f"l{i}.", L.mixer
        mp = p + "mix."
        if m.kind == "linear_attention":
            mixer = linear(m, mp, i, False)[0]
        elif m.kind == "attention":
            mixer = attention(m, mp, i, False)[0]
        else:
            left, lp, lo = attention(m.left, mp + "left.", i, True, m.left_scale)
            right, rp, ro = linear(m.right, mp + "right.", i, True, m.right_scale)
            mixer = ParallelMixer(m, i, LinearRows(_matrix(np.concatenate(lp + rp), dtype)),
                                  LinearRows(_matrix(np.concatenate([lo, ro], axis=1), dtype)), left, right)
        mlp = norm2 = conv2 = None
        if L.mlp is not None:
            f, q = L.mlp, p + "mlp."
            mlp = SquaredReluRows(f, LinearRows(_matrix(t.f32(q + "up", (f.ff, W)), dtype)),
                                  LinearRows(_matrix(t.f32(q + "down", (W, f.ff)), dtype)))
            norm2, conv2 = norm(p + "norm2"), conv(p + "canon2")
        blocks.append(PreNormBlock(norm(p + "norm1"), conv(p + "canon1"), mixer, norm2, conv2, mlp, mult))
    head = LinearRows(_matrix(t.f32("head", (V, W)), dtype), epilogue=2, scale=config.logit_scale, cap=0.0)
    return LayeredCausalModel(config, _matrix(t.f32("embed", (V, W)), dtype), blocks, norm("final.norm"), head, dtype)


def _build_sumitar(config: LayeredConfig, t: _Tensors, dtype: str) -> LayeredCausalModel:
    W, V, eps = config.hidden_size, config.vocab_size, config.norm_eps

    def norm(name):
        return RowNorm("dyt", _vector(t.f32(name, (W,))), _vector(t.f32(name + ".b", (W,))), eps,
                       alpha=float(t.f32(name + ".alpha").reshape(-1)[0]))

    def per_head(name, heads, vdim):          # a weight vector shared by the heads, laid out per head
        return _vector(np.tile(t.f32(name, (vdim,)), heads))

    blocks = []
    for i, L in enumerate(config.layers):
        p, m = f"l{i}.", L.mixer
        mp = p + "mix."
        if m.kind == "parallel":
            a, r = m.left, m.right
            lp, rp = mp + "left.", mp + "right."
            qd, kd, vd = a.heads * a.dim, a.kv_heads * a.dim, a.kv_heads * a.vdim
            rq, rv = r.heads * r.dim, r.heads * r.vdim
            fused = np.concatenate([t.f32(lp + "q", (qd, W)), t.f32(lp + "k", (kd, W)), t.f32(lp + "v", (vd, W)),
                                    t.f32(rp + "q", (rq, W)), t.f32(rp + "f", (rq, W)), t.f32(rp + "v", (rv, W))])
            left = PagedAttentionMixer(a, i, None, None, None, None, eps, q_bias=_vector(t.f32(lp + "q.b", (qd,))),
                                       k_bias=_vector(t.f32(lp + "k.b", (kd,))), v_bias=_vector(t.f32(lp + "v.b", (vd,))),
                                       head_temp=_vector(t.f32(lp + "temp", (a.heads,))))
            right = GatedLinearMixer(r, i, None, None, _vector(t.f32(rp + "f.b", (rq,))), _vector(t.f32(rp + "lower", (rq,))),
                                     per_head(rp + "norm", r.heads, r.vdim), eps)
            mixer = ParallelMixer(m, i, LinearRows(_matrix(fused, dtype)), None, left, right,
                                  o_left=LinearRows(_matrix(t.f32(lp + "o", (W, a.heads * a.vdim)), dtype)),
                                  o_right=LinearRows(_matrix(t.f32(rp + "o", (W, rv)), dtype)),
                                  out_weights=(_vector(t.f32(lp + "out", (W,))), _vector(t.f32(rp + "out", (W,)))), eps=eps)
        else:
            qk, vd, H = m.qk_heads * m.dim, m.heads * m.vdim, m.heads
            fused = np.concatenate([t.f32(mp + "q", (qk, W)), t.f32(mp + "k", (qk, W)), t.f32(mp + "v", (vd, W)),
                                    t.f32(mp + "g", (vd, W)), t.f32(mp + "b", (H, W)), t.f32(mp + "a", (H, W))])
            taps = m.conv_taps
            conv = np.concatenate([t.f32(mp + "q.conv", (qk, taps)), t.f32(mp + "k.conv", (qk, taps)), t.f32(mp + "v.conv", (vd, taps))])
            mixer = DeltaRuleMixer(m, i, LinearRows(_matrix(fused, dtype)), LinearRows(_matrix(t.f32(mp + "o", (W, vd)), dtype)),
                                   _vector(conv), _vector(t.f32(mp + "A_log", (H,))), _vector(t.f32(mp + "dt_bias", (H,))),
                                   per_head(mp + "norm", H, m.vdim), eps)
        mlp = norm2 = norm2b = None
        f = L.mlp
        if f is not None:
            q = p + "mlp."
            if f.kind == "dense":
                mlp = PolyNormRows(f, LinearRows(_matrix(t.f32(q + "up", (f.ff, W)), dtype)),
                                   LinearRows(_matrix(t.f32(q + "down", (W, f.ff)), dtype)), _vector(t.f32(q + "act", (4,))), eps)
            else:
                gu = dn = sgu = sdn = None
                if f.experts:
                    gu = LinearRows(_matrix(np.stack([interleave_gate_up(t.f32(f"{q}e{e}.gate", (f.ff, W)), t.f32(f"{q}e{e}.up", (f.ff, W)))
                                                      for e in range(f.experts)]), dtype), epilogue=1)
                    dn = LinearRows(_matrix(np.stack([t.f32(f"{q}e{e}.down", (W, f.ff)) for e in range(f.experts)]), dtype))
                rows = [t.f32(q + "router", (f.routes, W))]
                if f.shared_ff:
                    sq = q + "shared."
                    sgu = LinearRows(_matrix(interleave_gate_up(t.f32(sq + "gate", (f.shared_ff, W)), t.f32(sq + "up", (f.shared_ff, W))),
                                             dtype), epilogue=1)
                    sdn = LinearRows(_matrix(t.f32(sq + "down", (W, f.shared_ff)), dtype))
                    if f.shared_gate:
                        rows.append(t.f32(sq + "sg", (1, W)))
                # the router (and the gate row it carries) stays float32 in both modes
                mlp = BiasedRouterMoE(f, _matrix(np.concatenate(rows), "float32"), _vector(t.f32(q + "correction", (f.routes,))),
                                      gu, dn, sgu, sdn)
            norm2, norm2b = norm(p + "norm2"), norm(p + "norm2b")
        blocks.append(SandwichBlock(norm(p + "norm1"), mixer, norm(p + "norm1b"), norm2, mlp, norm2b))
    embed = _matrix(t.f32("embed", (V, W)), dtype)
    return LayeredCausalModel(config, embed, blocks, norm("final.norm"), LinearRows(embed), dtype)


# architecture (lower case) -> builder of its blocks from the checkpoint's tensors
_BUILDERS = {"dolurax": _build_dolurax, "turutar": _build_turutar, "rezulorn": _build_rezulorn, "sumitar": _build_sumitar}


def load_layered_model(model_path: str, dtype: str = "bfloat16", config: dict | None = None) -> LayeredCausalModel:
    """`model_path`: a folder holding config.json + model.safetensors, or the safetensors file itself."""
    folder = model_path if os.path.isdir(model_path) else os.path.dirname(os.path.abspath(model_path))
    st_path = os.path.join(folder, "model.safetensors") if os.path.isdir(model_path) else model_path
    if config is None:
        with open(os.path.join(folder, "config.json"), encoding="utf-8") as f:
            config = json.load(f)
    cfg = layered_config_from_json(config)
    if cfg is None:
        raise ValueError(f"config.json names no layered architecture (got {config.get('architecture')!r})")
    return build_layered_model(cfg, _Tensors(load_safetensors(st_path)), dtype)


__all__ = ["build_layered_model", "load_layered_model"]
