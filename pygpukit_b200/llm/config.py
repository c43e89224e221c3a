"""Model configuration (mirror of pygpukit/llm/config.py:20-615).

`ModelSpec` here keeps only the architecture flags the decode path reads (the reference's HF
tensor-name patterns belong to checkpoint loading, which is out of scope: SURVEY.md section 8f-3);
`TransformerConfig` has the reference's fields, defaults and derived properties
(config.py:440-510) plus `tp_size` / `tp_rank` for the net-new tensor-parallel path.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Literal


@dataclass(frozen=True)
class ModelSpec:
    name: str
    norm_type: Literal["rmsnorm", "layernorm"] = "rmsnorm"
    activation: Literal["gelu", "silu"] = "silu"
    use_rope: bool = True
    use_qk_norm: bool = False
    use_position_embed: bool = False
    qkv_combined: bool = False
    weight_transpose: bool = False
    is_moe: bool = False
    qkv_bias: bool = False
    default_norm_eps: float = 1e-5
    default_rope_theta: float = 10000.0
    hf_model_type: str = ""


GPT2_SPEC = ModelSpec(name="gpt2", norm_type="layernorm", activation="gelu", use_rope=False,
                      use_position_embed=True, qkv_combined=True, weight_transpose=True, qkv_bias=True,
                      hf_model_type="gpt2")
LLAMA_SPEC = ModelSpec(name="llama", hf_model_type="llama")
QWEN2_SPEC = ModelSpec(name="qwen2", qkv_bias=True, default_norm_eps=1e-6, default_rope_theta=1000000.0,
                       hf_model_type="qwen2")
QWEN3_SPEC = ModelSpec(name="qwen3", use_qk_norm=True, default_norm_eps=1e-6, default_rope_theta=1000000.0,
                       hf_model_type="qwen3")
QWEN3_MOE_SPEC = ModelSpec(name="qwen3_moe", use_qk_norm=True, is_moe=True, default_norm_eps=1e-6,
                           default_rope_theta=1000000.0, hf_model_type="qwen3_moe")
MIXTRAL_SPEC = ModelSpec(name="mixtral", is_moe=True, default_rope_theta=1000000.0, hf_model_type="mixtral")

MODEL_SPECS: dict[str, ModelSpec] = {
    "gpt2": GPT2_SPEC, "llama": LLAMA_SPEC, "qwen3": QWEN3_SPEC, "qwen3_moe": QWEN3_MOE_SPEC,
    "qwen2": QWEN2_SPEC, "mixtral": MIXTRAL_SPEC,
}


def detect_model_spec(tensor_names: list[str]) -> ModelSpec:
    """Same decision order as config.py:391-428."""
    if any("block_sparse_moe" in n for n in tensor_names):
        return MIXTRAL_SPEC
    has_moe = any("mlp.experts" in n for n in tensor_names)
    has_qk = any("q_norm" in n for n in tensor_names)
    if has_moe and has_qk:
        return QWEN3_MOE_SPEC
    if has_qk:
        return QWEN3_SPEC
    if "model.embed_tokens.weight" in tensor_names and "model.layers.0.self_attn.q_proj.bias" in tensor_names:
        return QWEN2_SPEC
    if "model.embed_tokens.weight" in tensor_names:
        return LLAMA_SPEC
    if "wte.weight" in tensor_names:
        return GPT2_SPEC
    raise ValueError(f"Cannot detect model type from tensor names. First 10 names: {tensor_names[:10]}")


@dataclass
class TransformerConfig:
    vocab_size: int = 32000
    hidden_size: int = 2048
    num_layers: int = 22
    num_heads: int = 32
    num_kv_heads: int | None = None
    intermediate_size: int | None = None
    _head_dim: int | None = None

    num_experts: int | None = None
    num_experts_per_tok: int = 2
    moe_intermediate_size: int | None = None

    norm_type: Literal["rmsnorm", "layernorm"] = "rmsnorm"
    activation: Literal["gelu", "silu"] = "silu"
    use_rope: bool = True
    causal: bool = True

    max_position_embeddings: int = 2048
    norm_eps: float = 1e-5
    rope_theta: float = 10000.0

    tie_word_embeddings: bool = True

    # net-new: tensor parallelism (the reference is single-GPU, docs/scheduler.md:358)
    tp_size: int = 1
    tp_rank: int = 0

    def __post_init__(self):
        if self.num_kv_heads is None:
            self.num_kv_heads = self.num_heads
        if self.intermediate_size is None:
            self.intermediate_size = 4 * self.hidden_size
        if self.moe_intermediate_size is None:
            self.moe_intermediate_size = self.intermediate_size

    @property
    def is_moe(self) -> bool:
        return self.num_experts is not None and self.num_experts > 1

    @property
    def head_dim(self) -> int:
        if self._head_dim is not None:
            return self._head_dim
        return self.hidden_size // self.num_heads

    @property
    def num_kv_groups(self) -> int:
        assert self.num_kv_heads is not None
        return self.num_heads // self.num_kv_heads


@dataclass
class GPT2Config:
    vocab_size: int = 50257
    n_embd: int = 768
    n_layer: int = 12
    n_head: int = 12
    n_positions: int = 1024
    layer_norm_eps: float = 1e-5

    @property
    def n_inner(self) -> int:
        return 4 * self.n_embd

    def to_transformer_config(self) -> TransformerConfig:
        return TransformerConfig(vocab_size=self.vocab_size, hidden_size=self.n_embd, num_layers=self.n_layer,
                                 num_heads=self.n_head, num_kv_heads=self.n_head, intermediate_size=self.n_inner,
                                 norm_type="layernorm", activation="gelu", use_rope=False, causal=True,
                                 max_position_embeddings=self.n_positions, norm_eps=self.layer_norm_eps)


@dataclass
class LlamaConfig:
    vocab_size: int = 32000
    hidden_size: int = 2048
    intermediate_size: int = 5632
    num_hidden_layers: int = 22
    num_attention_heads: int = 32
    num_key_value_heads: int = 4
    max_position_embeddings: int = 2048
    rms_norm_eps: float = 1e-5
    rope_theta: float = 10000.0

    @property
    def head_dim(self) -> int:
        return self.hidden_size // self.num_attention_heads

    def to_transformer_config(self) -> TransformerConfig:
        return TransformerConfig(vocab_size=self.vocab_size, hidden_size=self.hidden_size,
                                 num_layers=self.num_hidden_layers, num_heads=self.num_attention_heads,
                                 num_kv_heads=self.num_key_value_heads, intermediate_size=self.intermediate_size,
                                 norm_type="rmsnorm", activation="silu", use_rope=True, causal=True,
                                 max_position_embeddings=self.max_position_embeddings, norm_eps=self.rms_norm_eps,
                                 rope_theta=self.rope_theta)


@dataclass
class Qwen3Config:
    vocab_size: int = 151936
    hidden_size: int = 4096
    intermediate_size: int = 12288
    num_hidden_layers: int = 36
    num_attention_heads: int = 32
    num_key_value_heads: int = 8
    head_dim: int = 128
    max_position_embeddings: int = 40960
    rms_norm_eps: float = 1e-6
    rope_theta: float = 1000000.0

    def to_transformer_config(self) -> TransformerConfig:
        return TransformerConfig(vocab_size=self.vocab_size, hidden_size=self.hidden_size,
                                 num_layers=self.num_hidden_layers, num_heads=self.num_attention_heads,
                                 num_kv_heads=self.num_key_value_heads, intermediate_size=self.intermediate_size,
                                 _head_dim=self.head_dim, norm_type="rmsnorm", activation="silu", use_rope=True,
                                 causal=True, max_position_embeddings=self.max_position_embeddings,
                                 norm_eps=self.rms_norm_eps, rope_theta=self.rope_theta)


# ---- the shapes BASELINE.json's configs name (SURVEY.md section 8 header)
def named_config(name: str, max_seq: int = 4096, tp_size: int = 1, tp_rank: int = 0) -> tuple[TransformerConfig, ModelSpec]:
    """(config, spec) of a benchmark model: 'gpt2', 'qwen3-8b', 'llama3-8b', 'llama3-70b', 'qwen3-30b-a3b'
    (and 'tiny-*' variants used by the tests)."""
    kw = dict(max_position_embeddings=max_seq, tp_size=tp_size, tp_rank=tp_rank, tie_word_embeddings=False)
    n = name.lower()
    if n == "gpt2":
        c = GPT2Config().to_transformer_config()
        return c, GPT2_SPEC
    if n == "qwen3-8b":
        return TransformerConfig(vocab_size=151936, hidden_size=4096, num_layers=36, num_heads=32, num_kv_heads=8,
                                 intermediate_size=12288, _head_dim=128, norm_eps=1e-6, rope_theta=1e6, **kw), QWEN3_SPEC
    if n == "llama3-8b":
        return TransformerConfig(vocab_size=128256, hidden_size=4096, num_layers=32, num_heads=32, num_kv_heads=8,
                                 intermediate_size=14336, norm_eps=1e-5, rope_theta=5e5, **kw), LLAMA_SPEC
    if n == "llama3-70b":
        return TransformerConfig(vocab_size=128256, hidden_size=8192, num_layers=80, num_heads=64, num_kv_heads=8,
                                 intermediate_size=28672, norm_eps=1e-5, rope_theta=5e5, **kw), LLAMA_SPEC
    if n == "qwen3-30b-a3b":
        return TransformerConfig(vocab_size=151936, hidden_size=2048, num_layers=48, num_heads=32, num_kv_heads=4,
                                 intermediate_size=6144, _head_dim=128, num_experts=128, num_experts_per_tok=8,
                                 moe_intermediate_size=768, norm_eps=1e-6, rope_theta=1e7, **kw), QWEN3_MOE_SPEC
    if n == "tiny-llama":
        return TransformerConfig(vocab_size=1024, hidden_size=256, num_layers=2, num_heads=4, num_kv_heads=2,
                                 intermediate_size=512, _head_dim=64, norm_eps=1e-5, rope_theta=1e4, **kw), LLAMA_SPEC
    if n == "tiny-qwen3":
        return TransformerConfig(vocab_size=1024, hidden_size=256, num_layers=2, num_heads=4, num_kv_heads=2,
                                 intermediate_size=512, _head_dim=128, norm_eps=1e-6, rope_theta=1e6, **kw), QWEN3_SPEC
    if n == "small-qwen3":      # hidden >= 512: exercises the fused RMSNorm->GEMV prologue
        return TransformerConfig(vocab_size=2048, hidden_size=512, num_layers=2, num_heads=8, num_kv_heads=2,
                                 intermediate_size=1024, _head_dim=128, norm_eps=1e-6, rope_theta=1e6, **kw), QWEN3_SPEC
    if n == "small-llama":
        return TransformerConfig(vocab_size=2048, hidden_size=512, num_layers=2, num_heads=8, num_kv_heads=4,
                                 intermediate_size=1536, _head_dim=64, norm_eps=1e-5, rope_theta=5e5, **kw), LLAMA_SPEC
    if n == "tiny-moe":
        return TransformerConfig(vocab_size=1024, hidden_size=256, num_layers=2, num_heads=4, num_kv_heads=2,
                                 intermediate_size=512, _head_dim=64, num_experts=8, num_experts_per_tok=2,
                                 moe_intermediate_size=128, norm_eps=1e-6, rope_theta=1e6, **kw), QWEN3_MOE_SPEC
    raise ValueError(f"unknown model name {name!r}")



# ---- per-layer ("layered") configurations: models whose config.json lists every layer with its own mixer and
# feed-forward (net-new; the reference's families are uniform stacks described by TransformerConfig)
@dataclass(frozen=True)
class AttentionMixerSpec:
    """One attention mixer: H query heads of size `dim`, G key/value heads, values of size `vdim`; score =
    scale q.k, squashed to softcap tanh(. / softcap) when softcap > 0, minus a per-head distance slope when
    `distance_bias`; `chunk` > 0 limits a query to the keys of its own chunk of positions; RMS norm on q and k
    (`qk_norm`), value mixing with the first mixing layer (`v_mix`), sigmoid output gate (`out_gate`).

    `window` > 0: a query sees itself and the window - 1 positions before it.  `sink`: "none", "zero" (the softmax
    denominator gains exp(0) = 1) or "learned" (it gains exp(s_h), one number per head).  `norm_scope` "head": q and k are
    normalised head by head with one weight vector of size dim; "all": over the whole projection with weights of the
    projection's size.  `qk_bias`: the q and k projections have biases.  `values` "own": a value projection; "keys": the
    values are the keys as projected, before their norm (no value matrix; vdim == dim).  `gate_per_head`: the output
    gate is one number per head instead of one per output element.

    `keep_first` > 0 (with a window): the first positions of a sequence stay visible from every later query.
    `distance_bias` "slopes": the fixed per-head slopes above (True means the same); "log": r1_h ln(1 + r2_h (i - j)) with two
    learned numbers per head.  `rot`: rotary positions on q and k (a RotarySpec).  `norm_scope` "head" with
    `norm_weight` False divides q and k by their root mean square and multiplies by nothing.  `weights` "softmax", or
    "sigmoid": the weight of a visible key is sigmoid(score + b_h) with a learned number per head, not normalised.
    `qkv_bias`: the q, k and v projections have biases (added before the rotation).  `head_temp`: the score is also
    multiplied by a learned number per head."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    softcap: float = 0.0
    chunk: int = 0
    v_mix: bool = False
    qk_norm: bool = True
    out_gate: bool = True
    distance_bias: bool = True
    window: int = 0
    sink: str = "none"
    norm_scope: str = "head"
    qk_bias: bool = False
    values: str = "own"
    gate_per_head: bool = False
    keep_first: int = 0
    rot: "RotarySpec | None" = None
    norm_weight: bool = True
    weights: str = "softmax"
    qkv_bias: bool = False
    head_temp: bool = False

    kind = "attention"

    @property
    def gate_cols(self) -> int:
        return 0 if not self.out_gate else (self.heads if self.gate_per_head else self.heads * self.vdim)

    @property
    def proj_cols(self) -> int:
        """columns of the fused projection [q | k | v | gate]"""
        v = self.kv_heads * self.vdim if self.values == "own" else 0
        return self.heads * self.dim + self.kv_heads * self.dim + v + self.gate_cols

    @property
    def attn_cols(self) -> int:
        return self.heads * self.vdim

    def cache_shape(self) -> tuple[int, int, int]:
        """(key/value heads, key row size, value row size) of this mixer's cache pages"""
        return (self.kv_heads, self.dim, self.vdim)

    def slopes(self) -> list[float]:
        """slope of head h = 2^(-8 (h + 1) / H)"""
        return ([2.0 ** (-8.0 * (h + 1) / self.heads) for h in range(self.heads)]
                if self.distance_bias in (True, "slopes") else [])

    state_shapes = ()                    # no per-sequence state beside the cache pages


@dataclass(frozen=True)
class RotarySpec:
    """Rotary positions in the half layout: of the first `dims` elements of a head, element i is paired with element
    i + dims / 2 and the pair turns by position * base^(-2 i / dims) / factor (`factor`: linear position scaling)."""
    dims: int
    base: float
    factor: float = 1.0

    def inv_freq(self) -> list[float]:
        return [self.base ** (-2.0 * i / self.dims) / self.factor for i in range(self.dims // 2)]


@dataclass(frozen=True)
class LinearMixerSpec:
    """Linear attention with a fixed decay per head and a float32 state per sequence instead of cache pages:
    S_t = decay_h S_(t-1) + k_t v_t^T, o_t = S_t^T q_t; H heads, keys of size `dim`, values of size `vdim`.
    `activation` "silu" / "none" on q, k and v; `rot`: rotary positions on q and k; `k_scale` multiplies k after the
    rotation; `out_norm` "all": the heads' outputs are divided by their common root mean square and multiplied by a weight
    vector, "head": every head by its own, no weight; `gate` "sigmoid" / "silu" of a gate projection multiplies the result."""
    heads: int
    dim: int
    vdim: int
    decay: tuple
    activation: str = "none"
    rot: "RotarySpec | None" = None
    k_scale: float = 1.0
    out_norm: str = "head"
    gate: str = "sigmoid"

    kind = "linear_attention"
    kv_heads = 0
    chunk = 0
    window = 0
    keep_first = 0

    @property
    def proj_cols(self) -> int:
        """columns of the fused projection [q | k | v | gate]"""
        return 2 * self.heads * self.dim + 2 * self.heads * self.vdim

    @property
    def attn_cols(self) -> int:
        return self.heads * self.vdim

    def cache_shape(self) -> tuple[int, int, int]:
        return (0, 0, 0)                 # no cache pages

    @property
    def state_shapes(self) -> tuple:
        """float32 elements per sequence slot of every state array"""
        return (self.heads * self.dim * self.vdim,)


@dataclass(frozen=True)
class GatedLinearMixerSpec:
    """A linear recurrence that writes with the complement of its forget gate, with a float32 state per sequence:
    S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T, o_t = S_t^T q_t, per head; f_t = low + (1 - low) sigmoid(W_f h + b_f) per head
    and channel with a learned lower bound, q = silu(W_q h); there is no key.  Every head's output is divided by its root
    mean square and multiplied by a weight vector shared by the heads."""
    heads: int
    dim: int
    vdim: int

    kind = "gated_linear_attention"
    kv_heads = 0
    chunk = 0
    window = 0
    keep_first = 0

    @property
    def proj_cols(self) -> int:
        """columns of the fused projection [q | f | v]"""
        return 2 * self.heads * self.dim + self.heads * self.vdim

    @property
    def attn_cols(self) -> int:
        return self.heads * self.vdim

    def cache_shape(self) -> tuple[int, int, int]:
        return (0, 0, 0)                 # no cache pages

    @property
    def state_shapes(self) -> tuple:
        return (self.heads * self.dim * self.vdim,)


@dataclass(frozen=True)
class DeltaMixerSpec:
    """Gated delta rule with a float32 state per sequence: per head S <- g S; u = beta (v - S^T k); S <- S + k u^T;
    o = S^T q.  q and k have `qk_heads` heads of size `dim` (value head h reads head h // (heads / qk_heads)), v `heads` heads
    of size `vdim`; each passes a causal convolution over `conv_taps` positions per channel and SiLU; q and k are unit
    vectors (q times dim^-1/2); beta = sigmoid(W_b h), g = exp(-exp(A_log) softplus(W_a h + dt_bias)).  Every head's output
    is divided by its root mean square, multiplied by a weight vector shared by the heads and by silu of a gate projection.
    The last conv_taps - 1 inputs of the convolution are per-sequence state too (kept twice, see `CausalConvRows`)."""
    heads: int
    qk_heads: int
    dim: int
    vdim: int
    conv_taps: int

    kind = "delta_rule"
    kv_heads = 0
    chunk = 0
    window = 0
    keep_first = 0

    @property
    def conv_cols(self) -> int:
        """channels of the convolution: [q | k | v]"""
        return 2 * self.qk_heads * self.dim + self.heads * self.vdim

    @property
    def proj_cols(self) -> int:
        """columns of the fused projection [q | k | v | gate | beta | a]"""
        return self.conv_cols + self.heads * self.vdim + 2 * self.heads

    @property
    def attn_cols(self) -> int:
        return self.heads * self.vdim

    def cache_shape(self) -> tuple[int, int, int]:
        return (0, 0, 0)                 # no cache pages

    @property
    def state_shapes(self) -> tuple:
        return (self.heads * self.dim * self.vdim, 2 * max(0, self.conv_taps - 1) * self.conv_cols)


@dataclass(frozen=True)
class ParallelMixerSpec:
    """Two mixers side by side on the same input (an attention mixer with cache pages and a mixer with a state).  `join`
    "sum": left_scale * left + right_scale * right, one output projection over both sides' heads; "rms_mean": each side has
    its own output projection, whose result is divided by its root mean square over the width and multiplied by a weight
    vector, and the result is left_scale * left + right_scale * right of those (1/2 each for the mean)."""
    left: AttentionMixerSpec
    right: "LinearMixerSpec | GatedLinearMixerSpec"
    left_scale: float = 1.0
    right_scale: float = 1.0
    join: str = "sum"

    kind = "parallel"
    chunk = 0

    @property
    def heads(self) -> int:
        return self.left.heads

    @property
    def kv_heads(self) -> int:
        return self.left.kv_heads

    @property
    def window(self) -> int:
        return self.left.window

    @property
    def keep_first(self) -> int:
        return self.left.keep_first

    @property
    def proj_cols(self) -> int:
        return self.left.proj_cols + self.right.proj_cols

    @property
    def attn_cols(self) -> int:
        return self.left.attn_cols + self.right.attn_cols

    def cache_shape(self) -> tuple[int, int, int]:
        return self.left.cache_shape()

    @property
    def state_shapes(self) -> tuple:
        return self.right.state_shapes


@dataclass(frozen=True)
class LatentMixerSpec:
    """Latent attention: queries through a latent of size `q_rank` (0: projected directly), keys and values through one
    latent of size `kv_rank` per position plus `rot_dim` rotated key dimensions shared by the heads.  Per head `dim`
    unrotated + `rot_dim` rotated query/key dimensions and `vdim` value dimensions; the rotation turns the first
    `rot_dims` of the rotated part (interleaved pairs, base `rot_base`); causal; `sink` and the per-head gate as in
    AttentionMixerSpec.  Only the latent and the rotated key part are cached."""
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    q_rank: int
    scale: float
    rot_dims: int
    rot_base: float
    sink: str = "learned"
    out_gate: bool = True
    gate_per_head: bool = True

    kind = "latent_attention"
    kv_heads = 1
    chunk = 0
    window = 0
    keep_first = 0
    state_shapes = ()

    @property
    def gate_cols(self) -> int:
        return 0 if not self.out_gate else (self.heads if self.gate_per_head else self.heads * self.vdim)

    @property
    def proj_cols(self) -> int:
        """columns of the fused projection [query latent | key/value latent + rotated key | gate]"""
        return self.q_rank + self.kv_rank + self.rot_dim + self.gate_cols

    @property
    def attn_cols(self) -> int:
        """per token: the absorbed queries (and, later, the latent-space outputs) of all heads"""
        return self.heads * (self.kv_rank + self.rot_dim)

    def cache_shape(self) -> tuple[int, int, int]:
        return (1, self.kv_rank + self.rot_dim, 0)          # value rows are a prefix of the key rows

    def inv_freq(self) -> list[float]:
        """angle per position of pair i = rot_base^(-2 i / rot_dims)"""
        return [self.rot_base ** (-2.0 * i / self.rot_dims) for i in range(self.rot_dims // 2)]


@dataclass(frozen=True)
class DenseSpec:
    """Gated dense feed-forward: g = W_gate h, u = W_up h, output W_down act(g, u).  activation "silu": silu(g) u;
    "clamped_swish": g <- min(g, limit), u <- clamp(u, -limit, limit), g sigmoid(alpha g) (u + 1).  "relu2" has no gate:
    W_down max(W_up h, 0)^2.  "polynorm" has no gate either: W_down (a N(z) + b N(z^2) + c N(z^3) + e) with z = W_up h,
    powers element by element, N = division by the root mean square over the ff values, and four learned numbers."""
    ff: int
    activation: str = "silu"
    limit: float = 0.0
    alpha: float = 1.702

    kind = "dense"
    top = 1
    experts = 1
    shared_ff = 0


@dataclass(frozen=True)
class MoESpec:
    """Routed experts (gate/up/down, SiLU) + optional shared expert.  Router "grouped": softmax over all experts, the `top`
    best among the members of the `group_keep` best of `group_count` groups of neighbours, weights renormalised.  Router
    "biased": softmax over experts + identity router outputs, the `top` largest of score + a stored correction are chosen,
    the weights are the scores themselves (`renorm` False) -- the last `identity` outputs stand for experts that return
    their input and have no matrices; `shared_gate`: the shared expert's output is multiplied by sigmoid of one more
    projection, a number per token."""
    experts: int
    top: int
    ff: int
    group_count: int = 1
    group_keep: int = 1
    shared_ff: int = 0
    router: str = "grouped"
    identity: int = 0
    renorm: bool = True
    shared_gate: bool = False

    kind = "moe"

    @property
    def routes(self) -> int:
        """router outputs"""
        return self.experts + self.identity


@dataclass(frozen=True)
class LayerSpec:
    mixer: "AttentionMixerSpec | LatentMixerSpec | LinearMixerSpec | GatedLinearMixerSpec | DeltaMixerSpec | ParallelMixerSpec"
    mlp: "MoESpec | DenseSpec | None"


@dataclass
class LayeredConfig:
    """config.json of a layered model.  Every size is read from the file; nothing is assumed equal across layers
    except the width."""
    architecture: str
    vocab_size: int
    hidden_size: int
    layers: list[LayerSpec]
    norm_eps: float = 1e-5
    logit_scale: float = 1.0
    logit_softcap: float = 0.0
    # block form: "post_norm" x += LN(sublayer(x)) twice; "parallel" h = norm(x), x += s1 mixer(h) + s2 ff(h);
    # "pre_norm" x += m mixer(c1(norm1(x))), x += m ff(c2(norm2(x))) with m = residual_mult and c the input convolution;
    # "sandwich" x += norm1b(mixer(norm1(x))), x += norm2b(ff(norm2(x)))
    block: str = "post_norm"
    # "layernorm" (weight + bias), "layernorm_nobias", "rmsnorm_1p" (x / rms * (1 + w)) or "dyt" (tanh(alpha x) * w + b)
    norm: str = "layernorm"
    tied_head: bool = False            # the logits are products with the embedding table
    residual_mult: float = 1.0         # pre_norm blocks: factor on every sublayer's result before it joins the residual
    conv_taps: int = 0                 # > 0: h <- h + causal convolution over `conv_taps` positions in front of every sublayer
    embed_norm: bool = False           # the model's norm on the embedding output
    layer_scale: bool = False          # per-channel factors on the mixer's and the feed-forward's result
    side_dim: int = 0                  # > 0: a per-layer token input of this size after every layer
    # layers loop_start .. loop_stop - 1 run loop_times times in a row with the same weights (each pass with its own cache);
    # before every pass but the first the embedding output is added to the residual stream
    loop_start: int = 0
    loop_stop: int = 0
    loop_times: int = 1

    @property
    def num_layers(self) -> int:
        return len(self.layers)

    def layer_runs(self) -> list[tuple[int, bool]]:
        """The order in which layers run: (layer index, whether the embedding output is added first).  The position in
        this list names the run's cache."""
        n = len(self.layers)
        if self.loop_times <= 1 or self.loop_stop <= self.loop_start:
            return [(i, False) for i in range(n)]
        runs = [(i, False) for i in range(self.loop_start)]
        for t in range(self.loop_times):
            runs += [(i, t > 0 and i == self.loop_start) for i in range(self.loop_start, self.loop_stop)]
        return runs + [(i, False) for i in range(self.loop_stop, n)]


def _dolurax_config(d: dict) -> LayeredConfig:
    """Dolurax: post-sublayer LayerNorm blocks of chunked, distance-biased, gated attention and a grouped-router MoE."""
    layers = []
    for i, L in enumerate(d["layers"]):
        if L.get("type", "attention") != "attention":
            raise ValueError(f"Dolurax: layer {i} has unknown type {L.get('type')!r}")
        m = L["mixer"]
        mask = m.get("mask") or {}
        mixer = AttentionMixerSpec(heads=int(m["heads"]), kv_heads=int(m.get("kv_heads") or m["heads"]), dim=int(m["dim"]),
                                   vdim=int(m.get("vdim") or m["dim"]), scale=float(m["scale"]),
                                   softcap=float(m.get("softcap") or 0.0), chunk=int(mask.get("size") or 0),
                                   v_mix=bool(m.get("v_mix", False)))
        if mixer.heads % mixer.kv_heads:
            raise ValueError(f"Dolurax: layer {i}: {mixer.heads} heads over {mixer.kv_heads} key/value heads")
        mlp = None
        f = L.get("mlp")
        if f:
            if f.get("kind", "moe") != "moe":
                raise ValueError(f"Dolurax: layer {i} has unknown feed-forward kind {f.get('kind')!r}")
            r = f["router"]
            g = r.get("groups") or {}
            sh = f.get("shared") or {}
            mlp = MoESpec(experts=int(r["experts"]), top=int(r["top"]), ff=int(f["expert"]["ff"]),
                          group_count=int(g.get("count") or 1), group_keep=int(g.get("keep") or 1),
                          shared_ff=int(sh.get("ff") or 0))
            if mlp.experts % mlp.group_count:
                raise ValueError(f"Dolurax: layer {i}: {mlp.experts} experts do not split into {mlp.group_count} groups")
        layers.append(LayerSpec(mixer, mlp))
    return LayeredConfig(architecture="Dolurax", vocab_size=int(d["vocab"]), hidden_size=int(d["width"]), layers=layers,
                         norm_eps=float((d.get("norm") or {}).get("eps", 1e-5)), logit_scale=float(d.get("logit_scale") or 1.0),
                         logit_softcap=float(d.get("logit_softcap") or 0.0))


def _turutar_config(d: dict) -> LayeredConfig:
    """Turutar: parallel pre-norm blocks (one RMS norm with a weight stored around zero, mixer and feed-forward both read
    it, layer scales on both results) of windowed attention whose values are its keys, or latent attention with rotary
    positions; clamped gated feed-forward; a per-layer token input after every layer; an optional loop over a run of
    layers.  Constants the design fixes live here: the zero sink of the windowed mixer, the learned one of the latent
    mixer, per-head gates, alpha = 1.702."""
    W = int(d["width"])
    layers = []
    for i, L in enumerate(d["layers"]):
        m, kind = L["mixer"], L.get("type")
        if kind == "attention":
            heads, dim = int(m["heads"]), int(m["dim"])
            kv = int(m.get("kv_heads") or heads)
            vdim = int(m.get("vdim") or dim)
            if heads % kv:
                raise ValueError(f"Turutar: layer {i}: {heads} heads over {kv} key/value heads")
            if vdim != dim:
                raise ValueError(f"Turutar: layer {i}: the values are the keys, value size {vdim} must equal {dim}")
            mixer = AttentionMixerSpec(heads=heads, kv_heads=kv, dim=dim, vdim=vdim, scale=float(m["scale"]),
                                       window=int((m.get("mask") or {}).get("size") or 0), sink="zero", norm_scope="all",
                                       qk_bias=True, values="keys", gate_per_head=True, distance_bias=False)
        elif kind == "latent_attention":
            rot = m.get("rot") or {}
            rot_dim = int(m["rot_dim"])
            mixer = LatentMixerSpec(heads=int(m["heads"]), dim=int(m["dim"]), rot_dim=rot_dim, vdim=int(m["vdim"]),
                                    kv_rank=int(m["kv_rank"]), q_rank=int(m["q_rank"]), scale=float(m["scale"]),
                                    rot_dims=int(rot.get("dims", rot_dim)), rot_base=float(rot.get("base", 10000.0)))
            if mixer.rot_dims % 2 or mixer.rot_dims > rot_dim:
                raise ValueError(f"Turutar: layer {i}: {mixer.rot_dims} rotated dimensions in a part of {rot_dim}")
        else:
            raise ValueError(f"Turutar: layer {i} has unknown type {kind!r}")
        mlp = None
        f = L.get("mlp")
        if f:
            if f.get("kind") != "dense":
                raise ValueError(f"Turutar: layer {i} has unknown feed-forward kind {f.get('kind')!r}")
            mlp = DenseSpec(ff=int(f["ff"]), activation="clamped_swish", limit=float(f["limit"]))
        layers.append(LayerSpec(mixer, mlp))
    lp = d.get("loop") or {}
    start, stop, times = int(lp.get("start", 0)), int(lp.get("stop", 0)), int(lp.get("times", 1))
    if not 0 <= start <= stop <= len(layers) or times < 1:
        raise ValueError(f"Turutar: loop {start}..{stop} x {times} does not fit {len(layers)} layers")
    return LayeredConfig(architecture="Turutar", vocab_size=int(d["vocab"]), hidden_size=W, layers=layers,
                         norm_eps=float((d.get("norm") or {}).get("eps", 1e-6)), block="parallel", norm="rmsnorm_1p",
                         embed_norm=True, layer_scale=True, side_dim=int((d.get("token_side") or {}).get("dim") or 0),
                         loop_start=start, loop_stop=stop, loop_times=times)


def _rotary(rot: dict | None, dim: int, where: str) -> RotarySpec | None:
    if not rot:
        return None
    dims = int(rot.get("dims", dim))
    if dims % 2 or not 0 < dims <= dim:
        raise ValueError(f"{where}: {dims} rotated dimensions in heads of {dim}")
    return RotarySpec(dims=dims, base=float(rot.get("base", 10000.0)), factor=float((rot.get("scaling") or {}).get("factor", 1.0)))


def _rezulorn_config(d: dict) -> LayeredConfig:
    """Rezulorn: pre-norm blocks (LayerNorm without bias, a short causal convolution in front of every sublayer, one factor
    on every sublayer's result) of three mixers -- "lightning" (decayed linear attention on SiLU features, common output
    norm, sigmoid gate), "attention" (sliding window with kept first positions, logarithmic distance term, softmax) and
    "parallel" (sigmoid-weighted rotary attention with unit-norm q / k beside rotary retention with per-head output norm
    and SiLU gate) -- and a squared-ReLU feed-forward.  What the design fixes is set here; sizes and constants come from
    the file."""

    def heads_of(m, where):
        heads, dim = int(m["heads"]), int(m["dim"])
        kv = int(m.get("kv_heads") or heads)
        if heads < 1 or dim < 1 or heads % kv:
            raise ValueError(f"{where}: {heads} heads over {kv} key/value heads")
        return heads, kv, dim, int(m.get("vdim") or dim)

    def decays(m, heads, where):
        dec = tuple(float(v) for v in m["decay"])
        if len(dec) != heads:
            raise ValueError(f"{where}: {len(dec)} decays for {heads} heads")
        return dec

    layers = []
    for i, L in enumerate(d["layers"]):
        m, kind, where = L["mixer"], L.get("type"), f"Rezulorn: layer {i}"
        if kind == "lightning":
            heads, _, dim, vdim = heads_of(m, where)
            mixer = LinearMixerSpec(heads=heads, dim=dim, vdim=vdim, decay=decays(m, heads, where), activation="silu",
                                    out_norm="all", gate="sigmoid")
        elif kind == "attention":
            heads, kv, dim, vdim = heads_of(m, where)
            mask = m.get("mask") or {}
            window = int(mask.get("size") or 0)
            mixer = AttentionMixerSpec(heads=heads, kv_heads=kv, dim=dim, vdim=vdim, scale=float(m["scale"]), window=window,
                                       keep_first=int(mask.get("keep_first") or 0) if window > 0 else 0,   # no window: all visible
                                       qk_norm=False, out_gate=False, distance_bias="log")
        elif kind == "parallel":
            lm, rm = m["left"], m["right"]
            heads, kv, dim, vdim = heads_of(lm, where + " (left)")
            left = AttentionMixerSpec(heads=heads, kv_heads=kv, dim=dim, vdim=vdim, scale=float(lm["scale"]), qk_norm=True,
                                      norm_weight=False, out_gate=False, distance_bias=False,
                                      rot=_rotary(lm.get("rot"), dim, where + " (left)"), weights="sigmoid")
            heads, _, dim, vdim = heads_of(rm, where + " (right)")
            right = LinearMixerSpec(heads=heads, dim=dim, vdim=vdim, decay=decays(rm, heads, where + " (right)"),
                                    rot=_rotary(rm.get("rot"), dim, where + " (right)"), k_scale=dim ** -0.5, out_norm="head",
                                    gate="silu")
            mixer = ParallelMixerSpec(left, right, float(m.get("left_scale", 1.0)), float(m.get("right_scale", 1.0)))
        else:
            raise ValueError(f"{where} has unknown type {kind!r}")
        mlp = None
        f = L.get("mlp")
        if f:
            if f.get("kind") != "dense":
                raise ValueError(f"{where} has unknown feed-forward kind {f.get('kind')!r}")
            mlp = DenseSpec(ff=int(f["ff"]), activation="relu2")
        layers.append(LayerSpec(mixer, mlp))
    taps = int((d.get("canon") or {}).get("taps") or 0)
    if taps < 0:
        raise ValueError(f"Rezulorn: {taps} convolution taps")
    return LayeredConfig(architecture="Rezulorn", vocab_size=int(d["vocab"]), hidden_size=int(d["width"]), layers=layers,
                         norm_eps=float((d.get("norm") or {}).get("eps", 1e-6)), logit_scale=float(d.get("logit_scale") or 1.0),
                         block="pre_norm", norm="layernorm_nobias", residual_mult=float(d.get("residual_mult", 1.0)),
                         conv_taps=taps)


def _sumitar_config(d: dict) -> LayeredConfig:
    """Sumitar: sandwich blocks (a dynamic-tanh norm before and after every sublayer) of two mixers -- "parallel" (sliding-window
    rotary softmax attention with q / k / v biases and a per-head temperature beside a gated linear recurrence without keys,
    each side RMS-normed over the width, the mean of the two) and "delta" (gated delta rule behind short convolutions) -- with a
    PolyNorm feed-forward or a mixture of experts whose router has a choice bias, experts without matrices and a gated shared
    expert; the logits are products with the embedding table.  What the design fixes is set here; sizes and constants come
    from the file."""

    def sizes(m, where, kv_key="kv_heads"):
        heads, dim = int(m["heads"]), int(m["dim"])
        kv = int(m.get(kv_key) or heads)
        if heads < 1 or dim < 1 or kv < 1 or heads % kv:
            raise ValueError(f"{where}: {heads} heads over {kv} key/value heads")
        return heads, kv, dim, int(m.get("vdim") or dim)

    layers = []
    for i, L in enumerate(d["layers"]):
        m, kind, where = L["mixer"], L.get("type"), f"Sumitar: layer {i}"
        if kind == "parallel":
            lm, rm = m["left"], m["right"]
            heads, kv, dim, vdim = sizes(lm, where + " (left)")
            left = AttentionMixerSpec(heads=heads, kv_heads=kv, dim=dim, vdim=vdim, scale=float(lm["scale"]),
                                      window=int((lm.get("mask") or {}).get("size") or 0), qk_norm=False, out_gate=False,
                                      distance_bias=False, rot=_rotary(lm.get("rot"), dim, where + " (left)"), qkv_bias=True,
                                      head_temp=True)
            heads, _, dim, vdim = sizes(rm, where + " (right)")
            mixer = ParallelMixerSpec(left, GatedLinearMixerSpec(heads=heads, dim=dim, vdim=vdim), 0.5, 0.5, join="rms_mean")
        elif kind == "delta":
            heads, qk, dim, vdim = sizes(m, where)
            taps = int(m.get("conv") or 1)
            if taps < 1 or dim > 256:
                raise ValueError(f"{where}: {taps} convolution taps, heads of {dim}")
            mixer = DeltaMixerSpec(heads=heads, qk_heads=qk, dim=dim, vdim=vdim, conv_taps=taps)
        else:
            raise ValueError(f"{where} has unknown type {kind!r}")
        mlp = None
        f = L.get("mlp")
        if f:
            if f.get("kind") == "dense":
                mlp = DenseSpec(ff=int(f["ff"]), activation="polynorm")
            elif f.get("kind") == "moe":
                r = f["router"]
                sh = f.get("shared") or {}
                mlp = MoESpec(experts=int(r["experts"]), top=int(r["top"]), ff=int(f["expert"]["ff"]),
                              shared_ff=int(sh.get("ff") or 0), router="biased", identity=int(r.get("identity") or 0),
                              renorm=False, shared_gate=bool(sh.get("ff")))
                if mlp.experts < 0 or mlp.identity < 0 or not 1 <= mlp.top <= mlp.routes:
                    raise ValueError(f"{where}: top {mlp.top} of {mlp.experts} + {mlp.identity} experts")
            else:
                raise ValueError(f"{where} has unknown feed-forward kind {f.get('kind')!r}")
        layers.append(LayerSpec(mixer, mlp))
    return LayeredConfig(architecture="Sumitar", vocab_size=int(d["vocab"]), hidden_size=int(d["width"]), layers=layers,
                         norm_eps=float((d.get("norm") or {}).get("eps", 1e-6)), block="sandwich", norm="dyt", tied_head=True)


# config.json "architecture" -> parser (the model registry of the layered families)
LAYERED_ARCHITECTURES = {"dolurax": _dolurax_config, "turutar": _turutar_config, "rezulorn": _rezulorn_config,
                         "sumitar": _sumitar_config}


def layered_config_from_json(d: dict) -> LayeredConfig | None:
    """LayeredConfig when config.json names a layered architecture, else None (a uniform Hugging Face config)."""
    arch = str(d.get("architecture", "")).lower()
    return LAYERED_ARCHITECTURES[arch](d) if arch in LAYERED_ARCHITECTURES else None


__all__ = ["ModelSpec", "TransformerConfig", "GPT2Config", "LlamaConfig", "Qwen3Config", "GPT2_SPEC", "LLAMA_SPEC",
           "QWEN2_SPEC", "QWEN3_SPEC", "QWEN3_MOE_SPEC", "MIXTRAL_SPEC", "MODEL_SPECS", "detect_model_spec",
           "named_config", "AttentionMixerSpec", "LatentMixerSpec", "RotarySpec", "LinearMixerSpec", "GatedLinearMixerSpec", "DeltaMixerSpec", "ParallelMixerSpec", "DenseSpec", "MoESpec", "LayerSpec", "LayeredConfig",
           "LAYERED_ARCHITECTURES", "layered_config_from_json"]
