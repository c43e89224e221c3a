"""CPU tests of the Rezulorn design: config parsing and registry (every size different, rejections), the state the cache
manager is asked for, and the oracle's own mechanisms on hand-made cases where the answer is known in closed form."""
import numpy as np
import pytest

from pygpukit_b200.llm.config import (AttentionMixerSpec, LinearMixerSpec, ParallelMixerSpec, LAYERED_ARCHITECTURES,
                                      layered_config_from_json)
from tests import rezulorn_ref as R


def test_config_reads_every_size_and_constant_from_the_file():
    cfg = R.make_config([R.parallel_layer(heads=6, kv_heads=3, dim=10, vdim=14, dims=6, base=777.0, factor=3.0, scale=0.21, r_heads=5,
                                          r_dim=12, r_vdim=7, r_dims=8, r_base=55.0, left_scale=1.7, right_scale=0.3, ff=50),
                         R.lightning_layer(heads=2, dim=9, vdim=11, decay=[0.5, 0.75], ff=0),
                         R.attention_layer(heads=8, kv_heads=2, dim=6, vdim=5, window=13, keep=3, scale=0.4, ff=31)],
                        vocab=77, width=44, taps=5, eps=3e-6, residual_mult=0.6, logit_scale=0.125)
    c = layered_config_from_json(cfg)
    assert "rezulorn" in LAYERED_ARCHITECTURES and c.architecture == "Rezulorn"
    assert (c.vocab_size, c.hidden_size, c.conv_taps, c.norm_eps, c.residual_mult, c.logit_scale) == (77, 44, 5, 3e-6, 0.6, 0.125)
    assert c.block == "pre_norm" and c.norm == "layernorm_nobias" and c.layer_runs() == [(0, False), (1, False), (2, False)]
    p, l, a = (L.mixer for L in c.layers)
    assert isinstance(p, ParallelMixerSpec) and (p.left_scale, p.right_scale) == (1.7, 0.3)
    assert (p.left.heads, p.left.kv_heads, p.left.dim, p.left.vdim, p.left.scale) == (6, 3, 10, 14, 0.21)
    assert (p.left.rot.dims, p.left.rot.base, p.left.rot.factor) == (6, 777.0, 3.0) and p.left.weights == "sigmoid"
    assert p.left.qk_norm and not p.left.norm_weight and not p.left.out_gate and p.left.window == 0
    assert (p.right.heads, p.right.dim, p.right.vdim, p.right.rot.dims, p.right.rot.base, p.right.rot.factor) == (5, 12, 7, 8, 55.0, 1.0)
    assert p.right.k_scale == 12 ** -0.5 and p.right.out_norm == "head" and p.right.gate == "silu" and p.right.activation == "none"
    assert p.proj_cols == (6 * 10 + 3 * 10 + 3 * 14) + (2 * 5 * 12 + 2 * 5 * 7) and p.attn_cols == 6 * 14 + 5 * 7
    assert p.cache_shape() == (3, 10, 14) and p.state_shapes == (5 * 12 * 7,)
    assert isinstance(l, LinearMixerSpec) and l.decay == (0.5, 0.75) and l.activation == "silu" and l.out_norm == "all"
    assert l.gate == "sigmoid" and l.rot is None and l.k_scale == 1.0 and l.cache_shape() == (0, 0, 0) and l.state_shapes == (2 * 9 * 11,)
    assert isinstance(a, AttentionMixerSpec) and (a.window, a.keep_first, a.distance_bias, a.weights) == (13, 3, "log", "softmax")
    assert not a.qk_norm and a.rot is None and a.slopes() == [] and a.state_shapes == ()
    assert c.layers[1].mlp is None and c.layers[2].mlp.activation == "relu2" and c.layers[2].mlp.ff == 31
    assert p.left.rot.inv_freq() == pytest.approx([777.0 ** (-2.0 * i / 6) / 3.0 for i in range(3)])


@pytest.mark.parametrize("change,match", [
    (lambda c: c["layers"][0].update(type="conv"), "unknown type"),
    (lambda c: c["layers"][0]["mixer"]["left"].update(kv_heads=3), "key/value heads"),
    (lambda c: c["layers"][0]["mixer"]["left"]["rot"].update(dims=7), "rotated dimensions"),
    (lambda c: c["layers"][0]["mixer"]["right"]["rot"].update(dims=40), "rotated dimensions"),
    (lambda c: c["layers"][1]["mixer"].update(decay=[0.5]), "decays"),
    (lambda c: c["layers"][1]["mlp"].update(kind="moe"), "feed-forward kind"),
])
def test_config_rejections(change, match):
    cfg = R.make_config([R.parallel_layer(), R.lightning_layer()])
    change(cfg)
    with pytest.raises(ValueError, match=match):
        layered_config_from_json(cfg)


def test_oracle_input_convolution_on_an_impulse():
    w = np.array([[1.0, 2.0, 3.0, 4.0], [0.5, 0.0, -1.0, 2.0]])          # [channels, taps]; the last tap meets the token itself
    h = np.zeros((6, 2))
    h[1] = [1.0, 10.0]
    out = R.input_conv(h, w)
    assert np.allclose(out[:, 0], [0, 1 + 4, 3, 2, 1, 0]) and np.allclose(out[:, 1], [0, 10 + 20, -10, 0, 5, 0])
    assert np.allclose(R.input_conv(h[:2], w), out[:2])                  # causal: later tokens change nothing before them


def test_oracle_decayed_state_in_closed_form():
    T, a = 9, 0.8
    q, k, v = np.ones((T, 1, 2)), np.ones((T, 1, 2)), np.ones((T, 1, 3))
    o = R.decayed_linear_attention(q, k, v, [a])
    assert np.allclose(o[:, 0, 0], [2 * (1 - a ** (t + 1)) / (1 - a) for t in range(T)])
    assert np.allclose(R.decayed_linear_attention(q, k, v, [1.0])[:, 0, 1], 2 * np.arange(1, T + 1))


def test_oracle_mask_keeps_the_first_positions_and_the_window():
    m = R.keep_first_window_mask(10, window=3, keep=2)
    assert m[9].tolist() == [True, True, False, False, False, False, False, True, True, True]
    assert m[2].tolist() == [True, True, True] + [False] * 7 and not np.triu(m, 1).any()
    assert np.array_equal(R.keep_first_window_mask(6, 0, 0), np.tril(np.ones((6, 6), bool)))


def test_oracle_rotation_pairs_halves_keeps_the_rest_and_preserves_inner_products():
    x = np.arange(1.0, 7.0).reshape(1, 1, 6)
    r = R.rotate_half(np.repeat(x, 3, 0), [0, 1, 2], dims=4, base=100.0, factor=2.0)
    assert np.allclose(r[0], x[0]) and np.allclose(r[:, 0, 4:], [[5.0, 6.0]] * 3)
    ang = 1.0 / 2.0                                                      # position 1, pair 0: elements 0 and 2
    assert np.allclose(r[1, 0, [0, 2]], [1 * np.cos(ang) - 3 * np.sin(ang), 3 * np.cos(ang) + 1 * np.sin(ang)])
    rng = np.random.default_rng(0)
    a, b = rng.standard_normal((1, 1, 8)), rng.standard_normal((1, 1, 8))
    d1 = (R.rotate_half(a, [7], 8, 50.0) * R.rotate_half(b, [4], 8, 50.0)).sum()
    d2 = (R.rotate_half(a, [13], 8, 50.0) * R.rotate_half(b, [10], 8, 50.0)).sum()
    assert abs(d1 - d2) < 1e-12                                          # only the distance matters


def test_oracle_sigmoid_weights_add_up_without_normalisation():
    T = 5
    q, k = np.zeros((T, 1, 2)), np.zeros((T, 1, 2))
    v = np.ones((T, 1, 1))
    o = R.sigmoid_attention(q, k, v, 1.0, [0.0])
    assert np.allclose(o[:, 0, 0], 0.5 * np.arange(1, T + 1))


def test_oracle_forward_is_causal_and_layers_are_reported():
    cfg = R.make_config([R.parallel_layer(), R.lightning_layer(), R.attention_layer()])
    P = R.random_params(cfg, seed=3)
    toks = [int(t) for t in np.random.default_rng(1).integers(0, cfg["vocab"], 20)]
    full, layers = R.forward(cfg, P, toks, True)
    assert layers.shape == (3, 20, cfg["width"]) and np.allclose(R.forward(cfg, P, toks[:11]), full[:11])
