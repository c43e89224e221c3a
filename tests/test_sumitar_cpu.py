"""CPU tests of the Sumitar design: config parsing and registry (every size different, rejections), the state the cache
manager is asked for, and the oracle's own mechanisms on hand-made cases where the answer is known in closed form."""
import numpy as np
import pytest

from pygpukit_b200.llm.config import (AttentionMixerSpec, DeltaMixerSpec, GatedLinearMixerSpec, ParallelMixerSpec,
                                      LAYERED_ARCHITECTURES, layered_config_from_json)
from tests import sumitar_ref as R


def test_config_reads_every_size_and_constant_from_the_file():
    cfg = R.make_config([R.parallel_layer(heads=6, kv_heads=3, dim=10, vdim=14, dims=6, base=777.0, scale=0.21, window=13, r_heads=5,
                                          r_dim=12, r_vdim=7, mlp=R.dense_ff(50)),
                         R.delta_layer(heads=8, kv_heads=2, dim=9, vdim=11, conv=5, mlp=R.moe_ff(experts=7, identity=3, top=4, ff=21, shared_ff=33)),
                         R.delta_layer(heads=2, kv_heads=2, dim=4, vdim=4, conv=1, mlp=R.moe_ff(experts=3, identity=0, top=1, ff=5, shared_ff=0))],
                        vocab=77, width=44, eps=3e-6)
    c = layered_config_from_json(cfg)
    assert "sumitar" in LAYERED_ARCHITECTURES and c.architecture == "Sumitar"
    assert (c.vocab_size, c.hidden_size, c.norm_eps, c.block, c.norm, c.tied_head) == (77, 44, 3e-6, "sandwich", "dyt", True)
    assert c.layer_runs() == [(0, False), (1, False), (2, False)]
    p, d, d2 = (L.mixer for L in c.layers)
    assert isinstance(p, ParallelMixerSpec) and p.join == "rms_mean" and (p.left_scale, p.right_scale) == (0.5, 0.5)
    a, r = p.left, p.right
    assert isinstance(a, AttentionMixerSpec) and (a.heads, a.kv_heads, a.dim, a.vdim, a.scale, a.window) == (6, 3, 10, 14, 0.21, 13)
    assert (a.rot.dims, a.rot.base, a.rot.factor) == (6, 777.0, 1.0) and a.qkv_bias and a.head_temp and a.weights == "softmax"
    assert not a.qk_norm and not a.out_gate and a.sink == "none" and a.keep_first == 0 and a.slopes() == []
    assert isinstance(r, GatedLinearMixerSpec) and (r.heads, r.dim, r.vdim) == (5, 12, 7)
    assert p.proj_cols == (6 * 10 + 3 * 10 + 3 * 14) + (2 * 5 * 12 + 5 * 7) and p.attn_cols == 6 * 14 + 5 * 7
    assert p.cache_shape() == (3, 10, 14) and p.state_shapes == (5 * 12 * 7,)
    assert isinstance(d, DeltaMixerSpec) and (d.heads, d.qk_heads, d.dim, d.vdim, d.conv_taps) == (8, 2, 9, 11, 5)
    assert d.conv_cols == 2 * 2 * 9 + 8 * 11 and d.proj_cols == d.conv_cols + 8 * 11 + 16 and d.cache_shape() == (0, 0, 0)
    assert d.state_shapes == (8 * 9 * 11, 2 * 4 * d.conv_cols) and d2.state_shapes == (2 * 4 * 4, 0)
    f0, f1, f2 = (L.mlp for L in c.layers)
    assert (f0.kind, f0.ff, f0.activation) == ("dense", 50, "polynorm")
    assert (f1.experts, f1.identity, f1.routes, f1.top, f1.ff, f1.shared_ff) == (7, 3, 10, 4, 21, 33)
    assert f1.router == "biased" and not f1.renorm and f1.shared_gate
    assert (f2.experts, f2.identity, f2.top, f2.shared_ff, f2.shared_gate) == (3, 0, 1, 0, False)


def test_config_without_a_window_or_a_rotation():
    cfg = R.make_config([R.parallel_layer(window=0)])
    del cfg["layers"][0]["mixer"]["left"]["rot"]
    a = layered_config_from_json(cfg).layers[0].mixer.left
    assert a.window == 0 and a.rot is None and layered_config_from_json(cfg).layers[0].mlp is None


@pytest.mark.parametrize("change,match", [
    (lambda c: c["layers"][0].update(type="conv"), "unknown type"),
    (lambda c: c["layers"][0]["mixer"]["left"].update(kv_heads=3), "key/value heads"),
    (lambda c: c["layers"][0]["mixer"]["left"]["rot"].update(dims=7), "rotated dimensions"),
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=3), "key/value heads"),
    (lambda c: c["layers"][1]["mixer"].update(dim=300), "heads of 300"),
    (lambda c: c["layers"][1]["mlp"].update(kind="gated"), "feed-forward kind"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=9), "top 9"),
])
def test_config_rejections(change, match):
    cfg = R.make_config([R.parallel_layer(), R.delta_layer(mlp=R.moe_ff())])
    change(cfg)
    with pytest.raises(ValueError, match=match):
        layered_config_from_json(cfg)


def test_oracle_short_convolution_on_an_impulse():
    w = np.array([[1.0, 2.0, 3.0, 4.0], [0.5, 0.0, -1.0, 2.0]])          # [channels, taps]; the last tap meets the token itself
    h = np.zeros((6, 2))
    h[1] = [1.0, 10.0]
    out = R.short_conv(h, w)
    assert np.allclose(out[:, 0], [0, 4, 3, 2, 1, 0]) and np.allclose(out[:, 1], [0, 20, -10, 0, 5, 0])
    assert np.allclose(R.short_conv(h[:2], w), out[:2])                  # causal: later tokens change nothing before them


def test_oracle_gated_outer_recurrence_in_closed_form():
    T = 5
    q, v = np.ones((T, 1, 2)), np.arange(1.0, T + 1).reshape(T, 1, 1)
    f = np.full((T, 1, 2), 0.5)
    f[:, :, 1] = 1.0                                                     # a channel that keeps everything writes nothing
    o = R.gated_outer_recurrence(q, f, v)[:, 0, 0]
    want, s = [], 0.0
    for t in range(T):
        s = 0.5 * s + 0.5 * (t + 1)
        want.append(s)
    assert np.allclose(o, want)


def test_oracle_delta_rule_overwrites_along_a_key_and_leaves_the_rest():
    e0, e1 = np.array([1.0, 0.0, 0.0]), np.array([0.0, 1.0, 0.0])
    k = np.stack([e0, e1, e0, e1])[:, None, :]
    v = np.array([[1.0], [2.0], [3.0], [4.0]])[:, None, :]
    ones = np.ones((4, 1))
    assert np.allclose(R.delta_rule(k, k, v, ones, ones)[:, 0, 0], [1, 2, 3, 4])         # beta 1: the value along a key is replaced
    o = R.delta_rule(np.stack([e0] * 4)[:, None, :], k, v, ones, ones)[:, 0, 0]
    assert np.allclose(o, [1, 1, 3, 3])                                                   # writes along e1 leave e0 alone
    o = R.delta_rule(np.stack([e0] * 4)[:, None, :], k, v, 0.5 * ones, 0.5 * ones)[:, 0, 0]
    assert np.allclose(o, [0.5, 0.25, 0.125 + 0.5 * (3 - 0.125), (0.125 + 0.5 * (3 - 0.125)) * 0.5])


def test_oracle_window_and_router():
    T = 6
    q = np.zeros((T, 1, 2))
    k = np.zeros((T, 1, 2))
    v = np.arange(1.0, T + 1).reshape(T, 1, 1)
    o = R.window_softmax_attention(q, k, v, 1.0, [1.0], 2)[:, 0, 0]      # equal scores: the mean of the visible values
    assert np.allclose(o, [1, 1.5, 2.5, 3.5, 4.5, 5.5])
    o = R.window_softmax_attention(q, k, v, 1.0, [1.0], 0)[:, 0, 0]
    assert np.allclose(o, [1, 1.5, 2, 2.5, 3, 3.5])
    h = np.array([[1.0, 0.0]])
    router = np.array([[0.0, 0.0], [1.0, 0.0], [2.0, 0.0]])
    chosen, w = R.route(h, router, np.array([0.0, 5.0, 0.0]), 2)         # the correction changes the choice, not the weight
    s = np.exp([0.0, 1.0, 2.0]) / np.exp([0.0, 1.0, 2.0]).sum()
    assert list(chosen[0]) == [1, 2] and np.allclose(w[0], [s[1], s[2]])


def test_oracle_model_is_causal_and_identity_experts_return_their_input():
    cfg = R.make_config([R.parallel_layer(mlp=R.dense_ff()), R.delta_layer(mlp=R.moe_ff())])
    P = R.random_params(cfg, seed=3)
    toks = [int(t) for t in np.random.default_rng(0).integers(0, cfg["vocab"], 20)]
    full = R.forward(cfg, P, toks)
    assert np.allclose(R.forward(cfg, P, toks[:11]), full[:11])
    f = R.moe_ff(experts=0, identity=2, top=2, shared_ff=0)
    h = np.random.default_rng(1).standard_normal((4, cfg["width"]))
    Q = {"m.router": P["l1.mlp.router"][:2], "m.correction": np.zeros(2)}
    assert np.allclose(R.feed_forward(h, Q, "m.", f, 1e-6), h)           # both experts return h and the weights sum to one
