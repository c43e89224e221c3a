"""GPU tests of the Sumitar design in the layered family against the NumPy oracle tests/sumitar_ref.py: the new kernels alone
(dynamic-tanh norm, the join of two RMS-normed branches, PolyNorm, the router with a choice bias and experts without matrices,
the gated outer-product recurrence and the gated delta rule with their states, the short convolution with SiLU, the rotary
preparation with biases and a per-head temperature), then whole models under every schedule the step function admits, and
greedy generation through the scheduler and the command line.  Configurations are small and random; where random weights would
hide a fault (a key at the window's edge, a far key among hundreds, a state carried over many tokens) the inputs are made so
that it decides the answer.  float32 mode is held to 2e-4."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

import pygpukit_b200 as gk
from pygpukit_b200 import llm
from pygpukit_b200._lib import api
from pygpukit_b200.llm.config import layered_config_from_json
from pygpukit_b200.llm.paged_cache import PagedKVCache
from tests import sumitar_ref as R

pytestmark = pytest.mark.gpu

F32_TOL = 2e-4
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
_KEEP = []


def keep(g):
    """Park a device array until the test ends (kernels run asynchronously)."""
    _KEEP.append(g)
    return g


@pytest.fixture(autouse=True)
def _release_parked_arrays():
    yield
    gk.synchronize()
    _KEEP.clear()


def i32(a):
    return keep(gk.from_numpy(np.ascontiguousarray(a, np.int32)))


def f32(a):
    return keep(gk.from_numpy(np.ascontiguousarray(a, np.float32)))


def f64(a):
    return keep(gk.from_numpy(np.ascontiguousarray(a, np.float64)))


def cuts_of(sizes):
    at = [0]
    for n in sizes:
        at.append(at[-1] + n)
    return list(zip(at, at[1:]))


# ================================================================ kernels alone
@pytest.mark.parametrize("W", [5, 40, 300, 5000])
def test_dynamic_tanh_rows_gathered_and_accumulated(W):
    rng = np.random.default_rng(W)
    x, w, b = 2 * rng.standard_normal((9, W)), rng.standard_normal(W), rng.standard_normal(W)
    out = f32(np.ones((9, W)))
    api.dyt_rows_f32(f32(x).device_ptr, None, 0.7, f32(w).device_ptr, f32(b).device_ptr, out.device_ptr, 9, W, 1, None)
    assert np.abs(out.to_numpy() - (1 + R.dyt(x, 0.7, w, b))).max() < 1e-5
    rows = [7, 0, 7, 3]
    api.dyt_rows_f32(f32(x).device_ptr, i32(rows).device_ptr, 1.3, f32(w).device_ptr, None, out.device_ptr, 4, W, 0, None)
    assert np.abs(out.to_numpy()[:4] - R.dyt(x[rows], 1.3, w, 0.0)).max() < 1e-5


@pytest.mark.parametrize("W", [7, 256, 1111])
def test_two_branches_joined_after_their_rms_norms(W):
    rng = np.random.default_rng(W)
    a, b = 3 * rng.standard_normal((6, W)), 0.01 * rng.standard_normal((6, W))
    wa, wb = rng.standard_normal(W), rng.standard_normal(W)
    da = f32(a)
    api.rms_pair_rows_f32(da.device_ptr, f32(wa).device_ptr, f32(b).device_ptr, f32(wb).device_ptr, 1e-5, 0.5, da.device_ptr, 6, W,
                          None)                                          # in place on the first branch
    want = 0.5 * (R.unit_rms(a, 1e-5) * wa + R.unit_rms(b, 1e-5) * wb)
    assert np.abs(da.to_numpy() - want).max() < 1e-5


@pytest.mark.parametrize("n", [3, 64, 1000])
def test_polynomial_activation_with_a_norm_per_power(n):
    rng = np.random.default_rng(n)
    z, coef = 1.5 * rng.standard_normal((5, n)), np.array([0.7, -0.4, 0.25, 0.1])
    ld = n + 3
    buf = np.zeros((5, ld))
    buf[:, :n] = z
    d = f32(buf)
    api.polynorm_rows_f32(d.device_ptr, ld, f32(coef).device_ptr, 1e-6, 5, n, None)
    got = d.to_numpy()
    assert np.abs(got[:, :n] - R.polynorm(z, coef, 1e-6)).max() < 2e-5 and not got[:, n:].any()


@pytest.mark.parametrize("E,real,top,renorm", [(10, 8, 3, 0), (5, 5, 1, 0), (70, 60, 40, 1), (4, 0, 2, 0), (9, 8, 9, 1)])
def test_router_with_a_choice_bias_and_experts_without_matrices(E, real, top, renorm):
    rng = np.random.default_rng(E * 7 + top)
    T = 37
    z = np.zeros((T, E + 2))
    z[:, :E] = 2 * rng.standard_normal((T, E))
    z[:, E:] = 50.0                                                      # columns beyond the router's outputs are not its business
    bias = 0.3 * rng.standard_normal(E)
    idx, mat, wt = i32(np.zeros(T * top)), i32(np.zeros(T * top)), f32(np.zeros(T * top))
    rank, counts = i32(np.zeros(T * top)), i32(np.zeros(E))
    api.moe_route_biased(f32(z).device_ptr, E + 2, T, E, real, top, f32(bias).device_ptr, renorm, idx.device_ptr, mat.device_ptr,
                         wt.device_ptr, rank.device_ptr, counts.device_ptr, None)
    s = np.exp(z[:, :E] - z[:, :E].max(-1, keepdims=True))
    s /= s.sum(-1, keepdims=True)
    order = np.argsort(-(s + bias), axis=-1, kind="stable")[:, :top]
    want_w = np.take_along_axis(s, order, -1)
    if renorm:
        want_w = want_w / want_w.sum(-1, keepdims=True)
    got_i = idx.to_numpy().reshape(T, top)
    assert (got_i == order).all()
    assert (mat.to_numpy().reshape(T, top) == np.where(order < real, order, -1)).all()
    assert np.abs(wt.to_numpy().reshape(T, top) - want_w).max() < 1e-6
    assert (counts.to_numpy() == np.bincount(order.reshape(-1), minlength=E)).all()
    r = rank.to_numpy().reshape(-1)
    for e in range(E):                                                   # the ranks of an expert's rows are 0 .. count - 1
        assert sorted(r[got_i.reshape(-1) == e]) == list(range(int((order == e).sum())))


def test_weighted_sum_of_experts_own_rows_and_the_gated_shared_expert():
    rng = np.random.default_rng(3)
    T, W, top = 11, 50, 3
    parts, own, shared = rng.standard_normal((T * top, W)), rng.standard_normal((T, W)), rng.standard_normal((T, W))
    inv = rng.permutation(T * top)
    mat = rng.integers(-1, 4, T * top)
    mat[mat > 0] = 2
    w, gate = rng.uniform(0, 1, T * top), rng.standard_normal((T, 4))
    out = f32(np.zeros((T, W)))
    api.moe_combine_rows_f32(f32(parts).device_ptr, i32(inv).device_ptr, i32(mat).device_ptr, f32(w).device_ptr, top,
                             f32(own).device_ptr, f32(shared).device_ptr, f32(gate).device_ptr, 4, 3, out.device_ptr, T, W, None)
    want = R.sigmoid(gate[:, 3:4]) * shared
    for t in range(T):
        for k in range(top):
            o = t * top + k
            want[t] += w[o] * (own[t] if mat[o] < 0 else parts[inv[o]])
    assert np.abs(out.to_numpy() - want).max() < 1e-5
    api.moe_combine_rows_f32(f32(parts).device_ptr, i32(inv).device_ptr, None, f32(w).device_ptr, 1, None, None, None, 0, 0,
                             out.device_ptr, T, W, None)                # one expert per token, no shared expert
    assert np.abs(out.to_numpy() - w[:T, None] * parts[inv[:T]]).max() < 1e-5


class GatedHarness:
    """pgk_seq_gated_prep + pgk_seq_gated_recurrence + pgk_seq_linear_finish on raw rows [q | f | v]."""

    def __init__(self, H, D, Dv, slots=3, raw=False):
        self.H, self.D, self.Dv, self.raw = H, D, Dv, raw
        rng = np.random.default_rng(H * 13 + D)
        self.state = f32(7.0 * np.ones((slots, H * D * Dv)))            # dirty
        self.fb, self.low = rng.standard_normal(H * D), rng.uniform(0.0, 0.95, H * D)
        self.w = 1 + 0.2 * rng.standard_normal(Dv)
        self.pos = {}
        self.cols = 2 * H * D + H * Dv

    def run(self, batch):
        """batch: [(slot, q [n, H, D], f [n, H, D], v [n, H, Dv])] -> [n, H * Dv] per entry"""
        H, D, Dv = self.H, self.D, self.Dv
        rows = np.concatenate([np.concatenate([q.reshape(len(q), -1), f.reshape(len(q), -1), v.reshape(len(q), -1)], axis=1)
                               for _, q, f, v in batch])
        seqs, row = [], 0
        for s, q, _, _ in batch:
            p0 = self.pos.get(s, 0)
            seqs.append((row, len(q), s, p0))
            self.pos[s] = p0 + len(q)
            row += len(q)
        T = len(rows)
        proj, out = f32(rows), keep(gk.zeros((T, H * Dv), gk.float32))
        if not self.raw:
            api.seq_gated_prep(proj.device_ptr, self.cols, T, H, D, 0, H * D, f32(self.fb).device_ptr, f32(self.low).device_ptr, None)
        api.seq_gated_recurrence(0, proj.device_ptr, self.cols, 0, None, 0, 0, proj.device_ptr, self.cols, H * D, None, 0, 0,
                                 proj.device_ptr, self.cols, 2 * H * D, out.device_ptr, H * Dv, self.state.device_ptr,
                                 i32(seqs).device_ptr, len(seqs), H, H, D, Dv, None)
        if not self.raw:
            api.seq_linear_finish(out.device_ptr, H * Dv, None, 0, 0, f32(np.tile(self.w, H)).device_ptr, T, H, Dv, 1, 0, 1e-6, 1.0,
                                  None)
        o, at, res = out.to_numpy(), 0, []
        for _, q, _, _ in batch:
            res.append(o[at:at + len(q)])
            at += len(q)
        return res

    def oracle(self, q, f, v):
        T = len(q)
        if self.raw:
            return R.gated_outer_recurrence(q, f, v).reshape(T, -1)
        low = self.low.reshape(self.H, self.D)
        f = low + (1 - low) * R.sigmoid(f + self.fb.reshape(self.H, self.D))
        return (R.unit_rms(R.gated_outer_recurrence(R.silu(q), f, v), 1e-6) * self.w).reshape(T, -1)


GATED_LAYOUTS = [dict(H=3, D=8, Dv=6), dict(H=1, D=44, Dv=60), dict(H=2, D=70, Dv=9), dict(H=2, D=130, Dv=20), dict(H=5, D=16, Dv=33)]


@pytest.mark.parametrize("layout", GATED_LAYOUTS)
def test_gated_recurrence_whole_portions_and_single_tokens_agree_with_the_oracle(layout):
    h = GatedHarness(**layout)
    rng = np.random.default_rng(h.D)
    T = 75
    q, f, v = rng.standard_normal((T, h.H, h.D)), 2 * rng.standard_normal((T, h.H, h.D)), rng.standard_normal((T, h.H, h.Dv))
    ref = h.oracle(q, f, v)
    for s, sizes in enumerate([[T], [2] * 10 + [33, 1, 1, 20], [1] * 12 + [63]]):
        got = np.concatenate([h.run([(s % 3, q[a:b], f[a:b], v[a:b])])[0] for a, b in cuts_of(sizes)])
        assert np.abs(got - ref).max() < 2e-5, sizes
        h.pos.pop(s % 3)                                                 # the slot is used again from position 0, state dirty


def test_gated_recurrence_unequal_sequences_in_one_step():
    h = GatedHarness(2, 12, 10)
    rng = np.random.default_rng(5)
    data = [(rng.standard_normal((n, 2, 12)), rng.standard_normal((n, 2, 12)), rng.standard_normal((n, 2, 10))) for n in (40, 3, 17)]
    refs = [h.oracle(*d) for d in data]
    first = h.run([(s, q[:n], f[:n], v[:n]) for s, ((q, f, v), n) in enumerate(zip(data, (35, 1, 9)))])
    rest = h.run([(s, q[n:], f[n:], v[n:]) for s, ((q, f, v), n) in enumerate(zip(data, (35, 1, 9)))])
    for a, b, r in zip(first, rest, refs):
        assert np.abs(np.concatenate([a, b]) - r).max() < 2e-5


@pytest.mark.parametrize("decoded", [False, True])
def test_gated_recurrence_carries_one_early_token_over_hundreds(decoded):
    H, D, Dv, T, star = 2, 20, 12, 330, 4
    rng = np.random.default_rng(1)
    h = GatedHarness(H, D, Dv, raw=True)
    f = np.ones((T, H, D))                                               # everything is kept and nothing written ...
    f[star, :, 3] = 0.0                                                  # ... but one token writes channel 3 in full
    f[:, :, 5:] = rng.uniform(0.0, 0.5, (T, H, D - 5))                   # and the other channels forget fast
    q = np.zeros((T, H, D))
    q[:, :, 3] = 1.0
    v = rng.standard_normal((T, H, Dv))
    sizes = [star + 2] + [1] * (T - star - 2) if decoded else [100, 130, 100]
    got = np.concatenate([h.run([(0, q[a:b], f[a:b], v[a:b])])[0] for a, b in cuts_of(sizes)]).reshape(T, H, Dv)
    assert np.abs(got[:star]).max() == 0 and np.abs(got[star:] - v[star]).max() < 1e-6


class DeltaHarness:
    """pgk_causal_conv_rows_ex_f32 + pgk_seq_delta_prep + pgk_seq_gated_recurrence + pgk_seq_linear_finish on raw rows
    [q | k | v | gate | beta | a]."""

    def __init__(self, H, G, D, Dv, taps, slots=3):
        self.H, self.G, self.D, self.Dv, self.taps = H, G, D, Dv, taps
        rng = np.random.default_rng(H * 17 + D + taps)
        self.C = 2 * G * D + H * Dv
        self.cols = self.C + H * Dv + 2 * H
        self.cw = 0.6 * rng.standard_normal((self.C, taps))
        self.A_log, self.dt = np.log(rng.uniform(0.3, 3.0, H)), rng.uniform(-3, 0, H)
        self.w = 1 + 0.2 * rng.standard_normal(Dv)
        self.state = f32(7.0 * np.ones((slots, H * D * Dv)))            # dirty
        self.ring = f32(7.0 * np.ones((slots, 2 * max(1, taps - 1) * self.C)))
        self.pos, self.steps = {}, {}

    def run(self, batch):
        """batch: [(slot, rows [n, cols])]"""
        H, G, D, Dv, C = self.H, self.G, self.D, self.Dv, self.C
        rows = np.concatenate([r for _, r in batch])
        seqs, slot, pos, par, row = [], [], [], [], 0
        for s, r in batch:
            p0, n = self.pos.get(s, 0), len(r)
            seqs.append((row, n, s, p0))
            slot += [s] * n
            pos += list(range(p0, p0 + n))
            par += [self.steps.get(s, 0) & 1] * n
            self.pos[s], self.steps[s] = p0 + n, self.steps.get(s, 0) + 1
            row += n
        T = len(rows)
        proj, conv, out = f32(rows), keep(gk.zeros((T, C), gk.float32)), keep(gk.zeros((T, H * Dv), gk.float32))
        api.causal_conv_rows_ex_f32(proj.device_ptr, self.cols, conv.device_ptr, C, f32(self.cw).device_ptr,
                                    self.ring.device_ptr if self.taps > 1 else None, i32(slot).device_ptr, i32(pos).device_ptr,
                                    i32(par).device_ptr, T, C, self.taps, 0, 1, None)
        g_off = C
        b_off, a_off = g_off + H * Dv, g_off + H * Dv + H
        api.seq_delta_prep(conv.device_ptr, C, 0, G * D, proj.device_ptr, self.cols, b_off, a_off, f32(self.A_log).device_ptr,
                           f32(self.dt).device_ptr, T, H, G, D, D ** -0.5, None)
        api.seq_gated_recurrence(1, conv.device_ptr, C, 0, conv.device_ptr, C, G * D, proj.device_ptr, self.cols, a_off,
                                 proj.device_ptr, self.cols, b_off, conv.device_ptr, C, 2 * G * D, out.device_ptr, H * Dv,
                                 self.state.device_ptr, i32(seqs).device_ptr, len(seqs), H, G, D, Dv, None)
        api.seq_linear_finish(out.device_ptr, H * Dv, proj.device_ptr, self.cols, g_off, f32(np.tile(self.w, H)).device_ptr, T, H,
                              Dv, 1, 2, 1e-6, 1.0, None)
        o, at, res = out.to_numpy(), 0, []
        for _, r in batch:
            res.append(o[at:at + len(r)])
            at += len(r)
        return res

    def oracle(self, rows):
        H, G, D, Dv, C = self.H, self.G, self.D, self.Dv, self.C
        T = len(rows)
        c = R.silu(R.short_conv(rows[:, :C], self.cw))
        q, k, v = c[:, :G * D].reshape(T, G, D), c[:, G * D:2 * G * D].reshape(T, G, D), c[:, 2 * G * D:].reshape(T, H, Dv)
        q = q / np.sqrt((q * q).sum(-1, keepdims=True) + 1e-6) * D ** -0.5
        k = k / np.sqrt((k * k).sum(-1, keepdims=True) + 1e-6)
        q, k = np.repeat(q, H // G, axis=1), np.repeat(k, H // G, axis=1)
        gate = rows[:, C:C + H * Dv].reshape(T, H, Dv)
        beta = R.sigmoid(rows[:, C + H * Dv:C + H * Dv + H])
        g = np.exp(-np.exp(self.A_log) * R.softplus(rows[:, C + H * Dv + H:] + self.dt))
        o = R.unit_rms(R.delta_rule(q, k, v, beta, g), 1e-6) * self.w * R.silu(gate)
        return o.reshape(T, -1)


DELTA_LAYOUTS = [dict(H=4, G=2, D=8, Dv=6, taps=3), dict(H=1, G=1, D=60, Dv=28, taps=4), dict(H=3, G=3, D=70, Dv=9, taps=1),
                 dict(H=2, G=1, D=130, Dv=20, taps=2), dict(H=6, G=2, D=12, Dv=33, taps=5)]


@pytest.mark.parametrize("layout", DELTA_LAYOUTS)
def test_delta_rule_whole_portions_and_single_tokens_agree_with_the_oracle(layout):
    h = DeltaHarness(**layout)
    rng = np.random.default_rng(h.D)
    T = 70
    rows = rng.standard_normal((T, h.cols))
    ref = h.oracle(rows)
    for s, sizes in enumerate([[T], [2] * 10 + [28, 1, 1, 20], [1] * 9 + [61]]):
        got = np.concatenate([h.run([(s % 3, rows[a:b])])[0] for a, b in cuts_of(sizes)])
        assert np.abs(got - ref).max() < 5e-5, sizes
        h.pos.pop(s % 3)                                                 # the slot is used again from position 0: state and ring dirty


def test_delta_rule_unequal_sequences_in_one_step_and_a_reused_slot():
    h = DeltaHarness(4, 2, 10, 7, 4)
    rng = np.random.default_rng(9)
    data = [rng.standard_normal((n, h.cols)) for n in (30, 2, 11)]
    refs = [h.oracle(d) for d in data]
    cut = (25, 1, 4)
    first = h.run([(s, d[:n]) for s, (d, n) in enumerate(zip(data, cut))])
    rest = [[] for _ in data]
    for j in range(7):                                                   # then token by token, sequences ending at different steps
        live = [s for s, (d, n) in enumerate(zip(data, cut)) if n + j < len(d)]
        for s, o in zip(live, h.run([(s, data[s][cut[s] + j:cut[s] + j + 1]) for s in live])):
            rest[s].append(o)
    for a, b, r in zip(first, rest, refs):
        assert np.abs(np.concatenate([a] + b) - r).max() < 5e-5


def test_delta_rule_keeps_what_one_early_token_wrote():
    """One key direction is written once and never touched again: hundreds of tokens later a query along it still reads the value."""
    H, G, D, Dv, T, star = 2, 2, 16, 8, 300, 3
    h = DeltaHarness(H, G, D, Dv, 1)
    h.cw[:] = 1.0                                                        # one tap of weight 1: the convolution is the identity
    h.A_log[:], h.dt[:] = -30.0, -30.0                                   # g = 1: nothing decays
    rng = np.random.default_rng(2)
    rows = np.zeros((T, h.cols))
    C = h.C
    k = np.full((T, G, D), -20.0)                                        # silu(-20) ~ 0
    k[:, :, 1] = 20.0
    k[star, :, 1], k[star, :, 0] = -20.0, 20.0                           # the star's key is e0, everybody else's e1
    q = np.full((T, G, D), -20.0)
    q[:, :, 0] = 20.0                                                    # every query reads along e0
    v = rng.uniform(1.0, 2.0, (T, H, Dv))
    rows[:, :G * D], rows[:, G * D:2 * G * D], rows[:, 2 * G * D:C] = q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1)
    rows[:, C:C + H * Dv] = 1.0
    rows[:, C + H * Dv:C + H * Dv + H] = 30.0                            # beta = 1
    ref = h.oracle(rows)
    got = np.concatenate([h.run([(1, rows[a:b])])[0] for a, b in cuts_of([star + 2] + [1] * 40 + [T - star - 42])])
    assert np.abs(got - ref).max() < 5e-5
    want = R.unit_rms(R.silu(v[star]), 1e-6) * h.w * R.silu(1.0)         # the read-out of the star's value, normalised
    assert np.abs(got[star:].reshape(-1, H, Dv) - want).max() < 1e-3 and np.abs(got[:star]).max() < 1e-3


class AttentionHarness:
    """pgk_seq_mixer_prep_rot_ex + pgk_seq_attention_ex2 on raw rows [q | k | v] with biases and a per-head temperature."""

    def __init__(self, H, G, D, Dv, window, scale=0.3, page=4, dims=0, base=50.0, splits=1, bias=True):
        self.H, self.G, self.D, self.Dv, self.window, self.scale, self.dims, self.base, self.splits = H, G, D, Dv, window, scale, dims, base, splits
        self.cache = PagedKVCache([(G, D, Dv)], "float32", page, 64, 2)
        self.qt = api.seq_queries_per_tile(H, G)
        rng = np.random.default_rng(H * 31 + D)
        self.qb, self.kb, self.vb = (0.5 * rng.standard_normal(n) if bias else np.zeros(n) for n in (H * D, G * D, G * Dv))
        self.temp = rng.uniform(0.5, 2.0, H)
        self.inv_freq = [base ** (-2.0 * i / dims) for i in range(dims // 2)] if dims else []
        self.tickets = gk.zeros((4096,), gk.int32)
        self.cols = H * D + G * D + G * Dv

    def run(self, seq, q, k, v):
        n = q.shape[0]
        slot, pos0 = self.cache.extend(seq, n)
        self.cache.sync_table()
        c, H, G, D, Dv = self.cache, self.H, self.G, self.D, self.Dv
        proj = f32(np.concatenate([q.reshape(n, -1), k.reshape(n, -1), v.reshape(n, -1)], axis=1))
        api.seq_mixer_prep_rot_ex(proj.device_ptr, self.cols, n, H, G, D, Dv, 0, H * D, H * D + G * D, self.dims,
                                  f64(self.inv_freq).device_ptr if self.dims else None, 0, None, None, 1e-6, f32(self.qb).device_ptr,
                                  f32(self.kb).device_ptr, f32(self.vb).device_ptr, f32(self.temp).device_ptr, c.k[0].device_ptr,
                                  c.v[0].device_ptr, c.dtype_code, c.table_dev.device_ptr, c.pool.max_pages, c.page_size,
                                  i32([slot] * n).device_ptr, i32(np.arange(pos0, pos0 + n)).device_ptr, None)
        tiles = [(i, min(self.qt, n - i), slot, pos0 + i) for i in range(0, n, self.qt)]
        out = keep(gk.zeros((n, H * Dv), gk.float32))
        api.seq_attention_ex2(proj.device_ptr, self.cols, 0, None, 0, 0, 0, out.device_ptr, H * Dv, c.k[0].device_ptr,
                              c.v[0].device_ptr, D, Dv, c.dtype_code, c.table_dev.device_ptr, c.pool.max_pages, c.page_size,
                              i32(tiles).device_ptr, len(tiles), None, None, None, H, G, D, Dv, 0, self.window, 0, self.scale, 0.0, 0,
                              None, 1.0, self.splits, keep(gk.zeros((n * H * self.splits * (Dv + 2),), gk.float32)).device_ptr,
                              self.tickets.device_ptr, 1 if n == 1 else 0, None)
        return out.to_numpy().reshape(n, H, Dv)

    def oracle(self, q, k, v):
        T = len(q)
        q, k, v = q + self.qb.reshape(self.H, self.D), k + self.kb.reshape(self.G, self.D), v + self.vb.reshape(self.G, self.Dv)
        if self.dims:
            q, k = R.rotate_half(q, np.arange(T), self.dims, self.base), R.rotate_half(k, np.arange(T), self.dims, self.base)
        return R.window_softmax_attention(q, k, v, self.scale, self.temp, self.window)


ATTENTION_LAYOUTS = [dict(H=4, G=2, D=16, Dv=8, window=7, dims=8), dict(H=6, G=2, D=8, Dv=12, window=3, dims=8, page=3),
                     dict(H=3, G=3, D=12, Dv=20, window=100, dims=4), dict(H=2, G=1, D=40, Dv=72, window=33, dims=12, page=8),
                     dict(H=1, G=1, D=6, Dv=70, window=1, dims=0), dict(H=2, G=2, D=10, Dv=10, window=0, dims=10, bias=False)]


@pytest.mark.parametrize("layout", ATTENTION_LAYOUTS)
def test_attention_with_biases_and_temperature_agrees_with_the_oracle(layout):
    h = AttentionHarness(**layout)
    rng = np.random.default_rng(h.H * 7 + h.D)
    T = 45
    q, k, v = rng.standard_normal((T, h.H, h.D)), rng.standard_normal((T, h.G, h.D)), rng.standard_normal((T, h.G, h.Dv))
    ref = h.oracle(q, k, v)
    for name, sizes in (("whole", [T]), ("portions", [2, 2, 9, 1, 17, 14]), ("decoded", [5] + [1] * 40)):
        got = np.concatenate([h.run(name, q[a:b], k[a:b], v[a:b]) for a, b in cuts_of(sizes)])
        assert np.abs(got - ref).max() < 2e-5, name
        h.cache.release(name)


@pytest.mark.parametrize("decoded", [False, True])
@pytest.mark.parametrize("window,page", [(9, 4), (64, 16), (65, 64), (130, 64)])
def test_standout_key_just_inside_and_just_outside_the_window(window, page, decoded):
    """One key outweighs all others for every query: its value shows in exactly the `window` positions from its own on."""
    H, G, D, Dv = 2, 1, 8, 4
    for star in (0, 3, page - 1, page):
        T = star + window + 6
        rng = np.random.default_rng(star)
        q = np.zeros((T, H, D))
        q[:, :, 4] = 8.0
        k = 0.1 * rng.standard_normal((T, G, D))
        k[:, :, 4] = -1.0
        k[star, 0, 4] = 1.0
        v = 0.01 * rng.standard_normal((T, G, Dv))
        v[star, 0, 1] = 2.0
        h = AttentionHarness(H, G, D, Dv, window, scale=4.0, page=page, dims=4, bias=False)
        h.temp[:] = 1.0
        n0 = star + 1 if decoded else T - 3
        got = np.concatenate([h.run("a", q[:n0], k[:n0], v[:n0])] + [h.run("a", q[i:i + 1], k[i:i + 1], v[i:i + 1]) for i in range(n0, T)])
        assert np.abs(got - h.oracle(q, k, v)).max() < 1e-5
        for i in range(T):
            seen = 0 <= i - star < window
            assert (got[i, :, 1] > 1.9).all() == seen and ((got[i, :, 1] < 0.1).all() or seen), (star, i)


def test_short_convolution_with_silu_on_strided_rows():
    rng = np.random.default_rng(4)
    C, taps, ld = 300, 4, 310
    w = rng.standard_normal((C, taps))
    a, b = rng.standard_normal((23, ld)), rng.standard_normal((9, ld))
    ring = f32(7.0 * np.ones((2, 2 * (taps - 1) * C)))
    steps = {0: 0, 1: 0}
    pos = {0: 0, 1: 0}

    def run(batch):
        rows = np.concatenate([r for _, r in batch])
        slot = sum(([s] * len(r) for s, r in batch), [])
        p = sum((list(range(pos[s], pos[s] + len(r))) for s, r in batch), [])
        par = sum(([steps[s] & 1] * len(r) for s, r in batch), [])
        for s, r in batch:
            pos[s] += len(r)
            steps[s] += 1
        out = keep(gk.zeros((len(rows), C), gk.float32))
        api.causal_conv_rows_ex_f32(f32(rows).device_ptr, ld, out.device_ptr, C, f32(w).device_ptr, ring.device_ptr,
                                    i32(slot).device_ptr, i32(p).device_ptr, i32(par).device_ptr, len(rows), C, taps, 0, 1, None)
        return out.to_numpy()

    got_a, got_b = [], []
    o = run([(0, a[:2]), (1, b[:5])])
    got_a.append(o[:2]); got_b.append(o[2:])
    o = run([(1, b[5:6]), (0, a[2:3])])
    got_b.append(o[:1]); got_a.append(o[1:])
    o = run([(0, a[3:20]), (1, b[6:])])
    got_a.append(o[:17]); got_b.append(o[17:])
    for i in range(20, 23):
        got_a.append(run([(0, a[i:i + 1])]))
    assert np.abs(np.concatenate(got_a) - R.silu(R.short_conv(a[:, :C], w))).max() < 1e-5
    assert np.abs(np.concatenate(got_b) - R.silu(R.short_conv(b[:, :C], w))).max() < 1e-5


# ================================================================ whole models
def variants():
    """Sizes that the mechanisms must not assume equal or 1: key and value sizes, head counts on the two sides of a parallel
    mixer and between query/key and value heads of a delta mixer, rotated dimensions below the head size and equal to it, no
    rotation, a window of one, a window beyond the sequence and none at all, one tap and five, one chosen expert, no experts
    without matrices, more of them than real ones, no shared expert, layers without feed-forward, odd widths, every order of
    layers."""
    yield "base", R.make_config([R.parallel_layer(mlp=R.dense_ff()), R.delta_layer(mlp=R.moe_ff()), R.parallel_layer(mlp=R.moe_ff())])
    yield "delta_first", R.make_config([R.delta_layer(heads=6, kv_heads=2, dim=10, vdim=7, conv=2, mlp=R.dense_ff(31)),
                                        R.parallel_layer(heads=2, kv_heads=1, dim=16, vdim=4, dims=16, window=3, r_heads=3, r_dim=5,
                                                         r_vdim=9, mlp=R.moe_ff(experts=4, identity=0, top=1, ff=9, shared_ff=0)),
                                        R.delta_layer(heads=2, kv_heads=2, dim=20, vdim=20, conv=1)], vocab=61, width=52)
    yield "no_window", R.make_config([R.parallel_layer(heads=3, kv_heads=3, dim=10, vdim=10, dims=0, window=0, r_heads=1, r_dim=70,
                                                       r_vdim=12, mlp=R.moe_ff(experts=2, identity=3, top=4, ff=8, shared_ff=14)),
                                      R.delta_layer(heads=1, kv_heads=1, dim=6, vdim=40, conv=5, mlp=R.moe_ff(experts=40, identity=1, top=35))],
                                     width=36)
    yield "window_of_one", R.make_config([R.parallel_layer(window=1, mlp=None), R.parallel_layer(window=1000, dims=12, mlp=R.dense_ff(7))])


VARIANTS = dict(variants())


def config_of(cfg):
    d = json.loads(json.dumps(cfg))
    for L in d["layers"]:
        left = L["mixer"].get("left")
        if left and not left["rot"]["dims"]:
            del left["rot"]
    return d


def make(name, dtype="float32", page=4, seed=1, tokens_hint=64, slots=2):
    cfg = config_of(VARIANTS[name])
    P = R.random_params(cfg, seed=seed)
    m = llm.build_layered_model(layered_config_from_json(cfg), P, dtype)
    m.init_cache(tokens_hint, page_size=page, slots=slots)
    return cfg, P, m


def tokens(cfg, n, seed=0):
    return [int(t) for t in np.random.default_rng(seed).integers(0, cfg["vocab"], n)]


@pytest.mark.parametrize("name", list(VARIANTS))
def test_whole_prompt_and_every_layer_match_the_oracle_float32(name):
    cfg, P, m = make(name, tokens_hint=128)
    toks = tokens(cfg, 75)
    ref, layers = R.forward(cfg, P, toks, True)
    seen = []
    m.trace_hook = lambda run, x: seen.append(x)
    got = m.step([("a", toks, list(range(len(toks))))])
    assert len(seen) == len(layers)
    for run, (a, b) in enumerate(zip(seen, layers)):
        assert np.abs(a - b).max() < F32_TOL, run
    assert np.abs(got - ref).max() < F32_TOL


@pytest.mark.parametrize("name", list(VARIANTS))
def test_prefill_then_token_by_token_decoding(name):
    cfg, P, m = make(name)
    toks = tokens(cfg, 50, seed=3)
    ref = R.forward(cfg, P, toks)
    got = [m.step([("a", toks[:9], list(range(9)))])]
    got += [m.step([("a", [t], [0])]) for t in toks[9:]]                 # the windows pass over decoded tokens
    assert np.abs(np.concatenate(got) - ref).max() < F32_TOL


@pytest.mark.parametrize("name", ["base", "delta_first"])
def test_first_tokens_and_decoding_from_position_zero(name):
    cfg, P, m = make(name)
    toks = tokens(cfg, 12, seed=4)
    ref = R.forward(cfg, P, toks)
    got = np.concatenate([m.step([("a", [t], [0])]) for t in toks])
    assert np.abs(got - ref).max() < F32_TOL


@pytest.mark.parametrize("sizes", [[2] * 20, [3, 2, 7, 1, 11, 6, 10], [16, 24], [1, 39], [33, 3, 4]])
def test_prompt_portions(sizes):
    cfg, P, m = make("delta_first")
    toks = tokens(cfg, sum(sizes), seed=5)
    ref = R.forward(cfg, P, toks)
    got, at = [], 0
    for n in sizes:
        got.append(m.step([("a", toks[at:at + n], list(range(n)))]))
        at += n
    assert np.abs(np.concatenate(got) - ref).max() < F32_TOL


@pytest.mark.parametrize("name", ["base", "no_window"])
def test_batch_of_unequal_requests_equals_each_alone(name):
    cfg, P, m = make(name, tokens_hint=16)                               # small pool: pages and slots (with their state) grow
    lens, new = [1, 23, 7, 40], 6
    seqs = [tokens(cfg, n + new, seed=10 + i) for i, n in enumerate(lens)]
    refs = [R.forward(cfg, P, s) for s in seqs]
    got = m.step([(i, s[:n], list(range(n))) for i, (s, n) in enumerate(zip(seqs, lens))])
    assert np.abs(got - np.concatenate([r[:n] for r, n in zip(refs, lens)])).max() < F32_TOL
    for j in range(new):                                                 # request 0 ends after two more tokens
        live = [i for i in range(4) if i != 0 or j < 2]
        got = m.step([(i, [seqs[i][lens[i] + j]], [0]) for i in live], end=[0] if j == 1 else [])
        assert np.abs(got - np.stack([refs[i][lens[i] + j] for i in live])).max() < F32_TOL
    assert m.cache.pool.live_sequences == 3


def test_more_than_eight_decoding_requests():
    cfg, P, m = make("base", tokens_hint=256)
    seqs = [tokens(cfg, 5 + i, seed=30 + i) for i in range(11)]
    refs = [R.forward(cfg, P, s) for s in seqs]
    m.step([(i, s[:-2], []) for i, s in enumerate(seqs)])
    for back in (2, 1):
        got = m.step([(i, [s[-back]], [0]) for i, s in enumerate(seqs)])
        assert np.abs(got - np.stack([r[-back] for r in refs])).max() < F32_TOL


def test_pages_slots_and_state_are_used_again():
    cfg, P, m = make("base", page=4)
    a, b, c = tokens(cfg, 19, seed=20), tokens(cfg, 14, seed=21), tokens(cfg, 22, seed=22)
    m.step([("a", a, []), ("b", b[:6], [])])
    pages_a, slot_a = m.cache.pool.page_list("a"), m.cache.pool.slot("a")
    m.step([("b", b[6:], [])], end=["a"])
    got = m.step([("c", c[:13], list(range(13)))])                       # c inherits a's slot (dirty state and rings) and pages
    assert m.cache.pool.slot("c") == slot_a and set(m.cache.pool.page_list("c")) <= set(pages_a)
    got = np.concatenate([got] + [m.step([("c", [t], [0]), ("b", [1], [])])[:1] for t in c[13:]])
    assert np.abs(got - R.forward(cfg, P, c)).max() < F32_TOL
    m.release("c")
    got = np.concatenate([m.step([("d", [t], [0]), ("b", [2], [])])[:1] for t in c[:6]])      # and a sequence decoded from 0 in it
    assert np.abs(got - R.forward(cfg, P, c[:6])).max() < F32_TOL


def test_long_decoding_and_wanted_places_subset():
    cfg, P, m = make("base", page=8)
    toks = tokens(cfg, 170, seed=6)
    ref = R.forward(cfg, P, toks)
    want = [0, 6, 7, 8, 30, 69]
    got = m.step([("a", toks[:70], want)])
    assert np.abs(got - ref[want]).max() < F32_TOL
    got = np.concatenate([m.step([("a", [t], [0])]) for t in toks[70:]])
    assert np.abs(got - ref[70:]).max() < F32_TOL


@pytest.mark.parametrize("name", list(VARIANTS))
def test_bfloat16_mode_stays_within_bfloat16_rounding(name):
    cfg, P, m = make(name, dtype="bfloat16")
    toks = tokens(cfg, 40, seed=7)
    ref = R.forward(cfg, P, toks)
    whole = m.step([("a", toks, list(range(40)))])
    scale = np.abs(ref).max()
    assert np.abs(whole - ref).max() < 0.05 * scale
    got = np.concatenate([m.step([("b", toks[:20], list(range(20)))])] + [m.step([("b", [t], [0])]) for t in toks[20:]])
    assert np.abs(got - whole).max() < 0.05 * scale                      # the same sequence cut differently: rounding only


def test_a_sequence_with_state_cannot_be_cut_back():
    cfg, P, m = make("base")
    m.step([("a", tokens(cfg, 9), [])])
    with pytest.raises(ValueError, match="cut back"):
        m.cache.truncate("a", 5)


def test_greedy_generation_through_the_scheduler():
    cfg, P, m = make("base", tokens_hint=256)
    prompts = [tokens(cfg, n, seed=40 + n) for n in (3, 17, 9)]
    outs = m.generate(prompts, max_new_tokens=12, temperature=0.0, prefill_chunk=5)
    for p, o in zip(prompts, outs):
        assert o[:len(p)] == p and len(o) == len(p) + 12
        seq = list(p)
        for t in o[len(p):]:
            z = R.forward(cfg, P, seq)[-1]
            top2 = np.sort(z)[-2:]
            if top2[1] - top2[0] < 1e-3:                                 # a near tie: either token is right, stop comparing
                break
            assert t == int(np.argmax(z))
            seq.append(t)
    assert m.cache.pool.live_sequences == 0 and m.generate(prompts[0], 2) == outs[0][:len(prompts[0]) + 2]


def test_random_model_of_the_design_runs_in_bfloat16():
    cfg = layered_config_from_json(config_of(R.make_config([R.parallel_layer(heads=4, kv_heads=2, dim=32, vdim=32, dims=16, window=20,
                                                                              r_heads=2, r_dim=32, r_vdim=32, mlp=R.dense_ff(128)),
                                                            R.delta_layer(heads=4, kv_heads=2, dim=32, vdim=32, conv=4,
                                                                          mlp=R.moe_ff(experts=4, identity=1, top=2, ff=64, shared_ff=64))],
                                                           vocab=256, width=128)))
    m = llm.random_layered_model(cfg, "bfloat16", seed=3)
    m.init_cache(256)
    toks = tokens({"vocab": 256}, 60)
    whole = m.step([("a", toks, [58, 59])])
    m.step([("b", toks[:59], [])])
    one = m.step([("b", toks[59:], [0])])
    assert np.isfinite(whole).all() and np.abs(one - whole[1:]).max() < 0.05 * np.abs(whole).max()


def _save(cfg, P, folder):
    tensors = {k: ((np.ascontiguousarray(v, np.float32).view(np.uint32) >> 16).astype(np.uint16).reshape(v.shape), "BF16")
               for k, v in P.items()}
    llm.save_safetensors(os.path.join(folder, "model.safetensors"), tensors)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    return {k: (np.ascontiguousarray(v, np.float32).view(np.uint32) >> 16 << 16).view(np.float32) for k, v in P.items()}


def test_loader_picks_the_family_from_config_json(tmp_path):
    cfg = config_of(VARIANTS["delta_first"])
    P = _save(cfg, R.random_params(cfg, seed=8), str(tmp_path))
    m = llm.load_model_from_safetensors(str(tmp_path), dtype="float32")
    assert isinstance(m, llm.LayeredCausalModel) and m.config.architecture == "Sumitar"
    toks = tokens(cfg, 10)
    assert np.abs(m.step([("a", toks, list(range(10)))]) - R.forward(cfg, P, toks)).max() < F32_TOL
    with pytest.raises(ValueError, match="shape"):
        bad = dict(P)
        bad["l0.mix.q.conv"] = P["l0.mix.q.conv"][:-1]
        llm.build_layered_model(layered_config_from_json(cfg), bad, "float32")


def test_trace_replay_command_line(tmp_path):
    cfg = config_of(VARIANTS["base"])
    model_dir, out_dir = tmp_path / "model", tmp_path / "out"
    model_dir.mkdir()
    P = _save(cfg, R.random_params(cfg, seed=9), str(model_dir))
    a, b = tokens(cfg, 14, seed=1), tokens(cfg, 6, seed=2)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:11], "want": [0, 10]}, {"id": "b", "tokens": b[:5], "want": [4]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": [a[11]], "want": []}, {"id": "b", "tokens": [b[5]], "want": [0]}], "end": ["b"]},
             {"step": 2, "entries": [{"id": "a", "tokens": [a[12]], "want": [0]}], "end": []},
             {"step": 3, "entries": [{"id": "a", "tokens": [a[13]], "want": [0]}], "end": ["a"]}]
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", str(model_dir), "--dtype", "float32",
                        "--out", str(out_dir), "--max-tokens", "64"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [ln for ln in r.stdout.splitlines() if ln.startswith("done")] == [f"done {i}" for i in range(4)]
    ra, rb = R.forward(cfg, P, a), R.forward(cfg, P, b)
    V = cfg["vocab"]
    got0 = np.fromfile(out_dir / "0.f32", "<f4").reshape(-1, V)
    assert np.abs(got0 - np.stack([ra[0], ra[10], rb[4]])).max() < F32_TOL
    assert np.abs(np.fromfile(out_dir / "1.f32", "<f4").reshape(-1, V) - rb[5:6]).max() < F32_TOL
    assert np.abs(np.fromfile(out_dir / "3.f32", "<f4").reshape(-1, V) - ra[13:14]).max() < F32_TOL
