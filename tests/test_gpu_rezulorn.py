"""GPU tests of the Rezulorn design in the layered family against the NumPy oracle tests/rezulorn_ref.py: the new kernels
alone (input convolution with its ring, decayed linear attention with its state, rotary preparation, attention with kept
first positions, the logarithmic distance term and sigmoid weights, the squared-ReLU epilogue, LayerNorm without bias), then
whole models under every schedule the step function admits, and greedy generation through the scheduler and the command
line.  Configurations are small and random; where random weights would hide a fault (a key at the window's edge, a kept
first position, a far key among hundreds, a state carried over many tokens) the inputs are made so that it decides the
answer.  float32 mode is held to 2e-4."""
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
from tests import rezulorn_ref as R

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


def bf16_round(a):
    u = np.ascontiguousarray(a, np.float32).view(np.uint32)
    return (((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16).astype(np.uint32).view(np.float32)


def dev_w(a, wdt):
    a = np.ascontiguousarray(a, np.float32)
    return keep(gk.from_numpy((a.view(np.uint32) >> 16).astype(np.uint16).reshape(a.shape)) if wdt == 2 else gk.from_numpy(a))


def cuts_of(sizes):
    at = [0]
    for n in sizes:
        at.append(at[-1] + n)
    return list(zip(at, at[1:]))


# ================================================================ kernels alone
@pytest.mark.parametrize("wdt", [0, 2])
@pytest.mark.parametrize("M", [3, 70])
def test_gemm_squared_relu_epilogue(M, wdt):
    rng = np.random.default_rng(M + wdt)
    K, N = 44, 13
    x = rng.standard_normal((M, K)).astype(np.float32)
    w = bf16_round(rng.standard_normal((N, K)) / 3)
    out = gk.zeros((M, N), gk.float32)
    api.gemm_seq_f32(f32(x).device_ptr, K, 0, dev_w(w, wdt).device_ptr, wdt, 0, out.device_ptr, N, 0, M, N, K, 1, 6, 0.0, 0.0, None,
                     None, 0, None, 0, 0, 8 if M <= 8 else 0, None)
    xr = bf16_round(x) if wdt == 2 else x
    assert np.abs(out.to_numpy() - np.maximum(xr.astype(np.float64) @ w.T, 0.0) ** 2).max() < 2e-5


@pytest.mark.parametrize("W", [40, 1030])
def test_layer_norm_without_bias(W):
    rng = np.random.default_rng(W)
    x, w = 3.0 + rng.standard_normal((5, W)), 1 + 0.2 * rng.standard_normal(W)
    out = gk.zeros((5, W), gk.float32)
    api.combine_layernorm_f32(f32(x).device_ptr, None, None, None, None, 0, f32(w).device_ptr, None, 1e-5, out.device_ptr, 5, W, 0, None)
    assert np.abs(out.to_numpy() - R.layer_norm(x, w, 1e-5)).max() < 1e-5


class ConvHarness:
    def __init__(self, W, taps, slots=3):
        rng = np.random.default_rng(W + taps)
        self.W, self.taps = W, taps
        self.w = rng.standard_normal((W, taps))
        # the rings start dirty: a sequence that begins in a slot must not see what the slot held
        self.state = f32(50.0 * np.ones((slots, max(1, taps - 1) * W)))
        self.pos = {}

    def run(self, batch):
        """batch: [(slot, rows [n, W])] -> list of outputs; positions continue per slot"""
        h = np.concatenate([r for _, r in batch])
        slot = np.concatenate([[s] * len(r) for s, r in batch])
        pos, seqs, row = [], [], 0
        for s, r in batch:
            p0 = self.pos.get(s, 0)
            pos += list(range(p0, p0 + len(r)))
            seqs.append((row, len(r), s, p0))
            self.pos[s] = p0 + len(r)
            row += len(r)
        hd, u = f32(h), gk.zeros(h.shape, gk.float32)
        api.causal_conv_rows_f32(hd.device_ptr, u.device_ptr, f32(self.w).device_ptr, self.state.device_ptr, i32(slot).device_ptr,
                                 i32(pos).device_ptr, None, len(h), self.W, self.taps, None)
        api.causal_conv_state_f32(hd.device_ptr, self.state.device_ptr, i32(seqs).device_ptr, len(seqs), self.W, self.taps, None)
        out, at = u.to_numpy(), 0
        res = []
        for _, r in batch:
            res.append(out[at:at + len(r)])
            at += len(r)
        return res


@pytest.mark.parametrize("W,taps", [(40, 4), (300, 2), (33, 5), (16, 1), (520, 3)])
def test_input_convolution_whole_portions_single_tokens_and_two_sequences(W, taps):
    rng = np.random.default_rng(taps)
    a, b = rng.standard_normal((23, W)), rng.standard_normal((9, W))
    c = ConvHarness(W, taps)
    ra, rb = R.input_conv(a, c.w), R.input_conv(b, c.w)
    assert np.abs(c.run([(0, a)])[0] - ra).max() < 1e-5
    c.pos.clear()                                                        # the same slots again, rings dirty from the run before
    for sizes in ([2] * 4 + [1] * 3 + [5, 7], [1] * 23, [3, 20]):
        got = []
        for n, (lo, hi) in enumerate(cuts_of(sizes)):
            batch = [(0, a[lo:hi])]
            if n < len(b):                                               # a second sequence decodes beside it, one token a step
                batch.append((2, b[n:n + 1]))
            out = c.run(batch)
            got.append(out[0])
            if n < len(b):
                assert np.abs(out[1] - rb[n:n + 1]).max() < 1e-5
        assert np.abs(np.concatenate(got) - ra).max() < 1e-5
        c.pos.clear()


class DoubleRingHarness(ConvHarness):
    """pgk_causal_conv_rows_f32 with the ring kept twice per slot: rows and ring update in one launch."""

    def __init__(self, W, taps, slots=3):
        super().__init__(W, taps, slots)
        self.state = f32(50.0 * np.ones((slots, 2 * max(1, taps - 1) * W)))
        self.steps = {}

    def run(self, batch):
        h = np.concatenate([r for _, r in batch])
        slot = np.concatenate([[s] * len(r) for s, r in batch])
        pos, par = [], []
        for s, r in batch:
            p0 = self.pos.get(s, 0)
            pos += list(range(p0, p0 + len(r)))
            par += [self.steps.get(s, 0) & 1] * len(r)
            self.pos[s] = p0 + len(r)
            self.steps[s] = self.steps.get(s, 0) + 1
        u = gk.zeros(h.shape, gk.float32)
        api.causal_conv_rows_f32(f32(h).device_ptr, u.device_ptr, f32(self.w).device_ptr, self.state.device_ptr, i32(slot).device_ptr,
                                 i32(pos).device_ptr, i32(par).device_ptr, len(h), self.W, self.taps, None)
        out, at, res = u.to_numpy(), 0, []
        for _, r in batch:
            res.append(out[at:at + len(r)])
            at += len(r)
        return res

    def restart(self):
        self.pos.clear()
        self.steps.clear()


@pytest.mark.parametrize("W,taps", [(40, 4), (300, 2), (33, 5), (16, 1), (3000, 3)])
def test_input_convolution_with_the_ring_kept_twice(W, taps):
    rng = np.random.default_rng(taps)
    a, b = rng.standard_normal((23, W)), rng.standard_normal((9, W))
    c = DoubleRingHarness(W, taps)
    ra, rb = R.input_conv(a, c.w), R.input_conv(b, c.w)
    assert np.abs(c.run([(0, a)])[0] - ra).max() < 1e-5
    c.restart()                                                          # the same slots again, both ring copies dirty
    for sizes in ([2] * 4 + [1] * 3 + [5, 7], [1] * 23, [3, 20], [1, 1, 2, 1, 18]):
        got = []
        for n, (lo, hi) in enumerate(cuts_of(sizes)):
            batch = [(0, a[lo:hi])]
            if n < len(b):                                               # a second sequence decodes beside it, before or after
                batch.insert(n % 2, (2, b[n:n + 1]))
            out = c.run(batch)
            got.append(out[[i for i, (s_, _) in enumerate(batch) if s_ == 0][0]])
            if n < len(b):
                assert np.abs(out[[i for i, (s_, _) in enumerate(batch) if s_ == 2][0]] - rb[n:n + 1]).max() < 1e-5
        assert np.abs(np.concatenate(got) - ra).max() < 1e-5, sizes
        c.restart()


class LinearHarness:
    """pgk_seq_linear_prep + pgk_seq_linear_attention + pgk_seq_linear_finish on raw rows [q | k | v | gate]."""

    def __init__(self, H, D, Dv, decay, act=False, dims=0, base=100.0, k_scale=1.0, per_head=True, gate_act=2, mult=1.0, slots=3):
        self.H, self.D, self.Dv, self.decay = H, D, Dv, np.asarray(decay, np.float64)
        self.act, self.dims, self.base, self.k_scale, self.per_head, self.gate_act, self.mult = act, dims, base, k_scale, per_head, gate_act, mult
        self.state = f32(7.0 * np.ones((slots, H * D * Dv)))            # dirty
        self.w = None if per_head else 1 + 0.2 * np.random.default_rng(H).standard_normal(H * Dv)
        self.inv_freq = [base ** (-2.0 * i / dims) for i in range(dims // 2)] if dims else []
        self.pos = {}
        self.cols = 2 * H * D + 2 * H * Dv
        self.slice = None
        self.segment = 0                                                 # > 0: the three-pass form, this many chunks per call

    def run(self, batch):
        """batch: [(slot, q [n, H, D], k, v [n, H, Dv], gate [n, H * Dv])]"""
        H, D, Dv = self.H, self.D, self.Dv
        rows = np.concatenate([np.concatenate([q.reshape(len(q), -1), k.reshape(len(q), -1), v.reshape(len(q), -1), g], axis=1)
                               for _, q, k, v, g in batch])
        pos, seqs, row = [], [], 0
        for s, q, _, _, _ in batch:
            p0 = self.pos.get(s, 0)
            pos += list(range(p0, p0 + len(q)))
            seqs.append((row, len(q), s, p0))
            self.pos[s] = p0 + len(q)
            row += len(q)
        T = len(rows)
        proj, out = f32(rows), gk.zeros((T, H * Dv), gk.float32)
        api.seq_linear_prep(proj.device_ptr, self.cols, T, H, D, Dv, 0, H * D, 2 * H * D, 1 if self.act else 0, self.dims,
                            f64(self.inv_freq).device_ptr if self.dims else None, self.k_scale, i32(pos).device_ptr, None)
        if self.segment:
            n_chunks = -(-max(n for _, n, _, _ in seqs) // int(api.seq_linear_chunk_tokens()))
            ws = keep(gk.zeros((len(seqs) * self.segment * H * D * Dv,), gk.float32))
            for c0 in range(0, n_chunks, self.segment):
                api.seq_linear_attention_chunks(proj.device_ptr, self.cols, 0, H * D, 2 * H * D, out.device_ptr, H * Dv,
                                                self.state.device_ptr, f32(self.decay).device_ptr, i32(seqs).device_ptr, len(seqs),
                                                H, D, Dv, c0, min(self.segment, n_chunks - c0), ws.device_ptr, None)
        else:
            ds = self.slice or int(api.seq_linear_value_slice(H, D, Dv, len(seqs)))
            api.seq_linear_attention(proj.device_ptr, self.cols, 0, H * D, 2 * H * D, out.device_ptr, H * Dv, self.state.device_ptr,
                                     f32(self.decay).device_ptr, i32(seqs).device_ptr, len(seqs), H, D, Dv, ds, None)
        api.seq_linear_finish(out.device_ptr, H * Dv, proj.device_ptr, self.cols, 2 * H * D + H * Dv,
                              f32(self.w).device_ptr if self.w is not None else None, T, H, Dv, 1 if self.per_head else 0,
                              self.gate_act, 1e-6, self.mult, None)
        o, at, res = out.to_numpy(), 0, []
        for _, q, _, _, _ in batch:
            res.append(o[at:at + len(q)])
            at += len(q)
        return res

    def oracle(self, q, k, v, g):
        T = len(q)
        f = R.silu if self.act else (lambda z: z)
        q, k, v = f(q), f(k), f(v)
        if self.dims:
            q = R.rotate_half(q, np.arange(T), self.dims, self.base)
            k = R.rotate_half(k, np.arange(T), self.dims, self.base)
        o = R.decayed_linear_attention(q, k * self.k_scale, v, self.decay)
        o = R.unit_rms(o, 1e-6).reshape(T, -1) if self.per_head else R.unit_rms(o.reshape(T, -1), 1e-6) * self.w
        gate = {0: 1.0, 1: R.sigmoid(g), 2: R.silu(g)}[self.gate_act]
        return o * gate * self.mult


LINEAR_LAYOUTS = [dict(H=3, D=8, Dv=6, decay=[0.5, 0.9, 0.999], dims=6, k_scale=8 ** -0.5),
                  dict(H=1, D=32, Dv=32, decay=[0.97], act=True, per_head=False, gate_act=1),
                  dict(H=5, D=20, Dv=70, decay=[1.0, 0.3, 0.99, 0.9, 0.0], dims=20, mult=0.5),
                  dict(H=2, D=130, Dv=9, decay=[0.95, 0.8], act=True, per_head=False, gate_act=0),
                  dict(H=4, D=16, Dv=16, decay=[0.9] * 4, dims=16, base=1e6, gate_act=2)]


@pytest.mark.parametrize("layout", LINEAR_LAYOUTS)
def test_linear_attention_whole_portions_and_single_tokens_agree_with_the_oracle(layout):
    h = LinearHarness(**layout)
    rng = np.random.default_rng(h.D)
    T = 75                                                               # more than two chunks of 32
    q, k = rng.standard_normal((T, h.H, h.D)), rng.standard_normal((T, h.H, h.D))
    v, g = rng.standard_normal((T, h.H, h.Dv)), rng.standard_normal((T, h.H * h.Dv))
    ref = h.oracle(q, k, v, g)
    tol = 2e-5 * max(1.0, np.abs(ref).max())
    assert np.abs(h.run([(0, q, k, v, g)])[0] - ref).max() < tol
    for sizes in ([2] * 10 + [31, 1, 23], [32, 32, 11], [1] * 75, [33, 42]):
        h.pos.clear()                                                    # the slot's state is dirty from the run before
        got = [h.run([(1, q[a:b], k[a:b], v[a:b], g[a:b])])[0] for a, b in cuts_of(sizes)]
        assert np.abs(np.concatenate(got) - ref).max() < tol, sizes
    h.pos.clear()
    h.slice = 4                                                          # narrow value slices give the same answer
    assert np.abs(h.run([(0, q, k, v, g)])[0] - ref).max() < tol
    for segment in (1, 2, 8):                                            # all chunks at once, in segments of 1, 2, all
        h.segment = segment
        h.pos.clear()
        assert np.abs(h.run([(0, q, k, v, g)])[0] - ref).max() < tol, segment
        h.pos.clear()                                                    # a prompt in two portions beside a short sequence
        first = h.run([(1, q[:40], k[:40], v[:40], g[:40]), (2, q[:3], k[:3], v[:3], g[:3])])
        rest = h.run([(2, q[3:5], k[3:5], v[3:5], g[3:5]), (1, q[40:], k[40:], v[40:], g[40:])])
        assert np.abs(np.concatenate([first[0], rest[1]]) - ref).max() < tol, segment
        assert np.abs(np.concatenate([first[1], rest[0]]) - ref[:5]).max() < tol, segment


def test_linear_attention_unequal_sequences_in_one_step_and_a_reused_slot():
    h = LinearHarness(H=2, D=12, Dv=10, decay=[0.9, 0.99], dims=8)
    rng = np.random.default_rng(5)

    def seq(n):
        return (rng.standard_normal((n, 2, 12)), rng.standard_normal((n, 2, 12)), rng.standard_normal((n, 2, 10)),
                rng.standard_normal((n, 20)))

    a, b, c = seq(40), seq(3), seq(17)
    ra, rb, rc = h.oracle(*a), h.oracle(*b), h.oracle(*c)
    out = h.run([(0, *[x[:37] for x in a]), (1, *[x[:1] for x in b])])
    assert np.abs(out[0] - ra[:37]).max() < 2e-5 and np.abs(out[1] - rb[:1]).max() < 2e-5
    for i in range(2):
        out = h.run([(0, *[x[37 + i:38 + i] for x in a]), (1, *[x[1 + i:2 + i] for x in b])])
        assert np.abs(out[0] - ra[37 + i:38 + i]).max() < 2e-5 and np.abs(out[1] - rb[1 + i:2 + i]).max() < 2e-5
    h.pos.pop(1)                                                         # b is over; c starts in its slot
    out = h.run([(1, *[x[:9] for x in c]), (0, *[x[39:] for x in a])])
    assert np.abs(out[0] - rc[:9]).max() < 2e-5 and np.abs(out[1] - ra[39:]).max() < 2e-5
    assert np.abs(h.run([(1, *[x[9:] for x in c])])[0] - rc[9:]).max() < 2e-5


@pytest.mark.parametrize("decoded", [False, True])
def test_linear_attention_carries_one_early_token_over_hundreds(decoded):
    """Only token `star` has a key along the queries' direction and a value with a large component: the output of every later
    token is that value times decay^(distance), nothing else -- through chunk borders, portions and single tokens."""
    H, D, Dv, T = 2, 8, 6, 330
    dec = [0.999, 0.99]
    rng = np.random.default_rng(3)
    for star in (0, 31, 32, 200):
        q, k = np.zeros((T, H, D)), 1e-3 * rng.standard_normal((T, H, D))
        q[:, :, 0] = 1.0
        k[:, :, 0] = 0.0
        k[star, :, 0] = 1.0
        v = 1e-3 * rng.standard_normal((T, H, Dv))
        v[star, :, 2] = 5.0
        h = LinearHarness(H, D, Dv, dec, gate_act=0)
        h.oracle = lambda q, k, v, g: R.decayed_linear_attention(q, k, v, h.decay).reshape(len(q), -1)
        g = np.zeros((T, H * Dv))
        # raw outputs: skip the norm by comparing before it -- run prep + recurrence only
        api_finish = api.seq_linear_finish
        try:
            api.seq_linear_finish = lambda *a: None
            if decoded:
                n0 = min(star + 1, T - 1)
                got = [h.run([(0, q[:n0], k[:n0], v[:n0], g[:n0])])[0]] + [h.run([(0, q[i:i + 1], k[i:i + 1], v[i:i + 1], g[i:i + 1])])[0]
                                                                        for i in range(n0, T)]
                got = np.concatenate(got)
            else:
                h.segment = 3                                            # the three-pass form, two segments per portion
                got = np.concatenate([h.run([(0, q[a:b], k[a:b], v[a:b], g[a:b])])[0] for a, b in cuts_of([100, 130, 100])])
        finally:
            api.seq_linear_finish = api_finish
        got = got.reshape(T, H, Dv)
        for i in range(T):
            for hh in range(H):
                want = 5.0 * dec[hh] ** (i - star) if i >= star else 0.0
                assert abs(got[i, hh, 2] - want) < 2e-3 + 1e-4 * want, (star, i, hh)


class AttentionHarness:
    """pgk_seq_mixer_prep_rot + pgk_seq_attention_ex2 on raw rows [q | k | v]."""

    def __init__(self, H, G, D, Dv, window=0, keep_first=0, scale=0.3, page=4, dtype="float32", log=True, sigmoid=False, dims=0,
                 factor=1.0, norm=0, splits=1, mult=1.0):
        self.H, self.G, self.D, self.Dv, self.window, self.keep, self.scale = H, G, D, Dv, window, keep_first, scale
        self.splits, self.dims, self.factor, self.norm, self.sigmoid, self.mult = splits, dims, factor, norm, sigmoid, mult
        self.cache = PagedKVCache([(G, D, Dv)], dtype, page, 64, 2)
        self.qt = api.seq_queries_per_tile(H, G)
        rng = np.random.default_rng(H * 31 + D)
        self.r1, self.r2 = (rng.uniform(0.2, 1.5, H), rng.uniform(0.1, 2.0, H)) if log else (None, None)
        self.pb = rng.uniform(-2.0, 0.0, H) if sigmoid else None
        self.base = 50.0
        self.inv_freq = [self.base ** (-2.0 * i / dims) / factor for i in range(dims // 2)] if dims else []
        self.tickets = gk.zeros((4096,), gk.int32)
        self.cols = H * D + G * D + G * Dv
        self.decode_kernel = True

    def run(self, seq, q, k, v):
        n = q.shape[0]
        slot, pos0 = self.cache.extend(seq, n)
        self.cache.sync_table()
        c, H, G, D, Dv = self.cache, self.H, self.G, self.D, self.Dv
        proj = f32(np.concatenate([q.reshape(n, -1), k.reshape(n, -1), v.reshape(n, -1)], axis=1))
        api.seq_mixer_prep_rot(proj.device_ptr, self.cols, n, H, G, D, Dv, 0, H * D, H * D + G * D, self.dims,
                               f64(self.inv_freq).device_ptr if self.dims else None, self.norm, None, None, 1e-6, c.k[0].device_ptr,
                               c.v[0].device_ptr, c.dtype_code, c.table_dev.device_ptr, c.pool.max_pages, c.page_size,
                               i32([slot] * n).device_ptr, i32(np.arange(pos0, pos0 + n)).device_ptr, None)
        tiles = [(i, min(self.qt, n - i), slot, pos0 + i) for i in range(0, n, self.qt)]
        out = gk.zeros((n, H * Dv), gk.float32)
        api.seq_attention_ex2(proj.device_ptr, self.cols, 0, None, 0, 0, 0, out.device_ptr, H * Dv, c.k[0].device_ptr,
                              c.v[0].device_ptr, D, Dv, c.dtype_code, c.table_dev.device_ptr, c.pool.max_pages, c.page_size,
                              i32(tiles).device_ptr, len(tiles), f32(self.r1).device_ptr if self.r1 is not None else None,
                              f32(self.r2).device_ptr if self.r2 is not None else None, None, H, G, D, Dv, 0, self.window, self.keep,
                              self.scale, 0.0, 1 if self.sigmoid else 0, f32(self.pb).device_ptr if self.sigmoid else None, self.mult,
                              self.splits, keep(gk.zeros((n * H * self.splits * (Dv + 2),), gk.float32)).device_ptr,
                              self.tickets.device_ptr, 1 if (n == 1 and self.decode_kernel) else 0, None)
        assert not self.tickets.to_numpy().any()
        return out.to_numpy().reshape(n, H, Dv)

    def oracle(self, q, k, v):
        T = len(q)
        if self.dims:
            q = R.rotate_half(q, np.arange(T), self.dims, self.base, self.factor)
            k = R.rotate_half(k, np.arange(T), self.dims, self.base, self.factor)
        if self.norm:
            q, k = R.unit_rms(q, 1e-6), R.unit_rms(k, 1e-6)
        if self.sigmoid:
            return R.sigmoid_attention(q, k, v, self.scale, self.pb) * self.mult
        r1 = self.r1 if self.r1 is not None else np.zeros(self.H)
        r2 = self.r2 if self.r2 is not None else np.zeros(self.H)
        return R.log_distance_attention(q, k, v, self.scale, r1, r2, self.window, self.keep) * self.mult


ATTENTION_LAYOUTS = [dict(H=4, G=2, D=16, Dv=8, window=7, keep_first=2, page=4),
                     dict(H=6, G=2, D=8, Dv=12, window=3, keep_first=5, page=3),             # more kept positions than the window
                     dict(H=3, G=3, D=12, Dv=12, window=100, keep_first=4, page=4),           # window beyond the sequence
                     dict(H=2, G=1, D=20, Dv=6, window=33, keep_first=1, page=8),
                     dict(H=40, G=1, D=8, Dv=8, window=5, keep_first=3, page=4),
                     dict(H=1, G=1, D=6, Dv=70, window=9, keep_first=0, page=4, mult=1.5),
                     dict(H=2, G=2, D=10, Dv=10, window=0, keep_first=0, page=4),              # no window at all
                     dict(H=4, G=2, D=12, Dv=10, sigmoid=True, log=False, dims=8, factor=4.0, norm=1, page=4, scale=0.8, mult=1.2),
                     dict(H=2, G=1, D=16, Dv=16, sigmoid=True, log=False, dims=16, norm=1, page=8, scale=2.0),
                     dict(H=3, G=1, D=8, Dv=5, sigmoid=True, log=False, dims=0, norm=0, page=4)]


@pytest.mark.parametrize("layout", ATTENTION_LAYOUTS)
def test_attention_whole_portions_and_single_tokens_agree_with_the_oracle(layout):
    h = AttentionHarness(**layout)
    rng = np.random.default_rng(h.H * 7 + h.D)
    T = 75
    q, k, v = rng.standard_normal((T, h.H, h.D)), rng.standard_normal((T, h.G, h.D)), rng.standard_normal((T, h.G, h.Dv))
    ref = h.oracle(q, k, v)
    tol = 1e-5 * max(1.0, np.abs(ref).max())
    assert np.abs(h.run("w", q, k, v) - ref).max() < tol
    cuts = [0, 2, 5, 6, 19, 20, 31, 45, 75]
    parts = np.concatenate([h.run("p", q[a:b], k[a:b], v[a:b]) for a, b in zip(cuts, cuts[1:])])
    assert np.abs(parts - ref).max() < tol
    h.cache.release("w")                                                 # its pages serve the next sequence
    single = np.concatenate([h.run("s", q[i:i + 1], k[i:i + 1], v[i:i + 1]) for i in range(T)])
    assert np.abs(single - ref).max() < tol
    h.cache.release("p")
    h.decode_kernel = False                                              # the same through the tile kernel
    single = np.concatenate([h.run("t", q[i:i + 1], k[i:i + 1], v[i:i + 1]) for i in range(T)])
    assert np.abs(single - ref).max() < tol


@pytest.mark.parametrize("decoded", [False, True])
@pytest.mark.parametrize("window,keep_first,page", [(6, 2, 4), (8, 4, 8), (33, 1, 16), (1, 3, 4), (40, 33, 8)])
def test_standout_key_at_the_window_edge_and_among_the_kept_first_positions(window, keep_first, page, decoded):
    """One key has a score far above the rest and its value is the only one with a large component.  Query i must see it
    exactly while 0 <= i - star < window, or for good when star < keep_first."""
    H, G, D, Dv = 2, 1, 8, 4
    T = 2 * window + 40
    rng = np.random.default_rng(window)
    for star in (0, keep_first - 1, keep_first, window + 3, 63):         # the last kept position, the first that is not, a page's last row
        if not 0 <= star < T:
            continue
        q, k = 0.01 * rng.standard_normal((T, H, D)), 0.01 * rng.standard_normal((T, G, D))
        q[:, :, 0] = 3.0
        k[:, :, 0] = -3.0                                                # every other key points away from the queries
        k[star, 0, 0] = 3.0
        v = 0.01 * rng.standard_normal((T, G, Dv))
        v[:, 0, 0] = -1.0
        v[star, 0, 0] = 3.0
        h = AttentionHarness(H, G, D, Dv, window, keep_first, scale=6.0, page=page)
        h.r1[:] = 0.3                                                    # the distance term must not hide a far kept key
        ref = h.oracle(q, k, v)
        n0 = T if not decoded else min(star + 1, T - 1)
        got = h.run("a", q[:n0], k[:n0], v[:n0])
        if decoded:
            got = np.concatenate([got] + [h.run("a", q[i:i + 1], k[i:i + 1], v[i:i + 1]) for i in range(n0, T)])
        assert np.abs(got - ref).max() < 1e-5
        for i in range(T):
            sees = i >= star and (i - star < window or star < keep_first)
            assert (got[i, :, 0] > 2.5).all() == sees and (sees or (got[i, :, 0] < 0).all()), (star, i)


@pytest.mark.parametrize("splits", [2, 3, 7])
@pytest.mark.parametrize("sigmoid", [False, True])
def test_key_slices_fold_to_the_same_answer(splits, sigmoid):
    kw = dict(sigmoid=True, log=False, dims=8, norm=1) if sigmoid else dict(window=150, keep_first=40)
    h = AttentionHarness(4, 2, 16, 8, page=8, splits=splits, **kw)
    rng = np.random.default_rng(splits)
    T = 330                                                              # keys far away, across many pages
    q, k, v = rng.standard_normal((T, 4, 16)), rng.standard_normal((T, 2, 16)), rng.standard_normal((T, 2, 8))
    ref = h.oracle(q, k, v)
    tol = 2e-5 * max(1.0, np.abs(ref).max())
    got = np.concatenate([h.run("a", q[:300], k[:300], v[:300])] + [h.run("a", q[i:i + 1], k[i:i + 1], v[i:i + 1]) for i in range(300, T)])
    assert np.abs(got - ref).max() < tol


def test_sigmoid_weights_see_a_far_key_among_hundreds_at_page_borders():
    """Without normalisation every key adds on its own: one far key whose weight is near 1 among hundreds near 0."""
    H, G, D, Dv, T = 2, 1, 8, 4, 300
    rng = np.random.default_rng(1)
    for star in (0, 15, 16, 255):
        q, k = np.zeros((T, H, D)), np.zeros((T, G, D))
        q[:, :, 4] = 1.0                                                 # dimension 4 is not rotated
        k[:, :, 4] = -1.0
        k[star, 0, 4] = 1.0
        v = 0.01 * rng.standard_normal((T, G, Dv))
        v[star, 0, 1] = 2.0
        h = AttentionHarness(H, G, D, Dv, sigmoid=True, log=False, dims=4, norm=1, page=16, scale=4.0)
        h.pb[:] = 0.0                                                    # weights: sigmoid(32) for the star, sigmoid(-32) for the rest
        got = np.concatenate([h.run("a", q[:280], k[:280], v[:280])] + [h.run("a", q[i:i + 1], k[i:i + 1], v[i:i + 1]) for i in range(280, T)])
        assert np.abs(got - h.oracle(q, k, v)).max() < 1e-5
        for i in range(T):
            assert (got[i, :, 1] > 1.9).all() == (i >= star) and ((got[i, :, 1] < 0.1).all() or i >= star), (star, i)


# ================================================================ whole models
def variants():
    """Sizes that the mechanisms must not assume equal or 1: key and value sizes, head counts on the two sides of a parallel
    mixer, rotated dimensions below the head size and equal to it, no position scaling, more kept positions than the window, a
    window beyond the sequence, one tap, five taps, layers without feed-forward, odd widths, every order of layers."""
    yield "base", R.make_config([R.parallel_layer(), R.lightning_layer(), R.attention_layer()])
    yield "attention_first", R.make_config([R.attention_layer(heads=6, kv_heads=2, dim=8, vdim=12, window=3, keep=5),
                                            R.parallel_layer(heads=2, kv_heads=1, dim=16, vdim=4, dims=16, factor=1.0, r_heads=3,
                                                             r_dim=6, r_vdim=10, r_dims=4, ff=0),
                                            R.lightning_layer(heads=1, dim=20, vdim=5, ff=18)], vocab=61, width=52, taps=5,
                                           residual_mult=1.0, logit_scale=1.0)
    yield "one_tap", R.make_config([R.lightning_layer(heads=2, dim=6, vdim=6, decay=[1.0, 0.25], ff=0),
                                    R.attention_layer(heads=1, kv_heads=1, dim=10, vdim=10, window=1000, keep=0)], taps=1)
    yield "two_taps_twice", R.make_config([R.lightning_layer(), R.lightning_layer(heads=4, dim=4, vdim=3),
                                           R.parallel_layer(left_scale=1.0, right_scale=1.0), R.parallel_layer(dims=12, r_dims=8)],
                                          taps=2, width=36)


VARIANTS = dict(variants())


def make(name, dtype="float32", page=4, seed=1, tokens_hint=64, slots=2):
    cfg = VARIANTS[name]
    P = R.random_params(cfg, seed=seed)
    m = llm.build_layered_model(layered_config_from_json(cfg), P, dtype)
    m.init_cache(tokens_hint, page_size=page, slots=slots)
    return cfg, P, m


def tokens(cfg, n, seed=0):
    return [int(t) for t in np.random.default_rng(seed).integers(0, cfg["vocab"], n)]


@pytest.mark.parametrize("name", list(VARIANTS))
def test_whole_prompt_and_every_layer_match_the_oracle_float32(name):
    cfg, P, m = make(name, tokens_hint=128)
    toks = tokens(cfg, 75)                                               # long enough for the three-pass linear attention
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


@pytest.mark.parametrize("name", ["base", "attention_first"])
def test_first_tokens_and_decoding_from_position_zero(name):
    cfg, P, m = make(name)
    toks = tokens(cfg, 12, seed=4)
    ref = R.forward(cfg, P, toks)
    got = np.concatenate([m.step([("a", [t], [0])]) for t in toks])
    assert np.abs(got - ref).max() < F32_TOL


@pytest.mark.parametrize("sizes", [[2] * 20, [3, 2, 7, 1, 11, 6, 10], [16, 24], [1, 39], [33, 3, 4]])
def test_prompt_portions(sizes):
    cfg, P, m = make("attention_first")
    toks = tokens(cfg, sum(sizes), seed=5)
    ref = R.forward(cfg, P, toks)
    got, at = [], 0
    for n in sizes:
        got.append(m.step([("a", toks[at:at + n], list(range(n)))]))
        at += n
    assert np.abs(np.concatenate(got) - ref).max() < F32_TOL


@pytest.mark.parametrize("name", ["base", "attention_first"])
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


def test_slots_grow_while_sequences_hold_state():
    cfg, P, m = make("base", tokens_hint=64, slots=2)
    seqs = [tokens(cfg, 8 + i, seed=50 + i) for i in range(5)]
    refs = [R.forward(cfg, P, s) for s in seqs]
    m.step([(0, seqs[0][:5], []), (1, seqs[1][:5], [])])                 # two sequences hold state in the two slots
    m.step([(i, seqs[i][:5], []) for i in (2, 3, 4)])                    # three more: the slot arrays are reallocated
    got = m.step([(i, s[5:], list(range(len(s) - 5))) for i, s in enumerate(seqs)])
    assert np.abs(got - np.concatenate([r[5:] for r in refs])).max() < F32_TOL


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


def test_decoding_over_a_long_context_in_key_slices():
    cfg, P, m = make("one_tap", page=16, tokens_hint=512)
    toks = tokens(cfg, 300, seed=8)
    ref = R.forward(cfg, P, toks)
    m.step([("a", toks[:288], [])])
    got = np.concatenate([m.step([("a", [t], [0])]) for t in toks[288:]])
    assert m._ws is not None                                             # the sliced path ran
    assert np.abs(got - ref[288:]).max() < F32_TOL


@pytest.mark.parametrize("name", list(VARIANTS))
def test_bfloat16_mode_stays_within_bfloat16_rounding(name):
    cfg, P, m = make(name, dtype="bfloat16")
    toks = tokens(cfg, 40, seed=7)
    ref = R.forward(cfg, P, toks)
    whole = m.step([("a", toks, list(range(40)))])
    scale = np.abs(ref).max()
    assert np.abs(whole - ref).max() < 0.04 * scale
    got = np.concatenate([m.step([("b", toks[:20], list(range(20)))])] + [m.step([("b", [t], [0])]) for t in toks[20:]])
    assert np.abs(got - whole).max() < 0.04 * scale                      # the same sequence cut differently: rounding only


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


def _save(cfg, P, folder):
    tensors = {k: ((np.ascontiguousarray(v, np.float32).view(np.uint32) >> 16).astype(np.uint16).reshape(v.shape), "BF16")
               for k, v in P.items()}
    llm.save_safetensors(os.path.join(folder, "model.safetensors"), tensors)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    return {k: (np.ascontiguousarray(v, np.float32).view(np.uint32) >> 16 << 16).view(np.float32) for k, v in P.items()}


def test_loader_picks_the_family_from_config_json(tmp_path):
    cfg = VARIANTS["attention_first"]
    P = _save(cfg, R.random_params(cfg, seed=8), str(tmp_path))
    m = llm.load_model_from_safetensors(str(tmp_path), dtype="float32")
    assert isinstance(m, llm.LayeredCausalModel) and m.config.architecture == "Rezulorn"
    toks = tokens(cfg, 10)
    assert np.abs(m.step([("a", toks, list(range(10)))]) - R.forward(cfg, P, toks)).max() < F32_TOL
    with pytest.raises(ValueError, match="shape"):
        bad = dict(P)
        bad["l1.mix.right.g"] = P["l1.mix.right.g"][:-1]
        llm.build_layered_model(layered_config_from_json(cfg), bad, "float32")


def test_trace_replay_command_line(tmp_path):
    cfg = VARIANTS["base"]
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
