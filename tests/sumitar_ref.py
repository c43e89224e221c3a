"""NumPy float64 oracle of the Sumitar design: whole sequences at once, no cache, no state, one function per mechanism,
no code shared with the package.  Notation: T tokens, W width, H heads, G key/value (or query/key) heads, D key size, Dv
value size.

    layer        x += N1b(mixer(N1(x)));  x += N2b(ff(N2(x)))          N = dyt
    dyt(x)       tanh(alpha x) * w + b                                  (alpha a scalar; pointwise)
    parallel     ( rms(left) * w_l + rms(right) * w_r ) / 2            rms over the width, both sides read the same input
      left       q, k, v = W h + bias;  q, k rotated (half layout, first `dims`, angle p * base^(-2i/dims));
                 s_ij = scale temp_h q_i.k_j;  j visible when 0 <= i - j < window;  softmax;  W_o
      right      q = silu(W_q h);  f = l + (1 - l) sigmoid(W_f h + b_f);  S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T;
                 o_t = S_t^T q_t;  every head's o: rms * w;  W_o
    delta        q, k, v = silu(conv(W h));  q, k unit vectors per head, q *= D^(-1/2);  beta = sigmoid(W_b h);
                 g = exp(-exp(A_log) softplus(W_a h + dt_bias));  S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q;
                 W_o (rms(o) * w * silu(W_g h))
    dense ff     W_down polynorm(W_up h);  polynorm(z) = a rms(z) + b rms(z^2) + c rms(z^3) + e
    moe          s = softmax(W_r h);  the `top` largest of s + correction are chosen, weights s (not renormalised);  the last
                 `identity` router outputs stand for experts that return h;  + sigmoid(w_sg . h) * shared(h)
    expert       W_down (silu(W_gate h) * W_up h)
    output       embed . dyt_final(x)
"""
import numpy as np


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.logaddexp(0.0, z)


def dyt(x, alpha, w, b):
    return np.tanh(float(np.asarray(alpha).reshape(-1)[0]) * x) * w + b


def unit_rms(x, eps):
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def rotate_half(x, positions, dims, base):
    """x [T, heads, n]: element i < dims / 2 pairs with element i + dims / 2, angle position * base^(-2i/dims)"""
    out = np.array(x, np.float64)
    half = dims // 2
    f = base ** (-2.0 * np.arange(half) / dims)
    ang = np.asarray(positions, np.float64)[:, None] * f
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    a, b = out[..., :half].copy(), out[..., half:dims].copy()
    out[..., :half] = a * c - b * s
    out[..., half:dims] = b * c + a * s
    return out


def window_softmax_attention(q, k, v, scale, temp, window):
    """q [T, H, D], k [T, G, D], v [T, G, Dv] -> [T, H, Dv]; head h reads key/value head h // (H / G); window 0: all
    earlier keys"""
    T, H, _ = q.shape
    G = k.shape[1]
    out = np.zeros((T, H, v.shape[2]))
    i, j = np.arange(T)[:, None], np.arange(T)[None, :]
    seen = (j <= i) & ((i - j < window) if window > 0 else True)
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale * float(temp[h])
        s = np.where(seen, s, -np.inf)
        s = s - s.max(-1, keepdims=True)
        p = np.exp(s)
        p /= p.sum(-1, keepdims=True)
        out[:, h] = p @ v[:, g]
    return out


def gated_outer_recurrence(q, f, v):
    """q, f [T, H, D], v [T, H, Dv]: S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T, o_t = S_t^T q_t -> [T, H, Dv]"""
    T, H, D = q.shape
    S = np.zeros((H, D, v.shape[2]))
    out = np.zeros((T, H, v.shape[2]))
    for t in range(T):
        S = f[t][:, :, None] * S + (1.0 - f[t])[:, :, None] * v[t][:, None, :]
        out[t] = np.einsum("hd,hdv->hv", q[t], S)
    return out


def short_conv(x, w):
    """x [T, C], w [C, taps], the last column weighs the current token; zeros before the sequence"""
    T, taps = x.shape[0], w.shape[1]
    out = np.zeros_like(x, dtype=np.float64)
    for j in range(taps):
        back = taps - 1 - j
        if back < T:
            out[back:] += w[:, j] * x[:T - back]
    return out


def delta_rule(q, k, v, beta, g):
    """q, k [T, H, D] (already per value head), v [T, H, Dv], beta, g [T, H] -> [T, H, Dv]"""
    T, H, D = q.shape
    S = np.zeros((H, D, v.shape[2]))
    out = np.zeros((T, H, v.shape[2]))
    for t in range(T):
        S = g[t][:, None, None] * S
        u = beta[t][:, None] * (v[t] - np.einsum("hdv,hd->hv", S, k[t]))
        S = S + k[t][:, :, None] * u[:, None, :]
        out[t] = np.einsum("hdv,hd->hv", S, q[t])
    return out


def polynorm(z, coef, eps):
    a, b, c, e = (float(t) for t in coef)
    return a * unit_rms(z, eps) + b * unit_rms(z ** 2, eps) + c * unit_rms(z ** 3, eps) + e


def gated_expert(h, gate, up, down):
    return (silu(h @ gate.T) * (h @ up.T)) @ down.T


def route(h, router, correction, top):
    """-> (chosen [T, top] router outputs, their weights)"""
    z = h @ router.T
    z = z - z.max(-1, keepdims=True)
    s = np.exp(z)
    s /= s.sum(-1, keepdims=True)
    order = np.argsort(-(s + correction), axis=-1, kind="stable")[:, :top]
    return order, np.take_along_axis(s, order, -1)


# ---------------------------------------------------------------- mixers and feed-forwards from named tensors
def left_mixer(h, P, pre, m, positions):
    T = h.shape[0]
    H, G, D, Dv = m["heads"], m.get("kv_heads") or m["heads"], m["dim"], m.get("vdim") or m["dim"]
    q = (h @ P[pre + "q"].T + P[pre + "q.b"]).reshape(T, H, D)
    k = (h @ P[pre + "k"].T + P[pre + "k.b"]).reshape(T, G, D)
    v = (h @ P[pre + "v"].T + P[pre + "v.b"]).reshape(T, G, Dv)
    rot = m.get("rot")
    if rot:
        q = rotate_half(q, positions, rot["dims"], rot["base"])
        k = rotate_half(k, positions, rot["dims"], rot["base"])
    o = window_softmax_attention(q, k, v, m["scale"], P[pre + "temp"], int((m.get("mask") or {}).get("size") or 0))
    return o.reshape(T, H * Dv) @ P[pre + "o"].T


def right_mixer(h, P, pre, m, eps):
    T = h.shape[0]
    H, D, Dv = m["heads"], m["dim"], m.get("vdim") or m["dim"]
    q = silu(h @ P[pre + "q"].T).reshape(T, H, D)
    low = P[pre + "lower"].astype(np.float64)
    f = (low + (1.0 - low) * sigmoid(h @ P[pre + "f"].T + P[pre + "f.b"])).reshape(T, H, D)
    v = (h @ P[pre + "v"].T).reshape(T, H, Dv)
    o = unit_rms(gated_outer_recurrence(q, f, v), eps) * P[pre + "norm"]
    return o.reshape(T, H * Dv) @ P[pre + "o"].T


def parallel_mixer(h, P, pre, m, eps, positions):
    a = unit_rms(left_mixer(h, P, pre + "left.", m["left"], positions), eps) * P[pre + "left.out"]
    b = unit_rms(right_mixer(h, P, pre + "right.", m["right"], eps), eps) * P[pre + "right.out"]
    return 0.5 * (a + b)


def delta_mixer(h, P, pre, m, eps):
    T = h.shape[0]
    H, G, D, Dv = m["heads"], m.get("kv_heads") or m["heads"], m["dim"], m.get("vdim") or m["dim"]
    q = silu(short_conv(h @ P[pre + "q"].T, P[pre + "q.conv"])).reshape(T, G, D)
    k = silu(short_conv(h @ P[pre + "k"].T, P[pre + "k.conv"])).reshape(T, G, D)
    v = silu(short_conv(h @ P[pre + "v"].T, P[pre + "v.conv"])).reshape(T, H, Dv)
    q = q / np.sqrt((q * q).sum(-1, keepdims=True) + 1e-6) * D ** -0.5
    k = k / np.sqrt((k * k).sum(-1, keepdims=True) + 1e-6)
    rep = H // G
    q, k = np.repeat(q, rep, axis=1), np.repeat(k, rep, axis=1)
    beta = sigmoid(h @ P[pre + "b"].T)
    g = np.exp(-np.exp(P[pre + "A_log"].astype(np.float64)) * softplus(h @ P[pre + "a"].T + P[pre + "dt_bias"]))
    o = unit_rms(delta_rule(q, k, v, beta, g), eps) * P[pre + "norm"]
    o = o * silu(h @ P[pre + "g"].T).reshape(T, H, Dv)
    return o.reshape(T, H * Dv) @ P[pre + "o"].T


def feed_forward(h, P, pre, f, eps):
    if f["kind"] == "dense":
        return polynorm(h @ P[pre + "up"].T, P[pre + "act"], eps) @ P[pre + "down"].T
    r = f["router"]
    E, top = r["experts"], r["top"]
    chosen, wts = route(h, P[pre + "router"], P[pre + "correction"], top)
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for e, w in zip(chosen[t], wts[t]):
            if e >= E:
                out[t] += w * h[t]
            else:
                out[t] += w * gated_expert(h[t], P[f"{pre}e{e}.gate"], P[f"{pre}e{e}.up"], P[f"{pre}e{e}.down"])
    if f.get("shared"):
        s = pre + "shared."
        out += sigmoid(h @ P[s + "sg"].T) * gated_expert(h, P[s + "gate"], P[s + "up"], P[s + "down"])
    return out


def forward(cfg, P, tokens, want_layers=False):
    """-> logits [T, vocab] (and the residual stream after every layer, [layers, T, W])"""
    P = {n: np.asarray(a, np.float64) for n, a in P.items()}
    eps = cfg["norm"]["eps"]
    x = P["embed"][np.asarray(tokens)]
    pos = np.arange(len(tokens))
    seen = []

    def norm(name, v):
        return dyt(v, P[name + ".alpha"], P[name], P[name + ".b"])

    for i, L in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = norm(p + "norm1", x)
        if L["type"] == "parallel":
            y = parallel_mixer(h, P, p + "mix.", L["mixer"], eps, pos)
        elif L["type"] == "delta":
            y = delta_mixer(h, P, p + "mix.", L["mixer"], eps)
        else:
            raise ValueError(L["type"])
        x = x + norm(p + "norm1b", y)
        if L.get("mlp"):
            x = x + norm(p + "norm2b", feed_forward(norm(p + "norm2", x), P, p + "mlp.", L["mlp"], eps))
        seen.append(x.copy())
    logits = norm("final.norm", x) @ P["embed"].T
    return (logits, np.stack(seen)) if want_layers else logits


# ---------------------------------------------------------------- small configurations and random weights for the tests
def parallel_layer(heads=4, kv_heads=2, dim=12, vdim=10, dims=8, base=300.0, scale=0.4, window=9, r_heads=2, r_dim=8, r_vdim=6,
                   mlp=None):
    left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "mask": {"size": window},
            "rot": {"dims": dims, "base": base}}
    if not window:
        del left["mask"]
    return {"type": "parallel", "mixer": {"left": left, "right": {"heads": r_heads, "dim": r_dim, "vdim": r_vdim}}, "mlp": mlp}


def delta_layer(heads=4, kv_heads=2, dim=8, vdim=6, conv=3, mlp=None):
    return {"type": "delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}, "mlp": mlp}


def dense_ff(ff=24):
    return {"kind": "dense", "ff": ff}


def moe_ff(experts=5, identity=2, top=3, ff=12, shared_ff=10):
    f = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "identity": identity, "top": top}}
    if shared_ff:
        f["shared"] = {"ff": shared_ff}
    return f


def make_config(layers, vocab=90, width=40, eps=1e-5):
    return {"architecture": "Sumitar", "vocab": vocab, "width": width, "layers": layers, "norm": {"eps": eps}}


def bf16_round(a):
    b = np.ascontiguousarray(a, np.float32).view(np.uint32)
    b = ((b + 0x7FFF + ((b >> 16) & 1)) & 0xFFFF0000).astype(np.uint32)
    return b.view(np.float32)


def random_params(cfg, seed=0):
    """{tensor name: float32 array}, rounded to bfloat16-representable values so that both modes load the same numbers"""
    rng = np.random.default_rng(seed)
    W, V = cfg["width"], cfg["vocab"]
    bf = bf16_round

    def mat(n, k, gain=1.0):
        return bf(rng.standard_normal((n, k)) * gain / np.sqrt(k))

    P = {"embed": bf(rng.standard_normal((V, W)))}

    def norm(name):
        P[name] = bf(1.0 + 0.1 * rng.standard_normal(W))
        P[name + ".b"] = bf(0.1 * rng.standard_normal(W))
        P[name + ".alpha"] = bf(np.asarray(rng.uniform(0.4, 1.2))).reshape(())

    norm("final.norm")
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        for n in ("norm1", "norm1b") + (("norm2", "norm2b") if L.get("mlp") else ()):
            norm(p + n)
        mp = p + "mix."
        if L["type"] == "parallel":
            a, r = m["left"], m["right"]
            G = a.get("kv_heads") or a["heads"]
            lp, rp = mp + "left.", mp + "right."
            P[lp + "q"], P[lp + "k"] = mat(a["heads"] * a["dim"], W, 2.0), mat(G * a["dim"], W, 2.0)
            P[lp + "v"], P[lp + "o"] = mat(G * a["vdim"], W), mat(W, a["heads"] * a["vdim"])
            P[lp + "q.b"], P[lp + "k.b"] = bf(0.3 * rng.standard_normal(a["heads"] * a["dim"])), bf(0.3 * rng.standard_normal(G * a["dim"]))
            P[lp + "v.b"] = bf(0.3 * rng.standard_normal(G * a["vdim"]))
            P[lp + "temp"] = bf(rng.uniform(0.5, 2.0, a["heads"]))
            P[rp + "q"], P[rp + "f"] = mat(r["heads"] * r["dim"], W, 2.0), mat(r["heads"] * r["dim"], W, 2.0)
            P[rp + "f.b"] = bf(rng.standard_normal(r["heads"] * r["dim"]))
            P[rp + "lower"] = bf(rng.uniform(0.0, 0.9, r["heads"] * r["dim"]))
            P[rp + "v"], P[rp + "o"] = mat(r["heads"] * r["vdim"], W), mat(W, r["heads"] * r["vdim"])
            P[rp + "norm"] = bf(1.0 + 0.1 * rng.standard_normal(r["vdim"]))
            P[lp + "out"], P[rp + "out"] = bf(1.0 + 0.1 * rng.standard_normal(W)), bf(1.0 + 0.1 * rng.standard_normal(W))
        else:
            G = m.get("kv_heads") or m["heads"]
            H, D, Dv, taps = m["heads"], m["dim"], m["vdim"], m["conv"]
            P[mp + "q"], P[mp + "k"], P[mp + "v"] = mat(G * D, W, 2.0), mat(G * D, W, 2.0), mat(H * Dv, W, 2.0)
            for n, c in (("q", G * D), ("k", G * D), ("v", H * Dv)):
                P[mp + n + ".conv"] = bf(0.6 * rng.standard_normal((c, taps)))
            P[mp + "b"], P[mp + "a"], P[mp + "g"] = mat(H, W), mat(H, W), mat(H * Dv, W)
            P[mp + "A_log"] = bf(np.log(rng.uniform(0.5, 4.0, H)))
            P[mp + "dt_bias"] = bf(rng.uniform(-3.0, 0.0, H))
            P[mp + "norm"] = bf(1.0 + 0.1 * rng.standard_normal(Dv))
            P[mp + "o"] = mat(W, H * Dv)
        f = L.get("mlp")
        if not f:
            continue
        q = p + "mlp."
        if f["kind"] == "dense":
            P[q + "up"], P[q + "down"] = mat(f["ff"], W), mat(W, f["ff"])
            P[q + "act"] = bf(np.array([0.6, 0.3, 0.2, 0.05]) + 0.1 * rng.standard_normal(4))
        else:
            r = f["router"]
            for e in range(r["experts"]):
                P[f"{q}e{e}.gate"], P[f"{q}e{e}.up"] = mat(f["expert"]["ff"], W), mat(f["expert"]["ff"], W)
                P[f"{q}e{e}.down"] = mat(W, f["expert"]["ff"])
            n = r["experts"] + r.get("identity", 0)
            P[q + "router"] = mat(n, W, 3.0)
            P[q + "correction"] = bf(0.2 * rng.standard_normal(n))
            if f.get("shared"):
                s = q + "shared."
                sf = f["shared"]["ff"]
                P[s + "gate"], P[s + "up"], P[s + "down"], P[s + "sg"] = mat(sf, W), mat(sf, W), mat(W, sf), mat(1, W)
    return P
