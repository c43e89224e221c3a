"""NumPy float64 oracle of the Rezulorn design: whole sequences at once, no cache, no state, one function per mechanism,
no code shared with the package.  Notation: T tokens, W width, H query heads, G key/value heads, D key size, Dv value size.

    layer        x += m * mixer(u1),  u1 = c1(LN1(x));   x += m * ff(u2),  u2 = c2(LN2(x))
    LN(x)        (x - mean) / sqrt(var + eps) * w                       (no bias)
    c(h)_t       h_t + sum_j w[:, j] h_(t - taps + 1 + j)               (zeros before the sequence)
    lightning    q, k, v = silu(W h);  S_t = a_h S_(t-1) + k_t v_t^T;  o_t = S_t^T q_t;
                 W_o (rms_w(all heads of o) * sigmoid(W_g h))
    attention    s_ij = scale q_i.k_j - r1_h ln(1 + r2_h (i - j));  j visible when j <= i and (i - j < window or j < keep);
                 softmax;  W_o
    parallel     left_scale * left + right_scale * right on the same input
      left       q, k rotated (half layout, first `dims`, angle p * base^(-2i/dims) / factor), then divided by their root
                 mean square per head;  weight of key j <= i: sigmoid(scale q.k + pb_h), not normalised;  W_o
      right      q, k rotated;  k *= D^(-1/2);  S_t = a_h S_(t-1) + k_t v_t^T;  o_t = S_t^T q_t;  every head's o divided by
                 its root mean square;  W_o (o * silu(W_g h))
    ff           W_down relu(W_up h)^2
    output       head LN(x) * logit_scale
"""
import numpy as np


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def layer_norm(x, w, eps):
    mu = x.mean(-1, keepdims=True)
    var = ((x - mu) ** 2).mean(-1, keepdims=True)
    return (x - mu) / np.sqrt(var + eps) * w


def unit_rms(x, eps):
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def input_conv(h, w):
    """h [T, W], w [W, taps] -> h + causal convolution over time, channel by channel"""
    T, taps = h.shape[0], w.shape[1]
    out = np.array(h, np.float64)
    for j in range(taps):
        back = taps - 1 - j
        if back < T:
            out[back:] += w[:, j] * h[:T - back]
    return out


def rotate_half(x, positions, dims, base, factor=1.0):
    """x [T, heads, n]: element i < dims / 2 pairs with element i + dims / 2; angle position * base^(-2i/dims) / factor"""
    out = np.array(x, np.float64)
    half = dims // 2
    f = base ** (-2.0 * np.arange(half) / dims) / factor
    ang = np.asarray(positions, np.float64)[:, None] * f
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    a, b = out[..., :half].copy(), out[..., half:dims].copy()
    out[..., :half] = a * c - b * s
    out[..., half:dims] = b * c + a * s
    return out


def decayed_linear_attention(q, k, v, decay):
    """q, k [T, H, D], v [T, H, Dv], decay [H] -> o [T, H, Dv] by the recurrence itself, token by token"""
    T, H, D = q.shape
    out = np.zeros((T, H, v.shape[2]))
    for h in range(H):
        S = np.zeros((D, v.shape[2]))
        for t in range(T):
            S = decay[h] * S + np.outer(k[t, h], v[t, h])
            out[t, h] = S.T @ q[t, h]
    return out


def keep_first_window_mask(T, window, keep):
    i, j = np.arange(T)[:, None], np.arange(T)[None, :]
    near = (i - j < window) if window > 0 else np.ones((T, T), bool)
    return (j <= i) & (near | (j < keep))


def log_distance_attention(q, k, v, scale, r1, r2, window, keep):
    """q [T, H, D], k [T, G, D], v [T, G, Dv] -> [T, H, Dv]; softmax over the visible keys"""
    T, H, _ = q.shape
    G = k.shape[1]
    vis = keep_first_window_mask(T, window, keep)
    dist = np.maximum(np.arange(T)[:, None] - np.arange(T)[None, :], 0).astype(np.float64)
    out = np.zeros((T, H, v.shape[2]))
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale - r1[h] * np.log1p(r2[h] * dist)
        s = np.where(vis, s, -np.inf)
        e = np.exp(s - s.max(-1, keepdims=True))
        out[:, h] = (e / e.sum(-1, keepdims=True)) @ v[:, g]
    return out


def sigmoid_attention(q, k, v, scale, pb):
    """causal, weight sigmoid(scale q.k + pb_h), no normalisation over the keys"""
    T, H, _ = q.shape
    G = k.shape[1]
    vis = np.tril(np.ones((T, T), bool))
    out = np.zeros((T, H, v.shape[2]))
    for h in range(H):
        g = h // (H // G)
        p = np.where(vis, sigmoid((q[:, h] @ k[:, g].T) * scale + pb[h]), 0.0)
        out[:, h] = p @ v[:, g]
    return out


def lightning_mixer(h, P, pre, mx, eps):
    T = h.shape[0]
    H, D, Dv = mx["heads"], mx["dim"], mx["vdim"]
    q = silu(h @ P[pre + "q"].T).reshape(T, H, D)
    k = silu(h @ P[pre + "k"].T).reshape(T, H, D)
    v = silu(h @ P[pre + "v"].T).reshape(T, H, Dv)
    o = decayed_linear_attention(q, k, v, mx["decay"]).reshape(T, H * Dv)
    o = unit_rms(o, eps) * P[pre + "norm"] * sigmoid(h @ P[pre + "g"].T)
    return o @ P[pre + "o"].T


def attention_mixer(h, P, pre, mx, eps):
    T = h.shape[0]
    H, G, D, Dv = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
    q = (h @ P[pre + "q"].T).reshape(T, H, D)
    k = (h @ P[pre + "k"].T).reshape(T, G, D)
    v = (h @ P[pre + "v"].T).reshape(T, G, Dv)
    mask = mx.get("mask") or {}
    o = log_distance_attention(q, k, v, mx["scale"], P[pre + "r1"], P[pre + "r2"], int(mask.get("size") or 0),
                               int(mask.get("keep_first") or 0))
    return o.reshape(T, H * Dv) @ P[pre + "o"].T


def left_mixer(h, P, pre, mx, eps):
    T = h.shape[0]
    H, G, D, Dv = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
    rot = mx["rot"]
    factor = float((rot.get("scaling") or {}).get("factor", 1.0))
    pos = np.arange(T)
    q = rotate_half((h @ P[pre + "q"].T).reshape(T, H, D), pos, rot["dims"], rot["base"], factor)
    k = rotate_half((h @ P[pre + "k"].T).reshape(T, G, D), pos, rot["dims"], rot["base"], factor)
    v = (h @ P[pre + "v"].T).reshape(T, G, Dv)
    o = sigmoid_attention(unit_rms(q, eps), unit_rms(k, eps), v, mx["scale"], P[pre + "pb"])
    return o.reshape(T, H * Dv) @ P[pre + "o"].T


def right_mixer(h, P, pre, mx, eps):
    T = h.shape[0]
    H, D, Dv = mx["heads"], mx["dim"], mx["vdim"]
    rot = mx["rot"]
    factor = float((rot.get("scaling") or {}).get("factor", 1.0))
    pos = np.arange(T)
    q = rotate_half((h @ P[pre + "q"].T).reshape(T, H, D), pos, rot["dims"], rot["base"], factor)
    k = rotate_half((h @ P[pre + "k"].T).reshape(T, H, D), pos, rot["dims"], rot["base"], factor) * D ** -0.5
    v = (h @ P[pre + "v"].T).reshape(T, H, Dv)
    o = unit_rms(decayed_linear_attention(q, k, v, mx["decay"]), eps).reshape(T, H * Dv)
    return (o * silu(h @ P[pre + "g"].T)) @ P[pre + "o"].T


def parallel_mixer(h, P, pre, mx, eps):
    return (mx["left_scale"] * left_mixer(h, P, pre + "left.", mx["left"], eps)
            + mx["right_scale"] * right_mixer(h, P, pre + "right.", mx["right"], eps))


def relu2_ffn(h, P, pre):
    return (np.maximum(h @ P[pre + "up"].T, 0.0) ** 2) @ P[pre + "down"].T


MIXERS = {"lightning": lightning_mixer, "attention": attention_mixer, "parallel": parallel_mixer}


def forward(cfg, P, tokens, return_layers=False):
    """cfg: the config.json dictionary; P: {tensor name: float64 array}; -> logits [T, vocab] (and the residual rows after
    every layer)"""
    eps, m = cfg["norm"]["eps"], cfg["residual_mult"]
    x = np.asarray(P["embed"], np.float64)[np.asarray(tokens)]
    rows = []
    for i, L in enumerate(cfg["layers"]):
        p = f"l{i}."
        u = input_conv(layer_norm(x, P[p + "norm1"], eps), P[p + "canon1"])
        x = x + m * MIXERS[L["type"]](u, P, p + "mix.", L["mixer"], eps)
        if L.get("mlp"):
            u = input_conv(layer_norm(x, P[p + "norm2"], eps), P[p + "canon2"])
            x = x + m * relu2_ffn(u, P, p + "mlp.")
        rows.append(x.copy())
    logits = (layer_norm(x, P["final.norm"], eps) @ P["head"].T) * cfg["logit_scale"]
    return (logits, np.stack(rows)) if return_layers else logits


# ---------------------------------------------------------------- small configurations and random weights for the tests
def lightning_layer(heads=3, dim=8, vdim=12, decay=None, ff=24):
    decay = decay or [0.5 + 0.45 * (h + 1) / heads for h in range(heads)]
    return {"type": "lightning", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)},
            "mlp": {"kind": "dense", "ff": ff} if ff else None}


def attention_layer(heads=4, kv_heads=2, dim=16, vdim=8, window=7, keep=2, scale=0.3, ff=24):
    return {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale,
                                           "mask": {"size": window, "keep_first": keep}},
            "mlp": {"kind": "dense", "ff": ff} if ff else None}


def parallel_layer(heads=4, kv_heads=2, dim=12, vdim=10, dims=8, base=300.0, factor=2.0, scale=0.4, r_heads=2, r_dim=8,
                   r_vdim=6, r_dims=None, r_base=1000.0, decay=None, left_scale=1.3, right_scale=0.6, ff=24):
    decay = decay or [0.6 + 0.39 * (h + 1) / r_heads for h in range(r_heads)]
    left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale,
            "rot": {"dims": dims, "base": base, "scaling": {"factor": factor}}}
    right = {"heads": r_heads, "dim": r_dim, "vdim": r_vdim, "decay": list(decay),
             "rot": {"dims": r_dim if r_dims is None else r_dims, "base": r_base}}
    return {"type": "parallel", "mixer": {"left": left, "right": right, "left_scale": left_scale, "right_scale": right_scale},
            "mlp": {"kind": "dense", "ff": ff} if ff else None}


def make_config(layers, vocab=90, width=40, taps=3, eps=1e-5, residual_mult=0.8, logit_scale=0.5):
    return {"architecture": "Rezulorn", "vocab": vocab, "width": width, "layers": layers, "canon": {"taps": taps},
            "norm": {"eps": eps}, "residual_mult": residual_mult, "logit_scale": logit_scale}


def random_params(cfg, seed=0):
    """{tensor name: float32 array}, rounded to bfloat16-representable values so that both modes load the same numbers"""
    rng = np.random.default_rng(seed)
    W, V, taps = cfg["width"], cfg["vocab"], cfg["canon"]["taps"]

    def bf(a):
        b = np.ascontiguousarray(a, np.float32).view(np.uint32)
        b = ((b + 0x7FFF + ((b >> 16) & 1)) & 0xFFFF0000).astype(np.uint32)
        return b.view(np.float32)

    def mat(n, k, gain=1.0):
        return bf(rng.standard_normal((n, k)) * gain / np.sqrt(k))

    P = {"embed": bf(rng.standard_normal((V, W))), "head": mat(V, W), "final.norm": bf(1.0 + 0.1 * rng.standard_normal(W))}
    for i, L in enumerate(cfg["layers"]):
        p, mx = f"l{i}.", L["mixer"]
        P[p + "norm1"] = bf(1.0 + 0.1 * rng.standard_normal(W))
        P[p + "canon1"] = bf(0.3 * rng.standard_normal((W, taps)))
        mp = p + "mix."

        def attn(pre, a, extra):
            P[pre + "q"] = mat(a["heads"] * a["dim"], W, 2.0)
            P[pre + "k"] = mat(a.get("kv_heads", a["heads"]) * a["dim"], W, 2.0)
            P[pre + "v"] = mat(a.get("kv_heads", a["heads"]) * a["vdim"], W)
            P[pre + "o"] = mat(W, a["heads"] * a["vdim"])
            for name, fn in extra.items():
                P[pre + name] = bf(fn())

        if L["type"] == "lightning":
            attn(mp, mx, {"g": lambda: mat(mx["heads"] * mx["vdim"], W),
                          "norm": lambda: 1.0 + 0.1 * rng.standard_normal(mx["heads"] * mx["vdim"])})
        elif L["type"] == "attention":
            attn(mp, mx, {"r1": lambda: rng.uniform(0.2, 1.5, mx["heads"]), "r2": lambda: rng.uniform(0.1, 2.0, mx["heads"])})
        else:
            attn(mp + "left.", mx["left"], {"pb": lambda: rng.uniform(-3.0, -1.0, mx["left"]["heads"])})
            r = mx["right"]
            attn(mp + "right.", r, {"g": lambda: mat(r["heads"] * r["vdim"], W)})
        if L.get("mlp"):
            P[p + "norm2"] = bf(1.0 + 0.1 * rng.standard_normal(W))
            P[p + "canon2"] = bf(0.3 * rng.standard_normal((W, taps)))
            P[p + "mlp.up"] = mat(L["mlp"]["ff"], W)
            P[p + "mlp.down"] = mat(W, L["mlp"]["ff"])
    return P
