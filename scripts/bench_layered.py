"""Prefill and decode throughput of the layered (Dolurax) family at layer sizes of real models, beside the
closest existing family (Qwen3-MoE: QK-norm attention + routed experts) at equal sizes.  Run through
`python bench.py --layered [--layered-sizes a,b]`; prints ONE JSON line.  Random weights, synthetic tokens.

  dolurax     bfloat16 matrices, float32 residual / norms / softmax / router, paged cache, ragged steps:
              prefill = one step over a P-token prompt; decode = steps of one token for each of B requests.
  qwen3_moe   the package's Qwen3-MoE model with FP8 weights (its experts exist in FP8 / NVF4 only): prefill runs the
              prompt through its fixed-cache path in slabs of 64 rows, decode replays its one-graph step.

Per configuration: tokens/s, ms per step, and the step's roofline fraction -- decode against the measured HBM copy
bandwidth (weight bytes the step touches + KV bytes read), prefill against the measured bfloat16 GEMM throughput
(2 x tokens x active matrix parameters + attention products).  Timing: CUDA events on the launching stream,
3+ warm-up iterations, the weights of a step (> 1 GB) exceed the 126 MB L2.
"""
from __future__ import annotations

import json
import os
import time

import numpy as np

SIZES = {
    # name: width, heads, kv_heads, dim, vdim, chunk, experts, top, ff, groups, shared_ff, layers, vocab
    "a3b-2048": dict(width=2048, heads=32, kv_heads=4, dim=128, vdim=128, chunk=1024, experts=128, top=8, ff=768,
                     groups=(8, 4), shared_ff=0, layers=2, vocab=32768),
    "moe-4096": dict(width=4096, heads=32, kv_heads=8, dim=128, vdim=128, chunk=2048, experts=16, top=2, ff=2048,
                     groups=(4, 2), shared_ff=2048, layers=2, vocab=32768),
}


# Turutar: parallel blocks of latent attention (one cached row of kv_rank + rot per position) and windowed attention whose
# values are its keys, gated dense feed-forward, token side input; the two layers run twice (loop), i.e. four layer runs
TURUTAR_SIZES = {
    "t-2048": dict(width=2048, heads=16, kv_heads=4, dim=128, window=1024, ldim=128, rot=64, lvdim=128, kv_rank=512, q_rank=768,
                   ff=8192, side=256, times=2, vocab=32768),
    "t-4096": dict(width=4096, heads=32, kv_heads=8, dim=128, window=2048, ldim=128, rot=64, lvdim=128, kv_rank=512, q_rank=1536,
                   ff=12288, side=256, times=2, vocab=32768),
}


# Rezulorn: pre-norm blocks with input convolutions; a parallel layer (sigmoid-weighted rotary attention over the whole
# context beside rotary retention), a lightning layer (decayed linear attention, state only) and a windowed attention layer
# with kept first positions; squared-ReLU feed-forward
REZULORN_SIZES = {
    "r-2048": dict(width=2048, heads=16, kv_heads=4, dim=128, window=1024, keep=4, lin_heads=16, lin_dim=128, lin_vdim=128,
                   ff=8192, taps=4, vocab=32768),
    "r-4096": dict(width=4096, heads=32, kv_heads=8, dim=128, window=2048, keep=4, lin_heads=32, lin_dim=128, lin_vdim=128,
                   ff=12288, taps=4, vocab=32768),
}


# Sumitar: sandwich blocks with dynamic-tanh norms; a parallel layer (windowed rotary attention beside a gated linear
# recurrence, each side RMS-normed over the width) with a PolyNorm feed-forward, and a gated-delta-rule layer with a mixture of
# experts (choice bias, experts without matrices, gated shared expert)
SUMITAR_SIZES = {
    "s-2048": dict(width=2048, heads=16, kv_heads=4, dim=128, window=1024, rot=64, lin_heads=16, lin_dim=128, lin_vdim=128,
                   qk_heads=4, taps=4, ff=8192, experts=16, identity=2, top=4, eff=2048, shared_ff=2048, vocab=32768),
    "s-4096": dict(width=4096, heads=32, kv_heads=8, dim=128, window=2048, rot=64, lin_heads=32, lin_dim=128, lin_vdim=128,
                   qk_heads=8, taps=4, ff=12288, experts=16, identity=2, top=4, eff=3072, shared_ff=3072, vocab=32768),
}


def peaks(root: str) -> tuple[float, float, str]:
    p = os.path.join(root, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), float(d["bf16_tflops"]), "measured"
    return 6650.0, 1590.0, "fallback"


def layered_config(s: dict):
    from pygpukit_b200.llm.config import layered_config_from_json
    mixer = {"dim": s["dim"], "heads": s["heads"], "kv_heads": s["kv_heads"], "mask": {"size": s["chunk"]},
             "scale": s["dim"] ** -0.5, "softcap": 50.0, "v_mix": True, "vdim": s["vdim"]}
    mlp = {"expert": {"ff": s["ff"]}, "kind": "moe",
           "router": {"experts": s["experts"], "groups": {"count": s["groups"][0], "keep": s["groups"][1]}, "top": s["top"]},
           "shared": {"ff": s["shared_ff"]} if s["shared_ff"] else None}
    return layered_config_from_json({"architecture": "Dolurax", "layers": [{"type": "attention", "mixer": mixer, "mlp": mlp}
                                                                            for _ in range(s["layers"])],
                                     "logit_scale": 1.0, "logit_softcap": 30.0, "norm": {"eps": 1e-5}, "vocab": s["vocab"],
                                     "width": s["width"]})


def turutar_config(s: dict):
    from pygpukit_b200.llm.config import layered_config_from_json
    mlp = {"kind": "dense", "ff": s["ff"], "limit": 7.0}
    latent = {"type": "latent_attention", "mlp": mlp,
              "mixer": {"heads": s["heads"], "dim": s["ldim"], "rot_dim": s["rot"], "vdim": s["lvdim"], "kv_rank": s["kv_rank"],
                        "q_rank": s["q_rank"], "scale": (s["ldim"] + s["rot"]) ** -0.5, "rot": {"dims": s["rot"], "base": 10000.0}}}
    windowed = {"type": "attention", "mlp": mlp,
                "mixer": {"heads": s["heads"], "kv_heads": s["kv_heads"], "dim": s["dim"], "vdim": s["dim"], "scale": s["dim"] ** -0.5,
                          "mask": {"size": s["window"]}}}
    return layered_config_from_json({"architecture": "Turutar", "layers": [latent, windowed], "loop": {"start": 0, "stop": 2, "times": s["times"]},
                                     "norm": {"eps": 1e-6}, "token_side": {"dim": s["side"]}, "vocab": s["vocab"], "width": s["width"]})


def dense_twin_config(s: dict):
    """The closest existing model at equal size: as many Dolurax layers as Turutar layer runs, attention with the windowed
    mixer's heads and a chunk of the window's size, one expert of the same feed-forward size (top 1), no shared expert."""
    from pygpukit_b200.llm.config import layered_config_from_json
    mixer = {"dim": s["dim"], "heads": s["heads"], "kv_heads": s["kv_heads"], "mask": {"size": s["window"]},
             "scale": s["dim"] ** -0.5, "softcap": 50.0, "v_mix": False, "vdim": s["dim"]}
    mlp = {"expert": {"ff": s["ff"]}, "kind": "moe", "router": {"experts": 1, "groups": {"count": 1, "keep": 1}, "top": 1}, "shared": None}
    return layered_config_from_json({"architecture": "Dolurax", "layers": [{"type": "attention", "mixer": mixer, "mlp": mlp}
                                                                            for _ in range(int(2 * s["times"]))],
                                     "logit_scale": 1.0, "logit_softcap": 0.0, "norm": {"eps": 1e-5}, "vocab": s["vocab"], "width": s["width"]})


def rezulorn_config(s: dict):
    from pygpukit_b200.llm.config import layered_config_from_json
    mlp = {"kind": "dense", "ff": s["ff"]}
    H, G, D, Hl, Dl, Dvl = s["heads"], s["kv_heads"], s["dim"], s["lin_heads"], s["lin_dim"], s["lin_vdim"]
    decay = [1.0 - 2.0 ** (-5.0 - 5.0 * h / max(1, Hl - 1)) for h in range(Hl)]
    left = {"heads": H, "kv_heads": G, "dim": D, "vdim": D, "scale": D ** -0.5, "rot": {"dims": D, "base": 10000.0, "scaling": {"factor": 4.0}}}
    right = {"heads": Hl, "dim": Dl, "vdim": Dvl, "decay": decay, "rot": {"dims": Dl, "base": 100000.0}}
    layers = [{"type": "parallel", "mlp": mlp, "mixer": {"left": left, "right": right, "left_scale": 1.0, "right_scale": 0.75}},
              {"type": "lightning", "mlp": mlp, "mixer": {"heads": Hl, "dim": Dl, "vdim": Dvl, "decay": decay}},
              {"type": "attention", "mlp": mlp, "mixer": {"heads": H, "kv_heads": G, "dim": D, "vdim": D, "scale": D ** -0.5,
                                                           "mask": {"size": s["window"], "keep_first": s["keep"]}}}]
    return layered_config_from_json({"architecture": "Rezulorn", "layers": layers, "canon": {"taps": s["taps"]}, "norm": {"eps": 1e-6},
                                     "residual_mult": 0.5, "logit_scale": 1.0, "vocab": s["vocab"], "width": s["width"]})


def rezulorn_twin_config(s: dict):
    """The closest existing model at equal size: three Dolurax layers, attention with the same heads and a chunk of the
    window's size, one expert of the same feed-forward size (top 1, gated: three matrices to Rezulorn's two)."""
    return dense_twin_config(dict(s, times=1.5))


def rezulorn_bytes_flops(s: dict, T: int, B: int, ctx: int) -> tuple[float, float]:
    """(bytes a decode step of B tokens touches, FLOPs of a T-token prefill; linear attention counted in its recurrent form)"""
    W, H, G, D = s["width"], s["heads"], s["kv_heads"], s["dim"]
    Hl, Dl, Dvl = s["lin_heads"], s["lin_dim"], s["lin_vdim"]
    att_w = (H * D + 2 * G * D) * W + W * H * D
    lin_w = (2 * Hl * Dl + 2 * Hl * Dvl) * W + W * Hl * Dvl
    ff_w = 2 * s["ff"] * W
    weights = 2 * att_w + 2 * lin_w + 3 * ff_w
    seen = min(ctx, s["window"] + s["keep"])
    state = 2 * 4 * Hl * Dl * Dvl                                         # float32, read and written
    dec = 2 * weights + B * (2 * 2 * G * D * (ctx + seen) + 2 * state) + 2 * s["vocab"] * W
    win = s["window"]
    seen_avg = min(T, win) / 2 if T <= win else win * (1 - win / (2 * T))
    attn_fl = 2 * T * H * (T / 2) * 2 * D + 2 * T * H * seen_avg * 2 * D + 2 * T * Hl * 4 * Dl * Dvl
    return float(dec), float(2 * T * weights + attn_fl + 2 * s["vocab"] * W)


def turutar_bytes_flops(s: dict, T: int, B: int, ctx: int) -> tuple[float, float]:
    """(bytes a decode step of B tokens touches, FLOPs of a T-token prefill) over the 2 x times layer runs"""
    W, H, G, D = s["width"], s["heads"], s["kv_heads"], s["dim"]
    R, rot, hd = s["kv_rank"], s["rot"], s["ldim"] + s["rot"]
    ff_w = 3 * s["ff"] * W + 2 * s["side"] * W
    win_w = (H * D + G * D + H) * W + W * H * D
    lat_w = (s["q_rank"] + R + rot + H) * W + H * hd * s["q_rank"] + H * s["ldim"] * R + H * s["lvdim"] * R + W * H * s["lvdim"]
    seen_w = min(ctx, s["window"])
    dec = s["times"] * (2 * (win_w + lat_w + 2 * ff_w) + B * 2 * (2 * G * seen_w * D + ctx * (R + rot))) + 2 * s["vocab"] * W
    seen_avg = min(T, s["window"]) / 2 if T <= s["window"] else s["window"] * (1 - s["window"] / (2 * T))
    attn_fl = 2 * T * H * seen_avg * 2 * D + 2 * T * H * (T / 2) * (2 * R + rot)
    fl = s["times"] * (2 * T * (win_w + lat_w + 2 * ff_w) + attn_fl) + 2 * s["vocab"] * W
    return float(dec), float(fl)


def twin_bytes_flops(s: dict, T: int, B: int, ctx: int) -> tuple[float, float]:
    W, H, G, D = s["width"], s["heads"], s["kv_heads"], s["dim"]
    layer_w = (H * D + 2 * G * D + H * D) * W + W * H * D + W + 3 * s["ff"] * W
    seen = min(ctx, s["window"])
    n = 2 * s["times"]
    dec = n * (2 * layer_w + B * 2 * 2 * G * seen * D) + 2 * s["vocab"] * W
    seen_avg = min(T, s["window"]) / 2
    fl = n * (2 * T * layer_w + 2 * T * H * seen_avg * 2 * D) + 2 * s["vocab"] * W
    return float(dec), float(fl)


def sumitar_config(s: dict):
    from pygpukit_b200.llm.config import layered_config_from_json
    H, G, D, Hl, Dl, Dvl = s["heads"], s["kv_heads"], s["dim"], s["lin_heads"], s["lin_dim"], s["lin_vdim"]
    left = {"heads": H, "kv_heads": G, "dim": D, "vdim": D, "scale": D ** -0.5, "mask": {"size": s["window"]},
            "rot": {"dims": s["rot"], "base": 10000.0}}
    moe = {"kind": "moe", "expert": {"ff": s["eff"]}, "router": {"experts": s["experts"], "identity": s["identity"], "top": s["top"]},
           "shared": {"ff": s["shared_ff"]}}
    layers = [{"type": "parallel", "mlp": {"kind": "dense", "ff": s["ff"]},
               "mixer": {"left": left, "right": {"heads": Hl, "dim": Dl, "vdim": Dvl}}},
              {"type": "delta", "mlp": moe, "mixer": {"heads": Hl, "kv_heads": s["qk_heads"], "dim": Dl, "vdim": Dvl, "conv": s["taps"]}}]
    return layered_config_from_json({"architecture": "Sumitar", "layers": layers, "norm": {"eps": 1e-6}, "vocab": s["vocab"],
                                     "width": s["width"]})


def sumitar_twin_config(s: dict):
    """The closest existing model at equal size: a Rezulorn stack of a parallel layer (rotary attention beside rotary retention
    with per-sequence state) and a lightning layer (decayed linear attention, state only), the same heads, squared-ReLU
    feed-forward of the dense size in both."""
    from pygpukit_b200.llm.config import layered_config_from_json
    mlp = {"kind": "dense", "ff": s["ff"]}
    H, G, D, Hl, Dl, Dvl = s["heads"], s["kv_heads"], s["dim"], s["lin_heads"], s["lin_dim"], s["lin_vdim"]
    decay = [1.0 - 2.0 ** (-5.0 - 5.0 * h / max(1, Hl - 1)) for h in range(Hl)]
    left = {"heads": H, "kv_heads": G, "dim": D, "vdim": D, "scale": D ** -0.5, "rot": {"dims": D, "base": 10000.0}}
    right = {"heads": Hl, "dim": Dl, "vdim": Dvl, "decay": decay, "rot": {"dims": Dl, "base": 100000.0}}
    layers = [{"type": "parallel", "mlp": mlp, "mixer": {"left": left, "right": right, "left_scale": 1.0, "right_scale": 0.75}},
              {"type": "lightning", "mlp": mlp, "mixer": {"heads": Hl, "dim": Dl, "vdim": Dvl, "decay": decay}}]
    return layered_config_from_json({"architecture": "Rezulorn", "layers": layers, "canon": {"taps": s["taps"]}, "norm": {"eps": 1e-6},
                                     "residual_mult": 0.5, "logit_scale": 1.0, "vocab": s["vocab"], "width": s["width"]})


def sumitar_bytes_flops(s: dict, T: int, B: int, ctx: int) -> tuple[float, float]:
    """(bytes a decode step of B tokens touches, FLOPs of a T-token prefill; the recurrences counted in their recurrent form)"""
    W, H, G, D = s["width"], s["heads"], s["kv_heads"], s["dim"]
    Hl, Dl, Dvl, Gq = s["lin_heads"], s["lin_dim"], s["lin_vdim"], s["qk_heads"]
    par_w = (H * D + 2 * G * D + 2 * Hl * Dl + Hl * Dvl) * W + W * H * D + W * Hl * Dvl
    delta_w = (2 * Gq * Dl + 2 * Hl * Dvl + 2 * Hl) * W + W * Hl * Dvl
    dense_w = 2 * s["ff"] * W
    routes = s["experts"] + s["identity"]
    moe_fix = (routes + 1) * W * 2 + 3 * s["shared_ff"] * W              # the router is float32: twice the bytes per element
    act = min(s["experts"], B * s["top"])
    state = 2 * 4 * Hl * Dl * Dvl                                         # float32, read and written, per recurrent mixer
    seen = min(ctx, s["window"])
    dec = 2 * (par_w + delta_w + dense_w + moe_fix + act * 3 * s["eff"] * W) + B * (2 * 2 * G * D * seen + 2 * state) + 2 * s["vocab"] * W
    win = s["window"]
    seen_avg = min(T, win) / 2 if T <= win else win * (1 - win / (2 * T))
    share = s["experts"] / routes                                         # chosen experts that have matrices, on average
    per_tok = par_w + delta_w + dense_w + routes * W + 3 * s["shared_ff"] * W + s["top"] * share * 3 * s["eff"] * W
    attn_fl = 2 * T * H * seen_avg * 2 * D + 2 * T * Hl * 3 * Dl * Dvl + 2 * T * Hl * 4 * Dl * Dvl
    return float(dec), float(2 * T * per_tok + attn_fl + 2 * s["vocab"] * W)


def sumitar_twin_bytes_flops(s: dict, T: int, B: int, ctx: int) -> tuple[float, float]:
    W, H, G, D = s["width"], s["heads"], s["kv_heads"], s["dim"]
    Hl, Dl, Dvl = s["lin_heads"], s["lin_dim"], s["lin_vdim"]
    att_w = (H * D + 2 * G * D) * W + W * H * D
    lin_w = (2 * Hl * Dl + 2 * Hl * Dvl) * W + W * Hl * Dvl
    weights = att_w + 2 * lin_w + 2 * 2 * s["ff"] * W
    state = 2 * 4 * Hl * Dl * Dvl
    dec = 2 * weights + B * (2 * 2 * G * D * ctx + 2 * state) + 2 * s["vocab"] * W
    attn_fl = 2 * T * H * (T / 2) * 2 * D + 2 * 2 * T * Hl * 4 * Dl * Dvl
    return float(dec), float(2 * T * weights + attn_fl + 2 * s["vocab"] * W)


def _timed(fn, iters: int, warm: int) -> float:
    """ms per call of fn() (CUDA events on the default stream)."""
    from pygpukit_b200._lib import api
    from pygpukit_b200.core.stream import CudaEvent, event_elapsed_ms
    for _ in range(warm):
        fn()
    api.device_sync()
    e0, e1 = CudaEvent(), CudaEvent()
    api.event_record(e0.handle, None)
    for _ in range(iters):
        fn()
    api.event_record(e1.handle, None)
    e1.synchronize()
    return event_elapsed_ms(e0, e1) / iters


def dolurax_bytes_flops(s: dict, T: int, B: int, ctx: int) -> tuple[float, float]:
    """(bytes a decode step of B tokens touches, FLOPs of a T-token prefill)"""
    W, H, G, D, Dv = s["width"], s["heads"], s["kv_heads"], s["dim"], s["vdim"]
    attn_w = (H * D + G * D + G * Dv + H * Dv) * W + W * H * Dv
    expert_w = 3 * s["ff"] * W
    shared_w = 3 * s["shared_ff"] * W
    act_experts = min(s["experts"], B * s["top"])
    seen = min(ctx, s["chunk"]) if s["chunk"] else ctx
    layer_bytes = 2 * (attn_w + s["experts"] * W + act_experts * expert_w + shared_w) + B * 2 * G * seen * (D + Dv)
    dec = s["layers"] * layer_bytes + 2 * s["vocab"] * W
    per_tok = attn_w + s["experts"] * W + s["top"] * expert_w + shared_w
    seen_avg = min(T, s["chunk"] or T) / 2
    fl = s["layers"] * (2 * T * per_tok + 2 * T * H * seen_avg * (D + Dv)) + 2 * s["vocab"] * W
    return float(dec), float(fl)


def run_dolurax(s: dict, prompt: int, decode_batches, steps: int, warm: int, hbm: float, tflops: float) -> dict:
    return run_layered(layered_config(s), lambda T, B, ctx: dolurax_bytes_flops(s, T, B, ctx), s["vocab"], prompt, decode_batches,
                       steps, warm, hbm, tflops)


def run_layered(cfg, bytes_flops, vocab: int, prompt: int, decode_batches, steps: int, warm: int, hbm: float, tflops: float) -> dict:
    from pygpukit_b200 import llm
    from pygpukit_b200._lib import api, load
    s = {"vocab": vocab}
    t0 = time.perf_counter()
    model = llm.random_layered_model(cfg)
    model.init_cache(max_tokens=prompt * (max(decode_batches) + 1) + 4096, page_size=64, slots=16)
    api.device_sync()
    out = {"build_s": round(time.perf_counter() - t0, 2)}
    rng = np.random.default_rng(0)
    toks = [int(t) for t in rng.integers(0, s["vocab"], prompt)]
    n = [0]

    def prefill():
        n[0] += 1
        model.step([(("p", n[0]), toks, [prompt - 1])], end=[("p", n[0])])
    lib = load()
    prefill()
    lib.pgk_launch_count_reset()
    prefill()
    out["prefill_launches"] = int(lib.pgk_launch_count())
    ms = _timed(prefill, max(3, steps // 8), 2)
    _, fl = bytes_flops(prompt, 1, prompt)
    out["prefill"] = {"tokens": prompt, "ms": round(ms, 3), "tokens_per_s": round(prompt / ms * 1e3, 1),
                      "tflops": round(fl / ms / 1e9, 2), "frac_of_bf16_peak": round(fl / ms / 1e9 / tflops, 4)}
    out["decode"] = {}
    for B in decode_batches:
        ids = [("d", B, i) for i in range(B)]
        model.step([(i, toks, []) for i in ids])
        cur = [1]

        def dec():
            cur[0] += 1
            model.step([(i, [(cur[0] * 7919 + k) % s["vocab"]], [0]) for k, i in enumerate(ids)])
        lib.pgk_launch_count_reset()
        dec()
        launches = int(lib.pgk_launch_count())
        ms = _timed(dec, steps, warm)
        by, _ = bytes_flops(1, B, prompt)
        out["decode"][f"b{B}"] = {"ms_per_step": round(ms, 4), "tokens_per_s": round(B / ms * 1e3, 1), "launches": launches,
                                  "bytes_per_step": by, "gbs": round(by / ms / 1e6, 1), "frac_of_hbm_peak": round(by / ms / 1e6 / hbm, 4)}
        for i in ids:
            model.release(i)
    return out


def run_qwen3_moe(s: dict, prompt: int, decode_batches, steps: int, warm: int, hbm: float, tflops: float) -> dict:
    from pygpukit_b200 import llm
    from pygpukit_b200._lib import api
    from pygpukit_b200.core.stream import use_stream
    from pygpukit_b200.llm.config import QWEN3_MOE_SPEC, TransformerConfig
    ctx = prompt + steps + warm + 64
    cfg = TransformerConfig(vocab_size=s["vocab"], hidden_size=s["width"], num_layers=s["layers"], num_heads=s["heads"],
                            num_kv_heads=s["kv_heads"], intermediate_size=s["ff"], _head_dim=s["dim"], num_experts=s["experts"],
                            num_experts_per_tok=s["top"], moe_intermediate_size=s["ff"], norm_eps=1e-6, rope_theta=1e6,
                            max_position_embeddings=ctx, tie_word_embeddings=False)
    t0 = time.perf_counter()
    model = llm.build_random_model("bench", "fp8", max_seq=ctx, config=cfg, spec=QWEN3_MOE_SPEC)
    model.init_decode(ctx, max_batch_size=64)
    api.device_sync()
    out = {"build_s": round(time.perf_counter() - t0, 2), "weights": "fp8"}
    rng = np.random.default_rng(0)
    toks = [int(t) for t in rng.integers(0, s["vocab"], prompt)]
    ms = _timed(lambda: model.prefill(toks), 3, 1)
    W, H, G, D = s["width"], s["heads"], s["kv_heads"], s["dim"]
    per_tok = (H * D + 2 * G * D) * W + W * H * D + s["experts"] * W + s["top"] * 3 * s["ff"] * W
    fl = s["layers"] * (2 * prompt * per_tok + 2 * prompt * H * (prompt / 2) * 2 * D) + 2 * s["vocab"] * W
    out["prefill"] = {"tokens": prompt, "ms": round(ms, 3), "tokens_per_s": round(prompt / ms * 1e3, 1),
                      "tflops": round(fl / ms / 1e9, 2), "frac_of_bf16_peak": round(fl / ms / 1e9 / tflops, 4)}
    out["decode"] = {}
    for B in decode_batches:
        model.init_decode(ctx, max_batch_size=1, num_sequences=B) if B > 1 else model.init_decode(ctx, max_batch_size=1)
        model.init_decode_graph()
        with use_stream(model._graph_stream):
            model.set_decode_state([5] * B if B > 1 else 5, prompt)
            for _ in range(warm):
                model.decode_graph_replay()
            model._graph_stream.synchronize()
            from pygpukit_b200.core.stream import CudaEvent, event_elapsed_ms
            e0, e1 = CudaEvent(), CudaEvent()
            api.event_record(e0.handle, model._graph_stream.handle)
            for _ in range(steps):
                model.decode_graph_replay()
            api.event_record(e1.handle, model._graph_stream.handle)
            e1.synchronize()
            ms = event_elapsed_ms(e0, e1) / steps
        by = model.weight_bytes_per_token() + B * model.kv_bytes_per_token(prompt)
        if B > 1:       # weight_bytes_per_token counts `top` experts: B tokens touch up to B x top
            by += s["layers"] * (min(s["experts"], B * s["top"]) - s["top"]) * 3 * s["ff"] * W
        out["decode"][f"b{B}"] = {"ms_per_step": round(ms, 4), "tokens_per_s": round(B / ms * 1e3, 1), "bytes_per_step": float(by),
                                  "gbs": round(by / ms / 1e6, 1), "frac_of_hbm_peak": round(by / ms / 1e6 / hbm, 4)}
    return out


def main_turutar(root: str, sizes: list[str], steps: int, warm: int, prompt: int = 2000) -> dict:
    """Turutar beside its dense twin of the same family at equal size: prefill of `prompt` tokens, decode of 1 and 8
    requests at that context."""
    from pygpukit_b200._lib import api
    hbm, tflops, src = peaks(root)
    res = {"metric": "turutar_prefill_decode_tokens_per_s", "data": "synthetic", "dtype": "bf16 matrices and cache, f32 residual / norms / softmax",
           "peaks": {"hbm_gbs": hbm, "bf16_tflops": tflops, "source": src}, "prompt": prompt, "steps": steps, "warmup": warm, "sizes": {}}
    for name in sizes:
        s = TURUTAR_SIZES[name]
        entry = {"shape": dict(s)}
        entry["turutar"] = run_layered(turutar_config(s), lambda T, B, ctx: turutar_bytes_flops(s, T, B, ctx), s["vocab"], prompt,
                                       (1, 8), steps, max(3, warm), hbm, tflops)
        api.device_sync()
        entry["dolurax_dense_twin"] = run_layered(dense_twin_config(s), lambda T, B, ctx: twin_bytes_flops(s, T, B, ctx), s["vocab"],
                                                  prompt, (1, 8), steps, max(3, warm), hbm, tflops)
        api.device_sync()
        res["sizes"][name] = entry
    return res


def main_rezulorn(root: str, sizes: list[str], steps: int, warm: int, prompt: int = 2000) -> dict:
    """Rezulorn beside a dense Dolurax stack of the same family at equal size: prefill of `prompt` tokens, decode of 1 and 8
    requests at that context."""
    from pygpukit_b200._lib import api
    hbm, tflops, src = peaks(root)
    res = {"metric": "rezulorn_prefill_decode_tokens_per_s", "data": "synthetic",
           "dtype": "bf16 matrices and cache, f32 residual / norms / scores / recurrent state",
           "peaks": {"hbm_gbs": hbm, "bf16_tflops": tflops, "source": src}, "prompt": prompt, "steps": steps, "warmup": warm, "sizes": {}}
    for name in sizes:
        s = REZULORN_SIZES[name]
        entry = {"shape": dict(s)}
        entry["rezulorn"] = run_layered(rezulorn_config(s), lambda T, B, ctx: rezulorn_bytes_flops(s, T, B, ctx), s["vocab"], prompt,
                                        (1, 8), steps, max(3, warm), hbm, tflops)
        api.device_sync()
        twin = dict(s, times=1.5)
        entry["dolurax_dense_twin"] = run_layered(rezulorn_twin_config(s), lambda T, B, ctx: twin_bytes_flops(twin, T, B, ctx), s["vocab"],
                                                  prompt, (1, 8), steps, max(3, warm), hbm, tflops)
        api.device_sync()
        res["sizes"][name] = entry
    return res


def main_sumitar(root: str, sizes: list[str], steps: int, warm: int, prompt: int = 2000) -> dict:
    """Sumitar beside a Rezulorn stack of the same family at equal size (a parallel layer and a state-only layer): prefill of
    `prompt` tokens, decode of 1 and 8 requests at that context."""
    from pygpukit_b200._lib import api
    hbm, tflops, src = peaks(root)
    res = {"metric": "sumitar_prefill_decode_tokens_per_s", "data": "synthetic",
           "dtype": "bf16 matrices and cache, f32 residual / norms / scores / router / recurrent state",
           "peaks": {"hbm_gbs": hbm, "bf16_tflops": tflops, "source": src}, "prompt": prompt, "steps": steps, "warmup": warm, "sizes": {}}
    for name in sizes:
        s = SUMITAR_SIZES[name]
        entry = {"shape": dict(s)}
        entry["sumitar"] = run_layered(sumitar_config(s), lambda T, B, ctx: sumitar_bytes_flops(s, T, B, ctx), s["vocab"], prompt,
                                       (1, 8), steps, max(3, warm), hbm, tflops)
        api.device_sync()
        entry["rezulorn_twin"] = run_layered(sumitar_twin_config(s), lambda T, B, ctx: sumitar_twin_bytes_flops(s, T, B, ctx), s["vocab"],
                                             prompt, (1, 8), steps, max(3, warm), hbm, tflops)
        api.device_sync()
        res["sizes"][name] = entry
    return res


def main(root: str, sizes: list[str], steps: int, warm: int, prompt: int = 2000) -> dict:
    from pygpukit_b200._lib import api
    hbm, tflops, src = peaks(root)
    res = {"metric": "layered_prefill_decode_tokens_per_s", "data": "synthetic", "dtype": "bf16 matrices, f32 residual (dolurax); fp8 weights, bf16 activations (qwen3_moe)",
           "peaks": {"hbm_gbs": hbm, "bf16_tflops": tflops, "source": src}, "prompt": prompt, "steps": steps, "warmup": warm, "sizes": {}}
    for name in sizes:
        s = SIZES[name]
        entry = {"shape": {k: (list(v) if isinstance(v, tuple) else v) for k, v in s.items()}}
        entry["dolurax"] = run_dolurax(s, prompt, (1, 8), steps, max(3, warm), hbm, tflops)
        api.device_sync()
        try:
            entry["qwen3_moe"] = run_qwen3_moe(s, prompt, (1, 8), steps, max(3, warm), hbm, tflops)
        except Exception as e:      # a shape the older family's kernels refuse is reported, not hidden
            entry["qwen3_moe"] = {"unavailable": f"{type(e).__name__}: {e}"[:300]}
        res["sizes"][name] = entry
    return res
