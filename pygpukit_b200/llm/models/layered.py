"""LayeredCausalModel: decoder-only models described layer by layer (`LayeredConfig`), served token-major on the
paged cache (net-new; the reference's `CausalTransformerModel`, models/causal.py:78-1493, runs uniform stacks, one
sequence at a time, in 16 bits).

One step = one ragged batch: for every request its next tokens (a whole prompt, a portion of one, or one decoded
token), concatenated into T rows.  The residual stream, the norms, softmax, the router and every other
non-matrix-product step are float32; matrix products take bfloat16 weights with float32 accumulation (dtype
"bfloat16", the serving mode, cache in bfloat16) or float32 weights and cache (dtype "float32").  The logits of a
position depend only on the sequence's own tokens: rows of different requests meet in no reduction.

    model.step([(id, tokens, want), ...], end=[ids]) -> float32 logits [sum(len(want)), vocab] on the host
    model.generate(prompts, max_new_tokens, temperature, ...) -> list of token lists (llm/decode/ragged.py)

The step function is the only forward pass; `generate`, the scheduler and bin/trace_run all go through it.
"""
from __future__ import annotations

import os

import numpy as np

from ..._lib import api
from ...core.array import GPUArray
from ...core.dtypes import float32, int32
from ...core.stream import CudaGraph, Stream, current_stream_handle as _st
from ..buffers import RowBuffers
from ..config import LayeredConfig
from ..layers.linear import LinearRows
from ..layers.norm import RowNorm
from ..paged_cache import PagedKVCache


class StepContext:
    """Device-side description of one ragged batch (one int32 upload per step)."""

    def __init__(self, model: "LayeredCausalModel", entries, tile_sizes: set[int], tops: set[int]):
        cache = model.cache
        toks, slots, poss, want_rows, seqs, pars = [], [], [], [], [], []
        row = 0
        for seq_id, tokens, want in entries:
            n = len(tokens)
            if n < 1:
                raise ValueError(f"request {seq_id!r}: a step needs at least one token")
            slot, pos0 = cache.extend(seq_id, n)
            toks.extend(int(t) for t in tokens)
            slots.extend([slot] * n)
            poss.extend(range(pos0, pos0 + n))
            pars.extend([(cache.pool.steps(seq_id) - 1) & 1] * n)      # which copy of double-buffered state the step reads
            for w in want:
                if not 0 <= int(w) < n:
                    raise ValueError(f"request {seq_id!r}: wanted place {w} outside its {n} tokens")
                want_rows.append(row + int(w))
            seqs.append((row, n, slot, pos0))
            row += n
        self.T, self.n_want = row, len(want_rows)
        self.max_rows = max(n for _, n, _, _ in seqs)          # the longest portion of the step
        self._seqs, self._model = seqs, model
        self.decode_only = all(n == 1 and p0 > 0 for _, n, _, p0 in seqs)
        parts = [np.asarray(toks, np.int32), np.asarray(slots, np.int32), np.asarray(poss, np.int32),
                 np.asarray(want_rows, np.int32)]
        off = {"tok": 0, "slot": self.T, "pos": 2 * self.T, "want": 3 * self.T}
        cur = 3 * self.T + self.n_want
        self._rows_off = {}
        if self.T <= LinearRows.FEW:
            for top in sorted(tops):
                n = self.T * top
                parts += [np.repeat(np.arange(self.T, dtype=np.int32), top), np.arange(n, dtype=np.int32)]
                self._rows_off[top] = (cur, cur + n)
                cur += 2 * n
        self._tiles_off = {}
        for qt in sorted(tile_sizes):
            pad = (-cur) % 4                       # int4 loads: 16-byte aligned
            if pad:
                parts.append(np.zeros(pad, np.int32))
                cur += pad
            t = [(r0 + i, min(qt, n - i), slot, p0 + i) for r0, n, slot, p0 in seqs for i in range(0, n, qt)]
            parts.append(np.asarray(t, np.int32).reshape(-1))
            self._tiles_off[qt] = (cur, len(t))
            cur += 4 * len(t)
        pad = (-cur) % 4                           # one (first row, rows, slot, first position) per sequence, int4 loads
        if pad:
            parts.append(np.zeros(pad, np.int32))
            cur += pad
        parts.append(np.asarray(seqs, np.int32).reshape(-1))
        self._seqs_off = cur
        cur += 4 * len(seqs)
        parts.append(np.asarray(pars, np.int32))
        par_off = cur
        cur += self.T
        meta = np.concatenate(parts)
        self.meta = model._meta_buffer(meta.size)
        api.memcpy_h2d(self.meta.device_ptr, meta.ctypes.data, meta.nbytes, _st())
        api.stream_sync(_st()) if _st() is not None else api.device_sync()
        base = self.meta.device_ptr
        self.tok_ptr, self.slot_ptr, self.pos_ptr, self.want_ptr = (base + 4 * off[k] for k in ("tok", "slot", "pos", "want"))
        self._base = base
        self.parity_ptr = base + 4 * par_off
        cache.sync_table()
        self.cache = cache
        self.buf = model._buffers(self.T)

    def max_keys(self, chunk: int, window: int = 0, keep_first: int = 0) -> int:
        """The longest key range any tile of the step reads under a chunk size and a window (0: none) that keeps the first
        `keep_first` positions visible."""
        keys = max(p0 + n - ((p0 // chunk) * chunk if chunk > 0 else 0) for _, n, _, p0 in self._seqs)
        return min(keys, window + 64 + keep_first) if window > 0 else keys

    def seqs(self) -> tuple[int, int]:
        """(device pointer, count) of the step's sequences as (first row, rows, slot, first position)"""
        return self._base + 4 * self._seqs_off, len(self._seqs)

    def workspace(self, n_floats: int) -> GPUArray:
        return self._model._workspace(n_floats)

    def tiles(self, queries_per_tile: int) -> tuple[int, int]:
        off, n = self._tiles_off[queries_per_tile]
        return self._base + 4 * off, n

    def slot_rows(self, top: int) -> tuple[int, int]:
        """(token of every (token, slot) row, 0 .. T * top - 1) for the few-row expert path"""
        a, b = self._rows_off[top]
        return self._base + 4 * a, self._base + 4 * b


class LayeredCausalModel:
    def __init__(self, config: LayeredConfig, embed_tokens: GPUArray, blocks: list, final_norm, lm_head: LinearRows,
                 dtype: str = "bfloat16", embed_norm: RowNorm | None = None):
        """blocks: one PostNormBlock / ParallelBlock per layer of the config; final_norm: a RowNorm, or the (weight, bias)
        pair of a LayerNorm; embed_norm: the norm applied to the embedding rows (configs with `embed_norm`)."""
        self.config, self.embed_tokens, self.blocks = config, embed_tokens, blocks
        if isinstance(final_norm, tuple):
            final_norm = RowNorm("layernorm", final_norm[0], final_norm[1], config.norm_eps)
        self.final_norm, self.lm_head, self.dtype = final_norm, lm_head, dtype
        self.embed_norm = embed_norm
        if bool(config.embed_norm) != (embed_norm is not None):
            raise ValueError("LayeredCausalModel: the config and the embedding norm do not agree")
        self.runs = config.layer_runs()                 # (layer, add the embedding output first); index = cache
        self.trace_hook = None                          # debugging aid: called with (run index, residual rows array)
        self.embed_dt = 2 if embed_tokens.dtype.name == "bfloat16" else 0
        self.cache: PagedKVCache | None = None
        self._buf: RowBuffers | None = None
        self._meta: GPUArray | None = None
        self._out: GPUArray | None = None
        self._ws: GPUArray | None = None
        self.use_graphs = os.environ.get("PGK_LAYERED_GRAPH", "1") != "0"
        self._graphs: dict = {}
        self._graph_warm: set = set()
        self._gstream: Stream | None = None
        self._tile_sizes = {b.mixer.queries_per_tile for b in blocks if b.mixer.queries_per_tile}
        self._tops = {b.mlp.spec.top for b in blocks if b.mlp is not None and b.mlp.spec.kind == "moe"}

    # ------------------------------------------------------------------ setup
    def init_cache(self, max_tokens: int = 4096, page_size: int = 64, slots: int = 8) -> PagedKVCache:
        """Allocate the paged cache for about `max_tokens` live positions (it grows when more arrive)."""
        shapes = [self.blocks[li].mixer.spec.cache_shape() for li, _ in self.runs]
        states = [tuple(getattr(self.blocks[li], "state_shapes", ())) for li, _ in self.runs]
        self.cache = PagedKVCache(shapes, self.dtype, page_size, max_tokens, slots, state_shapes=states)
        self._graphs.clear()
        self._graph_warm.clear()
        return self.cache

    def _buffers(self, rows: int) -> RowBuffers:
        if self._buf is None or self._buf.rows < rows:
            self._buf = RowBuffers(self.config, max(rows, 2 * self._buf.rows if self._buf else 0))
        return self._buf

    def _workspace(self, n_floats: int) -> GPUArray:
        if self._ws is None or self._ws.size < n_floats:
            self._ws = GPUArray((max(1 << 20, 2 * n_floats),), float32)
        return self._ws

    def _meta_buffer(self, n: int) -> GPUArray:
        if self._meta is None or self._meta.size < n:
            self._meta = GPUArray((max(1024, 2 * n),), int32)
        return self._meta

    # ------------------------------------------------------------------ the step
    def _forward(self, ctx: StepContext) -> None:
        """Every launch of a step: embedding, the blocks, final norm + head of the wanted rows (into self._out)."""
        cfg = self.config
        W, V = cfg.hidden_size, cfg.vocab_size
        b, T = ctx.buf, ctx.T
        x = b.x
        en = self.embed_norm
        if en is not None and en.kind == "rmsnorm":    # embedding rows, their norm and the copy kept for later loop passes
            api.embed_norm_rows_f32(self.embed_tokens.device_ptr, self.embed_dt, ctx.tok_ptr, en.weight.device_ptr, en.offset,
                                    en.eps, x.device_ptr, b.x0.device_ptr if b.x0 is not None else None, T, W, V, _st())
        else:
            api.embed_rows_f32(self.embed_tokens.device_ptr, self.embed_dt, ctx.tok_ptr, x.device_ptr, T, W, V, _st())
            if en is not None:
                en.forward(x.device_ptr, x.device_ptr, T, W)
            if b.x0 is not None:
                api.memcpy_d2d(b.x0.device_ptr, x.device_ptr, T * W * 4, _st())
        normed, hook = False, self.trace_hook
        for run, (li, add_first) in enumerate(self.runs):
            nxt = self.runs[run + 1] if run + 1 < len(self.runs) else None
            # the block may hand the next one its normed rows (not while a hook wants to see x between the two)
            next_norm = self.blocks[nxt[0]].norm if nxt is not None and hook is None else None
            normed = self.blocks[li].forward(ctx, x, run, b.x0.device_ptr if add_first and not normed else None, normed, next_norm,
                                             b.x0.device_ptr if nxt is not None and nxt[1] else None)
            if hook is not None:
                hook(run, x.to_numpy()[:T].copy())
        if ctx.n_want:
            n = ctx.n_want
            xn = b.y                                   # free after the last block
            self.final_norm.forward(x.device_ptr, xn.device_ptr, n, W, src_rows=ctx.want_ptr)
            self.lm_head.forward(xn.device_ptr, W, n, self._out.device_ptr, V)

    def _graph_key(self, ctx: StepContext):
        """Decode steps (one token per request, few requests) replay a captured CUDA graph: the step's description
        lives in device buffers whose addresses, and every launch shape, are fixed by this key."""
        if not self.use_graphs or ctx.T > LinearRows.FEW or not ctx.decode_only:
            return None
        c = self.cache
        arrays = tuple(a.device_ptr for a in c.k if a is not None)[:1] + tuple(a.device_ptr for st in c.state for a in st)[:1]
        return (ctx.T, ctx.n_want, c.pool.max_pages, c.table_dev.device_ptr, arrays, id(ctx.buf),
                self._meta.device_ptr, self._out.device_ptr, self._ws.device_ptr if self._ws is not None else 0,
                tuple(blk.mixer.key_slices(ctx) for blk in self.blocks))

    def step_device(self, entries, end=()) -> tuple[GPUArray | None, int]:
        """Run one ragged batch; returns (float32 logits [n_want, vocab] on the device or None, n_want).  `end` names
        the requests whose cache is given back after the step."""
        if self.cache is None:
            self.init_cache()
        V = self.config.vocab_size
        if not entries:                                # nothing to run: only give back what `end` names
            for seq_id in end:
                self.cache.release(seq_id)
            return None, 0
        ctx = StepContext(self, entries, self._tile_sizes, self._tops)
        if self._out is None or self._out.shape[0] < max(ctx.n_want, 1):
            self._out = GPUArray((max(ctx.n_want, 16), V), float32)
        key = self._graph_key(ctx)
        if key is None:
            self._forward(ctx)
        else:
            g = self._graphs.get(key)
            if g is None and key not in self._graph_warm:
                self._graph_warm.add(key)              # first sight: run eagerly (kernel attributes, workspaces)
                self._forward(ctx)
                if self._graph_key(ctx) != key:        # the eager run grew a workspace: forget the stale key
                    self._graph_warm.discard(key)
            else:
                if self._gstream is None:
                    self._gstream = Stream()
                if g is None:
                    if len(self._graphs) >= 64:
                        self._graphs.clear()
                    g = CudaGraph()
                    api.device_sync()
                    with g.capture(self._gstream):
                        self._forward(ctx)
                    self._graphs[key] = g
                g.replay(self._gstream)
                self._gstream.synchronize()
        for seq_id in end:
            self.cache.release(seq_id)
        return (self._out if ctx.n_want else None), ctx.n_want

    def step(self, entries, end=()) -> np.ndarray:
        """`step_device` with the wanted logits copied to the host ([n_want, vocab] float32)."""
        out, n = self.step_device(entries, end)
        V = self.config.vocab_size
        if not n:
            api.stream_sync(_st()) if _st() is not None else api.device_sync()
            return np.zeros((0, V), np.float32)
        host = np.empty((n, V), np.float32)
        api.memcpy_d2h(host.ctypes.data, out.device_ptr, host.nbytes, _st())
        api.stream_sync(_st()) if _st() is not None else api.device_sync()
        return host

    def release(self, seq_id) -> None:
        self.cache.release(seq_id)

    def residual_rows(self, n: int) -> np.ndarray:
        """The first n rows of the residual stream as the last step left them (debugging aid)."""
        return self._buf.x.to_numpy()[:n].copy()

    # ------------------------------------------------------------------ generation
    def generate(self, prompts, max_new_tokens: int = 20, temperature: float = 0.0, top_k: int = 0, top_p: float = 1.0,
                 eos_token_id: int | None = None, prefill_chunk: int | None = None) -> list[list[int]]:
        """Generate for one prompt (a list of ints) or several (a list of lists) through the batch scheduler."""
        from ..decode.ragged import RaggedScheduler
        single = bool(prompts) and isinstance(prompts[0], (int, np.integer))
        sched = RaggedScheduler(self, prefill_chunk=prefill_chunk)
        for i, p in enumerate([prompts] if single else prompts):
            sched.add_request(i, list(p), max_new_tokens, temperature, top_k, top_p, eos_token_id)
        done = sched.run()
        outs = [done[i] for i in range(len(done))]
        return outs[0] if single else outs

    # ------------------------------------------------------------------ accounting
    def weight_bytes_per_token(self) -> int:
        return sum(self.blocks[li].weight_bytes for li, _ in self.runs) + self.lm_head.nbytes


__all__ = ["LayeredCausalModel", "StepContext"]
