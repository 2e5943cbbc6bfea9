"""Buzopel language model: the call surface the generation loops use (`__call__`, `make_cache`,
`make_cache_row`, `make_pool`, `fused_greedy_decode_n`, `prefill_rows`) over the engine's one step function.

A request's cache is a slot of a `LatentPool`; per layer a `LatentCache` view (the layers that borrow another
layer's latent hold shared views of that layer's rows).  `step()` is the core: the tokens that every request of
the step brings are concatenated, each token knows its slot and position."""
from __future__ import annotations

from typing import List, Optional, Sequence

import numpy as np
import torch

from ..base import LanguageModelOutput
from ..cache import LatentCache, LatentPool


def _np(x, dtype=np.int64):
    if x is None:
        return None
    if isinstance(x, torch.Tensor):
        return x.detach().cpu().numpy().astype(dtype)
    return np.asarray(x, dtype=dtype)


class LanguageModel:
    supports_logits_to_keep = True

    def __init__(self, args, core, engine_getter):
        self.args = args
        self.config = args
        self.core = core
        self.model_type = "buzopel"
        self._engine = engine_getter

    # ------------------------------------------------------------------ cache
    @property
    def layers(self):
        return list(range(len(self.core.layers)))

    def make_pool(self, rows: int = 1, capacity: int = 0) -> LatentPool:
        eng = self._engine()
        with torch.cuda.stream(eng.stream):
            return LatentPool(self.core.n_cache_layers, self.core.row_dim, eng.device, batch=rows, capacity=capacity,
                              dtype=eng.ops.cache_dtype)

    def make_cache_row(self, pool: LatentPool, row: int) -> List[LatentCache]:
        return [LatentCache(pool, L.mixer.cache_index, row, latent_dim=L.mixer.kv_rank, shared=not L.mixer.own_kv)
                for L in self.core.layers]

    def make_cache(self) -> List[LatentCache]:
        return self.make_cache_row(self.make_pool(1), 0)

    def _bind(self, caches: Sequence[List[LatentCache]], need_tokens: int) -> LatentPool:
        pool = caches[0][0]._pool
        if any(c[0]._pool is not pool for c in caches):
            raise ValueError("the requests of a step live in slots of ONE pool")
        eng = self._engine()
        if pool.capacity < need_tokens:
            eng.stream.synchronize()
            with torch.cuda.stream(eng.stream):
                pool.reserve(need_tokens, live_tokens=pool.capacity)
        eng.bind_pool(pool)
        return pool

    # ------------------------------------------------------------------ the step
    def step(self, token_lists: Sequence[Sequence[int]], caches: Sequence[List[LatentCache]],
             want: Optional[Sequence[Sequence[int]]] = None, reserve_tokens: int = 0,
             embeds: Optional[torch.Tensor] = None) -> torch.Tensor:
        """One forward over the tokens each request brings (request g: token_lists[g], continuing the cache
        caches[g]).  want[g]: places among request g's tokens whose logits are returned (default: its last token),
        in the order of the requests.  Returns fp32 logits (sum len(want[g]), vocab) on the device."""
        eng = self._engine()
        lens = [len(t) for t in token_lists]
        offs = [int(c[0].offset) for c in caches]
        self._bind(caches, max([o + n for o, n in zip(offs, lens)] + [reserve_tokens]))
        T = sum(lens)
        meta = np.empty((3, T), dtype=np.int32)
        rows, at, segments = [], 0, []
        for g, (toks, c, n, o) in enumerate(zip(token_lists, caches, lens, offs)):
            segments.append((at, n, int(c[0]._row), o))
            meta[0, at:at + n] = np.asarray(toks, dtype=np.int32)
            meta[1, at:at + n] = c[0]._row
            meta[2, at:at + n] = np.arange(o, o + n, dtype=np.int32)
            w = [n - 1] if want is None else list(want[g])
            if any(k < 0 or k >= n for k in w):
                raise IndexError("want: a place outside the tokens of the step")
            rows += [at + k for k in w]
            at += n
        dev = eng.ops.to_device(meta)
        all_rows = len(rows) == T and rows == list(range(T))
        want_dev = None if all_rows else (eng.ops.to_device(np.asarray(rows, dtype=np.int32)) if rows else None)
        if not rows:   # nothing wanted: the cache is still filled
            want_dev = eng.ops.to_device(np.asarray([T - 1], dtype=np.int32))
        logits = eng.forward(dev[0], dev[1], dev[2], want_dev, embeds=embeds, segments=segments)
        for c, n in zip(caches, lens):
            for layer_cache in c:
                layer_cache.offset += n
        return logits if rows else logits[:0]

    # ------------------------------------------------------------------ call
    def __call__(self, inputs, inputs_embeds=None, mask=None, cache=None, **kwargs):
        logits_to_keep = kwargs.pop("logits_to_keep", None)
        reserve = int(kwargs.pop("reserve_tokens", 0))
        ids = _np(inputs)
        if ids.ndim == 1:
            ids = ids[None]
        B, L = ids.shape
        if B != 1:
            raise ValueError("several rows per call go through step() / prefill_rows() with one cache per request")
        if cache is None or cache[0] is None:
            cache = self.make_cache()
        eng = self._engine()
        keep_last = logits_to_keep == 1
        emb = None if inputs_embeds is None else inputs_embeds.reshape(-1, inputs_embeds.shape[-1])
        logits = self.step([ids[0].tolist()], [cache], want=None if keep_last else [list(range(L))],
                           reserve_tokens=reserve, embeds=emb)
        # the greedy pick of the last row goes to the token log and arms the device decode loop
        eng.sample_prefill(logits[-1:], [int(cache[0].offset)], [cache[0]._row])
        return LanguageModelOutput(logits=logits.unsqueeze(0))

    def fused_greedy_decode_n(self, n_steps: int, cache, reserve_tokens: int = 0):
        """`n_steps` greedy steps on the device (argmax feeds the next step); tokens land in the engine's log"""
        eng = self._engine()
        off = int(cache[0].offset)
        self._bind([cache], max(off + n_steps, reserve_tokens))
        eng.decode(n_steps)
        for c in cache:
            c.offset += n_steps

    def prefill_rows(self, ids_list, embeds_list, caches, position_ids_list=None, rope_deltas_list=None,
                     reserve_tokens: int = 0) -> List[int]:
        """fresh prompts admitted together: ONE step over all of them; returns each prompt's first greedy token"""
        eng = self._engine()
        toks = [_np(i).reshape(-1).tolist() for i in ids_list]
        logits = self.step(toks, caches, reserve_tokens=reserve_tokens)
        start = eng.tokens_launched
        eng.sample_prefill(logits, [int(c[0].offset) for c in caches], [c[0]._row for c in caches])
        host = torch.empty(len(toks), dtype=torch.int32).pin_memory()
        eng.fetch_tokens(start, len(toks), host)
        eng.stream.synchronize()
        return [int(t) for t in host]

    @property
    def n_kv_heads(self) -> int:
        return 1

    @property
    def head_dim(self) -> int:
        return self.core.row_dim
