"""Sonulorn `Model`: the per-model surface of the package (`language_model`, `get_input_embeddings`, `sanitize`,
`load_weights`, `engine`, `config`) for a text-only decoder whose layers read ONE normed input with all their
sublayers (decoder_blocks.SharedInputLayer): softmax attention with a sink logit and block-local keys, a decayed
outer-product state, an attention beside a gated delta rule, a clamped gated feed-forward.  A span of layers may run
several times with the same weights; every run has its own cache rows and state, and before every repetition the
stream is mixed with the embedding output through a (width, 2 width) matrix and a vector of the repetition is added.
All weights are packed into ONE device arena; the arithmetic is csrc/layer_ops.cu + csrc/mixer_ops.cu driven by
`LayerEngine`."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional

import numpy as np
import torch

from ...layer_engine import LayerEngine
from ..base import InputEmbeddingsFeatures
from ..decoder_blocks import SharedInputLayer
from ..qwen2_vl.qwen2_vl import WeightArena
from .config import ModelConfig
from .language import LanguageModel


@dataclass
class Run:
    layer: int
    repetition: Optional[int]     # which pass of the repeated span (None: outside it)
    opens_pass: bool              # the stream is re-mixed with the embedding output before this run
    kv_base: int                  # the pool's caching layer of this run's (first) attention
    state_base: int               # offset of this run's state in a slot


class Model:
    norm_offset = 0.0             # the norms' weights are stored plainly

    def __init__(self, config: ModelConfig, device=None, dtype: str = "bfloat16"):
        if dtype not in ("bfloat16", "float32"):
            raise ValueError("dtype: 'bfloat16' (serving) or 'float32' (everything in true 32-bit)")
        self.config = config
        self.exact = dtype == "float32"
        self._device = torch.device(device) if device is not None else torch.device("cuda", 0)
        self._eng: Optional[LayerEngine] = None
        self.width, self.vocab = config.width, config.vocab
        self.eps, self.embed_scale, self.logit_softcap = config.norm_eps, config.embedding_scale, None
        self.layers = [SharedInputLayer(i, c, config.width) for i, c in enumerate(config.layers)]
        self.runs, kv, st = [], 0, 0
        for i, rep, opens in config.layer_runs():
            self.runs.append(Run(i, rep, opens, kv, st))
            kv += self.layers[i].kv_layers
            st += self.layers[i].state_floats
        self.n_cache_layers, self.state_floats = kv, st
        self.row_dim = max([L.kv_dim for L in self.layers] + [0])
        self.loop = config.loop
        self.embed = self.final_norm = self.head = self.loop_in = self.loop_step = None
        self.arena: Optional[WeightArena] = None
        self.language_model = LanguageModel(config, self, self._engine)

    # ------------------------------------------------------------------ engine
    def _engine(self) -> LayerEngine:
        if self._eng is None:
            self._eng = LayerEngine(self._device, exact=self.exact)
            self._eng.bind_model(self)
        return self._eng

    @property
    def engine(self) -> LayerEngine:
        return self._engine()

    def run_layers(self, ctx, x: torch.Tensor, embed_again) -> torch.Tensor:
        """the layer runs of one step over the residual rows x (T, width) fp32; returns the rows after the last run.
        embed_again(): a fresh copy of the embedding output (the layers update x in place)"""
        ops, W = ctx.ops, self.width
        x0 = None
        for k, run in enumerate(self.runs):
            if run.opens_pass:
                if x0 is None:          # x itself is the embedding output while no layer has run
                    x0 = x if k == 0 else embed_again()
                mixed = ops.linear(x, self.loop_in[:, :W], bias=self.loop_step[run.repetition])
                x = ops.linear(x0, self.loop_in[:, W:], out=mixed, add=True)
            self.layers[run.layer].forward(ctx, x, run.kv_base, run.state_base)
        return x

    # ------------------------------------------------------------------ weights
    def _globals(self):
        W, V = self.width, self.vocab
        out = [("embed", (V, W)), ("final.norm", (W,)), ("head", (V, W))]
        if self.loop is not None:
            out += [("loop.in", (W, 2 * W)), ("loop.step", (self.loop["times"], W))]
        return out

    def manifest(self):
        out = self._globals()
        for i, L in enumerate(self.layers):
            out += L.manifest(f"l{i}.")
        return out

    def checkpoint_tensors(self) -> Dict[str, tuple]:
        """checkpoint name -> shape of every tensor this configuration reads"""
        out = dict(self._globals())
        for i, L in enumerate(self.layers):
            out.update(L.checkpoint_tensors(f"l{i}."))
        return out

    def expected_tensors(self):
        return list(self.checkpoint_tensors())

    @staticmethod
    def sanitize(weights: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
        return {k[len("model."):] if k.startswith("model.") else k: v for k, v in weights.items()}

    def _bind(self, view):
        for i, L in enumerate(self.layers):
            L.bind(f"l{i}.", view)
        self.embed, self.final_norm, self.head = view("embed"), view("final.norm"), view("head")
        if self.loop is not None:
            self.loop_in, self.loop_step = view("loop.in"), view("loop.step")

    def load_weights(self, weights: Dict[str, torch.Tensor], strict: bool = True):
        need = self.checkpoint_tensors()
        missing = [n for n in need if n not in weights]
        if missing:
            raise ValueError(f"checkpoint lacks {len(missing)} tensors, e.g. {missing[:4]}")
        wrong = [n for n, shape in need.items() if tuple(weights[n].shape) != tuple(shape)]
        if wrong:
            n = wrong[0]
            raise ValueError(f"checkpoint tensor {n} has shape {tuple(weights[n].shape)}, the configuration says {need[n]}")
        extra = sorted(set(weights) - set(need))
        if strict and extra:
            raise ValueError(f"checkpoint has {len(extra)} tensors this configuration does not use, e.g. {extra[:4]}")
        eng = self._engine()
        with torch.cuda.stream(eng.stream):
            self.arena = WeightArena(self.manifest(), eng.device)
            ck = {n: weights[n].to(device=eng.device, dtype=torch.bfloat16) for n in need}
            view = self.arena.view
            for n, _ in self._globals():
                view(n).copy_(ck[n])
            for i, L in enumerate(self.layers):
                L.pack(f"l{i}.", ck, view)
            self._bind(view)
        eng.stream.synchronize()
        return self

    def init_random(self, seed: int = 0):
        """seeded random weights of this configuration, generated on the device straight into the arena (benchmarks,
        no checkpoint): matrices N(0, 1/fan-in), norm weights around one, the other vectors small"""
        eng = self._engine()
        g = torch.Generator(device=eng.device).manual_seed(seed)
        with torch.cuda.stream(eng.stream):
            self.arena = WeightArena(self.manifest(), eng.device)
            view = self.arena.view
            for name, shape in self.manifest():
                v = view(name)
                if len(shape) == 1:
                    mean = 1.0 if name.endswith(("norm", "norm1")) else 0.0
                    v.copy_(mean + 0.05 * torch.randn(shape, generator=g, device=eng.device))
                else:
                    s = 1.0 / self.embed_scale if name == "embed" else 1.0 / float(shape[-1]) ** 0.5
                    v.copy_(torch.randn(shape, generator=g, device=eng.device) * s)
            self._bind(view)
        eng.stream.synchronize()
        return self

    # ------------------------------------------------------------------ inputs
    def get_input_embeddings(self, input_ids=None, pixel_values=None, **kwargs) -> InputEmbeddingsFeatures:
        """text only: the scaled embedding rows (1, T, width) fp32"""
        if pixel_values is not None:
            raise ValueError("Sonulorn is a text-only decoder")
        eng = self._engine()
        ids = np.asarray(input_ids.cpu() if isinstance(input_ids, torch.Tensor) else input_ids).reshape(-1)
        x = eng.ops.embed(eng.ops.to_device(ids), self.embed, self.embed_scale)
        return InputEmbeddingsFeatures(inputs_embeds=x.unsqueeze(0))
