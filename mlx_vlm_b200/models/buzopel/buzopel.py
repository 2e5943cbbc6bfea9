"""Buzopel `Model`: the per-model contract of the package (`language_model`, `get_input_embeddings`, `sanitize`,
`load_weights`, `engine`, `config`) for a text-only decoder built from decoder_blocks (latent attention with
borrowed latents, expert mixtures, norms on the sublayers' outputs, soft-capped logits).  All weights are packed
into ONE device arena; the arithmetic is csrc/layer_ops.cu driven by `LayerEngine`."""
from __future__ import annotations

from typing import Dict, Optional

import numpy as np
import torch

from ...layer_engine import LayerEngine
from ..base import InputEmbeddingsFeatures
from ..decoder_blocks import PostNormLayer, assign_cache_layers
from ..qwen2_vl.qwen2_vl import WeightArena
from .config import ModelConfig
from .language import LanguageModel


class Model:
    def __init__(self, config: ModelConfig, device=None, dtype: str = "bfloat16"):
        if dtype not in ("bfloat16", "float32"):
            raise ValueError("dtype: 'bfloat16' (serving) or 'float32' (everything in true 32-bit)")
        self.config = config
        self.exact = dtype == "float32"
        self._device = torch.device(device) if device is not None else torch.device("cuda", 0)
        self._eng: Optional[LayerEngine] = None
        # the core the engine runs: embedding, layers, final norm, head
        self.width, self.vocab = config.width, config.vocab
        self.eps, self.embed_scale, self.logit_softcap = config.norm_eps, config.embedding_scale, config.logit_softcap
        self.layers = [PostNormLayer(i, c, config.width) for i, c in enumerate(config.layers)]
        self.n_cache_layers = assign_cache_layers(self.layers)
        self.row_dim = max(L.mixer.row_dim for L in self.layers)
        self.embed = self.final_norm = self.head = None
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

    # ------------------------------------------------------------------ weights
    def manifest(self):
        out = [("embed", (self.vocab, self.width)), ("final.norm", (self.width,)), ("head", (self.vocab, self.width))]
        for i, L in enumerate(self.layers):
            out += L.manifest(f"l{i}.")
        return out

    @staticmethod
    def sanitize(weights: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
        return {k[len("model."):] if k.startswith("model.") else k: v for k, v in weights.items()}

    def expected_tensors(self):
        """checkpoint names this configuration needs"""
        names = ["embed", "final.norm", "head"]
        for i, L in enumerate(self.layers):
            p, m = f"l{i}.", L.mixer
            names += [p + "norm1"] + [p + "mix." + n for n in ("dq", "dq.norm", "uq", "uk", "uv", "o")]
            if m.own_kv:
                names += [p + "mix.dkv", p + "mix.dkv.norm"]
            if L.ff is not None:
                names += [p + "norm2", p + "mlp.router", p + "mlp.router.b"]
                names += [p + f"mlp.e{e}.{n}" for e in range(L.ff.E) for n in ("up", "down")]
        return names

    def load_weights(self, weights: Dict[str, torch.Tensor], strict: bool = True):
        need = self.expected_tensors()
        missing = [n for n in need if n not in weights]
        if missing:
            raise ValueError(f"checkpoint lacks {len(missing)} tensors, e.g. {missing[:4]}")
        extra = sorted(set(weights) - set(need))
        if strict and extra:
            raise ValueError(f"checkpoint has {len(extra)} tensors this configuration does not use, e.g. {extra[:4]}")
        eng = self._engine()
        with torch.cuda.stream(eng.stream):
            self.arena = WeightArena(self.manifest(), eng.device)
            ck = {n: weights[n].to(device=eng.device, dtype=torch.bfloat16) for n in need}
            view = self.arena.view
            for n in ("embed", "final.norm", "head"):
                view(n).copy_(ck[n])
            for i, L in enumerate(self.layers):
                L.pack(f"l{i}.", ck, view)
            self.embed, self.final_norm, self.head = view("embed"), view("final.norm"), view("head")
        eng.stream.synchronize()
        return self

    def init_random(self, seed: int = 0):
        """seeded random weights of this configuration, generated on the device straight into the arena
        (benchmarks, no checkpoint): matrices N(0, 1/fan-in), norm weights around their neutral value"""
        eng = self._engine()
        g = torch.Generator(device=eng.device).manual_seed(seed)
        with torch.cuda.stream(eng.stream):
            self.arena = WeightArena(self.manifest(), eng.device)
            view = self.arena.view
            for name, shape in self.manifest():
                v = view(name)
                if len(shape) == 1:
                    mean = 1.0 if name.endswith(("dq.norm", "dkv.norm")) else 0.0
                    v.copy_(mean + 0.05 * torch.randn(shape, generator=g, device=eng.device))
                else:
                    s = 1.0 / self.embed_scale if name == "embed" else 1.0 / float(shape[-1]) ** 0.5
                    for part in (v.unbind(0) if v.numel() > (1 << 28) else (v,)):     # bounded fp32 staging
                        part.copy_(torch.randn(part.shape, generator=g, device=eng.device) * s)
            for i, L in enumerate(self.layers):
                L.bind(f"l{i}.", view)
            self.embed, self.final_norm, self.head = view("embed"), view("final.norm"), view("head")
        eng.stream.synchronize()
        return self

    def _ckpt_shape(self, name: str):
        W, V = self.width, self.vocab
        if name in ("embed", "head"):
            return (V, W)
        if name == "final.norm":
            return (W,)
        i, rest = name[1:].split(".", 1)
        L = self.layers[int(i)]
        m, f = L.mixer, L.ff
        table = {"norm1": (W,), "norm2": (W,), "mix.dq": (m.q_rank, W), "mix.dq.norm": (m.q_rank,),
                 "mix.uq": (m.H * (m.dim + m.rot_dim), m.q_rank), "mix.dkv": (m.row_dim, W),
                 "mix.dkv.norm": (m.kv_rank,), "mix.uk": (m.H * m.dim, m.kv_rank), "mix.uv": (m.H * m.vdim, m.kv_rank),
                 "mix.o": (W, m.H * m.vdim)}
        if f is not None:
            table.update({"mlp.router": (f.E, W), "mlp.router.b": (f.E,)})
            if rest.endswith(".up"):
                return (f.ff, W)
            if rest.endswith(".down") and rest.startswith("mlp.e"):
                return (W, f.ff)
        return table[rest]

    # ------------------------------------------------------------------ contract
    def get_input_embeddings(self, input_ids=None, pixel_values=None, **kwargs) -> InputEmbeddingsFeatures:
        """text only: the scaled embedding rows (1, T, width) fp32"""
        if pixel_values is not None:
            raise ValueError("Buzopel is a text-only decoder")
        eng = self._engine()
        ids = np.asarray(input_ids.cpu() if isinstance(input_ids, torch.Tensor) else input_ids).reshape(-1)
        x = eng.ops.embed(eng.ops.to_device(ids), self.embed, self.embed_scale)
        return InputEmbeddingsFeatures(inputs_embeds=x.unsqueeze(0))
