"""Configuration of a Sonulorn checkpoint: `config.json` names every size and every constant that differs between
models of the design: vocabulary, width, the list of layers (each with its mixer's type and sizes and its
feed-forward, or none), the span of layers that repeats (`loop`: start, stop, times; absent: nothing repeats), the
embedding scale and the eps of the norms."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional


@dataclass
class ModelConfig:
    vocab: int = 0
    width: int = 0
    layers: List[Dict[str, Any]] = field(default_factory=list)
    loop: Optional[Dict[str, int]] = None
    embedding_scale: float = 1.0
    norm_eps: float = 1e-5
    architecture: str = "Sonulorn"
    model_type: str = "sonulorn"
    eos_token_id: Any = None

    @classmethod
    def from_dict(cls, params: dict) -> "ModelConfig":
        for key in ("vocab", "width", "layers"):
            if key not in params:
                raise ValueError(f"config.json: missing '{key}'")
        loop = params.get("loop")
        n = len(params["layers"])
        if loop is not None:
            loop = {k: int(loop[k]) for k in ("start", "stop", "times")}
            if not (0 <= loop["start"] < loop["stop"] <= n and loop["times"] >= 1):
                raise ValueError(f"config.json: loop {loop} does not fit {n} layers")
        return cls(vocab=int(params["vocab"]), width=int(params["width"]), layers=list(params["layers"]), loop=loop,
                   embedding_scale=float((params.get("embedding") or {}).get("scale", 1.0)),
                   norm_eps=float((params.get("norm") or {}).get("eps", 1e-5)),
                   architecture=params.get("architecture", "Sonulorn"), eos_token_id=params.get("eos_token_id"))

    def to_dict(self) -> dict:
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "layers": self.layers,
               "embedding": {"scale": self.embedding_scale}, "norm": {"eps": self.norm_eps}}
        if self.loop is not None:
            out["loop"] = dict(self.loop)
        return out

    def layer_runs(self):
        """(layer, repetition or None, first of its repetition) in the order the layers run"""
        n = len(self.layers)
        if self.loop is None:
            return [(i, None, False) for i in range(n)]
        a, b, times = self.loop["start"], self.loop["stop"], self.loop["times"]
        runs = [(i, None, False) for i in range(a)]
        for t in range(times):
            runs += [(i, t, i == a) for i in range(a, b)]
        return runs + [(i, None, False) for i in range(b, n)]

    # names the generic parts of the package read
    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def num_hidden_layers(self) -> int:
        return len(self.layer_runs())
