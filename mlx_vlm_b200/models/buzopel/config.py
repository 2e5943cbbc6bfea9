"""Configuration of a Buzopel checkpoint: `config.json` names every size and every constant that differs
between models of the design (vocabulary, width, the list of layers with each mixer's and feed-forward's sizes,
the embedding scale, the eps of the norms, the soft cap of the logits)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional


@dataclass
class ModelConfig:
    vocab: int = 0
    width: int = 0
    layers: List[Dict[str, Any]] = field(default_factory=list)
    embedding_scale: float = 1.0
    norm_eps: float = 1e-5
    logit_softcap: Optional[float] = None
    architecture: str = "Buzopel"
    model_type: str = "buzopel"
    eos_token_id: Any = None

    @classmethod
    def from_dict(cls, params: dict) -> "ModelConfig":
        for key in ("vocab", "width", "layers"):
            if key not in params:
                raise ValueError(f"config.json: missing '{key}'")
        cap = params.get("logit_softcap")
        return cls(vocab=int(params["vocab"]), width=int(params["width"]), layers=list(params["layers"]),
                   embedding_scale=float((params.get("embedding") or {}).get("scale", 1.0)),
                   norm_eps=float((params.get("norm") or {}).get("eps", 1e-5)),
                   logit_softcap=float(cap) if cap else None,
                   architecture=params.get("architecture", "Buzopel"), eos_token_id=params.get("eos_token_id"))

    def to_dict(self) -> dict:
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "layers": self.layers,
               "embedding": {"scale": self.embedding_scale}, "norm": {"eps": self.norm_eps}}
        if self.logit_softcap:
            out["logit_softcap"] = self.logit_softcap
        return out

    # names the generic parts of the package read
    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)
