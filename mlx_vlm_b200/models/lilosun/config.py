"""Configuration of a Lilosun checkpoint: `config.json` names every size and every constant that differs between
models of the design: vocabulary, width, the list of layers (each with its mixer's type and sizes and its
feed-forward, or none), the eps of the norms and the constant the logits are multiplied by."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List


@dataclass
class ModelConfig:
    vocab: int = 0
    width: int = 0
    layers: List[Dict[str, Any]] = field(default_factory=list)
    norm_eps: float = 1e-5
    logit_scale: float = 1.0
    architecture: str = "Lilosun"
    model_type: str = "lilosun"
    eos_token_id: Any = None

    @classmethod
    def from_dict(cls, params: dict) -> "ModelConfig":
        for key in ("vocab", "width", "layers"):
            if key not in params:
                raise ValueError(f"config.json: missing '{key}'")
        for i, L in enumerate(params["layers"]):
            if "type" not in L or "mixer" not in L:
                raise ValueError(f"config.json: layer {i} needs 'type' and 'mixer'")
        return cls(vocab=int(params["vocab"]), width=int(params["width"]), layers=list(params["layers"]),
                   norm_eps=float((params.get("norm") or {}).get("eps", 1e-5)),
                   logit_scale=float(params.get("logit_scale", 1.0)),
                   architecture=params.get("architecture", "Lilosun"), eos_token_id=params.get("eos_token_id"))

    def to_dict(self) -> dict:
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "layers": self.layers,
                "norm": {"eps": self.norm_eps}, "logit_scale": self.logit_scale}

    # names the generic parts of the package read
    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)
