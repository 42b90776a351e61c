"""Configuration of a Vadelix checkpoint: `config.json` names every size and every constant that differs between
models of the design: vocabulary, width, the list of layers (each with its mixer's type and sizes and its
feed-forward, or none), the eps and the number of groups of the norms, the multiplier of the residual branches and the
taps of the convolution in front of every mixer.  The rank of a 'wkv' mixer's decay projection is the first size of
its `w1` tensor in the checkpoint (`decay_rank` in a mixer's entry overrides it; models made without a checkpoint use
that or 64)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List


@dataclass
class ModelConfig:
    vocab: int = 0
    width: int = 0
    layers: List[Dict[str, Any]] = field(default_factory=list)
    norm_eps: float = 1e-6
    norm_groups: int = 1
    residual_mult: float = 1.0
    canon_taps: int = 0
    architecture: str = "Vadelix"
    model_type: str = "vadelix"
    eos_token_id: Any = None

    @classmethod
    def from_dict(cls, params: dict) -> "ModelConfig":
        for key in ("vocab", "width", "layers"):
            if key not in params:
                raise ValueError(f"config.json: missing '{key}'")
        for i, L in enumerate(params["layers"]):
            if "type" not in L or "mixer" not in L:
                raise ValueError(f"config.json: layer {i} needs 'type' and 'mixer'")
        norm = params.get("norm") or {}
        return cls(vocab=int(params["vocab"]), width=int(params["width"]), layers=list(params["layers"]),
                   norm_eps=float(norm.get("eps", 1e-6)), norm_groups=int(norm.get("groups", 1)),
                   residual_mult=float(params.get("residual_mult", 1.0)),
                   canon_taps=int((params.get("canon") or {}).get("taps", 0)),
                   architecture=params.get("architecture", "Vadelix"), eos_token_id=params.get("eos_token_id"))

    def to_dict(self) -> dict:
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "layers": self.layers,
               "norm": {"eps": self.norm_eps, "groups": self.norm_groups}, "residual_mult": self.residual_mult}
        if self.canon_taps:
            out["canon"] = {"taps": self.canon_taps}
        return out

    # names the generic parts of the package read
    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)
