"""Vadelix `Model`: the per-model surface of the package (`language_model`, `get_input_embeddings`, `sanitize`,
`load_weights`, `engine`, `config`) for a text-only decoder of pre-norm layers with an RMS norm in groups, one
multiplier on both residual branches and a causal convolution on what every mixer reads
(decoder_blocks.ConvPreNormLayer).  Mixers: grouped attention with norms over the whole query / key projection,
YaRN-scaled rotary, unit-length values and a sink logit per head; grouped attention without rotation, with a query
temperature, a distance bias per head, a sliding window and one in the softmax's denominator; a token-shift mixer with
a decay per key channel and a matrix state per head.  The attention layers that say so mix their values with those of
the first of them.  Feed-forwards: a gelu-gated unit and a mixture of ungated gelu experts whose choice is limited to
groups, with a shared expert.  All weights are packed into ONE device arena; the arithmetic is csrc/layer_ops.cu +
csrc/mixer_ops.cu driven by `LayerEngine`."""
from __future__ import annotations

from typing import Dict, Optional

import numpy as np
import torch

from ...layer_engine import LayerEngine
from ..base import InputEmbeddingsFeatures
from ..decoder_blocks import ConvPreNormLayer, GroupedAttention, TokenShiftState
from ..qwen2_vl.qwen2_vl import WeightArena
from .config import ModelConfig
from .language import LanguageModel

DEFAULT_DECAY_RANK = 64


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
        self.eps, self.embed_scale, self.logit_softcap = config.norm_eps, 1.0, None
        self.norm_groups = config.norm_groups
        self.layers = [ConvPreNormLayer(i, c, config.width, groups=config.norm_groups, mult=config.residual_mult,
                                        taps=config.canon_taps) for i, c in enumerate(config.layers)]
        kv, first = 0, None
        for L in self.layers:     # every caching layer gets its rows of the pool; the value mixing its source
            m = L.mixer
            if L.kv_dim:
                m.cache_index, kv = kv, kv + 1
            if isinstance(m, GroupedAttention) and m.v_mix:
                if first is None:
                    first, m.v_role = m, "first"
                elif m.n_v != first.n_v:
                    raise ValueError(f"layer {L.index} mixes values of {m.n_v} numbers with layer {first.index}'s {first.n_v}")
                else:
                    m.v_role = "blend"
            if isinstance(m, TokenShiftState) and not m.rank:
                m.set_rank(DEFAULT_DECAY_RANK)
        self.n_cache_layers = kv
        self._assign_state()
        self.row_dim = max([L.kv_dim for L in self.layers] + [0])
        self.embed = self.final_norm = self.head = None
        self.arena: Optional[WeightArena] = None
        self.language_model = LanguageModel(config, self, self._engine)

    def _assign_state(self):
        """every layer's span of a slot's state: [rows of the convolution | what its mixer keeps]"""
        st = 0
        for L in self.layers:
            L.state_off, L.mixer.state_off = st, st + L.conv_floats
            st += L.state_floats
        self.state_floats = st

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
        """the layers of one step over the residual rows x (T, width) fp32, updated in place.  The last residual update
        of a layer also norms the rows for the layer that follows (one launch for both)."""
        n = None
        for i, L in enumerate(self.layers):
            nxt = self.layers[i + 1].w["norm1"] if i + 1 < len(self.layers) else None
            n = L.forward(ctx, x, normed=n, next_norm=nxt)
        return x

    # ------------------------------------------------------------------ weights
    def _globals(self):
        return [("embed", (self.vocab, self.width)), ("final.norm", (self.width,)), ("head", (self.vocab, self.width))]

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

    def load_weights(self, weights: Dict[str, torch.Tensor], strict: bool = True):
        for i, L in enumerate(self.layers):      # a size that only the checkpoint gives: the rank of the decay projection
            t = weights.get(f"l{i}.mix.w1")
            if isinstance(L.mixer, TokenShiftState) and t is not None and "decay_rank" not in self.config.layers[i]["mixer"]:
                L.mixer.set_rank(t.shape[0])
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
        no checkpoint): matrices N(0, 1/fan-in), norm weights around one, token-shift mixes around one half, decay
        biases negative, the other vectors small"""
        eng = self._engine()
        g = torch.Generator(device=eng.device).manual_seed(seed)
        with torch.cuda.stream(eng.stream):
            self.arena = WeightArena(self.manifest(), eng.device)
            view = self.arena.view
            for name, shape in self.manifest():
                v = view(name)
                if len(shape) == 1:
                    last = name.rsplit(".", 1)[-1]
                    mean = {"w0": -1.0, "vmix": 0.3}.get(last, 1.0 if "norm" in last else 0.0)
                    v.copy_(mean + 0.05 * torch.randn(shape, generator=g, device=eng.device))
                elif name.endswith((".mu", ".u", ".canon1")):
                    v.copy_((0.5 if name.endswith(".mu") else 0.0) + 0.1 * torch.randn(shape, generator=g, device=eng.device))
                else:
                    s = 1.0 if name == "embed" else 1.0 / float(shape[-1]) ** 0.5
                    for part in (v.unbind(0) if v.numel() > (1 << 28) else (v,)):     # bounded fp32 staging
                        part.copy_(torch.randn(part.shape, generator=g, device=eng.device) * s)
            self._bind(view)
        eng.stream.synchronize()
        return self

    # ------------------------------------------------------------------ inputs
    def get_input_embeddings(self, input_ids=None, pixel_values=None, **kwargs) -> InputEmbeddingsFeatures:
        """text only: the embedding rows (1, T, width) fp32"""
        if pixel_values is not None:
            raise ValueError("Vadelix is a text-only decoder")
        eng = self._engine()
        ids = np.asarray(input_ids.cpu() if isinstance(input_ids, torch.Tensor) else input_ids).reshape(-1)
        x = eng.ops.embed(eng.ops.to_device(ids), self.embed, self.embed_scale)
        return InputEmbeddingsFeatures(inputs_embeds=x.unsqueeze(0))
