"""Vadelix language model: the call surface of the layer-assembled decoders (`step`, `__call__`, `make_cache`,
`make_cache_row`, `make_pool`, `fused_greedy_decode_n`, `prefill_rows`: models/buzopel/language.py) over a
`StatePool`: a request's slot holds the key/value rows of every attention layer and, per layer, one span of fp32
state: the last inputs of the convolution in front of the mixer and, for a 'wkv' mixer, the previous token's input and
the matrix state of every head."""
from __future__ import annotations

from typing import List

import torch

from ..buzopel.language import LanguageModel as _LayeredLanguageModel
from ..cache import RunCache, StatePool


class LanguageModel(_LayeredLanguageModel):
    def __init__(self, args, core, engine_getter):
        super().__init__(args, core, engine_getter)
        self.model_type = "vadelix"

    def make_pool(self, rows: int = 1, capacity: int = 0) -> StatePool:
        eng = self._engine()
        with torch.cuda.stream(eng.stream):
            return StatePool(self.core.n_cache_layers, self.core.row_dim, self.core.state_floats, eng.device, batch=rows,
                             capacity=capacity, dtype=eng.ops.cache_dtype)

    def make_cache_row(self, pool: StatePool, row: int) -> List[RunCache]:
        return [RunCache(pool, row, kv_layer=L.mixer.cache_index if L.kv_dim else None, kv_dim=L.kv_dim,
                         state_off=L.state_off, state_len=L.state_floats) for L in self.core.layers]

    def make_cache(self) -> List[RunCache]:
        return self.make_cache_row(self.make_pool(1), 0)
