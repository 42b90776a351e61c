"""Engine for decoder designs that are assembled layer by layer on the host (models/decoder_blocks.py over
csrc/layer_ops.cu).  It has the surface of `engine.Engine` that the generation loops and the batch scheduler use
— a dedicated stream, a device token log with `tokens_launched` / `fetch_tokens`, `set_next` / `decode` for one
request, `batch_begin` / `batch_decode` / `batch_fetch` for lock-step rows, `bind_pool`, `kv_copy_row`,
`snapshot` — so `generate_step`, `stream_generate` and `BatchGenerator` drive such a model unchanged.

ONE step function serves everything: `forward(tokens, slot, pos, want)` takes the tokens of a step concatenated
over its requests, each with the cache slot and the position it belongs to; prompts, portions of prompts, decoded
tokens and batches of unequal requests differ only in those arrays.  Greedy decoding keeps the token feedback on
the device (argmax -> next step's input) and the host reads tokens from the log.
"""
from __future__ import annotations

from typing import List, Optional

import numpy as np
import torch

from . import _native as N
from .models.decoder_blocks import StepCtx
from .models.layer_ops import EPI_NONE, EPI_SCALE, EPI_SOFTCAP, LayerOps


class LayerEngine:
    BATCH_LOG_STEPS, BATCH_LOG_ROWS = 4096, 16
    TOKEN_LOG = 8192

    def __init__(self, device, exact: bool = False):
        device = torch.device(device)
        if device.type != "cuda":
            raise N.B200Error("the layer engine needs a CUDA (sm_100a) device; no CPU fallback")
        self.device = device if device.index is not None else torch.device("cuda", torch.cuda.current_device())
        self.exact = bool(exact)
        self.stream = torch.cuda.Stream(device=self.device)
        self.ops = LayerOps(self.device, self.stream, exact=exact)
        self.lib = self.ops.lib
        sm = N.C.c_int(0)
        N.check(self.lib.b200_device_check(self.device.index, N.C.byref(sm)), "device_check", self.lib)
        self.core = None              # the bound model: embed / layers / final norm / head
        self.pool = None
        self.tokens_launched = 0
        with torch.cuda.stream(self.stream):
            self._log = torch.zeros(self.TOKEN_LOG, dtype=torch.int32, device=self.device)
            self._blog = torch.zeros((self.BATCH_LOG_STEPS, self.BATCH_LOG_ROWS), dtype=torch.int32, device=self.device)
            self._blp = torch.zeros((self.BATCH_LOG_STEPS, self.BATCH_LOG_ROWS), dtype=torch.float32, device=self.device)
            self._sampled = torch.zeros(128, dtype=torch.int32, device=self.device)
            self._lp = torch.zeros(128, dtype=torch.float32, device=self.device)
            self._lstep = torch.zeros(1, dtype=torch.int32, device=self.device)     # device step counters of the logs
            self._bstep_dev = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._tok = self._pos = self._slot = self._active = None     # device state of the decode loop
        self._states = {}
        self._graphs = {}             # captured decode steps: (mode, rows, pool buffer, capacity) -> (graph, logits)
        self._eager_steps = {}
        self.use_graphs = True
        self.graph_replays = 0
        self._logits: Optional[torch.Tensor] = None
        self._bstep = 0

    # ------------------------------------------------------------------ plumbing
    @property
    def s(self) -> int:
        return self.stream.cuda_stream

    @property
    def launch_count(self) -> int:
        return self.ops.launches

    @property
    def token_log_capacity(self) -> int:
        return self.TOKEN_LOG

    def empty(self, shape, dtype=torch.float32):
        return self.ops.empty(shape, dtype)

    def bind_model(self, core):
        self.core = core

    def bind_pool(self, pool):
        self.pool = pool

    def kv_copy_row(self, dst, dst_row: int, src, src_row: int, n_tokens: int):
        with torch.cuda.stream(self.stream):
            dst.copy_slot(int(dst_row), src, int(src_row), int(n_tokens))

    # ------------------------------------------------------------------ the step
    def forward(self, tokens: torch.Tensor, slot: torch.Tensor, pos: torch.Tensor, want: Optional[torch.Tensor] = None,
                embeds: Optional[torch.Tensor] = None, segments=None) -> torch.Tensor:
        """tokens / slot / pos: (T,) int32 device.  want: (n,) int32 device rows whose logits are wanted (None:
        every row).  Returns fp32 logits (n, vocab).  The cache rows of the tokens are written on the way."""
        with self.ops.on_stream():
            return self._forward(tokens, slot, pos, want, embeds, segments)

    def _forward(self, tokens, slot, pos, want, embeds, segments):
        c, ops = self.core, self.ops
        ctx = StepCtx(ops, slot, pos, self.pool, c.eps, segments)    # segments: the host's view of a prompt step
        if embeds is not None:
            with torch.cuda.stream(self.stream):
                x = embeds.to(torch.float32).reshape(-1, c.width).clone()
        else:
            x = ops.embed(tokens, c.embed, c.embed_scale)
        if hasattr(c, "run_layers"):      # a design with its own order of layer runs (a span that repeats)
            def embed_again():
                if embeds is not None:
                    with torch.cuda.stream(self.stream):
                        return embeds.to(torch.float32).reshape(-1, c.width).clone()
                return ops.embed(tokens, c.embed, c.embed_scale)
            x = c.run_layers(ctx, x, embed_again)
        else:
            for layer in c.layers:
                layer.forward(ctx, x)
        n = x.shape[0] if want is None else want.shape[0]
        xn = ops.empty((n, c.width))
        ops.norm_rows(x, c.final_norm, c.eps, xn, w_offset=getattr(c, "norm_offset", 1.0), rows=want,
                      center=getattr(c, "norm_center", False), groups=getattr(c, "norm_groups", 1))
        cap, mul = c.logit_softcap, float(getattr(c, "logit_scale", 1.0))
        if not cap and mul != 1.0:        # a design whose logits are the head's product times a constant
            return ops.linear(xn, c.head, epi=EPI_SCALE, epi_param=mul)
        return ops.linear(xn, c.head, epi=EPI_SOFTCAP if cap else EPI_NONE, epi_param=cap or 0.0)

    # ------------------------------------------------------------------ one request
    def _state(self, B: int):
        """device arrays of the decode loop, one fixed set per row count (captured steps point at them)"""
        if B not in self._states:
            with torch.cuda.stream(self.stream):
                self._states[B] = [torch.zeros(B, dtype=torch.int32, device=self.device) for _ in range(3)] + \
                                  [torch.ones(B, dtype=torch.int32, device=self.device)]
        self._tok, self._pos, self._slot, self._active = self._states[B]

    def _upload_state(self, tok, pos, slot, active=None):
        B = len(tok)
        self._state(B)
        host = np.stack([np.asarray(tok, dtype=np.int32), np.asarray(pos, dtype=np.int32),
                         np.asarray(slot, dtype=np.int32),
                         np.ones(B, dtype=np.int32) if active is None else np.asarray(active, dtype=np.int32)])
        dev = self.ops.to_device(host)
        with torch.cuda.stream(self.stream):
            self._tok.copy_(dev[0]); self._pos.copy_(dev[1]); self._slot.copy_(dev[2]); self._active.copy_(dev[3])

    def set_next(self, token: int, ctx: int, position: int, slot: int = 0):
        """the next decode step of a single request feeds `token` at `position` of cache slot `slot`"""
        self._upload_state([token], [position], [slot])

    def sample_prefill(self, logits_last: torch.Tensor, positions: List[int], slots: List[int]):
        """greedy first tokens after a prefill (one logits row per request): logged, and armed as the decode state"""
        B = logits_last.shape[0]
        self._logits = logits_last
        self.ops.argmax_rows(logits_last, self._sampled[:B], self._lp[:B])
        self._upload_state([0] * B, positions, slots)
        with torch.cuda.stream(self.stream):
            self._tok.copy_(self._sampled[:B])
            i = self.tokens_launched % self.TOKEN_LOG
            if i + B <= self.TOKEN_LOG:
                self._log[i:i + B].copy_(self._sampled[:B])
            else:
                for b in range(B):
                    self._log[(i + b) % self.TOKEN_LOG].copy_(self._sampled[b])
        self.tokens_launched += B
        with torch.cuda.stream(self.stream):
            self._lstep.fill_(self.tokens_launched)

    def _decode_step(self, batch: bool):
        """one greedy step of the armed rows: forward, pick, feed back.  Every argument is device state, so after
        two eager steps (first-use set-up) the step is captured as a CUDA graph per (rows, pool buffer) and replayed."""
        B = self._tok.shape[0]

        def body():
            logits = self.forward(self._tok, self._slot, self._pos)
            self.ops.argmax_rows(logits, self._sampled[:B], self._lp[:B])
            if batch:
                self.ops.advance_rows(self._sampled[:B], self._tok, self._pos, self._active, self._blog, self._bstep_dev,
                                      self._lp[:B], self._blp)
            else:
                self.ops.advance_rows(self._sampled[:B], self._tok, self._pos, None, self._log.view(-1, 1), self._lstep)
            return logits

        state = getattr(self.pool, "state", None)      # a pool with recurrent state: its buffer is an argument too
        key = (batch, B, self.pool.buf.data_ptr(), self.pool.capacity, 0 if state is None else state.data_ptr())
        if not self.use_graphs:
            self._logits = body()
        elif key in self._graphs:
            g, self._logits = self._graphs[key]
            with torch.cuda.stream(self.stream):
                g.replay()
            self.graph_replays += 1
        elif self._eager_steps.get(key, 0) < 2:
            self._eager_steps[key] = self._eager_steps.get(key, 0) + 1
            self._logits = body()
        else:
            if len(self._graphs) >= 8:       # pools that moved leave stale graphs behind
                self._graphs.clear()
            g = torch.cuda.CUDAGraph()
            self.stream.synchronize()
            with torch.cuda.graph(g, stream=self.stream):
                logits = body()
            self._graphs[key] = (g, logits)
            self._logits = logits
            with torch.cuda.stream(self.stream):
                g.replay()
            self.graph_replays += 1

    def decode(self, n_steps: int):
        """n greedy steps of the armed single request; the token feedback stays on the device"""
        assert self._tok is not None and self._tok.shape[0] == 1, "decode: arm one request first (set_next / prefill)"
        for _ in range(int(n_steps)):
            self._decode_step(batch=False)
            self.tokens_launched += 1

    def fetch_tokens(self, start: int, n: int, host: torch.Tensor):
        with torch.cuda.stream(self.stream):
            for k in range(n):
                i = (start + k) % self.TOKEN_LOG
                host[k:k + 1].copy_(self._log[i:i + 1], non_blocking=True)

    def snapshot(self, which: str = "logprobs") -> torch.Tensor:
        """stream-ordered copy of the last step's logits / log-probabilities of row 0 (fp32, (vocab,))"""
        with torch.cuda.stream(self.stream):
            z = self._logits[0].clone()
            return z if which == "logits" else z - torch.logsumexp(z, dim=-1)

    # ------------------------------------------------------------------ lock-step rows
    def batch_begin(self, tok, ctx, pos, active):
        B = len(tok)
        assert B <= self.BATCH_LOG_ROWS
        self._upload_state(tok, pos, list(range(B)), active)
        with torch.cuda.stream(self.stream):
            self._bstep_dev.zero_()
        self._batch_B, self._bstep = B, 0

    def batch_decode(self, n_steps: int, want_logprobs: bool = False):
        assert self._tok.shape[0] == self._batch_B, "batch_decode: arm the rows first (batch_begin)"
        for _ in range(int(n_steps)):
            assert self._bstep < self.BATCH_LOG_STEPS, "batch_decode: re-arm the rows (batch_begin)"
            self._decode_step(batch=True)
            self._bstep += 1

    def batch_fetch(self, first_step: int, n_steps: int, tok_host: torch.Tensor, lp_host: Optional[torch.Tensor] = None):
        B = self._batch_B
        with torch.cuda.stream(self.stream):
            tok_host.view(n_steps, B).copy_(self._blog[first_step:first_step + n_steps, :B], non_blocking=True)
            if lp_host is not None:
                lp_host.view(n_steps, B).copy_(self._blp[first_step:first_step + n_steps, :B], non_blocking=True)

    def batch_logits_view(self, which: str = "logits") -> torch.Tensor:
        if which == "logits":
            return self._logits
        with torch.cuda.stream(self.stream):
            return self._logits - torch.logsumexp(self._logits, dim=-1, keepdim=True)

    def batch_token_log_view(self) -> torch.Tensor:
        return self._blog

    def device_error(self) -> int:
        return 0
