"""Thin Python face of the layer-level ops (csrc/layer_ops.cu) — the sibling of tower_ops.py for decoder
layers that are assembled on the host: fp32 residual stream, norms on the sublayer's output, latent
attention over (slot, position)-addressed cache rows, rotate-half rotary, expert mixtures, row GEMMs.

Every call enqueues one kernel on the engine's stream.  torch is the memory container only.
`exact=True` is the true-fp32 mode (fp32 cache rows, no rounding of matrix operands); otherwise cache rows
are bf16 and the operands of the matrix products are rounded to bf16 on load (fp32 accumulation).
"""
from __future__ import annotations

from typing import Optional

import numpy as np
import torch

from .. import _native as N

EPI_NONE, EPI_RELU2, EPI_SOFTCAP, EPI_ADD, EPI_SCALE, EPI_GELU = 0, 1, 2, 3, 4, 5
ACT_NONE, ACT_RELU2, ACT_GELU, ACT_TANH = 0, 1, 2, 3     # activation codes of `to_bf16` (gelu: the exact, erf form)
GELU_TANH_ALPHA, GELU_TANH_CUBIC = 1.5957691216057308, 0.044715     # z sigmoid(alpha (z + cubic z^3)) = the tanh form of gelu
SM_COUNT = 148
TC_MIN_ROWS = 128     # from this many rows on, a product of the bf16 serving mode runs on the tcgen05 GEMM
WT_F32 = 3            # gemm_wt output mode: fp32 rows
SKINNY_ROWS = 16      # up to this many rows a product runs on the warp-per-weight-row kernel


class LayerOps:
    def __init__(self, device, stream: torch.cuda.Stream, exact: bool = False):
        if torch.device(device).type != "cuda":
            raise N.B200Error("the layer ops need a CUDA (sm_100a) device; there is no CPU fallback")
        self.lib = N.lm_lib()
        self.device, self.stream, self.exact = torch.device(device), stream, bool(exact)
        self.launches = 0
        self._inv_freq = {}
        self._unit_seqs = {}
        self._on_stream = False
        self.tc_enabled = True

    @property
    def s(self) -> int:
        return self.stream.cuda_stream

    @property
    def cache_dtype(self):
        return torch.float32 if self.exact else torch.bfloat16

    def _ok(self, rc, what):
        self.launches += 1
        N.check(rc, what, self.lib)

    def empty(self, shape, dtype=torch.float32) -> torch.Tensor:
        if self._on_stream:       # the caller already made the engine's stream current (one context per step,
            return torch.empty(shape, dtype=dtype, device=self.device)   # not one per buffer: ~10 us each)
        with torch.cuda.stream(self.stream):
            return torch.empty(shape, dtype=dtype, device=self.device)

    def on_stream(self):
        """context: the engine's stream is current for everything inside (buffers of a step come from its pool)"""
        ops = self

        class _Ctx:
            def __enter__(self):
                self.inner = torch.cuda.stream(ops.stream)
                self.inner.__enter__()
                self.prev, ops._on_stream = ops._on_stream, True

            def __exit__(self, *exc):
                ops._on_stream = self.prev
                return self.inner.__exit__(*exc)

        return _Ctx()

    def to_device(self, arr, dtype=np.int32) -> torch.Tensor:
        t = torch.from_numpy(np.ascontiguousarray(arr, dtype=dtype)).pin_memory()
        with torch.cuda.stream(self.stream):
            return t.to(self.device, non_blocking=True)

    # ------------------------------------------------------------------------------------------
    def embed(self, tokens: torch.Tensor, table: torch.Tensor, scale: float) -> torch.Tensor:
        T, (V, W) = tokens.shape[0], table.shape
        x = self.empty((T, W))
        self._ok(self.lib.b200_lm_embed(tokens.data_ptr(), table.data_ptr(), float(scale), x.data_ptr(), T, W, V,
                                        self.s), "lm_embed")
        return x

    def inv_freq(self, base: float, dims: int, scaling: Optional[tuple] = None) -> torch.Tensor:
        """f_i = base^(-2i/dims), i < dims/2, computed in double precision on the host (once per rotation).
        scaling = (factor, original, fast, slow), the YaRN rule (Peng et al., "YaRN: Efficient Context Window
        Extension of Large Language Models"): with d(t) = dims ln(original / (2 pi t)) / (2 ln base) the index at
        which a frequency makes t turns over `original` positions, lo = max(floor d(fast), 0),
        hi = min(ceil d(slow), dims - 1) and r_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1), the frequency is
        f_i (1 - r_i) + (f_i / factor) r_i."""
        key = (float(base), int(dims), scaling)
        if key not in self._inv_freq:
            half = dims // 2
            f = np.power(np.float64(base), -2.0 * np.arange(half, dtype=np.float64) / dims)
            if scaling is not None:
                factor, original, fast, slow = (float(v) for v in scaling)

                def index(turns):
                    return dims * np.log(original / (2.0 * np.pi * turns)) / (2.0 * np.log(base))

                lo, hi = max(np.floor(index(fast)), 0.0), min(np.ceil(index(slow)), dims - 1.0)
                ramp = np.clip((np.arange(half, dtype=np.float64) - lo) / max(hi - lo, 0.001), 0.0, 1.0)
                f = f / factor * ramp + f * (1.0 - ramp)
            self._inv_freq[key] = self.to_device(f, np.float64)
        return self._inv_freq[key]

    @staticmethod
    def rope_amplitude(scaling: Optional[tuple]) -> float:
        """what a frequency scaling multiplies cos and sin by: 0.1 ln(factor) + 1"""
        return 1.0 if scaling is None else 0.1 * float(np.log(float(scaling[0]))) + 1.0

    def rope_table(self, pos: torch.Tensor, base: float, dims: int, scaling: Optional[tuple] = None) -> torch.Tensor:
        T, half = pos.shape[0], dims // 2
        if half == 0:             # nothing is rotated: the kernels never read the table
            return self.empty((1, 1, 2))
        cs = self.empty((T, half, 2))
        self._ok(self.lib.b200_lm_rope_table(pos.data_ptr(), self.inv_freq(base, dims, scaling).data_ptr(), cs.data_ptr(),
                                             T, half, self.rope_amplitude(scaling), self.s), "lm_rope_table")
        return cs

    def norm_rows(self, y: torch.Tensor, w: torch.Tensor, eps: float, x: torch.Tensor, *, w_offset: float = 0.0,
                  add: bool = False, combine: Optional[torch.Tensor] = None, top: int = 0,
                  rows: Optional[torch.Tensor] = None, center: bool = False, groups: int = 1):
        """x (T, N) = or += rmsnorm(y rows) * (w_offset + w); `combine` (T, top): y holds `top` rows per token;
        center: the mean of the row is taken off first (a layer norm without bias); groups: the row is that many equal
        consecutive parts, each divided by its own root mean square"""
        T, n = x.shape
        self._ok(self.lib.b200_lm_norm_rows(y.data_ptr(), y.stride(0), N.ptr(combine), int(top), w.data_ptr(),
                                            float(w_offset), float(eps), x.data_ptr(), x.stride(0), int(add),
                                            N.ptr(rows), int(center), int(groups), T, n, self.s), "lm_norm_rows")

    def residual_rows(self, y: torch.Tensor, x: torch.Tensor, ls: Optional[torch.Tensor] = None, *,
                      combine: Optional[torch.Tensor] = None, top: int = 0, shared: Optional[torch.Tensor] = None,
                      shared_gate: Optional[torch.Tensor] = None, mult: float = 1.0):
        """x (T, N) += ls * mult * (y row, or the `combine`-weighted sum of `top` rows of y per token, + sigmoid(shared_gate)
        * shared row; without a gate the shared row counts fully): the residual update of a branch with a scale vector
        `ls` and / or a scale number `mult`"""
        T, n = x.shape
        self._ok(self.lib.b200_lm_residual_rows(y.data_ptr(), y.stride(0), N.ptr(combine), int(top), N.ptr(shared),
                                                shared.stride(0) if shared is not None else 0, N.ptr(shared_gate),
                                                shared_gate.stride(0) if shared_gate is not None else 0, N.ptr(ls),
                                                float(mult), x.data_ptr(), x.stride(0), T, n, self.s), "lm_residual_rows")

    def residual_norm_rows(self, y: torch.Tensor, x: torch.Tensor, ls: Optional[torch.Tensor], w: torch.Tensor, eps: float,
                           out: torch.Tensor, *, center: bool = False, w_offset: float = 0.0,
                           combine: Optional[torch.Tensor] = None, top: int = 0, shared: Optional[torch.Tensor] = None,
                           shared_gate: Optional[torch.Tensor] = None, mult: float = 1.0, groups: int = 1):
        """the update of `residual_rows` on x and, in the same launch, out = norm(updated x) * (w_offset + w): the
        branch's end and the next sublayer's norm read and write the row once"""
        T, n = x.shape
        self._ok(self.lib.b200_lm_residual_norm_rows(
            y.data_ptr(), y.stride(0), N.ptr(combine), int(top), N.ptr(shared), shared.stride(0) if shared is not None else 0,
            N.ptr(shared_gate), shared_gate.stride(0) if shared_gate is not None else 0, N.ptr(ls), x.data_ptr(), x.stride(0),
            w.data_ptr(), float(w_offset), float(eps), int(center), out.data_ptr(), out.stride(0), int(groups), float(mult),
            T, n, self.s),
            "lm_residual_norm_rows")

    def latent_post(self, D, wq, wkv, eps, cq, cache_layer, slot, pos, cs, q_rank, kv_rank, rot_dim, rot_dims,
                    pairs: bool = False):
        """cache_layer: (slots, capacity, kv_rank + rot_dim) view of the pool, or None for a layer that borrows;
        q_rank 0: no query latent (wq, cq None; D's rows start with the kv latent); pairs: rotation pairs (2i, 2i+1)"""
        own = cache_layer is not None
        self._ok(self.lib.b200_lm_latent_post(
            D.data_ptr(), D.stride(0), N.ptr(wq), N.ptr(wkv), float(eps), N.ptr(cq), cq.stride(0) if cq is not None else 0,
            N.ptr(cache_layer), int(own and cache_layer.dtype == torch.bfloat16),
            cache_layer.stride(0) if own else 0, cache_layer.stride(1) if own else 0, N.ptr(slot), N.ptr(pos),
            N.ptr(cs), q_rank, kv_rank, rot_dim, rot_dims, int(own), int(pairs), D.shape[0], self.s), "lm_latent_post")

    def rope_q(self, q, qa, cs, H, dim, rot_dim, rot_dims, kv_rank, pairs: bool = False):
        T = q.shape[0]
        self._ok(self.lib.b200_lm_rope_q(q.data_ptr(), q.stride(0), dim + rot_dim, dim, qa.data_ptr(), qa.stride(0),
                                         kv_rank + rot_dim, kv_rank, cs.data_ptr(), H, rot_dim, rot_dims, int(pairs), T,
                                         self.s), "lm_rope_q")

    def latent_attention(self, qa, cache_layer, slot, pos, out, H, kv_rank, scale, n_split=None, window: int = 0):
        """n_split: blocks per (token, head group) that share the keys (None: enough to fill the GPU when the
        step has few tokens — a decode step —, 1 for prompts)"""
        T, Dl = qa.shape[0], cache_layer.shape[-1]
        if n_split is None:
            groups = T * ((H + 7) // 8)
            n_split = max(1, min(64, (2 * SM_COUNT) // groups))
            if window > 0:       # a window holds at most this many key tiles (of 32): more splits would only be merged
                n_split = min(n_split, (window + 31) // 32)
        part = self.empty((T, H, n_split, kv_rank + 2)) if n_split > 1 else None
        self._ok(self.lib.b200_lm_latent_attention(
            qa.data_ptr(), qa.stride(0), cache_layer.data_ptr(), int(cache_layer.dtype == torch.bfloat16),
            cache_layer.stride(0), cache_layer.stride(1), slot.data_ptr(), pos.data_ptr(), out.data_ptr(),
            out.stride(0), H, Dl, kv_rank, float(scale), 0, int(window), N.ptr(part), n_split, T, self.s),
            "lm_latent_attention")

    def router_topk(self, z, top):
        T, E = z.shape
        idx, wgt = self.empty((T, top), torch.int32), self.empty((T, top))
        self._ok(self.lib.b200_lm_router_topk(z.data_ptr(), z.stride(0), E, top, idx.data_ptr(), wgt.data_ptr(), T,
                                              self.s), "lm_router_topk")
        return idx, wgt

    def router_group_topk(self, z, top, correction=None, n_groups: int = 1, keep: int = 1, E: Optional[int] = None,
                          softmax: bool = False, group_max: bool = False):
        """sigmoid scores (softmax: softmax over all experts); choice on score + correction among the experts of the
        `keep` best of `n_groups` groups (a group's score: the sum of its two largest, or, group_max, its largest);
        weights = the chosen scores over their sum.  z may hold more columns than experts (E of them are read)"""
        T = z.shape[0]
        E = z.shape[1] if E is None else E
        idx, wgt = self.empty((T, top), torch.int32), self.empty((T, top))
        self._ok(self.lib.b200_lm_router_group_topk(z.data_ptr(), z.stride(0), N.ptr(correction), E, top, int(n_groups),
                                                    int(keep), int(softmax), int(group_max), idx.data_ptr(),
                                                    wgt.data_ptr(), T, self.s),
                 "lm_router_group_topk")
        return idx, wgt

    def moe_group(self, idx, E):
        T, top = idx.shape
        lists, count = self.empty((E, T), torch.int32), self.empty((E,), torch.int32)
        self._ok(self.lib.b200_lm_moe_group(idx.data_ptr(), T * top, E, lists.data_ptr(), T, count.data_ptr(), self.s),
                 "lm_moe_group")
        return lists, count

    def gemm(self, X, W, Y, *, M, N_, K, ldx=None, xb=0, ldw=None, wb=0, ldy=None, yb=0, batch=1, bias=None,
             lists=None, count=None, x_div=1, epi=EPI_NONE, epi_param=0.0, compact=0, exact_x: bool = False):
        """Y[b][r][:] = epi(X[b][r'] . W[b]^T + bias); strides in elements (default: the tensors' own rows).
        compact: an upper bound of the batches that have rows (a decode step: rows x top experts of many);
        exact_x: the rows of X are not rounded to bf16 in the serving mode either (a router's input)"""
        self._ok(self.lib.b200_lm_gemm_rows(
            X.data_ptr(), X.stride(0) if ldx is None else ldx, xb, W.data_ptr(), K if ldw is None else ldw, wb,
            N.ptr(bias), Y.data_ptr(), Y.stride(0) if ldy is None else ldy, yb, N.ptr(lists),
            lists.stride(0) if lists is not None else 0, N.ptr(count), x_div, M, N_, K, batch, epi, float(epi_param),
            int(not self.exact and not exact_x), int(M <= SKINNY_ROWS), int(compact), self.s), "lm_gemm_rows")

    # ---- the tensor-core path of prompt steps (bf16 serving mode) ----------------------------------------
    def tc_ok(self, rows: int, *ks: int) -> bool:
        """a product with `rows` rows and inner sizes `ks` may run on the tcgen05 GEMM: serving mode, enough rows
        to fill a tile, 16-byte rows for the TMA"""
        return self.tc_enabled and (not self.exact) and rows >= TC_MIN_ROWS and all(k % 8 == 0 for k in ks)

    def tc_refused(self, err: Exception):
        """the tensor-core GEMM rejected a product's arguments (its checks run before any launch): say so once and
        keep to the general row kernels — still this library's CUDA path — from here on"""
        if self.tc_enabled:
            import sys
            print(f"layer ops: tensor-core path switched off, the row kernels take over ({err})", file=sys.stderr)
        self.tc_enabled = False

    def to_bf16(self, X: torch.Tensor, K: int, rows: Optional[int] = None, row_map: Optional[torch.Tensor] = None,
                div: int = 1, relu2: bool = False, act: int = ACT_NONE) -> torch.Tensor:
        """fp32 rows -> bf16 rows zero-padded to a multiple of 64 columns (the GEMM's k-block); act: an activation
        before the rounding (ACT_RELU2, also `relu2`; ACT_GELU; ACT_TANH)"""
        rows = X.shape[0] if rows is None else rows
        Kp = (K + 63) // 64 * 64
        out = self.empty((rows, Kp), torch.bfloat16)
        self._ok(self.lib.b200_lm_rows_to_bf16(X.data_ptr(), X.stride(0), N.ptr(row_map), div, out.data_ptr(), Kp, rows,
                                               K, Kp, ACT_RELU2 if relu2 else int(act), self.s), "lm_rows_to_bf16")
        return out

    def tc_gemm(self, Xb: torch.Tensor, W: torch.Tensor, Y: torch.Tensor, *, N_: int, K: int, ldw: Optional[int] = None,
                ldy: Optional[int] = None, bias=None, rows: Optional[int] = None, res: Optional[torch.Tensor] = None,
                parts: int = 1):
        """Y[rows, N_] (fp32) = Xb[rows, ceil64(K)] (bf16) . W[N_, K]^T (bf16, row pitch ldw) (+ res, which may be Y
        itself: a stream that accumulates in place) on tcgen05.  parts = 2: Xb holds [hi | lo] halves of fp32 rows
        (`to_split`), both multiplied by W and summed in the accumulator"""
        rows = Xb.shape[0] if rows is None else rows
        self._ok(self.lib.b200_gemm_wt_f32(Xb.data_ptr(), Xb.stride(0), W.data_ptr(), K if ldw is None else ldw,
                                           N.ptr(bias), N.ptr(res), res.stride(0) if res is not None else 0,
                                           Y.data_ptr(), Y.stride(0) if ldy is None else ldy, 0, 0, 0,
                                           rows, N_, K, int(parts), 0, WT_F32, self.s), "gemm_wt_f32")

    def to_split(self, X: torch.Tensor, K: int) -> torch.Tensor:
        """fp32 rows -> (T, 2 ceil64(K)) bf16 = [hi | lo] with hi = bf16(x), lo = bf16(x - hi): sixteen more mantissa
        bits of x reach the tensor cores than with one rounded part (K a multiple of 4)"""
        T, Kp = X.shape[0], (K + 63) // 64 * 64
        with torch.cuda.stream(self.stream):
            out = torch.zeros((T, 2 * Kp), dtype=torch.bfloat16, device=self.device)
        self._ok(self.lib.b200_f32_split(X.data_ptr(), X.stride(0), out.data_ptr(), 2 * Kp, Kp, T, K, self.s), "f32_split")
        return out

    def moe_order(self, lists: torch.Tensor, count: torch.Tensor) -> torch.Tensor:
        E, T = lists.shape
        order = self.empty((lists.numel(),), torch.int32)      # T * top entries at most (each entry is in one list)
        self._ok(self.lib.b200_lm_moe_order(lists.data_ptr(), lists.stride(0), count.data_ptr(), E, order.data_ptr(),
                                            self.s), "lm_moe_order")
        return order

    def moe_tiles(self, lists: torch.Tensor, count: torch.Tensor, n_entries: int, tile: int = 128):
        """-> (order (n_rows,), tile_group (n_rows / tile,)): the entries sorted by expert in segments padded to whole
        tiles; n_rows bounds any distribution of the entries over the experts"""
        E = lists.shape[0]
        n_rows = (n_entries + E * (tile - 1) + tile - 1) // tile * tile
        order, group = self.empty((n_rows,), torch.int32), self.empty((n_rows // tile,), torch.int32)
        self._ok(self.lib.b200_lm_moe_tiles(lists.data_ptr(), lists.stride(0), count.data_ptr(), E, tile,
                                            order.data_ptr(), n_rows, group.data_ptr(), self.s), "lm_moe_tiles")
        return order, group

    def tc_gemm_grouped(self, Xb: torch.Tensor, W: torch.Tensor, Y: torch.Tensor, tile_group: torch.Tensor, *, N_: int,
                        K: int, n_groups: int):
        """Y[tile y] = Xb[tile y] . W[tile_group[y]]^T for every token tile of 128 rows, ONE tcgen05 launch"""
        self._ok(self.lib.b200_gemm_wt_f32_grouped(Xb.data_ptr(), Xb.stride(0), W.data_ptr(), K, Y.data_ptr(),
                                                   Y.stride(0), tile_group.data_ptr(), tile_group.shape[0], n_groups,
                                                   N_, K, self.s), "gemm_wt_f32_grouped")

    def tc_gemm_heads(self, Xb: torch.Tensor, W: torch.Tensor, Y: torch.Tensor, *, H: int, N_: int, K: int,
                      x_cols: int, x_group_cols: int, c_group_cols: int):
        """Y[:, g * c_group_cols : + N_] = Xb[:, g * x_group_cols : + K] . W[g]^T for every head g, ONE tcgen05 launch"""
        self._ok(self.lib.b200_gemm_wt_f32_heads(Xb.data_ptr(), Xb.stride(0), x_cols, x_group_cols, W.data_ptr(), K,
                                                 Y.data_ptr(), Y.stride(0), c_group_cols, Xb.shape[0], H, N_, K, self.s),
                 "gemm_wt_f32_heads")

    def rows_scatter(self, X: torch.Tensor, dst_map: torch.Tensor, out: torch.Tensor, rows: int):
        self._ok(self.lib.b200_lm_rows_scatter(X.data_ptr(), X.stride(0), dst_map.data_ptr(), out.data_ptr(),
                                               out.stride(0), rows, X.shape[1], self.s), "lm_rows_scatter")

    def masked_softmax_bf16(self, S: torch.Tensor, pos: torch.Tensor, H: int, scale: float, P: torch.Tensor):
        self._ok(self.lib.b200_lm_masked_softmax_bf16(S.data_ptr(), S.stride(0), pos.data_ptr(), H, float(scale),
                                                      P.data_ptr(), P.stride(0), S.shape[0], P.shape[1], self.s),
                 "lm_masked_softmax_bf16")

    def cache_transpose(self, rows: torch.Tensor, S: int, Sp: int, kv_rank: int) -> torch.Tensor:
        out = self.empty((kv_rank, Sp), torch.bfloat16)
        self._ok(self.lib.b200_lm_cache_transpose(rows.data_ptr(), rows.stride(0), S, Sp, kv_rank, out.data_ptr(), self.s),
                 "lm_cache_transpose")
        return out

    def linear(self, X: torch.Tensor, W: torch.Tensor, bias=None, epi=EPI_NONE, epi_param=0.0,
               out: Optional[torch.Tensor] = None, add: bool = False, exact_x: bool = False) -> torch.Tensor:
        """Y = epi(X . W^T + bias).  X and W may be column ranges of wider rows (their row pitch is taken from the
        tensors).  out: the rows to write (else fresh ones); add: the product is added to what `out` holds;
        exact_x: the rows of X are not rounded to one bf16 part in the serving mode (small products whose result
        decides something: a router): fp32 rows on the row kernels, or, for a long step, [hi | lo] halves on the
        tensor cores."""
        (T, K), n = X.shape, W.shape[0]
        Y = self.empty((T, n)) if out is None else out
        ldw = W.stride(0) if n > 1 else K
        if add:
            assert out is not None and epi == EPI_NONE, "linear: adding needs the rows to add to and no other epilogue"
        if epi == EPI_NONE and self.tc_ok(T, K, ldw) and W.data_ptr() % 16 == 0 and \
                (not exact_x or (X.stride(0) % 4 == 0 and X.data_ptr() % 16 == 0)):
            try:
                if exact_x:
                    self.tc_gemm(self.to_split(X, K), W, Y, N_=n, K=K, ldw=ldw, bias=bias, res=Y if add else None, parts=2)
                else:
                    self.tc_gemm(self.to_bf16(X, K), W, Y, N_=n, K=K, ldw=ldw, bias=bias, res=Y if add else None)
                return Y
            except N.B200Error as e:
                self.tc_refused(e)
        self.gemm(X, W, Y, M=T, N_=n, K=K, ldw=ldw, bias=bias, epi=EPI_ADD if add else epi, epi_param=epi_param,
                  exact_x=exact_x)
        return Y

    # ---- sequences of a step, and the mixers that carry a state along them (csrc/mixer_ops.cu) -------------------
    def seq_tables(self, segments, T: int):
        """-> (first (T,), seqs (G, 2), G) on the device.  segments: (first row, rows, slot, first position) per
        sequence of the step, or None: every row is a sequence of its own (a decode step; tables made once per T)"""
        if segments is None:
            if T not in self._unit_seqs:
                idx = np.arange(T, dtype=np.int32)
                both = self.to_device(np.concatenate([idx, np.stack([idx, np.ones(T, np.int32)], 1).reshape(-1)]))
                self._unit_seqs[T] = (both[:T], both[T:].view(T, 2), T)
            return self._unit_seqs[T]
        first = np.empty(T, dtype=np.int32)
        seqs = np.empty((len(segments), 2), dtype=np.int32)
        for g, (start, n, _, _) in enumerate(segments):
            first[start:start + n] = start
            seqs[g] = (start, n)
        both = self.to_device(np.concatenate([first, seqs.reshape(-1)]))
        return both[:T], both[T:].view(len(segments), 2), len(segments)

    def short_conv(self, U: torch.Tensor, w: torch.Tensor, state: torch.Tensor, ctx, act: bool = False,
                   bias: Optional[torch.Tensor] = None, residual: bool = False) -> torch.Tensor:
        """U (T, C) column range of projected rows; w (C, taps); state (slots, >= (taps-1) * C) fp32 view of the pool;
        residual: the result is U + conv(U)"""
        T, C = U.shape
        first, seqs, G = ctx.seq_tables()
        Y = self.empty((T, C))
        self._ok(self.lib.b200_lm_short_conv(U.data_ptr(), U.stride(0), w.data_ptr(), Y.data_ptr(), Y.stride(0),
                                             state.data_ptr() if state.numel() else 0, state.stride(0), ctx.slot.data_ptr(),
                                             ctx.pos.data_ptr(),
                                             first.data_ptr(), seqs.data_ptr(), G, C, w.shape[1], int(act), N.ptr(bias),
                                             int(residual), int(ctx.segments is None), T, self.s),
                 "lm_short_conv")
        return Y

    def token_shift(self, h: torch.Tensor, mu: torch.Tensor, state: torch.Tensor, ctx, operands: bool = False) -> torch.Tensor:
        """-> M (n_mix, T, C): M[s][t] = h[t] + (h[t - 1] - h[t]) * mu[s]; state (slots, C) fp32 view of the pool: the
        last input of every slot's sequence (read by the first token of a step, then replaced).  operands: M is
        (n_mix, T, ceil64(C)) bf16, zero-padded: the rows `tc_gemm` reads"""
        T, C = h.shape
        first, seqs, G = ctx.seq_tables()
        M = self.empty((mu.shape[0], T, (C + 63) // 64 * 64), torch.bfloat16) if operands else self.empty((mu.shape[0], T, C))
        self._ok(self.lib.b200_lm_token_shift(h.data_ptr(), h.stride(0), mu.data_ptr(), M.data_ptr(), M.stride(1), M.stride(0),
                                              state.data_ptr(), state.stride(0), ctx.slot.data_ptr(), ctx.pos.data_ptr(),
                                              first.data_ptr(), seqs.data_ptr(), G, C, mu.shape[0],
                                              int(ctx.segments is None), int(operands), T, self.s), "lm_token_shift")
        return M

    def qkv_post(self, Q, K, V, cache_layer, slot, pos, cs, H, G, dim, vdim, rot_dims, *, q_norm=None, k_norm=None,
                 eps: float = 0.0, v_unit: bool = False, q_temp: Optional[tuple] = None, vmix=None, v_first=None, v_keep=None):
        """Q rotated in place; cache_layer (slots, capacity, >= G * (dim + vdim)) gets the rotated K and V of the rows.
        Before that: q_norm / k_norm: RMS norm over the whole projection times these weights; q_temp (coef, every): Q times
        1 + coef ln(floor((pos + 1) / every) + 1); v_unit: every value head over its root mean square; vmix (one
        number lam) with v_first (T, G vdim): V <- (1 - lam) V + lam v_first; v_keep (T, G vdim): gets the cached values"""
        self._ok(self.lib.b200_lm_qkv_post(Q.data_ptr(), Q.stride(0), K.data_ptr(), K.stride(0), V.data_ptr(), V.stride(0),
                                           cache_layer.data_ptr(), int(cache_layer.dtype == torch.bfloat16),
                                           cache_layer.stride(0), cache_layer.stride(1), slot.data_ptr(), pos.data_ptr(),
                                           cs.data_ptr(), H, G, dim, vdim, rot_dims, N.ptr(q_norm), N.ptr(k_norm), float(eps),
                                           int(v_unit), float(q_temp[0]) if q_temp else 0.0, int(q_temp[1]) if q_temp else 0,
                                           N.ptr(vmix), N.ptr(v_first), v_first.stride(0) if v_first is not None else 0,
                                           N.ptr(v_keep), v_keep.stride(0) if v_keep is not None else 0, Q.shape[0], self.s),
                 "lm_qkv_post")

    def sink_attention(self, Q, cache_layer, slot, pos, out, sink, H, G, dim, vdim, scale, chunk=0, window=0,
                       n_split=None, bias_exp: float = 0.0, unit_sink: bool = False):
        """n_split None: enough blocks per (token, kv head) to fill the GPU when the step has few tokens, 1 for prompts;
        bias_exp > 0: 2^(-bias_exp (h + 1) / H) times the distance to the key is taken off head h's scores; unit_sink:
        the softmax's denominator also holds 1"""
        T = Q.shape[0]
        if n_split is None:
            rep = H // G
            groups = T * G * ((rep + 7) // 8)
            n_split = max(1, min(64, (2 * SM_COUNT) // groups))
            if window > 0:       # a window holds at most this many key tiles (of 32): more splits would only be merged
                n_split = min(n_split, (window + 31) // 32)
        part = self.empty((T, H, n_split, vdim + 2)) if n_split > 1 else None
        self._ok(self.lib.b200_lm_sink_attention(
            Q.data_ptr(), Q.stride(0), cache_layer.data_ptr(), int(cache_layer.dtype == torch.bfloat16),
            cache_layer.stride(0), cache_layer.stride(1), slot.data_ptr(), pos.data_ptr(), out.data_ptr(), out.stride(0),
            N.ptr(sink), H, G, dim, vdim, float(scale), int(chunk), int(window), float(bias_exp), int(unit_sink),
            N.ptr(part), n_split, T, self.s),
            "lm_sink_attention")

    def heads_to_bf16(self, q: torch.Tensor, rep: int, dim: int) -> torch.Tensor:
        """q (n, >= rep * dim) fp32 columns of `rep` heads -> bf16 rows (n * rep, ceil64(dim))"""
        n, Kp = q.shape[0], (dim + 63) // 64 * 64
        out = self.empty((n * rep, Kp), torch.bfloat16)
        self._ok(self.lib.b200_lm_heads_to_bf16(q.data_ptr(), q.stride(0), rep, dim, out.data_ptr(), Kp, n, self.s),
                 "lm_heads_to_bf16")
        return out

    def sink_softmax_bf16(self, S, pos, rep, sink, scale, chunk, window, key0, P, bias_exp: float = 0.0, head0: int = 0,
                          H: int = 1, unit_sink: bool = False, split: bool = False):
        """head0, H: the first head of the rows' group and the number of heads (they fix the slopes of the distance bias);
        split: P (rows, 2 Sp) gets every probability as two bf16 parts [hi | lo], the operand of `tc_gemm(parts=2)`"""
        self._ok(self.lib.b200_lm_sink_softmax_bf16(S.data_ptr(), S.stride(0), pos.data_ptr(), rep, N.ptr(sink), float(scale),
                                                    int(chunk), int(window), int(key0), float(bias_exp), int(head0), int(H),
                                                    int(unit_sink), int(split), P.data_ptr(), P.stride(0),
                                                    S.shape[0], P.shape[1] // 2 if split else P.shape[1], self.s),
                 "lm_sink_softmax_bf16")

    def linear_state(self, q, k, v, out, state, ctx, *, H, rep, dim, vdim, act=False, unit_eps=0.0, q_scale=1.0,
                     decay_const=None, a=None, A_log=None, dt_bias=None, b=None, delta=False, dt_in=False, skip=None,
                     decay_logits=None, bonus=None, part_len: int = 0):
        """dt_in: the state-space form, u = softplus(a + dt_bias) v; skip (H,): out += skip[h] v;
        decay_logits (T, H dim) with bonus (H, dim): a decay per key channel w = exp(-exp(decay_logits)) and
        out = S^T q + (sum_i q_i bonus_i k_i) v with S the state before the token, then S <- diag(w) S + k v^T;
        part_len > 0 (with decay_logits, a prompt step): sequences longer than that are walked in parts of part_len
        tokens at the same time (the state is linear in its start state, so the parts' contributions chain exactly)"""
        _, seqs, G = ctx.seq_tables()
        T, Hk = q.shape[0], H // rep
        # a prompt step does the per-token work (activation, unit lengths, k . q, decay, beta) in one parallel pass first
        if decay_logits is not None:
            prep = self.empty((T * (3 * H * dim + H),)) if T > SKINNY_ROWS else None
        else:
            prep = self.empty((T * (2 * Hk * dim + Hk + 2 * H),)) if T > SKINNY_ROWS else None
        scratch, n_parts = None, 0
        if decay_logits is not None and prep is not None and part_len > 0 and ctx.segments:
            n_parts = max(-(-n // part_len) for _, n, _, _ in ctx.segments)
            if n_parts > 1:
                lanes = 1
                while lanes * 8 < dim:
                    lanes *= 2
                scratch = self.empty((G * n_parts * (H * 8 * vdim * lanes + H * lanes * 8),))
        self._ok(self.lib.b200_lm_linear_state(
            q.data_ptr(), q.stride(0), k.data_ptr(), k.stride(0), v.data_ptr(), v.stride(0), out.data_ptr(), out.stride(0),
            state.data_ptr(), state.stride(0), seqs.data_ptr(), G, ctx.slot.data_ptr(), ctx.pos.data_ptr(), H, rep, dim,
            vdim, int(act), float(unit_eps), float(q_scale), N.ptr(decay_const), N.ptr(a), a.stride(0) if a is not None else 0,
            N.ptr(A_log), N.ptr(dt_bias), N.ptr(b), b.stride(0) if b is not None else 0, int(delta), int(dt_in), N.ptr(skip),
            N.ptr(decay_logits), decay_logits.stride(0) if decay_logits is not None else 0, N.ptr(bonus),
            N.ptr(prep), int(part_len) if scratch is not None else 0, n_parts, N.ptr(scratch), T, self.s),
            "lm_linear_state")

    def head_post(self, o, out, *, dv, gate=None, gate_per_head=False, gate_silu=False, w=None, eps=0.0, span=0,
                  scale=1.0, gate_first=False):
        T, n = o.shape
        self._ok(self.lib.b200_lm_head_post(o.data_ptr(), o.stride(0), N.ptr(gate), gate.stride(0) if gate is not None else 0,
                                            N.ptr(w), w.numel() if w is not None else 0, float(eps), int(span),
                                            int(gate_per_head), int(gate_silu), dv, n, float(scale), out.data_ptr(),
                                            out.stride(0), int(gate_first), T, self.s), "lm_head_post")

    def glu_clamp(self, G, U, limit, alpha, Y, up_offset: float = 1.0, cubic: float = 0.0):
        """Y = g sigmoid(alpha (g + cubic g^3)) (u + up_offset), g = min(G, limit), u = clamp(U, +-limit); limit inf,
        alpha 1 and up_offset 0 give the plain silu-gated unit; GELU_TANH_ALPHA and GELU_TANH_CUBIC the tanh form of gelu"""
        T, n = G.shape
        self._ok(self.lib.b200_lm_glu_clamp(G.data_ptr(), G.stride(0), U.data_ptr(), U.stride(0), float(limit),
                                            float(alpha), float(cubic), float(up_offset), Y.data_ptr(), Y.stride(0), n, T,
                                            self.s),
                 "lm_glu_clamp")

    def glu_clamp_bf16(self, G, U, limit, alpha, up_offset: float = 1.0, live: Optional[torch.Tensor] = None,
                       cubic: float = 0.0) -> torch.Tensor:
        """the gated activation written as bf16 operand rows (T, ceil64(n)) of the next tensor-core product; live (T,)
        int32: rows with a negative entry (padding of sorted expert segments) become zeros without being read"""
        T, n = G.shape
        Kp = (n + 63) // 64 * 64
        Y = self.empty((T, Kp), torch.bfloat16)
        self._ok(self.lib.b200_lm_glu_clamp_bf16(G.data_ptr(), G.stride(0), U.data_ptr(), U.stride(0), float(limit),
                                                 float(alpha), float(cubic), float(up_offset), Y.data_ptr(), n, Kp,
                                                 N.ptr(live), T, self.s),
                 "lm_glu_clamp_bf16")
        return Y

    def argmax_rows(self, z, tok, logprob=None):
        B, V = z.shape
        self._ok(self.lib.b200_lm_argmax_rows(z.data_ptr(), z.stride(0), V, tok.data_ptr(), N.ptr(logprob), B, self.s),
                 "lm_argmax_rows")

    def advance_rows(self, sampled, tok, pos, active, log, step, lp=None, lp_log=None):
        """log (and lp_log): (rows, B-wide) rings, step: (1,) int32 device counter (row = step mod rows; counts up)"""
        B = tok.shape[0]
        self._ok(self.lib.b200_lm_advance_rows(sampled.data_ptr(), tok.data_ptr(), pos.data_ptr(), N.ptr(active),
                                               log.data_ptr(), log.stride(0), log.shape[0], step.data_ptr(),
                                               N.ptr(lp), N.ptr(lp_log), B, self.s), "lm_advance_rows")
