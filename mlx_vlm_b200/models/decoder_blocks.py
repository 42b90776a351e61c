"""Decoder mechanisms that a design picks by name in its configuration, each with its sizes and constants as
parameters, its packed weight layout and its launch sequence over the layer ops (layer_ops.py):

  mixers         MIXERS["latent_attention"]  -> LatentAttention
  feed-forwards  FEEDFORWARDS["moe"]         -> ExpertMixture
  layer          PostNormLayer: x += norm(mixer(x)); x += norm(ff(x)), weights of the norms stored around zero

and, for layers whose sublayers all read ONE normed input (so that all their input projections are one product and
all their output projections another), the parts of a `SharedInputLayer`:

  mixers         FUSED_MIXERS["attention"]  -> SinkAttention   (grouped heads, sink logit, block-local keys, gate)
                 FUSED_MIXERS["lightning"]  -> DecayedState    (outer-product state with a fixed decay per head)
                 FUSED_MIXERS["parallel"]   -> an attention and a GatedDeltaRule side by side, weighted
  feed-forwards  FUSED_FEEDFORWARDS["dense"] -> ClampedGLU
  layer          SharedInputLayer: n = norm(x); x += sum of the parts' outputs

and, for pre-norm layers with a layer norm before each sublayer and a scale vector on each branch:

  mixers         SCALED_MIXERS["latent_attention"] -> LatentAttention without a query latent, rotation in pairs
                                                       (2i, 2i + 1), YaRN-scaled frequencies, a window, an output gate
                 SCALED_MIXERS["mamba2"]           -> StateSpaceMixer (convolution + matrix state with a step size)
  feed-forwards  SCALED_FEEDFORWARDS["dense"]      -> GatedDense (silu-gated unit)
                 SCALED_FEEDFORWARDS["moe"]        -> GroupedExpertMixture (sigmoid scores with a selection bias, the
                                                       choice limited to the best groups, clamped gated experts, a shared
                                                       expert with a gate per token)
  layer          ScaledPreNormLayer: x += s1 * mixer(LN(x)); x += s2 * ff(LN(x))

and, for pre-norm layers with an RMS norm in groups, ONE multiplier on both branches and a causal convolution over time
on what the mixer reads:

  mixers         CONV_MIXERS["attention"]    -> GroupedAttention with norms over the whole query / key projection,
                                                 YaRN-scaled rotate-half rotary, unit-length values, a sink logit per head
                 CONV_MIXERS["attention_2"]  -> GroupedAttention without rotation: a query temperature that grows with the
                                                 position, a distance bias per head, a sliding window, one in the denominator
                 (both: values mixed with those of the first such layer)
                 CONV_MIXERS["wkv"]          -> TokenShiftState (token shift, a decay per key channel made from the input,
                                                 a bonus for the current token, a matrix state per head)
  feed-forwards  CONV_FEEDFORWARDS["dense"]  -> GatedDense with the tanh form of gelu on the gate
                 CONV_FEEDFORWARDS["moe"]    -> UngatedExpertMixture (softmax scores, the choice limited to the best groups,
                                                 erf-gelu experts, a shared expert)
  layer          ConvPreNormLayer: h = N1(x); h += conv(h); x += m * mixer(h); x += m * ff(N2(x))

A block declares `manifest(prefix)` (packed name, shape) and `pack(prefix, checkpoint tensors, arena)`; the model
packs all blocks into ONE device arena (the layout the other models of this package use).  `forward(ctx, x)`
enqueues the block's kernels; `ctx` carries the per-token slot / position arrays of the step and the cache pool,
so a prompt, a portion of a prompt, a decoded token and a batch of unequal requests are the same code.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch

from .._native import B200Error as _B200Error
from .layer_ops import ACT_GELU, ACT_TANH, EPI_GELU, EPI_RELU2, EPI_SOFTCAP, GELU_TANH_ALPHA, GELU_TANH_CUBIC, LayerOps


@dataclass
class StepCtx:
    ops: LayerOps
    slot: torch.Tensor            # (T,) int32 device: cache slot of every token of the step
    pos: torch.Tensor             # (T,) int32 device: position of every token in its sequence
    pool: object                  # LatentPool
    eps: float
    segments: Optional[List] = None   # host view of the step: (first token, tokens, slot, first position) per request
    _rope: Dict = field(default_factory=dict)
    _seq: Optional[tuple] = None
    carry: Dict = field(default_factory=dict)     # what one layer of the step leaves for later ones (rows of the step)

    def seq_tables(self):
        """(first (T,), seqs (G, 2), G): the sequences of the step for the mixers that walk them in order; without a
        host view every token is a sequence of its own (a decode step)"""
        if self._seq is None:
            self._seq = self.ops.seq_tables(self.segments, self.pos.shape[0])
        return self._seq

    def rope(self, base: float, dims: int, scaling: Optional[tuple] = None) -> torch.Tensor:
        key = (float(base), int(dims), scaling)
        if key not in self._rope:
            self._rope[key] = self.ops.rope_table(self.pos, base, dims, scaling)
        return self._rope[key]


class LatentAttention:
    """Attention whose keys and values are expanded from one cached latent row per token.

    q = W_uq rmsnorm(W_dq h);  [c | r] = W_dkv h, c rms-normed, r rotated: the cache row of the token;
    per head  k = [W_uk c | r],  v = W_uv c;  softmax(scale * q.k) over the causal prefix;  W_o on the heads.
    `kv_from = j`: no W_dkv, the rows that layer j cached are read instead (same rank and rotation).
    The rotation is on the first `rot_dims` of the rotated part, frequency base `rot_base`; its pairs are
    (i, i + rot_dims / 2) (`rotation="half"`) or (2i, 2i + 1) (`rotation="pairs"`); `rot.scaling` (factor, original,
    fast, slow) rescales the frequencies by the YaRN rule and cos / sin by 0.1 ln(factor) + 1.
    Without `q_rank` there is no query latent: q = W_q h.  `mask.size = w`: a query at position p sees the keys
    p - w + 1 .. p.  `gated`: the heads' outputs are multiplied by sigmoid(W_g h) before W_o."""

    def __init__(self, index: int, cfg: dict, width: int, rotation: str = "half", gated: bool = False):
        self.index, self.W = index, width
        self.H, self.dim, self.rot_dim, self.vdim = cfg["heads"], cfg["dim"], cfg["rot_dim"], cfg["vdim"]
        self.kv_rank, self.q_rank, self.scale = cfg["kv_rank"], int(cfg.get("q_rank") or 0), float(cfg["scale"])
        rot = cfg.get("rot") or {}
        self.rot_base, self.rot_dims = float(rot.get("base", 10000.0)), int(rot.get("dims", self.rot_dim))
        sc = rot.get("scaling")
        self.rot_scaling = None if not sc else (float(sc["factor"]), float(sc["original"]), float(sc["fast"]),
                                                float(sc["slow"]))
        if rotation not in ("half", "pairs"):
            raise ValueError(f"layer {index}: rotation {rotation!r} (have 'half', 'pairs')")
        self.pairs, self.gated = rotation == "pairs", bool(gated)
        self.window = int((cfg.get("mask") or {}).get("size", 0))
        self.kv_from: Optional[int] = cfg.get("kv_from")
        if not self.q_rank and self.kv_from is not None:
            raise ValueError(f"layer {index}: a layer that borrows its latent needs a query latent")
        self.n_q = self.H * (self.dim + self.rot_dim)
        self.cache_index = -1     # set by the model: which caching layer of the pool this mixer reads (and writes)
        self.kv_dim, self.state_floats, self.state_off = self.kv_rank + self.rot_dim, 0, 0
        self.w: Dict[str, torch.Tensor] = {}

    @property
    def own_kv(self) -> bool:
        return self.kv_from is None

    @property
    def row_dim(self) -> int:
        return self.kv_rank + self.rot_dim

    def manifest(self, p: str):
        # `down`: every product that reads the layer's input, stacked: [query latent, or the queries themselves |
        # kv latent, rotated key part | gate]
        n_down = (self.q_rank or self.n_q) + (self.row_dim if self.own_kv else 0) + (self.H * self.vdim if self.gated else 0)
        out = [(p + "down", (n_down, self.W))]
        if self.q_rank:
            out += [(p + "dq.norm", (self.q_rank,)), (p + "uq", (self.n_q, self.q_rank))]
        out += [(p + "ukT", (self.H, self.kv_rank, self.dim)), (p + "uv", (self.H * self.vdim, self.kv_rank)),
                (p + "o", (self.W, self.H * self.vdim))]
        if self.own_kv:
            out.append((p + "dkv.norm", (self.kv_rank,)))
        return out

    def checkpoint_tensors(self, p: str) -> Dict[str, tuple]:
        """checkpoint name -> shape of everything this mixer reads"""
        out = {p + "uk": (self.H * self.dim, self.kv_rank), p + "uv": (self.H * self.vdim, self.kv_rank),
               p + "o": (self.W, self.H * self.vdim)}
        if self.q_rank:
            out.update({p + "dq": (self.q_rank, self.W), p + "dq.norm": (self.q_rank,), p + "uq": (self.n_q, self.q_rank)})
        else:
            out[p + "q"] = (self.n_q, self.W)
        if self.own_kv:
            out.update({p + "dkv": (self.row_dim, self.W), p + "dkv.norm": (self.kv_rank,)})
        if self.gated:
            out[p + "g"] = (self.H * self.vdim, self.W)
        return out

    def pack(self, p: str, ck: Dict[str, torch.Tensor], view):
        """ck: checkpoint tensors '<p>dq', '<p>dq.norm', '<p>uq' (or '<p>q'), '<p>dkv', '<p>dkv.norm', '<p>uk', '<p>uv',
        '<p>o' (and '<p>g')"""
        down = view(p + "down")
        at = self.q_rank or self.n_q
        down[:at].copy_(ck[p + "dq"] if self.q_rank else ck[p + "q"])
        if self.own_kv:
            down[at:at + self.row_dim].copy_(ck[p + "dkv"])  # one product for everything that reads the input
            view(p + "dkv.norm").copy_(ck[p + "dkv.norm"])
            at += self.row_dim
        if self.gated:
            down[at:].copy_(ck[p + "g"])
        for n in (("dq.norm", "uq") if self.q_rank else ()) + ("uv", "o"):
            view(p + n).copy_(ck[p + n])
        # the key up-projection per head, transposed: it is applied to the QUERY (absorbed form)
        view(p + "ukT").copy_(ck[p + "uk"].view(self.H, self.dim, self.kv_rank).transpose(1, 2))
        self.bind(p, view)

    def bind(self, p: str, view):
        self.w = {n[len(p):]: view(n) for n, _ in self.manifest(p)}

    def forward(self, ctx: StepCtx, x: torch.Tensor) -> torch.Tensor:
        ops, w, T = ctx.ops, self.w, x.shape[0]
        H, dn, dr, r, dv = self.H, self.dim, self.rot_dim, self.kv_rank, self.vdim
        Dl = r + dr
        D = ops.linear(x, w["down"])
        cache_layer = ctx.pool.buf[self.cache_index][..., :Dl]    # a pool row may be wider than this layer's
        cs = ctx.rope(self.rot_base, self.rot_dims, self.rot_scaling)
        if self.q_rank:
            cq = ops.empty((T, self.q_rank))
            ops.latent_post(D, w["dq.norm"], w.get("dkv.norm"), ctx.eps, cq, cache_layer if self.own_kv else None,
                            ctx.slot, ctx.pos, cs, self.q_rank, r, dr, self.rot_dims, pairs=self.pairs)
            q = ops.linear(cq, w["uq"])
            n_read = self.q_rank + (Dl if self.own_kv else 0)
        else:             # the queries come straight from the input: the first columns of D
            ops.latent_post(D[:, self.n_q:], None, w["dkv.norm"], ctx.eps, None, cache_layer, ctx.slot, ctx.pos, cs, 0, r,
                            dr, self.rot_dims, pairs=self.pairs)
            q = D[:, :self.n_q]
            n_read = self.n_q + Dl
        qa = ops.empty((T, H * Dl))
        heads_tc = ops.tc_ok(T, dn, dn + dr, r) and dn % 64 == 0 and r % 64 == 0 and Dl % 4 == 0 and dv % 4 == 0
        if heads_tc:     # a prompt: the heads' products as ONE tcgen05 launch (inner sizes are whole k-blocks)
            try:
                qb = ops.to_bf16(q, H * (dn + dr))
                ops.tc_gemm_heads(qb, w["ukT"], qa, H=H, N_=r, K=dn, x_cols=qb.shape[1], x_group_cols=dn + dr,
                                  c_group_cols=Dl)
            except _B200Error as e:
                ops.tc_refused(e)
                heads_tc = False
        if not heads_tc:
            ops.gemm(q, w["ukT"], qa, M=T, N_=r, K=dn, xb=dn + dr, ldw=dn, wb=r * dn, yb=Dl, batch=H)
        ops.rope_q(q, qa, cs, H, dn, dr, self.rot_dims, r, pairs=self.pairs)
        ol = ops.empty((T, H * r))
        segs = ctx.segments or []
        done = False
        if any(ops.tc_ok(n, Dl, r, cache_layer.stride(1)) for _, n, _, _ in segs) and cache_layer.dtype == torch.bfloat16:
            try:
                for start, n, slot, p0 in segs:      # long portions on the tensor cores, the rest on the row kernel
                    sl = slice(start, start + n)
                    if ops.tc_ok(n, Dl, r, cache_layer.stride(1)):
                        self._attend_prompt(ops, qa[sl], cache_layer[slot], ctx.pos[sl], ol[sl], p0, n)
                    else:
                        ops.latent_attention(qa[sl], cache_layer, ctx.slot[sl], ctx.pos[sl], ol[sl], H, r, self.scale,
                                             n_split=1, window=self.window)
                done = True
            except _B200Error as e:
                ops.tc_refused(e)
        if not done:
            ops.latent_attention(qa, cache_layer, ctx.slot, ctx.pos, ol, H, r, self.scale, window=self.window,
                                 n_split=1 if ctx.segments is not None and T > 16 else None)
        att = ops.empty((T, H * dv))
        if heads_tc:
            try:
                ob = ops.to_bf16(ol, H * r)
                ops.tc_gemm_heads(ob, w["uv"], att, H=H, N_=dv, K=r, x_cols=ob.shape[1], x_group_cols=r, c_group_cols=dv)
            except _B200Error as e:
                ops.tc_refused(e)
                heads_tc = False
        if not heads_tc:
            ops.gemm(ol, w["uv"], att, M=T, N_=dv, K=r, xb=r, ldw=r, wb=dv * r, yb=dv, batch=H)
        if self.gated:       # the gate reads the layer's input like the projections: the last columns of D
            ops.head_post(att, att, dv=dv, gate=D[:, n_read:])
        return ops.linear(att, w["o"])


    def _attend_prompt(self, ops: LayerOps, qa, rows, pos, ol, p0: int, n: int):
        """A portion of a prompt (positions p0 .. p0 + n - 1) against the cached rows of its slot as two tcgen05
        products: the cache rows are the weight-major operand of the scores (absorbed queries x rows), the softmax
        over the visible keys runs in fp32 over the score rows, and the transposed latent columns are the operand of
        the weighted sum.  Queries are taken in chunks that bound the score buffer; with a window a chunk is about a
        window long and meets only the rows from its first query's first visible key on."""
        H, r, Dl = self.H, self.kv_rank, self.kv_rank + self.rot_dim
        if not self.window:
            S = p0 + n
            Sp = (S + 63) // 64 * 64
            ct = ops.cache_transpose(rows, S, Sp, r)
            step = max(1, min(n, (1 << 27) // (H * Sp)))
            for a in range(0, n, step):
                m = min(step, n - a)
                qb = ops.to_bf16(qa[a:a + m].view(m * H, Dl), Dl)
                sc = ops.empty((m * H, S))
                ops.tc_gemm(qb, rows, sc, N_=S, K=Dl, ldw=rows.stride(0))
                P = ops.empty((m * H, Sp), torch.bfloat16)
                ops.masked_softmax_bf16(sc, pos[a:a + m], H, self.scale, P)
                ops.tc_gemm(P, ct, ol[a:a + m].view(m * H, r), N_=r, K=Sp)
            return
        step = max(128, min(self.window, (1 << 27) // (H * 2 * self.window)))
        step = -(-n // -(-n // step))          # equal chunks: no short one at the end
        for a in range(0, n, step):
            m = min(step, n - a)
            key0 = max(p0 + a - self.window + 1, 0)
            S = p0 + a + m - key0
            Sp = (S + 63) // 64 * 64
            ct = ops.cache_transpose(rows[key0:], S, Sp, r)
            qb = ops.to_bf16(qa[a:a + m].view(m * H, Dl), Dl)
            sc = ops.empty((m * H, S))
            ops.tc_gemm(qb, rows[key0:], sc, N_=S, K=Dl, ldw=rows.stride(0))
            P = ops.empty((m * H, Sp), torch.bfloat16)
            ops.sink_softmax_bf16(sc, pos[a:a + m], H, None, self.scale, 0, self.window, key0, P)
            ops.tc_gemm(P, ct, ol[a:a + m].view(m * H, r), N_=r, K=Sp)


class ExpertMixture:
    """`experts` small feed-forwards W_down relu(W_up h)^2 without biases; a token uses the `top` experts with the
    largest router logits (fp32, with a bias), weighted by the softmax over those logits only."""

    def __init__(self, index: int, cfg: dict, width: int):
        self.index, self.W = index, width
        self.E, self.top, self.ff = cfg["router"]["experts"], cfg["router"]["top"], cfg["expert"]["ff"]
        self.w: Dict[str, torch.Tensor] = {}

    def manifest(self, p: str):
        return [(p + "router", (self.E, self.W)), (p + "router.b", (self.E,)), (p + "up", (self.E, self.ff, self.W)),
                (p + "down", (self.E, self.W, self.ff))]

    def pack(self, p: str, ck: Dict[str, torch.Tensor], view):
        view(p + "router").copy_(ck[p + "router"])
        view(p + "router.b").copy_(ck[p + "router.b"])
        up, down = view(p + "up"), view(p + "down")
        for e in range(self.E):
            up[e].copy_(ck[p + f"e{e}.up"])
            down[e].copy_(ck[p + f"e{e}.down"])
        self.bind(p, view)

    def bind(self, p: str, view):
        self.w = {n[len(p):]: view(n) for n, _ in self.manifest(p)}

    def forward(self, ctx: StepCtx, x: torch.Tensor):
        """-> (rows (T * top, W) of the chosen experts' outputs, weights (T, top)): the layer's norm sums them"""
        ops, w, T = ctx.ops, self.w, x.shape[0]
        z = ops.linear(x, w["router"], bias=w["router.b"])
        idx, wgt = ops.router_topk(z, self.top)
        lists, count = ops.moe_group(idx, self.E)
        if ops.tc_ok(T, self.W, self.ff):
            try:
                return self._experts_prompt(ops, x, lists, count), wgt
            except _B200Error as e:
                ops.tc_refused(e)
        hid = ops.empty((T * self.top, self.ff))
        ops.gemm(x, w["up"], hid, M=T, N_=self.ff, K=self.W, wb=self.ff * self.W, batch=self.E, lists=lists,
                 count=count, x_div=self.top, epi=EPI_RELU2, compact=min(self.E, T * self.top))
        out = ops.empty((T * self.top, self.W))
        ops.gemm(hid, w["down"], out, M=T, N_=self.W, K=self.ff, wb=self.W * self.ff, batch=self.E, lists=lists,
                 count=count, x_div=1, compact=min(self.E, T * self.top))
        return out, wgt


    def _experts_prompt(self, ops: LayerOps, x, lists, count):
        """A prompt step on the tensor cores, without the host knowing how the tokens spread over the experts: the
        (token, choice) entries are sorted by expert into segments padded to whole token tiles, with the expert of
        every tile in a device table; ONE launch gathers and rounds all input rows in that order, ONE grouped tcgen05
        launch per projection multiplies every tile by its expert's weights (empty tiles leave at once), ONE launch
        applies relu^2 and rounds the hidden rows, ONE launch scatters the outputs back to entry order."""
        w, T = self.w, x.shape[0]
        n_all = T * self.top
        order, group = ops.moe_tiles(lists, count, n_all)
        n_rows = order.shape[0]
        xs = ops.to_bf16(x, self.W, rows=n_rows, row_map=order, div=self.top)
        hs = ops.empty((n_rows, self.ff))
        ops.tc_gemm_grouped(xs, w["up"], hs, group, N_=self.ff, K=self.W, n_groups=self.E)
        hb = ops.to_bf16(hs, self.ff, relu2=True)
        ys = ops.empty((n_rows, self.W))
        ops.tc_gemm_grouped(hb, w["down"], ys, group, N_=self.W, K=self.ff, n_groups=self.E)
        out = ops.empty((n_all, self.W))
        ops.rows_scatter(ys, order, out, n_rows)
        return out


MIXERS = {"latent_attention": LatentAttention}
FEEDFORWARDS = {"moe": ExpertMixture}


class PostNormLayer:
    """x <- x + N1(mixer(x)); x <- x + N2(ff(x)), N = RMS norm with weight (1 + w); the sublayers read x itself."""

    def __init__(self, index: int, cfg: dict, width: int):
        self.index, self.W = index, width
        if cfg["type"] not in MIXERS:
            raise ValueError(f"layer {index}: unknown mixer type {cfg['type']!r} (have {sorted(MIXERS)})")
        self.mixer = MIXERS[cfg["type"]](index, cfg["mixer"], width)
        f = cfg.get("mlp")
        if f is not None and f.get("kind") not in FEEDFORWARDS:
            raise ValueError(f"layer {index}: unknown feed-forward kind {f.get('kind')!r} (have {sorted(FEEDFORWARDS)})")
        self.ff = None if f is None else FEEDFORWARDS[f["kind"]](index, f, width)
        self.w: Dict[str, torch.Tensor] = {}

    def manifest(self, p: str):
        out = [(p + "norm1", (self.W,))] + self.mixer.manifest(p + "mix.")
        if self.ff is not None:
            out += [(p + "norm2", (self.W,))] + self.ff.manifest(p + "mlp.")
        return out

    def pack(self, p: str, ck, view):
        view(p + "norm1").copy_(ck[p + "norm1"])
        self.mixer.pack(p + "mix.", ck, view)
        if self.ff is not None:
            view(p + "norm2").copy_(ck[p + "norm2"])
            self.ff.pack(p + "mlp.", ck, view)
        self.bind(p, view)

    def bind(self, p: str, view):
        """point the blocks at their views of the arena (after packing a checkpoint or filling the arena directly)"""
        self.w["norm1"] = view(p + "norm1")
        self.mixer.bind(p + "mix.", view)
        if self.ff is not None:
            self.w["norm2"] = view(p + "norm2")
            self.ff.bind(p + "mlp.", view)

    def forward(self, ctx: StepCtx, x: torch.Tensor):
        ops = ctx.ops
        y = self.mixer.forward(ctx, x)
        ops.norm_rows(y, self.w["norm1"], ctx.eps, x, w_offset=1.0, add=True)
        if self.ff is not None:
            rows, wgt = self.ff.forward(ctx, x)
            ops.norm_rows(rows, self.w["norm2"], ctx.eps, x, w_offset=1.0, add=True, combine=wgt, top=self.ff.top)


# ----------------------------------------------------------------------------------------------------------------
# Parts of a layer whose sublayers share their input.  A part names the rows it adds to the layer's input projection
# (`in_names`, stacked in that order; `n_in` rows in all), the columns it adds to the output projection (`out_name`,
# `n_out`), its other tensors (`small`), what it keeps per request (`kv_dim` numbers per cached token, `state_floats`
# fp32 numbers per slot), and `forward(ctx, D, cat, kv_layer, state_off, out_scale)`: D (T, n_in) its columns of the
# projected rows (scratch: it may overwrite them), cat (T, n_out) its columns of the output projection's input.
class SinkAttention:
    """Softmax attention with `heads` query heads over `kv_heads` key/value heads (query head h reads key/value head
    h // (heads / kv_heads)), rotate-half rotary on the first `rot.dims` numbers of every query and key head, an
    optional short causal convolution on q, k, v before the rotation (`conv` taps), keys limited to the query's own
    block of `mask.size` positions (absent: all earlier positions), a learned logit per head that joins the softmax's
    denominator without a key or a value (`sink`), and a sigmoid gate on the heads' outputs computed from the layer's
    input: one number per output element (`gate="element"`) or per head (`gate="head"`)."""

    def __init__(self, index: int, cfg: dict, width: int, gate: str = "element"):
        self.index, self.W, self.gate = index, width, gate
        self.H, self.dim = int(cfg["heads"]), int(cfg["dim"])
        self.G, self.vdim = int(cfg.get("kv_heads", self.H)), int(cfg.get("vdim", self.dim))
        if self.H % self.G:
            raise ValueError(f"layer {index}: {self.H} query heads do not divide over {self.G} key/value heads")
        self.scale = float(cfg.get("scale", float(self.dim) ** -0.5))
        rot = cfg.get("rot") or {}
        self.rot_base, self.rot_dims = float(rot.get("base", 10000.0)), int(rot.get("dims", 0))
        self.chunk = int((cfg.get("mask") or {}).get("size", 0))
        self.window = int(cfg.get("window", 0))
        self.taps = int(cfg.get("conv") or 0)
        self.n_q, self.n_k, self.n_v = self.H * self.dim, self.G * self.dim, self.G * self.vdim
        self.n_gate = self.H * self.vdim if gate == "element" else self.H
        self.in_names, self.out_name = ["q", "k", "v", "g"], "o"
        self.n_in, self.n_out = self.n_q + self.n_k + self.n_v + self.n_gate, self.H * self.vdim
        self.kv_dim = self.n_k + self.n_v
        self.state_floats = max(self.taps - 1, 0) * (self.n_q + self.n_k + self.n_v)
        self.w: Dict[str, torch.Tensor] = {}

    def in_rows(self, name: str) -> int:
        return {"q": self.n_q, "k": self.n_k, "v": self.n_v, "g": self.n_gate}[name]

    def small(self):
        out = [("sink", (self.H,))]
        if self.taps:
            out.append(("conv", (self.n_q + self.n_k + self.n_v, self.taps)))
        return out

    def checkpoint_small(self):
        """packed name -> the checkpoint tensors it is stacked from"""
        out = {"sink": ["sink"]}
        if self.taps:
            out["conv"] = ["q.conv", "k.conv", "v.conv"]
        return out

    def forward(self, ctx: StepCtx, D, cat, kv_layer: int, state_off: int, out_scale: float = 1.0):
        ops, w, T = ctx.ops, self.w, D.shape[0]
        nq, nk, nv = self.n_q, self.n_k, self.n_v
        src = D
        if self.taps:
            src = ops.short_conv(D[:, :nq + nk + nv], w["conv"], ctx.pool.state[:, state_off:state_off + self.state_floats],
                                 ctx)
        q, k, v = src[:, :nq], src[:, nq:nq + nk], src[:, nq + nk:nq + nk + nv]
        rows = ctx.pool.buf[kv_layer][..., :self.kv_dim]
        ops.qkv_post(q, k, v, rows, ctx.slot, ctx.pos, ctx.rope(self.rot_base, self.rot_dims), self.H, self.G, self.dim,
                     self.vdim, self.rot_dims)
        o = ops.empty((T, self.n_out))
        segs = ctx.segments or []
        done = False
        if rows.dtype == torch.bfloat16 and not self.window and any(self._tc_portion(ops, n, rows) for _, n, _, _ in segs):
            try:
                for start, n, slot, p0 in segs:      # long portions on the tensor cores, the rest on the row kernel
                    sl = slice(start, start + n)
                    if self._tc_portion(ops, n, rows):
                        self._attend_prompt(ctx, q[sl], rows, slot, ctx.slot[sl], ctx.pos[sl], o[sl], p0, n)
                    else:
                        self._attend_rows(ctx, q[sl], rows, ctx.slot[sl], ctx.pos[sl], o[sl], prompt=True)
                done = True
            except _B200Error as e:
                ops.tc_refused(e)
        if not done:
            self._attend_rows(ctx, q, rows, ctx.slot, ctx.pos, o, prompt=ctx.segments is not None)
        ops.head_post(o, cat, dv=self.vdim, gate=D[:, nq + nk + nv:], gate_per_head=self.gate == "head", scale=out_scale)

    def _tc_portion(self, ops: LayerOps, n: int, rows) -> bool:
        return ops.tc_ok(n, self.dim, rows.stride(1)) and rows.stride(0) % 8 == 0

    def _attend_rows(self, ctx: StepCtx, q, rows, slot, pos, o, prompt: bool):
        """the row kernel: every query finds its keys by (slot, position); a step of few tokens (decoding) spreads the
        keys of a query over several blocks"""
        ctx.ops.sink_attention(q, rows, slot, pos, o, self.w["sink"], self.H, self.G, self.dim, self.vdim, self.scale,
                               chunk=self.chunk, window=self.window, n_split=1 if prompt and q.shape[0] > 16 else None)

    def _attend_prompt(self, ctx: StepCtx, q, all_rows, slot_index: int, slot, pos, o, p0: int, n: int):
        """A portion of a prompt (positions p0 .. p0 + n - 1 of one slot) as two tcgen05 products per key/value head:
        the cached key columns of that head are the weight-major operand of the scores of the query heads that share
        it, an fp32 softmax over the visible keys (with the sink logit in the denominator) writes bf16 probabilities,
        and the head's value columns, transposed, are the operand of the weighted sum.  With block-local keys the
        portion is taken block by block, each against the keys of its own block only.  Queries are taken in chunks
        that bound the score buffer; a block's share of fewer rows than a tile goes to the row kernel."""
        ops, H, G, d, dv = ctx.ops, self.H, self.G, self.dim, self.vdim
        rep, rows = H // G, all_rows[slot_index]
        if self.chunk:
            spans = [(max(p0, b * self.chunk), min(p0 + n, (b + 1) * self.chunk), b * self.chunk)
                     for b in range(p0 // self.chunk, (p0 + n - 1) // self.chunk + 1)]
        else:
            spans = [(p0, p0 + n, 0)]
        for qa, qb, key0 in spans:
            m, a0 = qb - qa, qa - p0
            if not ops.tc_ok(m, d):
                sl = slice(a0, a0 + m)
                self._attend_rows(ctx, q[sl], all_rows, slot[sl], pos[sl], o[sl], prompt=True)
                continue
            S = qb - key0
            Sp = (S + 63) // 64 * 64
            step = max(1, min(m, (1 << 27) // (rep * Sp)))
            for g in range(G):
                keys = rows[key0:key0 + S, g * d:(g + 1) * d]
                vt = ops.cache_transpose(rows[key0:, G * d + g * dv:], S, Sp, dv)
                for a in range(a0, a0 + m, step):
                    mm = min(step, a0 + m - a)
                    qb16 = ops.heads_to_bf16(q[a:a + mm, g * rep * d:], rep, d)
                    sc = ops.empty((mm * rep, S))
                    ops.tc_gemm(qb16, keys, sc, N_=S, K=d, ldw=rows.stride(0))
                    P = ops.empty((mm * rep, Sp), torch.bfloat16)
                    ops.sink_softmax_bf16(sc, pos[a:a + mm], rep, self.w["sink"][g * rep:], self.scale, self.chunk, 0, key0, P)
                    og = ops.empty((mm * rep, dv))
                    ops.tc_gemm(P, vt, og, N_=dv, K=Sp)
                    ops.head_post(og.view(mm, rep * dv), o[a:a + mm, g * rep * dv:(g + 1) * rep * dv], dv=dv)


STATE_ROWS = 8     # rows of a matrix state's column that one thread holds (csrc/mixer_ops.cu: LS_R)


def state_lanes(dim: int) -> int:
    """threads that share a column of a matrix state (STATE_ROWS rows each; a power of two up to a warp): it fixes
    the layout of the state in the slot, [heads][STATE_ROWS][vdim][lanes]"""
    if dim > 32 * STATE_ROWS:
        raise ValueError(f"a matrix state with {dim} rows is not supported (at most {32 * STATE_ROWS})")
    lanes = 1
    while lanes * STATE_ROWS < dim:
        lanes *= 2
    return lanes


def state_floats(heads: int, dim: int, vdim: int) -> int:
    return heads * STATE_ROWS * vdim * state_lanes(dim)


class GatedDeltaRule:
    """Gated delta rule: per head a (dim, vdim) state with  S <- g S;  S <- S + k (beta (v - S^T k))^T;  o = S^T q.
    q, k (`kv_heads` heads, shared by heads / kv_heads value heads) and v pass a short causal convolution and silu; q, k
    are then scaled to unit length (q also by dim^-1/2); beta = sigmoid(W_b n); g = exp(-exp(A_log) softplus(W_a n +
    dt_bias)); every head's output is RMS-normed over vdim, weighted, and gated by silu(W_g n)."""

    def __init__(self, index: int, cfg: dict, width: int, unit_eps: float = 1e-6):
        self.index, self.W, self.unit_eps = index, width, unit_eps
        self.H, self.dim, self.taps = int(cfg["heads"]), int(cfg["dim"]), int(cfg.get("conv") or 1)
        self.G, self.vdim = int(cfg.get("kv_heads", self.H)), int(cfg.get("vdim", self.dim))
        if self.H % self.G:
            raise ValueError(f"layer {index}: {self.H} value heads do not divide over {self.G} query/key heads")
        self.n_qk, self.n_v = self.G * self.dim, self.H * self.vdim
        self.n_conv = 2 * self.n_qk + self.n_v
        self.in_names, self.out_name = ["q", "k", "v", "b", "a", "g"], "o"
        self.n_in, self.n_out = self.n_conv + 2 * self.H + self.n_v, self.n_v
        self.kv_dim = 0
        self.conv_floats = max(self.taps - 1, 0) * self.n_conv
        self.state_floats = self.conv_floats + state_floats(self.H, self.dim, self.vdim)
        self.w: Dict[str, torch.Tensor] = {}

    def in_rows(self, name: str) -> int:
        return {"q": self.n_qk, "k": self.n_qk, "v": self.n_v, "b": self.H, "a": self.H, "g": self.n_v}[name]

    def small(self):
        return [("conv", (self.n_conv, self.taps)), ("A_log", (self.H,)), ("dt_bias", (self.H,)), ("norm", (self.vdim,))]

    def checkpoint_small(self):
        return {"conv": ["q.conv", "k.conv", "v.conv"], "A_log": ["A_log"], "dt_bias": ["dt_bias"], "norm": ["norm"]}

    def forward(self, ctx: StepCtx, D, cat, kv_layer: int, state_off: int, out_scale: float = 1.0):
        ops, w, T = ctx.ops, self.w, D.shape[0]
        n, nc, H = self.n_qk, self.n_conv, self.H
        st = ctx.pool.state
        c = ops.short_conv(D[:, :nc], w["conv"], st[:, state_off:state_off + self.conv_floats], ctx, act=True)
        o = ops.empty((T, self.n_out))
        ops.linear_state(c[:, :n], c[:, n:2 * n], c[:, 2 * n:], o, st[:, state_off + self.conv_floats:state_off + self.state_floats],
                         ctx, H=H, rep=H // self.G, dim=self.dim, vdim=self.vdim, unit_eps=self.unit_eps,
                         q_scale=float(self.dim) ** -0.5, a=D[:, nc + H:nc + 2 * H], A_log=w["A_log"], dt_bias=w["dt_bias"],
                         b=D[:, nc:nc + H], delta=True)
        ops.head_post(o, cat, dv=self.vdim, gate=D[:, nc + 2 * H:], gate_silu=True, w=w["norm"], eps=ctx.eps, span=self.vdim,
                      scale=out_scale)


class DecayedState:
    """Outer-product state with a fixed decay per head:  S <- decay_h S + k v^T,  o = S^T q,  q, k, v = silu of their
    projections; the heads' outputs are RMS-normed together, weighted, and gated by sigmoid(W_g n)."""

    def __init__(self, index: int, cfg: dict, width: int):
        self.index, self.W = index, width
        self.H, self.dim = int(cfg["heads"]), int(cfg["dim"])
        self.vdim = int(cfg.get("vdim", self.dim))
        decay = cfg["decay"]
        self.decay = [float(d) for d in decay] if isinstance(decay, (list, tuple)) else [float(decay)] * self.H
        if len(self.decay) != self.H:
            raise ValueError(f"layer {index}: {len(self.decay)} decays for {self.H} heads")
        self.n_qk, self.n_v = self.H * self.dim, self.H * self.vdim
        self.in_names, self.out_name = ["q", "k", "v", "g"], "o"
        self.n_in, self.n_out = 2 * self.n_qk + 2 * self.n_v, self.n_v
        self.kv_dim = 0
        self.state_floats = state_floats(self.H, self.dim, self.vdim)
        self.w: Dict[str, torch.Tensor] = {}
        self._decay_dev = None

    def in_rows(self, name: str) -> int:
        return {"q": self.n_qk, "k": self.n_qk, "v": self.n_v, "g": self.n_v}[name]

    def small(self):
        return [("norm", (self.n_v,))]

    def checkpoint_small(self):
        return {"norm": ["norm"]}

    def forward(self, ctx: StepCtx, D, cat, kv_layer: int, state_off: int, out_scale: float = 1.0):
        ops, T = ctx.ops, D.shape[0]
        n, nv = self.n_qk, self.n_v
        if self._decay_dev is None:       # first used by a prompt step, never inside a captured decode step
            import numpy as np
            self._decay_dev = ops.to_device(np.asarray(self.decay, dtype=np.float32), np.float32)
        o = ops.empty((T, nv))
        ops.linear_state(D[:, :n], D[:, n:2 * n], D[:, 2 * n:2 * n + nv], o,
                         ctx.pool.state[:, state_off:state_off + self.state_floats], ctx, H=self.H, rep=1, dim=self.dim,
                         vdim=self.vdim, act=True, decay_const=self._decay_dev)
        ops.head_post(o, cat, dv=self.vdim, gate=D[:, 2 * n + nv:], w=self.w["norm"], eps=ctx.eps, span=nv, scale=out_scale)


class ClampedGLU:
    """Gated feed-forward with clamps: g = min(W_gate n, limit), u = clamp(W_up n, -limit, limit),
    W_down (g sigmoid(alpha g) (u + 1))."""

    def __init__(self, index: int, cfg: dict, width: int, alpha: float = 1.702):
        self.index, self.W, self.alpha = index, width, alpha
        self.ff, self.limit = int(cfg["ff"]), float(cfg["limit"])
        self.in_names, self.out_name = ["gate", "up"], "down"
        self.n_in, self.n_out = 2 * self.ff, self.ff
        self.kv_dim = self.state_floats = 0
        self.w: Dict[str, torch.Tensor] = {}

    def in_rows(self, name: str) -> int:
        return self.ff

    def small(self):
        return []

    def checkpoint_small(self):
        return {}

    def forward(self, ctx: StepCtx, D, cat, kv_layer: int, state_off: int, out_scale: float = 1.0):
        ctx.ops.glu_clamp(D[:, :self.ff], D[:, self.ff:], self.limit, self.alpha, cat)


def _side_by_side(index: int, cfg: dict, width: int):
    """an attention (gate per head) and a gated delta rule reading the same input; their outputs are weighted"""
    return [("left.", SinkAttention(index, cfg["left"], width, gate="head"), float(cfg["left_scale"])),
            ("right.", GatedDeltaRule(index, cfg["right"], width), float(cfg["right_scale"]))]


FUSED_MIXERS = {"attention": lambda i, c, w: [("", SinkAttention(i, c, w, gate="element"), 1.0)],
                "lightning": lambda i, c, w: [("", DecayedState(i, c, w), 1.0)],
                "parallel": _side_by_side}
FUSED_FEEDFORWARDS = {"dense": ClampedGLU}


class SharedInputLayer:
    """n = rmsnorm(x) * w;  x <- x + sum_parts scale_part * part(n).  The parts' input projections are stacked into ONE
    weight (one product per layer gives every part its rows), their output projections are laid side by side into ONE
    weight whose input is the parts' outputs side by side — the sum over the parts and the residual add happen inside
    that product.  A part's scale is applied to its output before the product."""

    def __init__(self, index: int, cfg: dict, width: int):
        self.index, self.W = index, width
        if cfg["type"] not in FUSED_MIXERS:
            raise ValueError(f"layer {index}: unknown mixer type {cfg['type']!r} (have {sorted(FUSED_MIXERS)})")
        self.parts = [("mix." + p, part, s) for p, part, s in FUSED_MIXERS[cfg["type"]](index, cfg["mixer"], width)]
        f = cfg.get("mlp")
        if f is not None:
            if f.get("kind") not in FUSED_FEEDFORWARDS:
                raise ValueError(f"layer {index}: unknown feed-forward kind {f.get('kind')!r} (have {sorted(FUSED_FEEDFORWARDS)})")
            self.parts.append(("mlp.", FUSED_FEEDFORWARDS[f["kind"]](index, f, width), 1.0))
        self.n_in = sum(part.n_in for _, part, _ in self.parts)
        self.n_out = sum(part.n_out for _, part, _ in self.parts)
        self.kv_layers = sum(1 for _, part, _ in self.parts if part.kv_dim)
        self.kv_dim = max(part.kv_dim for _, part, _ in self.parts)
        self.state_floats = sum(part.state_floats for _, part, _ in self.parts)
        self.w: Dict[str, torch.Tensor] = {}

    def manifest(self, p: str):
        out = [(p + "norm1", (self.W,)), (p + "in", (self.n_in, self.W)), (p + "out", (self.W, self.n_out))]
        for pre, part, _ in self.parts:
            out += [(p + pre + n, shape) for n, shape in part.small()]
        return out

    def checkpoint_tensors(self, p: str):
        """checkpoint name -> shape of everything this layer reads"""
        out = {p + "norm1": (self.W,)}
        for pre, part, _ in self.parts:
            for n in part.in_names:
                out[p + pre + n] = (part.in_rows(n), self.W)
            out[p + pre + part.out_name] = (self.W, part.n_out)
            shapes = dict(part.small())
            for packed, names in part.checkpoint_small().items():
                if len(names) == 1:
                    out[p + pre + names[0]] = shapes[packed]
                else:       # the convolutions of q, k, v stacked: rows split like the projections'
                    for n in names:
                        out[p + pre + n] = (part.in_rows(n.split(".")[0]), shapes[packed][1])
        return out

    def pack(self, p: str, ck, view):
        view(p + "norm1").copy_(ck[p + "norm1"])
        w_in, w_out = view(p + "in"), view(p + "out")
        r = c = 0
        for pre, part, _ in self.parts:
            for n in part.in_names:
                t = ck[p + pre + n]
                w_in[r:r + t.shape[0]].copy_(t)
                r += t.shape[0]
            w_out[:, c:c + part.n_out].copy_(ck[p + pre + part.out_name])
            c += part.n_out
            for packed, names in part.checkpoint_small().items():
                dst, at = view(p + pre + packed), 0
                for n in names:
                    t = ck[p + pre + n]
                    dst[at:at + t.shape[0]].copy_(t)
                    at += t.shape[0]
        self.bind(p, view)

    def bind(self, p: str, view):
        self.w = {n: view(p + n) for n in ("norm1", "in", "out")}
        for pre, part, _ in self.parts:
            part.w = {n: view(p + pre + n) for n, _ in part.small()}

    def forward(self, ctx: StepCtx, x: torch.Tensor, kv_base: int = 0, state_base: int = 0):
        """kv_base: the pool's caching layer of this RUN's first attention; state_base: its offset in the slot's state"""
        ops, T = ctx.ops, x.shape[0]
        n = ops.empty((T, self.W))
        ops.norm_rows(x, self.w["norm1"], ctx.eps, n)
        D = ops.linear(n, self.w["in"])
        cat = ops.empty((T, self.n_out))
        a = c = 0
        for _, part, scale in self.parts:
            part.forward(ctx, D[:, a:a + part.n_in], cat[:, c:c + part.n_out], kv_base, state_base, scale)
            a, c = a + part.n_in, c + part.n_out
            kv_base += 1 if part.kv_dim else 0
            state_base += part.state_floats
        ops.linear(cat, self.w["out"], out=x, add=True)


# ----------------------------------------------------------------------------------------------------------------
# Pre-norm layers with a scale vector on each branch.  A mixer of such a layer has `forward(ctx, n) -> rows (T, width)`,
# `kv_dim` (numbers it caches per token; the model sets `cache_index`) and `state_floats` (fp32 numbers it keeps per
# slot; the model sets `state_off`); a feed-forward has `forward(ctx, n) -> keyword arguments of ops.residual_rows`.
class StateSpaceMixer:
    """Mamba-2 style state-space mixer (Dao and Gu, "Transformers are SSMs").  inner = heads * vdim, N = state, G = groups.
    W_in n = [z: inner | x: inner | B: G N | C: G N | dt: heads]; x, B, C pass a causal convolution per channel (`conv`
    taps, with bias; the slot keeps the last taps - 1 inputs) and silu; dt <- softplus(dt + dt_bias); per head h (group
    h // (heads / G)):  S <- exp(-exp(A_log_h) dt) S + dt B x^T  (S: N x vdim, fp32 in the slot, zero at position 0),
    y = S^T C + D_h x;  y <- y * silu(z), RMS-normed in `norm_groups` equal parts, times `norm`; then W_o."""

    def __init__(self, index: int, cfg: dict, width: int):
        self.index, self.W = index, width
        self.H, self.vdim, self.N = int(cfg["heads"]), int(cfg["vdim"]), int(cfg["state"])
        self.G, self.NG, self.taps = int(cfg.get("groups", 1)), int(cfg.get("norm_groups", 1)), int(cfg.get("conv") or 1)
        self.inner = self.H * self.vdim
        if self.H % self.G or self.inner % self.NG:
            raise ValueError(f"layer {index}: {self.H} heads in {self.G} groups, {self.inner} numbers in {self.NG} norm groups")
        self.n_conv = self.inner + 2 * self.G * self.N
        self.n_in = 2 * self.inner + 2 * self.G * self.N + self.H
        self.kv_dim = 0
        self.conv_floats = max(self.taps - 1, 0) * self.n_conv
        self.state_floats = self.conv_floats + state_floats(self.H, self.N, self.vdim)
        self.cache_index, self.state_off = -1, 0
        self.w: Dict[str, torch.Tensor] = {}

    def manifest(self, p: str):
        return [(p + "in", (self.n_in, self.W)), (p + "conv", (self.n_conv, self.taps)), (p + "conv.b", (self.n_conv,)),
                (p + "dt_bias", (self.H,)), (p + "A_log", (self.H,)), (p + "D", (self.H,)), (p + "norm", (self.inner,)),
                (p + "o", (self.W, self.inner))]

    def checkpoint_tensors(self, p: str) -> Dict[str, tuple]:
        return dict(self.manifest(p))        # the packed layout is the checkpoint's

    def pack(self, p: str, ck, view):
        for n, _ in self.manifest(p):
            view(n).copy_(ck[n])
        self.bind(p, view)

    def bind(self, p: str, view):
        self.w = {n[len(p):]: view(n) for n, _ in self.manifest(p)}

    def forward(self, ctx: StepCtx, x: torch.Tensor) -> torch.Tensor:
        ops, w, T = ctx.ops, self.w, x.shape[0]
        inner, gn, nc = self.inner, self.G * self.N, self.n_conv
        D = ops.linear(x, w["in"])
        st, off = ctx.pool.state, self.state_off
        c = ops.short_conv(D[:, inner:inner + nc], w["conv"], st[:, off:off + self.conv_floats], ctx, act=True,
                           bias=w["conv.b"])
        y = ops.empty((T, inner))
        ops.linear_state(c[:, inner + gn:], c[:, inner:inner + gn], c[:, :inner], y,
                         st[:, off + self.conv_floats:off + self.state_floats], ctx, H=self.H, rep=self.H // self.G,
                         dim=self.N, vdim=self.vdim, a=D[:, inner + nc:], A_log=w["A_log"], dt_bias=w["dt_bias"],
                         dt_in=True, skip=w["D"])
        ops.head_post(y, y, dv=self.vdim, gate=D[:, :inner], gate_silu=True, w=w["norm"], eps=ctx.eps,
                      span=inner // self.NG, gate_first=True)
        return ops.linear(y, w["o"])


class GatedDense:
    """Gated feed-forward W_down (g sigmoid(alpha g) (u + offset)), g = min(W_gate n, limit), u = clamp(W_up n, +-limit);
    without a limit, alpha = 1 and offset = 0 it is the silu-gated unit W_down (silu(W_gate n) * W_up n).  Gate and up
    are one stacked product.  act = "gelu_tanh": the gate passes the tanh form of gelu instead,
    g sigmoid(2 sqrt(2 / pi) (g + 0.044715 g^3)) = 0.5 g (1 + tanh(sqrt(2 / pi) (g + 0.044715 g^3)))."""

    def __init__(self, index: int, cfg: dict, width: int, clamped: bool = False, alpha: float = 1.702, act: str = "silu"):
        self.index, self.W, self.ff = index, width, int(cfg["ff"])
        self.limit = float(cfg["limit"]) if clamped else float("inf")
        self.alpha, self.offset = (alpha, 1.0) if clamped else (1.0, 0.0)
        if act not in ("silu", "gelu_tanh"):
            raise ValueError(f"layer {index}: activation {act!r} (have 'silu', 'gelu_tanh')")
        self.cubic = 0.0
        if act == "gelu_tanh":
            self.alpha, self.cubic = GELU_TANH_ALPHA, GELU_TANH_CUBIC
        self.w: Dict[str, torch.Tensor] = {}

    def manifest(self, p: str):
        return [(p + "gu", (2 * self.ff, self.W)), (p + "down", (self.W, self.ff))]

    def checkpoint_tensors(self, p: str) -> Dict[str, tuple]:
        return {p + "gate": (self.ff, self.W), p + "up": (self.ff, self.W), p + "down": (self.W, self.ff)}

    def pack(self, p: str, ck, view):
        gu = view(p + "gu")
        gu[:self.ff].copy_(ck[p + "gate"])
        gu[self.ff:].copy_(ck[p + "up"])
        view(p + "down").copy_(ck[p + "down"])
        self.bind(p, view)

    def bind(self, p: str, view):
        self.w = {n[len(p):]: view(n) for n, _ in self.manifest(p)}

    def rows(self, ctx: StepCtx, x: torch.Tensor) -> torch.Tensor:
        ops = ctx.ops
        D = ops.linear(x, self.w["gu"])
        down = self.w["down"]
        if ops.tc_ok(x.shape[0], self.ff, down.stride(0)) and down.data_ptr() % 16 == 0:
            try:          # a prompt: the activation is written as the bf16 operand of the down product, in one pass
                hb = ops.glu_clamp_bf16(D[:, :self.ff], D[:, self.ff:], self.limit, self.alpha, up_offset=self.offset,
                                        cubic=self.cubic)
                y = ops.empty((x.shape[0], self.W))
                ops.tc_gemm(hb, down, y, N_=self.W, K=self.ff, ldw=down.stride(0))
                return y
            except _B200Error as e:
                ops.tc_refused(e)
        hid = ops.empty((x.shape[0], self.ff))
        ops.glu_clamp(D[:, :self.ff], D[:, self.ff:], self.limit, self.alpha, hid, up_offset=self.offset, cubic=self.cubic)
        return ops.linear(hid, down)

    def forward(self, ctx: StepCtx, x: torch.Tensor) -> dict:
        return {"y": self.rows(ctx, x)}


class GroupedExpertMixture:
    """`experts` clamped gated feed-forwards (GatedDense with a limit) of which a token uses `top`.  Scores
    s = sigmoid(W_router n) in fp32; the choice is made on s + `correction` among the experts of the `groups.keep` best
    of `groups.count` equal groups of neighbours (a group's score: the sum of its two largest s + correction); the
    weights are the chosen s over their sum.  `shared`: one more such unit that every token uses, times
    sigmoid(W_sg n) (one number per token); its gate row rides at the end of the router's matrix."""

    def __init__(self, index: int, cfg: dict, width: int, alpha: float = 1.702):
        self.index, self.W, self.alpha = index, width, alpha
        r = cfg["router"]
        self.E, self.top, self.ff, self.limit = int(r["experts"]), int(r["top"]), int(cfg["expert"]["ff"]), float(cfg["expert"]["limit"])
        g = r.get("groups") or {}
        self.n_groups, self.keep = int(g.get("count", 1)), int(g.get("keep", g.get("count", 1)))
        if self.E % self.n_groups or not 1 <= self.keep <= self.n_groups or self.top > self.keep * (self.E // self.n_groups):
            raise ValueError(f"layer {index}: {self.E} experts in {self.n_groups} groups, {self.keep} kept, {self.top} chosen")
        self.shared = GatedDense(index, cfg["shared"], width, clamped=True, alpha=alpha) if cfg.get("shared") else None
        self.w: Dict[str, torch.Tensor] = {}

    def manifest(self, p: str):
        out = [(p + "router", (self.E + (1 if self.shared else 0), self.W)), (p + "correction", (self.E,)),
               (p + "gu", (self.E, 2 * self.ff, self.W)), (p + "down", (self.E, self.W, self.ff))]
        return out + (self.shared.manifest(p + "shared.") if self.shared else [])

    def checkpoint_tensors(self, p: str) -> Dict[str, tuple]:
        out = {p + "router": (self.E, self.W), p + "correction": (self.E,)}
        for e in range(self.E):
            out.update({p + f"e{e}.gate": (self.ff, self.W), p + f"e{e}.up": (self.ff, self.W), p + f"e{e}.down": (self.W, self.ff)})
        if self.shared:
            out.update(self.shared.checkpoint_tensors(p + "shared."))
            out[p + "shared.sg"] = (1, self.W)
        return out

    def pack(self, p: str, ck, view):
        router = view(p + "router")
        router[:self.E].copy_(ck[p + "router"])
        view(p + "correction").copy_(ck[p + "correction"])
        gu, down = view(p + "gu"), view(p + "down")
        for e in range(self.E):
            gu[e, :self.ff].copy_(ck[p + f"e{e}.gate"])
            gu[e, self.ff:].copy_(ck[p + f"e{e}.up"])
            down[e].copy_(ck[p + f"e{e}.down"])
        if self.shared:
            router[self.E:].copy_(ck[p + "shared.sg"])
            self.shared.pack(p + "shared.", ck, view)
        self.bind(p, view)

    def bind(self, p: str, view):
        self.w = {n: view(p + n) for n in ("router", "correction", "gu", "down")}
        if self.shared:
            self.shared.bind(p + "shared.", view)

    def forward(self, ctx: StepCtx, x: torch.Tensor) -> dict:
        ops, w, T, ff = ctx.ops, self.w, x.shape[0], self.ff
        z = ops.linear(x, w["router"], exact_x=True)      # scores decide the choice: fp32 input rows in every mode
        idx, wgt = ops.router_group_topk(z, self.top, w["correction"], self.n_groups, self.keep, E=self.E)
        lists, count = ops.moe_group(idx, self.E)
        out = None
        if ops.tc_ok(T, self.W, ff):
            try:
                out = self._experts_prompt(ops, x, lists, count)
            except _B200Error as e:
                ops.tc_refused(e)
        if out is None:
            n_act = min(self.E, T * self.top)
            hid = ops.empty((T * self.top, 2 * ff))
            ops.gemm(x, w["gu"], hid, M=T, N_=2 * ff, K=self.W, wb=2 * ff * self.W, batch=self.E, lists=lists, count=count,
                     x_div=self.top, compact=n_act)
            act = ops.empty((T * self.top, ff))
            ops.glu_clamp(hid[:, :ff], hid[:, ff:], self.limit, self.alpha, act)
            out = ops.empty((T * self.top, self.W))
            ops.gemm(act, w["down"], out, M=T, N_=self.W, K=ff, wb=self.W * ff, batch=self.E, lists=lists, count=count,
                     x_div=1, compact=n_act)
        res = {"y": out, "combine": wgt, "top": self.top}
        if self.shared:
            res.update(shared=self.shared.rows(ctx, x), shared_gate=z[:, self.E:])
        return res

    def _experts_prompt(self, ops: LayerOps, x, lists, count):
        """A prompt step on the tensor cores (see ExpertMixture._experts_prompt): entries sorted by expert into
        segments of whole token tiles, ONE grouped tcgen05 launch per projection — gate and up are one stacked
        product —, the clamped activation between them."""
        w, T, ff = self.w, x.shape[0], self.ff
        n_all = T * self.top
        order, group = ops.moe_tiles(lists, count, n_all)
        n_rows = order.shape[0]
        xs = ops.to_bf16(x, self.W, rows=n_rows, row_map=order, div=self.top)
        hs = ops.empty((n_rows, 2 * ff))
        ops.tc_gemm_grouped(xs, w["gu"], hs, group, N_=2 * ff, K=self.W, n_groups=self.E)
        act = ops.glu_clamp_bf16(hs[:, :ff], hs[:, ff:], self.limit, self.alpha, live=order)   # activation and rounding in one pass
        ys = ops.empty((n_rows, self.W))
        ops.tc_gemm_grouped(act, w["down"], ys, group, N_=self.W, K=ff, n_groups=self.E)
        out = ops.empty((n_all, self.W))
        ops.rows_scatter(ys, order, out, n_rows)
        return out


SCALED_MIXERS = {"latent_attention": lambda i, c, w: LatentAttention(i, c, w, rotation="pairs", gated=True),
                 "mamba2": StateSpaceMixer}
SCALED_FEEDFORWARDS = {"dense": GatedDense, "moe": GroupedExpertMixture}


class ScaledPreNormLayer:
    """x <- x + s1 * mixer(LN1(x));  x <- x + s2 * ff(LN2(x)),  LN(y) = (y - mean) / sqrt(var + eps) * w without bias,
    s1, s2 vectors of the layer (`ls1`, `ls2`).  The residual stream and both updates are fp32."""

    def __init__(self, index: int, cfg: dict, width: int):
        self.index, self.W = index, width
        if cfg["type"] not in SCALED_MIXERS:
            raise ValueError(f"layer {index}: unknown mixer type {cfg['type']!r} (have {sorted(SCALED_MIXERS)})")
        self.mixer = SCALED_MIXERS[cfg["type"]](index, cfg["mixer"], width)
        f = cfg.get("mlp")
        if f is not None and f.get("kind") not in SCALED_FEEDFORWARDS:
            raise ValueError(f"layer {index}: unknown feed-forward kind {f.get('kind')!r} (have {sorted(SCALED_FEEDFORWARDS)})")
        self.ff = None if f is None else SCALED_FEEDFORWARDS[f["kind"]](index, f, width)
        self.kv_dim, self.state_floats = self.mixer.kv_dim, self.mixer.state_floats
        self.w: Dict[str, torch.Tensor] = {}

    def _own(self):
        return ["norm1", "ls1"] + (["norm2", "ls2"] if self.ff is not None else [])

    def manifest(self, p: str):
        out = [(p + n, (self.W,)) for n in self._own()] + self.mixer.manifest(p + "mix.")
        return out + (self.ff.manifest(p + "mlp.") if self.ff is not None else [])

    def checkpoint_tensors(self, p: str) -> Dict[str, tuple]:
        out = {p + n: (self.W,) for n in self._own()}
        out.update(self.mixer.checkpoint_tensors(p + "mix."))
        if self.ff is not None:
            out.update(self.ff.checkpoint_tensors(p + "mlp."))
        return out

    def pack(self, p: str, ck, view):
        for n in self._own():
            view(p + n).copy_(ck[p + n])
        self.mixer.pack(p + "mix.", ck, view)
        if self.ff is not None:
            self.ff.pack(p + "mlp.", ck, view)
        self.bind(p, view)

    def bind(self, p: str, view):
        self.w = {n: view(p + n) for n in self._own()}
        self.mixer.bind(p + "mix.", view)
        if self.ff is not None:
            self.ff.bind(p + "mlp.", view)

    def forward(self, ctx: StepCtx, x: torch.Tensor, normed: Optional[torch.Tensor] = None,
                next_norm: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
        """normed: LN1(x) if the layer before already made it; next_norm: the weight of the norm that follows this layer
        — then the layer's last residual update also norms the updated rows, and the result is returned"""
        ops = ctx.ops
        n = normed
        if n is None:
            n = ops.empty(tuple(x.shape))
            ops.norm_rows(x, self.w["norm1"], ctx.eps, n, center=True)
        y = self.mixer.forward(ctx, n)
        if self.ff is None:
            return self._close(ctx, x, self.w["ls1"], {"y": y}, next_norm)
        n2 = self._close(ctx, x, self.w["ls1"], {"y": y}, self.w["norm2"])
        return self._close(ctx, x, self.w["ls2"], self.ff.forward(ctx, n2), next_norm)

    def _close(self, ctx: StepCtx, x, ls, branch: dict, norm_w):
        """x += ls * branch; with a norm weight: also the norm of the updated rows (one launch), returned"""
        if norm_w is None:
            ctx.ops.residual_rows(x=x, ls=ls, **branch)
            return None
        n = ctx.ops.empty(tuple(x.shape))
        ctx.ops.residual_norm_rows(x=x, ls=ls, w=norm_w, eps=ctx.eps, out=n, center=True, **branch)
        return n


# ----------------------------------------------------------------------------------------------------------------
# Pre-norm layers with an RMS norm in groups, one multiplier on both branches and a causal convolution on the mixer's
# input.  A mixer has `forward(ctx, h) -> rows (T, width)`, `kv_dim` / `cache_index` and `state_floats` / `state_off` like
# the mixers of a ScaledPreNormLayer; a feed-forward has `forward(ctx, n) -> keyword arguments of ops.residual_rows`.
class GroupedAttention:
    """Softmax attention with `heads` query heads over `kv_heads` key/value heads (query head h reads key/value head
    h // (heads / kv_heads)), q, k, v one stacked product of the mixer's input.  Optional, each by a parameter:
      qk_norm     q and k are RMS-normed over their WHOLE projection (all heads at once) and weighted (`q.norm`, `k.norm`)
      rot         rotate-half rotary on the first `rot.dims` numbers of every head, YaRN-scaled by `rot.scaling`
      v_unit      every value head is divided by its root mean square; the cache holds it so
      sink        "learned": a logit per head (`sink`) joins the softmax's denominator without a key or a value;
                  "unit": the denominator holds one more 1 (a sink logit of zero)
      q_temp      queries times 1 + coef ln(floor((p + 1) / every) + 1) at position p
      bias_exp    slope_h (i - j) is taken off the score of query i and key j, slope_h = 2^(-bias_exp (h + 1) / heads)
      mask.size   query i sees the keys j with 0 <= i - j < size (absent: every j <= i)
      v_mix       the model marks the first mixing layer (`v_role = "first"`: its cached values are also kept for the
                  step) and the later ones (`"blend"`: v <- (1 - lam) v + lam v_first, lam = `vmix`, after the value norm)."""

    def __init__(self, index: int, cfg: dict, width: int, qk_norm: bool = False, v_unit: bool = False,
                 sink: Optional[str] = None, bias_exp: float = 0.0):
        self.index, self.W = index, width
        self.H, self.dim = int(cfg["heads"]), int(cfg["dim"])
        self.G, self.vdim = int(cfg.get("kv_heads", self.H)), int(cfg.get("vdim", self.dim))
        if self.H % self.G:
            raise ValueError(f"layer {index}: {self.H} query heads do not divide over {self.G} key/value heads")
        self.scale = float(cfg.get("scale", float(self.dim) ** -0.5))
        rot = cfg.get("rot") or {}
        self.rot_base, self.rot_dims = float(rot.get("base", 10000.0)), int(rot.get("dims", 0))
        sc = rot.get("scaling")
        self.rot_scaling = None if not sc else (float(sc["factor"]), float(sc["original"]), float(sc["fast"]), float(sc["slow"]))
        if self.rot_dims % 2 or self.rot_dims > self.dim:
            raise ValueError(f"layer {index}: {self.rot_dims} rotated numbers in heads of {self.dim}")
        self.window = int((cfg.get("mask") or {}).get("size", 0))
        qt = cfg.get("q_temp")
        self.q_temp = None if not qt else (float(qt["coef"]), int(qt["every"]))
        if sink not in (None, "learned", "unit"):
            raise ValueError(f"layer {index}: sink {sink!r} (have None, 'learned', 'unit')")
        self.qk_norm, self.v_unit, self.sink, self.bias_exp = bool(qk_norm), bool(v_unit), sink, float(bias_exp)
        self.v_mix = bool(cfg.get("v_mix"))
        self.v_role: Optional[str] = None      # set by the model: "first" / "blend"
        self.n_q, self.n_k, self.n_v = self.H * self.dim, self.G * self.dim, self.G * self.vdim
        self.kv_dim, self.state_floats = self.n_k + self.n_v, 0
        self.cache_index, self.state_off = -1, 0
        self.w: Dict[str, torch.Tensor] = {}

    def manifest(self, p: str):
        out = [(p + "qkv", (self.n_q + self.n_k + self.n_v, self.W)), (p + "o", (self.W, self.H * self.vdim))]
        if self.qk_norm:
            out += [(p + "q.norm", (self.n_q,)), (p + "k.norm", (self.n_k,))]
        if self.sink == "learned":
            out.append((p + "sink", (self.H,)))
        if self.v_mix:
            out.append((p + "vmix", (1,)))
        return out

    def checkpoint_tensors(self, p: str) -> Dict[str, tuple]:
        out = {p + "q": (self.n_q, self.W), p + "k": (self.n_k, self.W), p + "v": (self.n_v, self.W),
               p + "o": (self.W, self.H * self.vdim)}
        if self.qk_norm:
            out.update({p + "q.norm": (self.n_q,), p + "k.norm": (self.n_k,)})
        if self.sink == "learned":
            out[p + "sink"] = (self.H,)
        if self.v_mix:
            out[p + "vmix"] = ()
        return out

    def pack(self, p: str, ck, view):
        qkv = view(p + "qkv")
        qkv[:self.n_q].copy_(ck[p + "q"])
        qkv[self.n_q:self.n_q + self.n_k].copy_(ck[p + "k"])
        qkv[self.n_q + self.n_k:].copy_(ck[p + "v"])
        for n, shape in self.manifest(p)[1:]:
            view(n).copy_(ck[n].reshape(shape))
        self.bind(p, view)

    def bind(self, p: str, view):
        self.w = {n[len(p):]: view(n) for n, _ in self.manifest(p)}

    def forward(self, ctx: StepCtx, h: torch.Tensor) -> torch.Tensor:
        ops, w, T = ctx.ops, self.w, h.shape[0]
        nq, nk, nv = self.n_q, self.n_k, self.n_v
        D = ops.linear(h, w["qkv"])
        q, k, v = D[:, :nq], D[:, nq:nq + nk], D[:, nq + nk:]
        rows = ctx.pool.buf[self.cache_index][..., :self.kv_dim]
        v_first = keep = None
        if self.v_role == "first":
            keep = ctx.carry["v_first"] = ops.empty((T, nv))
        elif self.v_role == "blend":
            v_first = ctx.carry["v_first"]
        ops.qkv_post(q, k, v, rows, ctx.slot, ctx.pos, ctx.rope(self.rot_base, self.rot_dims, self.rot_scaling), self.H, self.G,
                     self.dim, self.vdim, self.rot_dims, q_norm=w.get("q.norm"), k_norm=w.get("k.norm"), eps=ctx.eps,
                     v_unit=self.v_unit, q_temp=self.q_temp, vmix=w["vmix"] if v_first is not None else None,
                     v_first=v_first, v_keep=keep)
        o = ops.empty((T, self.H * self.vdim))
        segs = ctx.segments or []
        done = False
        if rows.dtype == torch.bfloat16 and any(self._tc_portion(ops, n, rows) for _, n, _, _ in segs):
            try:
                for start, n, slot, p0 in segs:      # long portions on the tensor cores, the rest on the row kernel
                    sl = slice(start, start + n)
                    if self._tc_portion(ops, n, rows):
                        self._attend_prompt(ctx, q[sl], rows, slot, ctx.pos[sl], o[sl], p0, n)
                    else:
                        self._attend_rows(ctx, q[sl], rows, ctx.slot[sl], ctx.pos[sl], o[sl], prompt=True)
                done = True
            except _B200Error as e:
                ops.tc_refused(e)
        if not done:
            self._attend_rows(ctx, q, rows, ctx.slot, ctx.pos, o, prompt=ctx.segments is not None)
        return ops.linear(o, w["o"])

    def _tc_portion(self, ops: LayerOps, n: int, rows) -> bool:
        return ops.tc_ok(n, self.dim, rows.stride(1)) and rows.stride(0) % 8 == 0

    def _attend_rows(self, ctx: StepCtx, q, rows, slot, pos, o, prompt: bool):
        """the row kernel: every query finds its keys by (slot, position); a step of few tokens (decoding) spreads the
        keys of a query over several blocks"""
        ctx.ops.sink_attention(q, rows, slot, pos, o, self.w.get("sink"), self.H, self.G, self.dim, self.vdim, self.scale,
                               window=self.window, n_split=1 if prompt and q.shape[0] > 16 else None,
                               bias_exp=self.bias_exp, unit_sink=self.sink == "unit")

    def _attend_prompt(self, ctx: StepCtx, q, all_rows, slot_index: int, pos, o, p0: int, n: int):
        """A portion of a prompt (positions p0 .. p0 + n - 1 of one slot) as two tcgen05 products per key/value head:
        the head's cached key columns are the weight-major operand of the scores of the query heads that share it, an
        fp32 softmax over the visible keys (distance bias and sink included) writes every probability as two bf16 parts
        (the second the rounding error of the first, so the weights keep 16 mantissa bits), and the head's value
        columns, transposed, are the operand of the weighted sum over both parts.  Queries are taken in chunks that bound the
        score buffer; with a window a chunk is about a window long and meets only the keys from its first query's
        first visible key on."""
        ops, H, G, d, dv = ctx.ops, self.H, self.G, self.dim, self.vdim
        rep, rows = H // G, all_rows[slot_index]
        sink = self.w.get("sink")
        step = n
        if self.window:
            step = max(128, min(self.window, (1 << 27) // (rep * 2 * self.window)))
            step = -(-n // -(-n // step))          # equal chunks: no short one at the end
        for a in range(0, n, step):
            m = min(step, n - a)
            key0 = max(p0 + a - self.window + 1, 0) if self.window else 0
            S = p0 + a + m - key0
            Sp = (S + 63) // 64 * 64
            sub = max(1, min(m, (1 << 27) // (rep * Sp)))
            for g in range(G):
                keys = rows[key0:key0 + S, g * d:(g + 1) * d]
                vt = ops.cache_transpose(rows[key0:, G * d + g * dv:], S, Sp, dv)
                for b in range(a, a + m, sub):
                    mm = min(sub, a + m - b)
                    qb16 = ops.heads_to_bf16(q[b:b + mm, g * rep * d:], rep, d)
                    sc = ops.empty((mm * rep, S))
                    ops.tc_gemm(qb16, keys, sc, N_=S, K=d, ldw=rows.stride(0))
                    P = ops.empty((mm * rep, 2 * Sp), torch.bfloat16)
                    ops.sink_softmax_bf16(sc, pos[b:b + mm], rep, None if sink is None else sink[g * rep:], self.scale, 0,
                                          self.window, key0, P, bias_exp=self.bias_exp, head0=g * rep, H=H,
                                          unit_sink=self.sink == "unit", split=True)
                    og = ops.empty((mm * rep, dv))
                    ops.tc_gemm(P, vt, og, N_=dv, K=Sp, parts=2)
                    ops.head_post(og.view(mm, rep * dv), o[b:b + mm, g * rep * dv:(g + 1) * rep * dv], dv=dv)


class TokenShiftState:
    """Time mixing with a token shift and a matrix state per head (the RWKV family's form).  With h' the input of the
    token before (zeros for a sequence's first token; the slot keeps the last one), each of r, k, v, g, w reads its own
    mix h + (h' - h) mu_s.  r, k, v = W_r, W_k, W_v of their mixes (`heads` x `dim`), gate = silu(W_g mix_g), and the
    decay per head and key channel  w = exp(-exp(W_w2 tanh(W_w1 mix_w) + w0)).  Per head, with S (dim, dim) fp32 in the slot,
    zero at position 0:  o = (S + diag(u) k v^T)^T r  (the bonus u counts for the current token only),  then
    S <- diag(w) S + k v^T.  Every head's o is divided by its root mean square, the heads side by side are multiplied by
    `norm` and the gate, then W_o."""
    MIXES = ("r", "k", "v", "g", "w")
    PART_LEN = 256        # a prompt's sequences are walked in parts of this many tokens at the same time

    def __init__(self, index: int, cfg: dict, width: int):
        self.index, self.W = index, width
        self.H, self.dim = int(cfg["heads"]), int(cfg["dim"])
        self.n = self.H * self.dim
        self.rank = int(cfg.get("decay_rank", 0))      # 0: taken from the checkpoint's `w1` when the weights are packed
        self.kv_dim = 0
        self.cache_index, self.state_off = -1, 0
        self.w: Dict[str, torch.Tensor] = {}

    @property
    def state_floats(self) -> int:
        return self.W + state_floats(self.H, self.dim, self.dim)

    def set_rank(self, rank: int):
        self.rank = int(rank)

    def manifest(self, p: str):
        return [(p + "mu", (len(self.MIXES), self.W)), (p + "rkvg", (4, self.n, self.W)), (p + "w1", (self.rank, self.W)),
                (p + "w2", (self.n, self.rank)), (p + "w0", (self.n,)), (p + "u", (self.H, self.dim)), (p + "norm", (self.n,)),
                (p + "o", (self.W, self.n))]

    def checkpoint_tensors(self, p: str) -> Dict[str, tuple]:
        out = {p + "mu." + s: (self.W,) for s in self.MIXES}
        out.update({p + s: (self.n, self.W) for s in "rkvg"})
        out.update({p + "w1": (self.rank, self.W), p + "w2": (self.n, self.rank), p + "w0": (self.n,),
                    p + "u": (self.H, self.dim), p + "norm": (self.n,), p + "o": (self.W, self.n)})
        return out

    def pack(self, p: str, ck, view):
        mu, rkvg = view(p + "mu"), view(p + "rkvg")
        for i, s in enumerate(self.MIXES):
            mu[i].copy_(ck[p + "mu." + s])
        for i, s in enumerate("rkvg"):
            rkvg[i].copy_(ck[p + s])
        for n in ("w1", "w2", "w0", "u", "norm", "o"):
            view(p + n).copy_(ck[p + n])
        self.bind(p, view)

    def bind(self, p: str, view):
        self.w = {n[len(p):]: view(n) for n, _ in self.manifest(p)}

    def forward(self, ctx: StepCtx, h: torch.Tensor) -> torch.Tensor:
        ops, w, T, n, W = ctx.ops, self.w, h.shape[0], self.n, self.W
        st, off = ctx.pool.state, self.state_off
        D = ops.empty((T, 4 * n))                                          # r | k | v | gate
        logit = M = Mb = None
        if ops.tc_ok(T, W, self.rank) and n % 4 == 0 and w["rkvg"].data_ptr() % 16 == 0:
            # a prompt: the mixes are written as the bf16 operands of five tensor-core products; the tanh of the decay
            # projection is applied while its latent rows are rounded to the next operand
            try:
                Mb = ops.token_shift(h, w["mu"], st[:, off:off + W], ctx, operands=True)      # (5, T, ceil64(W)) bf16
                for i in range(4):
                    ops.tc_gemm(Mb[i], w["rkvg"][i], D[:, i * n:(i + 1) * n], N_=n, K=W)
                lat = ops.empty((T, self.rank))
                ops.tc_gemm(Mb[4], w["w1"], lat, N_=self.rank, K=W)
                logit = ops.empty((T, n))
                ops.tc_gemm(ops.to_bf16(lat, self.rank, act=ACT_TANH), w["w2"], logit, N_=n, K=self.rank, bias=w["w0"])
            except _B200Error as e:       # the slot's previous input is already replaced: the shift is not run again,
                ops.tc_refused(e)         # the row kernels read the rounded mixes
                logit = None
                if Mb is None:
                    raise
                with torch.cuda.stream(ops.stream):
                    M = Mb[..., :W].float()
        if logit is None:             # few rows: ONE launch over the four (input, weight) pairs
            if M is None:
                M = ops.token_shift(h, w["mu"], st[:, off:off + W], ctx)      # (5, T, W)
            ops.gemm(M, w["rkvg"], D, M=T, N_=n, K=W, ldx=W, xb=T * W, wb=n * W, ldy=4 * n, yb=n, batch=4)
            lat = ops.linear(M[4], w["w1"], epi=EPI_SOFTCAP, epi_param=1.0)    # tanh
            logit = ops.linear(lat, w["w2"], bias=w["w0"])
        o = ops.empty((T, n))
        ops.linear_state(D[:, :n], D[:, n:2 * n], D[:, 2 * n:3 * n], o, st[:, off + W:off + self.state_floats], ctx, H=self.H,
                         rep=1, dim=self.dim, vdim=self.dim, decay_logits=logit, bonus=w["u"], part_len=self.PART_LEN)
        ops.head_post(o, o, dv=self.dim, gate=D[:, 3 * n:], gate_silu=True, w=w["norm"], eps=ctx.eps, span=self.dim)
        return ops.linear(o, w["o"])


class UngatedDense:
    """W_down act(W_up n), act = the exact (erf) gelu."""

    def __init__(self, index: int, cfg: dict, width: int):
        self.index, self.W, self.ff = index, width, int(cfg["ff"])
        self.w: Dict[str, torch.Tensor] = {}

    def manifest(self, p: str):
        return [(p + "up", (self.ff, self.W)), (p + "down", (self.W, self.ff))]

    def checkpoint_tensors(self, p: str) -> Dict[str, tuple]:
        return dict(self.manifest(p))

    def pack(self, p: str, ck, view):
        for n, _ in self.manifest(p):
            view(n).copy_(ck[n])
        self.bind(p, view)

    def bind(self, p: str, view):
        self.w = {n[len(p):]: view(n) for n, _ in self.manifest(p)}

    def rows(self, ctx: StepCtx, x: torch.Tensor) -> torch.Tensor:
        ops, up, down = ctx.ops, self.w["up"], self.w["down"]
        if ops.tc_ok(x.shape[0], self.W, self.ff):
            try:          # a prompt: the activation is written as the bf16 operand of the down product, in one pass
                hid = ops.linear(x, up)
                y = ops.empty((x.shape[0], self.W))
                ops.tc_gemm(ops.to_bf16(hid, self.ff, act=ACT_GELU), down, y, N_=self.W, K=self.ff)
                return y
            except _B200Error as e:
                ops.tc_refused(e)
        return ops.linear(ops.linear(x, up, epi=EPI_GELU), down)

    def forward(self, ctx: StepCtx, x: torch.Tensor) -> dict:
        return {"y": self.rows(ctx, x)}


class UngatedExpertMixture:
    """`experts` ungated feed-forwards W_down gelu(W_up n) (exact gelu, no biases) of which a token uses `top`.  Scores
    s = softmax(W_router n) over all experts, in fp32; the experts form `groups.count` equal groups of neighbours, a
    group's score is its largest s, and only experts of the `groups.keep` best groups can be chosen; the `top` largest s
    among them are chosen and weighted by s over the sum of the chosen s (+ 1e-20).  `shared`: one more such
    feed-forward that every token uses, added with weight one."""

    def __init__(self, index: int, cfg: dict, width: int):
        self.index, self.W = index, width
        r = cfg["router"]
        self.E, self.top, self.ff = int(r["experts"]), int(r["top"]), int(cfg["expert"]["ff"])
        g = r.get("groups") or {}
        self.n_groups, self.keep = int(g.get("count", 1)), int(g.get("keep", g.get("count", 1)))
        if self.E % self.n_groups or not 1 <= self.keep <= self.n_groups or self.top > self.keep * (self.E // self.n_groups):
            raise ValueError(f"layer {index}: {self.E} experts in {self.n_groups} groups, {self.keep} kept, {self.top} chosen")
        self.shared = UngatedDense(index, cfg["shared"], width) if cfg.get("shared") else None
        self.w: Dict[str, torch.Tensor] = {}

    def manifest(self, p: str):
        out = [(p + "router", (self.E, self.W)), (p + "up", (self.E, self.ff, self.W)), (p + "down", (self.E, self.W, self.ff))]
        return out + (self.shared.manifest(p + "shared.") if self.shared else [])

    def checkpoint_tensors(self, p: str) -> Dict[str, tuple]:
        out = {p + "router": (self.E, self.W)}
        for e in range(self.E):
            out.update({p + f"e{e}.up": (self.ff, self.W), p + f"e{e}.down": (self.W, self.ff)})
        if self.shared:
            out.update(self.shared.checkpoint_tensors(p + "shared."))
        return out

    def pack(self, p: str, ck, view):
        view(p + "router").copy_(ck[p + "router"])
        up, down = view(p + "up"), view(p + "down")
        for e in range(self.E):
            up[e].copy_(ck[p + f"e{e}.up"])
            down[e].copy_(ck[p + f"e{e}.down"])
        if self.shared:
            self.shared.pack(p + "shared.", ck, view)
        self.bind(p, view)

    def bind(self, p: str, view):
        self.w = {n: view(p + n) for n in ("router", "up", "down")}
        if self.shared:
            self.shared.bind(p + "shared.", view)

    def forward(self, ctx: StepCtx, x: torch.Tensor) -> dict:
        ops, w, T, ff = ctx.ops, self.w, x.shape[0], self.ff
        z = ops.linear(x, w["router"], exact_x=True)      # scores decide the choice: fp32 input rows in every mode
        idx, wgt = ops.router_group_topk(z, self.top, None, self.n_groups, self.keep, E=self.E, softmax=True, group_max=True)
        lists, count = ops.moe_group(idx, self.E)
        out = None
        if ops.tc_ok(T, self.W, ff):
            try:
                out = self._experts_prompt(ops, x, lists, count)
            except _B200Error as e:
                ops.tc_refused(e)
        if out is None:
            n_act = min(self.E, T * self.top)
            hid = ops.empty((T * self.top, ff))
            ops.gemm(x, w["up"], hid, M=T, N_=ff, K=self.W, wb=ff * self.W, batch=self.E, lists=lists, count=count,
                     x_div=self.top, epi=EPI_GELU, compact=n_act)
            out = ops.empty((T * self.top, self.W))
            ops.gemm(hid, w["down"], out, M=T, N_=self.W, K=ff, wb=self.W * ff, batch=self.E, lists=lists, count=count,
                     x_div=1, compact=n_act)
        res = {"y": out, "combine": wgt, "top": self.top}
        if self.shared:
            res["shared"] = self.shared.rows(ctx, x)
        return res

    def _experts_prompt(self, ops: LayerOps, x, lists, count):
        """A prompt step on the tensor cores (see ExpertMixture._experts_prompt): entries sorted by expert into
        segments of whole token tiles, ONE grouped tcgen05 launch per projection, the gelu between them applied while
        the hidden rows are rounded to the next product's operand."""
        w, T, ff = self.w, x.shape[0], self.ff
        n_all = T * self.top
        order, group = ops.moe_tiles(lists, count, n_all)
        n_rows = order.shape[0]
        xs = ops.to_bf16(x, self.W, rows=n_rows, row_map=order, div=self.top)
        hs = ops.empty((n_rows, ff))
        ops.tc_gemm_grouped(xs, w["up"], hs, group, N_=ff, K=self.W, n_groups=self.E)
        hb = ops.to_bf16(hs, ff, act=ACT_GELU)
        ys = ops.empty((n_rows, self.W))
        ops.tc_gemm_grouped(hb, w["down"], ys, group, N_=self.W, K=ff, n_groups=self.E)
        out = ops.empty((n_all, self.W))
        ops.rows_scatter(ys, order, out, n_rows)
        return out


DISTANCE_BIAS_EXP = 8.0       # 'attention_2': head h of H takes 2^(-8 (h + 1) / H) per position of distance off its scores

CONV_MIXERS = {"attention": lambda i, c, w: GroupedAttention(i, c, w, qk_norm=True, v_unit=True, sink="learned"),
               "attention_2": lambda i, c, w: GroupedAttention(i, c, w, sink="unit", bias_exp=DISTANCE_BIAS_EXP),
               "wkv": TokenShiftState}
CONV_FEEDFORWARDS = {"dense": lambda i, c, w: GatedDense(i, c, w, act="gelu_tanh"), "moe": UngatedExpertMixture}


class ConvPreNormLayer:
    """h = N1(x);  h <- h + conv(h);  x <- x + m * mixer(h);  x <- x + m * ff(N2(x)).
    N: the row in `groups` equal consecutive parts, each divided by sqrt(mean(part^2) + eps), the whole times w.
    conv: a causal convolution over time per channel (`canon1`, (width, taps), no bias), conv(h)_t = sum_j c[:, j]
    h_(t - taps + 1 + j); the slot keeps the last taps - 1 rows of N1(x) of its sequence (taps 0: no convolution).
    The residual stream and both updates are fp32."""

    def __init__(self, index: int, cfg: dict, width: int, groups: int = 1, mult: float = 1.0, taps: int = 0):
        self.index, self.W, self.groups, self.mult, self.taps = index, width, int(groups), float(mult), int(taps)
        if width % self.groups:
            raise ValueError(f"layer {index}: rows of {width} numbers in {self.groups} norm groups")
        if cfg["type"] not in CONV_MIXERS:
            raise ValueError(f"layer {index}: unknown mixer type {cfg['type']!r} (have {sorted(CONV_MIXERS)})")
        self.mixer = CONV_MIXERS[cfg["type"]](index, cfg["mixer"], width)
        f = cfg.get("mlp")
        if f is not None and f.get("kind") not in CONV_FEEDFORWARDS:
            raise ValueError(f"layer {index}: unknown feed-forward kind {f.get('kind')!r} (have {sorted(CONV_FEEDFORWARDS)})")
        self.ff = None if f is None else CONV_FEEDFORWARDS[f["kind"]](index, f, width)
        self.kv_dim = self.mixer.kv_dim
        self.conv_floats = max(self.taps - 1, 0) * width
        self.state_off = 0            # set by the model: the layer's span of the slot's state = [conv rows | the mixer's]
        self.w: Dict[str, torch.Tensor] = {}

    @property
    def state_floats(self) -> int:
        return self.conv_floats + self.mixer.state_floats

    def _own(self):
        return [("norm1", (self.W,))] + ([("canon1", (self.W, self.taps))] if self.taps else []) + \
               ([("norm2", (self.W,))] if self.ff is not None else [])

    def manifest(self, p: str):
        out = [(p + n, shape) for n, shape in self._own()] + self.mixer.manifest(p + "mix.")
        return out + (self.ff.manifest(p + "mlp.") if self.ff is not None else [])

    def checkpoint_tensors(self, p: str) -> Dict[str, tuple]:
        out = {p + n: shape for n, shape in self._own()}
        out.update(self.mixer.checkpoint_tensors(p + "mix."))
        if self.ff is not None:
            out.update(self.ff.checkpoint_tensors(p + "mlp."))
        return out

    def pack(self, p: str, ck, view):
        for n, _ in self._own():
            view(p + n).copy_(ck[p + n])
        self.mixer.pack(p + "mix.", ck, view)
        if self.ff is not None:
            self.ff.pack(p + "mlp.", ck, view)
        self.bind(p, view)

    def bind(self, p: str, view):
        self.w = {n: view(p + n) for n, _ in self._own()}
        self.mixer.bind(p + "mix.", view)
        if self.ff is not None:
            self.ff.bind(p + "mlp.", view)

    def forward(self, ctx: StepCtx, x: torch.Tensor, normed: Optional[torch.Tensor] = None,
                next_norm: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
        """normed: N1(x) if the layer before already made it; next_norm: the weight of the norm that follows this layer
        — then the layer's last residual update also norms the updated rows, and the result is returned"""
        ops = ctx.ops
        n = normed
        if n is None:
            n = ops.empty(tuple(x.shape))
            ops.norm_rows(x, self.w["norm1"], ctx.eps, n, groups=self.groups)
        if self.taps:
            st = ctx.pool.state[:, self.state_off:self.state_off + self.conv_floats]
            n = ops.short_conv(n, self.w["canon1"], st, ctx, residual=True)
        y = self.mixer.forward(ctx, n)
        if self.ff is None:
            return self._close(ctx, x, {"y": y}, next_norm)
        n2 = self._close(ctx, x, {"y": y}, self.w["norm2"])
        return self._close(ctx, x, self.ff.forward(ctx, n2), next_norm)

    def _close(self, ctx: StepCtx, x, branch: dict, norm_w):
        """x += m * branch; with a norm weight: also the norm of the updated rows (one launch), returned"""
        if norm_w is None:
            ctx.ops.residual_rows(x=x, ls=None, mult=self.mult, **branch)
            return None
        n = ctx.ops.empty(tuple(x.shape))
        ctx.ops.residual_norm_rows(x=x, ls=None, w=norm_w, eps=ctx.eps, out=n, mult=self.mult, groups=self.groups, **branch)
        return n


def assign_cache_layers(layers: List[PostNormLayer]) -> int:
    """number the layers that cache rows of their own; a borrowing layer gets its source's number"""
    n = 0
    for L in layers:
        if L.mixer.own_kv:
            L.mixer.cache_index = n
            n += 1
    for L in layers:
        m = L.mixer
        if not m.own_kv:
            if not 0 <= m.kv_from < m.index:
                raise ValueError(f"layer {m.index} borrows the latent of layer {m.kv_from}, which does not run before it")
            src = layers[m.kv_from].mixer
            if not src.own_kv or (src.kv_rank, src.rot_dim, src.rot_base, src.rot_dims) != \
                    (m.kv_rank, m.rot_dim, m.rot_base, m.rot_dims):
                raise ValueError(f"layer {m.index} borrows the latent of layer {m.kv_from}, which does not fit")
            m.cache_index = src.cache_index
    return n
