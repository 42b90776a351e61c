"""ORACLE — TEST INFRASTRUCTURE ONLY. Not imported by the product path.

Plain, slow restatement of the Vadelix decoder, one function per mechanism, written from the design's equations
with torch on the CPU.  It shares no code with mlx_vlm_b200/: no cache, no state objects, no batching; every call
walks the whole sequence.

Notation: x (T, W) residual stream, m the residual multiplier of the model.  A layer is pre-norm:
    h = N1(x);  h <- h + conv(h);  x <- x + m * mixer(h);   x <- x + m * ff(N2(x)),
    N(y): y in `groups` equal consecutive parts, each divided by sqrt(mean(part^2) + eps), the whole times w,
    conv(h)_t = sum_j c[:, j] * h_(t - taps + 1 + j)     (per channel, zeros before the sequence).
Mixers:
  'attention'    grouped heads, RMS norm (with weights) over the whole query and the whole key projection, rotate-half
                 rotary on the first dims numbers of a head with YaRN-scaled frequencies, values divided by their root
                 mean square per head, causal softmax with a learned sink logit per head in the denominator;
  'attention_2'  grouped heads, no rotation, queries scaled by a temperature that grows with the logarithm of the
                 position, a distance bias slope_h * (i - j) taken off the scores, a sliding window, one added to the
                 softmax's denominator;
  both           optional value mixing: from the second layer that has it on, v <- (1 - lam) v + lam v_first with
                 v_first the values of the first such layer for the same token;
  'wkv'          token shift (every projection reads its own mix of the current and the previous input), a decay per
                 key channel made from the input, a bonus for the current token, a (dim, dim) state per head, RMS
                 norm per head, a silu gate.
Feed-forwards: W_down (gelu_tanh(W_gate h) * W_up h); or a mixture of ungated erf-gelu experts chosen by softmax
scores within the best groups of experts, weighted by the chosen scores over their sum, plus a shared expert.
Output: N with 'final.norm', then the head.

Weights: dict name -> tensor with the checkpoint's names ('embed', 'l<i>.norm1', 'l<i>.canon1', 'l<i>.mix.q', ...).
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

BIAS_EXP = 8.0          # slope of head h of H in 'attention_2': 2^(-BIAS_EXP (h + 1) / H)


# ------------------------------------------------------------------------------------------------ pieces
def group_norm(y: torch.Tensor, w: Optional[torch.Tensor], eps: float, groups: int = 1) -> torch.Tensor:
    T, n = y.shape
    p = y.reshape(T, groups, n // groups)
    p = p / torch.sqrt((p * p).mean(-1, keepdim=True) + eps)
    p = p.reshape(T, n)
    return p if w is None else p * w


def input_conv(h: torch.Tensor, c: torch.Tensor) -> torch.Tensor:
    """h (T, W), c (W, taps) -> h + conv(h)"""
    T, taps = h.shape[0], c.shape[1]
    out = h.clone()
    for t in range(T):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                out[t] += c[:, j] * h[s]
    return out


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def gelu_erf(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.erf(z / math.sqrt(2.0)))


def yarn_frequencies(base: float, dims: int, scaling: Optional[dict]):
    """-> (f (dims/2,) float64, amplitude of cos and sin)"""
    half = dims // 2
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=torch.float64)
    if not scaling:
        return f, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def index(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(index(float(scaling["fast"]))), 0)
    hi = min(math.ceil(index(float(scaling["slow"]))), dims - 1)
    ramp = torch.tensor([min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0) for i in range(half)], dtype=torch.float64)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_half(v: torch.Tensor, pos: torch.Tensor, rot: Optional[dict]) -> torch.Tensor:
    """v (T, heads, D): of the first `dims` numbers of a head, (i, i + dims/2) is a pair turned by pos * f_i"""
    if not rot or int(rot.get("dims", 0)) < 2:
        return v.clone()
    dims = int(rot["dims"])
    half = dims // 2
    f, amp = yarn_frequencies(float(rot["base"]), dims, rot.get("scaling"))
    a = pos.to(torch.float64)[:, None] * f[None, :]
    cos, sin = (torch.cos(a) * amp).to(v.dtype)[:, None, :], (torch.sin(a) * amp).to(v.dtype)[:, None, :]
    lo, hi = v[..., :half], v[..., half:dims]
    out = v.clone()
    out[..., :half] = lo * cos - hi * sin
    out[..., half:dims] = hi * cos + lo * sin
    return out


def mix_values(v: torch.Tensor, lam: Optional[torch.Tensor], shared: Optional[dict]) -> torch.Tensor:
    """value mixing across layers.  shared: the dict of one forward pass ({} at its start), or None when the layer has
    no mixing.  The first layer that mixes leaves its values there; the later ones blend with them."""
    if shared is None:
        return v
    if "v_first" not in shared:
        shared["v_first"] = v
        return v
    return (1.0 - lam) * v + lam * shared["v_first"]


def softmax_with_sink(s: torch.Tensor, visible: torch.Tensor, sink: torch.Tensor) -> torch.Tensor:
    """s (H, T, T) scores, visible (T, T) bool, sink (H,) logits that join the denominator -> weights (H, T, T)"""
    s = s.masked_fill(~visible[None], float("-inf"))
    m = torch.maximum(s.max(-1, keepdim=True).values, sink[:, None, None])
    e = torch.exp(s - m)
    return e / (e.sum(-1, keepdim=True) + torch.exp(sink[:, None, None] - m))


def attention(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, c: dict, pos: torch.Tensor, eps: float,
              shared: Optional[dict]) -> torch.Tensor:
    T = h.shape[0]
    H, G, d, dv = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
    q, k, v = h @ w[p + "q"].T, h @ w[p + "k"].T, h @ w[p + "v"].T
    q = group_norm(q, w[p + "q.norm"], eps)
    k = group_norm(k, w[p + "k.norm"], eps)
    q = rotate_half(q.view(T, H, d), pos, c.get("rot"))
    k = rotate_half(k.view(T, G, d), pos, c.get("rot"))
    v = group_norm(v.reshape(T * G, dv), None, eps).view(T, G * dv)
    v = mix_values(v, w.get(p + "vmix"), shared if c.get("v_mix") else None).view(T, G, dv)
    rep = H // G
    s = torch.einsum("thd,shd->hts", q, k.repeat_interleave(rep, dim=1)) * float(c["scale"])
    i = torch.arange(T)
    a = softmax_with_sink(s, i[:, None] >= i[None, :], w[p + "sink"].to(s.dtype))
    o = torch.einsum("hts,shd->thd", a, v.repeat_interleave(rep, dim=1))
    return o.reshape(T, H * dv) @ w[p + "o"].T


def attention_2(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, c: dict, pos: torch.Tensor, eps: float,
                shared: Optional[dict]) -> torch.Tensor:
    T = h.shape[0]
    H, G, d, dv = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
    q, k, v = h @ w[p + "q"].T, h @ w[p + "k"].T, h @ w[p + "v"].T
    qt = c.get("q_temp")
    if qt:
        temp = 1.0 + float(qt["coef"]) * torch.log(torch.floor((pos.to(torch.float64) + 1.0) / float(qt["every"])) + 1.0)
        q = q * temp.to(q.dtype)[:, None]
    v = mix_values(v, w.get(p + "vmix"), shared if c.get("v_mix") else None).view(T, G, dv)
    rep = H // G
    s = torch.einsum("thd,shd->hts", q.view(T, H, d), k.view(T, G, d).repeat_interleave(rep, dim=1)) * float(c["scale"])
    dist = (pos[:, None] - pos[None, :]).to(s.dtype)
    slope = torch.tensor([2.0 ** (-BIAS_EXP * (hh + 1) / H) for hh in range(H)], dtype=s.dtype)
    s = s - slope[:, None, None] * dist[None]
    visible = dist >= 0
    size = int((c.get("mask") or {}).get("size", 0))
    if size:
        visible &= dist < size
    a = softmax_with_sink(s, visible, torch.zeros(H, dtype=s.dtype))
    o = torch.einsum("hts,shd->thd", a, v.repeat_interleave(rep, dim=1))
    return o.reshape(T, H * dv) @ w[p + "o"].T


def wkv(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, c: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, d = c["heads"], c["dim"]
    prev = torch.cat([torch.zeros_like(h[:1]), h[:-1]], 0)

    def mixed(name):
        return h + (prev - h) * w[p + "mu." + name]

    r, k, v = mixed("r") @ w[p + "r"].T, mixed("k") @ w[p + "k"].T, mixed("v") @ w[p + "v"].T
    g = torch.nn.functional.silu(mixed("g") @ w[p + "g"].T)
    decay = torch.exp(-torch.exp(torch.tanh(mixed("w") @ w[p + "w1"].T) @ w[p + "w2"].T + w[p + "w0"]))
    r, k, v, decay = r.view(T, H, d), k.view(T, H, d), v.view(T, H, d), decay.view(T, H, d)
    u = w[p + "u"]
    S = torch.zeros(H, d, d, dtype=h.dtype)
    o = torch.zeros(T, H, d, dtype=h.dtype)
    for t in range(T):
        kv = k[t][:, :, None] * v[t][:, None, :]                 # (H, key channel, value channel)
        o[t] = torch.einsum("hij,hi->hj", S + u[:, :, None] * kv, r[t])
        S = decay[t][:, :, None] * S + kv
    o = group_norm(o.reshape(T * H, d), None, eps).view(T, H * d) * w[p + "norm"] * g
    return o @ w[p + "o"].T


def dense_ff(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    return (gelu_tanh(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def expert(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    return gelu_erf(h @ w[p + "up"].T) @ w[p + "down"].T


def route(h: torch.Tensor, router: torch.Tensor, top: int, count: int, keep: int):
    """-> (idx (T, top), weights (T, top)): softmax scores over all experts; a group's score is its largest score;
    only experts of the `keep` best of `count` groups can be chosen"""
    s = torch.softmax(h.to(torch.float32) @ router.to(torch.float32).T, -1)
    T, E = s.shape
    c = s.clone()
    if count > 1 and keep < count:
        gs = s.view(T, count, E // count).max(-1).values
        best = gs.topk(keep, dim=-1).indices
        ok = torch.zeros(T, count, dtype=torch.bool)
        ok.scatter_(1, best, True)
        c = c.masked_fill(~ok.repeat_interleave(E // count, dim=1), float("-inf"))
    idx = c.topk(top, dim=-1).indices
    chosen = s.gather(1, idx)
    return idx, chosen / (chosen.sum(-1, keepdim=True) + 1e-20)


def moe_ff(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, c: dict) -> torch.Tensor:
    r = c["router"]
    g = r.get("groups") or {}
    idx, wgt = route(h, w[p + "router"], int(r["top"]), int(g.get("count", 1)), int(g.get("keep", g.get("count", 1))))
    out = torch.zeros(h.shape[0], w[p + "e0.down"].shape[0], dtype=h.dtype)
    for t in range(h.shape[0]):
        for s in range(idx.shape[1]):
            out[t] += wgt[t, s].to(h.dtype) * expert(h[t:t + 1], w, p + f"e{int(idx[t, s])}.")[0]
    if c.get("shared"):
        out = out + expert(h, w, p + "shared.")
    return out


# ------------------------------------------------------------------------------------------------ the model
def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens, return_layers: bool = False, dtype=torch.float64):
    """tokens: one sequence from position 0.  -> logits (T, vocab) (and the residual stream after every layer)"""
    w = {k: v.to(dtype) if v.is_floating_point() else v for k, v in w.items()}
    eps, groups, m = float(cfg["norm"]["eps"]), int(cfg["norm"].get("groups", 1)), float(cfg.get("residual_mult", 1.0))
    taps = int((cfg.get("canon") or {}).get("taps", 0))
    tok = torch.as_tensor(tokens, dtype=torch.long)
    pos = torch.arange(tok.shape[0])
    x = w["embed"][tok]
    shared: dict = {}
    after: List[torch.Tensor] = []
    for i, L in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = group_norm(x, w[p + "norm1"], eps, groups)
        if taps:
            h = input_conv(h, w[p + "canon1"])
        kind = L["type"]
        if kind == "attention":
            y = attention(h, w, p + "mix.", L["mixer"], pos, eps, shared)
        elif kind == "attention_2":
            y = attention_2(h, w, p + "mix.", L["mixer"], pos, eps, shared)
        elif kind == "wkv":
            y = wkv(h, w, p + "mix.", L["mixer"], eps)
        else:
            raise ValueError(kind)
        x = x + m * y
        f = L.get("mlp")
        if f is not None:
            h2 = group_norm(x, w[p + "norm2"], eps, groups)
            y = dense_ff(h2, w, p + "mlp.") if f["kind"] == "dense" else moe_ff(h2, w, p + "mlp.", f)
            x = x + m * y
        after.append(x)
    logits = group_norm(x, w["final.norm"], eps, groups) @ w["head"].T
    return (logits, after) if return_layers else logits


# ------------------------------------------------------------------------------------------------ test weights
def tensor_shapes(cfg: dict, decay_rank: int = 8) -> Dict[str, tuple]:
    """checkpoint name -> shape of every tensor of a configuration"""
    W, V = int(cfg["width"]), int(cfg["vocab"])
    taps = int((cfg.get("canon") or {}).get("taps", 0))
    out = {"embed": (V, W), "final.norm": (W,), "head": (V, W)}
    for i, L in enumerate(cfg["layers"]):
        p, c = f"l{i}.", L["mixer"]
        out[p + "norm1"] = (W,)
        if taps:
            out[p + "canon1"] = (W, taps)
        if L["type"] == "wkv":
            n = c["heads"] * c["dim"]
            rank = int(c.get("decay_rank", decay_rank))
            for s in "rkvgw":
                out[p + "mix.mu." + s] = (W,)
            for s in "rkvg":
                out[p + "mix." + s] = (n, W)
            out.update({p + "mix.w1": (rank, W), p + "mix.w2": (n, rank), p + "mix.w0": (n,), p + "mix.u": (c["heads"], c["dim"]),
                        p + "mix.norm": (n,), p + "mix.o": (W, n)})
        else:
            H, G, d, dv = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
            out.update({p + "mix.q": (H * d, W), p + "mix.k": (G * d, W), p + "mix.v": (G * dv, W), p + "mix.o": (W, H * dv)})
            if L["type"] == "attention":
                out.update({p + "mix.q.norm": (H * d,), p + "mix.k.norm": (G * d,), p + "mix.sink": (H,)})
            if c.get("v_mix"):
                out[p + "mix.vmix"] = ()
        f = L.get("mlp")
        if f is None:
            continue
        out[p + "norm2"] = (W,)
        if f["kind"] == "dense":
            out.update({p + "mlp.gate": (f["ff"], W), p + "mlp.up": (f["ff"], W), p + "mlp.down": (W, f["ff"])})
        else:
            out[p + "mlp.router"] = (f["router"]["experts"], W)
            for e in range(f["router"]["experts"]):
                out.update({p + f"mlp.e{e}.up": (f["expert"]["ff"], W), p + f"mlp.e{e}.down": (W, f["expert"]["ff"])})
            if f.get("shared"):
                out.update({p + "mlp.shared.up": (f["shared"]["ff"], W), p + "mlp.shared.down": (W, f["shared"]["ff"])})
    return out


def random_weights(cfg: dict, seed: int = 0, gain: float = 1.0, decay_rank: int = 8) -> Dict[str, torch.Tensor]:
    """bf16-valued random weights (stored as float32): matrices N(0, gain^2 / fan-in), norm weights around one, token
    shift mixes in (0, 1), decays that keep a state for tens of tokens, a router whose scores are well apart"""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(cfg, decay_rank).items():
        last = name.rsplit(".", 1)[-1]
        if name.endswith(("norm1", "norm2", "final.norm", "q.norm", "k.norm", "mix.norm")):
            t = 1.0 + 0.1 * torch.randn(shape, generator=g)
        elif ".mix.mu." in name:
            t = torch.rand(shape, generator=g)
        elif last == "w0":
            t = -1.5 + torch.randn(shape, generator=g)
        elif last == "u":
            t = 0.5 * torch.randn(shape, generator=g)
        elif last == "sink":
            t = torch.randn(shape, generator=g)
        elif last == "vmix":
            t = 0.2 + 0.5 * torch.rand(shape, generator=g)
        elif last == "canon1":
            t = 0.3 * torch.randn(shape, generator=g)
        elif last == "router":
            t = 4.0 * torch.randn(shape, generator=g) / math.sqrt(shape[-1])
        elif name == "embed":
            t = torch.randn(shape, generator=g)
        else:
            t = torch.randn(shape, generator=g) * gain / math.sqrt(shape[-1])
        out[name] = t.to(torch.bfloat16).to(torch.float32)
    return out
