"""ORACLE — TEST INFRASTRUCTURE ONLY. Not imported by the product path.

Plain, slow restatement of the Lilosun decoder, one function per mechanism, written from the design's equations
with torch on the CPU.  It shares no code with mlx_vlm_b200/: no cache, no state objects, no batching; the
recurrent mixer walks the whole sequence token by token on every call.

Notation: x (T, W) residual stream.  A layer is pre-norm with a scale vector on every branch:
    x <- x + s1 * mixer(LN1(x));   x <- x + s2 * ff(LN2(x)),
    LN(y) = (y - mean y) / sqrt(var y + eps) * w      (no bias; var = mean of squared deviations).
Mixers: a latent attention (keys and values expanded from one low-rank row per token plus one rotated key part
shared by the heads, interleaved rotary with YaRN-scaled frequencies, a sliding window of visible keys, a sigmoid
gate on the heads' outputs) and a Mamba-2 state-space mixer (short causal convolution with bias, a (state, vdim)
matrix state per head with an input-dependent decay, gated group RMS norm).
Feed-forwards: a silu-gated unit, and a mixture of clamped gated experts chosen by sigmoid scores with a selection
bias and a limit to the best groups of experts, plus an always-on shared expert with a per-token sigmoid gate.
Output: LN with 'final.norm', head, times a constant.

Weights: dict name -> tensor with the checkpoint's names ('embed', 'l<i>.norm1', 'l<i>.mix.q', ..., 'head').
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch
import torch.nn.functional as F


# ------------------------------------------------------------------------------------------------ pieces
def layer_norm(y: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    d = y - y.mean(-1, keepdim=True)
    return d / torch.sqrt((d * d).mean(-1, keepdim=True) + eps) * w


def rms(y: torch.Tensor, eps: float) -> torch.Tensor:
    return y / torch.sqrt((y * y).mean(-1, keepdim=True) + eps)


def yarn_frequencies(base: float, dims: int, scaling: Optional[dict]):
    """-> (f (dims/2,) float64, amplitude).  Without scaling: f_i = base^(-2i/dims), amplitude 1.  With (factor,
    original, fast, slow): the index at which a frequency makes t turns over `original` positions is
    d(t) = dims ln(original / (2 pi t)) / (2 ln base); between lo = floor d(fast) and hi = ceil d(slow) the
    frequency goes linearly (in the index) from f_i to f_i / factor, and cos and sin are scaled by
    0.1 ln(factor) + 1."""
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


def rotate_pairs(v: torch.Tensor, pos: torch.Tensor, base: float, dims: int, scaling: Optional[dict] = None):
    """v (T, heads, D): of the first `dims` numbers, (2i, 2i + 1) is a pair turned by the angle pos * f_i"""
    half = dims // 2
    if half == 0:
        return v.clone()
    f, amp = yarn_frequencies(base, dims, scaling)
    a = pos.to(torch.float64)[:, None] * f[None, :]
    cos, sin = (torch.cos(a) * amp).to(v.dtype)[:, None, :], (torch.sin(a) * amp).to(v.dtype)[:, None, :]
    even, odd = v[..., 0:dims:2], v[..., 1:dims:2]
    out = v.clone()
    out[..., 0:dims:2] = even * cos - odd * sin
    out[..., 1:dims:2] = odd * cos + even * sin
    return out


def window_visible(T: int, window: Optional[int]) -> torch.Tensor:
    """(T, T) bool: query i sees key j with 0 <= i - j < window (no window: every j <= i)"""
    d = torch.arange(T)[:, None] - torch.arange(T)[None, :]
    ok = d >= 0
    if window:
        ok &= d < window
    return ok


def window_attention(q, k, v, scale: float, window: Optional[int]) -> torch.Tensor:
    """q, k (T, H, D), v (T, H, dv), token t at position t: softmax over the visible keys of scale * q . k, times v"""
    T, H, _ = q.shape
    ok = window_visible(T, window)
    out = torch.zeros(T, H, v.shape[-1], dtype=q.dtype)
    for a in range(H):
        s = (q[:, a] @ k[:, a].T * scale).masked_fill(~ok, float("-inf"))
        out[:, a] = torch.softmax(s, dim=-1) @ v[:, a]
    return out


def latent_attention(h, W, p, m, eps, pos):
    """h (T, width) -> (T, width).  m: heads, dim, rot_dim, vdim, kv_rank, scale, rot, mask"""
    T = h.shape[0]
    H, d, dr, dv, r = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    rot = m.get("rot") or {}
    base, dims, scaling = float(rot.get("base", 10000.0)), int(rot.get("dims", dr)), rot.get("scaling")
    q = (h @ W[p + "q"].T).view(T, H, d + dr)
    q_plain, q_rot = q[..., :d], rotate_pairs(q[..., d:], pos, base, dims, scaling)
    down = h @ W[p + "dkv"].T
    c = rms(down[:, :r], eps) * W[p + "dkv.norm"]
    k_rot = rotate_pairs(down[:, None, r:], pos, base, dims, scaling)[:, 0]         # one part for all heads
    k_plain = (c @ W[p + "uk"].T).view(T, H, d)
    v = (c @ W[p + "uv"].T).view(T, H, dv)
    k = torch.cat([k_plain, k_rot[:, None, :].expand(T, H, dr)], dim=-1)
    out = window_attention(torch.cat([q_plain, q_rot], dim=-1), k, v, float(m["scale"]), (m.get("mask") or {}).get("size"))
    gated = out.reshape(T, H * dv) * torch.sigmoid(h @ W[p + "g"].T)
    return gated @ W[p + "o"].T


def causal_conv(u: torch.Tensor, w: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """u (T, C), w (C, taps), b (C,): y[t] = b + sum_j w[:, j] u[t - (taps - 1) + j], zeros before the first token"""
    T, taps = u.shape[0], w.shape[1]
    y = b.expand(T, -1).clone()
    for j in range(taps):
        back = taps - 1 - j
        if back < T:
            y[back:] += w[:, j] * u[:T - back]
    return y


def ssm_walk(xh, B, C, dt, A, D):
    """xh (T, H, P), B, C (T, H, N) (already spread over the heads), dt (T, H) > 0, A (H,) > 0, D (H,):
    S_t = exp(-A dt_t) S_(t-1) + dt_t B_t x_t^T (S: N x P, from zero);  y_t = S_t^T C_t + D x_t"""
    T, H, P = xh.shape
    S = torch.zeros(H, B.shape[-1], P, dtype=xh.dtype)
    y = torch.zeros_like(xh)
    for t in range(T):
        S = torch.exp(-A * dt[t])[:, None, None] * S + dt[t][:, None, None] * B[t][:, :, None] * xh[t][:, None, :]
        y[t] = torch.einsum("hnp,hn->hp", S, C[t]) + D[:, None] * xh[t]
    return y


def mamba2(h, W, p, m, eps):
    """h (T, width) -> (T, width).  m: heads, vdim, state, groups, norm_groups, conv"""
    T = h.shape[0]
    H, P, N, G, NG = m["heads"], m["vdim"], m["state"], m.get("groups", 1), m.get("norm_groups", 1)
    inner = H * P
    proj = h @ W[p + "in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xbc = F.silu(causal_conv(xbc, W[p + "conv"], W[p + "conv.b"]))
    xh = xbc[:, :inner].view(T, H, P)
    per = H // G
    B = xbc[:, inner:inner + G * N].view(T, G, N).repeat_interleave(per, dim=1)
    C = xbc[:, inner + G * N:].view(T, G, N).repeat_interleave(per, dim=1)
    dt = F.softplus(dt + W[p + "dt_bias"])
    y = ssm_walk(xh, B, C, dt, torch.exp(W[p + "A_log"]), W[p + "D"]).reshape(T, inner)
    y = y * F.silu(z)
    y = rms(y.view(T, NG, inner // NG), eps).reshape(T, inner) * W[p + "norm"]
    return y @ W[p + "o"].T


def silu_glu(h, W, p):
    return (F.silu(h @ W[p + "gate"].T) * (h @ W[p + "up"].T)) @ W[p + "down"].T


def clamped_expert(h, W, p, limit: float):
    g = torch.clamp(h @ W[p + "gate"].T, max=limit)
    u = torch.clamp(h @ W[p + "up"].T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ W[p + "down"].T


def route(h, Wr, correction, top: int, n_groups: int, keep: int):
    """-> (idx (T, top), weights (T, top)).  s = sigmoid(W_r h); the choice is made on s + correction among the
    experts of the `keep` groups (of `n_groups` equal groups of neighbours) whose two best choice scores sum
    highest; the weights are the chosen s, normalised"""
    s = torch.sigmoid(h.to(torch.float32) @ Wr.to(torch.float32).T)
    choice = s + correction.to(torch.float32)
    T, E = s.shape
    if n_groups > 1:
        per = E // n_groups
        by_group = choice.view(T, n_groups, per)
        group_score = by_group.topk(min(2, per), dim=-1).values.sum(-1)
        kept = torch.zeros(T, n_groups, dtype=torch.bool)
        kept.scatter_(1, group_score.topk(keep, dim=-1).indices, True)
        choice = choice.masked_fill(~kept.repeat_interleave(per, dim=1), float("-inf"))
    idx = choice.topk(top, dim=-1).indices
    w = s.gather(1, idx)
    return idx, w / (w.sum(-1, keepdim=True) + 1e-20)


def expert_mixture(h, W, p, f):
    r = f["router"]
    groups = r.get("groups") or {}
    idx, wgt = route(h, W[p + "router"], W[p + "correction"], r["top"], int(groups.get("count", 1)),
                     int(groups.get("keep", 1)))
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, a in zip(idx[t].tolist(), wgt[t].tolist()):
            out[t] += a * clamped_expert(h[t:t + 1], W, f"{p}e{e}.", float(f["expert"]["limit"]))[0]
    if f.get("shared"):
        gate = torch.sigmoid(h @ W[p + "shared.sg"].T)                       # (T, 1)
        out = out + gate * clamped_expert(h, W, p + "shared.", float(f["shared"]["limit"]))
    return out


def feed_forward(h, W, p, f):
    return silu_glu(h, W, p) if f["kind"] == "dense" else expert_mixture(h, W, p, f)


def layer(x, W, i, L, eps, pos):
    p = f"l{i}."
    n = layer_norm(x, W[p + "norm1"], eps)
    y = latent_attention(n, W, p + "mix.", L["mixer"], eps, pos) if L["type"] == "latent_attention" else \
        mamba2(n, W, p + "mix.", L["mixer"], eps)
    x = x + W[p + "ls1"] * y
    if L.get("mlp") is not None:
        x = x + W[p + "ls2"] * feed_forward(layer_norm(x, W[p + "norm2"], eps), W, p + "mlp.", L["mlp"])
    return x


def forward(cfg: dict, W: Dict[str, torch.Tensor], tokens: List[int], dtype=torch.float64,
            layers_out: Optional[list] = None) -> torch.Tensor:
    """logits (T, vocab) of one sequence from position 0; layers_out collects the stream after every layer"""
    W = {k: (v if v.dtype in (torch.int32, torch.int64) else v.to(dtype)) for k, v in W.items()}
    eps = float((cfg.get("norm") or {}).get("eps", 1e-5))
    x = W["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    pos = torch.arange(len(tokens))
    for i, L in enumerate(cfg["layers"]):
        x = layer(x, W, i, L, eps, pos)
        if layers_out is not None:
            layers_out.append(x.clone())
    return layer_norm(x, W["final.norm"], eps) @ W["head"].T * float(cfg.get("logit_scale", 1.0))


# ------------------------------------------------------------------------------------------------ checkpoints
def tensor_shapes(cfg: dict) -> Dict[str, tuple]:
    Wd, V = cfg["width"], cfg["vocab"]
    out = {"embed": (V, Wd), "final.norm": (Wd,), "head": (V, Wd)}
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        out[p + "norm1"] = out[p + "ls1"] = (Wd,)
        if L["type"] == "latent_attention":
            H, d, dr, dv, r = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
            out.update({p + "mix.q": (H * (d + dr), Wd), p + "mix.dkv": (r + dr, Wd), p + "mix.dkv.norm": (r,),
                        p + "mix.uk": (H * d, r), p + "mix.uv": (H * dv, r), p + "mix.g": (H * dv, Wd),
                        p + "mix.o": (Wd, H * dv)})
        else:
            H, P, N, G = m["heads"], m["vdim"], m["state"], m.get("groups", 1)
            ch = H * P + 2 * G * N
            out.update({p + "mix.in": (2 * H * P + 2 * G * N + H, Wd), p + "mix.conv": (ch, m["conv"]),
                        p + "mix.conv.b": (ch,), p + "mix.dt_bias": (H,), p + "mix.A_log": (H,), p + "mix.D": (H,),
                        p + "mix.norm": (H * P,), p + "mix.o": (Wd, H * P)})
        f = L.get("mlp")
        if f is None:
            continue
        out[p + "norm2"] = out[p + "ls2"] = (Wd,)
        if f["kind"] == "dense":
            out.update({p + "mlp.gate": (f["ff"], Wd), p + "mlp.up": (f["ff"], Wd), p + "mlp.down": (Wd, f["ff"])})
        else:
            E, ff = f["router"]["experts"], f["expert"]["ff"]
            out.update({p + "mlp.router": (E, Wd), p + "mlp.correction": (E,)})
            for e in range(E):
                out.update({p + f"mlp.e{e}.gate": (ff, Wd), p + f"mlp.e{e}.up": (ff, Wd), p + f"mlp.e{e}.down": (Wd, ff)})
            if f.get("shared"):
                fs = f["shared"]["ff"]
                out.update({p + "mlp.shared.gate": (fs, Wd), p + "mlp.shared.up": (fs, Wd),
                            p + "mlp.shared.down": (Wd, fs), p + "mlp.shared.sg": (1, Wd)})
    return out


def random_weights(cfg: dict, seed: int = 0, gain: float = 1.0) -> Dict[str, torch.Tensor]:
    """bf16-valued random weights (stored as float32): matrices N(0, gain^2 / fan-in), norm weights around one,
    branch scales around one half, the recurrent constants in their usual ranges"""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        last = name.rsplit(".", 1)[-1]
        if name.endswith(("norm1", "norm2", "final.norm", "dkv.norm", "mix.norm")):
            t = 1.0 + 0.1 * torch.randn(shape, generator=g)
        elif last in ("ls1", "ls2"):
            t = 0.5 + 0.1 * torch.randn(shape, generator=g)
        elif last == "A_log":
            t = torch.log(0.5 + 3.0 * torch.rand(shape, generator=g))
        elif last == "dt_bias":
            t = -2.0 + torch.randn(shape, generator=g)
        elif last == "D":
            t = 1.0 + 0.2 * torch.randn(shape, generator=g)
        elif last == "correction":
            t = 0.3 * torch.randn(shape, generator=g)
        elif name.endswith("conv.b"):
            t = 0.1 * torch.randn(shape, generator=g)
        elif name.endswith("mix.conv"):
            t = torch.randn(shape, generator=g) / math.sqrt(shape[-1])
        elif name == "embed":
            t = torch.randn(shape, generator=g)
        else:
            t = torch.randn(shape, generator=g) * gain / math.sqrt(shape[-1])
        out[name] = t.to(torch.bfloat16).to(torch.float32)
    return out
