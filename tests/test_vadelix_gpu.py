"""Vadelix on the GPU against the plain restatement in oracle/vadelix.py: every mechanism alone (with inputs made so
that a fault shows: a key that stands out just inside and just outside the window, at a staging tile's edge and far
back; a sink that dominates; a state that must survive a step), whole prompts with the residual stream after every
layer, prefill against token-by-token decoding, portions, batches of unequal requests, slots released and used again,
long decoding, other sizes, and greedy generation through generate_step and the batch scheduler.  Small random
configurations; none of them is a real model's."""
import copy
import math
import types

import numpy as np
import pytest
import torch

from oracle import vadelix as O

pytestmark = pytest.mark.gpu


# ------------------------------------------------------------------------------------------------ configurations
def att(heads=6, kv_heads=3, dim=16, vdim=12, dims=8, base=5000.0, scaling=(4.0, 32, 16.0, 2.0), scale=None, v_mix=True):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "v_mix": v_mix,
         "rot": {"base": base, "dims": dims}, "scale": scale if scale is not None else 1.0 / math.sqrt(dim)}
    if scaling:
        m["rot"]["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return m


def att2(heads=6, kv_heads=3, dim=8, vdim=12, window=13, temp=(0.4, 7), scale=None, v_mix=True):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "v_mix": v_mix,
         "scale": scale if scale is not None else 1.0 / math.sqrt(dim)}
    if window:
        m["mask"] = {"size": window}
    if temp:
        m["q_temp"] = {"coef": temp[0], "every": temp[1]}
    return m


def wkv(heads=3, dim=12):
    return {"heads": heads, "dim": dim}


def dense(ff=56):
    return {"kind": "dense", "ff": ff}


def moe(experts=8, top=3, ff=24, count=4, keep=2, shared=40):
    f = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top, "groups": {"count": count, "keep": keep}}}
    if shared:
        f["shared"] = {"ff": shared}
    return f


def layer(kind, mixer, mlp="dense"):
    return {"type": kind, "mixer": mixer, "mlp": dense() if mlp == "dense" else (moe() if mlp == "moe" else mlp)}


def config(layers=None, width=72, vocab=101, eps=1e-5, groups=3, mult=0.4, taps=3):
    layers = layers or [layer("attention_2", att2(), "moe"), layer("wkv", wkv()), layer("attention", att(), "dense"),
                        layer("wkv", wkv(heads=2, dim=20), None),
                        layer("attention_2", att2(window=40, temp=(0.7, 16), dim=24), moe(experts=6, top=2, count=1, keep=1, shared=None))]
    c = {"architecture": "Vadelix", "vocab": vocab, "width": width, "layers": layers, "norm": {"eps": eps, "groups": groups},
         "residual_mult": mult}
    if taps:
        c["canon"] = {"taps": taps}
    return c


_MODELS = {}


def build(cfg, dtype="float32", seed=1):
    from mlx_vlm_b200.models.vadelix import Model, ModelConfig
    key = (repr(cfg), dtype, seed)
    if key not in _MODELS:
        W = O.random_weights(cfg, seed)
        _MODELS[key] = (Model(ModelConfig.from_dict(copy.deepcopy(cfg)), dtype=dtype).load_weights(W), W)
    return _MODELS[key]


def host(eng, t):
    eng.stream.synchronize()
    return t.detach().to("cpu", torch.float64)


def rel_rows(got, want):
    d = got - want
    d = d - d.mean(-1, keepdim=True)
    return d.square().mean(-1).sqrt() / (want - want.mean(-1, keepdim=True)).square().mean(-1).sqrt()


def rel(got, want):
    return rel_rows(got, want).max().item()


TOL = {"float32": 3e-5, "bfloat16": 8e-2}


def close(got, want, dtype):
    """float32: every row within 3e-5 of the logits' spread.  bfloat16: nine rows of ten within 8e-2 and none beyond
    0.25 — an expert choice that flips on a close call of the rounded scores moves a row by more than rounding alone"""
    r = rel_rows(got, want)
    if dtype == "float32":
        return bool(r.max() < TOL[dtype])
    return bool(r.quantile(0.9) < TOL[dtype] and r.max() < 0.25)


def tokens(n, vocab, seed=0):
    return np.random.default_rng(seed).integers(0, vocab, n).tolist()


def run_alone(model, toks, cuts=None):
    """one request in its own fresh pool, its tokens cut into portions; logits of every position"""
    lm = model.language_model
    cache = lm.make_cache()
    out, at = [], 0
    for n in (cuts or [len(toks)]):
        part = toks[at:at + n]
        out.append(host(model.engine, lm.step([part], [cache], want=[list(range(len(part)))])))
        at += n
    assert at == len(toks)
    return torch.cat(out)


# ------------------------------------------------------------------------------------------------ mechanisms
def _eng(exact=True):
    from mlx_vlm_b200.layer_engine import LayerEngine
    key = "eng" if exact else "eng16"
    if key not in _MODELS:
        _MODELS[key] = LayerEngine("cuda:0", exact=exact)
    return _MODELS[key]


def dev(a, dtype=torch.float32):
    return torch.as_tensor(a).to(device="cuda:0", dtype=dtype).contiguous()


def bf(t):
    return t.to(torch.bfloat16).to(torch.float32)


class _Pool:
    """what the mixers read of a pool: rows (caching layers, slots, capacity, row) and state (slots, floats)"""

    def __init__(self, slots=3, capacity=0, row=0, state=0, dtype=torch.float32):
        self.buf = torch.zeros((1, slots, max(capacity, 1), max(row, 1)), device="cuda:0", dtype=dtype)
        self.state = torch.full((slots, max(state, 1)), 7.0, device="cuda:0")     # stale numbers: never to be read
        torch.cuda.synchronize()


def _ctx(eng, pool, segments, eps=1e-5):
    """segments: (first row, rows, slot, first position) per sequence; None rows of a decode step are given as such"""
    from mlx_vlm_b200.models.decoder_blocks import StepCtx
    T = sum(n for _, n, _, _ in segments)
    slot, pos = np.zeros(T, np.int32), np.zeros(T, np.int32)
    for a, n, s, p0 in segments:
        slot[a:a + n], pos[a:a + n] = s, np.arange(p0, p0 + n)
    return StepCtx(eng.ops, dev(slot, torch.int32), dev(pos, torch.int32), pool, eps, segments)


def _decode_ctx(eng, pool, slots, positions, eps=1e-5):
    from mlx_vlm_b200.models.decoder_blocks import StepCtx
    return StepCtx(eng.ops, dev(np.asarray(slots, np.int32), torch.int32), dev(np.asarray(positions, np.int32), torch.int32),
                   pool, eps, None)


@pytest.mark.parametrize("groups,N", [(1, 150), (3, 150), (5, 40), (8, 1024), (150, 150)])
def test_norm_in_groups_and_scalar_residual(groups, N):
    eng = _eng()
    ops = eng.ops
    g = torch.Generator().manual_seed(groups)
    T = 7
    y = torch.randn(T, N, generator=g) * torch.linspace(0.1, 30.0, N)        # parts of very different size
    w = bf(1 + 0.2 * torch.randn(N, generator=g))
    out = dev(torch.zeros(T, N))
    ops.norm_rows(dev(y), dev(w, torch.bfloat16), 1e-3, out, groups=groups)
    want = O.group_norm(y.double(), w.double(), 1e-3, groups)
    assert (host(eng, out) - want).abs().max() < 1e-5 * want.abs().max()
    rows = dev(np.asarray([4, 0], np.int32), torch.int32)
    two = dev(torch.zeros(2, N))
    ops.norm_rows(dev(y), dev(w, torch.bfloat16), 1e-3, two, groups=groups, rows=rows)
    assert (host(eng, two) - want[[4, 0]]).abs().max() < 1e-5 * want.abs().max()
    # x += m * (weighted rows + shared row), alone and with the norm of the updated rows in the same launch
    top, m = 3, 0.37
    for n_rows in (T, 70):
        xr, yr = torch.randn(n_rows, N, generator=g) + 2.0, torch.randn(n_rows * top, N, generator=g)
        wr, sh = torch.rand(n_rows, top, generator=g), torch.randn(n_rows, N, generator=g)
        upd = xr.double() + m * ((yr.double().view(n_rows, top, N) * wr.double()[:, :, None]).sum(1) + sh.double())
        x = dev(xr)
        ops.residual_rows(dev(yr), x, None, combine=dev(wr), top=top, shared=dev(sh), mult=m)
        assert (host(eng, x) - upd).abs().max() < 1e-5
        x, n = dev(xr), dev(torch.zeros(n_rows, N))
        ops.residual_norm_rows(dev(yr), x, None, dev(w, torch.bfloat16), 1e-3, n, combine=dev(wr), top=top, shared=dev(sh),
                               mult=m, groups=groups)
        assert (host(eng, x) - upd).abs().max() < 1e-5
        ref = O.group_norm(upd, w.double(), 1e-3, groups)
        assert (host(eng, n) - ref).abs().max() < 2e-5 * max(1.0, ref.abs().max().item())


@pytest.mark.parametrize("taps", [1, 2, 4, 6])
def test_input_convolution_in_portions_and_slots(taps):
    """h + conv(h) over a sequence cut into portions (down to one token), two sequences in one step, a slot used again"""
    eng = _eng()
    ops = eng.ops
    g = torch.Generator().manual_seed(taps)
    C, n = 37, 23
    c = bf(torch.randn(C, taps, generator=g))
    ha, hb = torch.randn(n, C, generator=g), torch.randn(9, C, generator=g)
    want_a, want_b = O.input_conv(ha.double(), c.double()), O.input_conv(hb.double(), c.double())
    pool = _Pool(slots=3, state=(taps - 1) * C + 5)
    st = pool.state[:, 2:2 + (taps - 1) * C]
    got_a, got_b, at = [], [], 0
    for k, cut in enumerate([5, 1, 1, 9, 2, 5]):
        segs = [(0, cut, 2, at)]
        rows = [ha[at:at + cut]]
        if k == 1:                    # b joins for one step, whole, in slot 0
            segs.append((cut, 9, 0, 0))
            rows.append(hb)
        ctx = _ctx(eng, pool, segs) if (cut > 1 or k == 1) else _decode_ctx(eng, pool, [2], [at])
        y = host(eng, ops.short_conv(dev(torch.cat(rows)), dev(c, torch.bfloat16), st, ctx, residual=True))
        got_a.append(y[:cut])
        if k == 1:
            got_b.append(y[cut:])
        at += cut
    assert (torch.cat(got_a) - want_a).abs().max() < 1e-5
    assert (got_b[0] - want_b).abs().max() < 1e-5
    # slot 2 again, from position 0: what a left there is not read
    y = host(eng, ops.short_conv(dev(hb), dev(c, torch.bfloat16), st, _ctx(eng, pool, [(0, 9, 2, 0)]), residual=True))
    assert (y - want_b).abs().max() < 1e-5


def test_token_shift_keeps_the_last_input_per_slot():
    eng = _eng()
    ops = eng.ops
    g = torch.Generator().manual_seed(3)
    C, n = 45, 17
    mu = bf(torch.rand(5, C, generator=g))
    ha, hb = torch.randn(n, C, generator=g), torch.randn(6, C, generator=g)

    def ref(h):
        prev = torch.cat([torch.zeros(1, C), h[:-1]]).double()
        return torch.stack([h.double() + (prev - h.double()) * mu[s].double() for s in range(5)])

    pool = _Pool(slots=2, state=C + 3)
    st = pool.state[:, 3:3 + C]
    got, at = [], 0
    for k, cut in enumerate([4, 1, 1, 7, 2, 2]):
        if cut == 1:
            ctx, rows = _decode_ctx(eng, pool, [1], [at]), ha[at:at + 1]
        elif k == 3:                  # b joins, whole, in slot 0
            ctx, rows = _ctx(eng, pool, [(0, cut, 1, at), (cut, 6, 0, 0)]), torch.cat([ha[at:at + cut], hb])
        else:
            ctx, rows = _ctx(eng, pool, [(0, cut, 1, at)]), ha[at:at + cut]
        M = host(eng, ops.token_shift(dev(rows), dev(mu, torch.bfloat16), st, ctx))
        got.append(M[:, :cut])
        if k == 3:
            assert (M[:, cut:] - ref(hb)).abs().max() < 1e-6
        at += cut
    assert (torch.cat(got, 1) - ref(ha)).abs().max() < 1e-6
    assert (host(eng, st[1]) - ha[-1].double()).abs().max() == 0


def _attend(eng, q, k, v, H, G, d, dv, scale, pos0=0, window=0, bias_exp=0.0, sink=None, unit_sink=False, n_split=None,
            dtype=torch.float32):
    """the row kernel over a cache that holds k, v at positions pos0 .. (queries at the same positions)"""
    ops = eng.ops
    T = q.shape[0]
    pool = _Pool(slots=2, capacity=pos0 + T + 3, row=G * (d + dv), dtype=dtype)
    pool.buf[0, 1, pos0:pos0 + T, :G * d] = dev(k.reshape(T, G * d)).to(dtype)
    pool.buf[0, 1, pos0:pos0 + T, G * d:] = dev(v.reshape(T, G * dv)).to(dtype)
    slot, pos = dev(np.full(T, 1, np.int32), torch.int32), dev(np.arange(pos0, pos0 + T, dtype=np.int32), torch.int32)
    out = dev(torch.zeros(T, H * dv))
    ops.sink_attention(dev(q.reshape(T, H * d)), pool.buf[0], slot, pos, out, None if sink is None else dev(sink, torch.bfloat16),
                       H, G, d, dv, scale, window=window, n_split=n_split, bias_exp=bias_exp, unit_sink=unit_sink)
    return host(eng, out).view(T, H, dv)


def _attend_ref(q, k, v, H, G, scale, window=0, slopes=None, sink=None):
    T = q.shape[0]
    rep = H // G
    s = torch.einsum("thd,shd->hts", q.double(), k.double().repeat_interleave(rep, dim=1)) * scale
    i = torch.arange(T)
    dist = (i[:, None] - i[None, :]).double()
    if slopes is not None:
        s = s - slopes[:, None, None] * dist[None]
    vis = dist >= 0
    if window:
        vis &= dist < window
    a = O.softmax_with_sink(s, vis, sink if sink is not None else torch.full((H,), float("-inf"), dtype=torch.float64))
    return torch.einsum("hts,shd->thd", a, v.double().repeat_interleave(rep, dim=1))


@pytest.mark.parametrize("window", [1, 2, 31, 32, 33, 64, 100])
@pytest.mark.parametrize("n_split", [1, None])
def test_window_edges_with_a_key_that_stands_out(window, n_split):
    """one key far louder than the rest, placed just inside and just outside the window of the last query: inside it
    takes the whole output, outside it must not be seen"""
    eng = _eng()
    g = torch.Generator().manual_seed(window)
    H, G, d, dv, T = 4, 2, 8, 6, 140
    q, k, v = torch.randn(T, H, d, generator=g), 0.1 * torch.randn(T, G, d, generator=g), torch.randn(T, G, dv, generator=g)
    slopes = torch.tensor([2.0 ** (-8.0 * (h + 1) / H) for h in range(H)], dtype=torch.float64)
    zero = torch.zeros(H, dtype=torch.float64)
    for back in (window - 1, window):                 # distance of the loud key from the last query
        if back >= T:
            continue
        kk = k.clone()
        kk[T - 1 - back] = 30.0 * q[T - 1].view(G, H // G, d)[:, 0] / q[T - 1].view(G, H // G, d)[:, 0].norm(dim=-1, keepdim=True)
        got = _attend(eng, q, kk, v, H, G, d, dv, 0.5, window=window, bias_exp=8.0, unit_sink=True,
                      n_split=n_split if n_split else 4)
        want = _attend_ref(q, kk, v, H, G, 0.5, window, slopes, zero)
        assert (got - want).abs().max() < 2e-5
        loud = (got[T - 1, 0] - v[T - 1 - back, 0].double()).abs().max()
        assert (loud < 1e-3) == (back < window)


def test_far_key_sink_and_distance_bias():
    """full causal attention: a loud key 700 positions back is found; a sink logit that dominates empties the output;
    the distance bias, not the sink, decides between two equal keys"""
    eng = _eng()
    g = torch.Generator().manual_seed(5)
    H, G, d, dv, T = 3, 1, 12, 10, 750
    q, k, v = torch.randn(T, H, d, generator=g), 0.1 * torch.randn(T, G, d, generator=g), torch.randn(T, G, dv, generator=g)
    k[40, 0] = 25.0 * q[T - 1, 1] / q[T - 1, 1].norm()
    sink = bf(torch.tensor([0.3, -1.0, 300.0]))
    for n_split in (1, 8):
        got = _attend(eng, q, k, v, H, G, d, dv, 0.7, sink=sink, n_split=n_split)
        want = _attend_ref(q, k, v, H, G, 0.7, sink=sink.double())
        assert (got - want).abs().max() < 2e-5
        assert (got[T - 1, 1] - v[40, 0].double()).abs().max() < 1e-3          # the far key
        assert got[:, 2].abs().max() < 1e-6                                      # the sink took everything
    # cached rows rounded to bf16 (the serving mode's cache) and a first position that is not a tile's start
    # (the 29 rows before it are zeros in the cache: keys with score 0 and no value)
    got = _attend(eng, q[:90], bf(k[:90]), bf(v[:90]), H, G, d, dv, 0.7, pos0=29, sink=sink, dtype=torch.bfloat16)
    pad = lambda t: torch.cat([torch.zeros(29, *t.shape[1:]), t])
    want = _attend_ref(pad(q[:90]), pad(bf(k[:90])), pad(bf(v[:90])), H, G, 0.7, sink=sink.double())[29:]
    assert (got - want).abs().max() < 2e-5
    slopes = torch.tensor([2.0 ** (-8.0 * (h + 1) / H) for h in range(H)], dtype=torch.float64)
    kk = torch.zeros(T, G, d)
    got = _attend(eng, q, kk, v, H, G, d, dv, 0.7, bias_exp=8.0, unit_sink=True)
    want = _attend_ref(q, kk, v, H, G, 0.7, slopes=slopes, sink=torch.zeros(H, dtype=torch.float64))
    assert (got - want).abs().max() < 2e-5


@pytest.mark.parametrize("case", ["norms", "temperature", "mix", "plain"])
def test_projection_post_steps(case):
    """what happens between the projections and the cache: norms over the whole projection, the query temperature, unit
    values, value mixing — against the plain functions"""
    eng = _eng()
    ops = eng.ops
    g = torch.Generator().manual_seed(11)
    H, G, d, dv, T, eps = 4, 2, 10, 6, 9, 1e-3
    q, k, v = 3 * torch.randn(T, H * d, generator=g), 2 * torch.randn(T, G * d, generator=g), torch.randn(T, G * dv, generator=g)
    qw, kw = bf(1 + 0.3 * torch.randn(H * d, generator=g)), bf(1 + 0.3 * torch.randn(G * d, generator=g))
    vf, lam = torch.randn(T, G * dv, generator=g), bf(torch.tensor([0.3]))
    rot = {"base": 77.0, "dims": 6, "scaling": {"factor": 3.0, "original": 16, "fast": 4.0, "slow": 1.0}}
    p0 = 120
    pos = torch.arange(p0, p0 + T)
    pool = _Pool(slots=2, capacity=p0 + T, row=G * (d + dv) + 3)
    ctx = _ctx(eng, pool, [(0, T, 1, p0)], eps)
    kw_args, qr, kr, vr = {}, q.double(), k.double(), v.double()
    if case == "norms":
        kw_args = dict(q_norm=dev(qw, torch.bfloat16), k_norm=dev(kw, torch.bfloat16), eps=eps, v_unit=True)
        qr, kr = O.group_norm(qr, qw.double(), eps), O.group_norm(kr, kw.double(), eps)
        vr = O.group_norm(vr.reshape(T * G, dv), None, eps).view(T, G * dv)
    elif case == "temperature":
        kw_args = dict(q_temp=(0.6, 50))
        qr = qr * (1.0 + 0.6 * torch.log(torch.floor((pos.double() + 1) / 50) + 1))[:, None]
    elif case == "mix":
        keep = dev(torch.zeros(T, G * dv))
        kw_args = dict(eps=eps, v_unit=True, vmix=dev(lam, torch.bfloat16), v_first=dev(vf), v_keep=keep)
        vr = O.group_norm(vr.reshape(T * G, dv), None, eps).view(T, G * dv)
        vr = (1 - lam.double()) * vr + lam.double() * vf.double()
    dims = 0 if case == "temperature" else rot["dims"]
    cs = ctx.rope(rot["base"], dims, (3.0, 16.0, 4.0, 1.0))
    Q = dev(q)
    ops.qkv_post(Q, dev(k), dev(v), pool.buf[0][..., :G * (d + dv)], ctx.slot, ctx.pos, cs, H, G, d, dv, dims, **kw_args)
    if dims:
        qr = O.rotate_half(qr.view(T, H, d), pos, rot).reshape(T, H * d)
        kr = O.rotate_half(kr.view(T, G, d), pos, rot).reshape(T, G * d)
    row = host(eng, pool.buf[0, 1, p0:p0 + T])
    assert (host(eng, Q) - qr).abs().max() < 2e-5
    assert (row[:, :G * d] - kr).abs().max() < 2e-5
    assert (row[:, G * d:G * (d + dv)] - vr).abs().max() < 2e-5
    assert row[:, G * (d + dv):].abs().max() == 0
    if case == "mix":
        assert (host(eng, keep) - vr).abs().max() < 2e-5


@pytest.mark.parametrize("part_len", [0, 8, 5])
@pytest.mark.parametrize("H,d", [(3, 8), (2, 12), (4, 32), (1, 64), (2, 100), (5, 4)])
def test_state_with_a_decay_per_channel_in_portions_and_slots(H, d, part_len):
    """part_len: long portions are walked in parts of that many tokens at the same time (a portion of 17 tokens in 3 or 4
    parts, one of 2 tokens beside one of 19 in one step, a last part of one token)"""
    eng = _eng()
    ops = eng.ops
    from mlx_vlm_b200.models.decoder_blocks import state_floats
    g = torch.Generator().manual_seed(H * 100 + d)
    n = H * d
    u = bf(0.5 * torch.randn(H, d, generator=g))

    def rand(T):
        return [torch.randn(T, n, generator=g) for _ in range(3)] + [-1.0 + torch.randn(T, n, generator=g)]

    def ref(r, k, v, x):
        T = r.shape[0]
        r, k, v, w = (t.double().view(T, H, d) for t in (r, k, v, torch.exp(-torch.exp(x.double()))))
        S, o = torch.zeros(H, d, d, dtype=torch.float64), torch.zeros(T, H, d, dtype=torch.float64)
        for t in range(T):
            kv = k[t][:, :, None] * v[t][:, None, :]
            o[t] = torch.einsum("hij,hi->hj", S + u.double()[:, :, None] * kv, r[t])
            S = w[t][:, :, None] * S + kv
        return o.view(T, n)

    a, b = rand(41), rand(19)
    want_a, want_b = ref(*a), ref(*b)
    sf = state_floats(H, d, d)
    pool = _Pool(slots=3, state=sf + 4)
    st = pool.state[:, 4:4 + sf]

    def run(ctx, parts):
        r, k, v, x = (dev(torch.cat(p)) for p in parts)
        o = dev(torch.zeros(r.shape[0], n))
        ops.linear_state(r, k, v, o, st, ctx, H=H, rep=1, dim=d, vdim=d, decay_logits=x, bonus=dev(u, torch.bfloat16),
                         part_len=part_len)
        return host(eng, o)

    got, at = [], 0
    for kk, cut in enumerate([17, 1, 1, 2, 20] if part_len != 5 else [21, 1, 1, 2, 16]):
        part = [[t[at:at + cut]] for t in a]
        if kk == 3:                   # b joins for one step, whole, in another slot
            y = run(_ctx(eng, pool, [(0, cut, 2, at), (cut, 19, 0, 0)]), [p + [t] for p, t in zip(part, b)])
            assert (y[cut:] - want_b).abs().max() < 5e-5 * max(1.0, want_b.abs().max().item())
        elif cut == 1:
            y = run(_decode_ctx(eng, pool, [2], [at]), part)
        else:
            y = run(_ctx(eng, pool, [(0, cut, 2, at)]), part)
        got.append(y[:cut])
        at += cut
    assert (torch.cat(got) - want_a).abs().max() < 5e-5 * max(1.0, want_a.abs().max().item())
    y = run(_ctx(eng, pool, [(0, 19, 2, 0)]), [[t] for t in b])          # slot 2 again, from position 0
    assert (y - want_b).abs().max() < 5e-5 * max(1.0, want_b.abs().max().item())


@pytest.mark.parametrize("E,top,count,keep", [(8, 3, 4, 2), (12, 2, 3, 1), (6, 6, 1, 1), (6, 2, 6, 3), (16, 4, 2, 2), (5, 1, 5, 1),
                                              (64, 8, 8, 3)])
def test_router_softmax_scores_and_group_maximum(E, top, count, keep):
    eng = _eng()
    g = torch.Generator().manual_seed(E + top)
    T, W = 33, 24
    h, router = torch.randn(T, W, generator=g), bf(torch.randn(E, W, generator=g))
    z = h @ router.T
    idx, wgt = eng.ops.router_group_topk(dev(z), top, None, count, keep, softmax=True, group_max=True)
    ridx, rw = O.route(h, router, top, count, keep)
    gi, gw = host(eng, idx).long(), host(eng, wgt)
    for t in range(T):
        assert sorted(gi[t].tolist()) == sorted(ridx[t].tolist())
        order = {int(e): float(w) for e, w in zip(ridx[t], rw[t])}
        for e, w in zip(gi[t].tolist(), gw[t].tolist()):
            assert abs(w - order[e]) < 1e-5


def test_gelu_forms():
    """the erf form in the row product's epilogue and in the operand rounding; the tanh form on the gate"""
    eng, eng16 = _eng(), _eng(False)
    g = torch.Generator().manual_seed(2)
    T, K, n = 5, 40, 28
    x, w = torch.randn(T, K, generator=g) * 2, bf(torch.randn(n, K, generator=g) * 0.5)
    from mlx_vlm_b200.models.layer_ops import ACT_GELU, EPI_GELU, GELU_TANH_ALPHA, GELU_TANH_CUBIC
    y = host(eng, eng.ops.linear(dev(x), dev(w, torch.bfloat16), epi=EPI_GELU))
    assert (y - O.gelu_erf(x.double() @ w.double().T)).abs().max() < 1e-5
    big = torch.randn(130, K, generator=g) * 3
    hb = host(eng16, eng16.ops.to_bf16(dev(big), K, act=ACT_GELU))
    want = O.gelu_erf(big.double())
    assert ((hb[:, :K] - want).abs() <= want.abs() / 256 + 1e-6).all() and hb[:, K:].abs().max() == 0
    a, b = torch.randn(T, n, generator=g) * 3, torch.randn(T, n, generator=g)
    out = dev(torch.zeros(T, n))
    eng.ops.glu_clamp(dev(a), dev(b), float("inf"), GELU_TANH_ALPHA, out, up_offset=0.0, cubic=GELU_TANH_CUBIC)
    assert (host(eng, out) - O.gelu_tanh(a.double()) * b.double()).abs().max() < 2e-6


@pytest.mark.parametrize("window,p0,n", [(40, 0, 300), (150, 0, 330), (150, 70, 260), (128, 5, 256), (0, 30, 170), (0, 0, 260)])
def test_prompt_attention_on_the_tensor_cores(window, p0, n):
    """a long portion (serving mode) through the two tensor-core products against the row kernel on the same cache: the
    window's edge, the distance bias and the sink must agree"""
    eng = _eng(False)
    from mlx_vlm_b200.models.decoder_blocks import GroupedAttention
    g = torch.Generator().manual_seed(window + n)
    for kind in ("unit", "learned"):
        cfg = att2(heads=4, kv_heads=2, dim=16, vdim=24, window=window, temp=None) if kind == "unit" else \
            att(heads=4, kv_heads=2, dim=16, vdim=24, dims=0, scaling=None)
        m = GroupedAttention(0, cfg, 32, sink="learned" if kind == "learned" else "unit", bias_exp=8.0 if kind == "unit" else 0.0)
        m.cache_index = 0
        m.w = {"sink": dev(bf(torch.randn(4, generator=g)), torch.bfloat16)} if kind == "learned" else {}
        T = p0 + n
        pool = _Pool(slots=2, capacity=T + 5, row=m.kv_dim, dtype=torch.bfloat16)
        pool.buf[0, 1, :T] = dev(torch.randn(T, m.kv_dim, generator=g)).to(torch.bfloat16)
        q = dev(torch.randn(n, m.n_q, generator=g))
        ctx = _ctx(eng, pool, [(0, n, 1, p0)])
        rows = pool.buf[0][..., :m.kv_dim]
        a, b = dev(torch.zeros(n, 4 * 24)), dev(torch.zeros(n, 4 * 24))
        with eng.ops.on_stream():
            m._attend_prompt(ctx, q, rows, 1, ctx.pos, a, p0, n)
            m._attend_rows(ctx, q, rows, ctx.slot, ctx.pos, b, prompt=True)
        assert eng.ops.tc_enabled
        assert (host(eng, a) - host(eng, b)).abs().max() < 2e-2


# ------------------------------------------------------------------------------------------------ the model
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_prompt_and_every_layer(dtype):
    cfg = config()
    model, W = build(cfg, dtype)
    toks = tokens(150, cfg["vocab"], 1)
    ref, layers_ref = O.forward(cfg, W, toks, return_layers=True)
    assert close(run_alone(model, toks), ref, dtype)
    if dtype == "float32":
        eng, lm = model.engine, model.language_model
        seen = []
        real = [L.forward for L in model.layers]
        try:
            for L, f in zip(model.layers, real):
                def wrapped(c, xx, f=f, **kw):
                    out = f(c, xx, **kw)
                    seen.append(host(eng, xx))
                    return out
                L.forward = wrapped
            lm.step([toks], [lm.make_cache()])
        finally:
            for L, f in zip(model.layers, real):
                L.forward = f
        assert len(seen) == len(layers_ref) == 5
        for got, want in zip(seen, layers_ref):
            assert (got - want).abs().max() < 3e-5 * max(1.0, want.abs().max().item())


def test_first_tokens():
    cfg = config()
    model, W = build(cfg)
    for n in (1, 2, 3, 4):
        toks = tokens(n, cfg["vocab"], 10 + n)
        assert rel(run_alone(model, toks), O.forward(cfg, W, toks)) < TOL["float32"]
        assert rel(run_alone(model, toks, [1] * n), O.forward(cfg, W, toks)) < TOL["float32"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prefill_then_token_by_token(dtype):
    cfg = config()
    model, W = build(cfg, dtype)
    toks = tokens(110, cfg["vocab"], 2)
    ref = O.forward(cfg, W, toks)
    got = run_alone(model, toks, [50] + [1] * 60)       # both windows pass over decoded tokens
    assert close(got, ref, dtype)
    if dtype == "float32":
        assert rel(got, run_alone(model, toks)) < TOL[dtype]


@pytest.mark.parametrize("cuts", [[2] * 35, [3, 64, 3], [31, 1, 32, 6], [12, 1, 13, 14, 30], [69, 1], [11, 11, 22, 26]])
def test_portions(cuts):
    cfg = config()
    model, W = build(cfg)
    toks = tokens(70, cfg["vocab"], 3)
    assert rel(run_alone(model, toks, cuts), O.forward(cfg, W, toks)) < TOL["float32"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_unequal_batch_against_each_alone(dtype):
    cfg = config()
    model, W = build(cfg, dtype)
    lm, eng = model.language_model, model.engine
    lens = [1, 45, 130, 18]
    reqs = [tokens(n + 12, cfg["vocab"], 20 + n) for n in lens]
    pool = lm.make_pool(4, 64)                       # too short on purpose: it grows under the batch
    caches = [lm.make_cache_row(pool, s) for s in (2, 0, 3, 1)]
    first = host(eng, lm.step([r[:n] for r, n in zip(reqs, lens)], caches, want=[list(range(n)) for n in lens]))
    got = list(torch.split(first, lens))
    for k in range(12):                              # then all go on by one token, together
        step = host(eng, lm.step([[r[n + k]] for r, n in zip(reqs, lens)], caches))
        got = [torch.cat([g, step[i:i + 1]]) for i, g in enumerate(got)]
    for g, r in zip(got, reqs):
        assert close(g, O.forward(cfg, W, r), dtype)
        if dtype == "float32":
            assert rel(g, run_alone(model, r)) < TOL[dtype]


def test_slots_released_and_used_again_and_more_slots():
    from mlx_vlm_b200.models.cache import SlotTable
    cfg = config()
    model, W = build(cfg)
    lm, eng = model.language_model, model.engine
    pool, table = lm.make_pool(2, 64), SlotTable(2)
    a, b, c, d = (tokens(n, cfg["vocab"], 40 + n) for n in (40, 25, 33, 50))
    ca, cb = lm.make_cache_row(pool, table.acquire("a")), lm.make_cache_row(pool, table.acquire("b"))
    lm.step([a[:30], b], [ca, cb])
    table.release("b")                                   # b is finished; c takes its slot (and b's stale rows and state)
    cc = lm.make_cache_row(pool, table.acquire("c"))
    assert cc[0]._row == 1 and cc[0].offset == 0
    got = host(eng, lm.step([a[30:], c], [ca, cc], want=[list(range(10)), list(range(33))]))
    assert rel(got[:10], O.forward(cfg, W, a)[30:]) < TOL["float32"]
    assert rel(got[10:], O.forward(cfg, W, c)) < TOL["float32"]
    with torch.cuda.stream(eng.stream):                  # a third live request: the pool gets more slots
        pool.add_slots(4, live_tokens=pool.capacity)
    table.grow(4)
    cd = lm.make_cache_row(pool, table.acquire("d"))
    assert cd[0]._row == 2
    got = host(eng, lm.step([[a[0]], d], [ca, cd], want=[[], list(range(50))]))
    assert rel(got, O.forward(cfg, W, d)) < TOL["float32"]
    got = host(eng, lm.step([[5]], [cc]))                # c's rows and state survived the move
    assert rel(got, O.forward(cfg, W, c + [5])[-1:]) < TOL["float32"]
    eng.kv_copy_row(pool, 3, pool, 1, cc[0].offset)      # a slot copied to another row (the scheduler's compaction)
    moved = lm.make_cache_row(pool, 3)
    for m in moved:
        m.offset = cc[0].offset
    got = host(eng, lm.step([[9]], [moved]))
    assert rel(got, O.forward(cfg, W, c + [5, 9])[-1:]) < TOL["float32"]


def test_long_prompt_paths_of_the_serving_mode():
    """prompts of 128 tokens and more take the tensor-core products (projections, attention in chunks, the experts as
    grouped products); a long portion after a cached prefix; a batch whose short member stays on the row kernels"""
    cfg = config([layer("attention_2", att2(heads=4, kv_heads=2, dim=16, vdim=16, window=150), moe(experts=8, top=2, ff=32, count=2, keep=1)),
                  layer("wkv", wkv(heads=4, dim=16)),
                  layer("attention", att(heads=4, kv_heads=2, dim=24, vdim=16, dims=16), "dense"),
                  layer("attention_2", att2(heads=2, kv_heads=1, dim=8, vdim=16, window=40, v_mix=False), "dense")], width=64, groups=4)
    model, W = build(cfg, "bfloat16", seed=4)
    exact, _ = build(cfg, "float32", seed=4)
    lm, eng = model.language_model, model.engine
    toks = tokens(400, cfg["vocab"], 9)
    ref = O.forward(cfg, W, toks)
    assert close(run_alone(model, toks), ref, "bfloat16")
    assert close(run_alone(model, toks, [140, 220, 40]), ref, "bfloat16")
    assert rel(run_alone(exact, toks, [140, 220, 40]), ref) < TOL["float32"]
    assert model.engine.ops.tc_enabled
    pool = lm.make_pool(2, 512)
    ca, cb = lm.make_cache_row(pool, 0), lm.make_cache_row(pool, 1)
    both = host(eng, lm.step([toks[:200], toks[:30]], [ca, cb], want=[list(range(200)), list(range(30))]))
    assert close(both[:200], ref[:200], "bfloat16") and close(both[200:], ref[:30], "bfloat16")


def test_long_decoding():
    cfg = config()
    model, W = build(cfg)
    toks = tokens(330, cfg["vocab"], 5)
    got = run_alone(model, toks, [20] + [1] * 310)
    assert rel(got, O.forward(cfg, W, toks)) < TOL["float32"]


OTHER = {
    "recurrent layers first, no feed-forward on the attention, no convolution": config(
        [layer("wkv", wkv(heads=2, dim=20), dense(20)), layer("wkv", wkv(heads=1, dim=36)),
         layer("attention", att(heads=2, kv_heads=2, dim=12, vdim=12, dims=12, scaling=None, v_mix=False), None)], taps=0, groups=1),
    "one head, one group, one expert, one tap, a window of one": config(
        [layer("attention_2", att2(heads=1, kv_heads=1, dim=4, vdim=4, window=1, temp=None, v_mix=False)),
         layer("wkv", wkv(heads=1, dim=8), moe(experts=1, top=1, count=1, keep=1, shared=None)),
         layer("attention", att(heads=1, kv_heads=1, dim=4, vdim=4, dims=2), moe(experts=4, top=4, count=2, keep=2, shared=8))],
        width=40, vocab=37, taps=1, groups=1, mult=1.0),
    "attention first in the value mixing, many kv heads, no window": config(
        [layer("attention", att(heads=4, kv_heads=4, dim=8, vdim=10, dims=4, base=50.0, scaling=(8.0, 16, 2.0, 1.0)), "moe"),
         layer("attention_2", att2(heads=8, kv_heads=4, dim=6, vdim=10, window=0, temp=(1.5, 2)), None),
         layer("attention", att(heads=8, kv_heads=4, dim=10, vdim=10, dims=10), dense(30)),
         layer("attention_2", att2(heads=4, kv_heads=4, dim=12, vdim=10, window=3, v_mix=False), "moe")], width=48, groups=6, taps=5, mult=0.2),
    "wide heads and an odd vocabulary": config(
        [layer("wkv", wkv(heads=1, dim=72), "moe"), layer("attention_2", att2(heads=3, kv_heads=1, dim=40, vdim=72, window=64), "dense")],
        width=72, vocab=257, groups=2, taps=2),
}


@pytest.mark.parametrize("name", sorted(OTHER))
def test_other_sizes(name):
    cfg = OTHER[name]
    model, W = build(cfg, seed=7)
    toks = tokens(75, cfg["vocab"], 6)
    ref = O.forward(cfg, W, toks)
    assert rel(run_alone(model, toks), ref) < TOL["float32"]
    assert rel(run_alone(model, toks, [40] + [1] * 35), ref) < TOL["float32"]
    assert rel(run_alone(model, toks, [7, 2, 66]), ref) < TOL["float32"]
    served, _ = build(cfg, "bfloat16", seed=7)
    assert close(run_alone(served, toks, [40] + [1] * 35), ref, "bfloat16")


# ------------------------------------------------------------------------------------------------ generation
def oracle_greedy(cfg, W, prompt, n):
    toks, margins = list(prompt), []
    for _ in range(n):
        z = O.forward(cfg, W, toks)[-1]
        top2 = torch.topk(z, 2).values
        margins.append(float(top2[0] - top2[1]))
        toks.append(int(torch.argmax(z)))
    return toks[len(prompt):], margins


def same_until_tie(got, want, margins, what):
    for i, (g, w) in enumerate(zip(got, want)):
        if margins[i] < 1e-3:
            return
        assert g == w, f"{what}: token {i} is {g}, the plain implementation says {w}"


def test_greedy_generate_step():
    from mlx_vlm_b200.generate import generate_step
    cfg = config()
    model, W = build(cfg)
    prompt = tokens(21, cfg["vocab"], 8)
    want, margins = oracle_greedy(cfg, W, prompt, 20)       # past two eager steps the step is a replayed graph
    got = [t for t, _ in generate_step(np.asarray([prompt]), model, None, None, max_tokens=20)]
    same_until_tie(got, want, margins, "generate_step")
    from mlx_vlm_b200.sample_utils import make_sampler
    got = [t for t, _ in generate_step(np.asarray([prompt]), model, None, None, max_tokens=6,
                                       sampler=make_sampler(temp=0.0), logit_bias={0: 0.0})]
    same_until_tie(got, want[:6], margins, "generate_step with a sampler")


def test_batch_scheduler_lock_step_rows():
    from mlx_vlm_b200.generate_batch import BatchGenerator
    cfg = config()
    model, W = build(cfg)
    model.config.eos_token_id = []
    prompts = [tokens(n, cfg["vocab"], 60 + n) for n in (5, 30, 12, 44, 9)]
    n_new = [6, 9, 4, 7, 5]
    proc = types.SimpleNamespace(tokenizer=types.SimpleNamespace(stopping_criteria=None))
    g = BatchGenerator(model, proc, completion_batch_size=3, prefill_batch_size=2, decode_slice=2)
    uids = g.insert(prompts, n_new)
    out = {u: [] for u in uids}
    while g.has_work:
        for r in g.next()[1]:
            out[r.uid].append(r.token)
    for u, p, n in zip(uids, prompts, n_new):
        want, margins = oracle_greedy(cfg, W, p, n)
        assert len(out[u]) == n
        same_until_tie(out[u], want, margins, f"row {u}")


def test_trace_runner_from_a_checkpoint_folder(tmp_path):
    """bin/trace_run on a checkpoint folder: the registry picks the class from `architecture`, the decay rank comes from
    the checkpoint's shapes, requests are prefilled together, decoded together, one ends and a later one takes its
    slot; both number formats"""
    import json
    import os
    import subprocess
    import sys
    from safetensors.torch import save_file
    cfg = config()
    W = O.random_weights(cfg, 11, decay_rank=5)
    model_dir = tmp_path / "model"
    model_dir.mkdir()
    (model_dir / "config.json").write_text(json.dumps(cfg))
    save_file({k: v.to(torch.bfloat16).contiguous() for k, v in W.items()}, str(model_dir / "model.safetensors"))
    a, b, c = (tokens(n, cfg["vocab"], 70 + n) for n in (40, 9, 25))
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:30], "want": [0, 29]}, {"id": "b", "tokens": b[:8], "want": [7]}],
              "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[30:31], "want": [0]}, {"id": "b", "tokens": b[8:], "want": [0]}],
              "end": ["b"]},
             {"step": 2, "entries": [{"id": "a", "tokens": a[31:32], "want": []}], "end": []},
             {"step": 3, "entries": [{"id": "a", "tokens": a[32:], "want": [7]}, {"id": "c", "tokens": c, "want": [0, 24]}],
              "end": ["a", "c"]}]
    want = {0: [(a, 0), (a, 29), (b, 7)], 1: [(a, 30), (b, 8)], 3: [(a, 39), (c, 0), (c, 24)]}
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    for dtype in ("bfloat16", "float32"):
        out = tmp_path / dtype
        r = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", str(model_dir), "--dtype", dtype,
                            "--out", str(out), "--max-tokens", "80"], input="".join(json.dumps(x) + "\n" for x in steps),
                           capture_output=True, text=True, timeout=600)
        assert r.returncode == 0, r.stderr[-2000:]
        assert [ln for ln in r.stdout.splitlines() if ln.startswith("done")] == [f"done {i}" for i in range(4)]
        assert not (out / "2.f32").exists()
        for st, rows in want.items():
            got = torch.from_numpy(np.fromfile(out / f"{st}.f32", dtype="<f4").reshape(len(rows), cfg["vocab"])).double()
            ref = torch.stack([O.forward(cfg, W, t)[i] for t, i in rows])
            assert close(got, ref, dtype)
