"""Lilosun on the GPU against the plain restatement in oracle/lilosun.py: every mechanism alone (with inputs made so
that a fault shows: a key that stands out just inside and just outside the window, at a staging tile's edge and far
back; choice scores that are negative; a state that must survive a step), whole prompts with the residual stream
after every layer, prefill against token-by-token decoding, portions, batches of unequal requests, slots released and
used again, long decoding, other sizes, and greedy generation through generate_step and the batch scheduler.  Small
random configurations; none of them is a real model's."""
import copy
import math
import types

import numpy as np
import pytest
import torch

from oracle import lilosun as O

pytestmark = pytest.mark.gpu
F = torch.nn.functional


# ------------------------------------------------------------------------------------------------ configurations
def attn(heads=3, dim=16, rot_dim=8, vdim=24, kv_rank=40, window=13, base=5000.0, scaling=(4.0, 32, 16.0, 2.0), scale=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "mask": {"size": window},
         "rot": {"base": base, "dims": rot_dim}, "scale": scale if scale is not None else 1.0 / math.sqrt(dim + rot_dim)}
    if scaling:
        m["rot"]["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return m


def ssm(heads=4, vdim=12, state=16, groups=2, norm_groups=2, conv=3):
    return {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "norm_groups": norm_groups, "conv": conv}


def dense(ff=56):
    return {"kind": "dense", "ff": ff}


def moe(experts=8, top=3, ff=24, limit=1.25, count=4, keep=2, shared=(40, 1.75)):
    f = {"kind": "moe", "expert": {"ff": ff, "limit": limit},
         "router": {"experts": experts, "top": top, "groups": {"count": count, "keep": keep}}}
    if shared:
        f["shared"] = {"ff": shared[0], "limit": shared[1]}
    return f


def L_attn(mlp="dense", **kw):
    return {"type": "latent_attention", "mixer": attn(**kw), "mlp": dense() if mlp == "dense" else mlp}


def L_ssm(mlp="moe", **kw):
    return {"type": "mamba2", "mixer": ssm(**kw), "mlp": moe() if mlp == "moe" else mlp}


def config(layers=None, width=72, vocab=101, eps=1e-5, logit_scale=0.7):
    layers = layers or [L_attn(), L_ssm(), L_ssm(mlp=None, heads=3, vdim=8, state=20, groups=1, norm_groups=1, conv=4),
                        L_attn(mlp=moe(experts=6, top=2, count=1, keep=1, shared=None), heads=5, dim=8, rot_dim=12, vdim=8,
                               kv_rank=24, window=40, scaling=None)]
    return {"architecture": "Lilosun", "vocab": vocab, "width": width, "layers": layers, "norm": {"eps": eps},
            "logit_scale": logit_scale}


_MODELS = {}


def build(cfg, dtype="float32", seed=1):
    from mlx_vlm_b200.models.lilosun import Model, ModelConfig
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


class _Pool:
    """what the mixers read of a pool: rows (caching layers, slots, capacity, row) and state (slots, floats)"""

    def __init__(self, slots=3, capacity=0, row=0, state=0, dtype=torch.float32):
        self.buf = torch.zeros((1, slots, max(capacity, 1), max(row, 1)), device="cuda:0", dtype=dtype)
        self.state = torch.full((slots, max(state, 1)), 7.0, device="cuda:0")     # stale numbers: never to be read
        torch.cuda.synchronize()


def _ctx(eng, pool, segments, eps=1e-5):
    """segments: (first row, rows, slot, first position) per sequence"""
    from mlx_vlm_b200.models.decoder_blocks import StepCtx
    T = sum(n for _, n, _, _ in segments)
    slot, pos = np.zeros(T, np.int32), np.zeros(T, np.int32)
    for a, n, s, p0 in segments:
        slot[a:a + n], pos[a:a + n] = s, np.arange(p0, p0 + n)
    return StepCtx(eng.ops, dev(slot, torch.int32), dev(pos, torch.int32), pool, eps, segments)


def test_layer_norm_and_scaled_residual():
    eng = _eng()
    ops = eng.ops
    g = torch.Generator().manual_seed(0)
    T, N = 7, 150
    y = torch.randn(T, N, generator=g) * 3 + 5.0                 # a mean far from zero: a plain RMS norm would differ
    w = (1 + 0.2 * torch.randn(N, generator=g)).bfloat16()
    out = dev(torch.zeros(T, N))
    ops.norm_rows(dev(y), dev(w, torch.bfloat16), 1e-3, out, center=True)
    assert (host(eng, out) - O.layer_norm(y.double(), w.double(), 1e-3)).abs().max() < 1e-5
    rows = dev(np.asarray([4, 0], np.int32), torch.int32)        # gathered rows (the model's norm of the wanted rows)
    two = dev(torch.zeros(2, N))
    ops.norm_rows(dev(y), dev(w, torch.bfloat16), 1e-3, two, center=True, rows=rows)
    assert (host(eng, two) - O.layer_norm(y[[4, 0]].double(), w.double(), 1e-3)).abs().max() < 1e-5
    # x += s * y;  x += s * (sum of weighted rows + sigmoid(gate) * shared row)
    x0, ls = torch.randn(T, N, generator=g), torch.randn(N, generator=g).bfloat16()
    x = dev(x0)
    ops.residual_rows(dev(y), x, dev(ls, torch.bfloat16))
    assert (host(eng, x) - (x0.double() + ls.double() * y.double())).abs().max() < 1e-5
    top = 3
    ye, wg = torch.randn(T * top, N, generator=g), torch.rand(T, top, generator=g)
    sh, sg = torch.randn(T, N + 5, generator=g), torch.randn(T, 9, generator=g)
    x = dev(x0)
    ops.residual_rows(dev(ye), x, dev(ls, torch.bfloat16), combine=dev(wg), top=top, shared=dev(sh)[:, 5:], shared_gate=dev(sg)[:, 8:])
    want = x0.double() + ls.double() * ((ye.double().view(T, top, N) * wg.double()[:, :, None]).sum(1)
                                        + torch.sigmoid(sg[:, 8:].double()) * sh[:, 5:].double())
    assert (host(eng, x) - want).abs().max() < 1e-5
    # the same update and the norm of the updated rows in one launch; few rows and many (two block sizes)
    for rows in (T, 70):
        xr, yr = torch.randn(rows, N, generator=g) + 2.0, torch.randn(rows * top, N, generator=g)
        wr, shr, sgr = torch.rand(rows, top, generator=g), torch.randn(rows, N, generator=g), torch.randn(rows, 1, generator=g)
        x, n = dev(xr), dev(torch.zeros(rows, N))
        ops.residual_norm_rows(dev(yr), x, dev(ls, torch.bfloat16), dev(w, torch.bfloat16), 1e-3, n, center=True, combine=dev(wr),
                               top=top, shared=dev(shr), shared_gate=dev(sgr))
        want = xr.double() + ls.double() * ((yr.double().view(rows, top, N) * wr.double()[:, :, None]).sum(1)
                                            + torch.sigmoid(sgr.double()) * shr.double())
        assert (host(eng, x) - want).abs().max() < 1e-5
        assert (host(eng, n) - O.layer_norm(want, w.double(), 1e-3)).abs().max() < 2e-5
        x, n = dev(xr), dev(torch.zeros(rows, N))
        ops.residual_norm_rows(dev(shr), x, None, dev(w, torch.bfloat16), 1e-3, n, center=True)
        assert (host(eng, n) - O.layer_norm(xr.double() + shr.double(), w.double(), 1e-3)).abs().max() < 2e-5


@pytest.mark.parametrize("scaling", [None, (4.0, 32, 16.0, 2.0), (16.0, 4096, 32.0, 1.0), (2.0, 8, 1.0, 1.0)])
@pytest.mark.parametrize("dims,width", [(8, 8), (6, 10), (2, 2)])
def test_rotation_in_pairs_with_scaled_frequencies(scaling, dims, width):
    """the rotated key part of the cached row and the rotated query parts, at the first positions and far out"""
    eng = _eng()
    ops = eng.ops
    g = torch.Generator().manual_seed(dims)
    H, dn, r, base = 3, 5, 7, 300.0
    pos = torch.tensor([0, 1, 2, 31, 32, 33, 1000, 99999])
    T = len(pos)
    sc = None if scaling is None else dict(zip(("factor", "original", "fast", "slow"), scaling))
    f, amp = O.yarn_frequencies(base, dims, sc)
    got_f = host(eng, ops.inv_freq(base, dims, scaling))
    assert (got_f - f).abs().max() < 1e-12 * f.abs().max() and abs(ops.rope_amplitude(scaling) - amp) < 1e-12
    if scaling is not None and scaling[0] > 2:
        assert (f - O.yarn_frequencies(base, dims, None)[0]).abs().max() > 0 or dims == 2
    cs = ops.rope_table(dev(pos, torch.int32), base, dims, scaling)
    D = torch.randn(T, r + width, generator=g)
    wkv = (1 + 0.1 * torch.randn(r, generator=g)).bfloat16()
    pool = _Pool(slots=2, capacity=100000, row=r + width)
    ops.latent_post(dev(D), None, dev(wkv, torch.bfloat16), 1e-4, None, pool.buf[0], dev(np.ones(T), torch.int32),
                    dev(pos, torch.int32), cs, 0, r, width, dims, pairs=True)
    rows = host(eng, pool.buf[0][1][pos])
    assert (rows[:, :r] - O.rms(D[:, :r].double(), 1e-4) * wkv.double()).abs().max() < 1e-5
    want = O.rotate_pairs(D[:, None, r:].double(), pos, base, dims, sc)[:, 0]
    assert (rows[:, r:] - want).abs().max() < 2e-5
    q = torch.randn(T, H, dn + width, generator=g)
    qa = dev(torch.zeros(T, H * (r + width)))
    ops.rope_q(dev(q.reshape(T, -1)), qa, cs, H, dn, width, dims, r, pairs=True)
    got = host(eng, qa).view(T, H, r + width)[..., r:]
    assert (got - O.rotate_pairs(q[..., dn:].double(), pos, base, dims, sc)).abs().max() < 2e-5


def _latent_rows(S, r, dr, seed):
    g = torch.Generator().manual_seed(seed)
    return F.normalize(torch.randn(S, r + dr, generator=g), dim=-1), g


def _plain_window(rows, q, r, scale, window):
    """every query t at position t over the rows: the rows are the keys of all heads, their first r numbers the values"""
    S, H = q.shape[0], q.shape[1]
    k = rows.double()[:, None, :].expand(S, H, -1)
    return O.window_attention(q.double(), k, k[..., :r], scale, window)


@pytest.mark.parametrize("window", [1, 2, 31, 32, 33, 100, 1000])
@pytest.mark.parametrize("r,dr", [(24, 8), (21, 5)])
def test_window_of_visible_keys(window, r, dr):
    """head 1 of every query points at the key just OUTSIDE its window, then at the first key INSIDE it: a prompt
    (many queries in a launch), and single queries with the keys split over several blocks"""
    eng = _eng()
    ops = eng.ops
    H, S, slot = 3, 300, 1
    rows, g = _latent_rows(S, r, dr, window)
    pool = _Pool(slots=2, capacity=S + 5, row=r + dr + 3)
    layer = pool.buf[0][..., :r + dr]
    layer[slot, :S] = dev(rows)
    layer[slot, S:] = 50.0                          # rows past the sequence: never to be seen
    pos, sl = dev(np.arange(S), torch.int32), dev(np.full(S, slot), torch.int32)
    for inside in (False, True):
        q = torch.randn(S, H, r + dr, generator=g) * 0.2
        for p in range(S):
            key = p - window + (1 if inside else 0)
            if key >= 0:
                q[p, 1] = rows[key] * 100.0
        want = _plain_window(rows, q, r, 1.0, window)
        out = dev(torch.zeros(S, H * r))
        ops.latent_attention(dev(q.reshape(S, -1)), layer, sl, pos, out, H, r, 1.0, n_split=1, window=window)
        got = host(eng, out).view(S, H, r)
        assert (got - want).abs().max() < 2e-5
        for p in (S - 1, window, 150):
            key = p - window + (1 if inside else 0)
            if not 0 <= key < S or p >= S:
                continue
            hit = (got[p, 1] - rows[key, :r].double()).abs().max()
            assert (hit < 1e-3) if inside else (hit > 0.02)
            for split in (None, 1, 4, 64):
                one = dev(torch.zeros(1, H * r))
                ops.latent_attention(dev(q[p:p + 1].reshape(1, -1)), layer, sl[p:p + 1], pos[p:p + 1], one, H, r, 1.0,
                                     n_split=split, window=window)
                assert (host(eng, one).view(H, r) - want[p]).abs().max() < 2e-5


def test_far_key_without_a_window_and_at_tile_edges():
    eng = _eng()
    ops = eng.ops
    H, S, r, dr, slot = 2, 700, 16, 8, 0
    rows, g = _latent_rows(S, r, dr, 3)
    pool = _Pool(slots=1, capacity=S, row=r + dr)
    pool.buf[0][slot, :S] = dev(rows)
    for key in (0, 31, 32, 33, 64, 350, 698):
        for p in (key, key + 1, 699):
            q = torch.randn(1, H, r + dr, generator=g) * 0.2
            q[0, 1] = rows[key] * 100.0
            for window, seen in ((0, True), (p - key + 1, True), (p - key, p == key)):
                out = dev(torch.zeros(1, H * r))
                ops.latent_attention(dev(q.reshape(1, -1)), pool.buf[0], dev([slot], torch.int32), dev([p], torch.int32), out,
                                     H, r, 1.0, window=window)
                hit = (host(eng, out).view(H, r)[1] - rows[key, :r].double()).abs().max()
                assert (hit < 1e-3) if seen else (hit > 0.02), (key, p, window)


@pytest.mark.parametrize("window,p0,n", [(40, 0, 300), (150, 0, 330), (150, 70, 260), (128, 5, 256), (1000, 0, 200), (0, 30, 170)])
def test_prompt_attention_on_the_tensor_cores_keeps_the_window(window, p0, n):
    """the two-product form of a long portion (serving mode): chunks of queries against the rows from the chunk's
    first visible key on; a crafted key just outside every query's window gets no weight, the one just inside all"""
    from mlx_vlm_b200.models.decoder_blocks import LatentAttention
    eng = _eng(exact=False)
    ops = eng.ops
    H, r, dr = 3, 32, 8
    S = p0 + n
    rows, g = _latent_rows(S, r, dr, window + n)
    rows = rows.bfloat16().float()
    m = LatentAttention(0, {"heads": H, "dim": 8, "rot_dim": dr, "vdim": 8, "kv_rank": r, "scale": 1.0,
                            "mask": {"size": window} if window else None}, 64, rotation="pairs", gated=True)
    pool = _Pool(slots=2, capacity=S + 8, row=r + dr, dtype=torch.bfloat16)
    pool.buf[0][1, :S] = dev(rows, torch.bfloat16)
    pos = dev(np.arange(p0, S), torch.int32)
    for inside in (False, True):
        q = torch.randn(S, H, r + dr, generator=g) * 0.2
        for p in range(S):
            key = p - window + (1 if inside else 0) if window else (0 if inside else p + 1)
            if 0 <= key < S:
                q[p, 1] = rows[key] * 60.0
        q = q.bfloat16().float()
        want = _plain_window(rows, q, r, 1.0, window or None)[p0:]
        ol = dev(torch.zeros(n, H * r))
        with ops.on_stream():
            m._attend_prompt(ops, dev(q[p0:].reshape(n, -1)), pool.buf[0][1], pos, ol, p0, n)
        got = host(eng, ol).view(n, H, r)
        assert (got - want).abs().max() < 2e-2
        if window and window < S:
            p = S - 1
            hit = (got[p - p0, 1] - rows[p - window + (1 if inside else 0), :r].double()).abs().max()
            assert (hit < 2e-2) if inside else (hit > 0.05)


@pytest.mark.parametrize("E,top,count,keep", [(8, 3, 4, 2), (12, 2, 3, 1), (6, 6, 1, 1), (6, 2, 6, 3), (16, 4, 2, 2), (5, 1, 5, 1),
                                              (64, 6, 8, 3), (70, 5, 1, 1)])
def test_router_with_groups(E, top, count, keep):
    """choice scores are negative for many experts (a correction far below zero), so an expert outside the kept groups
    that counted as zero instead of minus infinity would be chosen"""
    eng = _eng()
    ops = eng.ops
    g = torch.Generator().manual_seed(E + top)
    T = 50
    z = torch.randn(T, E + 2, generator=g) * 2
    corr = (torch.randn(E, generator=g) * 0.5 - 1.5).bfloat16()
    idx, wgt = ops.router_group_topk(dev(z), top, dev(corr, torch.bfloat16), count, keep, E=E)
    # the restatement takes a weight matrix: the identity makes its logits the given z
    ri, rw = O.route(z[:, :E], torch.eye(E), corr.float(), top, count, keep)
    gi, gw = host(eng, idx).long(), host(eng, wgt)
    order = torch.argsort(gi, dim=1)
    rorder = torch.argsort(ri, dim=1)
    assert torch.equal(torch.gather(gi, 1, order), torch.gather(ri, 1, rorder))
    assert (torch.gather(gw, 1, order) - torch.gather(rw.double(), 1, rorder)).abs().max() < 1e-6
    assert (gw.sum(1) - 1).abs().max() < 1e-5
    if count > keep:
        per = E // count
        assert all(len({int(e) // per for e in row}) <= keep for row in gi)


@pytest.mark.parametrize("taps", [1, 2, 4])
def test_convolution_with_bias(taps):
    eng = _eng()
    C, cuts = 37, [2, 1, 3, 24]
    T = sum(cuts)
    g = torch.Generator().manual_seed(taps)
    u = torch.randn(2, T, C + 3, generator=g)
    w, b = torch.randn(C, taps, generator=g).bfloat16(), torch.randn(C, generator=g).bfloat16()
    pool = _Pool(slots=3, state=(taps - 1) * C + 6)
    st = pool.state[:, 5:5 + max((taps - 1) * C, 1)]
    got, at = [[], []], [0, 0]
    for na, nb in zip(cuts, cuts[::-1]):
        segs = [(0, na, 2, at[0]), (na, nb, 0, at[1])]
        rows = dev(torch.cat([u[0, at[0]:at[0] + na], u[1, at[1]:at[1] + nb]]))
        y = host(eng, eng.ops.short_conv(rows[:, 3:], dev(w, torch.bfloat16), st, _ctx(eng, pool, segs), act=True,
                                         bias=dev(b, torch.bfloat16)))
        got[0].append(y[:na])
        got[1].append(y[na:])
        at = [at[0] + na, at[1] + nb]
    for i in (0, 1):
        want = F.silu(O.causal_conv(u[i, :, 3:].double(), w.double(), b.double()))
        assert (torch.cat(got[i]) - want).abs().max() < 1e-5


@pytest.mark.parametrize("N,P,H,G", [(16, 12, 4, 2), (20, 8, 3, 1), (64, 40, 2, 2), (128, 64, 2, 1), (8, 130, 1, 1), (100, 24, 6, 3)])
def test_state_space_walk_in_portions_and_slots(N, P, H, G):
    """S <- exp(-A dt) S + dt B x^T, y = S^T C + D x: the state survives from step to step in its slot, a slot that held
    another sequence starts anew; a step size near zero keeps an old input alive for hundreds of tokens"""
    eng = _eng()
    ops = eng.ops
    from mlx_vlm_b200.models.decoder_blocks import state_floats
    T = 45
    g = torch.Generator().manual_seed(N + P)
    x = torch.randn(T, H, P, generator=g)
    B, C = torch.randn(T, G, N, generator=g), torch.randn(T, G, N, generator=g)
    a = torch.randn(T, H, generator=g)
    A_log = torch.log(0.5 + 2 * torch.rand(H, generator=g)).bfloat16()
    dtb = (torch.randn(H, generator=g) - 1).bfloat16()
    Dk = (1 + 0.3 * torch.randn(H, generator=g)).bfloat16()
    dt = F.softplus(a.double() + dtb.double())
    per = H // G
    want = O.ssm_walk(x.double(), B.double().repeat_interleave(per, 1), C.double().repeat_interleave(per, 1), dt,
                      torch.exp(A_log.double()), Dk.double())
    floats = state_floats(H, N, P)
    pool = _Pool(slots=3, state=floats + 3)
    st = pool.state[:, 3:3 + floats]
    for cuts in ([T], [1] * 6 + [17, 2, 20], [20, 25]):
        got, at = [], 0
        for n in cuts:
            ctx = _ctx(eng, pool, [(0, n, 1, at)])
            o = dev(torch.zeros(n, H * P))
            sl = slice(at, at + n)
            ops.linear_state(dev(C[sl].reshape(n, -1)), dev(B[sl].reshape(n, -1)), dev(x[sl].reshape(n, -1)), o, st, ctx,
                             H=H, rep=per, dim=N, vdim=P, a=dev(a[sl]), A_log=dev(A_log, torch.bfloat16),
                             dt_bias=dev(dtb, torch.bfloat16), dt_in=True, skip=dev(Dk, torch.bfloat16))
            got.append(host(eng, o).view(n, H, P))
            at += n
        err = (torch.cat(got) - want).abs().max() / want.abs().max()
        assert err < 2e-5, (cuts, err)


def test_gate_before_the_group_norm_and_plain_gated_unit():
    eng = _eng()
    ops = eng.ops
    g = torch.Generator().manual_seed(2)
    T, H, dv = 5, 4, 18
    o, z = torch.randn(T, H * dv, generator=g) * 3, torch.randn(T, H * dv + 2, generator=g)
    w = (1 + 0.2 * torch.randn(H * dv, generator=g)).bfloat16()
    for groups in (1, 2, 4):
        out = dev(o)
        ops.head_post(out, out, dv=dv, gate=dev(z)[:, 2:], gate_silu=True, w=dev(w, torch.bfloat16), eps=1e-3,
                      span=H * dv // groups, gate_first=True)
        y = o.double() * F.silu(z[:, 2:].double())
        want = O.rms(y.view(T, groups, -1), 1e-3).reshape(T, -1) * w.double()
        assert (host(eng, out) - want).abs().max() < 1e-5
        after = O.rms(o.double().view(T, groups, -1), 1e-3).reshape(T, -1) * w.double() * F.silu(z[:, 2:].double())
        assert (want - after).abs().max() > 0.1                      # the order matters
    # few tokens with long groups: a whole block per group
    big, zb, wb = torch.randn(2, 1536, generator=g) * 2, torch.randn(2, 1536, generator=g), torch.randn(1536, generator=g).bfloat16()
    for groups in (1, 3, 6):
        out = dev(torch.zeros(2, 1536))
        ops.head_post(dev(big), out, dv=64, gate=dev(zb), gate_silu=True, w=dev(wb, torch.bfloat16), eps=1e-5, span=1536 // groups,
                      gate_first=True)
        want = O.rms((big.double() * F.silu(zb.double())).view(2, groups, -1), 1e-5).reshape(2, -1) * wb.double()
        assert (host(eng, out) - want).abs().max() < 1e-5
    a, b = torch.randn(T, 300, generator=g) * 3, torch.randn(T, 300, generator=g) * 3
    y = dev(torch.zeros(T, 300))
    ops.glu_clamp(dev(a), dev(b), float("inf"), 1.0, y, up_offset=0.0)
    assert (host(eng, y) - F.silu(a.double()) * b.double()).abs().max() < 1e-5
    wide = dev(torch.cat([a, b], dim=1))                                 # the same as bf16 operand rows, zero-padded
    yb = ops.glu_clamp_bf16(wide[:, :300], wide[:, 300:], 1.25, 1.702, up_offset=1.0)
    gg, uu = a.double().clamp(max=1.25), b.double().clamp(-1.25, 1.25)
    want = (gg * torch.sigmoid(1.702 * gg) * (uu + 1)).float().bfloat16().double()
    got = host(eng, yb)
    assert got.shape == (T, 320) and got[:, 300:].abs().max() == 0
    assert ((got[:, :300] - want).abs() <= 2.0 ** -7 * want.abs() + 1e-6).all()
    live = dev(np.asarray([0, -1, 7, -1, 2], np.int32), torch.int32)      # padding rows become zeros, their inputs may hold anything
    junk = wide.clone()
    junk[1], junk[3] = float("nan"), float("inf")
    masked = host(eng, ops.glu_clamp_bf16(junk[:, :300], junk[:, 300:], 1.25, 1.702, up_offset=1.0, live=live))
    assert torch.equal(masked[[0, 2, 4]], got[[0, 2, 4]]) and masked[[1, 3]].abs().max() == 0
    odd = host(eng, ops.glu_clamp_bf16(wide[:, 1:78], wide[:, 301:378], 1.25, 1.702, up_offset=1.0))    # rows that are no vectors
    assert odd.shape == (T, 128) and torch.equal(odd[:, :77], got[:, 1:78]) and odd[:, 77:].abs().max() == 0


@pytest.mark.parametrize("K", [64, 100, 77])
def test_operand_rows_gathered_and_scattered(K):
    """fp32 rows -> bf16 operand rows through a row map with padding entries, and product rows back to entry order"""
    eng = _eng()
    ops = eng.ops
    g = torch.Generator().manual_seed(K)
    x = torch.randn(9, K + 4, generator=g)
    order = np.asarray([5, -1, 0, 17, 16, -1, -1, 3], np.int32)           # entry e reads row e // 2
    xb = host(eng, ops.to_bf16(dev(x)[:, 4:], K, rows=8, row_map=dev(order, torch.int32), div=2))
    Kp = (K + 63) // 64 * 64
    assert xb.shape == (8, Kp)
    for i, e in enumerate(order):
        want = torch.zeros(Kp, dtype=torch.float64) if e < 0 else F.pad(x[e // 2, 4:].bfloat16().double(), (0, Kp - K))
        assert torch.equal(xb[i], want)
    y = torch.randn(8, K, generator=g)
    out = dev(torch.full((18, K + 4), -5.0))
    ops.rows_scatter(dev(y), dev(order, torch.int32), out[:, 4:], 8)
    got = host(eng, out)[:, 4:]
    for i, e in enumerate(order):
        if e >= 0:
            assert torch.equal(got[e], y[i].double())
    untouched = [r for r in range(18) if r not in set(order.tolist())]
    assert (got[untouched] == -5.0).all()


def test_logits_times_a_constant():
    from mlx_vlm_b200.models.layer_ops import EPI_SCALE
    eng = _eng()
    g = torch.Generator().manual_seed(4)
    for M in (1, 5, 40):
        x, W = torch.randn(M, 48, generator=g), (torch.randn(70, 48, generator=g) / 7).bfloat16()
        z = eng.ops.linear(dev(x), dev(W, torch.bfloat16), epi=EPI_SCALE, epi_param=0.37)
        assert (host(eng, z) - 0.37 * (x.double() @ W.double().T)).abs().max() < 1e-5


@pytest.mark.parametrize("M", [3, 40, 130, 300])
def test_router_product_keeps_its_input_unrounded_in_the_serving_mode(M):
    """few rows: fp32 rows on the row kernels; a long step: [hi | lo] halves on the tensor cores (2^-17 of the input)"""
    eng = _eng(exact=False)
    g = torch.Generator().manual_seed(M)
    K, N_ = 72, 9
    x = torch.randn(M, K + 4, generator=g) * 3
    W = (torch.randn(N_, K, generator=g) / 8).bfloat16()
    xd = dev(x)
    want = x[:, 4:].double() @ W.double().T
    with eng.ops.on_stream():
        z = eng.ops.linear(xd[:, 4:], dev(W, torch.bfloat16), exact_x=True)
        rounded = eng.ops.linear(xd[:, 4:], dev(W, torch.bfloat16))
    assert (host(eng, z) - want).abs().max() < 2e-4
    assert (host(eng, rounded) - want).abs().max() > 2e-3          # one rounded part is two orders further off
    assert eng.ops.tc_enabled


# ------------------------------------------------------------------------------------------------ the model
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_prompt_and_every_layer(dtype):
    cfg = config()
    model, W = build(cfg, dtype)
    toks = tokens(150, cfg["vocab"], 1)
    layers_ref = []
    ref = O.forward(cfg, W, toks, torch.float64, layers_ref)
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
        assert len(seen) == len(layers_ref) == 4
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
        assert close(run_alone(model, toks, [1] * 110), ref, dtype)


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
    """prompts of 128 tokens and more take the tensor-core products (projections, windowed attention in chunks, the
    experts as grouped products); a long portion after a cached prefix; a batch whose short member stays on the row
    kernels"""
    cfg = config([L_attn(heads=4, dim=16, rot_dim=8, vdim=16, kv_rank=32, window=150), L_ssm(heads=4, vdim=16, state=16),
                  L_attn(mlp=moe(experts=8, top=2, ff=32, count=2, keep=1), heads=2, dim=24, rot_dim=16, vdim=8, kv_rank=64,
                         window=40)], width=64)
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
    "state-space layers first, no feed-forward on the attention": config(
        [L_ssm(mlp=dense(20)), L_ssm(heads=2, vdim=20, state=24, groups=2, norm_groups=1, conv=2), L_attn(mlp=None, window=5)]),
    "one head, one group, one expert": config(
        [L_attn(heads=1, window=1), L_ssm(heads=1, groups=1, norm_groups=1, conv=1, mlp=moe(experts=1, top=1, count=1, keep=1)),
         L_attn(mlp=moe(experts=4, top=4, count=2, keep=2, shared=(8, 0.5)), heads=1, dim=4, rot_dim=2, vdim=4, kv_rank=4)],
        width=40, vocab=37, logit_scale=1.0),
    "equal sizes": config(
        [L_attn(heads=2, dim=32, rot_dim=32, vdim=32, kv_rank=32, window=32, base=32.0, scaling=(32.0, 32, 32.0, 1.0), scale=1 / 32),
         L_ssm(heads=2, vdim=32, state=32, groups=2, norm_groups=2, conv=2, mlp=moe(experts=2, top=2, ff=32, limit=2.0, count=2, keep=2, shared=(32, 2.0)))],
        width=32, vocab=32, logit_scale=2.0),
    "odd sizes, a window longer than the sequence, groups of one expert": config(
        [L_attn(heads=7, dim=9, rot_dim=6, vdim=11, kv_rank=19, window=500, base=123.0, scaling=(3.0, 20, 4.0, 0.5)),
         L_ssm(heads=6, vdim=7, state=9, groups=3, norm_groups=3, conv=5, mlp=moe(experts=9, top=3, ff=13, limit=0.4, count=9, keep=4, shared=(7, 3.0))),
         L_ssm(heads=2, vdim=80, state=136, groups=1, norm_groups=2, conv=2, mlp=dense(31))], width=50, vocab=61, eps=1e-3),
    "many heads and experts": config(
        [L_attn(heads=12, dim=8, rot_dim=4, vdim=8, kv_rank=16, window=7, mlp=moe(experts=40, top=5, ff=8, count=5, keep=2)),
         L_ssm(heads=8, vdim=8, state=8, groups=4, norm_groups=4, conv=3, mlp=None)], width=48),
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
    """bin/trace_run on a checkpoint folder: the registry picks the class from `architecture`, requests are prefilled
    together, decoded together, one ends and a later one takes its slot; both number formats"""
    import json
    import os
    import subprocess
    import sys
    from safetensors.torch import save_file
    cfg = config()
    W = O.random_weights(cfg, 11)
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
