"""Host-side parts of the Lilosun integration (no GPU): configuration, registry, the packed layout of its blocks against
the checkpoint names, cache rows and state spans of the layers, the frequency table of the scaled rotation, and sanity
properties of the plain restatement the GPU tests compare with."""
import math

import numpy as np
import pytest
import torch

from oracle import lilosun as O


def attn(**kw):
    m = {"heads": 2, "dim": 6, "rot_dim": 4, "vdim": 5, "kv_rank": 8, "mask": {"size": 4}, "scale": 0.3,
         "rot": {"base": 100.0, "dims": 4, "scaling": {"factor": 4.0, "original": 16, "fast": 8.0, "slow": 1.0}}}
    m.update(kw)
    return m


def ssm(**kw):
    m = {"heads": 4, "vdim": 3, "state": 10, "groups": 2, "norm_groups": 2, "conv": 3}
    m.update(kw)
    return m


MOE = {"kind": "moe", "expert": {"ff": 7, "limit": 1.5}, "shared": {"ff": 9, "limit": 2.5},
       "router": {"experts": 6, "top": 2, "groups": {"count": 3, "keep": 2}}}


def config():
    return {"architecture": "Lilosun", "vocab": 29, "width": 20, "norm": {"eps": 1e-4}, "logit_scale": 0.25,
            "layers": [{"type": "mamba2", "mixer": ssm(), "mlp": {"kind": "dense", "ff": 12}},
                       {"type": "latent_attention", "mixer": attn(), "mlp": MOE},
                       {"type": "mamba2", "mixer": ssm(heads=2, state=20, groups=1, norm_groups=1, conv=1), "mlp": None},
                       {"type": "latent_attention", "mixer": attn(kv_rank=5, rot_dim=2, rot={"base": 50.0, "dims": 2}), "mlp": None}]}


def test_config_and_registry():
    from mlx_vlm_b200.models.lilosun import ModelConfig
    from mlx_vlm_b200.utils import get_model_and_args
    c = ModelConfig.from_dict(config())
    assert (c.vocab, c.width, c.norm_eps, c.logit_scale, c.num_hidden_layers) == (29, 20, 1e-4, 0.25, 4)
    assert ModelConfig.from_dict(c.to_dict()).to_dict() == c.to_dict()
    arch, name = get_model_and_args(config())
    assert name == "lilosun" and hasattr(arch, "Model")
    assert ModelConfig.from_dict({"vocab": 3, "width": 2, "layers": []}).logit_scale == 1.0
    with pytest.raises(ValueError):
        ModelConfig.from_dict({"vocab": 3})
    with pytest.raises(ValueError):
        ModelConfig.from_dict({"vocab": 3, "width": 2, "layers": [{"mixer": {}}]})


def test_model_layout_matches_the_checkpoint_names():
    from mlx_vlm_b200.models.decoder_blocks import ScaledPreNormLayer, state_floats
    from mlx_vlm_b200.models.lilosun import Model, ModelConfig
    cfg = config()
    m = Model(ModelConfig.from_dict(cfg), device="cpu")       # no engine is made until something runs
    assert m.checkpoint_tensors() == O.tensor_shapes(cfg)
    L0, L1, L2, L3 = m.layers
    names = dict(m.manifest())
    # everything that reads a layer's input is one stacked product: queries, latent + rotated part, gate
    assert names["l1.mix.down"] == (2 * 10 + 12 + 10, 20) and names["l1.mix.ukT"] == (2, 8, 6)
    assert names["l3.mix.down"] == (2 * 8 + 7 + 10, 20)
    assert names["l0.mix.in"] == (2 * 12 + 2 * 20 + 4, 20) and names["l0.mix.conv"] == (12 + 40, 3)
    assert names["l0.mlp.gu"] == (24, 20)
    # the shared expert's gate row rides with the router; gate and up of every expert are stacked
    assert names["l1.mlp.router"] == (7, 20) and names["l1.mlp.gu"] == (6, 14, 20) and names["l1.mlp.shared.gu"] == (18, 20)
    assert "l2.norm2" not in names and "l2.ls2" not in names and "l3.ls1" in names
    # cache rows of the attention layers, state spans of the state-space layers
    assert m.n_cache_layers == 2 and m.row_dim == 12
    assert (L1.mixer.cache_index, L3.mixer.cache_index) == (0, 1)
    s0, s2 = 2 * 52 + state_floats(4, 10, 3), state_floats(2, 20, 3)
    assert (L0.state_floats, L1.state_floats, L2.state_floats) == (s0, 0, s2)
    assert (L0.mixer.state_off, L2.mixer.state_off, m.state_floats) == (0, s0, s0 + s2)
    assert (L1.mixer.window, L1.mixer.pairs, L1.mixer.gated, L1.mixer.q_rank) == (4, True, True, 0)
    assert L1.mixer.rot_scaling == (4.0, 16.0, 8.0, 1.0) and L3.mixer.rot_scaling is None
    for bad in ({"type": "other", "mixer": {}}, {"type": "mamba2", "mixer": ssm(heads=3), "mlp": None},
                {"type": "mamba2", "mixer": ssm(), "mlp": {"kind": "other"}},
                {"type": "mamba2", "mixer": ssm(), "mlp": dict(MOE, router={"experts": 6, "top": 5, "groups": {"count": 3, "keep": 2}})},
                {"type": "mamba2", "mixer": ssm(), "mlp": dict(MOE, router={"experts": 6, "top": 2, "groups": {"count": 4, "keep": 2}})}):
        with pytest.raises(ValueError):
            ScaledPreNormLayer(0, bad, 20)


def test_packing_stacks_the_projections():
    from mlx_vlm_b200.models.decoder_blocks import ScaledPreNormLayer
    cfg = config()
    W = O.random_weights(cfg, 2)
    L = ScaledPreNormLayer(1, cfg["layers"][1], 20)
    store = {n: torch.zeros(s, dtype=torch.bfloat16) for n, s in L.manifest("l1.")}
    L.pack("l1.", {k: v.bfloat16() for k, v in W.items()}, store.__getitem__)
    p = "l1.mix."
    assert torch.equal(store[p + "down"].float(), torch.cat([W[p + "q"], W[p + "dkv"], W[p + "g"]]))
    assert torch.equal(store[p + "ukT"].float(), W[p + "uk"].view(2, 6, 8).transpose(1, 2))
    f = "l1.mlp."
    assert torch.equal(store[f + "router"].float(), torch.cat([W[f + "router"], W[f + "shared.sg"]]))
    assert torch.equal(store[f + "gu"][4].float(), torch.cat([W[f + "e4.gate"], W[f + "e4.up"]]))
    assert torch.equal(store[f + "down"][5].float(), W[f + "e5.down"])
    assert torch.equal(store[f + "shared.gu"].float(), torch.cat([W[f + "shared.gate"], W[f + "shared.up"]]))
    assert L.w["ls2"] is store["l1.ls2"] and L.ff.shared.w["down"] is store[f + "shared.down"]


def test_scaled_frequencies_of_the_product_and_the_restatement():
    """the host-side table of the product (numpy, double precision) against the restatement's"""
    from mlx_vlm_b200.models.layer_ops import LayerOps
    ops = LayerOps.__new__(LayerOps)          # the table needs no device: catch the upload
    ops._inv_freq = {}
    ops.to_device = lambda arr, dtype=None: torch.from_numpy(np.asarray(arr, dtype=np.float64))
    for base, dims, sc in ((100.0, 4, (4.0, 16, 8.0, 1.0)), (50000.0, 64, (40.0, 4096, 24.0, 2.0)), (10.0, 2, (2.0, 8, 1.0, 1.0)),
                           (500.0, 12, None)):
        want, amp = O.yarn_frequencies(base, dims, None if sc is None else dict(zip(("factor", "original", "fast", "slow"), sc)))
        assert torch.allclose(ops.inv_freq(base, dims, sc), want, rtol=1e-13, atol=0)
        assert abs(LayerOps.rope_amplitude(sc) - amp) < 1e-15
    f, amp = O.yarn_frequencies(50000.0, 64, {"factor": 40.0, "original": 4096, "fast": 24.0, "slow": 2.0})
    plain, _ = O.yarn_frequencies(50000.0, 64, None)
    assert f[0] == plain[0] and abs(f[-1] - plain[-1] / 40.0) < 1e-18 and abs(amp - (0.1 * math.log(40.0) + 1)) < 1e-15
    assert all(plain[i] / 40.0 <= f[i] <= plain[i] for i in range(32))


# ---- the plain restatement itself ---------------------------------------------------------------------------
def test_restatement_is_causal_and_the_window_hides_earlier_keys():
    cfg = config()
    W = O.random_weights(cfg, 3)
    toks = [3, 1, 4, 1, 5, 9, 2, 6, 5, 3, 5, 8]
    full = O.forward(cfg, W, toks)
    assert torch.allclose(full[:7], O.forward(cfg, W, toks[:7]), atol=1e-9)
    ok = O.window_visible(6, 3)
    assert ok[5].tolist() == [False, False, False, True, True, True] and ok[1].tolist() == [True, True, False, False, False, False]
    assert O.window_visible(4, None).sum() == 10
    # attention alone forgets what left its window: two sequences that differ only before it give the same output
    only_attn = {"architecture": "Lilosun", "vocab": 29, "width": 20, "norm": {"eps": 1e-4},
                 "layers": [{"type": "latent_attention", "mixer": attn(), "mlp": None}]}
    W1 = O.random_weights(only_attn, 4)
    a, b = O.forward(only_attn, W1, [1, 2, 3, 4, 5, 6, 7]), O.forward(only_attn, W1, [9, 8, 7, 4, 5, 6, 7])
    assert torch.allclose(a[-1], b[-1], atol=1e-9) and not torch.allclose(a[3], b[3], atol=1e-3)


def test_restatement_router_and_state():
    g = torch.Generator().manual_seed(0)
    z = torch.randn(40, 8, generator=g)
    corr = torch.full((8,), -2.0)                    # every choice score is negative
    idx, w = O.route(z, torch.eye(8), corr, 2, 4, 1)
    assert ((idx[:, 0] // 2) == (idx[:, 1] // 2)).all() and torch.allclose(w.sum(1), torch.ones(40))
    s = torch.sigmoid(z)
    best_group = (s - 2.0).view(40, 4, 2).sum(-1).argmax(-1)
    assert torch.equal(idx[:, 0] // 2, best_group)
    free, _ = O.route(z, torch.eye(8), corr, 2, 1, 1)
    assert torch.equal(torch.sort(free, 1).values, torch.sort(s.topk(2, dim=1).indices, 1).values)
    # one head, a constant step: the state is a geometric sum of the inputs
    T = 6
    x, B, C = torch.ones(T, 1, 1, dtype=torch.float64), torch.ones(T, 1, 1, dtype=torch.float64), torch.ones(T, 1, 1, dtype=torch.float64)
    dt, A = torch.full((T, 1), 0.5, dtype=torch.float64), torch.tensor([2.0], dtype=torch.float64)
    y = O.ssm_walk(x, B, C, dt, A, torch.tensor([3.0], dtype=torch.float64))
    d = math.exp(-1.0)
    assert torch.allclose(y[:, 0, 0], torch.tensor([3.0 + 0.5 * sum(d ** k for k in range(t + 1)) for t in range(T)], dtype=torch.float64))
    u = torch.arange(12.0, dtype=torch.float64).view(6, 2)
    yc = O.causal_conv(u, torch.tensor([[1.0, 10.0], [0.0, 1.0]], dtype=torch.float64), torch.tensor([0.5, 0.0], dtype=torch.float64))
    assert yc[0].tolist() == [0.5, 1.0] and yc[2].tolist() == [2.0 + 40.0 + 0.5, 5.0]
