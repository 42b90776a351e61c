"""Host-side parts of the Vadelix integration (no GPU): configuration, registry, the packed layout of its blocks against
the checkpoint names, cache rows and state spans of the layers, the roles of the value mixing, and sanity properties
of the plain restatement the GPU tests compare with."""
import math

import pytest
import torch

from oracle import vadelix as O


def att(**kw):
    m = {"heads": 4, "kv_heads": 2, "dim": 6, "vdim": 5, "scale": 0.3, "v_mix": True,
         "rot": {"base": 100.0, "dims": 4, "scaling": {"factor": 4.0, "original": 16, "fast": 8.0, "slow": 1.0}}}
    m.update(kw)
    return m


def att2(**kw):
    m = {"heads": 4, "kv_heads": 2, "dim": 4, "vdim": 5, "scale": 0.5, "v_mix": True, "mask": {"size": 3},
         "q_temp": {"coef": 0.5, "every": 4}}
    m.update(kw)
    return m


MOE = {"kind": "moe", "expert": {"ff": 7}, "shared": {"ff": 9}, "router": {"experts": 6, "top": 2, "groups": {"count": 3, "keep": 2}}}


def config():
    return {"architecture": "Vadelix", "vocab": 29, "width": 20, "norm": {"eps": 1e-4, "groups": 5}, "residual_mult": 0.25,
            "canon": {"taps": 3},
            "layers": [{"type": "wkv", "mixer": {"heads": 2, "dim": 10}, "mlp": {"kind": "dense", "ff": 12}},
                       {"type": "attention", "mixer": att(v_mix=False), "mlp": MOE},
                       {"type": "attention_2", "mixer": att2(), "mlp": None},
                       {"type": "attention", "mixer": att(), "mlp": None},
                       {"type": "wkv", "mixer": {"heads": 1, "dim": 12, "decay_rank": 3}, "mlp": None}]}


def test_config_and_registry():
    from mlx_vlm_b200.models.vadelix import ModelConfig
    from mlx_vlm_b200.utils import get_model_and_args
    c = ModelConfig.from_dict(config())
    assert (c.vocab, c.width, c.norm_eps, c.norm_groups, c.residual_mult, c.canon_taps, c.num_hidden_layers) == \
        (29, 20, 1e-4, 5, 0.25, 3, 5)
    assert ModelConfig.from_dict(c.to_dict()).to_dict() == c.to_dict()
    arch, name = get_model_and_args(config())
    assert name == "vadelix" and hasattr(arch, "Model")
    plain = ModelConfig.from_dict({"vocab": 3, "width": 2, "layers": []})
    assert (plain.norm_groups, plain.residual_mult, plain.canon_taps) == (1, 1.0, 0)
    with pytest.raises(ValueError):
        ModelConfig.from_dict({"vocab": 3})
    with pytest.raises(ValueError):
        ModelConfig.from_dict({"vocab": 3, "width": 2, "layers": [{"mixer": {}}]})


def test_model_layout_matches_the_checkpoint_names():
    from mlx_vlm_b200.models.decoder_blocks import ConvPreNormLayer, state_floats
    from mlx_vlm_b200.models.vadelix import Model, ModelConfig
    cfg = config()
    m = Model(ModelConfig.from_dict(cfg), device="cpu")       # no engine is made until something runs
    for L in m.layers:                                        # the rank that a checkpoint's shapes would give
        if hasattr(L.mixer, "set_rank") and "decay_rank" not in cfg["layers"][L.index]["mixer"]:
            L.mixer.set_rank(8)
    assert m.checkpoint_tensors() == O.tensor_shapes(cfg)
    L0, L1, L2, L3, L4 = m.layers
    names = dict(m.manifest())
    # everything that reads the mixer's input is one stacked product
    assert names["l1.mix.qkv"] == (4 * 6 + 2 * 6 + 2 * 5, 20) and names["l2.mix.qkv"] == (4 * 4 + 2 * 4 + 2 * 5, 20)
    assert names["l0.mix.rkvg"] == (4, 20, 20) and names["l0.mix.mu"] == (5, 20) and names["l4.mix.w1"] == (3, 20)
    assert names["l0.mlp.gu"] == (24, 20) and names["l1.mlp.up"] == (6, 7, 20) and names["l1.mlp.shared.down"] == (20, 9)
    assert "l1.mix.sink" in names and "l2.mix.sink" not in names and "l2.mix.q.norm" not in names
    assert "l1.mix.vmix" not in names and names["l2.mix.vmix"] == (1,) and "l2.norm2" not in names
    assert names["l3.canon1"] == (20, 3)
    # cache rows of the attention layers; state spans: [rows of the convolution | previous input | matrix states]
    assert m.n_cache_layers == 3 and m.row_dim == 2 * 6 + 2 * 5
    assert (L1.mixer.cache_index, L2.mixer.cache_index, L3.mixer.cache_index) == (0, 1, 2)
    conv = 2 * 20
    s0, s4 = conv + 20 + state_floats(2, 10, 10), conv + 20 + state_floats(1, 12, 12)
    assert (L0.state_floats, L1.state_floats, L4.state_floats) == (s0, conv, s4)
    assert (L0.state_off, L0.mixer.state_off, L1.state_off, L4.mixer.state_off) == (0, conv, s0, s0 + 3 * conv + conv)
    assert m.state_floats == s0 + 3 * conv + s4
    # the first layer that mixes values keeps them, the later ones blend; a layer that does not say so does neither
    assert (L1.mixer.v_role, L2.mixer.v_role, L3.mixer.v_role) == (None, "first", "blend")
    assert (L2.mixer.window, L2.mixer.q_temp, L2.mixer.sink, L2.mixer.bias_exp, L2.mixer.rot_dims) == (3, (0.5, 4), "unit", 8.0, 0)
    assert (L3.mixer.window, L3.mixer.qk_norm, L3.mixer.v_unit, L3.mixer.sink, L3.mixer.rot_scaling) == \
        (0, True, True, "learned", (4.0, 16.0, 8.0, 1.0))
    for bad in ({"type": "other", "mixer": {}}, {"type": "attention", "mixer": att(heads=3), "mlp": None},
                {"type": "attention", "mixer": att(rot={"base": 10.0, "dims": 8}), "mlp": None},
                {"type": "wkv", "mixer": {"heads": 2, "dim": 10}, "mlp": {"kind": "other"}},
                {"type": "wkv", "mixer": {"heads": 2, "dim": 10}, "mlp": dict(MOE, router={"experts": 6, "top": 5, "groups": {"count": 3, "keep": 2}})},
                {"type": "wkv", "mixer": {"heads": 2, "dim": 10}, "mlp": dict(MOE, router={"experts": 6, "top": 2, "groups": {"count": 4, "keep": 2}})}):
        with pytest.raises(ValueError):
            ConvPreNormLayer(0, bad, 20)
    with pytest.raises(ValueError):
        ConvPreNormLayer(0, cfg["layers"][0], 20, groups=3)
    bad = config()
    bad["layers"][3]["mixer"]["vdim"] = 7                     # values of another size cannot be mixed
    with pytest.raises(ValueError):
        Model(ModelConfig.from_dict(bad), device="cpu")


def test_packing_stacks_the_projections():
    from mlx_vlm_b200.models.decoder_blocks import ConvPreNormLayer
    cfg = config()
    W = O.random_weights(cfg, 2)
    ck = {k: v.bfloat16() for k, v in W.items()}
    L = ConvPreNormLayer(2, cfg["layers"][2], 20, groups=5, mult=0.25, taps=3)
    store = {n: torch.zeros(s, dtype=torch.bfloat16) for n, s in L.manifest("l2.")}
    L.pack("l2.", ck, store.__getitem__)
    p = "l2.mix."
    assert torch.equal(store[p + "qkv"].float(), torch.cat([W[p + "q"], W[p + "k"], W[p + "v"]]))
    assert torch.equal(store[p + "vmix"].float(), W[p + "vmix"].reshape(1))
    assert L.w["canon1"] is store["l2.canon1"] and L.mixer.w["o"] is store[p + "o"]
    L = ConvPreNormLayer(0, cfg["layers"][0], 20, groups=5, taps=3)
    L.mixer.set_rank(8)
    store = {n: torch.zeros(s, dtype=torch.bfloat16) for n, s in L.manifest("l0.")}
    L.pack("l0.", ck, store.__getitem__)
    p = "l0.mix."
    assert torch.equal(store[p + "mu"].float(), torch.stack([W[p + "mu." + s] for s in "rkvgw"]))
    assert torch.equal(store[p + "rkvg"].float(), torch.stack([W[p + s] for s in "rkvg"]))
    assert torch.equal(store["l0.mlp.gu"].float(), torch.cat([W["l0.mlp.gate"], W["l0.mlp.up"]]))
    L = ConvPreNormLayer(1, cfg["layers"][1], 20, groups=5, taps=3)
    store = {n: torch.zeros(s, dtype=torch.bfloat16) for n, s in L.manifest("l1.")}
    L.pack("l1.", ck, store.__getitem__)
    assert torch.equal(store["l1.mlp.up"][4].float(), W["l1.mlp.e4.up"]) and torch.equal(store["l1.mlp.down"][5].float(), W["l1.mlp.e5.down"])
    assert L.ff.shared.w["down"] is store["l1.mlp.shared.down"]


# ---- the plain restatement itself ---------------------------------------------------------------------------
def test_restatement_norm_convolution_and_activations():
    g = torch.Generator().manual_seed(0)
    y = torch.randn(3, 12, generator=g, dtype=torch.float64)
    n = O.group_norm(y, None, 0.0, 4)
    assert torch.allclose((n.view(3, 4, 3) ** 2).mean(-1), torch.ones(3, 4, dtype=torch.float64))
    assert torch.allclose(O.group_norm(y, None, 1e-3, 1), y / torch.sqrt((y * y).mean(-1, keepdim=True) + 1e-3))
    c = torch.zeros(12, 3, dtype=torch.float64)
    c[:, 0] = 2.0                                             # only the oldest tap: h_t + 2 h_(t - 2)
    out = O.input_conv(y, c)
    assert torch.allclose(out[2], y[2] + 2 * y[0]) and torch.allclose(out[1], y[1]) and torch.allclose(out[0], y[0])
    z = torch.linspace(-4, 4, 41, dtype=torch.float64)
    assert torch.allclose(O.gelu_erf(z), torch.nn.functional.gelu(z)) and torch.allclose(O.gelu_tanh(z), torch.nn.functional.gelu(z, approximate="tanh"))
    # the tanh form equals z sigmoid(2 sqrt(2 / pi) (z + 0.044715 z^3)), the form the kernels compute
    assert torch.allclose(O.gelu_tanh(z), z * torch.sigmoid(2 * math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3)), atol=1e-14)


def test_restatement_attention_is_causal_windowed_and_position_dependent():
    cfg = {"architecture": "Vadelix", "vocab": 17, "width": 12, "norm": {"eps": 1e-5, "groups": 2}, "residual_mult": 0.5,
           "canon": {"taps": 2},
           "layers": [{"type": "attention_2", "mixer": att2(heads=2, kv_heads=1, vdim=4, mask={"size": 3}), "mlp": None}]}
    W = O.random_weights(cfg, 1)
    a = [3, 1, 4, 1, 5, 9, 2, 6]
    b = [7] + a[1:]                                            # another first token
    za, zb = O.forward(cfg, W, a), O.forward(cfg, W, b)
    # the window holds 3 tokens and the convolution reaches one further back: from position 4 on nothing of token 0 is left
    assert (za[:4] - zb[:4]).abs().max() > 1e-6 and (za[4:] - zb[4:]).abs().max() < 1e-12
    assert (O.forward(cfg, W, a[:5]) - za[:5]).abs().max() < 1e-12         # causal
    cfg2 = {**cfg, "layers": [{"type": "wkv", "mixer": {"heads": 2, "dim": 4}, "mlp": None}]}
    W2 = O.random_weights(cfg2, 1)
    za, zb = O.forward(cfg2, W2, a), O.forward(cfg2, W2, b)
    assert (za[-1] - zb[-1]).abs().max() > 1e-9                            # the state remembers the first token


def test_restatement_router_keeps_to_the_best_groups():
    g = torch.Generator().manual_seed(4)
    h, router = torch.randn(50, 16, generator=g), torch.randn(12, 16, generator=g)
    idx, w = O.route(h, router, top=3, count=4, keep=2)
    s = torch.softmax(h @ router.T, -1)
    best = s.view(50, 4, 3).max(-1).values.topk(2, -1).indices
    for t in range(50):
        assert all(int(e) // 3 in best[t].tolist() for e in idx[t])
        assert abs(float(w[t].sum()) - 1.0) < 1e-6
    idx1, _ = O.route(h, router, top=3, count=1, keep=1)
    assert all(sorted(idx1[t].tolist()) == sorted(s[t].topk(3).indices.tolist()) for t in range(50))
