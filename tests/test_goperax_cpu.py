"""Goperax without a GPU: the configuration reader and what it refuses, the tensor table, the C description, the oracle's
mechanisms against values worked out by hand, and that the oracle reacts to every constant the GPU tests rely on."""
import json

import numpy as np
import pytest

from distributed_inference_server_b200 import binding as B
from distributed_inference_server_b200 import models
from tests import _goperax_util as U
from tests import goperax_oracle as GO

LAYERS = [(U.attention(), U.dense()), (U.ssm(), U.moe()), (U.ssm(heads=6, vdim=4, state=5, groups=3, conv=2, norm_groups=1), None),
          (U.attention(heads=3, kv_heads=3, dim=10, window=0, softcap=0), U.moe(experts=3, top=3, shared=0))]


def test_reader_takes_every_size_and_constant_from_the_file():
    cfg = U.config(LAYERS, vocab=77, width=40, eps=3e-4, streams=5, loop=(1, 3, 4), embed_scale=2.5)
    sp = models.goperax_spec(cfg)
    assert (sp.name, sp.vocab, sp.width, sp.norm_eps, sp.streams, sp.loop, sp.embed_scale) == ("Goperax", 77, 40, 3e-4, 5, (1, 3, 4), 2.5)
    assert sp.pre_norm and sp.pos_sinus and sp.loop_plain and sp.tied_head and sp.norm_kind == "rms"
    a, s, s2, a2 = sp.layers
    assert (a.mixer, a.heads, a.kv_heads, a.dim, a.vdim, a.mask_window, a.score_softcap) == ("attention", 4, 2, 8, 8, 24, 12.0)
    assert a.attn_flags == B.ATTN_V_IS_K | B.ATTN_SINK_UNIT and a.rot_dims == 0
    assert (a.mlp, a.ff, a.mlp_act, a.gated) == ("dense", 40, "relu2", False)
    assert (s.mixer, s.heads, s.vdim, s.ssm_state, s.ssm_groups, s.conv_taps, s.ssm_norm_groups) == ("ssm", 4, 6, 8, 2, 3, 2)
    assert (s.mlp, s.experts, s.top, s.ff, s.shared_ff, s.shared_plain, s.route) == ("moe", 6, 2, 10, 14, True, "softmax_all")
    assert s2.mlp == "none" and (s2.ssm_groups, s2.conv_taps, s2.ssm_norm_groups) == (3, 2, 1)
    assert (a2.mask_window, a2.score_softcap, a2.shared_ff, a2.top) == (0, 0.0, 0, 3)
    assert sp.layer_runs() == [0, 1, 2, 1, 2, 1, 2, 1, 2, 3]
    assert models.read_config.__module__  # the registry names the design
    assert models.ARCHITECTURES["Goperax"][1] is models.goperax_spec


def test_reader_without_optional_parts():
    cfg = U.config(LAYERS[:2], streams=0)
    del cfg["embedding"]
    sp = models.goperax_spec(cfg)
    assert sp.streams == 0 and sp.loop == (0, 0, 0) and sp.embed_scale == 1.0
    assert not any(".hc" in n for n in sp.tensor_shapes())


@pytest.mark.parametrize("edit,msg", [
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "multiple of kv_heads"),
    (lambda c: c["layers"][0]["mixer"].update(vdim=9), "vdim must equal dim"),
    (lambda c: c["layers"][1]["mixer"].update(groups=3), "multiple of groups"),
    (lambda c: c["layers"][1]["mixer"].update(norm_groups=5), "norm_groups"),
    (lambda c: c["layers"][1].update(type="lstm"), "unknown mixer"),
    (lambda c: c["layers"][1]["mlp"].update(kind="glu"), "unknown feed-forward"),
    (lambda c: c.update(loop={"start": 2, "stop": 2, "times": 2}), "loop"),
])
def test_reader_refuses(edit, msg):
    cfg = U.config(LAYERS)
    edit(cfg)
    with pytest.raises(ValueError, match=msg):
        models.goperax_spec(cfg)


def test_tensor_table():
    cfg = U.config(LAYERS, vocab=77, width=40, streams=5)
    t = models.goperax_spec(cfg).tensor_shapes()
    assert "head" not in t and "loop.in" not in t and t["embed"] == (77, 40) and t["final.norm"] == (40,)
    assert t["l0.mix.q"] == (32, 40) and t["l0.mix.k"] == (16, 40) and t["l0.mix.o"] == (40, 32) and "l0.mix.v" not in t and "l0.mix.sink" not in t
    assert t["l0.mlp.up"] == (40, 40) and t["l0.mlp.down"] == (40, 40) and "l0.mlp.gate" not in t
    assert "l0.norm1b" not in t and "l0.norm2b" not in t and t["l0.norm2"] == (40,)
    assert t["l0.hc1.in"] == (5,) and t["l0.hc2.out"] == (5,) and t["l0.hc2.mix"] == (5, 5)
    # z | x | B | C | dt rows of the input projection; the convolution covers x | B | C
    assert t["l1.mix.in"] == (2 * 24 + 2 * 16 + 4, 40) and t["l1.mix.conv"] == (24 + 32, 3) and t["l1.mix.conv.b"] == (56,)
    assert t["l1.mix.dt_bias"] == t["l1.mix.A_log"] == t["l1.mix.D"] == (4,) and t["l1.mix.norm"] == (24,) and t["l1.mix.o"] == (40, 24)
    assert t["l1.mlp.router"] == (6, 40) and t["l1.mlp.e5.up"] == (10, 40) and t["l1.mlp.shared.down"] == (40, 14)
    assert "l1.mlp.shared.sg" not in t and "l1.mlp.e0.gate" not in t and "l1.mlp.correction" not in t
    assert "l2.norm2" not in t and "l2.hc2.in" not in t and "l3.mlp.shared.up" not in t
    W = U.weights(cfg)
    assert set(W) == set(t) and all(W[k].shape == tuple(v) for k, v in t.items())


def test_c_description_carries_the_new_fields():
    cfg = U.config(LAYERS, streams=5, loop=(1, 3, 2))
    sc, keep = models.goperax_spec(cfg).c(256, 16, True)
    assert sc.frame_flags == B.FRAME_PRE_NORM | B.FRAME_POS_SINUS | B.FRAME_LOOP_PLAIN | B.FRAME_TIED_HEAD
    assert sc.streams == 5 and sc.pos_base == 10000.0 and (sc.loop_start, sc.loop_stop, sc.loop_times) == (1, 3, 2)
    a, s = sc.layers[0], sc.layers[1]
    assert (a.mixer, a.mask_window, a.score_softcap, a.mlp_act, a.mask_chunk) == (B.MIX_ATTENTION, 24, 12.0, B.ACT_RELU2, 0)
    assert (s.mixer, s.ssm_state, s.ssm_groups, s.conv_taps, s.ssm_norm_groups, s.route_kind, s.mlp_flags) == \
        (B.MIX_SSM, 8, 2, 3, 2, B.ROUTE_SOFTMAX_ALL, B.MLP_SHARED_PLAIN)


# ---- the oracle's mechanisms, each against numbers worked out by hand

def test_position_vector():
    v = GO.position_vector(3, 6)
    f = [1.0, 10000.0 ** (-2 / 6), 10000.0 ** (-4 / 6)]
    assert np.allclose(v, [np.sin(3 * f[0]), np.cos(3 * f[0]), np.sin(3 * f[1]), np.cos(3 * f[1]), np.sin(3 * f[2]), np.cos(3 * f[2])])
    assert np.allclose(GO.position_vector(0, 4), [0, 1, 0, 1])


def test_window_and_cap_and_sink():
    assert [GO.window_visible(10, j, 3) for j in (7, 8, 9, 10, 11)] == [False, True, True, True, False]
    assert GO.window_visible(10, 0, 0) and not GO.window_visible(3, 4, 0)
    assert GO.capped(100.0, 5.0) == pytest.approx(5.0) and GO.capped(0.01, 5.0) == pytest.approx(0.01, rel=1e-4) and GO.capped(7.0, 0) == 7.0
    w = GO.unit_sink_weights([0.0])
    assert w[0] == pytest.approx(0.5)
    w = GO.unit_sink_weights([np.log(3.0), 0.0])
    assert np.allclose(w, [3 / 5, 1 / 5])
    assert GO.unit_sink_weights([-800.0])[0] == 0.0 and GO.unit_sink_weights([800.0])[0] == pytest.approx(1.0)


def test_convolution_last_tap_is_the_current_token():
    u = np.array([[1.0], [2.0], [4.0]])
    out = GO.causal_conv_silu(u, np.array([[100.0, 10.0, 1.0]]), np.array([0.5]))
    pre = np.array([1.5, 12.5, 124.5])
    assert np.allclose(out[:, 0], pre / (1 + np.exp(-pre)))


def test_state_space_by_hand():
    """One head, state 1, value size 1, a convolution of one tap of weight 1 without bias: everything is scalar."""
    mx = {"heads": 1, "vdim": 1, "state": 1, "groups": 1, "conv": 1, "norm_groups": 1}
    P = {"m.in": np.eye(5), "m.conv": np.ones((3, 1)), "m.conv.b": np.zeros(3), "m.dt_bias": np.array([0.3]), "m.A_log": np.array([0.2]),
         "m.D": np.array([0.7]), "m.norm": np.array([1.0]), "m.o": np.array([[1.0]])}
    h = np.array([[0.5, 1.0, -0.4, 0.8, 0.1], [1.5, -0.3, 0.9, 0.2, -0.6]])  # z, x, B, C, dt per token
    S, want = 0.0, []
    for z, x, b, c, dt in h:
        x, b, c = GO.silu(x), GO.silu(b), GO.silu(c)
        dt = np.log1p(np.exp(dt + 0.3))
        S = np.exp(-np.exp(0.2) * dt) * S + dt * b * x
        y = (S * c + 0.7 * x) * GO.silu(z)
        want.append(y / np.sqrt(y * y + 1e-6))
    got = GO.state_space(mx, P, "m.", h, 1e-6)
    assert np.allclose(got[:, 0], want)


def test_experts_choice_and_weights():
    idx, wt = GO.choose_experts([0.0, np.log(2.0), np.log(2.0), -5.0], 2)
    assert idx == [1, 2] and np.allclose(wt, [0.5, 0.5])
    idx, wt = GO.choose_experts([np.log(3.0), 0.0, -9.0], 2)
    assert idx == [0, 1] and np.allclose(wt, [0.75, 0.25])


def test_layer_order_with_a_loop():
    assert GO.layer_order({"layers": [0] * 5, "loop": {"start": 1, "stop": 3, "times": 3}}) == [0, 1, 2, 1, 2, 1, 2, 3, 4]
    assert GO.layer_order({"layers": [0] * 3}) == [0, 1, 2]


def test_streams_equal_one_residual_when_the_coefficients_say_so():
    """in = (1, 0, 0), out = (1, 0, 0) and mix = identity keep everything in the first stream; the other streams keep the
    embedding, so the sum of the streams is the plain residual plus (S - 1) embeddings: with S = 1 the two coincide."""
    cfg1 = U.config(LAYERS, streams=1)
    W = U.weights(cfg1, seed=2)
    for k in W:
        if ".hc" in k:
            W[k] = np.ones_like(W[k])
    cfg0 = U.config(LAYERS, streams=0)
    t = [3, 9, 1, 4, 4, 7, 30, 2]
    a = GO.forward(cfg1, W, t)[0]
    b = GO.forward(cfg0, {k: v for k, v in W.items() if ".hc" not in k}, t)[0]
    assert np.allclose(a, b)


@pytest.mark.parametrize("what", ["window", "softcap", "scale", "embed_scale", "streams_mix", "loop", "A_log", "dt_bias", "D", "conv", "norm_groups",
                                  "groups", "top", "shared", "eps", "position"])
def test_oracle_reacts_to(what):
    """Every constant and tensor the GPU tests compare through the oracle changes the oracle's output."""
    cfg = U.config(LAYERS, loop=(1, 3, 2))
    W = U.weights(cfg, seed=4)
    t = [int(x) for x in np.random.default_rng(0).integers(0, 50, 40)]
    base = GO.forward(cfg, W, t)[0]
    cfg2, W2, t2 = json.loads(json.dumps(cfg)), dict(W), list(t)
    if what == "window":
        cfg2["layers"][0]["mixer"]["mask"]["size"] = 23
    elif what == "softcap":
        cfg2["layers"][0]["mixer"]["softcap"] = 1.0
    elif what == "scale":
        cfg2["layers"][0]["mixer"]["scale"] *= 1.5
    elif what == "embed_scale":
        cfg2["embedding"]["scale"] = 4.0
    elif what == "streams_mix":
        W2["l1.hc2.mix"] = W["l1.hc2.mix"].T.copy()
    elif what == "loop":
        cfg2["loop"]["times"] = 3
    elif what in ("A_log", "dt_bias", "D"):
        W2["l1.mix." + what] = W["l1.mix." + what] + 0.5
    elif what == "conv":
        W2["l1.mix.conv"] = W["l1.mix.conv"][:, ::-1].copy()
    elif what == "norm_groups":
        cfg2["layers"][1]["mixer"]["norm_groups"] = 1
    elif what == "groups":
        cfg2["layers"][2]["mixer"]["groups"] = 6
        W2 = U.weights(cfg2, seed=4)
        cfg = cfg2
        base = GO.forward(cfg2, W2, t)[0]
        W2 = dict(W2)
        W2["l2.mix.in"] = W2["l2.mix.in"].copy()
        W2["l2.mix.in"][2 * 24 + 5:2 * 24 + 10] *= 2.0  # the B rows of the second group only
    elif what == "top":
        cfg2["layers"][1]["mlp"]["router"]["top"] = 3
    elif what == "shared":
        W2["l1.mlp.shared.down"] = W["l1.mlp.shared.down"] * 2
    elif what == "eps":
        cfg2["norm"]["eps"] = 0.5
    elif what == "position":
        base = GO.forward(cfg, W, [5, 5, 5, 5])[0]
        assert np.abs(base[3] - base[0]).max() > 1e-3  # equal tokens, different positions
        return
    other = GO.forward(cfg2, W2, t2)[0]
    assert np.abs(other - base).max() > 1e-4
