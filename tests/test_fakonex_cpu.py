"""Fakonex without a GPU: the configuration reader, the table of tensor names and shapes, and the oracle's own sensitivity to
every constant and mechanism the GPU tests rely on."""
import copy

import numpy as np
import pytest

from distributed_inference_server_b200 import binding as B
from distributed_inference_server_b200 import models
from tests import _fakonex_util as U
from tests import fakonex_oracle as FO


def toks(n, vocab=50, seed=0):
    return [int(x) for x in np.random.default_rng(seed).integers(0, vocab, n)]


LAYERS = [(U.attention(), U.moe()), (U.attention(heads=6, kv_heads=2, chunk=0, kv_from=0), None), (U.attention(chunk=9), U.moe(groups=None, shared=0))]


def test_registry_reads_the_configuration():
    cfg = U.config(LAYERS, width=40, vocab=77, eps=3e-4, softcap=11.0)
    assert models.architecture_of(cfg) == "Fakonex"
    family, reader = models.ARCHITECTURES["Fakonex"]
    spec = reader(cfg)
    assert family == "stack" and spec.norm_kind == "rms" and spec.logit_softcap == 11.0 and spec.norm_eps == 3e-4 and spec.loop[2] == 0
    a, b, c = spec.layers
    flags = B.ATTN_BIAS_QKV | B.ATTN_QK_NORM_HEAD | B.ATTN_SINK | B.ATTN_GATE
    assert a.mixer == "attention" and a.attn_flags == flags and (a.heads, a.kv_heads, a.dim, a.vdim) == (4, 2, 8, 12)
    assert a.mask_chunk == 24 and a.kv_from == -1 and a.rot_dims == 0 and a.scale == 8 ** -0.5
    assert (a.mlp, a.mlp_act, a.route, a.experts, a.top, a.ff) == ("moe", "silu", "sigmoid_groups", 6, 2, 10)
    assert (a.route_groups, a.route_keep, a.shared_ff) == (3, 2, 14)
    assert b.kv_from == 0 and b.mask_chunk == 0 and b.mlp == "none" and b.heads == 6
    assert (c.route_groups, c.route_keep, c.shared_ff, c.mask_chunk) == (0, 0, 0, 9)
    sc, _keep = spec.c(256, 8, False)
    assert sc.norm_kind == B.NORM_RMS and sc.logit_softcap == 11.0 and sc.layers[0].mask_chunk == 24 and sc.layers[1].kv_from == 0
    assert sc.layers[0].route_kind == B.ROUTE_SIGMOID_GROUPS and sc.layers[0].shared_ff == 14 and sc.layers[0].mlp_act == B.ACT_SILU


def test_reader_refuses_what_cannot_be():
    bad = U.config(LAYERS)
    bad["layers"][1]["mixer"]["kv_from"] = 2  # a later layer
    with pytest.raises(ValueError):
        models.fakonex_spec(bad)
    bad = U.config(LAYERS + [(U.attention(kv_from=1), None)])  # a layer that itself borrows
    with pytest.raises(ValueError):
        models.fakonex_spec(bad)
    bad = U.config([(U.attention(), U.moe(experts=6, top=3, groups=(3, 1)))])  # one group of two cannot give three experts
    with pytest.raises(ValueError):
        models.fakonex_spec(bad)
    bad = U.config([(U.attention(), U.moe(experts=6, groups=(4, 1)))])  # four groups do not divide six experts
    with pytest.raises(ValueError):
        models.fakonex_spec(bad)
    bad = U.config(LAYERS)
    bad["layers"][0]["type"] = "recurrent"
    with pytest.raises(ValueError):
        models.fakonex_spec(bad)


def test_tensor_table():
    shapes = models.fakonex_spec(U.config(LAYERS, width=40, vocab=77)).tensor_shapes()
    assert shapes["embed"] == (77, 40) and shapes["head"] == (77, 40) and shapes["final.norm"] == (40,) and "final.norm.b" not in shapes
    assert shapes["l0.norm1"] == (40,) and "l0.norm1.b" not in shapes and shapes["l0.norm2b"] == (40,) and "l1.norm2" not in shapes
    assert shapes["l0.mix.q"] == (32, 40) and shapes["l0.mix.k"] == (16, 40) and shapes["l0.mix.v"] == (24, 40)
    assert shapes["l0.mix.q.b"] == (32,) and shapes["l0.mix.k.b"] == (16,) and shapes["l0.mix.v.b"] == (24,) and "l0.mix.o.b" not in shapes
    assert shapes["l0.mix.q.norm"] == (8,) and shapes["l0.mix.k.norm"] == (8,) and shapes["l0.mix.sink"] == (4,)
    assert shapes["l0.mix.g"] == (4, 40) and shapes["l0.mix.o"] == (40, 48)
    # a layer that reads another's cache has queries, gate, sink and output only
    assert shapes["l1.mix.q"] == (48, 40) and shapes["l1.mix.q.norm"] == (8,) and shapes["l1.mix.o"] == (40, 72)
    assert not [k for k in shapes if k.startswith("l1.mix.k") or k.startswith("l1.mix.v")]
    assert shapes["l0.mlp.router"] == (6, 40) and shapes["l0.mlp.correction"] == (6,) and shapes["l0.mlp.e5.down"] == (40, 10)
    assert shapes["l0.mlp.shared.gate"] == (14, 40) and shapes["l0.mlp.shared.down"] == (40, 14) and shapes["l0.mlp.shared.sg"] == (1, 40)
    assert "l2.mlp.shared.sg" not in shapes and shapes["l2.mlp.correction"] == (6,)
    assert set(U.weights(U.config(LAYERS, width=40, vocab=77))) == set(shapes)


def test_mechanisms_of_the_oracle_one_by_one():
    assert FO.visible(9, 9, 0) and FO.visible(9, 0, 0) and not FO.visible(3, 4, 0)
    assert FO.visible(9, 5, 5) and not FO.visible(9, 4, 5) and FO.visible(10, 10, 5) and not FO.visible(10, 9, 5) and FO.visible(4, 0, 5)
    w = FO.sink_softmax([0.0, 0.0], 0.0)
    assert np.allclose(w, [1 / 3, 1 / 3]) and np.allclose(FO.sink_softmax([1.0], -1e9), [1.0]) and FO.sink_softmax([0.0], 50.0)[0] < 1e-20
    assert np.allclose(FO.rms_norm(np.array([3.0, -4.0]), np.array([2.0, 1.0]), 0.0), [6 / np.sqrt(12.5), -4 / np.sqrt(12.5)])
    s = np.array([0.9, 0.1, 0.5, 0.5, 0.6, 0.55])
    assert FO.choose_experts(s, np.zeros(6), 2) == [0, 4]
    assert FO.choose_experts(s, np.zeros(6), 2, (3, 1)) == [4, 5]          # 0.6 + 0.55 beats 0.9 + 0.1 and 0.5 + 0.5
    assert FO.choose_experts(s, np.array([0, 0, 0.3, 0, 0, 0]), 2, (3, 1)) == [2, 3]
    assert FO.choose_experts(s, np.array([0, 0, 0.3, 0, 0, 0]), 3, (3, 2)) == [2, 4, 5]
    assert FO.choose_experts(s, -10 * np.ones(6), 1, (3, 1)) == [4]          # below zero everywhere: the kept group still gives
    assert FO.choose_experts(s[:3], np.zeros(3), 2, (3, 2)) == [0, 2]        # groups of one
    assert np.allclose(FO.soft_cap(np.array([0.0, 100.0, -100.0]), 5.0), [0.0, 5.0, -5.0]) and FO.soft_cap(7.0, 0) == 7.0


def test_the_oracle_reacts_to_every_constant():
    """A constant or tensor that the engine and the oracle both ignored would pass the GPU tests unnoticed."""
    t = toks(60, seed=2)
    base = U.config(LAYERS)
    W = U.weights(base, seed=4)
    ref = U.oracle_logits(base, W, t)

    def moved(cfg=None, W2=None):
        return U.rel_err(U.oracle_logits(cfg or base, W2 or W, t), ref)
    for change in ("chunk", "no_mask", "scale", "groups", "keep", "top", "no_shared", "softcap", "eps", "kv_from"):
        cfg = copy.deepcopy(base)
        W2 = dict(W)
        if change == "chunk":
            cfg["layers"][0]["mixer"]["mask"]["size"] = 23
        elif change == "no_mask":
            del cfg["layers"][2]["mixer"]["mask"]
        elif change == "scale":
            cfg["layers"][1]["mixer"]["scale"] *= 2
        elif change == "groups":
            del cfg["layers"][0]["mlp"]["router"]["groups"]
        elif change == "keep":
            cfg["layers"][0]["mlp"]["router"]["groups"]["keep"] = 1
        elif change == "top":
            cfg["layers"][2]["mlp"]["router"]["top"] = 3
        elif change == "no_shared":
            del cfg["layers"][0]["mlp"]["shared"]
        elif change == "softcap":
            cfg["logit_softcap"] = 3.0
        elif change == "eps":
            cfg["norm"]["eps"] = 0.5
        else:
            cfg["layers"][1]["mixer"]["heads"] = 4
            cfg["layers"][1]["mixer"]["kv_from"] = None
            W2 = U.weights(cfg, seed=4)
            W2.update({k: v for k, v in W.items() if k in W2 and W2[k].shape == v.shape and not k.startswith("l1.mix")})
        assert moved(cfg, W2) > 1e-3, change
    for name in ("l0.mix.sink", "l1.mix.sink", "l0.mix.g", "l0.mix.q.b", "l0.mix.k.b", "l0.mix.v.b", "l0.mix.q.norm", "l2.mix.k.norm",
                 "l0.mlp.correction", "l0.mlp.shared.sg", "l0.mlp.shared.up", "l2.mlp.router", "l0.norm1b", "l2.norm2b", "final.norm"):
        W2 = dict(W)
        W2[name] = models.bf16_round(W[name] + np.random.default_rng(7).normal(0, 1.0, W[name].shape).astype(np.float32))
        assert moved(None, W2) > 1e-4, name
