"""Helpers of the Goperax tests: small made-up configurations, random weights, the oracle's logits and engines built from
them.  The step driver (Feeder) and the error measures are those of the other layer-list tests."""
import copy

import numpy as np

from distributed_inference_server_b200 import Engine, WorkerConfig, models
from tests import goperax_oracle as GO
from tests._stack_util import Feeder, bf16_close, rel_err, row_errs  # noqa: F401  (re-exported)


def attention(heads=4, kv_heads=2, dim=8, window=24, scale=None, softcap=12.0):
    mx = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": dim ** -0.5 if scale is None else scale}
    if window:
        mx["mask"] = {"size": window}
    if softcap:
        mx["softcap"] = softcap
    return {"type": "attention", "mixer": mx}


def ssm(heads=4, vdim=6, state=8, groups=2, conv=3, norm_groups=2):
    return {"type": "mamba2", "mixer": {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv,
                                        "norm_groups": norm_groups}}


def dense(ff=40):
    return {"kind": "dense", "ff": ff}


def moe(experts=6, top=2, ff=10, shared=14):
    ml = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared:
        ml["shared"] = {"ff": shared}
    return ml


def config(layers, vocab=50, width=32, eps=1e-5, streams=3, loop=None, embed_scale=3.0):
    """layers: list of (mixer dict, mlp dict or None); loop: (start, stop, times) or None."""
    cfg = {"architecture": "Goperax", "vocab": vocab, "width": width, "norm": {"eps": eps}, "embedding": {"scale": embed_scale},
           "layers": [dict(copy.deepcopy(m), mlp=copy.deepcopy(f)) for m, f in layers]}
    if streams:
        cfg["streams"] = streams
    if loop:
        cfg["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return cfg


def weights(cfg, seed=0, gain=1.0):
    """Random float32 tensors by name, every value representable in bfloat16 (both compute types then see one model)."""
    spec = models.goperax_spec(cfg)
    rng = np.random.default_rng(seed)
    out = {}
    for name, shape in spec.tensor_shapes().items():
        leaf = name.rsplit(".", 1)[-1]
        if ".hc" in name:
            n = shape[0]
            a = {"in": rng.normal(1.0 / n, 0.3, shape), "out": rng.normal(1.0, 0.4, shape), "mix": np.eye(n) + rng.normal(0, 0.3, shape)}[leaf]
        elif leaf in ("norm1", "norm2", "norm"):
            a = rng.uniform(0.5, 1.5, shape)
        elif leaf == "dt_bias":
            a = rng.normal(-1.0, 1.0, shape)
        elif leaf == "A_log":
            a = rng.uniform(-3.0, 1.0, shape)
        elif leaf == "D":
            a = rng.normal(1.0, 0.5, shape)
        elif leaf == "conv":
            a = rng.normal(0, 0.6, shape)
        elif leaf == "b":
            a = rng.normal(0, 0.4, shape)
        elif name == "embed":
            a = rng.normal(0, 1.0, shape)
        elif leaf == "router":
            a = rng.normal(0, 2.0 / np.sqrt(shape[-1]), shape)
        else:
            a = rng.normal(0, gain / np.sqrt(shape[-1]), shape)
        out[name] = models.bf16_round(np.asarray(a, np.float32))
    return out


def oracle_logits(cfg, W, tokens):
    return GO.forward(cfg, W, tokens)[0]


def engine(cfg, W, dtype="float32", max_batch=4, pool_tokens=512, page_size=8, max_step_tokens=0, rows=0):
    spec = models.goperax_spec(cfg)
    cap = max_step_tokens or pool_tokens
    e = Engine(WorkerConfig(None, max_batch=max_batch, max_step_tokens=cap, page_size=page_size,
                            kv_pages=(pool_tokens + page_size - 1) // page_size, stack=spec, context_size=pool_tokens + page_size,
                            compute_dtype=dtype, max_logit_rows=(rows or cap) + max_batch))
    for name, a in W.items():
        e.load_named(name, np.asarray(a, np.float32))
    e.finalize()
    return e


def feed(e, tokens, cuts, key="a"):
    """One sequence through a live engine: portions of the given sizes, the rest token by token; its logits; its slot and
    pages go back to the engine."""
    f = Feeder(e)
    fed = 0
    for n in cuts:
        n = min(n, len(tokens) - fed)
        if n > 0:
            f.step([(key, tokens, n)])
            fed += n
    while fed < len(tokens):
        f.step([(key, tokens, 1)])
        fed += 1
    return f.end(key)


def run_whole(cfg, W, tokens, dtype="float32", **kw):
    e = engine(cfg, W, dtype, **kw)
    out = feed(e, tokens, [len(tokens)])
    e.close()
    return out


def run_portions(cfg, W, tokens, sizes, dtype="float32", **kw):
    """The sequence in portions of the given sizes (the rest one token at a time)."""
    e = engine(cfg, W, dtype, **kw)
    out = feed(e, tokens, sizes)
    e.close()
    return out
