"""Helpers of the Fakonex tests: small made-up configurations, random weights, the oracle's logits and engines built from
them.  The step driver (Feeder) and the error measures are those of the other layer-list tests."""
import copy

import numpy as np

from distributed_inference_server_b200 import Engine, WorkerConfig, models
from tests import fakonex_oracle as FO
from tests._stack_util import Feeder, bf16_close, rel_err, row_errs  # noqa: F401  (re-exported)


def attention(heads=4, kv_heads=2, dim=8, vdim=12, chunk=24, scale=None, kv_from=None):
    mx = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": dim ** -0.5 if scale is None else scale}
    if chunk:
        mx["mask"] = {"size": chunk}
    if kv_from is not None:
        mx["kv_from"] = kv_from
    return {"type": "attention", "mixer": mx}


def moe(experts=6, top=2, ff=10, groups=(3, 2), shared=14):
    ml = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if groups:
        ml["router"]["groups"] = {"count": groups[0], "keep": groups[1]}
    if shared:
        ml["shared"] = {"ff": shared}
    return ml


def config(layers, vocab=50, width=32, eps=1e-5, softcap=9.0):
    """layers: list of (mixer dict, mlp dict or None)."""
    cfg = {"architecture": "Fakonex", "vocab": vocab, "width": width, "norm": {"eps": eps},
           "layers": [dict(copy.deepcopy(m), mlp=copy.deepcopy(f)) for m, f in layers]}
    if softcap:
        cfg["logit_softcap"] = softcap
    return cfg


def weights(cfg, seed=0, gain=1.0):
    """Random float32 tensors by name, every value representable in bfloat16 (both compute types then see one model)."""
    spec = models.fakonex_spec(cfg)
    rng = np.random.default_rng(seed)
    out = {}
    for name, shape in spec.tensor_shapes().items():
        leaf = name.rsplit(".", 1)[-1]
        if leaf == "b":
            a = rng.normal(0, 0.5, shape)
        elif leaf in ("norm1", "norm1b", "norm2", "norm2b", "norm"):
            a = rng.uniform(0.5, 1.5, shape)
        elif leaf == "sink":
            a = rng.normal(0.5, 1.0, shape)
        elif leaf == "correction":
            a = rng.normal(0, 0.4, shape)
        elif name == "embed":
            a = rng.normal(0, 1.0, shape)
        elif leaf in ("router", "sg", "g"):
            a = rng.normal(0, 2.0 / np.sqrt(shape[-1]), shape)
        else:
            a = rng.normal(0, gain / np.sqrt(shape[-1]), shape)
        out[name] = models.bf16_round(np.asarray(a, np.float32))
    return out


def oracle_logits(cfg, W, tokens, layers_out=None):
    return FO.forward(cfg, W, tokens, layers_out)


def engine(cfg, W, dtype="float32", max_batch=4, pool_tokens=512, page_size=8, max_step_tokens=0, rows=0):
    spec = models.fakonex_spec(cfg)
    cap = max_step_tokens or pool_tokens
    e = Engine(WorkerConfig(None, max_batch=max_batch, max_step_tokens=cap, page_size=page_size,
                            kv_pages=(pool_tokens + page_size - 1) // page_size, stack=spec, context_size=pool_tokens + page_size,
                            compute_dtype=dtype, max_logit_rows=(rows or cap) + max_batch))
    for name, a in W.items():
        e.load_named(name, np.asarray(a, np.float32))
    e.finalize()
    return e


def run_whole(cfg, W, tokens, dtype="float32", **kw):
    e = engine(cfg, W, dtype, **kw)
    f = Feeder(e)
    f.step([("a", tokens, len(tokens))])
    out = f.end("a")
    e.close()
    return out


def run_portions(cfg, W, tokens, sizes, dtype="float32", **kw):
    """The sequence in portions of the given sizes (the rest one token at a time)."""
    e = engine(cfg, W, dtype, **kw)
    f = Feeder(e)
    fed = 0
    for n in sizes:
        n = min(n, len(tokens) - fed)
        if n <= 0:
            break
        f.step([("a", tokens, n)])
        fed += n
    while fed < len(tokens):
        f.step([("a", tokens, 1)])
        fed += 1
    out = f.end("a")
    e.close()
    return out
