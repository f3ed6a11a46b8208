"""Model registry: which engine a model folder's config.json asks for, and how its weights get there.

A model folder holds config.json and model.safetensors.  `architecture` (or, for Hugging Face style folders,
`architectures[0]` / `model_type`) selects an entry of ARCHITECTURES; the entry turns the configuration into the
engine's description of the model and names every tensor.  Two families exist:

  llama     the fixed Llama decoder of engine.cu (ModelShape; tensors by kind and layer)
  Kidolorn  a layer-list decoder of stack.cu (StackSpec; tensors by name): per layer one mixer out of linear attention
            with a fixed per-head decay, a minimal gated recurrence, or latent attention over a compressed cache (which a
            later layer may share), and a dense or mixture-of-experts feed-forward, every sublayer behind a scalar-gain RMS
            norm and a short causal convolution.
  Motolix   a layer-list decoder of the same engine with layer norms (weight and bias) before and after every sublayer, a
            stretch of layers that runs several times with shared weights (each pass with its own cache and state, entered
            through a projection of [residual ; embedding] plus a per-pass vector), and two mixers: `attention` (grouped-query,
            values = unrotated keys, partial rotary with wavelength-dependent frequency scaling, sigmoid weights with a
            per-head temperature and bias instead of softmax) and `parallel` (softmax attention with whole-projection
            query/key norms and position-rotated values, beside gated linear attention with a per-channel decay; the two
            outputs are added with fixed weights); feed-forward gelu_tanh(gate) * up.
  Fakonex   a layer-list decoder of the same engine with RMS norms (gain vectors) before and after every sublayer; its
            `attention` mixer is grouped-query softmax attention without rotation, with biases on q, k and v, a per-head RMS
            norm of queries and keys, a causal mask cut into chunks of a fixed number of positions, a learned per-head sink
            logit in the softmax denominator and a per-head sigmoid gate on the output, and a layer may read an earlier layer's
            keys and values instead of projecting its own; the feed-forward is a mixture of SiLU-gated experts chosen by a
            sigmoid router with a correction vector and a limit on the groups of experts a token may use, plus a shared
            expert behind a sigmoid gate; the logits pass through a tanh soft cap.
  Goperax   a layer-list decoder of the same engine in the pre-norm frame (RMS norms with gain vectors in front of the
            sublayers only) whose residual is several streams mixed by small learned matrices around every sublayer; scaled
            embedding plus a sinusoidal position vector, logits from the embedding table itself; a stretch of layers that runs
            several times in a row with nothing in between; mixers `attention` (grouped-query, values = keys, no rotation, a
            tanh soft cap on the scores, a sliding window, and a softmax whose denominator carries one extra 1) and `mamba2`
            (selective state space with a short causal convolution, gated and group-normalised); feed-forward of ungated
            squared-ReLU units, dense or as a mixture chosen by a softmax router, with an optional always-on shared unit.

The reference has no model loading at all (crates/inference/src/worker.rs:1 is empty).
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from dataclasses import dataclass, field
from typing import Callable, Dict, Iterator, List, Optional, Tuple

import numpy as np

from . import binding as B

_MIXERS = {"lightning": B.MIX_LIGHTNING, "mingru": B.MIX_MINGRU, "latent_attention": B.MIX_LATENT,
           "attention": B.MIX_ATTENTION, "parallel": B.MIX_PARALLEL, "ssm": B.MIX_SSM}
_ACTS = {"clamped": B.ACT_CLAMPED, "gelu_tanh": B.ACT_GELU_TANH, "silu": B.ACT_SILU, "relu2": B.ACT_RELU2}
_ROUTES = {"softmax_top": B.ROUTE_SOFTMAX_TOP, "sigmoid_groups": B.ROUTE_SIGMOID_GROUPS, "softmax_all": B.ROUTE_SOFTMAX_ALL}


@dataclass
class LayerSpec:
    mixer: str
    heads: int = 0
    dim: int = 0
    vdim: int = 0
    width: int = 0
    kv_rank: int = 0
    rot_dim: int = 0
    rot_dims: int = 0
    kv_from: int = -1
    rot_base: float = 10000.0
    scale: float = 1.0
    decay: List[float] = field(default_factory=list)
    mlp: str = "none"  # none | dense | moe
    ff: int = 0
    experts: int = 0
    top: int = 0
    limit: float = 0.0
    # attention / parallel
    kv_heads: int = 0
    attn_flags: int = 0
    rot_factor: float = 0.0
    rot_low: float = 0.0
    rot_high: float = 0.0
    rot_original: int = 0
    gla_heads: int = 0
    gla_dim: int = 0
    gla_vdim: int = 0
    gla_rank: int = 0
    gla_tau: float = 1.0
    mix_scale: float = 1.0
    gla_scale: float = 1.0
    mlp_act: str = "clamped"  # clamped (with biases) | gelu_tanh (without) | silu (without) | relu2 (ungated, without)
    mask_chunk: int = 0  # attention: chunked causal mask (0 = plain causal)
    route: str = "softmax_top"  # softmax_top | sigmoid_groups | softmax_all
    route_groups: int = 0
    route_keep: int = 0
    shared_ff: int = 0  # mixture of experts: hidden size of the shared expert (0 = none)
    mask_window: int = 0  # attention: sliding window (0 = none)
    score_softcap: float = 0.0  # attention: tanh soft cap on the scaled scores (0 = none)
    ssm_state: int = 0  # state-space mixer: state size per head, groups sharing B and C, convolution taps, norm parts
    ssm_groups: int = 0
    conv_taps: int = 0
    ssm_norm_groups: int = 1
    shared_plain: bool = False  # the shared expert joins the sum without a gate

    @property
    def gated(self) -> bool:
        return self.mlp_act != "relu2"


@dataclass
class StackSpec:
    """A layer-list decoder: sizes, constants and the order of layers, all from the model's configuration."""
    name: str
    vocab: int
    width: int
    layers: List[LayerSpec]
    canon_taps: int = 0
    norm_eps: float = 1e-5
    norm_kind: str = "rms_scalar"  # rms_scalar | layer | rms
    embed_scale: float = 1.0
    logit_scale: float = 1.0
    loop: Tuple[int, int, int] = (0, 0, 0)  # start, stop, times (times 0 = no loop)
    logit_softcap: float = 0.0  # c > 0: logits -> c tanh(logits / c)
    pre_norm: bool = False  # sublayers are x += f(norm(x)): no norms behind them
    streams: int = 0  # residual streams mixed around every sublayer (0 = one plain residual); needs pre_norm
    pos_sinus: bool = False  # a sinusoidal position vector joins the scaled embedding
    pos_base: float = 10000.0
    loop_plain: bool = False  # the loop's passes follow each other without an input projection
    tied_head: bool = False  # logits from the embedding table: the file has no "head"

    def layer_runs(self) -> List[int]:
        """Layer index of every layer run of one forward pass, the looped stretch repeated."""
        a, b, n = self.loop
        if n <= 0:
            return list(range(len(self.layers)))
        return list(range(a)) + list(range(a, b)) * n + list(range(b, len(self.layers)))

    def tensor_shapes(self) -> Dict[str, Tuple[int, ...]]:
        """Every tensor of the model file, by name."""
        W, out = self.width, {"embed": (self.vocab, self.width), "head": (self.vocab, self.width)}
        if self.tied_head:
            del out["head"]
        vec = self.norm_kind in ("layer", "rms")
        post = not self.pre_norm

        def norm(name):
            out[name] = (W,) if vec else ()
            if self.norm_kind == "layer":
                out[name + ".b"] = (W,)
        norm("final.norm")
        if self.loop[2] > 0 and not self.loop_plain:
            out["loop.in"] = (W, 2 * W)
            out["loop.step"] = (self.loop[2], W)
        for i, L in enumerate(self.layers):
            p = f"l{i}."
            norm(p + "norm1")
            if post:
                norm(p + "norm1b")
            for q in ((1,) if L.mlp == "none" else (1, 2)) if self.streams > 0 else ():
                out.update({f"{p}hc{q}.in": (self.streams,), f"{p}hc{q}.out": (self.streams,), f"{p}hc{q}.mix": (self.streams, self.streams)})
            if self.canon_taps >= 1:
                out[p + "canon1"] = (W, self.canon_taps)
            if L.mixer == "lightning":
                out.update({p + "mix.q": (L.heads * L.dim, W), p + "mix.k": (L.heads * L.dim, W), p + "mix.v": (L.heads * L.vdim, W),
                            p + "mix.g": (L.heads * L.vdim, W), p + "mix.o": (W, L.heads * L.vdim), p + "mix.norm": (L.heads * L.vdim,)})
            elif L.mixer == "mingru":
                out.update({p + "mix.z": (L.width, W), p + "mix.z.b": (L.width,), p + "mix.x": (L.width, W), p + "mix.x.b": (L.width,),
                            p + "mix.g": (L.width, W), p + "mix.o": (W, L.width)})
            elif L.mixer == "ssm":
                inner, gn = L.heads * L.vdim, L.ssm_groups * L.ssm_state
                out.update({p + "mix.in": (2 * inner + 2 * gn + L.heads, W), p + "mix.conv": (inner + 2 * gn, L.conv_taps),
                            p + "mix.conv.b": (inner + 2 * gn,), p + "mix.dt_bias": (L.heads,), p + "mix.A_log": (L.heads,),
                            p + "mix.D": (L.heads,), p + "mix.norm": (inner,), p + "mix.o": (W, inner)})
            elif L.mixer in ("attention", "parallel"):
                a = p + ("mix.left." if L.mixer == "parallel" else "mix.")
                own = L.kv_from < 0  # a layer that reads another layer's cache has nothing of the keys and values
                out.update({a + "q": (L.heads * L.dim, W), a + "o": (W, L.heads * L.vdim)})
                if own:
                    out[a + "k"] = (L.kv_heads * L.dim, W)
                if own and not L.attn_flags & B.ATTN_V_IS_K:
                    out[a + "v"] = (L.kv_heads * L.vdim, W)
                if L.attn_flags & B.ATTN_BIAS:
                    out.update({a + "q.b": (L.heads * L.dim,), a + "k.b": (L.kv_heads * L.dim,), a + "o.b": (W,)})
                if L.attn_flags & B.ATTN_BIAS_QKV:
                    out[a + "q.b"] = (L.heads * L.dim,)
                    if own:
                        out.update({a + "k.b": (L.kv_heads * L.dim,), a + "v.b": (L.kv_heads * L.vdim,)})
                if L.attn_flags & B.ATTN_QK_NORM:
                    out.update({a + "q.norm": (L.heads * L.dim,), a + "k.norm": (L.kv_heads * L.dim,)})
                if L.attn_flags & B.ATTN_QK_NORM_HEAD:
                    out[a + "q.norm"] = (L.dim,)
                    if own:
                        out[a + "k.norm"] = (L.dim,)
                if L.attn_flags & B.ATTN_SINK:
                    out[a + "sink"] = (L.heads,)
                if L.attn_flags & B.ATTN_GATE:
                    out[a + "g"] = (L.heads, W)
                if L.attn_flags & B.ATTN_SIGMOID:
                    out.update({a + "temp": (L.heads,), a + "pb": (L.heads,)})
                if L.mixer == "parallel":
                    r, n, nv = p + "mix.right.", L.gla_heads * L.gla_dim, L.gla_heads * L.gla_vdim
                    out.update({r + "q": (n, W), r + "k": (n, W), r + "v": (nv, W), r + "g": (nv, W), r + "o": (W, nv),
                                r + "norm": (L.gla_vdim,), r + "a1": (L.gla_rank, W), r + "a2": (n, L.gla_rank), r + "a2.b": (n,)})
            else:
                out[p + "mix.q"] = (L.heads * (L.dim + L.rot_dim), W)
                if L.kv_from < 0:
                    out[p + "mix.dkv"] = (L.kv_rank + L.rot_dim, W)
                    out[p + "mix.dkv.norm"] = (L.kv_rank,)
                out.update({p + "mix.uk": (L.heads * L.dim, L.kv_rank), p + "mix.uv": (L.heads * L.vdim, L.kv_rank),
                            p + "mix.sink": (L.heads,), p + "mix.g": (L.heads * L.vdim, W), p + "mix.o": (W, L.heads * L.vdim)})
            if L.mlp == "none":
                continue
            norm(p + "norm2")
            if post:
                norm(p + "norm2b")
            if self.canon_taps >= 1:
                out[p + "canon2"] = (W, self.canon_taps)
            if not L.gated:  # ungated units: "up" and "down" only
                if L.mlp == "dense":
                    out.update({p + "mlp.up": (L.ff, W), p + "mlp.down": (W, L.ff)})
                else:
                    out[p + "mlp.router"] = (L.experts, W)
                    for e in range(L.experts):
                        out.update({f"{p}mlp.e{e}.up": (L.ff, W), f"{p}mlp.e{e}.down": (W, L.ff)})
                    if L.shared_ff > 0:
                        out.update({p + "mlp.shared.up": (L.shared_ff, W), p + "mlp.shared.down": (W, L.shared_ff)})
                        if not L.shared_plain:
                            out[p + "mlp.shared.sg"] = (1, W)
            elif L.mlp == "dense" and L.mlp_act in ("gelu_tanh", "silu"):
                out.update({p + "mlp.gate": (L.ff, W), p + "mlp.up": (L.ff, W), p + "mlp.down": (W, L.ff)})
            elif L.mlp == "dense":
                out.update({p + "mlp.gate": (L.ff, W), p + "mlp.gate.b": (L.ff,), p + "mlp.up": (L.ff, W), p + "mlp.up.b": (L.ff,),
                            p + "mlp.down": (W, L.ff), p + "mlp.down.b": (W,)})
            else:
                out[p + "mlp.router"] = (L.experts, W)
                for e in range(L.experts):
                    out.update({f"{p}mlp.e{e}.gate": (L.ff, W), f"{p}mlp.e{e}.up": (L.ff, W), f"{p}mlp.e{e}.down": (W, L.ff)})
                if L.route == "sigmoid_groups":
                    out[p + "mlp.correction"] = (L.experts,)
                if L.shared_ff > 0:
                    out.update({p + "mlp.shared.gate": (L.shared_ff, W), p + "mlp.shared.up": (L.shared_ff, W),
                                p + "mlp.shared.down": (W, L.shared_ff)})
                    if not L.shared_plain:
                        out[p + "mlp.shared.sg"] = (1, W)
        return out

    def c(self, max_ctx: int, max_logit_rows: int, f32: bool):
        """The C description (dis_stack_config) and the objects that must outlive the call that reads it."""
        arr = (B.LayerConfig * len(self.layers))()
        keep = [arr]
        for i, L in enumerate(self.layers):
            c = arr[i]
            c.mixer = _MIXERS[L.mixer]
            c.heads, c.dim, c.vdim, c.width = L.heads, L.dim, L.vdim, L.width
            c.kv_rank, c.rot_dim, c.rot_dims, c.kv_from = L.kv_rank, L.rot_dim, L.rot_dims, L.kv_from
            c.rot_base, c.scale = L.rot_base, L.scale
            if L.decay:
                d = (B.C.c_float * len(L.decay))(*L.decay)
                keep.append(d)
                c.decay = d
            c.mlp = {"none": B.MLP_NONE, "dense": B.MLP_DENSE, "moe": B.MLP_MOE}[L.mlp]
            c.ff, c.experts, c.top, c.limit = L.ff, L.experts, L.top, L.limit
            c.kv_heads, c.attn_flags = L.kv_heads, L.attn_flags
            c.rot_factor, c.rot_low, c.rot_high, c.rot_original = L.rot_factor, L.rot_low, L.rot_high, L.rot_original
            c.gla_heads, c.gla_dim, c.gla_vdim, c.gla_rank = L.gla_heads, L.gla_dim, L.gla_vdim, L.gla_rank
            c.gla_tau, c.mix_scale, c.gla_scale = L.gla_tau, L.mix_scale, L.gla_scale
            c.mlp_act = _ACTS[L.mlp_act]
            c.mask_chunk, c.shared_ff = L.mask_chunk, L.shared_ff
            c.route_kind = _ROUTES[L.route]
            c.route_groups, c.route_keep = L.route_groups, L.route_keep
            c.mask_window, c.score_softcap = L.mask_window, L.score_softcap
            c.ssm_state, c.ssm_groups, c.conv_taps, c.ssm_norm_groups = L.ssm_state, L.ssm_groups, L.conv_taps, L.ssm_norm_groups
            c.mlp_flags = B.MLP_SHARED_PLAIN if L.shared_plain else 0
        sc = B.StackConfig(self.vocab, self.width, len(self.layers), self.canon_taps, max_ctx, max_logit_rows,
                           B.F32 if f32 else B.BF16, self.norm_eps, arr,
                           {"rms_scalar": B.NORM_RMS_SCALAR, "layer": B.NORM_LAYER, "rms": B.NORM_RMS}[self.norm_kind],
                           self.embed_scale, self.logit_scale, *self.loop, self.logit_softcap,
                           (B.FRAME_PRE_NORM if self.pre_norm else 0) | (B.FRAME_POS_SINUS if self.pos_sinus else 0) |
                           (B.FRAME_LOOP_PLAIN if self.loop_plain else 0) | (B.FRAME_TIED_HEAD if self.tied_head else 0),
                           self.streams, self.pos_base)
        return sc, keep


def kidolorn_spec(cfg: dict) -> StackSpec:
    """Kidolorn's config.json -> StackSpec.  Every size and constant comes from the file; nothing is assumed."""
    layers = []
    for i, ly in enumerate(cfg["layers"]):
        kind, mx = ly["type"], ly["mixer"]
        if kind not in _MIXERS:
            raise ValueError(f"layer {i}: unknown mixer type {kind!r}")
        L = LayerSpec(kind)
        if kind == "lightning":
            L.heads, L.dim, L.vdim = int(mx["heads"]), int(mx["dim"]), int(mx["vdim"])
            L.decay = [float(a) for a in mx["decay"]]
            if len(L.decay) != L.heads:
                raise ValueError(f"layer {i}: decay must list one value per head")
        elif kind == "mingru":
            L.width = int(mx["width"])
        else:
            L.heads, L.dim, L.vdim = int(mx["heads"]), int(mx["dim"]), int(mx["vdim"])
            L.kv_rank, L.rot_dim = int(mx["kv_rank"]), int(mx["rot_dim"])
            rot = mx.get("rot") or {}
            L.rot_dims, L.rot_base = int(rot.get("dims", L.rot_dim)), float(rot.get("base", 10000.0))
            L.scale = float(mx["scale"])
            kf = mx.get("kv_from")
            L.kv_from = -1 if kf is None else int(kf)
        ml = ly.get("mlp")
        if ml is not None:
            if ml["kind"] == "dense":
                L.mlp, L.ff, L.limit = "dense", int(ml["ff"]), float(ml["limit"])
            elif ml["kind"] == "moe":
                L.mlp, L.ff, L.limit = "moe", int(ml["expert"]["ff"]), float(ml["expert"]["limit"])
                L.experts, L.top = int(ml["router"]["experts"]), int(ml["router"]["top"])
            else:
                raise ValueError(f"layer {i}: unknown feed-forward kind {ml['kind']!r}")
        layers.append(L)
    canon = cfg.get("canon") or {}
    return StackSpec("Kidolorn", int(cfg["vocab"]), int(cfg["width"]), layers, int(canon.get("taps", 0)),
                     float((cfg.get("norm") or {}).get("eps", 1e-5)))


def _attention_fields(L: LayerSpec, mx: dict, flags: int, where: str) -> None:
    L.heads, L.kv_heads, L.dim, L.vdim = int(mx["heads"]), int(mx["kv_heads"]), int(mx["dim"]), int(mx["vdim"])
    if L.heads % L.kv_heads:
        raise ValueError(f"{where}: heads must be a multiple of kv_heads")
    rot = mx.get("rot") or {}
    L.rot_dims, L.rot_base = int(rot.get("dims", 0)), float(rot.get("base", 10000.0))
    sc = rot.get("scaling")
    if sc:
        L.rot_factor, L.rot_low, L.rot_high = float(sc["factor"]), float(sc["low"]), float(sc["high"])
        L.rot_original = int(sc["original"])
    L.scale = float(mx["scale"])
    L.attn_flags = flags


def motolix_spec(cfg: dict, shapes: Optional[Dict[str, Tuple[int, ...]]] = None) -> StackSpec:
    """Motolix's config.json -> StackSpec.  Sizes the configuration does not state (the rank of the decay bottleneck of the
    gated-linear half) come from the shapes of the model file's tensors, or from a `rank` entry beside the other sizes."""
    layers = []
    for i, ly in enumerate(cfg["layers"]):
        kind, mx = ly["type"], ly["mixer"]
        if kind == "attention":
            L = LayerSpec("attention")
            _attention_fields(L, mx, B.ATTN_SIGMOID | B.ATTN_V_IS_K | B.ATTN_BIAS, f"layer {i}")
        elif kind == "parallel":
            L = LayerSpec("parallel")
            _attention_fields(L, mx["left"], B.ATTN_QK_NORM | B.ATTN_ROT_V, f"layer {i}")
            r = mx["right"]
            L.gla_heads, L.gla_dim, L.gla_vdim, L.gla_tau = int(r["heads"]), int(r["dim"]), int(r["vdim"]), float(r["tau"])
            a1 = (shapes or {}).get(f"l{i}.mix.right.a1")
            if a1 is not None:
                L.gla_rank = int(a1[0])
            elif "rank" in r:
                L.gla_rank = int(r["rank"])
            else:
                raise ValueError(f"layer {i}: the rank of the decay projection is given by neither a tensor nor the configuration")
            L.mix_scale, L.gla_scale = float(mx["left_scale"]), float(mx["right_scale"])
        else:
            raise ValueError(f"layer {i}: unknown mixer type {kind!r}")
        ml = ly.get("mlp")
        if ml is not None:
            if ml["kind"] != "dense":
                raise ValueError(f"layer {i}: unknown feed-forward kind {ml['kind']!r}")
            L.mlp, L.ff, L.mlp_act = "dense", int(ml["ff"]), "gelu_tanh"
        layers.append(L)
    lp = cfg.get("loop")
    loop = (int(lp["start"]), int(lp["stop"]), int(lp["times"])) if lp else (0, 0, 0)
    if loop[2] > 0 and not 0 <= loop[0] < loop[1] <= len(layers):
        raise ValueError("loop: start < stop must lie inside the layer list")
    return StackSpec("Motolix", int(cfg["vocab"]), int(cfg["width"]), layers, 0, float((cfg.get("norm") or {}).get("eps", 1e-5)),
                     "layer", float((cfg.get("embedding") or {}).get("scale", 1.0)), float(cfg.get("logit_scale", 1.0)), loop)


def fakonex_spec(cfg: dict) -> StackSpec:
    """Fakonex's config.json -> StackSpec: every size and constant from the file.  What the file leaves out is off: a mixer
    without `mask` sees the whole past, a router without `groups` chooses among all experts, a feed-forward without `shared`
    has no shared expert, a model without `logit_softcap` no cap."""
    layers = []
    for i, ly in enumerate(cfg["layers"]):
        kind, mx = ly["type"], ly["mixer"]
        if kind != "attention":
            raise ValueError(f"layer {i}: unknown mixer type {kind!r}")
        L = LayerSpec("attention")
        L.heads, L.kv_heads, L.dim, L.vdim = int(mx["heads"]), int(mx["kv_heads"]), int(mx["dim"]), int(mx["vdim"])
        if L.heads % L.kv_heads:
            raise ValueError(f"layer {i}: heads must be a multiple of kv_heads")
        L.scale = float(mx["scale"])
        L.attn_flags = B.ATTN_BIAS_QKV | B.ATTN_QK_NORM_HEAD | B.ATTN_SINK | B.ATTN_GATE
        mask = mx.get("mask") or {}
        L.mask_chunk = int(mask.get("size", 0))
        kf = mx.get("kv_from")
        L.kv_from = -1 if kf is None else int(kf)
        if L.kv_from >= 0:
            if L.kv_from >= i or layers[L.kv_from].kv_from >= 0:
                raise ValueError(f"layer {i}: kv_from must name an earlier layer that projects its own keys and values")
            src = layers[L.kv_from]
            if (src.kv_heads, src.dim, src.vdim) != (L.kv_heads, L.dim, L.vdim):
                raise ValueError(f"layer {i}: the layer named by kv_from has other key/value heads or sizes")
        ml = ly.get("mlp")
        if ml is not None:
            if ml.get("kind") != "moe":
                raise ValueError(f"layer {i}: unknown feed-forward kind {ml.get('kind')!r}")
            r = ml["router"]
            L.mlp, L.mlp_act, L.ff = "moe", "silu", int(ml["expert"]["ff"])
            L.experts, L.top, L.route = int(r["experts"]), int(r["top"]), "sigmoid_groups"
            gr = r.get("groups")
            if gr:
                L.route_groups, L.route_keep = int(gr["count"]), int(gr["keep"])
                if L.route_groups < 1 or L.experts % L.route_groups or not 1 <= L.route_keep <= L.route_groups:
                    raise ValueError(f"layer {i}: groups.count must divide experts and 1 <= groups.keep <= groups.count")
                if L.route_keep * (L.experts // L.route_groups) < L.top:
                    raise ValueError(f"layer {i}: the kept groups hold fewer experts than top")
            sh = ml.get("shared")
            if sh:
                L.shared_ff = int(sh["ff"])
        layers.append(L)
    return StackSpec("Fakonex", int(cfg["vocab"]), int(cfg["width"]), layers, 0, float((cfg.get("norm") or {}).get("eps", 1e-5)),
                     "rms", logit_softcap=float(cfg.get("logit_softcap") or 0.0))


def goperax_spec(cfg: dict) -> StackSpec:
    """Goperax's config.json -> StackSpec: every size and every constant that may differ between models comes from the file;
    what the design fixes (the base of the position vector, the activation, the unit sink) is set here.  A part the file
    leaves out is off: no `mask` = the whole past, no `softcap` = none, no `shared` = no shared unit, no `loop` = every layer
    once, no `streams` = one plain residual."""
    layers = []
    for i, ly in enumerate(cfg["layers"]):
        kind, mx = ly["type"], ly["mixer"]
        if kind == "attention":
            L = LayerSpec("attention")
            L.heads, L.kv_heads, L.dim, L.vdim = int(mx["heads"]), int(mx["kv_heads"]), int(mx["dim"]), int(mx["vdim"])
            if L.heads % L.kv_heads:
                raise ValueError(f"layer {i}: heads must be a multiple of kv_heads")
            if L.vdim != L.dim:
                raise ValueError(f"layer {i}: the values are the keys, so vdim must equal dim")
            L.scale = float(mx["scale"])
            L.attn_flags = B.ATTN_V_IS_K | B.ATTN_SINK_UNIT
            L.mask_window = int((mx.get("mask") or {}).get("size", 0))
            L.score_softcap = float(mx.get("softcap") or 0.0)
        elif kind == "mamba2":
            L = LayerSpec("ssm")
            L.heads, L.vdim, L.ssm_state, L.ssm_groups = int(mx["heads"]), int(mx["vdim"]), int(mx["state"]), int(mx["groups"])
            L.conv_taps, L.ssm_norm_groups = int(mx["conv"]), int(mx.get("norm_groups", 1))
            if L.ssm_groups < 1 or L.heads % L.ssm_groups:
                raise ValueError(f"layer {i}: heads must be a multiple of groups")
            if L.ssm_norm_groups < 1 or (L.heads * L.vdim) % L.ssm_norm_groups:
                raise ValueError(f"layer {i}: norm_groups must divide heads * vdim")
        else:
            raise ValueError(f"layer {i}: unknown mixer type {kind!r}")
        ml = ly.get("mlp")
        if ml is not None:
            L.mlp_act = "relu2"
            if ml.get("kind") == "dense":
                L.mlp, L.ff = "dense", int(ml["ff"])
            elif ml.get("kind") == "moe":
                L.mlp, L.ff, L.route = "moe", int(ml["expert"]["ff"]), "softmax_all"
                L.experts, L.top = int(ml["router"]["experts"]), int(ml["router"]["top"])
                sh = ml.get("shared")
                if sh:
                    L.shared_ff, L.shared_plain = int(sh["ff"]), True
            else:
                raise ValueError(f"layer {i}: unknown feed-forward kind {ml.get('kind')!r}")
        layers.append(L)
    lp = cfg.get("loop")
    loop = (int(lp["start"]), int(lp["stop"]), int(lp["times"])) if lp and int(lp.get("times", 0)) > 0 else (0, 0, 0)
    if loop[2] > 0 and not 0 <= loop[0] < loop[1] <= len(layers):
        raise ValueError("loop: start < stop must lie inside the layer list")
    return StackSpec("Goperax", int(cfg["vocab"]), int(cfg["width"]), layers, 0, float((cfg.get("norm") or {}).get("eps", 1e-5)), "rms",
                     embed_scale=float((cfg.get("embedding") or {}).get("scale", 1.0)), loop=loop, pre_norm=True,
                     streams=int(cfg.get("streams") or 0), pos_sinus=True, pos_base=10000.0, loop_plain=True, tied_head=True)


def llama_shape(cfg: dict):
    """A Hugging Face style Llama config.json -> ModelShape."""
    from .worker import ModelShape
    nh = int(cfg["num_attention_heads"])
    return ModelShape(int(cfg["vocab_size"]), int(cfg["hidden_size"]), int(cfg["num_hidden_layers"]), nh,
                      int(cfg.get("num_key_value_heads", nh)), int(cfg.get("head_dim", int(cfg["hidden_size"]) // nh)),
                      int(cfg["intermediate_size"]), int(cfg.get("max_position_embeddings", 8192)),
                      float(cfg.get("rope_theta", 10000.0)), float(cfg.get("rms_norm_eps", 1e-5)))


# architecture name -> (family, configuration reader)
ARCHITECTURES: Dict[str, Tuple[str, Callable[..., object]]] = {
    "Kidolorn": ("stack", kidolorn_spec),
    "Motolix": ("stack", motolix_spec),
    "Fakonex": ("stack", fakonex_spec),
    "Goperax": ("stack", goperax_spec),
    "LlamaForCausalLM": ("llama", llama_shape),
    "llama": ("llama", llama_shape),
}


def architecture_of(cfg: dict) -> str:
    name = cfg.get("architecture") or (cfg.get("architectures") or [None])[0] or cfg.get("model_type")
    if name not in ARCHITECTURES:
        raise ValueError(f"config.json names architecture {name!r}; known: {sorted(ARCHITECTURES)}")
    return name


def read_config(model_dir: str):
    """(family, description) of the model in `model_dir`."""
    cfg = json.load(open(os.path.join(model_dir, "config.json")))
    family, reader = ARCHITECTURES[architecture_of(cfg)]
    if reader is motolix_spec:
        st = os.path.join(model_dir, "model.safetensors")
        return family, reader(cfg, safetensors_shapes(st) if os.path.exists(st) else None)
    return family, reader(cfg)


def safetensors_shapes(path: str) -> Dict[str, Tuple[int, ...]]:
    """name -> shape of every tensor of a safetensors file (the header only)."""
    with open(path, "rb") as f:
        n = struct.unpack("<Q", f.read(8))[0]
        header = json.loads(f.read(n))
    return {k: tuple(int(d) for d in v["shape"]) for k, v in header.items() if k != "__metadata__"}


_ST_DTYPES = {"BF16": (np.uint16, B.BF16), "F32": (np.float32, B.F32), "I32": (np.int32, None)}


def read_safetensors(path: str) -> Iterator[Tuple[str, np.ndarray, Optional[int], Tuple[int, ...]]]:
    """Tensors of a safetensors file: (name, flat array, engine dtype code or None, shape).  The file is an 8-byte
    little-endian header length, that many bytes of JSON (name -> dtype, shape, data_offsets), then the data; bfloat16
    comes back as its uint16 bit patterns."""
    with open(path, "rb") as f:
        n = struct.unpack("<Q", f.read(8))[0]
        header = json.loads(f.read(n))
        mm = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ)
    base = 8 + n
    for name, info in header.items():
        if name == "__metadata__":
            continue
        if info["dtype"] not in _ST_DTYPES:
            raise ValueError(f"{name}: dtype {info['dtype']} is not supported")
        npdt, code = _ST_DTYPES[info["dtype"]]
        a, e = info["data_offsets"]
        arr = np.frombuffer(mm, dtype=npdt, count=(e - a) // np.dtype(npdt).itemsize, offset=base + a)
        yield name, arr, code, tuple(int(d) for d in info["shape"])


_LLAMA_NAMES = {"input_layernorm.weight": B.T_ATTN_NORM, "self_attn.q_proj.weight": B.T_WQ, "self_attn.k_proj.weight": B.T_WK,
                "self_attn.v_proj.weight": B.T_WV, "self_attn.o_proj.weight": B.T_WO, "post_attention_layernorm.weight": B.T_MLP_NORM,
                "mlp.gate_proj.weight": B.T_WGATE, "mlp.up_proj.weight": B.T_WUP, "mlp.down_proj.weight": B.T_WDOWN}


def load_model(model_dir: str, dtype: str = "bfloat16", max_batch: int = 32, max_tokens: int = 0, page_size: int = 64,
               max_step_tokens: int = 0, max_logit_rows: int = 0, max_ctx: int = 0, device: int = 0, flags: int = 0,
               eos_token: int = -1):
    """Create an engine for the model in `model_dir`, load its weights and finalize it.

    max_tokens: tokens the cache pool holds (rounded up to pages); 0 = a share of free memory.  dtype float32 is available
    for layer-list models only."""
    from .worker import Engine, WorkerConfig
    family, desc = read_config(model_dir)
    if dtype not in ("bfloat16", "float32"):
        raise ValueError("dtype must be bfloat16 or float32")
    pages = (max_tokens + page_size - 1) // page_size if max_tokens > 0 else 0
    st = os.path.join(model_dir, "model.safetensors")
    if family == "stack":
        ctx = max_ctx or (max_tokens + page_size if max_tokens > 0 else 8192)
        eng = Engine(WorkerConfig(None, device=device, max_batch=max_batch, max_step_tokens=max_step_tokens, page_size=page_size,
                                  kv_pages=pages, flags=flags, eos_token=eos_token, stack=desc, context_size=ctx,
                                  compute_dtype=dtype, max_logit_rows=max_logit_rows))
        want = desc.tensor_shapes()
        for name, arr, code, shape in read_safetensors(st):
            if name not in want:
                raise ValueError(f"{st}: tensor {name!r} is not part of this configuration")
            if code is None:
                raise ValueError(f"{st}: {name!r} is an integer table; this design has none")
            eng.load_named(name, arr, shape)
        eng.finalize()
        return eng
    if dtype != "bfloat16":
        raise ValueError("the Llama engine computes in bfloat16 only")
    import dataclasses
    shape = dataclasses.replace(desc, max_ctx=max_ctx) if max_ctx else desc
    eng = Engine(WorkerConfig(shape, device=device, max_batch=max_batch, max_step_tokens=max_step_tokens, page_size=page_size,
                              kv_pages=pages, flags=flags, eos_token=eos_token))
    seen_head = False
    for name, arr, code, _ in read_safetensors(st):
        if code is None:
            continue
        if name == "model.embed_tokens.weight":
            eng.load_tensor(B.T_EMBED, 0, arr)
        elif name == "model.norm.weight":
            eng.load_tensor(B.T_FINAL_NORM, 0, arr)
        elif name == "lm_head.weight":
            eng.load_tensor(B.T_LM_HEAD, 0, arr)
            seen_head = True
        elif name.startswith("model.layers."):
            _, _, li, rest = name.split(".", 3)
            if rest in _LLAMA_NAMES:
                eng.load_tensor(_LLAMA_NAMES[rest], int(li), arr)
    if not seen_head:  # tied embeddings
        for name, arr, code, _ in read_safetensors(st):
            if name == "model.embed_tokens.weight":
                eng.load_tensor(B.T_LM_HEAD, 0, arr)
    eng.finalize()
    return eng


def random_tensors(spec: StackSpec, seed: int = 0, scale: float = 1.0) -> Dict[str, np.ndarray]:
    """Random float32 weights for a layer-list model (benchmarks and tests): matrices ~ N(0, 1/fan_in), gains and
    convolution taps small, rounded to bfloat16-representable values so that every compute dtype sees the same model."""
    rng = np.random.default_rng(seed)
    out = {}
    for name, shape in spec.tensor_shapes().items():
        leaf = name.rsplit(".", 1)[-1]
        if shape == ():
            a = np.asarray(rng.uniform(0.5, 1.5), np.float32)
        elif leaf in ("norm1", "norm1b", "norm2", "norm2b") or name == "final.norm" or name.endswith(("q.norm", "k.norm")):
            a = rng.uniform(0.5, 1.5, shape).astype(np.float32)
        elif leaf == "temp":
            a = rng.uniform(0.5, 1.5, shape).astype(np.float32)
        elif leaf == "pb":
            a = rng.normal(-2.0, 1.0, shape).astype(np.float32)
        elif name == "loop.step":
            a = rng.normal(0, 0.3, shape).astype(np.float32)
        elif name.endswith("a2.b"):
            a = rng.normal(2.0, 1.5, shape).astype(np.float32)
        elif leaf.startswith("canon"):
            a = rng.normal(0, 0.3, shape).astype(np.float32)
        elif leaf in ("norm",) or name.endswith("dkv.norm"):
            a = rng.uniform(0.5, 1.5, shape).astype(np.float32)
        elif leaf == "sink":
            a = rng.normal(0, 1.0, shape).astype(np.float32)
        elif leaf == "correction":
            a = rng.normal(0, 0.3, shape).astype(np.float32)
        elif ".hc" in name:  # stream coefficients: readers and writers near 1 / S and 1, mixers near the identity
            n = shape[0]
            a = {"in": rng.normal(1.0 / n, 0.1, shape), "out": rng.normal(1.0, 0.2, shape),
                 "mix": np.eye(n) + rng.normal(0, 0.1, shape)}[leaf].astype(np.float32)
        elif leaf == "dt_bias":
            a = rng.normal(-1.0, 1.0, shape).astype(np.float32)
        elif leaf == "A_log":
            a = rng.uniform(-2.0, 1.0, shape).astype(np.float32)
        elif leaf == "D":
            a = rng.normal(1.0, 0.3, shape).astype(np.float32)
        elif leaf == "conv":
            a = rng.normal(0, 0.5, shape).astype(np.float32)
        elif leaf == "b":
            a = rng.normal(0, 0.3, shape).astype(np.float32)
        elif name in ("embed",):
            a = rng.normal(0, 1.0, shape).astype(np.float32)
        else:
            a = (rng.standard_normal(shape, dtype=np.float32) * np.float32(scale / np.sqrt(shape[-1])))
        out[name] = bf16_round(a)
    return out


def bf16_round(a: np.ndarray) -> np.ndarray:
    """float32 values rounded to the nearest bfloat16 (ties to even), returned as float32."""
    u = np.ascontiguousarray(a, np.float32).view(np.uint32).astype(np.uint64)
    u = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16
    return u.astype(np.uint32).view(np.float32).reshape(np.shape(a))
