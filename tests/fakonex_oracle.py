"""Plain float64 restatement of the Fakonex design, one function per mechanism, written for the tests only.  It shares no
code with the engine: numpy on the CPU, attention token by token over explicit lists of keys and values, experts looked up
per token.  Tensors come as a dict name -> array (names as in the model file).

Notation: W width of the residual, H query heads, G key/value heads, d query/key size, dv value size, c chunk length,
E experts, k experts per token.
"""
import numpy as np


def rms_norm(v, gain, eps):
    """v / sqrt(mean(v^2) + eps) * gain over the last axis."""
    v = np.asarray(v, np.float64)
    return v / np.sqrt(np.mean(v * v, axis=-1, keepdims=True) + eps) * gain


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-np.asarray(z, np.float64)))


def visible(i, j, chunk):
    """May position i look at position j?  Causal, and -- with a chunk length -- only inside i's own chunk, chunks being
    [0, c), [c, 2c), ... of the sequence."""
    if j > i:
        return False
    return chunk <= 0 or i // chunk == j // chunk


def sink_softmax(scores, sink):
    """Softmax weights of the listed scores when one more logit `sink` sits in the denominator (it has no value)."""
    scores = np.asarray(scores, np.float64)
    m = max(float(scores.max()), float(sink))
    e = np.exp(scores - m)
    return e / (e.sum() + np.exp(sink - m))


def attention(mx, P, p, h, eps, caches, layer):
    """The mixer of one layer on its input h [T][W].  caches[layer] receives (keys, values) as this layer would cache them;
    a layer with kv_from reads caches[kv_from] instead of projecting."""
    T = h.shape[0]
    H, G, d, dv = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
    q = (h @ P[p + "q"].T + P[p + "q.b"]).reshape(T, H, d)
    q = rms_norm(q, P[p + "q.norm"], eps)
    src = mx.get("kv_from")
    if src is None:
        k = rms_norm((h @ P[p + "k"].T + P[p + "k.b"]).reshape(T, G, d), P[p + "k.norm"], eps)
        v = (h @ P[p + "v"].T + P[p + "v.b"]).reshape(T, G, dv)
        caches[layer] = (k, v)
    else:
        k, v = caches[src]
    chunk = int((mx.get("mask") or {}).get("size", 0))
    gate = sigmoid(h @ P[p + "g"].T)  # [T][H]
    out = np.zeros((T, H, dv))
    for i in range(T):
        seen = [j for j in range(T) if visible(i, j, chunk)]
        for hd in range(H):
            g = hd // (H // G)
            s = np.array([q[i, hd] @ k[j, g] for j in seen]) * mx["scale"]
            w = sink_softmax(s, P[p + "sink"][hd])
            out[i, hd] = gate[i, hd] * sum(wj * v[j, g] for wj, j in zip(w, seen))
    return out.reshape(T, H * dv) @ P[p + "o"].T


def gated_unit(P, p, h):
    """W_down (silu(W_gate h) * (W_up h)) for one token or several."""
    g = h @ P[p + "gate"].T
    return (g * sigmoid(g) * (h @ P[p + "up"].T)) @ P[p + "down"].T


def choose_experts(scores, correction, top, groups=None):
    """Indices of the chosen experts of ONE token, best first.  scores: sigmoid of the router logits [E]; c = scores +
    correction decides.  groups = (count, keep): indices [g * E/count, (g + 1) * E/count) form block g, a block ranks by the
    sum of its top two c, and only members of the `keep` best blocks may be picked."""
    c = np.asarray(scores, np.float64) + np.asarray(correction, np.float64)
    E = len(c)
    allowed = np.ones(E, bool)
    if groups:
        count, keep = groups
        per = E // count
        gscore = [np.sort(c[g * per:(g + 1) * per])[-2:].sum() for g in range(count)]
        best = sorted(range(count), key=lambda g: (-gscore[g], g))[:keep]
        allowed = np.array([e // per in best for e in range(E)])
    order = sorted((e for e in range(E) if allowed[e]), key=lambda e: (-c[e], e))
    return order[:top]


def mixture(ml, P, p, h):
    """The feed-forward of one layer on its input h [T][W]."""
    r = ml["router"]
    gr = r.get("groups")
    y = np.zeros_like(h)
    for t in range(h.shape[0]):
        s = sigmoid(P[p + "router"] @ h[t])
        chosen = choose_experts(s, P[p + "correction"], r["top"], (gr["count"], gr["keep"]) if gr else None)
        total = sum(s[e] for e in chosen) + 1e-20
        for e in chosen:
            y[t] += s[e] / total * gated_unit(P, f"{p}e{e}.", h[t])
        if ml.get("shared"):
            y[t] += sigmoid(P[p + "shared.sg"] @ h[t])[0] * gated_unit(P, p + "shared.", h[t])
    return y


def soft_cap(z, cap):
    return cap * np.tanh(z / cap) if cap else z


def forward(cfg, W, tokens, layers_out=None):
    """Logits [T][vocab] of the token sequence; layers_out (a list) receives the residual after every layer."""
    P = {k: np.asarray(v, np.float64) for k, v in W.items()}
    eps = cfg["norm"]["eps"]
    x = P["embed"][np.asarray(tokens, np.int64)]
    caches = {}
    for i, ly in enumerate(cfg["layers"]):
        p = f"l{i}."
        a = attention(ly["mixer"], P, p + "mix.", rms_norm(x, P[p + "norm1"], eps), eps, caches, i)
        x = x + rms_norm(a, P[p + "norm1b"], eps)
        if ly.get("mlp"):
            f = mixture(ly["mlp"], P, p + "mlp.", rms_norm(x, P[p + "norm2"], eps))
            x = x + rms_norm(f, P[p + "norm2b"], eps)
        if layers_out is not None:
            layers_out.append(x.copy())
    return soft_cap(rms_norm(x, P["final.norm"], eps) @ P["head"].T, cfg.get("logit_softcap"))
