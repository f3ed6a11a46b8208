"""Plain float64 restatement of the Goperax design, one function per mechanism, written for the tests only.  It shares no
code with the engine: numpy on the CPU, recurrences token by token, attention over explicit lists of visible keys, experts
looked up per token.  Tensors come as a dict name -> array (names as in the model file).

Notation: W width, S residual streams, H heads, G key/value heads (attention) or groups of the state-space mixer, d
query/key size, P value size of a state-space head, N state size, w window length, E experts, k experts per token.
"""
import numpy as np


def rms_norm(v, gain, eps):
    """v / sqrt(mean(v^2) + eps) * gain over the last axis."""
    v = np.asarray(v, np.float64)
    return v / np.sqrt(np.mean(v * v, axis=-1, keepdims=True) + eps) * gain


def silu(z):
    z = np.asarray(z, np.float64)
    return z / (1.0 + np.exp(-z))


def softplus(z):
    z = np.asarray(z, np.float64)
    return np.maximum(z, 0.0) + np.log1p(np.exp(-np.abs(z)))


def position_vector(p, width, base=10000.0):
    """Entry 2i = sin(p * base^(-2i/width)), entry 2i+1 = cos of the same angle."""
    out = np.zeros(width)
    for c in range(width):
        i = c // 2
        a = p * base ** (-2.0 * i / width)
        out[c] = np.sin(a) if c % 2 == 0 else np.cos(a)
    return out


def embedding(cfg, P, tokens, pos0=0):
    sc = float((cfg.get("embedding") or {}).get("scale", 1.0))
    W = cfg["width"]
    return np.stack([np.asarray(P["embed"][t], np.float64) * sc + position_vector(pos0 + n, W) for n, t in enumerate(tokens)])


def window_visible(i, j, window):
    """Position i sees j iff 0 <= i - j < window (window <= 0: the whole past)."""
    return j <= i and (window <= 0 or i - j < window)


def capped(score, cap):
    return score if not cap else cap * np.tanh(score / cap)


def unit_sink_weights(scores):
    """exp(s_j) / (1 + sum_j exp(s_j)): a softmax with one more term of logit 0 in the denominator."""
    scores = np.asarray(scores, np.float64)
    m = max(float(scores.max()), 0.0)
    e = np.exp(scores - m)
    return e / (e.sum() + np.exp(-m))


def attention(mx, P, p, h):
    """Grouped-query attention whose values are its keys, no positions in the scores, a soft cap on the scaled scores, a
    sliding window and the unit sink.  h [T][W] -> [T][W]."""
    T = h.shape[0]
    H, G, d = mx["heads"], mx["kv_heads"], mx["dim"]
    window = int((mx.get("mask") or {}).get("size", 0))
    cap = float(mx.get("softcap") or 0.0)
    q = (h @ P[p + "q"].T).reshape(T, H, d)
    k = (h @ P[p + "k"].T).reshape(T, G, d)
    out = np.zeros((T, H, mx["vdim"]))
    for i in range(T):
        seen = [j for j in range(T) if window_visible(i, j, window)]
        for hd in range(H):
            g = hd // (H // G)
            s = np.array([capped(q[i, hd] @ k[j, g] * mx["scale"], cap) for j in seen])
            wts = unit_sink_weights(s)
            out[i, hd] = sum(wj * k[j, g] for wj, j in zip(wts, seen))
    return out.reshape(T, -1) @ P[p + "o"].T


def causal_conv_silu(u, taps_w, bias):
    """u [T][C]; taps_w [C][taps] with the last column weighing the current token; zeros before the start."""
    T, C = u.shape
    taps = taps_w.shape[1]
    out = np.zeros((T, C))
    for t in range(T):
        acc = np.array(bias, np.float64)
        for j in range(taps):
            src = t - (taps - 1 - j)
            if src >= 0:
                acc = acc + taps_w[:, j] * u[src]
        out[t] = silu(acc)
    return out


def state_space(mx, P, p, h, eps):
    """The selective state-space mixer, token by token.  Per head a matrix S [N][P], decayed by exp(-exp(A_log) dt) and fed
    dt * B x^T; read out through C, plus D x; gated by silu(z), then normalised in norm_groups equal parts."""
    T = h.shape[0]
    H, Pd, N, G = mx["heads"], mx["vdim"], mx["state"], mx["groups"]
    inner = H * Pd
    proj = h @ P[p + "in"].T
    z, rest, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    rest = causal_conv_silu(rest, np.asarray(P[p + "conv"], np.float64), np.asarray(P[p + "conv.b"], np.float64))
    x = rest[:, :inner].reshape(T, H, Pd)
    Bm = rest[:, inner:inner + G * N].reshape(T, G, N)
    Cm = rest[:, inner + G * N:].reshape(T, G, N)
    dt = softplus(dt + P[p + "dt_bias"])
    A = -np.exp(np.asarray(P[p + "A_log"], np.float64))
    S = np.zeros((H, N, Pd))
    y = np.zeros((T, H, Pd))
    for t in range(T):
        for hd in range(H):
            g = hd // (H // G)
            S[hd] = np.exp(A[hd] * dt[t, hd]) * S[hd] + dt[t, hd] * np.outer(Bm[t, g], x[t, hd])
            y[t, hd] = S[hd].T @ Cm[t, g] + P[p + "D"][hd] * x[t, hd]
    y = y.reshape(T, inner) * silu(z)
    parts = int(mx.get("norm_groups", 1))
    y = rms_norm(y.reshape(T, parts, inner // parts), 1.0, eps).reshape(T, inner) * P[p + "norm"]
    return y @ P[p + "o"].T


def relu_squared_unit(P, p, h):
    """W_down relu(W_up h)^2."""
    u = np.maximum(h @ P[p + "up"].T, 0.0)
    return (u * u) @ P[p + "down"].T


def choose_experts(logits, top):
    """(indices, weights) of one token: softmax over all experts, the `top` largest scores (lowest index wins a tie), the
    chosen scores divided by their sum."""
    z = np.asarray(logits, np.float64)
    s = np.exp(z - z.max())
    s = s / s.sum()
    order = sorted(range(len(s)), key=lambda e: (-s[e], e))[:top]
    wsum = sum(s[e] for e in order) + 1e-20
    return order, [s[e] / wsum for e in order]


def mixture(ml, P, p, h):
    T = h.shape[0]
    out = np.zeros((T, P[p + "e0.down"].shape[0]))
    z = h @ np.asarray(P[p + "router"], np.float64).T
    for t in range(T):
        idx, wt = choose_experts(z[t], int(ml["router"]["top"]))
        for e, w in zip(idx, wt):
            out[t] += w * relu_squared_unit(P, f"{p}e{e}.", h[t])
    if ml.get("shared"):
        out += relu_squared_unit(P, p + "shared.", h)
    return out


def layer_order(cfg):
    n = len(cfg["layers"])
    lp = cfg.get("loop")
    if not lp or int(lp.get("times", 0)) <= 0:
        return list(range(n))
    a, b, k = int(lp["start"]), int(lp["stop"]), int(lp["times"])
    return list(range(a)) + list(range(a, b)) * k + list(range(b, n))


def forward(cfg, P, tokens, upto=None):
    """Logits [T][vocab] of one sequence and the residual (the sum of the streams) after every layer run."""
    P = {k: np.asarray(v, np.float64) for k, v in P.items()}
    eps = float(cfg["norm"]["eps"])
    S = int(cfg.get("streams") or 0)
    x0 = embedding(cfg, P, tokens)
    xs = [x0.copy() for _ in range(max(S, 1))]
    trail = []
    runs = layer_order(cfg)
    for li in runs[:upto]:
        ly = cfg["layers"][li]
        pre = f"l{li}."
        subs = [(1, lambda h, ly=ly, pre=pre: attention(ly["mixer"], P, pre + "mix.", h) if ly["type"] == "attention"
                 else state_space(ly["mixer"], P, pre + "mix.", h, eps))]
        if ly.get("mlp"):
            ml = ly["mlp"]
            subs.append((2, lambda h, ml=ml, pre=pre: relu_squared_unit(P, pre + "mlp.", h) if ml["kind"] == "dense"
                         else mixture(ml, P, pre + "mlp.", h)))
        for q, fn in subs:
            if S:
                hin, hmix, hout = P[f"{pre}hc{q}.in"], P[f"{pre}hc{q}.mix"], P[f"{pre}hc{q}.out"]
                u = sum(hin[s] * xs[s] for s in range(S))
                y = fn(rms_norm(u, P[f"{pre}norm{q}"], eps))
                xs = [sum(hmix[s, t] * xs[s] for s in range(S)) + hout[t] * y for t in range(S)]
            else:
                xs = [xs[0] + fn(rms_norm(xs[0], P[f"{pre}norm{q}"], eps))]
        trail.append(sum(xs))
    x = sum(xs)
    logits = rms_norm(x, P["final.norm"], eps) @ P["embed"].T
    return logits, trail
