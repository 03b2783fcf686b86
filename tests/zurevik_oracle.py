"""Slow float64 restatement of the Zurevik design of the hybrid decoder family, one function per mechanism, used only by the tests.

A layer adds mixer(norm1(x)) + experts(norm2(x)) to the residual x, both norms RMS norms of the same x.  The mixers are windowed softmax
attention in two variants: a differential one (two score maps per head over the same values, a1 - lambda a2, unit RMS per head, per-channel
sigmoid gate, RMS-normed queries and keys, a sliding window that also keeps the first tokens of the sequence) and one with projection biases,
a per-head sink in the softmax denominator, a per-head sigmoid gate, and optionally the keys and values of an earlier layer.  The experts
are gate-less squared-ReLU layers weighted by the softmax over the chosen router logits.  Everything is computed for a whole sequence at
once with explicit masks; there is no cache, no page and no state, and nothing is shared with the CUDA path."""
import math

import numpy as np

from hybrid_oracle import bf16_round, rel_err, sigmoid, write_checkpoint  # noqa: F401  (helpers of the test side only)

F = np.float64


# ---- mechanisms --------------------------------------------------------------------------------------------------------------
def rms_norm(x, w, eps):
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps) * w


def visible(T, window, keep_first=0):
    """[T, T] bool: query i sees key j"""
    i, j = np.arange(T)[:, None], np.arange(T)[None, :]
    return (j <= i) & ((i - j < window) | (j < keep_first))


def masked_softmax(s, vis, sink=None):
    """softmax over the visible keys of each row; `sink` (a scalar) enlarges the denominator only"""
    s = np.where(vis, s, -np.inf)
    m = s.max(-1, keepdims=True)
    if sink is not None:
        m = np.maximum(m, sink)
    e = np.exp(s - m)
    den = e.sum(-1, keepdims=True)
    if sink is not None:
        den = den + np.exp(sink - m)
    return e / den


def differential_attention(h, W, p, m, eps):
    T = h.shape[0]
    H, G, d, vd = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rms_norm((h @ W[p + "q"].T).reshape(T, H, 2, d), W[p + "q.norm"], eps)
    k = rms_norm((h @ W[p + "k"].T).reshape(T, G, 2, d), W[p + "k.norm"], eps)
    v = (h @ W[p + "v"].T).reshape(T, G, vd)
    vis = visible(T, m["mask"]["size"], m["mask"].get("keep_first", 0))
    lam = math.exp(float(W[p + "lq1"] @ W[p + "lk1"])) - math.exp(float(W[p + "lq2"] @ W[p + "lk2"])) + m["diff"]
    out = np.zeros((T, H, vd), F)
    for hd in range(H):
        g = hd // (H // G)
        a = [masked_softmax(q[:, hd, mp] @ k[:, g, mp].T * m["scale"], vis) @ v[:, g] for mp in range(2)]
        o = a[0] - lam * a[1]
        out[:, hd] = o / np.sqrt((o * o).mean(-1, keepdims=True) + eps) * (1.0 - m["diff"])
    return (out.reshape(T, H * vd) * sigmoid(h @ W[p + "g"].T)) @ W[p + "o"].T


def sink_attention(h, W, p, m, kv):
    """kv: (k, v) of the layer this one reads, or None: then the layer's own projections, which are returned for later layers"""
    T = h.shape[0]
    H, G, d, vd = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ W[p + "q"].T + W[p + "q.b"]).reshape(T, H, d)
    if kv is None:
        kv = ((h @ W[p + "k"].T + W[p + "k.b"]).reshape(T, G, d), (h @ W[p + "v"].T + W[p + "v.b"]).reshape(T, G, vd))
    k, v = kv
    vis = visible(T, m["mask"]["size"])
    gate = sigmoid(h @ W[p + "g"].T)
    out = np.zeros((T, H, vd), F)
    for hd in range(H):
        g = hd // (H // G)
        out[:, hd] = masked_softmax(q[:, hd] @ k[:, g].T * m["scale"], vis, W[p + "sink"][hd]) @ v[:, g] * gate[:, hd:hd + 1]
    return out.reshape(T, H * vd) @ W[p + "o"].T, kv


def route(h, W, p, m):
    """-> chosen experts [T, top] (largest logit first) and their weights: softmax over the chosen logits only"""
    z = h @ W[p + "router"].T + W[p + "router.b"]
    idx = np.argsort(-z, -1, kind="stable")[:, :m["router"]["top"]]
    zc = np.take_along_axis(z, idx, -1)
    e = np.exp(zc - zc.max(-1, keepdims=True))
    return idx, e / e.sum(-1, keepdims=True)


def experts(h, W, p, m):
    idx, wgt = route(h, W, p, m)
    y = np.zeros_like(h)
    for t in range(h.shape[0]):
        for c in range(idx.shape[1]):
            e = idx[t, c]
            y[t] += wgt[t, c] * (W[p + "e%d.down" % e] @ np.maximum(W[p + "e%d.up" % e] @ h[t], 0.0) ** 2)
    return y


def forward(cfg, W, tokens, layers_out=None):
    """logits [T, vocab] of one sequence"""
    eps = cfg["norm"]["eps"]
    x = W["embed"][np.asarray(tokens)] * cfg["embedding"]["scale"]
    kvs = {}
    for i, l in enumerate(cfg["layers"]):
        p, m = "l%d." % i, l["mixer"]
        h = rms_norm(x, W[p + "norm1"], eps)
        if l["type"] == "attention":
            y = differential_attention(h, W, p + "mix.", m, eps)
        else:
            y, kvs[i] = sink_attention(h, W, p + "mix.", m, kvs[m["kv_from"]] if m.get("kv_from") is not None else None)
        if l.get("mlp"):
            y = y + experts(rms_norm(x, W[p + "norm2"], eps), W, p + "mlp.", l["mlp"])
        x = x + y
        if layers_out is not None:
            layers_out.append(x.copy())
    lg = rms_norm(x, W["final.norm"], eps) @ W["head"].T
    cap = cfg.get("logit_softcap")
    return cap * np.tanh(lg / cap) if cap else lg


# ---- random checkpoints ------------------------------------------------------------------------------------------------------
def diff_layer(heads=4, kv_heads=2, dim=8, vdim=24, window=20, keep_first=3, diff=0.3, mlp=None):
    return {"type": "attention", "mlp": mlp,
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "diff": diff, "scale": dim ** -0.5, "mask": {"size": window, "keep_first": keep_first}}}


def sink_layer(heads=4, kv_heads=2, dim=16, vdim=8, window=30, kv_from=None, mlp=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": dim ** -0.5, "mask": {"size": window}}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "attention_2", "mlp": mlp, "mixer": m}


def moe(experts=6, top=2, ff=24):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def make_config(layers, width=48, vocab=80, eps=1e-5, embed_scale=2.0, softcap=20.0):
    c = {"architecture": "Zurevik", "width": width, "vocab": vocab, "norm": {"eps": eps}, "embedding": {"scale": embed_scale}, "layers": layers}
    if softcap:
        c["logit_softcap"] = softcap
    return c


def random_weights(cfg, seed, sharp=1.0):
    """float64 arrays holding bf16-representable values.  `sharp` scales the query projections so that single keys dominate a softmax."""
    rng = np.random.default_rng(seed)
    Wd, V = cfg["width"], cfg["vocab"]
    W = {}

    def mat(n, k, gain=1.0):
        return bf16_round(rng.standard_normal((n, k)) * gain / math.sqrt(k)).astype(F)

    def vec(n, mean, spread):
        return bf16_round(mean + spread * rng.standard_normal(n)).astype(F)

    W["embed"], W["head"], W["final.norm"] = mat(V, Wd, math.sqrt(Wd)), mat(V, Wd, 3.0), vec(Wd, 1.0, 0.2)
    for i, l in enumerate(cfg["layers"]):
        p, m = "l%d." % i, l["mixer"]
        q = p + "mix."
        H, G, d, vd = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        W[p + "norm1"] = vec(Wd, 1.0, 0.2)
        if l["type"] == "attention":
            W[q + "q"], W[q + "k"], W[q + "v"] = mat(H * 2 * d, Wd, 2.0), mat(G * 2 * d, Wd, 2.0), mat(G * vd, Wd, 2.0)
            W[q + "q.norm"], W[q + "k.norm"] = vec(d, sharp, 0.2 * sharp), vec(d, 1.0, 0.2)
            for n in ("lq1", "lk1", "lq2", "lk2"):
                W[q + n] = vec(d, 0.0, 0.5 / math.sqrt(math.sqrt(d)))
            W[q + "g"], W[q + "o"] = mat(H * vd, Wd, 2.0), mat(Wd, H * vd)
        else:
            W[q + "q"], W[q + "q.b"] = mat(H * d, Wd, 2.0 * sharp), vec(H * d, 0.0, 0.3)
            if m.get("kv_from") is None:
                W[q + "k"], W[q + "k.b"], W[q + "v"], W[q + "v.b"] = mat(G * d, Wd, 2.0), vec(G * d, 0.0, 0.3), mat(G * vd, Wd, 2.0), vec(G * vd, 0.0, 0.3)
            W[q + "sink"], W[q + "g"], W[q + "o"] = vec(H, 1.0, 1.5), mat(H, Wd, 2.0), mat(Wd, H * vd)
        if l.get("mlp"):
            r, ff, q = l["mlp"]["router"], l["mlp"]["expert"]["ff"], p + "mlp."
            W[p + "norm2"] = vec(Wd, 1.0, 0.2)
            W[q + "router"], W[q + "router.b"] = mat(r["experts"], Wd, 3.0), vec(r["experts"], 0.0, 0.5)
            for e in range(r["experts"]):
                W[q + "e%d.up" % e], W[q + "e%d.down" % e] = mat(ff, Wd, 1.5), mat(Wd, ff, 1.0)
    return W
