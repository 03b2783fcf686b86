"""Slow float64 restatement of the Ratasun hybrid decoder family, one function per mechanism, used only by the tests.

It processes a whole sequence at once with explicit per-token loops for the recurrences; it has no cache, no pages, no state slots and
shares nothing with the CUDA path.  Also here: a generator of small random checkpoints (config.json + model.safetensors in bf16) so that
the tests choose their own sizes."""
import json
import math
import os
import struct

import numpy as np

F = np.float64


# ---- small helpers -----------------------------------------------------------------------------------------------------------
def bf16_round(a):
    a = np.asarray(a, dtype=np.float32)
    u = a.view(np.uint32).astype(np.uint64)
    u = (u + 0x7FFF + ((u >> 16) & 1)) >> 16
    return (u.astype(np.uint32) << 16).view(np.float32)


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.where(z > 30, z, np.log1p(np.exp(np.minimum(z, 30))))


def layer_norm(x, w, eps):
    mu = x.mean(-1, keepdims=True)
    var = ((x - mu) ** 2).mean(-1, keepdims=True)
    return (x - mu) / np.sqrt(var + eps) * w


def rms_unit(x, eps):
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps)


def causal_conv_silu(x, w, b=None):
    """x [T, C], w [C, taps] (last column multiplies the current token), zeros before the sequence"""
    T, C = x.shape
    taps = w.shape[1]
    xp = np.concatenate([np.zeros((taps - 1, C), F), x])
    y = np.zeros((T, C), F)
    for j in range(taps):
        y += xp[j:j + T] * w[:, j]
    return silu(y if b is None else y + b)


def rotate_pairs(x, pos, base, dims):
    """rotary embedding on the first `dims` channels of the last axis, channel 2i paired with 2i+1; x [T, ..., d]"""
    i = np.arange(dims // 2, dtype=F)
    ang = np.asarray(pos, F)[:, None] * base ** (-2.0 * i / dims)
    c, s = np.cos(ang), np.sin(ang)
    while c.ndim < x.ndim:
        c, s = c[:, None], s[:, None]
    y = x.copy()
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    y[..., 0:dims:2] = u * c - v * s
    y[..., 1:dims:2] = v * c + u * s
    return y


# ---- mechanisms --------------------------------------------------------------------------------------------------------------
def route(h, W, p, m):
    """-> chosen experts [T, top] and their weights [T, top]"""
    r = m["router"]
    E, top, G, keep = r["experts"], r["top"], r["groups"]["count"], r["groups"]["keep"]
    s = sigmoid(h @ W[p + "router"].T)
    choice = s + W[p + "correction"]
    T = h.shape[0]
    idx, wgt = np.zeros((T, top), np.int64), np.zeros((T, top), F)
    for t in range(T):
        c = choice[t].copy()
        grp = c.reshape(G, E // G)
        score = np.sort(grp, axis=1)[:, -2:].sum(1) if E // G >= 2 else grp[:, 0]
        kept = np.argsort(-score, kind="stable")[:keep]
        allowed = np.zeros(G, bool)
        allowed[kept] = True
        c[~np.repeat(allowed, E // G)] = -np.inf
        ch = np.argsort(-c, kind="stable")[:top]
        w = s[t, ch]
        idx[t], wgt[t] = ch, w / (w.sum() + 1e-20) * r["scale"]
    return idx, wgt


def experts(h, W, p, m):
    idx, wgt = route(h, W, p, m)
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for e, w in zip(idx[t], wgt[t]):
            q = p + "e%d." % e
            out[t] += w * (W[q + "down"] @ (silu(W[q + "gate"] @ h[t]) * (W[q + "up"] @ h[t])))
    return out


def latent_attention(h, W, p, m, eps):
    T, H, d, r, vd, R = h.shape[0], m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    q = (h @ W[p + "q"].T).reshape(T, H, d + r)
    down = h @ W[p + "dkv"].T
    lat = rms_unit(down[:, :R], eps) * W[p + "dkv.norm"]
    pos = np.arange(T)
    q_rot = rotate_pairs(q[..., d:], pos, m["rot"]["base"], m["rot"]["dims"])
    k_rot = rotate_pairs(down[:, R:], pos, m["rot"]["base"], m["rot"]["dims"])
    k = (lat @ W[p + "uk"].T).reshape(T, H, d)
    v = (lat @ W[p + "uv"].T).reshape(T, H, vd)
    out = np.zeros((T, H, vd), F)
    for i in range(T):
        sc = (np.einsum("hd,jhd->hj", q[i, :, :d], k[:i + 1]) + q_rot[i] @ k_rot[:i + 1].T) * m["scale"]
        sc = np.exp(sc - sc.max(-1, keepdims=True))
        out[i] = np.einsum("hj,jhd->hd", sc / sc.sum(-1, keepdims=True), v[:i + 1])
    return out.reshape(T, H * vd) @ W[p + "o"].T


def channel_delta(h, W, p, m, eps):
    T, H, KH, d, vd = h.shape[0], m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = causal_conv_silu(h @ W[p + "q"].T, W[p + "q.conv"]).reshape(T, KH, d)
    k = causal_conv_silu(h @ W[p + "k"].T, W[p + "k.conv"]).reshape(T, KH, d)
    v = causal_conv_silu(h @ W[p + "v"].T, W[p + "v.conv"]).reshape(T, H, vd)
    q = q / np.sqrt((q * q).sum(-1, keepdims=True) + 1e-6) * d ** -0.5
    k = k / np.sqrt((k * k).sum(-1, keepdims=True) + 1e-6)
    beta = sigmoid(h @ W[p + "b"].T)
    rate = np.exp(W[p + "A_log"])
    decay = np.exp(-rate[None, :, None] * softplus(((h @ W[p + "a1"].T) @ W[p + "a2"].T + W[p + "dt_bias"]).reshape(T, H, d)))
    gate = sigmoid(((h @ W[p + "g1"].T) @ W[p + "g2"].T).reshape(T, H, vd))
    o = np.zeros((T, H, vd), F)
    for hd in range(H):
        S, kh = np.zeros((d, vd), F), hd // (H // KH)
        for t in range(T):
            S = decay[t, hd][:, None] * S
            u = beta[t, hd] * (v[t, hd] - S.T @ k[t, kh])
            S = S + np.outer(k[t, kh], u)
            o[t, hd] = S.T @ q[t, kh]
    o = rms_unit(o, eps) * W[p + "norm"] * gate
    return o.reshape(T, H * vd) @ W[p + "o"].T


def mamba2(h, W, p, m, eps):
    T, H, vd, N, G, NG = h.shape[0], m["heads"], m["vdim"], m["state"], m["groups"], m["norm_groups"]
    inner = H * vd
    zx = h @ W[p + "in"].T
    z, dt = zx[:, :inner], zx[:, 2 * inner + 2 * G * N:]
    xbc = causal_conv_silu(zx[:, inner:2 * inner + 2 * G * N], W[p + "conv"], W[p + "conv.b"])
    x, B, C = xbc[:, :inner].reshape(T, H, vd), xbc[:, inner:inner + G * N].reshape(T, G, N), xbc[:, inner + G * N:].reshape(T, G, N)
    dt = softplus(dt + W[p + "dt_bias"])
    rate = np.exp(W[p + "A_log"])
    y = np.zeros((T, H, vd), F)
    for hd in range(H):
        S, g = np.zeros((N, vd), F), hd // (H // G)
        for t in range(T):
            S = math.exp(-rate[hd] * dt[t, hd]) * S + dt[t, hd] * np.outer(B[t, g], x[t, hd])
            y[t, hd] = S.T @ C[t, g] + W[p + "D"][hd] * x[t, hd]
    y = (y.reshape(T, inner) * silu(z)).reshape(T, NG, inner // NG)
    return (rms_unit(y, eps).reshape(T, inner) * W[p + "norm"]) @ W[p + "o"].T


MIXERS = {"latent_attention": latent_attention, "channel_delta": channel_delta, "mamba2": mamba2}


def forward(cfg, W, tokens):
    """logits [T, vocab] of one sequence"""
    eps, L, loop = cfg["norm"]["eps"], cfg["layers"], cfg.get("loop")
    x0 = W["embed"][np.asarray(tokens)]
    x = x0.copy()

    def layer(i, x):
        p = "l%d." % i
        h = layer_norm(x, W[p + "norm1"], eps)
        y = MIXERS[L[i]["type"]](h, W, p + "mix.", L[i]["mixer"], eps)
        if L[i].get("mlp"):
            y = y + experts(h, W, p + "mlp.", L[i]["mlp"])
        return x + y

    i = 0
    while i < len(L):
        if loop and i == loop["start"]:
            for t in range(loop["times"]):
                x = np.concatenate([x, x0], -1) @ W["loop.in"].T + W["loop.step"][t]
                for j in range(loop["start"], loop["stop"]):
                    x = layer(j, x)
            i = loop["stop"]
        else:
            x = layer(i, x)
            i += 1
    return layer_norm(x, W["final.norm"], eps) @ W["head"].T * cfg.get("logit_scale", 1.0)


# ---- random checkpoints ------------------------------------------------------------------------------------------------------
def attention_layer(heads=2, dim=16, rot_dim=8, vdim=16, kv_rank=24, base=10000.0, mlp=None):
    return {"type": "latent_attention", "mlp": mlp,
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "scale": (dim + rot_dim) ** -0.5, "rot": {"base": base, "dims": rot_dim}}}


def delta_layer(heads=2, kv_heads=1, dim=16, vdim=24, conv=4, mlp=None):
    return {"type": "channel_delta", "mlp": mlp, "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}}


def mamba_layer(heads=4, vdim=8, state=16, groups=2, norm_groups=1, conv=2, mlp=None):
    return {"type": "mamba2", "mlp": mlp, "mixer": {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "norm_groups": norm_groups, "conv": conv}}


def moe(experts=6, top=2, groups=3, keep=2, ff=24, scale=1.5):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top, "scale": scale, "groups": {"count": groups, "keep": keep}}}


def make_config(layers, width=48, vocab=80, loop=None, eps=1e-5, logit_scale=1.0):
    c = {"architecture": "Ratasun", "width": width, "vocab": vocab, "norm": {"eps": eps}, "logit_scale": logit_scale, "layers": layers}
    if loop:
        c["loop"] = loop
    return c


def random_weights(cfg, seed, low_rank=8, sharp=1.0):
    """float64 arrays holding bf16-representable values.  `sharp` scales the attention queries so that single keys dominate a softmax."""
    rng = np.random.default_rng(seed)
    Wd, V = cfg["width"], cfg["vocab"]
    W = {}

    def mat(n, k, gain=1.0):
        return bf16_round(rng.standard_normal((n, k)) * gain / math.sqrt(k)).astype(F)

    def vec(n, mean, spread):
        return bf16_round(mean + spread * rng.standard_normal(n)).astype(F)

    W["embed"], W["head"], W["final.norm"] = mat(V, Wd, math.sqrt(Wd)), mat(V, Wd), vec(Wd, 1.0, 0.2)
    if cfg.get("loop"):
        W["loop.in"], W["loop.step"] = mat(Wd, 2 * Wd, 1.2), bf16_round(0.3 * rng.standard_normal((cfg["loop"]["times"], Wd))).astype(F)
    for i, l in enumerate(cfg["layers"]):
        p, m = "l%d." % i, l["mixer"]
        W[p + "norm1"] = vec(Wd, 1.0, 0.2)
        q = p + "mix."
        if l["type"] == "latent_attention":
            H, d, r, vd, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
            W[q + "q"], W[q + "dkv"], W[q + "dkv.norm"] = mat(H * (d + r), Wd, sharp), mat(R + r, Wd, 2.0), vec(R, 1.0, 0.2)
            W[q + "uk"], W[q + "uv"], W[q + "o"] = mat(H * d, R, 2.0), mat(H * vd, R), mat(Wd, H * vd)
        elif l["type"] == "channel_delta":
            H, KH, d, vd, taps = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
            for n, rows in (("q", KH * d), ("k", KH * d), ("v", H * vd)):
                W[q + n] = mat(rows, Wd, 2.0)
                W[q + n + ".conv"] = bf16_round(rng.standard_normal((rows, taps)) * 0.6).astype(F)
            W[q + "b"], W[q + "A_log"], W[q + "norm"] = mat(H, Wd, 2.0), vec(H, -0.5, 0.5), vec(vd, 1.0, 0.2)
            W[q + "a1"], W[q + "a2"], W[q + "dt_bias"] = mat(low_rank, Wd), mat(H * d, low_rank, 2.0), vec(H * d, -1.0, 1.0)
            W[q + "g1"], W[q + "g2"], W[q + "o"] = mat(low_rank, Wd), mat(H * vd, low_rank, 2.0), mat(Wd, H * vd)
        else:
            H, vd, N, G, taps = m["heads"], m["vdim"], m["state"], m["groups"], m["conv"]
            inner, ch = H * vd, H * vd + 2 * G * N
            W[q + "in"], W[q + "conv"], W[q + "conv.b"] = mat(2 * inner + 2 * G * N + H, Wd, 2.0), bf16_round(rng.standard_normal((ch, taps)) * 0.6).astype(F), vec(ch, 0.0, 0.2)
            W[q + "dt_bias"], W[q + "A_log"], W[q + "D"] = vec(H, -1.0, 1.0), vec(H, -0.5, 0.5), vec(H, 1.0, 0.3)
            W[q + "norm"], W[q + "o"] = vec(inner, 1.0, 0.2), mat(Wd, inner)
        if l.get("mlp"):
            r, ff, q = l["mlp"]["router"], l["mlp"]["expert"]["ff"], p + "mlp."
            W[q + "router"], W[q + "correction"] = mat(r["experts"], Wd, 3.0), vec(r["experts"], 0.0, 0.3)
            for e in range(r["experts"]):
                W[q + "e%d.gate" % e], W[q + "e%d.up" % e], W[q + "e%d.down" % e] = mat(ff, Wd, 1.5), mat(ff, Wd, 1.5), mat(Wd, ff, 1.5)
    return W


def write_checkpoint(folder, cfg, W):
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    header, blobs, at = {}, [], 0
    for name, a in W.items():
        b = (np.ascontiguousarray(a, dtype=np.float32).view(np.uint32) >> 16).astype(np.uint16).tobytes()
        header[name] = {"dtype": "BF16", "shape": list(a.shape), "data_offsets": [at, at + len(b)]}
        blobs.append(b)
        at += len(b)
    hj = json.dumps(header).encode()
    hj += b" " * (-len(hj) % 8)
    with open(os.path.join(folder, "model.safetensors"), "wb") as f:
        f.write(struct.pack("<Q", len(hj)) + hj + b"".join(blobs))


def rel_err(got, want):
    """the per-row measure: rms over the vocabulary of the mean-free difference, over the rms of the mean-free reference"""
    d = got - want
    d = d - d.mean(-1, keepdims=True)
    w = want - want.mean(-1, keepdims=True)
    return np.sqrt((d * d).mean(-1)) / np.sqrt((w * w).mean(-1).mean())
