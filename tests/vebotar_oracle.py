"""Plain, slow float64 restatement of the Vebotar decoder, one function per mechanism.

Shares no code with the engine: numpy only, token-at-a-time loops, no cache.  Weights are a dict name -> float array, the
configuration is the nested dict of a model folder's config.json.

  streams:    S copies X[s] of the residual, all starting as scale_e * embed[token].  A sublayer reads u = sum_s a[s] X[s], computes
              y = f(rms(u) * g) and writes X'[t] = sum_s M[s, t] X[s] + b[t] * y for every t at once.  The model's output is sum_s X[s].
  mixer:      two score maps per head over one set of values: query rows [head][map][dim], key rows [kv head][map][dim];
              the first `dims` channels of every map rotate pairwise (2i, 2i+1) by p * f_i with long-context frequency blending;
              key j is visible from i iff j <= i and both lie in the same block of `size` positions; each map is a softmax of its own;
              o = A1 v - lam * A2 v, lam = exp(<lq1, lk1>) - exp(<lq2, lk2>) + d; o is scaled to unit RMS per head and by (1 - d).
  ff:         routed experts Wd relu(Wu h)^2, the `top` largest router logits, softmax over those only; plus a shared expert of the
              same form times sigmoid(<w_sg, h>).
"""
from __future__ import annotations

import math

import numpy as np


def rms_unit(x: np.ndarray, eps: float) -> np.ndarray:
    x = np.asarray(x, dtype=np.float64)
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def rms_norm(x, gain, eps):
    return rms_unit(x, eps) * np.asarray(gain, dtype=np.float64)


def rotary_frequencies(rot: dict):
    """(f_i for i < dims/2, magnitude multiplier of cos and sin)."""
    dims, base = int(rot["dims"]), float(rot["base"])
    f = np.array([base ** (-2.0 * i / dims) for i in range(dims // 2)])
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor, orig = float(sc["factor"]), float(sc["original"])

    def turn(t):
        return dims * math.log(orig / (2.0 * math.pi * t)) / (2.0 * math.log(base))

    lo = max(math.floor(turn(float(sc["fast"]))), 0)
    hi = min(math.ceil(turn(float(sc["slow"]))), dims - 1)
    ramp = np.clip((np.arange(dims // 2) - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate(x: np.ndarray, pos: int, rot: dict | None) -> np.ndarray:
    """x: one map of one head at position pos, [dim]."""
    x = np.array(x, dtype=np.float64)
    if not rot:
        return x
    f, mag = rotary_frequencies(rot)
    for i in range(len(f)):
        a = pos * f[i]
        c, s = math.cos(a) * mag, math.sin(a) * mag
        u, v = x[2 * i], x[2 * i + 1]
        x[2 * i], x[2 * i + 1] = u * c - v * s, v * c + u * s
    return x


def visible(i: int, j: int, size: int) -> bool:
    return j <= i and (size <= 0 or i // size == j // size)


def softmax(s):
    p = np.exp(s - np.max(s))
    return p / p.sum()


def diff_lambda(W: dict, prefix: str, d: float) -> float:
    g = lambda n: np.asarray(W[prefix + n], dtype=np.float64)
    return math.exp(float(g("lq1") @ g("lk1"))) - math.exp(float(g("lq2") @ g("lk2"))) + d


def rotated_qkv(h, W, own: str, kv: str, m: dict, pos0: int = 0):
    """q [T, H, maps, dim], k [T, G, maps, dim] (both rotated), v [T, G, vdim]; queries from layer `own`, keys / values from layer `kv`."""
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    mat = lambda n: np.asarray(W[n], dtype=np.float64)
    q = (h @ mat(own + "mix.q").T).reshape(T, H, 2, D)
    k = (h @ mat(kv + "mix.k").T).reshape(T, G, 2, D)
    v = (h @ mat(kv + "mix.v").T).reshape(T, G, V)
    for t in range(T):
        for a in range(2):
            for x in range(H):
                q[t, x, a] = rotate(q[t, x, a], pos0 + t, m.get("rot"))
            for x in range(G):
                k[t, x, a] = rotate(k[t, x, a], pos0 + t, m.get("rot"))
    return q, k, v


def diff_attention(q, k, v, m: dict, lam: float, eps: float) -> np.ndarray:
    """q [T, H, 2, dim], k [T, G, 2, dim], v [T, G, vdim] -> [T, H * vdim]."""
    H, G, V = m["heads"], m["kv_heads"], m["vdim"]
    T = q.shape[0]
    size = (m.get("mask") or {}).get("size", 0)
    d = float(m["diff"])
    out = np.zeros((T, H, V))
    for i in range(T):
        js = [j for j in range(T) if visible(i, j, size)]
        for x in range(H):
            g = x // (H // G)
            maps = []
            for a in range(2):
                s = np.array([float(q[i, x, a] @ k[j, g, a]) * m["scale"] for j in js])
                p = softmax(s)
                maps.append(sum(w * v[j, g] for w, j in zip(p, js)))
            o = maps[0] - lam * maps[1]
            out[i, x] = rms_unit(o, eps) * (1.0 - d)
    return out.reshape(T, H * V)


def expert(h, up, down):
    z = np.maximum(np.asarray(up, dtype=np.float64) @ h, 0.0)
    return np.asarray(down, dtype=np.float64) @ (z * z)


def route(h, router, top: int):
    """(chosen expert ids, their weights) for one token."""
    z = np.asarray(router, dtype=np.float64) @ h
    ids = np.argsort(-z, kind="stable")[:top]
    return ids, softmax(z[ids])


def moe(h: np.ndarray, W: dict, p: str, mlp: dict) -> np.ndarray:
    T = h.shape[0]
    out = np.zeros_like(h)
    for t in range(T):
        ids, ws = route(h[t], W[p + "router"], int(mlp["router"]["top"]))
        for e, w in zip(ids, ws):
            out[t] += w * expert(h[t], W[p + "e%d.up" % e], W[p + "e%d.down" % e])
        if mlp.get("shared"):
            gate = 1.0 / (1.0 + math.exp(-float(np.asarray(W[p + "shared.sg"], dtype=np.float64).reshape(-1) @ h[t])))
            out[t] += gate * expert(h[t], W[p + "shared.up"], W[p + "shared.down"])
    return out


def stream_read(X, W, p):
    """X [S, T, width] -> u [T, width]."""
    if p + "in" not in W:
        return X[0]
    return np.tensordot(np.asarray(W[p + "in"], dtype=np.float64), X, axes=(0, 0))


def stream_write(X, y, W, p):
    if p + "in" not in W:
        return X + y[None]
    M = np.asarray(W[p + "mix"], dtype=np.float64)          # [from, to]
    b = np.asarray(W[p + "out"], dtype=np.float64)
    return np.einsum("st,sij->tij", M, X) + b[:, None, None] * y[None]


def forward(cfg: dict, W: dict, tokens, layer_sums: list | None = None) -> np.ndarray:
    """Logits [T, vocab] of a whole sequence from position 0."""
    eps = float(cfg["norm"]["eps"])
    S = int(cfg.get("streams", 1))
    x0 = np.asarray(W["embed"], dtype=np.float64)[np.asarray(tokens)] * float((cfg.get("embedding") or {}).get("scale", 1.0))
    X = np.stack([x0] * S)
    kv = {}
    for i, e in enumerate(cfg["layers"]):
        p, m = "l%d." % i, e["mixer"]
        h = rms_norm(stream_read(X, W, p + "hc1."), W[p + "norm1"], eps)
        src = "l%d." % m["kv_from"] if "kv_from" in m else p
        if "kv_from" in m:
            hk = kv[m["kv_from"]]
        else:
            hk = kv[i] = h
        q, _, _ = rotated_qkv(h, W, p, src, m)
        _, k, v = rotated_qkv(hk, W, p, src, m)
        a = diff_attention(q, k, v, m, diff_lambda(W, p + "mix.", float(m["diff"])), eps)
        X = stream_write(X, a @ np.asarray(W[p + "mix.o"], dtype=np.float64).T, W, p + "hc1.")
        if e.get("mlp"):
            h = rms_norm(stream_read(X, W, p + "hc2."), W[p + "norm2"], eps)
            X = stream_write(X, moe(h, W, p + "mlp.", e["mlp"]), W, p + "hc2.")
        if layer_sums is not None:
            layer_sums.append(X.sum(0))
    x = rms_norm(X.sum(0), W["final.norm"], eps)
    return x @ np.asarray(W["head"], dtype=np.float64).T


# ---------------------------------------------------------------- random small models for the tests
def _bf16(a):
    """Round to the nearest bfloat16-representable value (ties to even), so a checkpoint written in bfloat16 holds the same numbers."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    u = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16
    return u.astype(np.uint32).view(np.float32).astype(np.float64).reshape(np.shape(a))


def random_model(rng, vocab=37, width=48, n_layers=3, heads=4, kv_heads=2, dim=8, vdim=12, chunk=7, rot_dims=4, base=50.0, scaling=True, diff=0.25,
                 scale=None, experts=5, top=2, ff=20, shared_ff=14, streams=3, embed_scale=0.7, kv_from=None, no_mlp=(), eps=1e-5):
    """(config dict, weights dict).  kv_from: {layer: earlier layer whose cache it reads}; streams 0: a single residual, no stream tensors."""
    kv_from = kv_from or {}
    layers = []
    for i in range(n_layers):
        m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": float(scale if scale is not None else dim ** -0.5), "diff": diff}
        if chunk:
            m["mask"] = {"size": chunk}
        if rot_dims:
            m["rot"] = {"dims": rot_dims, "base": base}
            if scaling:
                m["rot"]["scaling"] = {"factor": 3.0, "original": 24, "fast": 6.0, "slow": 1.5}
        if i in kv_from:
            m["kv_from"] = kv_from[i]
        mlp = None
        if i not in no_mlp:
            mlp = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
            if shared_ff:
                mlp["shared"] = {"ff": shared_ff}
        layers.append({"type": "attention", "mixer": m, "mlp": mlp})
    cfg = {"architecture": "Vebotar", "vocab": vocab, "width": width, "norm": {"eps": eps}, "embedding": {"scale": embed_scale}, "layers": layers}
    if streams:
        cfg["streams"] = streams
    mat = lambda r, c, s=1.0: _bf16(rng.standard_normal((r, c)) * s * c ** -0.5)
    vec = lambda n: _bf16(1.0 + 0.2 * rng.standard_normal(n))
    W = {"embed": _bf16(rng.standard_normal((vocab, width))), "final.norm": vec(width), "head": mat(vocab, width)}
    for i, e in enumerate(layers):
        p, m = "l%d." % i, e["mixer"]
        W[p + "norm1"] = vec(width)
        W[p + "mix.q"] = mat(heads * 2 * dim, width, 2.0)
        if "kv_from" not in m:
            W[p + "mix.k"] = mat(kv_heads * 2 * dim, width, 2.0)
            W[p + "mix.v"] = mat(kv_heads * vdim, width)
        for n in ("lq1", "lk1", "lq2", "lk2"):
            W[p + "mix." + n] = _bf16(rng.standard_normal(dim) * 0.3)
        W[p + "mix.o"] = mat(width, heads * vdim)
        subs = ["hc1."] + (["hc2."] if e["mlp"] else [])
        if streams:
            for q in subs:
                W[p + q + "in"] = _bf16(1.0 / streams + 0.3 * rng.standard_normal(streams))
                W[p + q + "out"] = _bf16(1.0 + 0.3 * rng.standard_normal(streams))
                W[p + q + "mix"] = _bf16(np.eye(streams) + 0.2 * rng.standard_normal((streams, streams)))
        if e["mlp"]:
            W[p + "norm2"] = vec(width)
            W[p + "mlp.router"] = mat(experts, width, 2.0)
            for x in range(experts):
                W[p + "mlp.e%d.up" % x] = mat(ff, width)
                W[p + "mlp.e%d.down" % x] = mat(width, ff)
            if shared_ff:
                W[p + "mlp.shared.up"] = mat(shared_ff, width)
                W[p + "mlp.shared.down"] = mat(width, shared_ff)
                W[p + "mlp.shared.sg"] = mat(1, width, 2.0)
    return cfg, W
