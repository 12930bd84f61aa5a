"""Plain, slow float64 restatement of the Zelunex decoder, one function per mechanism.

Shares no code with the engine: numpy only, a token-at-a-time double loop for the attention, no cache.
Weights are a dict name -> float array, the configuration is the nested dict of a model folder's config.json.

  block:      h = rms(x) * g ;  x' = x + m * (ls1 * mixer(h) + ls2 * ff(h))        (one norm feeds both branches)
  mixer:      q = Wq h, k = Wk h, v = Wv h ;  q, k each normalised over their FULL length (all heads at once) with a gain vector ;
              s_ij = c * tanh(scale * <q_i, k_j> / c) ;  j visible from i  <=>  j <= i and (i - j < window or j < keep) ;
              softmax over the visible j, weighted sum of v, then Wo on the concatenated heads
  ff:         Wdown (gelu_tanh(Wgate h) * (Wup h))
  a layer with `weights_of: j` reads layer j's tensors
"""
from __future__ import annotations

import math

import numpy as np


def rms_norm(x: np.ndarray, gain: np.ndarray, eps: float) -> np.ndarray:
    x = np.asarray(x, dtype=np.float64)
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps) * np.asarray(gain, dtype=np.float64)


def gelu_tanh(z: np.ndarray) -> np.ndarray:
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def visible(i: int, j: int, window: int, keep: int) -> bool:
    return j <= i and (i - j < window or j < keep)


def softcap(s: float, cap: float) -> float:
    return cap * math.tanh(s / cap)


def window_attention(q: np.ndarray, k: np.ndarray, v: np.ndarray, heads: int, kv_heads: int, dim: int, vdim: int, scale: float, cap: float,
                     window: int, keep: int) -> np.ndarray:
    """q [T, heads*dim], k [T, kv_heads*dim], v [T, kv_heads*vdim] -> [T, heads*vdim]."""
    T = q.shape[0]
    out = np.zeros((T, heads * vdim))
    group = heads // kv_heads
    for i in range(T):
        js = [j for j in range(T) if visible(i, j, window, keep)]
        for h in range(heads):
            g = h // group
            qi = q[i, h * dim:(h + 1) * dim]
            s = np.array([softcap(scale * float(qi @ k[j, g * dim:(g + 1) * dim]), cap) for j in js])
            p = np.exp(s - s.max())
            p /= p.sum()
            for w, j in zip(p, js):
                out[i, h * vdim:(h + 1) * vdim] += w * v[j, g * vdim:(g + 1) * vdim]
    return out


def window_attention_row(q_i: np.ndarray, k: np.ndarray, v: np.ndarray, i: int, heads: int, kv_heads: int, dim: int, vdim: int, scale: float,
                         cap: float, window: int, keep: int) -> np.ndarray:
    """The same for the single query at position i (long contexts, where the all-pairs loop above is too slow)."""
    js = np.array([j for j in range(i + 1) if visible(i, j, window, keep)])
    out = np.zeros(heads * vdim)
    for h in range(heads):
        g = h // (heads // kv_heads)
        s = cap * np.tanh(scale * (k[js, g * dim:(g + 1) * dim] @ q_i[h * dim:(h + 1) * dim]) / cap)
        p = np.exp(s - s.max())
        out[h * vdim:(h + 1) * vdim] = (p / p.sum()) @ v[js, g * vdim:(g + 1) * vdim]
    return out


def mixer_attention(h: np.ndarray, W: dict, pre: str, mc: dict, eps: float) -> np.ndarray:
    q = h @ W[pre + "mix.q"].T
    k = h @ W[pre + "mix.k"].T
    v = h @ W[pre + "mix.v"].T
    q = rms_norm(q, W[pre + "mix.q.norm"], eps)
    k = rms_norm(k, W[pre + "mix.k.norm"], eps)
    a = window_attention(q, k, v, mc["heads"], mc["kv_heads"], mc["dim"], mc["vdim"], mc["scale"], mc["softcap"], mc["mask"]["size"],
                         mc["mask"]["keep_first"])
    return a @ W[pre + "mix.o"].T


def feed_forward(h: np.ndarray, W: dict, pre: str) -> np.ndarray:
    return (gelu_tanh(h @ W[pre + "mlp.gate"].T) * (h @ W[pre + "mlp.up"].T)) @ W[pre + "mlp.down"].T


def forward(cfg: dict, W: dict, tokens, return_layers: bool = False):
    """Logits [T, vocab] (and the residual stream after every layer run, [L, T, width])."""
    W = {n: np.asarray(a, dtype=np.float64) for n, a in W.items()}
    eps = cfg["norm"]["eps"]
    m = cfg["residual_mult"]
    x = W["embed"][np.asarray(tokens)]
    per_layer = []
    for i, lc in enumerate(cfg["layers"]):
        assert lc["type"] == "attention"
        pre = "l%d." % lc.get("weights_of", i)
        h = rms_norm(x, W[pre + "norm1"], eps)
        y = mixer_attention(h, W, pre, lc["mixer"], eps) * W[pre + "ls1"]
        if lc.get("mlp") is not None:
            assert lc["mlp"]["kind"] == "dense"
            y = y + feed_forward(h, W, pre) * W[pre + "ls2"]
        x = x + m * y
        per_layer.append(x.copy())
    logits = rms_norm(x, W["final.norm"], eps) @ W["head"].T
    return (logits, np.stack(per_layer)) if return_layers else logits


def random_model(rng: np.random.Generator, *, vocab=96, width=64, n_layers=3, heads=4, kv_heads=2, dim=32, vdim=16, ff=96, window=8, keep=2,
                 softcap_c=15.0, scale=None, eps=4e-3, mult=0.6, share=None, no_mlp=()):
    """A small random configuration + weights (bf16-representable values). share: {layer: source layer}."""
    import torch

    def bf(a):
        return torch.from_numpy(np.asarray(a, dtype=np.float32)).to(torch.bfloat16).to(torch.float32).numpy()

    def r(*shape, s=1.0):
        return bf(rng.standard_normal(shape).astype(np.float32) * s)

    share = share or {}
    layers, W = [], {}
    for i in range(n_layers):
        mixer = {"dim": dim, "heads": heads, "kv_heads": kv_heads, "vdim": vdim, "scale": scale if scale is not None else 1.0 / math.sqrt(dim) * 1.5,
                 "softcap": softcap_c, "mask": {"size": window, "keep_first": keep}}
        entry = {"type": "attention", "mixer": mixer, "mlp": None if i in no_mlp else {"kind": "dense", "ff": ff}}
        if i in share:
            entry = dict(layers[share[i]])
            entry["weights_of"] = share[i]
            layers.append(entry)
            continue
        layers.append(entry)
        p = "l%d." % i
        W[p + "norm1"] = bf(1.0 + r(width, s=0.1))
        W[p + "mix.q"] = r(heads * dim, width, s=width ** -0.5)
        W[p + "mix.k"] = r(kv_heads * dim, width, s=width ** -0.5)
        W[p + "mix.v"] = r(kv_heads * vdim, width, s=width ** -0.5)
        W[p + "mix.q.norm"] = bf(1.0 + r(heads * dim, s=0.1))
        W[p + "mix.k.norm"] = bf(1.0 + r(kv_heads * dim, s=0.1))
        W[p + "mix.o"] = r(width, heads * vdim, s=(heads * vdim) ** -0.5)
        W[p + "ls1"] = bf(1.0 + r(width, s=0.2))
        if i not in no_mlp:
            W[p + "mlp.gate"] = r(ff, width, s=width ** -0.5)
            W[p + "mlp.up"] = r(ff, width, s=width ** -0.5)
            W[p + "mlp.down"] = r(width, ff, s=ff ** -0.5)
            W[p + "ls2"] = bf(1.0 + r(width, s=0.2))
    W["embed"] = r(vocab, width)
    W["final.norm"] = bf(1.0 + r(width, s=0.1))
    W["head"] = r(vocab, width, s=width ** -0.5)
    cfg = {"architecture": "Zelunex", "layers": layers, "norm": {"eps": eps}, "residual_mult": mult, "vocab": vocab, "width": width}
    return cfg, W
