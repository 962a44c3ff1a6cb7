"""A plain, slow Gubotar model in float64, one function per mechanism, written token by token.

Used by the tests only; it shares no code with the engine. Everything is a loop over the tokens
of one sequence: recurrences are stepped, attention is a sum over the visible keys.

Notation: W is the model width, a "layer" is a dict from config.json's ``layers`` list, ``P`` maps
tensor names to float64 tensors.
"""

from __future__ import annotations

import json
from pathlib import Path

import torch
from safetensors.torch import load_file

F = torch.float64


def load(folder):
    folder = Path(folder)
    cfg = json.loads((folder / "config.json").read_text())
    P = {k: v.to(F) for k, v in load_file(str(folder / "model.safetensors")).items()}
    return cfg, P


# ----------------------------------------------------------------------------- small pieces
def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def silu(z):
    return z / (1 + torch.exp(-z))


def sigmoid(z):
    return 1 / (1 + torch.exp(-z))


def token_shift(x, mu):
    """x [T, W]; every row is mixed with the row before it (zeros before the first)."""
    prev = torch.cat([torch.zeros_like(x[:1]), x[:-1]], 0)
    return x + (prev - x) * mu


def rotate_partial(x, pos, dims, base):
    """x [heads, dim] at position pos: the first ``dims`` dims are rotated, pairs (i, i + dims/2)."""
    half = dims // 2
    i = torch.arange(half, dtype=F)
    ang = pos * base ** (-2 * i / dims)
    c, s = torch.cos(ang), torch.sin(ang)
    u, v = x[:, :half], x[:, half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[:, dims:]], -1)


def decayed_outer_product_scan(q, k, v, decay):
    """q, k [T, H, dk], v [T, H, dv], decay [H]: S_t = decay S_{t-1} + k_t v_t^T, o_t = S_t^T q_t."""
    T, H, dk = q.shape
    dv = v.shape[-1]
    S = torch.zeros(H, dk, dv, dtype=F)
    out = torch.zeros(T, H, dv, dtype=F)
    for t in range(T):
        S = decay[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hkv,hk->hv", S, q[t])
    return out


# ----------------------------------------------------------------------------- mixers
def chunked_softmax(q, k, v, scale, temp, slopes, size, start=0):
    """q [T, H, D]; k, v [start + T, G, D] (``start`` earlier tokens are only keys). Query i
    (absolute position start + i) sees key j <= its position of the same chunk of ``size``;
    score = q.k * scale * temp[h] - slopes[h] * (distance)."""
    T, H, D = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[-1], dtype=F)
    for hd in range(H):
        g = hd // (H // G)
        for t in range(T):
            i = start + t
            lo = (i // size) * size
            js = torch.arange(lo, i + 1)
            s = (k[lo : i + 1, g] @ q[t, hd]) * scale * temp[hd] - slopes[hd] * (i - js).to(F)
            out[t, hd] = torch.softmax(s, 0) @ v[lo : i + 1, g]
    return out


def head_slopes(H):
    return torch.tensor([2.0 ** (-8.0 * (h + 1) / H) for h in range(H)], dtype=F)


def chunked_biased_attention(h, P, pre, m, eps):
    """The softmax half of the ``parallel`` mixer. h [T, W]."""
    T = h.shape[0]
    H, G, D = m["heads"], m["kv_heads"], m["dim"]
    q = (h @ P[pre + "q"].T).view(T, H, D)
    k_raw = (h @ P[pre + "k"].T).view(T, G, D)
    q = rms(q, eps) * P[pre + "q.norm"]
    k = rms(k_raw, eps) * P[pre + "k.norm"]
    # the values are the keys as projected
    out = chunked_softmax(q, k, k_raw, m["scale"], P[pre + "temp"], head_slopes(H), m["mask"]["size"])
    return out.reshape(T, H * D) @ P[pre + "o"].T


def lightning_attention(h, P, pre, m, eps):
    """The linear half of the ``parallel`` mixer."""
    T = h.shape[0]
    H, dk, dv = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ P[pre + "q"].T).view(T, H, dk)
    k = silu(h @ P[pre + "k"].T).view(T, H, dk)
    v = silu(h @ P[pre + "v"].T).view(T, H, dv)
    o = decayed_outer_product_scan(q, k, v, torch.tensor(m["decay"], dtype=F))
    o = rms(o.reshape(T, H * dv), eps) * P[pre + "norm"]
    return (o * sigmoid(h @ P[pre + "g"].T)) @ P[pre + "o"].T


def parallel_mixer(h, P, pre, m, eps):
    a = chunked_biased_attention(h, P, pre + "left.", m["left"], eps)
    b = lightning_attention(h, P, pre + "right.", m["right"], eps)
    return 0.5 * (rms(a, eps) * P[pre + "left.out"] + rms(b, eps) * P[pre + "right.out"])


def retention_mixer(h, P, pre, m, eps):
    T = h.shape[0]
    H, dk, dv = m["heads"], m["dim"], m["vdim"]
    q = (h @ P[pre + "q"].T).view(T, H, dk)
    k = (h @ P[pre + "k"].T).view(T, H, dk)
    v = (h @ P[pre + "v"].T).view(T, H, dv)
    rot = m["rot"]
    q = torch.stack([rotate_partial(q[t], t, rot["dims"], rot["base"]) for t in range(T)])
    k = torch.stack([rotate_partial(k[t], t, rot["dims"], rot["base"]) for t in range(T)])
    k = k * dk ** -0.5
    o = decayed_outer_product_scan(q, k, v, torch.tensor(m["decay"], dtype=F))
    o = rms(o, eps).reshape(T, H * dv)  # each head alone, no weight
    return (o * silu(h @ P[pre + "g"].T)) @ P[pre + "o"].T


MIXERS = {"parallel": parallel_mixer, "retention": retention_mixer}


def dense_feed_forward(h, P, pre):
    return (silu(h @ P[pre + "gate"].T) * (h @ P[pre + "up"].T)) @ P[pre + "down"].T


# ----------------------------------------------------------------------------- the model
def forward(cfg, P, tokens, layers_out=None):
    """Logits [T, vocab] of one sequence given whole. ``layers_out``: list that receives the
    residual stream after every layer."""
    eps = cfg["norm"]["eps"]
    x = P["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    for i, layer in enumerate(cfg["layers"]):
        pre = f"l{i}."
        h = token_shift(x, P[pre + "shift"])
        a = MIXERS[layer["type"]](h, P, pre + "mix.", layer["mixer"], eps)
        x = x + rms(a, eps) * (1 + P[pre + "norm1"])
        if layer.get("mlp") is not None:
            assert layer["mlp"]["kind"] == "dense"
            f = dense_feed_forward(x, P, pre + "mlp.")
            x = x + rms(f, eps) * (1 + P[pre + "norm2"])
        if layers_out is not None:
            layers_out.append(x.clone())
    x = rms(x, eps) * (1 + P["final.norm"])
    return x @ P["embed"].T


def model_logits(folder, tokens):
    cfg, P = load(folder)
    return forward(cfg, P, tokens).float()


def greedy(folder, prompt, n):
    """n tokens generated greedily after ``prompt`` (the whole sequence is run again each time)."""
    cfg, P = load(folder)
    tokens = list(prompt)
    for _ in range(n):
        tokens.append(int(forward(cfg, P, tokens)[-1].argmax()))
    return tokens[len(prompt):]
