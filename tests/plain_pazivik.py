"""The Pazivik architecture written out plainly in float64, one function per mechanism.

A slow oracle for the tests: whole sequences only, no cache, no batching, no kernels; it shares no
code with the engine. Weights come as a dict of tensors under the checkpoint's names and the
configuration as the plain dict of ``config.json``.

Notation: ``x`` is the residual stream ``[n, width]`` of one sequence whose tokens sit at
positions 0 .. n-1.
"""

from __future__ import annotations

import math

import torch

F64 = torch.float64


def rms_norm(x, w, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def bigram_rows(tokens, buckets, mul_prev, mul_cur):
    """Row of the bigram table for every token: the last row for a sequence's first token."""
    rows = [buckets]
    for prev, cur in zip(tokens[:-1], tokens[1:]):
        rows.append((prev * mul_prev + cur * mul_cur) % buckets)
    return rows


def sinusoid(n, width):
    """[n, width]: entry 2i is sin(p * 10000^(-2i/width)), entry 2i+1 the cosine of that angle."""
    out = torch.zeros(n, width, dtype=F64)
    p = torch.arange(n, dtype=F64)[:, None]
    i = torch.arange((width + 1) // 2, dtype=F64)[None, :]
    ang = p * 10000.0 ** (-2.0 * i / width)
    out[:, 0::2] = torch.sin(ang)[:, : out[:, 0::2].shape[1]]
    out[:, 1::2] = torch.cos(ang)[:, : out[:, 1::2].shape[1]]
    return out


def embed(tokens, w, cfg):
    width = cfg["width"]
    b = cfg["embedding"]["bigram"]
    x = w["embed"].to(F64)[tokens]
    x = x + w["bigram"].to(F64)[bigram_rows(list(tokens), b["buckets"], b["mul_prev"], b["mul_cur"])]
    return x + sinusoid(len(tokens), width)


def latent(h, w, prefix, eps):
    """The normed latent rows ``c`` that a layer with a down-projection of its own caches."""
    return rms_norm(h @ w[prefix + "dkv"].to(F64).T, w[prefix + "dkv.norm"].to(F64), eps)


def windowed_sink_softmax(scores, window, sink):
    """scores [n, n] of one head: causal, the last ``window`` keys (0: all), and a sink term
    exp(sink) in the denominator that has no value."""
    n = scores.shape[0]
    i = torch.arange(n)[:, None]
    j = torch.arange(n)[None, :]
    seen = (j <= i) & ((i - j < window) if window > 0 else torch.ones_like(j <= i))
    s = scores.masked_fill(~seen, -math.inf)
    m = torch.maximum(s.max(-1, keepdim=True).values, sink.reshape(1, 1))
    e = torch.exp(s - m)
    return e / (e.sum(-1, keepdim=True) + torch.exp(sink - m))


def latent_attention(h, c, w, prefix, m):
    """h [n, width] the normed input, c [n, kv_rank] the latent rows this layer reads."""
    H, D, V = m["heads"], m["dim"], m["vdim"]
    window = int((m.get("mask") or {}).get("size", 0) or 0)
    q = (h @ w[prefix + "q"].to(F64).T).view(-1, H, D)
    k = (c @ w[prefix + "uk"].to(F64).T).view(-1, H, D)
    v = (c @ w[prefix + "uv"].to(F64).T).view(-1, H, V)
    sink = w[prefix + "sink"].to(F64)
    outs = []
    for hd in range(H):
        p = windowed_sink_softmax(q[:, hd] @ k[:, hd].T * m["scale"], window, sink[hd])
        outs.append(p @ v[:, hd])
    return torch.cat(outs, -1) @ w[prefix + "o"].to(F64).T


def gated(h, w, prefix, act):
    return (act(h @ w[prefix + "gate"].to(F64).T) * (h @ w[prefix + "up"].to(F64).T)) @ w[prefix + "down"].to(F64).T


def route(h, w, prefix, top):
    """Chosen experts [n, top] and their weights: the sigmoid scores themselves."""
    s = torch.sigmoid(h @ w[prefix + "router"].to(F64).T)
    val, idx = torch.topk(s, top, dim=-1)
    return idx, val


def moe(h, w, prefix, mlp):
    E, top = mlp["router"]["experts"], mlp["router"]["top"]
    idx, val = route(h, w, prefix, top)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for k in range(top):
            e = int(idx[t, k])
            out[t] += gated((val[t, k] * h[t])[None], w, f"{prefix}e{e}.", silu)[0]
    if mlp.get("shared"):
        g = torch.sigmoid(h @ w[prefix + "shared.sg"].to(F64).T)  # [n, 1]
        out = out + g * gated(h, w, prefix + "shared.", silu)
    return out


def feed_forward(h, w, prefix, mlp):
    if mlp["kind"] == "dense":
        return gated(h, w, prefix, gelu_tanh)
    return moe(h, w, prefix, mlp)


def forward(tokens, w, cfg, return_layers=False):
    """Logits [n, vocab] of one whole sequence (and the residual stream after every layer)."""
    eps = cfg["norm"]["eps"]
    x = embed(tokens, w, cfg)
    latents = {}
    after = []
    for i, layer in enumerate(cfg["layers"]):
        m = layer["mixer"]
        pre = f"l{i}."
        h = rms_norm(x, w[pre + "norm1"].to(F64), eps)
        if "kv_from" in m and m["kv_from"] is not None:
            c = latents[m["kv_from"]]
        else:
            c = latents[i] = latent(h, w, pre + "mix.", eps)
        x = x + latent_attention(h, c, w, pre + "mix.", m)
        if layer["mlp"] is not None:
            h = rms_norm(x, w[pre + "norm2"].to(F64), eps)
            x = x + feed_forward(h, w, pre + "mlp.", layer["mlp"])
        after.append(x)
    h = rms_norm(x, w["final.norm"].to(F64), eps)
    logits = h @ w["embed"].to(F64).T
    cap = cfg.get("logit_softcap", 0.0)
    if cap:
        logits = cap * torch.tanh(logits / cap)
    return (logits, torch.stack(after)) if return_layers else logits


# ----------------------------------------------------------------------------- a model folder
def load(folder):
    import json
    from pathlib import Path

    from safetensors.torch import load_file

    folder = Path(folder)
    cfg = json.loads((folder / "config.json").read_text())
    return cfg, {k: v.to(F64) if v.is_floating_point() else v for k, v in load_file(str(folder / "model.safetensors")).items()}


def model_logits(folder, tokens):
    cfg, w = load(folder)
    return forward(list(tokens), w, cfg).float()


def greedy(folder, prompt, n):
    """n tokens generated greedily after ``prompt`` (the whole sequence is run again each time)."""
    cfg, w = load(folder)
    tokens = list(prompt)
    for _ in range(n):
        tokens.append(int(forward(tokens, w, cfg)[-1].argmax()))
    return tokens[len(prompt):]
