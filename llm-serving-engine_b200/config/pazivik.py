"""Typed configuration of the Pazivik architecture, read from its ``config.json``.

The file names the architecture (``"architecture": "Pazivik"``), ``vocab``, ``width``, the epsilon
of every norm (``norm.eps``), the soft cap of the logits (``logit_softcap``), the hashed bigram
embedding (``embedding.bigram``: ``buckets``, ``mul_prev``, ``mul_cur``) and a list ``layers``.
Each entry has ``type`` (the mixer: ``latent_attention``), the mixer's sizes under ``mixer``
(``heads``, ``dim``, ``vdim``, ``kv_rank``, ``scale``, ``mask.size``, and ``kv_from`` for a layer
that reads another layer's latent rows) and its feed-forward under ``mlp``: null,
``{"kind": "dense", "ff": F}`` or ``{"kind": "moe", "router": {"experts", "top"}, "expert":
{"ff"}, "shared": {"ff"}}`` (``shared`` may be absent or null). Layers may differ in every size.
A key that is absent is an error, and so is a key that this engine does not know, because it
would change the math silently.
"""

from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Any

from .gubotar import _take
from .llama import ConfigError


def _take_some(d: dict, required: tuple[str, ...], optional: tuple[str, ...], where: str) -> list:
    """Values of the required keys, then of the optional ones (None where absent)."""
    if not isinstance(d, dict):
        raise ConfigError(f"{where}: expected an object")
    missing = [k for k in required if k not in d]
    unknown = [k for k in d if k not in required + optional]
    if missing or unknown:
        raise ConfigError(f"{where}: missing keys {missing}, unknown keys {unknown}")
    return [d[k] for k in required] + [d.get(k) for k in optional]


@dataclass(frozen=True)
class LatentAttentionConfig:
    heads: int
    dim: int
    vdim: int
    kv_rank: int
    scale: float
    window: int  # 0: no mask beyond the causal one
    kv_from: int | None  # the layer whose latent rows this one reads; None: its own

    @classmethod
    def from_dict(cls, d, where):
        heads, dim, vdim, rank, scale, mask, kv_from = _take_some(
            d, ("heads", "dim", "vdim", "kv_rank", "scale"), ("mask", "kv_from"), where)
        window = 0
        if mask is not None:
            (window,) = _take(mask, ("size",), where + ".mask")
            if int(window) < 1:
                raise ConfigError(f"{where}: mask.size must be positive")
        if min(int(heads), int(dim), int(vdim), int(rank)) < 1:
            raise ConfigError(f"{where}: sizes must be positive")
        return cls(int(heads), int(dim), int(vdim), int(rank), float(scale), int(window),
                   None if kv_from is None else int(kv_from))

    def to_dict(self):
        d = {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "kv_rank": self.kv_rank,
             "scale": self.scale}
        if self.window:
            d["mask"] = {"size": self.window}
        if self.kv_from is not None:
            d["kv_from"] = self.kv_from
        return d


@dataclass(frozen=True)
class PazivikMlpConfig:
    kind: str  # "dense" or "moe"
    ff: int  # dense: the inner size; moe: an expert's inner size
    experts: int = 0
    top: int = 0
    shared_ff: int = 0  # 0: no shared expert

    @classmethod
    def from_dict(cls, d, where):
        if not isinstance(d, dict) or "kind" not in d:
            raise ConfigError(f"{where}: expected an object with a kind")
        if d["kind"] == "dense":
            _, ff = _take(d, ("kind", "ff"), where)
            return cls("dense", int(ff))
        if d["kind"] == "moe":
            _, router, expert, shared = _take_some(d, ("kind", "router", "expert"), ("shared",), where)
            experts, top = _take(router, ("experts", "top"), where + ".router")
            (ff,) = _take(expert, ("ff",), where + ".expert")
            shared_ff = 0
            if shared is not None:
                (shared_ff,) = _take(shared, ("ff",), where + ".shared")
            if not 1 <= int(top) <= int(experts):
                raise ConfigError(f"{where}.router: top must lie between 1 and experts")
            return cls("moe", int(ff), int(experts), int(top), int(shared_ff))
        raise ConfigError(f"{where}: kind {d['kind']!r} is not known (known: 'dense', 'moe')")

    def to_dict(self):
        if self.kind == "dense":
            return {"kind": "dense", "ff": self.ff}
        d = {"kind": "moe", "router": {"experts": self.experts, "top": self.top}, "expert": {"ff": self.ff}}
        if self.shared_ff:
            d["shared"] = {"ff": self.shared_ff}
        return d


@dataclass(frozen=True)
class PazivikLayerConfig:
    type: str
    mixer: LatentAttentionConfig
    mlp: PazivikMlpConfig | None

    @classmethod
    def from_dict(cls, d, where):
        kind, mixer, mlp = _take(d, ("type", "mixer", "mlp"), where)
        if kind != "latent_attention":
            raise ConfigError(f"{where}: layer type {kind!r} is not known (known: 'latent_attention')")
        return cls(kind, LatentAttentionConfig.from_dict(mixer, where + ".mixer"),
                   None if mlp is None else PazivikMlpConfig.from_dict(mlp, where + ".mlp"))

    def to_dict(self):
        return {"type": self.type, "mixer": self.mixer.to_dict(),
                "mlp": None if self.mlp is None else self.mlp.to_dict()}


@dataclass(frozen=True)
class PazivikConfig:
    vocab_size: int
    hidden_size: int
    norm_eps: float
    logit_softcap: float  # 0: none
    bigram_buckets: int
    bigram_mul_prev: int
    bigram_mul_cur: int
    layers: tuple[PazivikLayerConfig, ...]

    architecture = "Pazivik"
    max_position_embeddings = 1 << 20  # positions enter through a computed sinusoid and a window
    tie_word_embeddings = True
    eos_token_ids: tuple[int, ...] = ()

    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)

    def num_parameters(self) -> int:
        from ..models.pazivik import pazivik_checkpoint_layout

        total = 0
        for entry in pazivik_checkpoint_layout(self).entries:
            for src in entry.sources:
                n = 1
                for k in src.shape:
                    n *= k
                total += n
        return total

    @classmethod
    def from_dict(cls, d: dict[str, Any]) -> "PazivikConfig":
        required = ("architecture", "embedding", "layers", "norm", "vocab", "width")
        known = required + ("logit_softcap",)
        # keys beside these at the top describe the file, not the model (a name, a seed)
        arch, emb, layers, norm, vocab, width, cap = _take_some(
            {k: v for k, v in d.items() if k in known}, required, ("logit_softcap",), "config")
        if arch != cls.architecture:
            raise ConfigError(f"config: architecture {arch!r} is not {cls.architecture!r}")
        (eps,) = _take(norm, ("eps",), "config.norm")
        (bigram,) = _take(emb, ("bigram",), "config.embedding")
        buckets, mul_cur, mul_prev = _take(bigram, ("buckets", "mul_cur", "mul_prev"), "config.embedding.bigram")
        if int(buckets) < 1:
            raise ConfigError("config.embedding.bigram: buckets must be positive")
        if not layers:
            raise ConfigError("config: no layers")
        out = tuple(PazivikLayerConfig.from_dict(l, f"config.layers[{i}]") for i, l in enumerate(layers))
        for i, l in enumerate(out):
            j = l.mixer.kv_from
            if j is None:
                continue
            if not 0 <= j < i or out[j].mixer.kv_from is not None:
                raise ConfigError(f"config.layers[{i}].mixer: kv_from must name an earlier layer with a latent of its own")
            if out[j].mixer.kv_rank != l.mixer.kv_rank:
                raise ConfigError(f"config.layers[{i}].mixer: kv_rank differs from layer {j}'s")
        return cls(int(vocab), int(width), float(eps), float(cap or 0.0), int(buckets), int(mul_prev),
                   int(mul_cur), out)

    @classmethod
    def from_pretrained(cls, path: str | Path) -> "PazivikConfig":
        return cls.from_dict(json.loads((Path(path) / "config.json").read_text()))

    def to_dict(self) -> dict[str, Any]:
        d = {"architecture": self.architecture,
             "embedding": {"bigram": {"buckets": self.bigram_buckets, "mul_cur": self.bigram_mul_cur,
                                      "mul_prev": self.bigram_mul_prev}},
             "layers": [l.to_dict() for l in self.layers], "norm": {"eps": self.norm_eps},
             "vocab": self.vocab_size, "width": self.hidden_size}
        if self.logit_softcap:
            d["logit_softcap"] = self.logit_softcap
        return d
