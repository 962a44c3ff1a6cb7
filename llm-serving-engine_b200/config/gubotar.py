"""Typed configuration of the Gubotar architecture, read from its ``config.json``.

The file names the architecture (``"architecture": "Gubotar"``), the vocabulary and the width,
the epsilon of every norm (``norm.eps``) and a list ``layers``. Each entry of the list has a
``type`` (which mixer the layer has), the mixer's sizes and constants under ``mixer`` and its
feed-forward under ``mlp`` (``{"kind": "dense", "ff": F}`` or null). Layers may differ from one
another in every size. Nothing has a default: a key that is absent is an error, and so is a key
of a layer that this engine does not know, because it would change the math silently.

Mixers:

* ``parallel``: ``mixer.left`` (chunked softmax attention: ``heads``, ``kv_heads``, ``dim``,
  ``vdim``, ``scale``, ``mask.size``) beside ``mixer.right`` (linear attention with a decay per
  head: ``heads``, ``dim``, ``vdim``, ``decay``);
* ``retention``: ``heads``, ``dim``, ``vdim``, ``decay`` and rotary positions ``rot.dims``,
  ``rot.base``.
"""

from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Any

from .llama import ConfigError


def _take(d: dict, keys: tuple[str, ...], where: str) -> list:
    if not isinstance(d, dict):
        raise ConfigError(f"{where}: expected an object")
    missing = [k for k in keys if k not in d]
    unknown = [k for k in d if k not in keys]
    if missing or unknown:
        raise ConfigError(f"{where}: missing keys {missing}, unknown keys {unknown}")
    return [d[k] for k in keys]


def _decays(values, heads: int, where: str) -> tuple[float, ...]:
    out = tuple(float(v) for v in values)
    if len(out) != heads:
        raise ConfigError(f"{where}: {len(out)} decays for {heads} heads")
    return out


@dataclass(frozen=True)
class ChunkedAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    chunk: int  # a query sees the keys of its own chunk of this many positions

    @classmethod
    def from_dict(cls, d, where):
        heads, kv, dim, vdim, scale, mask = _take(d, ("heads", "kv_heads", "dim", "vdim", "scale", "mask"), where)
        (size,) = _take(mask, ("size",), where + ".mask")
        if heads % kv:
            raise ConfigError(f"{where}: heads must be a multiple of kv_heads")
        if vdim != dim:
            raise ConfigError(f"{where}: the values are the projected keys, so vdim must equal dim")
        if size < 1:
            raise ConfigError(f"{where}: mask.size must be positive")
        return cls(int(heads), int(kv), int(dim), int(vdim), float(scale), int(size))

    def to_dict(self):
        return {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim,
                "scale": self.scale, "mask": {"size": self.chunk}}


@dataclass(frozen=True)
class DecayAttentionConfig:
    heads: int
    dim: int
    vdim: int
    decay: tuple[float, ...]
    rot_dims: int = 0  # 0: no rotary positions
    rot_base: float = 0.0

    @classmethod
    def from_dict(cls, d, where, rotary: bool):
        if rotary:
            heads, dim, vdim, decay, rot = _take(d, ("heads", "dim", "vdim", "decay", "rot"), where)
            dims, base = _take(rot, ("dims", "base"), where + ".rot")
            if dims % 2 or not 0 < dims <= dim:
                raise ConfigError(f"{where}: rot.dims must be even and at most dim")
            return cls(int(heads), int(dim), int(vdim), _decays(decay, heads, where), int(dims), float(base))
        heads, dim, vdim, decay = _take(d, ("heads", "dim", "vdim", "decay"), where)
        return cls(int(heads), int(dim), int(vdim), _decays(decay, heads, where))

    def to_dict(self):
        d = {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "decay": list(self.decay)}
        if self.rot_dims:
            d["rot"] = {"dims": self.rot_dims, "base": self.rot_base}
        return d


@dataclass(frozen=True)
class GubotarLayerConfig:
    type: str  # "parallel" or "retention"
    left: ChunkedAttentionConfig | None
    right: DecayAttentionConfig | None  # the linear half of "parallel"
    retention: DecayAttentionConfig | None
    ff: int  # 0: the layer has no feed-forward

    @classmethod
    def from_dict(cls, d, where):
        kind, mixer, mlp = _take(d, ("type", "mixer", "mlp"), where)
        ff = 0
        if mlp is not None:
            mk, ff = _take(mlp, ("kind", "ff"), where + ".mlp")
            if mk != "dense":
                raise ConfigError(f"{where}.mlp: kind {mk!r} is not known (known: 'dense')")
        if kind == "parallel":
            left, right = _take(mixer, ("left", "right"), where + ".mixer")
            return cls(kind, ChunkedAttentionConfig.from_dict(left, where + ".mixer.left"),
                       DecayAttentionConfig.from_dict(right, where + ".mixer.right", False), None, int(ff))
        if kind == "retention":
            return cls(kind, None, None, DecayAttentionConfig.from_dict(mixer, where + ".mixer", True), int(ff))
        raise ConfigError(f"{where}: layer type {kind!r} is not known (known: 'parallel', 'retention')")

    def to_dict(self):
        mixer = (self.retention.to_dict() if self.type == "retention"
                 else {"left": self.left.to_dict(), "right": self.right.to_dict()})
        return {"type": self.type, "mixer": mixer,
                "mlp": {"kind": "dense", "ff": self.ff} if self.ff else None}


@dataclass(frozen=True)
class GubotarConfig:
    vocab_size: int
    hidden_size: int
    norm_eps: float
    layers: tuple[GubotarLayerConfig, ...]

    architecture = "Gubotar"
    # positions enter through a chunk's mask, a distance and rotation angles: nothing bounds them
    max_position_embeddings = 1 << 20
    tie_word_embeddings = True
    eos_token_ids: tuple[int, ...] = ()

    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)

    def num_parameters(self) -> int:
        """Every checkpoint tensor once (the embedding table is also the output projection)."""
        from ..models.gubotar import gubotar_checkpoint_layout

        total = 0
        for entry in gubotar_checkpoint_layout(self).entries:
            for src in entry.sources:
                n = 1
                for k in src.shape:
                    n *= k
                total += n
        return total

    @classmethod
    def from_dict(cls, d: dict[str, Any]) -> "GubotarConfig":
        known = ("architecture", "layers", "norm", "vocab", "width")
        # keys beside these at the top describe the file, not the model (a name, a seed)
        arch, layers, norm, vocab, width = _take({k: v for k, v in d.items() if k in known}, known, "config")
        if arch != cls.architecture:
            raise ConfigError(f"config: architecture {arch!r} is not {cls.architecture!r}")
        (eps,) = _take(norm, ("eps",), "config.norm")
        if not layers:
            raise ConfigError("config: no layers")
        return cls(int(vocab), int(width), float(eps),
                   tuple(GubotarLayerConfig.from_dict(l, f"config.layers[{i}]") for i, l in enumerate(layers)))

    @classmethod
    def from_pretrained(cls, path: str | Path) -> "GubotarConfig":
        return cls.from_dict(json.loads((Path(path) / "config.json").read_text()))

    def to_dict(self) -> dict[str, Any]:
        return {"architecture": self.architecture, "layers": [l.to_dict() for l in self.layers],
                "norm": {"eps": self.norm_eps}, "vocab": self.vocab_size, "width": self.hidden_size}
