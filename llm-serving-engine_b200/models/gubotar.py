"""The Gubotar architecture as data: which parts each layer has and where its tensors come from.

Every layer is a ``branchnorm`` block (the norm stands on a branch's output, weights stored
around zero) whose mixer reads the token-shifted residual stream. Two kinds of layer:

* ``parallel``: chunked softmax attention (keys double as values, query/key norm, a temperature
  per head, a distance penalty with slope ``2^(-8 (h+1) / H)`` for head h) beside linear attention
  with a decay per head (``silu`` on q, k, v; all heads normed together; sigmoid gate); the two
  outputs are normed one by one and averaged;
* ``retention``: linear attention with a decay per head, rotary positions on part of q and k,
  keys scaled by ``key_dim^(-1/2)``, every head's output divided by its root mean square, ``silu``
  gate.

The feed-forward is the dense gated one. The output projection is the embedding table.

Checkpoint tensors are named ``l<i>.<part>``; the matrices of one product are concatenated along
their rows (q | k, q | k | v | g, gate | up) when they are read.
"""

from __future__ import annotations

from ..config.gubotar import GubotarConfig, GubotarLayerConfig
from ..parts.attention import AttentionSpec
from ..parts.blocks import BranchNormBlockSpec
from ..parts.feed_forward import SwiGLUSpec
from ..parts.linear_attention import DecayLinearAttentionSpec
from ..parts.norms import RMSNormSpec
from ..parts.parallel import ParallelMixerSpec
from ..parts.positions import NoPositionSpec, RotarySpec
from ..parts.token_shift import TokenShiftSpec
from .plan import CheckpointLayout, ModelPlan, ParamSource, RunEntry, Source

SLOPE_EXPONENT = 8.0  # head h of H takes slope 2^(-SLOPE_EXPONENT (h+1) / H) per position of distance


def distance_slopes(heads: int) -> tuple[float, ...]:
    return tuple(2.0 ** (-SLOPE_EXPONENT * (h + 1) / heads) for h in range(heads))


def _mixer_spec(cfg: GubotarConfig, layer: GubotarLayerConfig):
    w, eps = cfg.hidden_size, cfg.norm_eps
    if layer.type == "retention":
        r = layer.retention
        return DecayLinearAttentionSpec(
            hidden_size=w, num_heads=r.heads, key_dim=r.dim, value_dim=r.vdim, decay=r.decay, eps=eps,
            activation="none", key_scale=r.dim ** -0.5,
            position=RotarySpec(head_dim=r.rot_dims, theta=r.rot_base),
            out_norm="heads", gate_activation="silu")
    a, b = layer.left, layer.right
    left = AttentionSpec(
        hidden_size=w, num_heads=a.heads, num_kv_heads=a.kv_heads, head_dim=a.dim, scale=a.scale,
        position=NoPositionSpec(), qk_norm_eps=eps, values_are_keys=True, head_temperature=True,
        distance_slopes=distance_slopes(a.heads), chunk=a.chunk)
    right = DecayLinearAttentionSpec(
        hidden_size=w, num_heads=b.heads, key_dim=b.dim, value_dim=b.vdim, decay=b.decay, eps=eps,
        activation="silu", key_scale=1.0, position=None, out_norm="row", gate_activation="sigmoid")
    return ParallelMixerSpec(hidden_size=w, names=("left", "right"), branches=(left, right),
                             coefficients=(0.5, 0.5), eps=eps)


def gubotar_plan(cfg: GubotarConfig) -> ModelPlan:
    norm = RMSNormSpec(cfg.hidden_size, cfg.norm_eps, unit_offset=True)
    layers = tuple(
        BranchNormBlockSpec(
            mixer=_mixer_spec(cfg, layer), norm_mixer=norm,
            feed_forward=SwiGLUSpec(cfg.hidden_size, layer.ff) if layer.ff else None,
            norm_ff=norm if layer.ff else None,
            input_filter=TokenShiftSpec(cfg.hidden_size))
        for layer in cfg.layers)
    n = len(layers)
    return ModelPlan(
        vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size, layers=layers,
        run_order=tuple(RunEntry(i, i) for i in range(n)), final_norm=norm, tie_head=True)


def _linear_attention_sources(src: str, dst: str, w: int, r) -> list[ParamSource]:
    qk, vg = r.heads * r.dim, r.heads * r.vdim
    return [
        ParamSource(dst + "qkvg.weight", (Source(src + "q", (qk, w)), Source(src + "k", (qk, w)),
                                          Source(src + "v", (vg, w)), Source(src + "g", (vg, w)))),
        ParamSource(dst + "o.weight", (Source(src + "o", (w, vg)),)),
    ]


def gubotar_checkpoint_layout(cfg: GubotarConfig) -> CheckpointLayout:
    w = cfg.hidden_size
    entries = [
        ParamSource("embed.weight", (Source("embed", (cfg.vocab_size, w)),), "embedding"),
        ParamSource("final_norm.weight", (Source("final.norm", (w,)),), "offset"),
    ]
    ignored = []
    for i, layer in enumerate(cfg.layers):
        src, dst = f"l{i}.", f"layers.{i}."
        entries += [
            ParamSource(dst + "norm_mixer.weight", (Source(src + "norm1", (w,)),), "offset"),
            ParamSource(dst + "filter.mix", (Source(src + "shift", (w,)),), "mix"),
        ]
        if layer.ff:
            entries += [
                ParamSource(dst + "norm_ff.weight", (Source(src + "norm2", (w,)),), "offset"),
                ParamSource(dst + "feed_forward.gate_up.weight",
                            (Source(src + "mlp.gate", (layer.ff, w)), Source(src + "mlp.up", (layer.ff, w)))),
                ParamSource(dst + "feed_forward.down.weight", (Source(src + "mlp.down", (w, layer.ff)),)),
            ]
        else:
            ignored.append(src + "norm2")  # a file may carry the unused norm of a layer without feed-forward
        if layer.type == "retention":
            entries += _linear_attention_sources(src + "mix.", dst + "mixer.", w, layer.retention)
            continue
        a, b = layer.left, layer.right
        ls, ld = src + "mix.left.", dst + "mixer.left."
        entries += [
            ParamSource(ld + "qkv.weight", (Source(ls + "q", (a.heads * a.dim, w)),
                                            Source(ls + "k", (a.kv_heads * a.dim, w)))),
            ParamSource(ld + "o.weight", (Source(ls + "o", (w, a.heads * a.dim)),)),
            ParamSource(ld + "q_norm.weight", (Source(ls + "q.norm", (a.dim,)),), "scale"),
            ParamSource(ld + "k_norm.weight", (Source(ls + "k.norm", (a.dim,)),), "scale"),
            ParamSource(ld + "temperature", (Source(ls + "temp", (a.heads,)),), "scale"),
        ]
        entries += _linear_attention_sources(src + "mix.right.", dst + "mixer.right.", w, b)
        entries += [
            ParamSource(dst + "mixer.right.norm.weight", (Source(src + "mix.right.norm", (b.heads * b.vdim,)),), "scale"),
            ParamSource(dst + "mixer.out.left.weight", (Source(src + "mix.left.out", (w,)),), "scale"),
            ParamSource(dst + "mixer.out.right.weight", (Source(src + "mix.right.out", (w,)),), "scale"),
        ]
    return CheckpointLayout(entries=tuple(entries), ignored_names=tuple(ignored))
