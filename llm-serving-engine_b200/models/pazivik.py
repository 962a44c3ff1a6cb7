"""The Pazivik architecture as data: which parts each layer has and where its tensors come from.

The embedded token is the sum of its row of the embedding table, a row of a second table chosen
by the token and the one before it (``hashed_pair``) and a sinusoidal position vector. Every layer
is a ``prenorm`` block whose mixer is latent attention with a window and a sink per head; a layer
may read the latent rows of an earlier layer instead of making its own (the two then share a
cache layer, which keeps the larger of their windows). The feed-forward is dense (gated, the tanh
form of gelu), a set of routed experts with a shared one, or absent. The output projection is the
embedding table; the logits are soft-capped.

Checkpoint tensors are named ``l<i>.<part>``; the matrices of one product are concatenated along
their rows (q | dkv, gate | up, all experts' gate | up, all experts' down, router | shared gate).
"""

from __future__ import annotations

from ..config.pazivik import PazivikConfig
from ..parts.blocks import PreNormBlockSpec
from ..parts.embed_terms import HashedPairSpec
from ..parts.feed_forward import SwiGLUSpec
from ..parts.latent_attention import LatentAttentionSpec, needs_materialized_heads
from ..parts.moe import RoutedExpertsSpec
from ..parts.norms import RMSNormSpec
from ..parts.positions import SinusoidSpec
from .plan import CheckpointLayout, ModelPlan, ParamSource, RunEntry, Source

SINUSOID_BASE = 10000.0


def _cache_of(cfg: PazivikConfig) -> list[int]:
    """Layer -> the layer whose cache it uses (itself, or the one it reads)."""
    return [i if l.mixer.kv_from is None else l.mixer.kv_from for i, l in enumerate(cfg.layers)]


def pazivik_plan(cfg: PazivikConfig) -> ModelPlan:
    w, eps = cfg.hidden_size, cfg.norm_eps
    norm = RMSNormSpec(w, eps)
    owner = _cache_of(cfg)
    # a shared cache layer keeps what its most far-sighted reader needs (0: everything)
    keep: dict[int, int] = {}
    for i, l in enumerate(cfg.layers):
        win = l.mixer.window
        keep[owner[i]] = 0 if (win == 0 or keep.get(owner[i], win) == 0) else max(keep.get(owner[i], 0), win)
    layers = []
    # a rank beyond the attention kernels' head sizes: such a layer keeps keys and values of its
    # own (every layer its own cache layer and window) and is handed the step's latent rows
    wide = [needs_materialized_heads(l.mixer.kv_rank) for l in cfg.layers]
    for i, l in enumerate(cfg.layers):
        m = l.mixer
        mixer = LatentAttentionSpec(
            hidden_size=w, num_heads=m.heads, head_dim=m.dim, value_dim=m.vdim, latent_rank=m.kv_rank,
            scale=m.scale, eps=eps, window=m.window, cache_window=m.window if wide[i] else keep[owner[i]],
            own_latent=m.kv_from is None, sinks=True, materialize=wide[i], latent_key=owner[i])
        if l.mlp is None:
            ff = None
        elif l.mlp.kind == "dense":
            ff = SwiGLUSpec(w, l.mlp.ff, activation="gelu_tanh")
        else:
            ff = RoutedExpertsSpec(w, l.mlp.experts, l.mlp.top, l.mlp.ff, l.mlp.shared_ff, activation="silu")
        layers.append(PreNormBlockSpec(norm_in=norm, mixer=mixer, norm_post=norm if ff is not None else None,
                                       feed_forward=ff))
    users = sorted({i if wide[i] else owner[i] for i in range(len(layers))})
    cache_id = {o: k for k, o in enumerate(users)}
    return ModelPlan(
        vocab_size=cfg.vocab_size, hidden_size=w, layers=tuple(layers),
        run_order=tuple(RunEntry(i, cache_id[i if wide[i] else owner[i]]) for i in range(len(layers))),
        final_norm=norm, tie_head=True, embed_position=SinusoidSpec(w, SINUSOID_BASE),
        embed_terms=(HashedPairSpec(w, cfg.bigram_buckets, cfg.bigram_mul_prev, cfg.bigram_mul_cur),),
        logit_softcap=cfg.logit_softcap)


def pazivik_checkpoint_layout(cfg: PazivikConfig) -> CheckpointLayout:
    w = cfg.hidden_size
    entries = [
        ParamSource("embed.weight", (Source("embed", (cfg.vocab_size, w)),), "embedding"),
        ParamSource("embed_terms.0.table", (Source("bigram", (cfg.bigram_buckets + 1, w)),), "embedding"),
        ParamSource("final_norm.weight", (Source("final.norm", (w,)),), "scale"),
    ]
    ignored = []
    for i, l in enumerate(cfg.layers):
        src, dst, m = f"l{i}.", f"layers.{i}.", l.mixer
        q = Source(src + "mix.q", (m.heads * m.dim, w))
        entries.append(ParamSource(dst + "norm_in.weight", (Source(src + "norm1", (w,)),), "scale"))
        if m.kv_from is None:
            entries += [
                ParamSource(dst + "mixer.in.weight", (q, Source(src + "mix.dkv", (m.kv_rank, w)))),
                ParamSource(dst + "mixer.latent_norm.weight", (Source(src + "mix.dkv.norm", (m.kv_rank,)),), "scale"),
            ]
        else:
            entries.append(ParamSource(dst + "mixer.in.weight", (q,)))
        entries += [
            ParamSource(dst + "mixer.uk.weight", (Source(src + "mix.uk", (m.heads * m.dim, m.kv_rank)),)),
            ParamSource(dst + "mixer.uv.weight", (Source(src + "mix.uv", (m.heads * m.vdim, m.kv_rank)),)),
            ParamSource(dst + "mixer.sink", (Source(src + "mix.sink", (m.heads,)),), "offset"),
            ParamSource(dst + "mixer.o.weight", (Source(src + "mix.o", (w, m.heads * m.vdim)),)),
        ]
        if l.mlp is None:
            ignored.append(src + "norm2")  # a file may carry the unused norm of a layer without feed-forward
            continue
        entries.append(ParamSource(dst + "norm_post.weight", (Source(src + "norm2", (w,)),), "scale"))
        ms, md = src + "mlp.", dst + "feed_forward."

        def gated(s_, d_, ff):
            return [ParamSource(d_ + "gate_up.weight", (Source(s_ + "gate", (ff, w)), Source(s_ + "up", (ff, w)))),
                    ParamSource(d_ + "down.weight", (Source(s_ + "down", (w, ff)),))]

        if l.mlp.kind == "dense":
            entries += gated(ms, md, l.mlp.ff)
            continue
        E, ff = l.mlp.experts, l.mlp.ff
        router = [Source(ms + "router", (E, w))]
        if l.mlp.shared_ff:
            router.append(Source(ms + "shared.sg", (1, w)))
            entries += gated(ms + "shared.", md + "shared.", l.mlp.shared_ff)
        entries += [
            ParamSource(md + "router.weight", tuple(router), "matrix32"),
            ParamSource(md + "experts.gate_up.weight",
                        tuple(Source(f"{ms}e{e}.{n}", (ff, w)) for e in range(E) for n in ("gate", "up"))),
            ParamSource(md + "experts.down.weight", tuple(Source(f"{ms}e{e}.down", (w, ff)) for e in range(E))),
        ]
    return CheckpointLayout(entries=tuple(entries), ignored_names=tuple(ignored))
