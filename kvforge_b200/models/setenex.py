"""The Setenex decoder as a ``ModelSpec``: which parts, with which constants, under which tensor
names.  Every layer is the parallel arrangement (one norm; the mixer and the feed-forward both read
its output and both add to the stream) with a norm whose tensor holds the weight's offset from one; its mixer is
grouped-query attention without rotation whose heads are normed and whose scores take a bias by
distance, under a window that keeps the first tokens (``attention``), or attention over a latent shared
by keys and values with a gate per head (``latent_attention``); its feed-forward, where it has one, is
made of routed experts.  A stretch of layers may run several times with the same weights; every pass
has cache entries of its own and is marked by a row added to the stream.  Tensors of layer ``i`` start
with ``l<i>.``."""

from __future__ import annotations

from ..config.setenex_config import BiasedAttentionConfig, ExpertsConfig, LatentAttentionConfig, SetenexConfig
from ..parts.base import PartSpec
from ..parts.model import LayerCall, LayerSpec, ModelSpec


def _attention(cfg: SetenexConfig, a: BiasedAttentionConfig) -> PartSpec:
    return PartSpec(
        "paged_attention",
        {
            "hidden_size": cfg.hidden_size, "num_heads": a.heads, "num_kv_heads": a.kv_heads, "head_dim": a.dim, "v_head_dim": a.vdim,
            "scale": a.scale, "window": a.window, "keep_first": a.keep_first if a.window is not None else 0, "position": None,
            "qk_norm": {"eps": cfg.eps}, "distance_bias": {"rows": a.bias_rows, "far": a.bias_max},
            "names": {
                "q_proj.weight": "q", "k_proj.weight": "k", "v_proj.weight": "v", "o_proj.weight": "o",
                "q_norm.weight": "q.norm", "k_norm.weight": "k.norm",
            },
        },
    )  # fmt: skip


def _latent(cfg: SetenexConfig, a: LatentAttentionConfig) -> PartSpec:
    position = PartSpec("rotary", {"head_dim": a.rot_dim, "rotary_dim": a.rot_dims, "theta": a.rot_base, "interleaved": True, "scaling": None})
    return PartSpec(
        "latent_attention",
        {
            "hidden_size": cfg.hidden_size, "num_heads": a.heads, "head_dim": a.dim, "rot_dim": a.rot_dim, "v_head_dim": a.vdim,
            "kv_rank": a.kv_rank, "eps": cfg.eps, "scale": a.scale, "window": a.window, "position": position, "gate": "sigmoid",
        },
    )  # fmt: skip


def _experts(cfg: SetenexConfig, e: ExpertsConfig) -> PartSpec:
    return PartSpec(
        "routed_experts",
        {
            "hidden_size": cfg.hidden_size, "experts": e.experts, "top": e.top, "intermediate_size": e.ff, "activation": "gelu",
            "groups": e.groups, "keep": e.keep, "correction": True,
        },
    )  # fmt: skip


def setenex_spec(cfg: SetenexConfig) -> ModelSpec:
    norm = lambda name: PartSpec("rmsnorm", {"dim": cfg.hidden_size, "eps": cfg.eps, "one_plus": True, "names": {"weight": name}})  # noqa: E731
    layers = []
    for i, lc in enumerate(cfg.layers):
        mixer = _attention(cfg, lc.mixer) if lc.type == "attention" else _latent(cfg, lc.mixer)
        block = PartSpec(
            "parallel",
            {"norm": norm("norm1"), "mixer": mixer, "ffn": _experts(cfg, lc.mlp) if lc.mlp is not None else None, "norm_name": "", "mixer_name": "mix", "ffn_name": "mlp"},
        )
        layers.append(LayerSpec(block=block, prefix=f"l{i}."))
    n = len(cfg.layers)
    if cfg.loop is None:
        execution, passes = [LayerCall(i) for i in range(n)], 0
    else:
        lp = cfg.loop
        execution = [LayerCall(i) for i in range(lp.start)]
        for t in range(lp.times):
            execution += [LayerCall(i, offset_row=t if i == lp.start else None) for i in range(lp.start, lp.stop)]
        execution += [LayerCall(i) for i in range(lp.stop, n)]
        passes = lp.times
    return ModelSpec(
        architecture=cfg.architecture,
        hidden_size=cfg.hidden_size,
        vocab_size=cfg.vocab_size,
        layers=layers,
        execution=execution,
        final_norm=norm("norm"),
        final_norm_prefix="final.",
        embedding_name="embed",
        lm_head_name="head",
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab_size, "hidden_size": cfg.hidden_size, "scale": cfg.embedding_scale}),
        ignore_suffixes=(),
        max_position_embeddings=cfg.max_position_embeddings,
        pass_offsets=passes,
        pass_offsets_name="loop.step",
    )
