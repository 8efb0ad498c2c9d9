"""The Mopilorn decoder as a ``ModelSpec``: which parts, with which constants, under which tensor
names.  Every layer is the pre-norm arrangement over several residual streams (or over one, with the
plain sum, when the configuration names no streams); its mixer is either attention and a delta rule
side by side (``parallel``) or a delta rule with one decay a key channel (``channel_delta``); its
feed-forward, where it has one, is the gated one.  Tensors of layer ``i`` start with ``l<i>.``."""

from __future__ import annotations

from ..config.mopilorn_config import AttentionConfig, DeltaConfig, MopilornConfig
from ..parts.base import PartSpec
from ..parts.model import LayerSpec, ModelSpec


def _attention(cfg: MopilornConfig, a: AttentionConfig) -> PartSpec:
    position = None
    if a.rot is not None:
        sc = a.rot.scaling
        position = PartSpec(
            "rotary",
            {
                "head_dim": a.dim,
                "rotary_dim": a.rot.dims,
                "theta": a.rot.base,
                "interleaved": True,
                "scaling": {
                    "factor": sc["factor"],
                    "low_freq_factor": sc["low"],
                    "high_freq_factor": sc["high"],
                    "original_max_position_embeddings": sc["original"],
                }
                if sc
                else None,
            },
        )
    return PartSpec(
        "paged_attention",
        {
            "hidden_size": cfg.hidden_size,
            "num_heads": a.heads,
            "num_kv_heads": a.kv_heads,
            "head_dim": a.dim,
            "v_head_dim": a.vdim,
            "conv": a.conv,
            "scale": a.scale,
            "window": a.window,
            "position": position,
            "names": {
                "q_proj.weight": "q", "k_proj.weight": "k", "v_proj.weight": "v", "o_proj.weight": "o",
                "q_proj.conv": "q.conv", "k_proj.conv": "k.conv", "v_proj.conv": "v.conv",
            },
        },
    )  # fmt: skip


def _delta(cfg: MopilornConfig, d: DeltaConfig, channel: bool) -> PartSpec:
    return PartSpec(
        "gated_delta_rule",
        {
            "hidden_size": cfg.hidden_size,
            "num_heads": d.heads,
            "num_kv_heads": d.kv_heads,
            "head_dim": d.dim,
            "v_head_dim": d.vdim,
            "conv": d.conv,
            "eps": cfg.eps,
            "decay": "channel" if channel else "head",
            "decay_rank": d.decay_rank if channel else None,
            "gate_rank": d.gate_rank if channel else None,
            "gate": "sigmoid" if channel else "silu",
        },
    )


def mopilorn_spec(cfg: MopilornConfig) -> ModelSpec:
    streams = cfg.streams
    layers = []
    for i, lc in enumerate(cfg.layers):
        if lc.type == "parallel":
            mixer = PartSpec(
                "parallel_mixers",
                {"hidden_size": cfg.hidden_size, "eps": cfg.eps, "branches": [("left", _attention(cfg, lc.left)), ("right", _delta(cfg, lc.right, False))]},
            )
        else:
            mixer = _delta(cfg, lc.right, True)
        ffn = None
        if lc.ff is not None:
            ffn = PartSpec(
                "gated_mlp",
                {
                    "hidden_size": cfg.hidden_size, "intermediate_size": lc.ff, "activation": "silu",
                    "names": {"gate_proj.weight": "gate", "up_proj.weight": "up", "down_proj.weight": "down"},
                },
            )  # fmt: skip
        if streams is not None:
            norm = lambda name: PartSpec("stream_rmsnorm", {"dim": cfg.hidden_size, "eps": cfg.eps, "streams": streams, "names": {"weight": name}})  # noqa: E731
            block = PartSpec("stream_prenorm", {"streams": streams, "norm1": norm("norm1"), "mixer": mixer, "norm2": norm("norm2") if ffn else None, "ffn": ffn})
            for part in ("norm1", "norm2"):
                block.params[part + "_name"] = ""  # the norm's tensor is l<i>.norm1 itself
        else:
            norm = lambda name: PartSpec("rmsnorm", {"dim": cfg.hidden_size, "eps": cfg.eps, "names": {"weight": name}})  # noqa: E731
            if ffn is None:
                raise ValueError("a layer without a feed-forward needs the arrangement over several streams")
            block = PartSpec(
                "prenorm",
                {"norm1": norm("norm1"), "mixer": mixer, "norm2": norm("norm2"), "ffn": ffn, "norm1_name": "", "norm2_name": "", "mixer_name": "mix", "ffn_name": "mlp"},
            )
        layers.append(LayerSpec(block=block, prefix=f"l{i}."))
    final_kind = "stream_rmsnorm" if streams is not None else "rmsnorm"
    final = {"dim": cfg.hidden_size, "eps": cfg.eps, "names": {"weight": "norm"}}
    if streams is not None:
        final["streams"] = streams
    return ModelSpec(
        architecture=cfg.architecture,
        hidden_size=cfg.hidden_size,
        vocab_size=cfg.vocab_size,
        layers=layers,
        final_norm=PartSpec(final_kind, final),
        final_norm_prefix="final.",
        embedding_name="embed",
        lm_head_name="head",
        head=PartSpec("linear_head", {"vocab_size": cfg.vocab_size, "hidden_size": cfg.hidden_size, "softcap": cfg.logit_softcap}),
        ignore_suffixes=(),
        max_position_embeddings=cfg.max_position_embeddings,
        residual_streams=streams if streams is not None else 1,
    )
