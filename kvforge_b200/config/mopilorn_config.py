"""Typed configuration of the Mopilorn decoder, read from its ``config.json``.

The file gives every size and every constant that differs between models of the design::

    {"architecture": "Mopilorn", "vocab": V, "width": W, "streams": S, "norm": {"eps": e},
     "logit_softcap": c, "layers": [{"type": "parallel" | "channel_delta", "mixer": {...},
                                     "mlp": {"kind": "dense", "ff": F} | null}, ...]}

A ``parallel`` mixer has a ``left`` part (attention: ``heads``, ``kv_heads``, ``dim``, ``vdim``,
``conv``, ``scale``, ``mask.size``, ``rot.{dims, base, scaling.{factor, low, high, original}}``) and a
``right`` part (delta rule with one decay a head: ``heads``, ``kv_heads``, ``dim``, ``vdim``,
``conv``); a ``channel_delta`` mixer has the delta rule's sizes (its low-rank inner sizes are read
from the tensors' shapes).  Nothing here has a default that stands for a size.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

from .model_config import ConfigError

ARCHITECTURE = "Mopilorn"


def _need(d: dict, key: str, where: str):
    if not isinstance(d, dict) or key not in d:
        raise ConfigError(f"config.json lacks {where}{key}")
    return d[key]


@dataclass(frozen=True)
class RotaryConfig:
    dims: int
    base: float
    scaling: dict[str, float] | None  # factor, low, high, original

    @classmethod
    def from_dict(cls, d: dict | None, where: str) -> RotaryConfig | None:
        if not d:
            return None
        sc = d.get("scaling")
        if sc:
            sc = {k: float(_need(sc, k, where + "scaling.")) for k in ("factor", "low", "high", "original")}
            if sc["high"] <= sc["low"]:
                raise ConfigError(f"{where}scaling needs high > low")
        dims = int(_need(d, "dims", where))
        if dims <= 0 or dims % 2:
            raise ConfigError(f"{where}dims must be positive and even")
        return cls(dims, float(_need(d, "base", where)), sc or None)


@dataclass(frozen=True)
class AttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int
    scale: float
    window: int | None
    rot: RotaryConfig | None

    @classmethod
    def from_dict(cls, d: dict, where: str) -> AttentionConfig:
        mask = d.get("mask")
        out = cls(
            heads=int(_need(d, "heads", where)), kv_heads=int(_need(d, "kv_heads", where)), dim=int(_need(d, "dim", where)),
            vdim=int(_need(d, "vdim", where)), conv=int(_need(d, "conv", where)), scale=float(_need(d, "scale", where)),
            window=int(_need(mask, "size", where + "mask.")) if mask else None,
            rot=RotaryConfig.from_dict(d.get("rot"), where + "rot."),
        )  # fmt: skip
        if out.kv_heads <= 0 or out.heads % out.kv_heads:
            raise ConfigError(f"{where}heads must be a multiple of kv_heads")
        if out.rot and out.rot.dims > out.dim:
            raise ConfigError(f"{where}rot.dims exceeds dim")
        if out.window is not None and out.window <= 0:
            raise ConfigError(f"{where}mask.size must be positive")
        return out


@dataclass(frozen=True)
class DeltaConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int
    decay_rank: int | None = None  # channel_delta: inner size of the step-size projection
    gate_rank: int | None = None  # channel_delta: inner size of the gate projection

    @classmethod
    def from_dict(cls, d: dict, where: str) -> DeltaConfig:
        out = cls(
            heads=int(_need(d, "heads", where)), kv_heads=int(_need(d, "kv_heads", where)), dim=int(_need(d, "dim", where)),
            vdim=int(_need(d, "vdim", where)), conv=int(_need(d, "conv", where)),
            decay_rank=d.get("decay_rank"), gate_rank=d.get("gate_rank"),
        )  # fmt: skip
        if out.kv_heads <= 0 or out.heads % out.kv_heads:
            raise ConfigError(f"{where}heads must be a multiple of kv_heads")
        return out


@dataclass(frozen=True)
class LayerConfig:
    type: str  # "parallel" or "channel_delta"
    left: AttentionConfig | None
    right: DeltaConfig | None  # the delta rule of either type
    ff: int | None  # None: the layer has no feed-forward


@dataclass
class MopilornConfig:
    vocab_size: int
    hidden_size: int
    streams: int | None  # None: a single residual stream with the plain sum
    eps: float
    logit_softcap: float | None
    layers: list[LayerConfig]
    architectures: list[str] = field(default_factory=lambda: [ARCHITECTURE])
    raw: dict[str, Any] = field(default_factory=dict, repr=False)

    @property
    def architecture(self) -> str:
        return self.architectures[0]

    @property
    def num_layers(self) -> int:
        return len(self.layers)

    @property
    def max_position_embeddings(self) -> int:
        return 1 << 30  # the design names no longest sequence

    @classmethod
    def from_dict(cls, d: dict[str, Any], tensor_shapes: dict[str, tuple[int, ...]] | None = None) -> MopilornConfig:
        """``tensor_shapes`` (checkpoint name -> shape), when given, supplies the inner sizes of
        low-rank projections, which the file does not name."""
        layers = []
        for i, ld in enumerate(_need(d, "layers", "")):
            where = f"layers[{i}]."
            kind, m = _need(ld, "type", where), _need(ld, "mixer", where)
            if kind == "parallel":
                left = AttentionConfig.from_dict(_need(m, "left", where + "mixer."), where + "mixer.left.")
                right = DeltaConfig.from_dict(_need(m, "right", where + "mixer."), where + "mixer.right.")
            elif kind == "channel_delta":
                left, right = None, DeltaConfig.from_dict(m, where + "mixer.")
                ranks = {}
                for key, stem in (("decay_rank", "a1"), ("gate_rank", "g1")):
                    shape = (tensor_shapes or {}).get(f"l{i}.mix.{stem}")
                    ranks[key] = int(shape[0]) if shape else getattr(right, key)
                    if not ranks[key]:
                        raise ConfigError(f"{where}mixer: the inner size of {stem} is neither in the file nor in the tensors")
                right = DeltaConfig(right.heads, right.kv_heads, right.dim, right.vdim, right.conv, **ranks)
            else:
                raise ConfigError(f"{where}type {kind!r} is not a mixer of this design ('parallel', 'channel_delta')")
            mlp = ld.get("mlp")
            if mlp is not None and _need(mlp, "kind", where + "mlp.") != "dense":
                raise ConfigError(f"{where}mlp.kind {mlp['kind']!r} is not supported (only 'dense')")
            layers.append(LayerConfig(kind, left, right, int(_need(mlp, "ff", where + "mlp.")) if mlp is not None else None))
        streams = d.get("streams")
        cap = d.get("logit_softcap")
        return cls(
            vocab_size=int(_need(d, "vocab", "")), hidden_size=int(_need(d, "width", "")),
            streams=int(streams) if streams is not None else None, eps=float(_need(_need(d, "norm", ""), "eps", "norm.")),
            logit_softcap=float(cap) if cap else None, layers=layers, raw=dict(d),
        )  # fmt: skip

    def to_hf_dict(self) -> dict[str, Any]:
        """The ``config.json`` of this configuration (low-rank inner sizes are written too; a reader
        that takes them from the tensors ignores them)."""

        def delta(c: DeltaConfig, ranks: bool) -> dict:
            out = {"conv": c.conv, "dim": c.dim, "heads": c.heads, "kv_heads": c.kv_heads, "vdim": c.vdim}
            if ranks:
                out.update(decay_rank=c.decay_rank, gate_rank=c.gate_rank)
            return out

        layers = []
        for lc in self.layers:
            if lc.type == "parallel":
                a = lc.left
                left = {"conv": a.conv, "dim": a.dim, "heads": a.heads, "kv_heads": a.kv_heads, "vdim": a.vdim, "scale": a.scale}
                if a.window is not None:
                    left["mask"] = {"size": a.window}
                if a.rot is not None:
                    left["rot"] = {"base": a.rot.base, "dims": a.rot.dims}
                    if a.rot.scaling:
                        left["rot"]["scaling"] = dict(a.rot.scaling)
                mixer = {"left": left, "right": delta(lc.right, False)}
            else:
                mixer = delta(lc.right, True)
            layers.append({"type": lc.type, "mixer": mixer, "mlp": {"kind": "dense", "ff": lc.ff} if lc.ff is not None else None})
        out = {"architecture": ARCHITECTURE, "vocab": self.vocab_size, "width": self.hidden_size, "norm": {"eps": self.eps}, "layers": layers}
        if self.streams is not None:
            out["streams"] = self.streams
        if self.logit_softcap:
            out["logit_softcap"] = self.logit_softcap
        return out


def alternating(
    *, vocab: int, width: int, num_layers: int, ff: int, streams: int | None, attn_heads: int, attn_kv_heads: int, dim: int, vdim: int,
    window: int | None, delta_heads: int, channel_heads: int, rank: int, conv: int = 4, rot_dims: int | None = None, base: float = 10000.0,
    eps: float = 1e-6, logit_softcap: float | None = 30.0,
) -> MopilornConfig:  # fmt: skip
    """A configuration whose layers alternate between the two mixers (the first is ``parallel``), with
    the same sizes in every layer of a kind: what the named shapes below are made with."""
    left = AttentionConfig(attn_heads, attn_kv_heads, dim, vdim, conv, dim**-0.5, window, RotaryConfig(rot_dims or dim, base, None))
    right = DeltaConfig(delta_heads, delta_heads, dim, vdim, conv)
    channel = DeltaConfig(channel_heads, channel_heads, dim, vdim, conv, rank, rank)
    layers = [LayerConfig("parallel", left, right, ff) if i % 2 == 0 else LayerConfig("channel_delta", None, channel, ff) for i in range(num_layers)]
    return MopilornConfig(vocab, width, streams, eps, logit_softcap, layers)


# Named shapes with random weights: a small one for demonstrations, and two with the widths of the Llama
# shapes this engine is measured on (equal width, layers, feed-forward and vocabulary).
MOPILORN_PRESETS: dict[str, MopilornConfig] = {
    "mopilorn-tiny": alternating(
        vocab=256, width=96, num_layers=3, ff=160, streams=2, attn_heads=4, attn_kv_heads=2, dim=32, vdim=48, window=24,
        delta_heads=2, channel_heads=3, rank=8, conv=3, rot_dims=16,
    ),
    "mopilorn-1b": alternating(
        vocab=128256, width=2048, num_layers=16, ff=8192, streams=4, attn_heads=16, attn_kv_heads=4, dim=128, vdim=128, window=1024,
        delta_heads=8, channel_heads=16, rank=64, rot_dims=64, base=500000.0,
    ),
    "mopilorn-3b": alternating(
        vocab=128256, width=3072, num_layers=28, ff=8192, streams=4, attn_heads=24, attn_kv_heads=8, dim=128, vdim=128, window=2048,
        delta_heads=8, channel_heads=24, rank=96, rot_dims=64, base=500000.0,
    ),
}  # fmt: skip
