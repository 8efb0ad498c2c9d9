"""Typed configuration of the Setenex decoder, read from its ``config.json``.

The file gives every size and every constant that differs between models of the design::

    {"architecture": "Setenex", "vocab": V, "width": W, "norm": {"eps": e}, "embedding": {"scale": s},
     "loop": {"start": a, "stop": b, "times": t} | absent,
     "layers": [{"type": "attention" | "latent_attention", "mixer": {...}, "mlp": {...} | null}, ...]}

An ``attention`` mixer: ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``, ``bias_max`` (the farthest
distance its bias table tells apart; the table's rows are read from the tensor ``rel``) and
``mask.{size, keep_first}``.  A ``latent_attention`` mixer: ``heads``, ``dim``, ``rot_dim``, ``vdim``,
``kv_rank``, ``scale``, ``rot.{dims, base}``, ``mask.size``.  A feed-forward: ``kind`` ``"moe"``,
``expert.ff``, ``router.{experts, top, groups.{count, keep}}``.  Nothing here has a default that stands
for a size.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

from .model_config import ConfigError

ARCHITECTURE = "Setenex"


def _need(d, key: str, where: str):
    if not isinstance(d, dict) or key not in d:
        raise ConfigError(f"config.json lacks {where}{key}")
    return d[key]


@dataclass(frozen=True)
class BiasedAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    bias_rows: int  # rows of the distance-bias table (the shape of the tensor ``rel``)
    bias_max: int
    window: int | None
    keep_first: int

    @classmethod
    def from_dict(cls, d: dict, where: str, bias_rows: int | None) -> BiasedAttentionConfig:
        mask = d.get("mask")
        rows = bias_rows if bias_rows is not None else d.get("bias_rows")
        if rows is None:
            raise ConfigError(f"{where}: the rows of the bias table are neither in the tensors nor in the file")
        out = cls(
            heads=int(_need(d, "heads", where)), kv_heads=int(_need(d, "kv_heads", where)), dim=int(_need(d, "dim", where)),
            vdim=int(_need(d, "vdim", where)), scale=float(_need(d, "scale", where)), bias_rows=int(rows),
            bias_max=int(_need(d, "bias_max", where)), window=int(_need(mask, "size", where + "mask.")) if mask else None,
            keep_first=int(mask.get("keep_first", 0)) if mask else 0,
        )  # fmt: skip
        if out.kv_heads <= 0 or out.heads % out.kv_heads:
            raise ConfigError(f"{where}heads must be a multiple of kv_heads")
        if out.window is not None and out.window <= 0:
            raise ConfigError(f"{where}mask.size must be positive")
        if out.bias_rows < 2 or out.bias_max <= out.bias_rows // 2:
            raise ConfigError(f"{where}bias_max must lie beyond half the rows of the bias table (at least two rows)")
        return out


@dataclass(frozen=True)
class LatentAttentionConfig:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    scale: float
    rot_dims: int
    rot_base: float
    window: int | None

    @classmethod
    def from_dict(cls, d: dict, where: str) -> LatentAttentionConfig:
        mask, rot = d.get("mask"), _need(d, "rot", where)
        out = cls(
            heads=int(_need(d, "heads", where)), dim=int(_need(d, "dim", where)), rot_dim=int(_need(d, "rot_dim", where)),
            vdim=int(_need(d, "vdim", where)), kv_rank=int(_need(d, "kv_rank", where)), scale=float(_need(d, "scale", where)),
            rot_dims=int(_need(rot, "dims", where + "rot.")), rot_base=float(_need(rot, "base", where + "rot.")),
            window=int(_need(mask, "size", where + "mask.")) if mask else None,
        )  # fmt: skip
        if out.rot_dims % 2 or not 0 < out.rot_dims <= out.rot_dim:
            raise ConfigError(f"{where}rot.dims must be even and at most rot_dim")
        if out.window is not None and out.window <= 0:
            raise ConfigError(f"{where}mask.size must be positive")
        return out


@dataclass(frozen=True)
class ExpertsConfig:
    experts: int
    top: int
    ff: int
    groups: int
    keep: int

    @classmethod
    def from_dict(cls, d: dict, where: str) -> ExpertsConfig:
        if _need(d, "kind", where) != "moe":
            raise ConfigError(f"{where}kind {d['kind']!r} is not supported (only 'moe')")
        r = _need(d, "router", where)
        g = r.get("groups") or {}
        groups = int(g.get("count", 1))
        out = cls(
            experts=int(_need(r, "experts", where + "router.")), top=int(_need(r, "top", where + "router.")),
            ff=int(_need(_need(d, "expert", where), "ff", where + "expert.")), groups=groups, keep=int(g.get("keep", groups)),
        )  # fmt: skip
        if out.experts % out.groups or not 0 < out.keep <= out.groups or not 0 < out.top <= out.keep * (out.experts // out.groups):
            raise ConfigError(f"{where}router: experts must divide into the groups, and the groups that stay must hold 'top' experts")
        return out


@dataclass(frozen=True)
class LayerConfig:
    type: str  # "attention" or "latent_attention"
    mixer: BiasedAttentionConfig | LatentAttentionConfig
    mlp: ExpertsConfig | None


@dataclass(frozen=True)
class LoopConfig:
    start: int
    stop: int
    times: int


@dataclass
class SetenexConfig:
    vocab_size: int
    hidden_size: int
    eps: float
    embedding_scale: float
    layers: list[LayerConfig]
    loop: LoopConfig | None = None
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
    def from_dict(cls, d: dict[str, Any], tensor_shapes: dict[str, tuple[int, ...]] | None = None) -> SetenexConfig:
        """``tensor_shapes`` (checkpoint name -> shape), when given, supplies the rows of the distance-bias
        tables, which the file does not name."""
        layers = []
        for i, ld in enumerate(_need(d, "layers", "")):
            where = f"layers[{i}]."
            kind, m = _need(ld, "type", where), _need(ld, "mixer", where)
            if kind == "attention":
                shape = (tensor_shapes or {}).get(f"l{i}.mix.rel")
                mixer = BiasedAttentionConfig.from_dict(m, where + "mixer.", int(shape[0]) if shape else None)
            elif kind == "latent_attention":
                mixer = LatentAttentionConfig.from_dict(m, where + "mixer.")
            else:
                raise ConfigError(f"{where}type {kind!r} is not a mixer of this design ('attention', 'latent_attention')")
            mlp = ld.get("mlp")
            layers.append(LayerConfig(kind, mixer, ExpertsConfig.from_dict(mlp, where + "mlp.") if mlp is not None else None))
        loop = d.get("loop")
        if loop:
            loop = LoopConfig(int(_need(loop, "start", "loop.")), int(_need(loop, "stop", "loop.")), int(_need(loop, "times", "loop.")))
            if not 0 <= loop.start < loop.stop <= len(layers) or loop.times < 1:
                raise ConfigError("loop: start < stop within the layers and at least one pass are needed")
        emb = d.get("embedding") or {}
        return cls(
            vocab_size=int(_need(d, "vocab", "")), hidden_size=int(_need(d, "width", "")),
            eps=float(_need(_need(d, "norm", ""), "eps", "norm.")), embedding_scale=float(emb.get("scale", 1.0)),
            layers=layers, loop=loop or None, raw=dict(d),
        )  # fmt: skip

    def to_hf_dict(self) -> dict[str, Any]:
        """The ``config.json`` of this configuration (the rows of the bias tables are written too; a reader that
        takes them from the tensors ignores them)."""
        layers = []
        for lc in self.layers:
            m = lc.mixer
            if lc.type == "attention":
                mixer = {"heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "scale": m.scale, "bias_max": m.bias_max, "bias_rows": m.bias_rows}
                if m.window is not None:
                    mixer["mask"] = {"size": m.window, "keep_first": m.keep_first}
            else:
                mixer = {
                    "heads": m.heads, "dim": m.dim, "rot_dim": m.rot_dim, "vdim": m.vdim, "kv_rank": m.kv_rank, "scale": m.scale,
                    "rot": {"dims": m.rot_dims, "base": m.rot_base},
                }  # fmt: skip
                if m.window is not None:
                    mixer["mask"] = {"size": m.window}
            mlp = None
            if lc.mlp is not None:
                e = lc.mlp
                mlp = {"kind": "moe", "expert": {"ff": e.ff}, "router": {"experts": e.experts, "top": e.top, "groups": {"count": e.groups, "keep": e.keep}}}
            layers.append({"type": lc.type, "mixer": mixer, "mlp": mlp})
        out = {
            "architecture": ARCHITECTURE, "vocab": self.vocab_size, "width": self.hidden_size, "norm": {"eps": self.eps},
            "embedding": {"scale": self.embedding_scale}, "layers": layers,
        }  # fmt: skip
        if self.loop is not None:
            out["loop"] = {"start": self.loop.start, "stop": self.loop.stop, "times": self.loop.times}
        return out


def interleaved(
    *, vocab: int, width: int, num_layers: int, latent_every: int, heads: int, kv_heads: int, dim: int, window: int, keep_first: int,
    bias_rows: int, bias_max: int, latent_heads: int, latent_dim: int, rot_dim: int, kv_rank: int, latent_window: int, experts: int, top: int,
    ff: int, groups: int, keep: int, loop: LoopConfig | None = None, eps: float = 1e-5, base: float = 10000.0,
) -> SetenexConfig:  # fmt: skip
    """A configuration whose every ``latent_every``-th layer is latent attention and whose other layers are
    attention with a distance bias, all with the same feed-forward: what the named shapes below are made with."""
    attn = BiasedAttentionConfig(heads, kv_heads, dim, dim, dim**-0.5, bias_rows, bias_max, window, keep_first)
    latent = LatentAttentionConfig(latent_heads, latent_dim, rot_dim, latent_dim, kv_rank, (latent_dim + rot_dim) ** -0.5, rot_dim, base, latent_window)
    mlp = ExpertsConfig(experts, top, ff, groups, keep)
    layers = [
        LayerConfig("latent_attention", latent, mlp) if (i + 1) % latent_every == 0 else LayerConfig("attention", attn, mlp)
        for i in range(num_layers)
    ]
    return SetenexConfig(vocab, width, eps, float(width) ** 0.5, layers, loop)


# Named shapes with random weights: a small one for demonstrations, and one with the width, depth and vocabulary
# of the 1B Llama shape this engine is measured on (its experts' inner sizes add up to that shape's feed-forward
# per token: 4 of 32 experts of 2,048).
SETENEX_PRESETS: dict[str, SetenexConfig] = {
    "setenex-tiny": interleaved(
        vocab=256, width=96, num_layers=3, latent_every=2, heads=4, kv_heads=2, dim=32, window=24, keep_first=4, bias_rows=12, bias_max=40,
        latent_heads=3, latent_dim=16, rot_dim=8, kv_rank=24, latent_window=20, experts=8, top=2, ff=48, groups=4, keep=2,
        loop=LoopConfig(0, 2, 2),
    ),
    "setenex-1b": interleaved(
        vocab=128256, width=2048, num_layers=16, latent_every=4, heads=32, kv_heads=8, dim=64, window=1024, keep_first=64, bias_rows=64,
        bias_max=4096, latent_heads=16, latent_dim=128, rot_dim=64, kv_rank=512, latent_window=2048, experts=32, top=4, ff=2048, groups=8,
        keep=4, base=500000.0,
    ),
}  # fmt: skip
