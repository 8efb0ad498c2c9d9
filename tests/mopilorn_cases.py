"""Small Mopilorn configurations for the tests, model folders with random weights made here (not by
the package's random-weights mode), and the plain implementation's logits for them.

The configurations differ from one another in every size and option: streams (none, 1, 2, 3),
heads and groups, key and value sizes (equal and not), taps, windows (and none), rotated dims (part
of a head, a whole head, none), frequency scaling, low-rank inner sizes (a multiple of 8 and not),
layers without a feed-forward, the order of layers, the soft cap.
"""

from __future__ import annotations

import json
from pathlib import Path

import torch

import plain_mopilorn as plain


def attention(heads, kv_heads, dim, vdim, conv, window, rot=None, scale=None):
    out = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv, "scale": scale if scale is not None else dim**-0.5}
    if window is not None:
        out["mask"] = {"size": window}
    if rot is not None:
        out["rot"] = rot
    return out


def delta(heads, kv_heads, dim, vdim, conv):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}


def layer(kind, mixer, ff):
    return {"type": kind, "mixer": mixer, "mlp": {"kind": "dense", "ff": ff} if ff else None}


SCALED = {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64}

CASES: dict[str, dict] = {
    # parallel first; key size != value size; a window shorter than a page; part of a head turns, with scaling
    "a": {
        "config": {
            "architecture": "Mopilorn", "vocab": 131, "width": 64, "streams": 3, "norm": {"eps": 1e-5}, "logit_softcap": 20.0,
            "layers": [
                layer("parallel", {"left": attention(4, 2, 16, 24, 3, 11, {"dims": 8, "base": 1000.0, "scaling": SCALED}), "right": delta(2, 1, 16, 8, 4)}, 96),
                layer("channel_delta", delta(4, 2, 24, 16, 2), 80),
                layer("parallel", {"left": attention(4, 2, 16, 24, 3, 11, {"dims": 8, "base": 1000.0, "scaling": SCALED}), "right": delta(2, 1, 16, 8, 4)}, None),
            ],
        },
        "ranks": (5, 8),
        "block_size": 16,
    },
    # channel_delta first; two layers of a kind in a row; as many key heads as heads; windows of two lengths
    # (two cache groups), one longer than several pages; a whole head turns, no scaling; no soft cap; two streams
    "b": {
        "config": {
            "architecture": "Mopilorn", "vocab": 97, "width": 48, "streams": 2, "norm": {"eps": 1e-6},
            "layers": [
                layer("channel_delta", delta(2, 2, 8, 40, 3), 64),
                layer("channel_delta", delta(3, 1, 16, 16, 4), 64),
                layer("parallel", {"left": attention(3, 3, 24, 8, 2, 37, {"dims": 24, "base": 10000.0}), "right": delta(3, 3, 8, 8, 2)}, 72),
                layer("parallel", {"left": attention(2, 1, 32, 32, 4, 5, {"dims": 16, "base": 10000.0}), "right": delta(1, 1, 32, 24, 3)}, 72),
            ],
        },
        "ranks": (8, 3),
        "block_size": 8,
    },
    # no streams at all (the plain residual sum), no window (every key), no rotation, one tap
    "c": {
        "config": {
            "architecture": "Mopilorn", "vocab": 150, "width": 40, "norm": {"eps": 1e-6}, "logit_softcap": 50.0,
            "layers": [
                layer("parallel", {"left": attention(2, 2, 16, 16, 1, None), "right": delta(2, 2, 16, 16, 1)}, 56),
                layer("channel_delta", delta(2, 1, 16, 8, 4), 56),
            ],
        },
        "ranks": (4, 4),
        "block_size": 4,
    },
    # one stream with its own in / mix / out; key and value heads of 64 with four heads a key head and pages
    # of 16: in bfloat16 the tensor-core attention kernels take this shape
    "d": {
        "config": {
            "architecture": "Mopilorn", "vocab": 211, "width": 96, "streams": 1, "norm": {"eps": 1e-6}, "logit_softcap": 30.0,
            "layers": [
                layer("parallel", {"left": attention(8, 2, 64, 64, 4, 48, {"dims": 32, "base": 50000.0}), "right": delta(2, 2, 64, 32, 4)}, 128),
                layer("channel_delta", delta(2, 2, 64, 64, 4), 128),
                layer("parallel", {"left": attention(8, 2, 64, 64, 4, None, {"dims": 64, "base": 50000.0}), "right": delta(2, 2, 64, 32, 4)}, 128),
            ],
        },
        "ranks": (16, 16),
        "block_size": 16,
    },
}  # fmt: skip


def tensor_shapes(config: dict, ranks: tuple[int, int]) -> dict[str, tuple[int, ...]]:
    """Checkpoint name -> shape, from the design's naming alone."""
    w, s = config["width"], config.get("streams")
    out = {"embed": (config["vocab"], w), "head": (config["vocab"], w), "final.norm": (w,)}

    def delta_tensors(p, m, channel):
        h, g, dk, dv, taps = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
        out.update({p + "q": (g * dk, w), p + "k": (g * dk, w), p + "v": (h * dv, w), p + "q.conv": (g * dk, taps), p + "k.conv": (g * dk, taps),
                    p + "v.conv": (h * dv, taps), p + "b": (h, w), p + "A_log": (h,), p + "norm": (dv,), p + "o": (w, h * dv)})  # fmt: skip
        if channel:
            out.update({p + "a1": (ranks[0], w), p + "a2": (h * dk, ranks[0]), p + "dt_bias": (h * dk,), p + "g1": (ranks[1], w), p + "g2": (h * dv, ranks[1])})
        else:
            out.update({p + "a": (h, w), p + "dt_bias": (h,), p + "g": (h * dv, w)})

    for i, ly in enumerate(config["layers"]):
        p = f"l{i}."
        out[p + "norm1"] = (w,)
        m = ly["mixer"]
        if ly["type"] == "parallel":
            a = m["left"]
            h, g, dk, dv, taps = a["heads"], a["kv_heads"], a["dim"], a["vdim"], a["conv"]
            q = p + "mix.left."
            out.update({q + "q": (h * dk, w), q + "k": (g * dk, w), q + "v": (g * dv, w), q + "q.conv": (h * dk, taps), q + "k.conv": (g * dk, taps),
                        q + "v.conv": (g * dv, taps), q + "o": (w, h * dv), p + "mix.left.out": (w,), p + "mix.right.out": (w,)})  # fmt: skip
            delta_tensors(p + "mix.right.", m["right"], False)
        else:
            delta_tensors(p + "mix.", m, True)
        subs = ["hc1"]
        if ly["mlp"]:
            out.update({p + "norm2": (w,), p + "mlp.gate": (ly["mlp"]["ff"], w), p + "mlp.up": (ly["mlp"]["ff"], w), p + "mlp.down": (w, ly["mlp"]["ff"])})
            subs.append("hc2")
        if s is not None:
            for hc in subs:
                out.update({p + hc + ".in": (s,), p + hc + ".out": (s,), p + hc + ".mix": (s, s)})
    return out


def random_tensors(config: dict, ranks: tuple[int, int], seed: int) -> dict[str, torch.Tensor]:
    """Weights of order one where it matters, rounded to bfloat16 (what the files hold), as float32."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(config, ranks).items():
        leaf = name.rsplit(".", 1)[-1]
        r = torch.randn(shape, generator=g)
        if name == "embed":
            t = r
        elif leaf in ("norm", "norm1", "norm2") or name.endswith((".left.out", ".right.out")):
            t = 1.0 + 0.2 * r
        elif leaf == "conv":
            t = 0.6 * r
        elif leaf in ("A_log", "dt_bias"):
            t = 0.7 * r
        elif ".hc" in name and leaf == "in":
            t = 1.0 / shape[0] + 0.2 * r
        elif ".hc" in name and leaf == "out":
            t = 1.0 + 0.2 * r
        elif ".hc" in name and leaf == "mix":
            t = torch.eye(shape[0]) + 0.15 * r
        else:
            t = r * (1.5 if leaf in ("q", "k", "b", "a", "a2") else 1.0) / shape[-1] ** 0.5
        out[name] = t.to(torch.bfloat16).to(torch.float32)
    return out


def write_folder(path: Path, config: dict, tensors: dict[str, torch.Tensor]) -> Path:
    """``config.json`` and ``model.safetensors`` (bfloat16), written with the standard layout of the format:
    eight bytes of header length, the JSON header, the data."""
    import struct

    path.mkdir(parents=True, exist_ok=True)
    (path / "config.json").write_text(json.dumps(config))
    header, blobs, at = {}, [], 0
    for name, t in tensors.items():
        raw = t.to(torch.bfloat16).contiguous().view(torch.int16).numpy().tobytes()
        header[name] = {"dtype": "BF16", "shape": list(t.shape), "data_offsets": [at, at + len(raw)]}
        blobs.append(raw)
        at += len(raw)
    hj = json.dumps(header).encode()
    hj += b" " * (-len(hj) % 8)
    with open(path / "model.safetensors", "wb") as f:
        f.write(struct.pack("<Q", len(hj)) + hj + b"".join(blobs))
    return path


def plain_logits(config: dict, tensors: dict[str, torch.Tensor], tokens: list[int]) -> torch.Tensor:
    w = {k: v.double() for k, v in tensors.items()}
    return plain.forward(config, w, tokens)


def row_error(got: torch.Tensor, want: torch.Tensor, scale: float) -> float:
    """Root mean square over the vocabulary of the difference (its mean taken off: a shift of all logits
    changes no probability), relative to ``scale`` (the root mean square of the reference logits)."""
    d = got.double() - want.double()
    d = d - d.mean()
    return float(d.pow(2).mean().sqrt()) / scale
