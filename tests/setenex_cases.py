"""Small Setenex configurations for the tests, model folders with random weights made here (not by
the package's random-weights mode), and the plain implementation's logits for them.

The configurations differ from one another in every size and option: the order of the layers, heads
and groups (as many key heads as heads, a single key head), key and value sizes (equal and not),
windows (none, shorter than a page, longer than several), kept first tokens (none, fewer and more than
the window), bias tables with an even and an odd number of rows, latent sizes, experts (one a token,
several; groups of one, of several, all groups kept), layers without a feed-forward, a loop from the
first layer, in the middle, to the last layer, and none.
"""

from __future__ import annotations

import random

import torch

import plain_setenex as plain
from mopilorn_cases import row_error, write_folder  # noqa: F401  (the folder writer and the error measure are the same)


def attention(heads, kv_heads, dim, vdim, rows, far, window=None, keep_first=0, scale=None):
    out = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "bias_max": far, "bias_rows": rows, "scale": scale if scale is not None else dim**-0.5}
    if window is not None:
        out["mask"] = {"size": window, "keep_first": keep_first}
    return out


def latent(heads, dim, rot_dim, vdim, rank, window=None, base=10000.0, scale=None):
    out = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank, "rot": {"dims": rot_dim, "base": base},
           "scale": scale if scale is not None else (dim + rot_dim) ** -0.5}  # fmt: skip
    if window is not None:
        out["mask"] = {"size": window}
    return out


def moe(experts, top, ff, groups=None, keep=None):
    router = {"experts": experts, "top": top}
    if groups:
        router["groups"] = {"count": groups, "keep": keep}
    return {"kind": "moe", "expert": {"ff": ff}, "router": router}


def layer(kind, mixer, mlp):
    return {"type": kind, "mixer": mixer, "mlp": mlp}


CASES: dict[str, dict] = {
    # a loop in the middle; two windows (two cache groups of attention), one shorter than a page; key size != value size
    "a": {
        "config": {
            "architecture": "Setenex", "vocab": 131, "width": 64, "norm": {"eps": 1e-5}, "embedding": {"scale": 3.0},
            "loop": {"start": 1, "stop": 3, "times": 2},
            "layers": [
                layer("attention", attention(4, 2, 16, 24, 8, 30, window=11, keep_first=3), moe(6, 2, 40, 3, 2)),
                layer("latent_attention", latent(3, 16, 8, 24, 24, window=13), moe(6, 2, 40, 3, 2)),
                layer("attention", attention(4, 2, 16, 24, 8, 30, window=29, keep_first=3), moe(6, 2, 40, 3, 2)),
                layer("attention", attention(2, 1, 24, 8, 6, 20, window=11, keep_first=3), None),
            ],
        },
        "block_size": 16,
    },
    # latent attention first, looped from the first layer; more kept tokens than the window is long; a table with an odd
    # number of rows; as many key heads as heads; one expert a token, no groups; a latent layer that sees every key
    "b": {
        "config": {
            "architecture": "Setenex", "vocab": 97, "width": 48, "norm": {"eps": 1e-6},
            "loop": {"start": 0, "stop": 1, "times": 3},
            "layers": [
                layer("latent_attention", latent(2, 8, 16, 8, 40, window=37, base=500.0), moe(4, 1, 32)),
                layer("attention", attention(3, 3, 24, 8, 5, 17, window=5, keep_first=7), moe(4, 1, 32)),
                layer("latent_attention", latent(4, 16, 8, 16, 16), None),
            ],
        },
        "block_size": 8,
    },
    # no loop; attention that sees every key (no mask) with a single key head; a window without kept tokens; three
    # experts a token out of groups that all stay; pages of four tokens
    "c": {
        "config": {
            "architecture": "Setenex", "vocab": 150, "width": 40, "norm": {"eps": 1e-6}, "embedding": {"scale": 0.5},
            "layers": [
                layer("attention", attention(4, 1, 16, 16, 10, 64), moe(8, 3, 24, 4, 4)),
                layer("attention", attention(2, 2, 8, 16, 4, 9, window=6, keep_first=0), moe(8, 3, 24, 2, 1)),
            ],
        },
        "block_size": 4,
    },
    # the loop runs to the last layer; heads of 64 with four heads a key head; a latent wider than a head; many experts
    "d": {
        "config": {
            "architecture": "Setenex", "vocab": 211, "width": 96, "norm": {"eps": 1e-5}, "embedding": {"scale": 9.0},
            "loop": {"start": 1, "stop": 3, "times": 2},
            "layers": [
                layer("attention", attention(8, 2, 64, 64, 16, 100, window=48, keep_first=4), moe(16, 4, 64, 4, 2)),
                layer("latent_attention", latent(4, 32, 32, 48, 64, window=40), moe(16, 4, 64, 4, 2)),
                layer("attention", attention(8, 2, 64, 64, 16, 100, window=48, keep_first=4), moe(16, 4, 64, 8, 3)),
            ],
        },
        "block_size": 16,
    },
}  # fmt: skip


def tensor_shapes(config: dict) -> dict[str, tuple[int, ...]]:
    """Checkpoint name -> shape, from the design's naming alone."""
    w = config["width"]
    out = {"embed": (config["vocab"], w), "head": (config["vocab"], w), "final.norm": (w,)}
    if config.get("loop"):
        out["loop.step"] = (config["loop"]["times"], w)
    for i, ly in enumerate(config["layers"]):
        p, m = f"l{i}.", ly["mixer"]
        out[p + "norm1"] = (w,)
        q = p + "mix."
        if ly["type"] == "attention":
            h, g, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            out.update({q + "q": (h * dk, w), q + "k": (g * dk, w), q + "v": (g * dv, w), q + "q.norm": (dk,), q + "k.norm": (dk,),
                        q + "rel": (m["bias_rows"], h), q + "o": (w, h * dv)})  # fmt: skip
        else:
            h, dk, dr, dv, r = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
            out.update({q + "q": (h * (dk + dr), w), q + "dkv": (r + dr, w), q + "dkv.norm": (r,), q + "uk": (h * dk, r), q + "uv": (h * dv, r),
                        q + "g": (h, w), q + "o": (w, h * dv)})  # fmt: skip
        if ly["mlp"]:
            e, ff = ly["mlp"]["router"]["experts"], ly["mlp"]["expert"]["ff"]
            q = p + "mlp."
            out.update({q + "router": (e, w), q + "correction": (e,)})
            for k in range(e):
                out.update({f"{q}e{k}.up": (ff, w), f"{q}e{k}.down": (w, ff)})
    return out


def random_tensors(config: dict, seed: int, fixed_choice: bool = False) -> dict[str, torch.Tensor]:
    """Weights of order one where it matters, rounded to bfloat16 (what the files hold), as float32.
    ``fixed_choice``: the corrections lie so far apart that they alone decide which experts a token uses
    (the weights of the chosen experts still follow the token): rounding cannot change the choice then."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(config).items():
        leaf = name.rsplit(".", 1)[-1]
        r = torch.randn(shape, generator=g)
        if name == "embed":
            t = r
        elif leaf in ("norm1",) or name == "final.norm":
            t = 0.2 * r  # an offset from one
        elif leaf == "norm":
            t = 1.0 + 0.2 * r
        elif leaf == "rel":
            t = 1.5 * r
        elif leaf == "step":
            t = 0.5 * r
        elif leaf == "correction":
            t = 0.7 * torch.randperm(shape[0], generator=g).float() if fixed_choice else 0.3 * r
        elif leaf == "router":
            t = r * (0.3 if fixed_choice else 1.5) / shape[-1] ** 0.5
        else:
            t = r * (1.5 if leaf in ("q", "k", "dkv", "uk") else 1.0) / shape[-1] ** 0.5
        out[name] = t.to(torch.bfloat16).to(torch.float32)
    return out


def plain_logits(config: dict, tensors: dict[str, torch.Tensor], tokens: list[int]) -> torch.Tensor:
    w = {k: v.double() for k, v in tensors.items()}
    return plain.logits(config, w, tokens)


def random_config(seed: int) -> dict:
    """A configuration drawn at random: widths that are and are not multiples of 8, one to twenty heads, one key head
    or several, key and value sizes from 8 to 128, tables of 2 to 40 rows, windows of 1 to 100 tokens or none, up to 40
    kept tokens, latents of 8 to 160 numbers, 4 to 24 experts in any grouping that divides them, layers without a
    feed-forward, a loop over any stretch (or none) with one to three passes."""
    rng = random.Random(seed)
    m8 = lambda lo, hi: 8 * rng.randint(lo, hi)  # noqa: E731
    width = rng.choice([m8(5, 24), 100, 132])
    n_layers = rng.randint(2, 5)
    experts = rng.choice([4, 6, 9, 10, 16, 24])
    divisors = [g for g in range(1, experts + 1) if experts % g == 0]
    layers = []
    for _ in range(n_layers):
        if rng.random() < 0.5:
            kv = rng.choice([1, 2, 3])
            heads = kv * rng.choice([1, 2, 3, 5])
            dim = rng.choice([8, 16, 24, 40, 64, 128])
            vdim = dim if rng.random() < 0.5 else rng.choice([8, 16, 48, 72])
            rows = rng.randint(2, 40)
            far = rng.randint(rows // 2 + 1, 300)
            window = rng.choice([None, rng.randint(1, 90)])
            keep = rng.randint(0, 40) if window else 0
            kind, mixer = "attention", attention(heads, kv, dim, vdim, rows, far, window, keep, scale=rng.uniform(0.05, 0.3))
        else:
            heads, dim, rot = rng.choice([1, 2, 5, 8, 16, 20]), rng.choice([8, 16, 32]), rng.choice([8, 16, 32, 64])
            rank, vdim = rng.choice([8, 24, 32, 48, 64, 96, 128, 160]), rng.choice([8, 24, 40])
            window = rng.choice([None, rng.randint(1, 100)])
            kind, mixer = "latent_attention", latent(heads, dim, rot, vdim, rank, window, base=rng.choice([100.0, 10000.0, 1e6]), scale=rng.uniform(0.05, 0.3))
        groups = rng.choice(divisors)
        keep_groups = rng.randint(1, groups)
        top = rng.randint(1, min(keep_groups * (experts // groups), 6))
        mlp = None if rng.random() < 0.2 else moe(experts, top, m8(2, 12), groups, keep_groups)
        layers.append(layer(kind, mixer, mlp))
    config = {"architecture": "Setenex", "vocab": rng.randint(30, 300), "width": width, "norm": {"eps": rng.choice([1e-5, 1e-6])},
              "embedding": {"scale": rng.uniform(0.5, 12)}, "layers": layers}  # fmt: skip
    if rng.random() < 0.7:
        start = rng.randint(0, n_layers - 1)
        config["loop"] = {"start": start, "stop": rng.randint(start + 1, n_layers), "times": rng.randint(1, 3)}
    return config
