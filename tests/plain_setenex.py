"""A plain, slow implementation of the Setenex decoder: whole sequences, no cache, no batching,
one function per mechanism, written from the design's equations.  It shares no code with the
package and is what the package's kernels are compared with.

Notation: ``T`` tokens, ``W`` model width, ``H`` heads, ``G`` key heads, ``dk`` / ``dv`` the key
and value sizes of a head.  Weights are a dict name -> tensor with the checkpoint's names; ``cfg``
is the parsed ``config.json``.  Everything runs in the dtype of the weights (float32 or float64)
on the CPU.
"""

from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import torch


# ---------------------------------------------------------------- reading a folder


def read_folder(folder, dtype=torch.float64):
    """(config dict, weights dict) of a model folder; floats widened to ``dtype``."""
    folder = Path(folder)
    cfg = json.loads((folder / "config.json").read_text())
    raw = (folder / "model.safetensors").read_bytes()
    (n,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8 : 8 + n])
    kinds = {"BF16": torch.bfloat16, "F32": torch.float32, "F16": torch.float16, "I32": torch.int32, "F64": torch.float64}
    weights = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        a, b = info["data_offsets"]
        t = torch.frombuffer(bytearray(raw[8 + n + a : 8 + n + b]), dtype=kinds[info["dtype"]]).reshape(info["shape"])
        weights[name] = t.to(dtype) if t.is_floating_point() else t
    return cfg, weights


# ---------------------------------------------------------------- small pieces


def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def norm_one_plus(x, w, eps):
    """The layers' and the model's norm: the tensor holds the weight's offset from one."""
    return rms(x, eps) * (1.0 + w)


def norm_plain(x, w, eps):
    return rms(x, eps) * w


def gelu_erf(z):
    return 0.5 * z * (1.0 + torch.erf(z / math.sqrt(2.0)))


def distance_bucket(n: int, rows: int, far: int) -> int:
    """Row of the distance-bias table for distance ``n >= 0``: one row per distance below half the
    table, logarithmic steps from there to ``far``, the last row beyond."""
    half = rows // 2
    if n < half:
        return n
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))


def rotate_pairs(x, positions, dims: int, base: float):
    """``x [T, ..., d]``: dims (2i, 2i+1), i < dims/2, turn by ``p * base^(-2i/dims)``; the other dims are left as they are."""
    freqs = torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=torch.float64)
    ang = positions.to(torch.float64)[:, None] * freqs[None, :]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [dims // 2]
    cos, sin = ang.cos().to(x.dtype).reshape(shape), ang.sin().to(x.dtype).reshape(shape)
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    y = x.clone()
    y[..., 0:dims:2] = u * cos - v * sin
    y[..., 1:dims:2] = v * cos + u * sin
    return y


def softmax_rows(scores, visible):
    scores = scores.masked_fill(~visible, float("-inf"))
    return torch.softmax(scores, dim=-1)


# ---------------------------------------------------------------- mixers


def biased_attention(h, w, p: str, m: dict, eps: float):
    """Grouped-query attention without rotation: per-head RMS norm of queries and keys, a learned
    bias by distance bucket, a window that also keeps the first tokens."""
    t = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T).reshape(t, H, dk)
    k = (h @ w[p + "k"].T).reshape(t, G, dk)
    v = (h @ w[p + "v"].T).reshape(t, G, dv)
    q = norm_plain(q, w[p + "q.norm"], eps)
    k = norm_plain(k, w[p + "k.norm"], eps)
    rel = w[p + "rel"]
    rows = rel.shape[0]
    i = torch.arange(t)[:, None]
    j = torch.arange(t)[None, :]
    visible = j <= i
    mask = m.get("mask")
    if mask:
        visible = visible & ((i - j < mask["size"]) | (j < mask.get("keep_first", 0)))
    buckets = torch.tensor([distance_bucket(n, rows, m["bias_max"]) for n in range(t)])
    bias = rel[buckets[(i - j).clamp(min=0)]]  # [T, T, H]
    out = h.new_zeros(t, H, dv)
    for head in range(H):
        g = head // (H // G)
        s = (q[:, head] @ k[:, g].T) * m["scale"] + bias[:, :, head]
        out[:, head] = softmax_rows(s, visible) @ v[:, g]
    return out.reshape(t, H * dv) @ w[p + "o"].T


def latent_attention(h, w, p: str, m: dict, eps: float):
    """Attention whose keys and values are made from one small latent per token, with a rotated key
    part shared by all heads, a window, and a logistic gate per head on the output."""
    t = h.shape[0]
    H, dk, dr, dv, r = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(t)
    q = (h @ w[p + "q"].T).reshape(t, H, dk + dr)
    q_plain, q_rot = q[..., :dk], q[..., dk:]
    down = h @ w[p + "dkv"].T
    c = norm_plain(down[:, :r], w[p + "dkv.norm"], eps)
    k_rot = down[:, r:]
    rot = m["rot"]
    q_rot = rotate_pairs(q_rot, pos, rot["dims"], rot["base"])
    k_rot = rotate_pairs(k_rot, pos, rot["dims"], rot["base"])
    k_plain = (c @ w[p + "uk"].T).reshape(t, H, dk)
    v = (c @ w[p + "uv"].T).reshape(t, H, dv)
    i = torch.arange(t)[:, None]
    j = torch.arange(t)[None, :]
    visible = j <= i
    mask = m.get("mask")
    if mask:
        visible = visible & (i - j < mask["size"])
    gate = torch.sigmoid(h @ w[p + "g"].T)  # [T, H]
    out = h.new_zeros(t, H, dv)
    for head in range(H):
        s = (q_plain[:, head] @ k_plain[:, head].T + q_rot[:, head] @ k_rot.T) * m["scale"]
        out[:, head] = (softmax_rows(s, visible) @ v[:, head]) * gate[:, head : head + 1]
    return out.reshape(t, H * dv) @ w[p + "o"].T


# ---------------------------------------------------------------- feed-forward


def route(h, w, p: str, r: dict):
    """(chosen experts ``[T, top]``, their weights ``[T, top]``)."""
    s = torch.sigmoid(h @ w[p + "router"].T)
    choice = s + w[p + "correction"]
    E, top = r["experts"], r["top"]
    groups = r.get("groups")
    if groups:
        per = E // groups["count"]
        by_group = choice.reshape(-1, groups["count"], per)
        score = by_group.topk(min(2, per), dim=-1).values.sum(-1)
        best = score.topk(groups["keep"], dim=-1).indices
        allowed = torch.zeros_like(score, dtype=torch.bool).scatter_(1, best, True)
        choice = choice.masked_fill(~allowed.repeat_interleave(per, dim=1), float("-inf"))
    chosen = choice.topk(top, dim=-1).indices
    picked = s.gather(1, chosen)
    return chosen, picked / (picked.sum(-1, keepdim=True) + 1e-20)


def mixture_of_experts(h, w, p: str, mlp: dict):
    chosen, weights = route(h, w, p, mlp["router"])
    out = torch.zeros(h.shape[0], w[p + "e0.down"].shape[0], dtype=h.dtype)
    for t in range(h.shape[0]):
        for e, g in zip(chosen[t].tolist(), weights[t]):
            out[t] += g * (gelu_erf(h[t] @ w[f"{p}e{e}.up"].T) @ w[f"{p}e{e}.down"].T)
    return out


# ---------------------------------------------------------------- the model


def layer_runs(cfg) -> list[tuple[int, int | None]]:
    """(layer, pass number if the run is the first of a pass of the loop)."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    runs = [(i, None) for i in range(loop["start"])]
    for t in range(loop["times"]):
        for i in range(loop["start"], loop["stop"]):
            runs.append((i, t if i == loop["start"] else None))
    return runs + [(i, None) for i in range(loop["stop"], n)]


def residual_after_every_run(cfg, w, tokens) -> list[torch.Tensor]:
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)] * (cfg.get("embedding") or {}).get("scale", 1.0)
    out = []
    for i, step in layer_runs(cfg):
        if step is not None:
            x = x + w["loop.step"][step]
        layer = cfg["layers"][i]
        h = norm_one_plus(x, w[f"l{i}.norm1"], eps)
        mix = {"attention": biased_attention, "latent_attention": latent_attention}[layer["type"]]
        y = mix(h, w, f"l{i}.mix.", layer["mixer"], eps)
        if layer.get("mlp") is not None:
            y = y + mixture_of_experts(h, w, f"l{i}.mlp.", layer["mlp"])
        x = x + y
        out.append(x)
    return out


def logits(cfg, w, tokens) -> torch.Tensor:
    x = residual_after_every_run(cfg, w, tokens)[-1]
    return norm_one_plus(x, w["final.norm"], cfg["norm"]["eps"]) @ w["head"].T


def greedy(cfg, w, prompt, n_new: int) -> list[int]:
    ids = list(prompt)
    for _ in range(n_new):
        ids.append(int(logits(cfg, w, ids)[-1].argmax()))
    return ids[len(prompt) :]
