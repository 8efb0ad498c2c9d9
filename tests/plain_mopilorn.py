"""A plain, slow implementation of the Mopilorn decoder: whole sequences, no cache, no batching,
one function per mechanism, written from the design's equations.  It shares no code with the
package and is what the package's kernels are compared with.

Notation: ``T`` tokens, ``W`` model width, ``H`` heads, ``G`` key heads, ``dk`` / ``dv`` the
key and value sizes of a head.  Weights are a dict name -> tensor with the checkpoint's names;
``cfg`` is the parsed ``config.json``.  Everything runs in the dtype of ``weights`` (float32 or
float64) on the CPU.
"""

from __future__ import annotations

import math

import torch
import torch.nn.functional as F


# ---------------------------------------------------------------- small pieces


def rms_norm(x: torch.Tensor, w: torch.Tensor | None, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis, times ``w`` when given."""
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if w is None else y * w


def short_conv(u: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """Causal convolution over time per channel: ``u [T, C]``, ``w [C, taps]``; the last column
    of ``w`` multiplies the current token, zeros stand before the first token."""
    t, c = u.shape
    taps = w.shape[1]
    padded = torch.cat([u.new_zeros(taps - 1, c), u], dim=0)
    y = u.new_zeros(t, c)
    for j in range(taps):
        y = y + padded[j : j + t] * w[:, j]
    return y


def rotary_frequencies(dims: int, base: float, scaling: dict | None) -> torch.Tensor:
    """f_i = base^(-2i/dims), i < dims/2, then the three-regime wavelength scaling."""
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=torch.float64)
    if scaling:
        factor, low, high, orig = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
        out = []
        for fi in f.tolist():
            lam = 2.0 * math.pi / fi
            if lam < orig / high:
                out.append(fi)
            elif lam > orig / low:
                out.append(fi / factor)
            else:
                s = (orig / lam - low) / (high - low)
                out.append((1.0 - s) * fi / factor + s * fi)
        f = torch.tensor(out, dtype=torch.float64)
    return f


def rotate_interleaved(x: torch.Tensor, positions: torch.Tensor, freqs: torch.Tensor) -> torch.Tensor:
    """``x [T, heads, d]``: dims (2i, 2i+1), i < len(freqs), turn by ``positions * freqs[i]``;
    the remaining dims pass."""
    rot = 2 * freqs.numel()
    ang = positions.to(torch.float64)[:, None] * freqs[None, :]
    cos, sin = ang.cos().to(x.dtype)[:, None, :], ang.sin().to(x.dtype)[:, None, :]
    a, b = x[..., 0:rot:2], x[..., 1:rot:2]
    y = x.clone()
    y[..., 0:rot:2] = a * cos - b * sin
    y[..., 1:rot:2] = b * cos + a * sin
    return y


def windowed_attention(q, k, v, scale: float, window: int | None) -> torch.Tensor:
    """``q [T, H, dk]``, ``k [T, G, dk]``, ``v [T, G, dv]`` -> ``[T, H, dv]``.  Query i sees key j
    iff ``0 <= i - j < window`` (all earlier keys without a window); head h reads key head
    ``h // (H / G)``."""
    t, h, _ = q.shape
    g = k.shape[1]
    rep = h // g
    out = q.new_zeros(t, h, v.shape[-1])
    i = torch.arange(t)
    diff = i[:, None] - i[None, :]
    visible = diff >= 0
    if window is not None:
        visible &= diff < window
    for hh in range(h):
        kh = hh // rep
        s = (q[:, hh] @ k[:, kh].T) * scale
        s = s.masked_fill(~visible, float("-inf"))
        out[:, hh] = torch.softmax(s, dim=-1) @ v[:, kh]
    return out


def delta_rule(q, k, v, beta, decay) -> torch.Tensor:
    """The gated delta rule, token by token, state ``S [dk, dv]`` per head from zero.

    ``q, k [T, H, dk]`` (already unit vectors, q scaled), ``v [T, H, dv]``, ``beta [T, H]``,
    ``decay [T, H]`` (one factor a head) or ``[T, H, dk]`` (one a key channel: it scales the
    rows of S).  Per token: ``S <- decay * S``; ``u = beta (v - S^T k)``; ``S <- S + k u^T``;
    ``o = S^T q``.
    """
    t, h, dk = q.shape
    dv = v.shape[-1]
    s = q.new_zeros(h, dk, dv)
    out = q.new_zeros(t, h, dv)
    for n in range(t):
        d = decay[n]
        s = s * (d[:, None, None] if d.dim() == 1 else d[:, :, None])
        u = beta[n][:, None] * (v[n] - torch.einsum("hkv,hk->hv", s, k[n]))
        s = s + torch.einsum("hk,hv->hkv", k[n], u)
        out[n] = torch.einsum("hkv,hk->hv", s, q[n])
    return out


def unit(x: torch.Tensor) -> torch.Tensor:
    return x / torch.sqrt((x * x).sum(-1, keepdim=True) + 1e-6)


# ---------------------------------------------------------------- mixers


def attention_branch(h, w, p: str, m: dict) -> torch.Tensor:
    """Projections, short convolution, rotation, windowed softmax attention, output product."""
    t = h.shape[0]
    heads, kvh, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = short_conv(h @ w[p + "q"].T, w[p + "q.conv"]).view(t, heads, dk)
    k = short_conv(h @ w[p + "k"].T, w[p + "k.conv"]).view(t, kvh, dk)
    v = short_conv(h @ w[p + "v"].T, w[p + "v.conv"]).view(t, kvh, dv)
    rot = m.get("rot")
    if rot:
        f = rotary_frequencies(int(rot["dims"]), float(rot["base"]), rot.get("scaling"))
        pos = torch.arange(t)
        q, k = rotate_interleaved(q, pos, f), rotate_interleaved(k, pos, f)
    window = m["mask"]["size"] if m.get("mask") else None
    o = windowed_attention(q, k, v, float(m["scale"]), window)
    return o.reshape(t, heads * dv) @ w[p + "o"].T


def delta_inputs(h, w, p: str, m: dict):
    """q, k, v of a delta-rule mixer after projection, convolution, silu and unit norms."""
    t = h.shape[0]
    heads, kvh, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = F.silu(short_conv(h @ w[p + "q"].T, w[p + "q.conv"])).view(t, kvh, dk)
    k = F.silu(short_conv(h @ w[p + "k"].T, w[p + "k.conv"])).view(t, kvh, dk)
    v = F.silu(short_conv(h @ w[p + "v"].T, w[p + "v.conv"])).view(t, heads, dv)
    q = unit(q) * dk**-0.5
    k = unit(k)
    rep = heads // kvh
    q = q.repeat_interleave(rep, dim=1)
    k = k.repeat_interleave(rep, dim=1)
    return q, k, v


def head_delta_branch(h, w, p: str, m: dict, eps: float) -> torch.Tensor:
    """Delta rule with one decay a head and a silu gate on the normed read-out."""
    t = h.shape[0]
    heads, dv = m["heads"], m["vdim"]
    q, k, v = delta_inputs(h, w, p, m)
    beta = torch.sigmoid(h @ w[p + "b"].T)
    decay = torch.exp(-torch.exp(w[p + "A_log"]) * F.softplus(h @ w[p + "a"].T + w[p + "dt_bias"]))
    o = delta_rule(q, k, v, beta, decay)
    gate = F.silu(h @ w[p + "g"].T).view(t, heads, dv)
    o = rms_norm(o, w[p + "norm"], eps) * gate
    return o.reshape(t, heads * dv) @ w[p + "o"].T


def channel_delta_mixer(h, w, p: str, m: dict, eps: float) -> torch.Tensor:
    """Delta rule with one decay a head and key channel (low-rank projection) and a sigmoid gate."""
    t = h.shape[0]
    heads, dk, dv = m["heads"], m["dim"], m["vdim"]
    q, k, v = delta_inputs(h, w, p, m)
    beta = torch.sigmoid(h @ w[p + "b"].T)
    a = ((h @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "dt_bias"]).view(t, heads, dk)
    decay = torch.exp(-torch.exp(w[p + "A_log"])[None, :, None] * F.softplus(a))
    o = delta_rule(q, k, v, beta, decay)
    gate = torch.sigmoid((h @ w[p + "g1"].T) @ w[p + "g2"].T).view(t, heads, dv)
    o = rms_norm(o, w[p + "norm"], eps) * gate
    return o.reshape(t, heads * dv) @ w[p + "o"].T


def parallel_mixer(h, w, p: str, m: dict, eps: float) -> torch.Tensor:
    """Attention and head-decay delta rule side by side on the same input; each result is
    normed over the width with its own weight, and the two are averaged."""
    left = attention_branch(h, w, p + "left.", m["left"])
    right = head_delta_branch(h, w, p + "right.", m["right"], eps)
    return 0.5 * (rms_norm(left, w[p + "left.out"], eps) + rms_norm(right, w[p + "right.out"], eps))


def mixer(kind: str, h, w, p: str, m: dict, eps: float) -> torch.Tensor:
    if kind == "parallel":
        return parallel_mixer(h, w, p, m, eps)
    if kind == "channel_delta":
        return channel_delta_mixer(h, w, p, m, eps)
    raise ValueError(f"unknown mixer {kind!r}")


def dense_ff(h, w, p: str) -> torch.Tensor:
    return (F.silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


# ---------------------------------------------------------------- layers and model


def hyper_sublayer(streams: torch.Tensor, fn, norm_w, eps: float, w_in, w_mix, w_out) -> torch.Tensor:
    """``streams [S, T, W]``: read ``u = sum_s in[s] x_s``, run ``y = fn(norm(u))``, write
    ``x_t <- sum_s mix[s, t] x_s + out[t] y`` for all t from the old streams."""
    u = torch.einsum("s,stw->tw", w_in, streams)
    y = fn(rms_norm(u, norm_w, eps))
    return torch.einsum("sr,stw->rtw", w_mix, streams) + w_out[:, None, None] * y[None]


def output(cfg: dict, w: dict, x: torch.Tensor, eps: float) -> torch.Tensor:
    logits = rms_norm(x, w["final.norm"], eps) @ w["head"].T
    cap = cfg.get("logit_softcap")
    if cap:
        logits = float(cap) * torch.tanh(logits / float(cap))
    return logits


def _forward_single_stream(cfg, w, x, eps, return_layers):
    """Without streams: x <- x + mixer(norm1(x)); x <- x + ff(norm2(x))."""
    per_layer = []
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        x = x + mixer(layer["type"], rms_norm(x, w[p + "norm1"], eps), w, p + "mix.", layer["mixer"], eps)
        if layer.get("mlp"):
            x = x + dense_ff(rms_norm(x, w[p + "norm2"], eps), w, p + "mlp.")
        per_layer.append(x)
    logits = output(cfg, w, x, eps)
    return (logits, torch.stack(per_layer)) if return_layers else logits


def forward(cfg: dict, w: dict, tokens, return_layers: bool = False):
    """Logits ``[T, vocab]`` of one whole sequence (and, on request, the sum of the streams
    after every layer, ``[layers, T, W]``)."""
    eps = float(cfg["norm"]["eps"])
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    if cfg.get("streams") is None:
        return _forward_single_stream(cfg, w, x, eps, return_layers)
    n_streams = int(cfg["streams"])
    streams = x[None].repeat(n_streams, 1, 1)
    per_layer = []
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        streams = hyper_sublayer(
            streams, lambda z: mixer(layer["type"], z, w, p + "mix.", layer["mixer"], eps),
            w[p + "norm1"], eps, w[p + "hc1.in"], w[p + "hc1.mix"], w[p + "hc1.out"],
        )  # fmt: skip
        if layer.get("mlp"):
            if layer["mlp"]["kind"] != "dense":
                raise ValueError("only dense feed-forwards exist")
            streams = hyper_sublayer(
                streams, lambda z: dense_ff(z, w, p + "mlp."),
                w[p + "norm2"], eps, w[p + "hc2.in"], w[p + "hc2.mix"], w[p + "hc2.out"],
            )  # fmt: skip
        per_layer.append(streams.sum(0))
    logits = output(cfg, w, streams.sum(0), eps)
    if return_layers:
        return logits, torch.stack(per_layer)
    return logits
