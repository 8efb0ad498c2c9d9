"""The gated delta rule as a mixer: a matrix state per head instead of pages of keys.

Per head a state ``S [dk, dv]`` (float, one per request, zero at its start) and per token::

    S <- g * S;   u = beta * (v - S^T k);   S <- S + k u^T;   o = S^T q

so the read-out sees the token's own write.  ``q`` and ``k`` (``kv_heads`` heads of ``dk``, shared by
``heads / kv_heads`` value heads each) and ``v`` (``heads`` heads of ``dv``) are bias-free
projections followed by a short causal convolution over time per channel and SiLU; ``q`` and ``k``
are then unit vectors per head (``x / sqrt(sum x^2 + 1e-6)``), ``q`` times ``dk^-1/2``;
``beta = sigmoid(W_b h)``; the decay is ``g = exp(-exp(A_log) * softplus(a + dt_bias))`` with ``a``
either one value a head (``decay="head"``, ``a = W_a h``) or one a head and key channel
(``decay="channel"``, ``g`` then scales the rows of ``S``), and in either case ``W_a`` may be a
product of two low-rank matrices (``decay_rank``).  The read-out of a head is divided by its root mean
square, multiplied by a weight shared by the heads and by ``act(gate)``, ``gate = W_g h`` (or
low-rank, ``gate_rank``), ``act`` SiLU or the logistic function; then the output projection.

What the recurrence reads besides the projections is float in both storage types: decay, step size,
beta, unit norms, the state.  A request's state is one row of floats: the last ``conv - 1`` inputs
of the convolution, then ``S``.
"""

from __future__ import annotations

import torch

from .. import ops
from .base import Mixer, WeightDecl, register_mixer
from .projection import project


def _pad8(n: int) -> int:
    return (n + 7) // 8 * 8


def product(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """``out = x @ w^T`` where ``x`` may be a column slice of a wider buffer and ``out`` float or the
    storage type: the decode product for a few aligned rows, else the engine's plain product."""
    if ops.skinny_ok(x, w) and x.data_ptr() % 16 == 0 and out.stride(1) == 1:
        ops.gemm_skinny(x, w, out)
    else:
        ops.linear(x, w, out)


@register_mixer("gated_delta_rule")
class GatedDeltaRule(Mixer):
    """params: ``hidden_size``, ``num_heads``, ``num_kv_heads``, ``head_dim`` (dk), ``v_head_dim``
    (dv), ``conv`` (taps), ``eps`` (of the read-out's norm); ``decay``: ``"head"`` or ``"channel"``;
    ``decay_rank`` / ``gate_rank``: ``None`` or the inner size of a low-rank projection; ``gate``:
    ``"silu"`` or ``"sigmoid"``.  Tensors: ``q``, ``k``, ``v``, ``q.conv``, ``k.conv``, ``v.conv``,
    ``b``, ``A_log``, ``dt_bias``, ``norm``, ``o`` and ``a`` (or ``a1``, ``a2``), ``g`` (or ``g1``,
    ``g2``)."""

    def __init__(self, params, prefix=""):
        super().__init__(params, prefix)
        p = params
        self.hidden = int(p["hidden_size"])
        self.H, self.G = int(p["num_heads"]), int(p["num_kv_heads"])
        self.dk, self.dv = int(p["head_dim"]), int(p["v_head_dim"])
        self.taps = int(p["conv"])
        self.eps = float(p["eps"])
        self.decay = p.get("decay", "head")
        self.gate = p.get("gate", "silu")
        self.decay_rank = p.get("decay_rank")
        self.gate_rank = p.get("gate_rank")
        if self.G <= 0 or self.H % self.G:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        if self.decay not in ("head", "channel") or self.gate not in ("silu", "sigmoid"):
            raise ValueError("decay must be 'head' or 'channel', gate 'silu' or 'sigmoid'")
        if self.taps < 1 or self.dk > 1024:
            raise ValueError("conv must be at least 1 tap and head_dim at most 1024")
        self.c_q, self.c_v = self.G * self.dk, self.H * self.dv
        self.c_qkv = 2 * self.c_q + self.c_v
        self.a_width = self.H * self.dk if self.decay == "channel" else self.H
        self.conv_floats = (self.taps - 1) * self.c_qkv
        self.state_floats = self.conv_floats + self.H * self.dk * self.dv

    @classmethod
    def weight_decls(cls, params):
        p = params
        w, H, G, dk, dv, taps = (int(p[k]) for k in ("hidden_size", "num_heads", "num_kv_heads", "head_dim", "v_head_dim", "conv"))
        a_width = H * dk if p.get("decay", "head") == "channel" else H
        out = {
            "q": WeightDecl((G * dk, w)),
            "k": WeightDecl((G * dk, w)),
            "v": WeightDecl((H * dv, w)),
            "q.conv": WeightDecl((G * dk, taps), kind="vector", init="conv"),
            "k.conv": WeightDecl((G * dk, taps), kind="vector", init="conv"),
            "v.conv": WeightDecl((H * dv, taps), kind="vector", init="conv"),
            "b": WeightDecl((H, w)),
            "A_log": WeightDecl((H,), kind="vector", init="small"),
            "dt_bias": WeightDecl((a_width,), kind="vector", init="small"),
            "norm": WeightDecl((dv,), kind="vector", init="ones"),
            "o": WeightDecl((w, H * dv)),
        }
        for stem, rank, width in (("a", p.get("decay_rank"), a_width), ("g", p.get("gate_rank"), H * dv)):
            if rank:
                out[stem + "1"] = WeightDecl((int(rank), w))
                out[stem + "2"] = WeightDecl((width, int(rank)), init="wide")
            else:
                out[stem] = WeightDecl((width, w))
        return out

    def state_shape(self):
        return (self.state_floats,)

    def bind(self, weights, rt):
        super().bind(weights, rt)
        W = weights
        dev, dt = rt.device, rt.dtype

        def stack(parts: list[torch.Tensor]) -> tuple[torch.Tensor, list[int]]:
            # rows of several projections in one matrix, each starting at a multiple of 8 columns of the result
            offs, rows, at = [], [], 0
            for t in parts:
                offs.append(at)
                rows.append(t)
                pad = _pad8(t.shape[0]) - t.shape[0]
                if pad:
                    rows.append(torch.zeros((pad, t.shape[1]), dtype=t.dtype, device=t.device))
                at += _pad8(t.shape[0])
            return torch.cat(rows, dim=0).contiguous(), offs

        # one product in the storage type: q, k, v, then what feeds the gate and a low-rank decay
        main = [torch.cat([W["q"], W["k"], W["v"]], dim=0), W["g1"] if self.gate_rank else W["g"]]
        if self.decay_rank:
            main.append(W["a1"])
        self.w_main, offs = stack(main)
        self.off_gate = offs[1]
        self.off_a1 = offs[2] if self.decay_rank else None
        # one product with a float result: the logits of beta, and of the step size when they come straight from h
        small = [W["b"]] if self.decay_rank else [W["b"], W["a"]]
        self.w_small, soffs = stack(small)
        self.off_a = soffs[1] if not self.decay_rank else None
        self.w_a2 = W.get("a2")
        self.w_g2 = W.get("g2")
        self.w_o = W["o"].contiguous()
        self.w_conv = torch.cat([W["q.conv"], W["k.conv"], W["v.conv"]], dim=0).contiguous()
        self.a_log, self.dt_bias, self.norm_w = W["A_log"], W["dt_bias"], W["norm"]
        del dev, dt

    def forward(self, ctx, x: torch.Tensor, cache):
        rt = self.rt
        n = x.shape[0]
        if cache is None or cache.state is None:
            raise RuntimeError("gated_delta_rule needs a state slot per request")
        H, dk, dv = self.H, self.dk, self.dv
        main = rt.buf("delta.main", n, self.w_main.shape[0])
        product(x, self.w_main, main)
        # the logits of beta (and of a per-head step size): few output rows, so for a few tokens the product runs over
        # slices of K in parallel and the kernel that prepares the delta rule's inputs sums the slices
        c_small = self.w_small.shape[0]
        slices = ops.skinny_splits(c_small, self.hidden, n) if (ops.skinny_ok(x, self.w_small) and n <= 8) else 1
        slices = min(slices, 8)
        if slices > 1:
            part = rt.buf("delta.small_part", 8 * 8, c_small, torch.float32, cap=64)[: slices * n].view(slices, n, c_small)
            ops.gemm_skinny(x, self.w_small, ops.Partials(part))
            small, slice_stride = part[0], part.stride(0)
        else:
            small, slice_stride = rt.buf("delta.small", n, c_small, torch.float32), 0
            product(x, self.w_small, small)
        qkv = rt.buf("delta.qkv", n, self.c_qkv)
        conv_state = cache.state[:, : self.conv_floats]
        ops.causal_conv(
            main[:, : self.c_qkv], self.w_conv, conv_state, ctx.query_start_loc, ctx.state_slots, ctx.num_seqs, qkv, activation="silu",
            max_query_len=ctx.max_query_len,
        )
        if self.decay_rank:
            r = int(self.decay_rank)
            step = rt.buf("delta.step", n, self.a_width, torch.float32)
            product(main[:, self.off_a1 : self.off_a1 + r], self.w_a2, step)
        else:
            step = small[:, self.off_a : self.off_a + self.a_width]
        if self.gate_rank:
            r = int(self.gate_rank)
            gate = rt.buf("delta.gate", n, self.c_v)
            product(main[:, self.off_gate : self.off_gate + r], self.w_g2, gate)
        else:
            gate = main[:, self.off_gate : self.off_gate + self.c_v]
        read = rt.buf("delta.read", n, self.c_v, torch.float32)
        f32 = torch.float32
        scratch = (
            rt.buf("delta.kn", n, H * dk, f32), rt.buf("delta.qn", n, H * dk, f32),
            rt.buf("delta.gn", n, H * dk, f32) if self.decay == "channel" else None, rt.buf("delta.sc", n, H * 4, f32),
        )  # fmt: skip
        ops.gated_delta(
            qkv[:, : self.c_q], qkv[:, self.c_q : 2 * self.c_q], qkv[:, 2 * self.c_q :], small[:, :H], step, self.a_log, self.dt_bias,
            cache.state[:, self.conv_floats :], read, ctx.query_start_loc, ctx.state_slots, ctx.num_seqs, H, self.G, dk, dv,
            q_scale=dk**-0.5, norm_eps=1e-6, max_query_len=ctx.max_query_len, scratch=scratch,
            logit_slices=slices if slices > 1 else 0, logit_slice_stride=slice_stride,
        )  # fmt: skip
        y = rt.buf("delta.y", n, self.c_v)
        ops.gated_head_norm(read, gate, self.norm_w, self.eps, y, H, dv, activation=self.gate)
        return project(rt, "delta.proj", y, self.w_o, ctx)
