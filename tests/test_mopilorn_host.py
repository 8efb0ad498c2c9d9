"""Host-side tests of the Mopilorn decoder: its configuration reader, the tensor names and shapes
its parts ask for, and the plain implementation's own mechanisms (each against a second way of
computing the same thing).  No GPU is needed."""

from __future__ import annotations

import math

import pytest
import torch

import plain_mopilorn as plain
from mopilorn_cases import CASES, plain_logits, random_tensors, tensor_shapes

from kvforge_b200 import PRESETS, ConfigError
from kvforge_b200.config.mopilorn_config import MopilornConfig
from kvforge_b200.config.registry import architecture_of
from kvforge_b200.engine.core import spec_from_config
from kvforge_b200.parts.model import DecoderModel


@pytest.mark.parametrize("name", sorted(CASES))
def test_parts_ask_for_the_designs_tensors(name):
    case = CASES[name]
    shapes = tensor_shapes(case["config"], case["ranks"])
    arch = architecture_of(case["config"])
    cfg = arch.parse_config(case["config"], shapes)
    model = DecoderModel(arch.build_spec(cfg))
    got = {k: tuple(v.shape) for k, v in model.expected_weights().items()}
    assert got == shapes
    # cache groups: one per distinct (window, sizes) among the attention parts; a state per layer
    windows = {(ly["mixer"]["left"].get("mask", {}).get("size"), ly["mixer"]["left"]["dim"]) for ly in case["config"]["layers"] if ly["type"] == "parallel"}
    assert len(model.groups) == len(windows)
    assert all(s is not None for s in model.state_shapes)


def test_configuration_round_trip_and_errors():
    for name, case in CASES.items():
        shapes = tensor_shapes(case["config"], case["ranks"])
        cfg = MopilornConfig.from_dict(case["config"], shapes)
        again = MopilornConfig.from_dict(cfg.to_hf_dict())  # ranks are written, so no shapes are needed
        assert again.layers == cfg.layers and again.streams == cfg.streams and again.logit_softcap == cfg.logit_softcap, name
    base = CASES["a"]["config"]
    with pytest.raises(ConfigError):
        MopilornConfig.from_dict({**base, "layers": [{**base["layers"][0], "type": "other"}]})
    with pytest.raises(ConfigError):
        MopilornConfig.from_dict({k: v for k, v in base.items() if k != "width"})
    with pytest.raises(ConfigError):  # a low-rank inner size that nothing gives
        MopilornConfig.from_dict(base)
    bad = {**base, "layers": [{**base["layers"][1], "mlp": {"kind": "sparse", "ff": 8}}]}
    with pytest.raises(ConfigError):
        MopilornConfig.from_dict(bad, tensor_shapes(base, (5, 8)))


def test_named_shapes_build():
    for name in ("mopilorn-tiny", "mopilorn-1b"):
        model = DecoderModel(spec_from_config(PRESETS[name]))
        assert model.spec.residual_streams == PRESETS[name].streams
        assert len(model.expected_weights()) > 10


# ------------------------------------------------------------------ the plain implementation's mechanisms


def test_short_conv_is_causal_and_ends_on_the_current_token():
    u = torch.randn(9, 3, dtype=torch.float64)
    w = torch.randn(3, 4, dtype=torch.float64)
    y = plain.short_conv(u, w)
    for t in range(9):
        want = sum(w[:, j] * (u[t - 3 + j] if t - 3 + j >= 0 else 0.0) for j in range(4))
        assert torch.allclose(y[t], want)


def test_rotation_pairs_neighbours_and_keeps_the_rest():
    x = torch.randn(5, 2, 12, dtype=torch.float64)
    f = plain.rotary_frequencies(8, 100.0, None)
    y = plain.rotate_interleaved(x, torch.arange(5), f)
    assert torch.equal(y[..., 8:], x[..., 8:])
    a = 3 * f[2]
    assert math.isclose(float(y[3, 1, 4]), float(x[3, 1, 4] * torch.cos(a) - x[3, 1, 5] * torch.sin(a)), rel_tol=1e-12)
    assert math.isclose(float(y[3, 1, 5]), float(x[3, 1, 5] * torch.cos(a) + x[3, 1, 4] * torch.sin(a)), rel_tol=1e-12)
    # scores depend on the distance alone
    q, k = torch.randn(1, 1, 8, dtype=torch.float64), torch.randn(1, 1, 8, dtype=torch.float64)
    s = lambda i, j: float((plain.rotate_interleaved(q, torch.tensor([i]), f) * plain.rotate_interleaved(k, torch.tensor([j]), f)).sum())  # noqa: E731
    assert math.isclose(s(7, 3), s(104, 100), rel_tol=1e-9)


def test_frequency_scaling_regimes():
    sc = {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64}
    f0 = plain.rotary_frequencies(16, 10000.0, None)
    f1 = plain.rotary_frequencies(16, 10000.0, sc)
    for a, b in zip(f0.tolist(), f1.tolist()):
        lam = 2 * math.pi / a
        if lam < 16:
            assert b == a
        elif lam > 64:
            assert math.isclose(b, a / 8)
        else:
            assert a / 8 <= b <= a
    assert f1[0] == f0[0] and math.isclose(float(f1[-1]), float(f0[-1]) / 8)


def test_window_counts_the_token_itself():
    t, win = 12, 4
    q = torch.zeros(t, 1, 2, dtype=torch.float64)
    k = torch.zeros(t, 1, 2, dtype=torch.float64)
    v = torch.eye(t, dtype=torch.float64)[:, None, :]  # the read-out shows the weights
    o = plain.windowed_attention(q, k, v, 1.0, win)[:, 0]
    for i in range(t):
        seen = [j for j in range(t) if o[i, j] > 0]
        assert seen == list(range(max(0, i - win + 1), i + 1))


def test_delta_rule_against_its_closed_form_for_two_tokens():
    torch.manual_seed(0)
    dk, dv = 3, 2
    q, k = torch.randn(2, 1, dk, dtype=torch.float64), torch.randn(2, 1, dk, dtype=torch.float64)
    v = torch.randn(2, 1, dv, dtype=torch.float64)
    beta = torch.rand(2, 1, dtype=torch.float64)
    g = torch.rand(2, 1, dk, dtype=torch.float64)
    o = plain.delta_rule(q, k, v, beta, g)
    s1 = torch.outer(k[0, 0], beta[0, 0] * v[0, 0])
    assert torch.allclose(o[0, 0], s1.T @ q[0, 0])
    s1d = g[1, 0][:, None] * s1
    s2 = s1d + torch.outer(k[1, 0], beta[1, 0] * (v[1, 0] - s1d.T @ k[1, 0]))
    assert torch.allclose(o[1, 0], s2.T @ q[1, 0])
    # one factor a head is the same as that factor on every key channel
    gh = torch.rand(2, 1, dtype=torch.float64)
    assert torch.allclose(plain.delta_rule(q, k, v, beta, gh), plain.delta_rule(q, k, v, beta, gh[..., None].expand(2, 1, dk)))


def test_a_prefix_has_the_logits_of_the_whole():
    for name in ("a", "c"):
        case = CASES[name]
        w = random_tensors(case["config"], case["ranks"], seed=3)
        toks = [int(t) for t in torch.randint(0, case["config"]["vocab"], (30,), generator=torch.Generator().manual_seed(1))]
        whole = plain_logits(case["config"], w, toks)
        part = plain_logits(case["config"], w, toks[:17])
        assert torch.allclose(whole[:17], part, atol=1e-9)


def test_streams_of_one_with_unit_weights_are_the_plain_sum():
    case = CASES["c"]
    cfg = dict(case["config"])
    w = random_tensors(cfg, case["ranks"], seed=5)
    toks = list(range(1, 20))
    ref = plain_logits(cfg, w, toks)
    cfg1 = {**cfg, "streams": 1}
    w1 = dict(w)
    for i, ly in enumerate(cfg["layers"]):
        for hc in ("hc1", "hc2"):
            w1[f"l{i}.{hc}.in"] = torch.ones(1)
            w1[f"l{i}.{hc}.out"] = torch.ones(1)
            w1[f"l{i}.{hc}.mix"] = torch.ones(1, 1)
    assert torch.allclose(plain_logits(cfg1, w1, toks), ref, atol=1e-10)
