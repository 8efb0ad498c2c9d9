"""What of the Setenex decoder needs no GPU: the configuration and its names, the bias buckets, the pages
that a window with kept first tokens holds, and the plain implementation's own pieces."""

from __future__ import annotations

import math

import pytest
import torch

import plain_setenex as plain
from setenex_cases import CASES, random_tensors, tensor_shapes


@pytest.mark.parametrize("name", sorted(CASES))
def test_names_and_shapes_follow_the_configuration(name):
    from kvforge_b200.config.registry import architecture_of
    from kvforge_b200.parts.model import DecoderModel

    config = CASES[name]["config"]
    arch = architecture_of(config)
    want = tensor_shapes(config)
    cfg = arch.parse_config(config, want)
    model = DecoderModel(arch.build_spec(cfg))
    got = {k: tuple(d.shape) for k, d in model.expected_weights().items()}
    assert got == want
    # what the file says comes back when it is written again
    again = arch.parse_config(cfg.to_hf_dict(), None)
    assert again.layers == cfg.layers and again.loop == cfg.loop and again.embedding_scale == cfg.embedding_scale
    # a pass of the loop has cache entries of its own
    runs = plain.layer_runs(config)
    assert [(c.layer, c.offset_row) for c in model.spec.execution] == runs
    assert sum(len(g.calls) for g in model.groups) == len(runs)


def test_the_rows_of_a_bias_table_come_from_the_tensor():
    from kvforge_b200.config.model_config import ConfigError
    from kvforge_b200.config.setenex_config import SetenexConfig

    config = {k: v for k, v in CASES["c"]["config"].items()}
    config["layers"] = [dict(ly, mixer={k: v for k, v in ly["mixer"].items() if k != "bias_rows"}) for ly in config["layers"]]
    with pytest.raises(ConfigError):
        SetenexConfig.from_dict(config, None)
    cfg = SetenexConfig.from_dict(config, {"l0.mix.rel": (14, 4), "l1.mix.rel": (6, 2)})
    assert [ly.mixer.bias_rows for ly in cfg.layers] == [14, 6]
    with pytest.raises(ConfigError):
        SetenexConfig.from_dict({**config, "layers": [{"type": "mamba", "mixer": {}, "mlp": None}]}, None)


@pytest.mark.parametrize("rows,far", [(8, 30), (5, 17), (32, 1000), (2, 3), (3, 9)])
def test_distance_buckets(rows, far):
    from kvforge_b200.parts.attention import distance_buckets

    got = distance_buckets(rows, far).tolist()
    assert got == [plain.distance_bucket(n, rows, far) for n in range(far + 1)]
    assert got[: rows // 2] == list(range(rows // 2)) and got[-1] == rows - 1 and got == sorted(got)
    assert plain.distance_bucket(10 * far, rows, far) == rows - 1


def test_a_window_group_keeps_the_pages_of_the_first_tokens():
    from kvforge_b200.cache.block_manager import BlockManager, GroupSpec

    bm = BlockManager(12, 4, groups=[GroupSpec("window", 6, keep_first=5), GroupSpec("window", 6), GroupSpec("full")])
    bm.allocate("r", 3, 3)
    pos = 3
    for n in (2, 7, 1, 1, 9, 1, 1, 1):
        bm.append_slots("r", pos + n, pos)
        pos += n
        first_live = max(0, pos - n - 6 + 1) // 4
        kept, plain_window, full = (bm.get_block_table("r", g) for g in range(3))
        assert all(b >= 0 for b in full)
        for i in range(len(kept)):
            assert (kept[i] >= 0) == (i < 2 or i >= first_live)  # two pages hold the five kept tokens
            assert (plain_window[i] >= 0) == (i >= first_live)
        bm.check_invariants()
    bm.free("r")
    assert all(bm.free_blocks_of(g) == 12 for g in range(3))
    windows_only = BlockManager(12, 4, groups=[GroupSpec("window", 6, keep_first=5)])
    assert windows_only.can_ever_fit(1000, 8) and not windows_only.can_ever_fit(1000, 40)


def test_plain_route_groups_and_weights():
    """The plain router on a hand-made case: groups ranked by the sum of their top two shifted scores, the
    choice with the correction, the weights without it."""
    w = {"m.router": torch.eye(8, dtype=torch.float64), "m.correction": torch.tensor([0.0, 0, 0, 0, 0, 0, 0.9, 0], dtype=torch.float64)}
    z = torch.tensor([[2.0, 1.9, -9, -9, 3.0, -9, -1.0, -9]], dtype=torch.float64)
    r = {"experts": 8, "top": 2, "groups": {"count": 4, "keep": 2}}
    chosen, weights = plain.route(z, w, "m.", r)
    # group scores: {0,1}: s(2)+s(1.9) = 1.75; {4,5}: 0.95; {6,7}: s(-1)+0.9 = 1.17 -> groups 0 and 3 stay, expert 4 cannot be chosen
    s = torch.sigmoid(z[0])
    assert chosen[0].tolist() == [6, 0]
    assert torch.allclose(weights[0], torch.stack([s[6], s[0]]) / (s[6] + s[0]))
    assert abs(float(plain.gelu_erf(torch.tensor(0.7))) - 0.5 * 0.7 * (1 + math.erf(0.7 / math.sqrt(2)))) < 1e-7


def test_plain_model_sees_the_kept_tokens_and_the_window():
    """In the plain model a change of a token shows in a later position's logits exactly when that token is
    kept, inside the window of some layer's reach, or neither (then nothing moves)."""
    config = {
        "architecture": "Setenex", "vocab": 50, "width": 32, "norm": {"eps": 1e-5},
        "layers": [{"type": "attention", "mlp": None, "mixer": {"heads": 2, "kv_heads": 1, "dim": 8, "vdim": 8, "scale": 0.35, "bias_max": 20, "bias_rows": 6,
                                                                "mask": {"size": 4, "keep_first": 2}}}],
    }  # fmt: skip
    w = {k: v.double() for k, v in random_tensors(config, 3).items()}
    base = list(range(10, 30))
    ref = plain.logits(config, w, base)
    for j in (1, 2, 15, 16):
        toks = list(base)
        toks[j] += 1
        moved = float((plain.logits(config, w, toks)[19] - ref[19]).abs().max())
        assert (moved > 1e-6) == (j < 2 or 19 - j < 4), (j, moved)
