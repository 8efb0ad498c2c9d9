"""The Setenex decoder on the GPU against the plain implementation (``plain_setenex``): each new
mechanism alone, then whole models with random weights made here, replayed whole, token by token, in
portions down to two tokens and mixed with other requests on few pages and slots; in 32-bit and in
bfloat16, eager and as captured graphs; and greedy generation through the engine's entry point."""

from __future__ import annotations

import json
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

import plain_setenex as plain
import traces
from setenex_cases import CASES, attention, latent, plain_logits, random_config, random_tensors, row_error, write_folder
from test_gpu_mopilorn import check, run_trace, tokens
from test_gpu_parts import context, runtime

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent
TOL = {"float32": 1e-4, "bfloat16": 0.25}
SHARP_TOL = 1e-3
LENGTHS = {"a": [70, 3, 41, 1, 26, 97], "b": [9, 120, 33, 2, 64, 50], "c": [45, 17, 5, 80, 30], "d": [130, 20, 75, 49, 9]}
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def build(tmp, name, config, w, lengths, seed=40):
    folder = write_folder(tmp / name, config, w)
    reqs = {f"{name}{i}": tokens(config["vocab"], n, seed + i) for i, n in enumerate(lengths)}
    ref = {rid: plain_logits(config, w, t) for rid, t in reqs.items()}
    scale = float(torch.cat(list(ref.values())).pow(2).mean().sqrt())
    return folder, reqs, ref, scale, w


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    """Per case and storage type: folder, requests, plain logits of every request whole, the logits' scale.
    32-bit runs on weights whose router follows the token; bfloat16 on weights whose corrections decide the
    choice of experts, so that rounding cannot move a token to other experts than the plain model's."""
    tmp = tmp_path_factory.mktemp("setenex")
    out = {}
    for k, (name, case) in enumerate(sorted(CASES.items())):
        out[name, "float32"] = build(tmp, name, case["config"], random_tensors(case["config"], 17 + k), LENGTHS[name])
        out[name, "bfloat16"] = build(tmp, name + "-fixed", case["config"], random_tensors(case["config"], 27 + k, fixed_choice=True), LENGTHS[name])
    return out


def regime_steps(reqs, regime):
    if regime == "whole":
        return traces.whole(reqs)
    if regime == "tail":
        return traces.tail_one_by_one(reqs, 40)
    if regime == "portions":
        return traces.portions(reqs)
    prompt_lens = {rid: max(1, len(t) - 14) for rid, t in reqs.items()}
    steps = traces.mixed(reqs, prompt_lens, max_live=4, seed=5)
    assert max(len(s["entries"]) for s in steps) >= 3
    return steps


# ------------------------------------------------------------------ whole models


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CASES))
@pytest.mark.parametrize("regime", ["whole", "tail", "portions", "mixed"])
def test_replay_regimes(models, name, dtype, regime):
    """Whole prompts; the last 40 tokens one by one (every window passes over decoded tokens); portions of
    1 to 33 tokens; up to four live requests on as few pages as they need (pages and slots are used again)."""
    folder, reqs, ref, scale, _ = models[name, dtype]
    steps = regime_steps(reqs, regime)
    outs, runner = run_trace(folder, dtype, steps, CASES[name]["block_size"])
    check(steps, outs, ref, scale, TOL[dtype])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CASES))
@pytest.mark.parametrize("regime", ["tail", "mixed"])
def test_replay_as_captured_graphs(models, name, dtype, regime):
    """The way generation runs by default: single-token steps and steps of more than 16 tokens as CUDA
    graphs made for padded shapes.  Padding sequences and rows must leave every cache alone."""
    folder, reqs, ref, scale, _ = models[name, dtype]
    steps = traces.last_only(regime_steps(reqs, regime))
    outs, runner = run_trace(folder, dtype, steps, CASES[name]["block_size"], cuda_graphs=True)
    check(steps, outs, ref, scale, TOL[dtype])
    assert runner.core.runner.num_graph_kernels > 0


def test_batch_and_cutting_change_float32_logits_by_rounding_only(models):
    folder, reqs, ref, scale, _ = models["a", "float32"]
    whole, _ = run_trace(folder, "float32", traces.whole(reqs), 16)
    by_place = {}
    for rows, got in zip(traces.wanted_places(traces.whole(reqs)), whole):
        for i, place in enumerate(rows):
            by_place[place] = got[i]
    steps = regime_steps(reqs, "mixed")
    outs, _ = run_trace(folder, "float32", steps, 16)
    worst = 0.0
    for rows, got in zip(traces.wanted_places(steps), outs):
        for i, place in enumerate(rows):
            worst = max(worst, float((got[i] - by_place[place]).abs().max()))
    assert worst <= 2e-5 * scale, worst


@pytest.mark.parametrize("seed", [3, 12, 29, 41, 57, 68])
def test_configurations_drawn_at_random(tmp_path, seed):
    """Sizes that no hand-made case has (widths and inner sizes that are no multiple of 8 or of 16, one head, twenty
    heads, one expert a token out of ungrouped experts, a single pass of a loop, ...), each replayed whole, in
    portions and mixed, in both storage types."""
    config = random_config(seed)
    block_size = [4, 8, 16, 32][seed % 4]
    for dtype, fixed in (("float32", False), ("bfloat16", True)):
        folder, reqs, ref, scale, _ = build(tmp_path, f"drawn-{dtype}", config, random_tensors(config, 100 + seed, fixed_choice=fixed), [90, 1, 37, 140], seed=seed)
        for regime in ("whole", "portions", "mixed"):
            steps = regime_steps(reqs, regime) if regime != "mixed" else traces.mixed(reqs, {r: max(1, len(t) - 10) for r, t in reqs.items()}, max_live=4, seed=seed)
            outs, _ = run_trace(folder, dtype, steps, block_size)
            check(steps, outs, ref, scale, TOL[dtype])


def sharpened(w):
    """Queries and keys scaled up until a few keys take nearly all the weight."""
    w = dict(w)
    for k in list(w):
        if k.endswith(("mix.q.norm", "mix.k.norm")):
            w[k] = (w[k] * 2.5).to(torch.bfloat16).float()
        if k.endswith(("mix.uk",)):
            w[k] = (w[k] * 5.0).to(torch.bfloat16).float()
    return w


def test_sharp_attention_far_keys_window_edges_and_kept_tokens(tmp_path):
    """With sharp scores over sequences of several hundred tokens, a far key among hundreds (case c: no
    mask), the keys at a window's two ends and the last kept token (cases a, b) decide the logits: the plain
    model with a window or a count of kept tokens one off is far outside the tolerance."""
    for name, edges in (("c", False), ("a", True), ("b", True)):
        case = CASES[name]
        w = sharpened(random_tensors(case["config"], seed=91))
        folder, reqs, ref, scale, _ = build(tmp_path, f"sharp-{name}", case["config"], w, [310, 150], seed=70)
        if edges:
            for key in ("size", "keep_first"):
                for d in (-1, 1):
                    cfg2 = json.loads(json.dumps(case["config"]))
                    for ly in cfg2["layers"]:
                        if key in ly["mixer"].get("mask", {}):
                            ly["mixer"]["mask"][key] += d
                    rid = f"sharp-{name}1"
                    off = plain_logits(cfg2, w, reqs[rid])
                    errs = sorted(row_error(off[i], ref[rid][i], scale) for i in range(60, 150))
                    # a window's edge moves half of the rows; the last kept token, far behind most queries, a tenth
                    assert errs[len(errs) // 2 if key == "size" else int(len(errs) * 0.9)] > 20 * SHARP_TOL, (name, key, d)
        for regime in ("whole", "tail", "portions"):
            steps = regime_steps(reqs, regime)
            outs, _ = run_trace(folder, "float32", steps, case["block_size"])
            check(steps, outs, ref, scale, SHARP_TOL, SHARP_TOL)


def test_long_decoding(models):
    """Three hundred tokens one by one after a prompt of five: windows pass over decoded tokens many times,
    pages of the windows are given back and taken again, the kept first pages stay."""
    for name in ("a", "b"):
        case = CASES[name]
        for dtype, graphs in (("float32", False), ("bfloat16", True)):
            w = models[name, dtype][4]
            folder = models[name, dtype][0]
            reqs = {"long": tokens(case["config"]["vocab"], 305, 7)}
            ref = {"long": plain_logits(case["config"], w, reqs["long"])}
            scale = float(ref["long"].pow(2).mean().sqrt())
            steps = traces.tail_one_by_one(reqs, 300)
            outs, _ = run_trace(folder, dtype, steps, case["block_size"], cuda_graphs=graphs)
            check(steps, outs, ref, scale, TOL[dtype])


def test_the_trace_program_reads_a_folder_and_writes_logits(models, tmp_path):
    folder, reqs, ref, scale, _ = models["b", "float32"]
    steps = traces.portions(dict(list(reqs.items())[:3]))
    lines = "\n".join(json.dumps(s) for s in steps) + "\n"
    out = tmp_path / "out"
    res = subprocess.run(
        [sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", "float32", "--out", str(out), "--max-tokens", "256", "--max-live", "4"],
        input=lines, capture_output=True, text=True, timeout=600,
    )  # fmt: skip
    assert res.returncode == 0, res.stderr[-2000:]
    assert [ln for ln in res.stdout.splitlines() if ln.startswith("done")] == [f"done {s['step']}" for s in steps]
    vocab = CASES["b"]["config"]["vocab"]
    outs = [torch.from_numpy(np.fromfile(out / f"{s['step']}.f32", dtype="<f4").reshape(-1, vocab).copy()) for s in steps]
    check(steps, outs, ref, scale, TOL["float32"])


# ------------------------------------------------------------------ generation through the entry point


@pytest.mark.parametrize("name", ["a", "b", "d"])
def test_greedy_generation_through_the_engine(models, name):
    """``InferenceEngine.generate`` with its scheduler: more requests than slots, prompts cut into portions,
    decode steps as graphs, tokens read a step late."""
    from kvforge_b200 import CacheConfig, EngineConfig, InferenceEngine, SamplingParams, SchedulerConfig

    folder, _, _, _, w = models[name, "float32"]
    case = CASES[name]
    prompts = [tokens(case["config"]["vocab"], n, 300 + i) for i, n in enumerate([3, 40, 11, 1, 25, 18])]
    cfg = EngineConfig(
        cache=CacheConfig(block_size=case["block_size"], num_blocks=128),
        scheduler=SchedulerConfig(max_num_seqs=3, max_num_batched_tokens=32, max_model_len=128),
        dtype="float32",
    )
    engine = InferenceEngine(cfg, model=folder)
    outs = engine.generate(prompts, SamplingParams(max_tokens=12, temperature=0.0, ignore_eos=True))
    wd = {k: v.double() for k, v in w.items()}
    for p, o in zip(prompts, outs):
        assert o.output_token_ids == plain.greedy(case["config"], wd, p, 12)
    assert engine.core.state_slots.num_free == 3


def test_generation_from_a_named_shape_with_random_weights():
    from kvforge_b200 import PRESETS, EngineConfig, InferenceEngine, SamplingParams, SchedulerConfig

    cfg = EngineConfig(model=PRESETS["setenex-tiny"], scheduler=SchedulerConfig(max_num_seqs=4, max_num_batched_tokens=64, max_model_len=96), dtype="bfloat16")
    engine = InferenceEngine(cfg)
    outs = engine.generate([[1, 2, 3], list(range(40))], SamplingParams(max_tokens=8, temperature=0.0, ignore_eos=True))
    assert all(len(o.output_token_ids) == 8 for o in outs)


# ------------------------------------------------------------------ mechanisms alone


def as_float(y, n):
    from kvforge_b200 import ops

    return y.t[:, :n].sum(0) if isinstance(y, ops.Partials) else y[:n].float()


def part_tol(dtype):
    return 2e-5 if dtype == torch.float32 else 3e-2


def rel_rows(got, want):
    return float((got.double() - want.double()).abs().max() / want.double().abs().max())


def step_mixer(part, rt, x, cache_k, cache_v, bs, table, cuts, group_cache):
    """Run a mixer over a sequence cut into steps on pages of a shuffled table."""
    t = x.shape[0]
    slots = [table[p // bs] * bs + p % bs for p in range(t)]
    got = []
    for a, b in cuts:
        ctx = context(rt, [b - a], [a], bs, [table], slots[a:b])
        got.append(as_float(part.forward(ctx, x[a:b].cuda(), group_cache), b - a).cpu().clone())
    return torch.cat(got)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window,keep", [(None, 0), (7, 0), (7, 3), (5, 9), (70, 66)])
@pytest.mark.parametrize("dk,dv,t", [(24, 16, 45), (64, 64, 200), (128, 128, 150)])
def test_attention_with_normed_heads_bias_and_kept_tokens(dtype, window, keep, dk, dv, t):
    """The whole sequence in one step, then portions and single tokens on top of the cache (the decode
    form: key ranges in parallel), against the plain mixer.  Heads of 64 in bfloat16 go to the tensor-core
    kernel while a step brings more than single tokens; 200 tokens are several of its tiles of keys, with the
    kept tokens in a tile of their own."""
    from kvforge_b200.parts.base import LayerCache, PartSpec, build_part

    rt = runtime(dtype)
    width, nh, nkv, bs, rows, far, eps = 80, 6, 3, 4, 7, 19, 1e-5
    m = attention(nh, nkv, dk, dv, rows, far, window, keep)
    names = {"q_proj.weight": "q", "k_proj.weight": "k", "v_proj.weight": "v", "o_proj.weight": "o", "q_norm.weight": "q.norm", "k_norm.weight": "k.norm"}
    part = build_part("mixer", PartSpec("paged_attention", {
        "hidden_size": width, "num_heads": nh, "num_kv_heads": nkv, "head_dim": dk, "v_head_dim": dv, "scale": m["scale"], "window": window,
        "keep_first": keep, "position": None, "qk_norm": {"eps": eps}, "distance_bias": {"rows": rows, "far": far}, "names": names}), "m.")  # fmt: skip
    g = torch.Generator().manual_seed(3)
    shapes = {"q": (nh * dk, width), "k": (nkv * dk, width), "v": (nkv * dv, width), "o": (width, nh * dv), "q.norm": (dk,), "k.norm": (dk,), "rel": (rows, nh)}
    w = {k: (torch.randn(s, generator=g) * (1.0 if k == "rel" else 0.2) + (1.5 if "norm" in k else 0.0)).to(dtype).float() for k, s in shapes.items()}
    kinds = type(part).weight_decls(part.params)
    bound = {}
    for local, decl in kinds.items():
        tensor = w[names.get(local, local)]
        bound[local] = tensor.cuda() if decl.kind == "vector" else tensor.to(dtype).cuda()
    part.bind(bound, rt)
    x = (torch.randn(t, width, generator=g)).to(dtype)
    ref = plain.biased_attention(x.double(), {"m." + k: v.double() for k, v in w.items()}, "m.", m, eps)
    nb = 64
    table = [int(i) for i in torch.randperm(nb, generator=g)]
    need = part.cache_need()
    assert (need.kind, need.keep_first) == (("window", keep) if window else ("full", 0))
    cache = LayerCache(torch.zeros(nb, nkv, bs, dk, device="cuda", dtype=dtype), torch.zeros(nb, nkv, bs, dv, device="cuda", dtype=dtype), 0)
    for cuts in ([(0, t)], [(0, 17), (17, 19), (19, 20), (20, 21), (21, 34), (34, 35), (35, 36), (36, t - 3), (t - 3, t - 2), (t - 2, t)]):
        got = step_mixer(part, rt, x, None, None, bs, table, cuts, cache)
        assert rel_rows(got, ref) < part_tol(dtype), cuts


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize(
    "heads,dk,dr,dv,rank,window",
    [(3, 16, 8, 24, 24, 9), (5, 8, 16, 8, 40, None), (2, 32, 32, 16, 264, 30), (16, 16, 32, 8, 64, 40), (5, 8, 16, 8, 96, None), (20, 8, 16, 8, 128, 33), (2, 32, 64, 16, 512, 70)],
)
def test_latent_attention(dtype, heads, dk, dr, dv, rank, window):
    """The cache holds one row of ``rank + rot_dim`` numbers per token; whole, in portions and token by token.  In
    bfloat16 latents of 64, 96, 128, 256 or 512 numbers (with rows that are a multiple of 16 wide) go to the
    tensor-core kernel: 16 heads a CTA, fewer heads with several tokens a CTA, more heads in chunks."""
    from kvforge_b200.parts.base import LayerCache, PartSpec, build_part

    rt = runtime(dtype)
    width, bs, eps = 64, 8, 1e-6
    m = latent(heads, dk, dr, dv, rank, window, base=300.0)
    pos = PartSpec("rotary", {"head_dim": dr, "rotary_dim": dr, "theta": 300.0, "interleaved": True})
    part = build_part("mixer", PartSpec("latent_attention", {
        "hidden_size": width, "num_heads": heads, "head_dim": dk, "rot_dim": dr, "v_head_dim": dv, "kv_rank": rank, "eps": eps, "scale": m["scale"],
        "window": window, "position": pos, "gate": "sigmoid"}), "m.")  # fmt: skip
    g = torch.Generator().manual_seed(5)
    shapes = {"q": (heads * (dk + dr), width), "dkv": (rank + dr, width), "dkv.norm": (rank,), "uk": (heads * dk, rank), "uv": (heads * dv, rank),
              "g": (heads, width), "o": (width, heads * dv)}  # fmt: skip
    w = {k: (torch.randn(s, generator=g) * (2.0 / s[-1] ** 0.5) + (1.0 if "norm" in k else 0.0)).to(dtype).float() for k, s in shapes.items()}
    kinds = type(part).weight_decls(part.params)
    part.bind({k: (w[k].cuda() if kinds[k].kind == "vector" else w[k].to(dtype).cuda()) for k in kinds}, rt)
    t = 50 if rank < 64 else 150
    x = torch.randn(t, width, generator=g).to(dtype)
    ref = plain.latent_attention(x.double(), {"m." + k: v.double() for k, v in w.items()}, "m.", m, eps)
    need = part.cache_need()
    assert need.v_in_k and need.kv_heads == 1 and need.head_dim == rank + dr and need.value_dim == rank
    table = [int(i) for i in torch.randperm(24, generator=g)]
    k = torch.zeros(24, 1, bs, rank + dr, device="cuda", dtype=dtype)
    cache = LayerCache(k, k, 0)
    for cuts in ([(0, t)], [(0, 21), (21, 23), (23, 24), (24, 25), (25, 41), (41, 42), (42, t - 2), (t - 2, t - 1), (t - 1, t)]):
        got = step_mixer(part, rt, x, None, None, bs, table, cuts, cache)
        assert rel_rows(got, ref) < part_tol(dtype), cuts


@pytest.mark.parametrize("experts,top,groups,keep", [(6, 2, 3, 2), (8, 3, 4, 4), (4, 1, 1, 1), (12, 4, 12, 5), (40, 6, 5, 2)])
def test_router_alone(experts, top, groups, keep):
    """Chosen experts and weights against the plain router, on tokens whose choice does not hang on the last
    bits (the gap between the last chosen and the first left out is wider than 32-bit rounding)."""
    from kvforge_b200 import ops

    g = torch.Generator().manual_seed(experts)
    width, n = 72, 200
    x = torch.randn(n, width, generator=g)
    w = {"m.router": torch.randn(experts, width, generator=g) * 0.3, "m.correction": torch.randn(experts, generator=g) * 0.3}
    r = {"experts": experts, "top": top, "groups": {"count": groups, "keep": keep}}
    chosen, weights = plain.route(x.double(), {k: v.double() for k, v in w.items()}, "m.", r)
    ids = torch.zeros(n, top, dtype=torch.int32, device="cuda")
    wts = torch.zeros(n, top, dtype=torch.float32, device="cuda")
    ops.moe_route(x.cuda(), w["m.router"].cuda(), w["m.correction"].cuda(), top, groups, keep, 1e-20, ids, wts)
    same = 0
    for i in range(n):
        if sorted(ids[i].tolist()) == sorted(chosen[i].tolist()):
            same += 1
            order = {e: k for k, e in enumerate(ids[i].tolist())}
            got = torch.stack([wts[i, order[e]] for e in chosen[i].tolist()]).cpu()
            assert torch.allclose(got.double(), weights[i], atol=1e-6)
            assert abs(float(wts[i].sum()) - 1.0) < 1e-6
    assert same >= n - 2  # a near tie may fall the other way in 32-bit


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n", [1, 7, 30, 150, 400])
def test_routed_experts(dtype, n):
    """The feed-forward part against the plain one, for one token, a few and many (several tiles an expert; in
    bfloat16 the tile sizes of the tensor-core product follow the rows an expert gets, and from 64 rows an expert
    on average the products run on the tcgen05 tensor cores)."""
    from kvforge_b200.parts.base import PartSpec, build_part

    rt = runtime(dtype, max_tokens=512)
    width, experts, top, ff = 48, 6, 2, 40
    part = build_part("ffn", PartSpec("routed_experts", {"hidden_size": width, "experts": experts, "top": top, "intermediate_size": ff, "groups": 3, "keep": 2}), "m.")
    g = torch.Generator().manual_seed(11)
    w = {"router": torch.randn(experts, width, generator=g) * 0.05, "correction": 0.7 * torch.randperm(experts, generator=g).float()}
    for e in range(experts):
        w[f"e{e}.up"] = (torch.randn(ff, width, generator=g) * 0.2).to(dtype).float()
        w[f"e{e}.down"] = (torch.randn(width, ff, generator=g) * 0.2).to(dtype).float()
    kinds = type(part).weight_decls(part.params)
    part.bind({k: (w[k].cuda() if kinds[k].kind == "vector" else w[k].to(dtype).cuda()) for k in kinds}, rt)
    x = torch.randn(n, width, generator=g).to(dtype)
    mlp = {"router": {"experts": experts, "top": top, "groups": {"count": 3, "keep": 2}}}
    ref = plain.mixture_of_experts(x.double(), {"m." + k: v.double() for k, v in w.items()}, "m.", mlp)
    ctx = context(rt, [n], [0], 4, [[0]], [0] * n)
    got = as_float(part.forward(ctx, x.cuda()), n).cpu()
    assert rel_rows(got, ref) < part_tol(dtype)
    # straight into the residual stream
    resid = torch.ones(n, width, device="cuda")
    ctx.residual = resid
    from kvforge_b200 import ops

    assert part.forward(ctx, x.cuda()) is ops.ADDED
    assert rel_rows(resid.cpu() - 1.0, ref) < part_tol(dtype) + 1e-6


def test_small_parts():
    """The norm that multiplies by one plus its weight, the scaled embedding, the row added between passes."""
    from kvforge_b200 import ops
    from kvforge_b200.parts.base import PartSpec, build_part

    rt = runtime(torch.float32)
    norm = build_part("norm", PartSpec("rmsnorm", {"dim": 40, "eps": 1e-5, "one_plus": True}), "n.")
    w, x = torch.randn(40) * 0.1, torch.randn(6, 40)
    norm.bind({"weight": w.cuda()}, rt)
    assert torch.allclose(norm.forward(None, x.cuda(), None).cpu(), plain.norm_one_plus(x, w, 1e-5), atol=1e-6)
    emb = build_part("embedding", PartSpec("token_embedding", {"vocab_size": 9, "hidden_size": 40, "scale": 2.5}), "e.")
    table = torch.randn(9, 40)
    emb.bind({"weight": table.cuda()}, rt)
    ctx = context(rt, [4], [0], 4, [[0]], [0] * 4)
    ctx.token_ids = torch.tensor([3, 0, 8, 3], dtype=torch.int32, device="cuda")
    resid = torch.zeros(4, 40, device="cuda")
    emb.forward(ctx, resid)
    assert torch.equal(resid.cpu(), table[[3, 0, 8, 3]] * 2.5)
    row = torch.randn(40)
    ops.add_row(resid, row.cuda())
    assert torch.equal(resid.cpu(), table[[3, 0, 8, 3]] * 2.5 + row)
