"""The Mopilorn decoder on the GPU against the plain implementation (``plain_mopilorn``): each new
kernel alone, then whole models with random weights made here, replayed whole, token by token, in
portions down to two tokens and mixed with other requests on few pages and slots; in 32-bit and
in bfloat16, eager and as captured graphs; and greedy generation through the engine's entry point."""

from __future__ import annotations

import json
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.nn.functional as F

import plain_mopilorn as plain
import traces
from mopilorn_cases import CASES, plain_logits, random_tensors, row_error, write_folder

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent
# row error: rms over the vocabulary of the difference, relative to the rms of the reference logits.
# bfloat16: weights are bfloat16 in both, so what differs is the rounding of activations (2^-8 each) through
# the layers; on models this narrow single rows lose up to a tenth, so a row may be off by a quarter and the
# mean over a trace by a twentieth (a wrong key, state or window is off by the whole scale)
TOL = {"float32": 1e-4, "bfloat16": 0.25}
MEAN_TOL = {"float32": 1e-4, "bfloat16": 0.05}
# with scores five times as large, rounding in 32-bit alone moves a row by 1e-4 (the plain implementation in 32-bit
# against itself in 64-bit: 8e-5); a window's edge off by one moves half of the rows by more than 0.08
SHARP_TOL = 1e-3
LENGTHS = {"a": [70, 3, 41, 1, 26, 97], "b": [9, 120, 33, 2, 64, 50], "c": [45, 17, 5, 80, 30], "d": [130, 20, 75, 49, 9]}
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def tokens(vocab, n, seed):
    g = torch.Generator().manual_seed(seed)
    return [int(t) for t in torch.randint(0, vocab, (n,), generator=g)]


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    """Per case: folder, requests, plain logits of every request whole, and the logits' scale."""
    tmp = tmp_path_factory.mktemp("mopilorn")
    out = {}
    for name, case in CASES.items():
        w = random_tensors(case["config"], case["ranks"], seed=17 + len(out))
        folder = write_folder(tmp / name, case["config"], w)
        reqs = {f"{name}{i}": tokens(case["config"]["vocab"], n, 40 + i) for i, n in enumerate(LENGTHS[name])}
        ref = {rid: plain_logits(case["config"], w, t) for rid, t in reqs.items()}
        scale = float(torch.cat(list(ref.values())).pow(2).mean().sqrt())
        out[name] = (folder, reqs, ref, scale, w)
    return out


def run_trace(folder, dtype, steps, block_size, max_tokens=None, max_live=4, **kw):
    from kvforge_b200.replay import TraceRunner

    page = max(64, block_size)
    runner = TraceRunner(str(folder), dtype, max_tokens or traces.tokens_needed(steps, page), max_live=max_live, block_size=block_size, **kw)
    outs = [runner.step(s) for s in steps]
    outs = [None if o is None else o.clone() for o in outs]
    runner.core.block_manager.check_invariants()
    runner.core.state_slots.check_invariants()
    assert runner.core.block_manager.num_free_blocks == runner.core.block_manager.num_blocks
    assert runner.core.state_slots.num_free == runner.core.state_slots.num_slots
    return outs, runner


def check(steps, outputs, ref, scale, tol, mean_tol=None):
    """Every wanted row against the plain logits.  32-bit: every row within ``tol``.  bfloat16: rounding
    through a badly conditioned place (a unit norm of eight small numbers) can throw a single row, so one row in
    fifty may exceed ``tol``; the mean over the trace is bounded as well."""
    errs = []
    for s, rows, got in zip(steps, traces.wanted_places(steps), outputs):
        if not rows:
            assert got is None
            continue
        assert got.shape[0] == len(rows)
        for i, (rid, pos) in enumerate(rows):
            errs.append((row_error(got[i], ref[rid][pos], scale), s["step"], rid, pos))
    assert errs
    over = [e for e in errs if not e[0] < tol]
    allowed = len(errs) // 50 if tol >= 0.1 else 0
    assert len(over) <= allowed, f"{len(over)} of {len(errs)} rows over {tol}; the worst: step {max(over)[1]} request {max(over)[2]} position {max(over)[3]}: {max(over)[0]:.3e}"
    mean_tol = mean_tol if mean_tol is not None else MEAN_TOL["float32" if tol < 0.1 else "bfloat16"]
    mean = sum(e[0] for e in errs) / len(errs)
    assert mean < mean_tol, f"mean row error {mean:.3e} (tolerance {mean_tol})"


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
    """Whole prompts; the last 40 tokens one by one (long enough for every window to pass over decoded
    tokens); portions of 1 to 33 tokens; up to four live requests on as few pages as they need (pages and
    the four state slots are used again)."""
    folder, reqs, ref, scale, _ = models[name]
    steps = regime_steps(reqs, regime)
    outs, runner = run_trace(folder, dtype, steps, CASES[name]["block_size"])
    check(steps, outs, ref, scale, TOL[dtype])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CASES))
@pytest.mark.parametrize("regime", ["tail", "mixed"])
def test_replay_as_captured_graphs(models, name, dtype, regime):
    """The way generation runs by default: single-token steps and steps of more than 16 tokens as CUDA
    graphs made for padded shapes.  Padding sequences and rows must leave every state alone."""
    folder, reqs, ref, scale, _ = models[name]
    steps = traces.last_only(regime_steps(reqs, regime))
    outs, runner = run_trace(folder, dtype, steps, CASES[name]["block_size"], cuda_graphs=True)
    check(steps, outs, ref, scale, TOL[dtype])
    assert runner.core.runner.num_graph_kernels > 0


def test_batch_and_cutting_change_float32_logits_by_rounding_only(models):
    """In 32-bit a request gives the same logits alone and whole as beside others in portions: every sum
    of the new kernels has an order that the sizes alone fix."""
    folder, reqs, ref, scale, _ = models["a"]
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
    assert worst <= 2e-5 * scale, worst  # attention's key tiles of a portion start elsewhere: rounding only


def test_sharp_attention_far_keys_and_window_edges(models, tmp_path):
    """Queries and keys scaled up until a few keys take nearly all the weight, over sequences of several
    hundred tokens: a far key among hundreds (no window, case c) or the keys at a window's two ends (case b)
    then decide the logits.  The plain implementation with a window one longer or one shorter is far outside
    the tolerance, so an edge that is off by one shows."""
    for name, edge in (("c", False), ("b", True)):
        case = CASES[name]
        w = dict(random_tensors(case["config"], case["ranks"], seed=91))
        for k in list(w):
            if k.endswith(("left.q", "left.k")):
                w[k] = (w[k] * 5.0).to(torch.bfloat16).float()
        folder = write_folder(tmp_path / f"sharp-{name}", case["config"], w)
        reqs = {f"s{name}{i}": tokens(case["config"]["vocab"], n, 70 + i) for i, n in enumerate([310, 150])}
        ref = {rid: plain_logits(case["config"], w, t) for rid, t in reqs.items()}
        scale = float(torch.cat(list(ref.values())).pow(2).mean().sqrt())
        if edge:
            for d in (-1, 1):
                cfg2 = json.loads(json.dumps(case["config"]))
                for ly in cfg2["layers"]:
                    if ly["type"] == "parallel":
                        ly["mixer"]["left"]["mask"]["size"] += d
                off = plain_logits(cfg2, w, reqs[f"s{name}1"])
                errs = sorted(row_error(off[i], ref[f"s{name}1"][i], scale) for i in range(60, 150))
                assert errs[len(errs) // 2] > 20 * SHARP_TOL  # half of the rows are off by more than that
        for regime in ("whole", "tail", "portions"):
            steps = regime_steps(reqs, regime)
            outs, _ = run_trace(folder, "float32", steps, case["block_size"])
            check(steps, outs, ref, scale, SHARP_TOL, SHARP_TOL)


def test_long_decoding_keeps_the_state(models):
    """Three hundred tokens one by one after a prompt of five: the state is carried through every step."""
    folder, _, _, _, w = models["a"]
    case = CASES["a"]
    reqs = {"long": tokens(case["config"]["vocab"], 305, 7)}
    ref = {"long": plain_logits(case["config"], w, reqs["long"])}
    scale = float(ref["long"].pow(2).mean().sqrt())
    steps = traces.tail_one_by_one(reqs, 300)
    for dtype, graphs in (("float32", False), ("bfloat16", True)):
        outs, _ = run_trace(folder, dtype, steps, 16, cuda_graphs=graphs)
        check(steps, outs, ref, scale, TOL[dtype])


def test_the_trace_program_reads_a_folder_and_writes_logits(models, tmp_path):
    folder, reqs, ref, scale, _ = models["b"]
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


def plain_greedy(config, w, prompt, n):
    toks = list(prompt)
    for _ in range(n):
        toks.append(int(plain_logits(config, w, toks)[-1].argmax()))
    return toks[len(prompt) :]


@pytest.mark.parametrize("name,dtype", [("a", "float32"), ("b", "float32"), ("d", "float32")])
def test_greedy_generation_through_the_engine(models, name, dtype):
    """``InferenceEngine.generate`` with its scheduler: more requests than state slots, prompts cut into
    portions, decode steps as graphs, tokens read a step late."""
    from kvforge_b200 import CacheConfig, EngineConfig, InferenceEngine, SamplingParams, SchedulerConfig

    folder, _, _, _, w = models[name]
    case = CASES[name]
    prompts = [tokens(case["config"]["vocab"], n, 300 + i) for i, n in enumerate([3, 40, 11, 1, 25, 18])]
    cfg = EngineConfig(
        cache=CacheConfig(block_size=case["block_size"], num_blocks=128),
        scheduler=SchedulerConfig(max_num_seqs=3, max_num_batched_tokens=32, max_model_len=128),
        dtype=dtype,
    )
    engine = InferenceEngine(cfg, model=folder)
    outs = engine.generate(prompts, SamplingParams(max_tokens=12, temperature=0.0, ignore_eos=True))
    for p, o in zip(prompts, outs):
        assert o.output_token_ids == plain_greedy(case["config"], w, p, 12)
    assert engine.core.state_slots.num_free == 3


def test_generation_from_a_named_shape_with_random_weights():
    from kvforge_b200 import PRESETS, EngineConfig, InferenceEngine, SamplingParams, SchedulerConfig

    cfg = EngineConfig(model=PRESETS["mopilorn-tiny"], scheduler=SchedulerConfig(max_num_seqs=4, max_num_batched_tokens=64, max_model_len=96), dtype="bfloat16")
    engine = InferenceEngine(cfg)
    outs = engine.generate([[1, 2, 3], list(range(40))], SamplingParams(max_tokens=8, temperature=0.0, ignore_eos=True))
    assert all(len(o.output_token_ids) == 8 for o in outs)


# ------------------------------------------------------------------ kernels alone


def flat_batch(lengths, slots, device):
    qsl = torch.tensor([0] + list(np.cumsum(lengths)), dtype=torch.int32, device=device)
    return qsl, torch.tensor(slots, dtype=torch.int32, device=device)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("taps,act,c", [(4, "silu", 40), (2, None, 40), (3, None, 40), (3, "silu", 30), (6, None, 36)])
def test_short_convolution_with_state(dtype, taps, act, c):
    """Three sequences cut into steps of unequal lengths (one shorter than the taps, one left out of a step,
    one padding sequence without rows and one without a slot), on slots in any order; a slot that is cleared
    and used again starts from zeros."""
    from kvforge_b200 import ops

    dev, dt = "cuda", DT[dtype]  # 40 channels: 16-byte loads; 30 and 36 (in bfloat16): one channel a thread
    g = torch.Generator().manual_seed(taps)
    w = torch.randn(c, taps, generator=g)
    seqs = [torch.randn(n, c, generator=g).to(dt).float() for n in (23, 9, 14)]
    want = [plain.short_conv(u.double(), w.double()) for u in seqs]
    if act:
        want = [F.silu(y) for y in want]
    state = torch.zeros(6, 7 + (taps - 1) * c, device=dev)  # the mixer's columns start at 7
    view = state[:, 7:]
    cuts = [[5, 1, 0, 2, 15], [2, 3, 4, 0, 0], [1, 1, 1, 8, 3]]  # steps 1 and 2 bring at most four rows a sequence
    slots = [4, 0, 2]
    got = [[] for _ in seqs]
    at = [0, 0, 0]
    for step in range(5):
        lens = [cuts[i][step] for i in range(3)]
        # after the three sequences: one without rows that holds slot 5, one without rows or slot, and three rows of no sequence
        x = torch.cat([seqs[i][at[i] : at[i] + lens[i]] for i in range(3)] + [torch.randn(3, c, generator=g)]).to(dev, dt)
        qsl, sl = flat_batch(lens + [0, 0], slots + [5, -1], dev)
        out = torch.full_like(x, 7.0)
        ops.causal_conv(x, w.to(dev), view, qsl, sl, 5, out, activation=act, max_query_len=max(lens) if step in (1, 2) else 0)
        assert bool((out[-3:] == 7.0).all())
        o = 0
        for i in range(3):
            got[i].append(out[o : o + lens[i]].float().cpu())
            o += lens[i]
            at[i] += lens[i]
    tol = 1e-5 if dtype == "float32" else 2e-2
    for i in range(3):
        assert torch.allclose(torch.cat(got[i]).double(), want[i], atol=tol, rtol=tol)
    assert float(state[:, :7].abs().max()) == 0 and float(state[[1, 3, 5]].abs().max()) == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("taps", [2, 4, 5])
def test_short_convolution_of_a_step_with_many_rows(dtype, taps):
    """More than a thousand rows in a step: rows come in tiles of four; a tile inside one sequence loads its inputs
    once, a tile that crosses from one sequence into the next (or ends the step) takes the rows one by one.  Both
    must give the same sums; the second step continues from the state the first left."""
    from kvforge_b200 import ops

    dev, dt = "cuda", DT[dtype]
    c = 72
    g = torch.Generator().manual_seed(taps)
    w = torch.randn(c, taps, generator=g)
    lens = [(701, 38), (9, 5), (602, 0), (3, 30)]
    seqs = [torch.randn(a + b, c, generator=g).to(dt).float() for a, b in lens]
    want = [plain.short_conv(u.double(), w.double()) for u in seqs]
    state = torch.zeros(5, (taps - 1) * c, device=dev)
    got = [[] for _ in seqs]
    for step in range(2):
        ls = [ab[step] for ab in lens]
        x = torch.cat([u[: ls[i]] if step == 0 else u[lens[i][0] :] for i, u in enumerate(seqs)]).to(dev, dt)
        qsl, sl = flat_batch(ls, [3, 0, 4, 1], dev)
        out = torch.empty_like(x)
        ops.causal_conv(x, w.to(dev), state, qsl, sl, 4, out)
        o = 0
        for i in range(4):
            got[i].append(out[o : o + ls[i]].float().cpu())
            o += ls[i]
    tol = 1e-5 if dtype == "float32" else 2e-2
    for i in range(4):
        assert torch.allclose(torch.cat(got[i]).double(), want[i], atol=tol, rtol=tol)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("h,g,dk,dv,channel", [(4, 2, 16, 8, False), (3, 3, 24, 40, True), (2, 1, 64, 32, True), (2, 2, 128, 128, False), (1, 1, 8, 300, True)])
def test_gated_delta_rule_through_the_state(dtype, h, g, dk, dv, channel):
    """Two sequences cut into steps (single tokens among them) against the rule applied token by token to
    whole sequences; unit norms, beta and the decay are computed by the kernel from their inputs."""
    from kvforge_b200 import ops

    dev, dt = "cuda", DT[dtype]
    gen = torch.Generator().manual_seed(dk + dv)
    lens = (37, 12)
    aw = h * dk if channel else h
    a_log, dt_bias = 0.5 * torch.randn(h, generator=gen), 0.5 * torch.randn(aw, generator=gen)
    seqs = []
    for n in lens:
        qkv = torch.randn(n, 2 * g * dk + h * dv, generator=gen).to(dt).float()
        seqs.append((qkv, torch.randn(n, h, generator=gen), torch.randn(n, aw, generator=gen)))
    want = []
    for qkv, b, a in seqs:
        n = qkv.shape[0]
        q = plain.unit(qkv[:, : g * dk].double().view(n, g, dk)) * dk**-0.5
        k = plain.unit(qkv[:, g * dk : 2 * g * dk].double().view(n, g, dk))
        v = qkv[:, 2 * g * dk :].double().view(n, h, dv)
        rep = h // g
        step = F.softplus((a + dt_bias).double())
        decay = torch.exp(-torch.exp(a_log.double()).repeat_interleave(dk if channel else 1) * step)
        decay = decay.view(n, h, dk) if channel else decay
        want.append(plain.delta_rule(q.repeat_interleave(rep, 1), k.repeat_interleave(rep, 1), v, torch.sigmoid(b.double()), decay).reshape(n, h * dv))
    state = torch.zeros(3, 5 + h * dk * dv, device=dev)
    cuts = [[1, 20, 1, 15], [4, 0, 7, 1]]
    got = [[], []]
    at = [0, 0]
    for step in range(4):
        ls = [cuts[i][step] for i in range(2)]
        cat = lambda j: torch.cat([seqs[i][j][at[i] : at[i] + ls[i]] for i in range(2)])  # noqa: E731
        qkv = cat(0).to(dev, dt)
        b, a = cat(1).to(dev), cat(2).to(dev)
        qsl, sl = flat_batch(ls, [2, 0], dev)
        out = torch.empty(sum(ls), h * dv, device=dev)
        extra = {}
        if step % 2 == 1 and not channel:
            # the logits as three float slices that sum to them (what a product over slices of K leaves)
            both = torch.cat([b, a], dim=1)
            parts = torch.randn(3, *both.shape, device=dev)
            parts[0] = both - parts[1] - parts[2]
            b, a = parts[0][:, :h], parts[0][:, h:]
            extra = dict(logit_slices=3, logit_slice_stride=parts.stride(0))
        ops.gated_delta(
            qkv[:, : g * dk], qkv[:, g * dk : 2 * g * dk], qkv[:, 2 * g * dk :], b, a, a_log.to(dev), dt_bias.to(dev), state[:, 5:], out,
            qsl, sl, 2, h, g, dk, dv, q_scale=dk**-0.5, max_query_len=max(ls) if step >= 2 else 0, **extra,
        )  # fmt: skip
        o = 0
        for i in range(2):
            got[i].append(out[o : o + ls[i]].cpu())
            o += ls[i]
            at[i] += ls[i]
    for i in range(2):
        assert torch.allclose(torch.cat(got[i]).double(), want[i], atol=5e-5, rtol=5e-4)
    assert float(state[1].abs().max()) == 0 and float(state[:, :5].abs().max()) == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_gated_head_norm_and_branch_mean(dtype):
    from kvforge_b200 import ops

    dev, dt = "cuda", DT[dtype]
    gen = torch.Generator().manual_seed(2)
    n, h, dv, width = 19, 3, 24, 72
    o = torch.randn(n, h * dv, generator=gen)
    gate = torch.randn(n, h * dv, generator=gen).to(dt).float()
    w = 1 + 0.3 * torch.randn(dv, generator=gen)
    tol = 1e-5 if dtype == "float32" else 2e-2
    for act, fn in (("silu", F.silu), ("sigmoid", torch.sigmoid)):
        out = torch.empty(n, h * dv, device=dev, dtype=dt)
        ops.gated_head_norm(o.to(dev), gate.to(dev, dt), w.to(dev), 1e-5, out, h, dv, activation=act)
        want = (plain.rms_norm(o.double().view(n, h, dv), w.double(), 1e-5) * fn(gate.double().view(n, h, dv))).view(n, h * dv)
        assert torch.allclose(out.float().cpu().double(), want, atol=tol, rtol=tol)
    ys = [torch.randn(n, width, generator=gen).to(dt).float() for _ in range(2)]
    parts = torch.randn(3, n, width, generator=gen)
    ws = [1 + 0.3 * torch.randn(width, generator=gen) for _ in range(3)]
    out = torch.empty(n, width, device=dev, dtype=dt)
    ops.branch_norm_mean([ys[0].to(dev, dt), ops.Partials(parts.to(dev)), ys[1].to(dev, dt)], [x.to(dev) for x in ws], 1e-6, out)
    want = sum(plain.rms_norm(y.double(), x.double(), 1e-6) for y, x in zip([ys[0], parts.sum(0), ys[1]], ws)) / 3
    assert torch.allclose(out.float().cpu().double(), want, atol=tol, rtol=tol)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("s", [1, 2, 4, 5])
def test_stream_step(dtype, s):
    """A pending write moves the streams on and the next read is normed, in one kernel; the gather before the
    output head leaves the streams alone."""
    from kvforge_b200 import ops

    dev, dt = "cuda", DT[dtype]
    gen = torch.Generator().manual_seed(s)
    n, w = 11, 56
    x = torch.randn(n, s, w, generator=gen)
    y = torch.randn(n, w, generator=gen).to(dt).float()
    mix, ow, rd = torch.randn(s, s, generator=gen), torch.randn(s, generator=gen), torch.randn(s, generator=gen)
    nw = 1 + 0.2 * torch.randn(w, generator=gen)
    new = torch.einsum("st,nsw->ntw", mix.double(), x.double()) + ow.double()[None, :, None] * y.double()[:, None, :]
    tol = 1e-5 if dtype == "float32" else 2e-2
    streams = x.reshape(n, s * w).to(dev)
    out = torch.empty(n, w, device=dev, dtype=dt)
    ops.stream_step(streams, ops.StreamWrite(y.to(dev, dt), mix.to(dev), ow.to(dev)), rd.to(dev), nw.to(dev), out, 1e-6, s)
    assert torch.allclose(streams.cpu().double().view(n, s, w), new, atol=1e-5, rtol=1e-5)
    want = plain.rms_norm(torch.einsum("t,ntw->nw", rd.double(), new), nw.double(), 1e-6)
    assert torch.allclose(out.float().cpu().double(), want, atol=tol, rtol=tol)
    # the final read: the plain sum of the streams after a pending write of split-K slices, two rows gathered
    parts = torch.randn(2, n, w, generator=gen)
    before = streams.clone()
    rows = torch.tensor([7, 2], dtype=torch.int32, device=dev)
    out2 = torch.empty(2, w, device=dev, dtype=dt)
    ops.stream_step(streams, ops.StreamWrite(ops.Partials(parts.to(dev)), mix.to(dev), ow.to(dev)), None, nw.to(dev), out2, 1e-6, s, rows=rows)
    assert torch.equal(streams, before)
    new2 = torch.einsum("st,nsw->ntw", mix.double(), new) + ow.double()[None, :, None] * parts.sum(0).double()[:, None, :]
    want2 = plain.rms_norm(new2.sum(1), nw.double(), 1e-6)[[7, 2]]
    assert torch.allclose(out2.float().cpu().double(), want2, atol=tol * 3, rtol=tol * 3)
    rep = torch.empty(n, s * w, device=dev)
    ops.replicate_streams(x[:, 0].contiguous().to(dev), rep, s)
    assert torch.equal(rep.view(n, s, w).cpu(), x[:, :1].expand(n, s, w))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("interleaved,rot", [(True, 8), (True, 24), (False, 16), (True, 0)])
def test_general_rotation_and_cache_write(dtype, interleaved, rot):
    from kvforge_b200 import ops

    dev, dt = "cuda", DT[dtype]
    gen = torch.Generator().manual_seed(rot + 1)
    n, nh, nkv, dk, dv, bs, blocks = 13, 4, 2, 24, 40, 4, 9
    qkv = torch.randn(n, (nh + nkv) * dk + nkv * dv, generator=gen).to(dt).float()
    pos = torch.tensor([0, 1, 2, 3, 4, 5, 90, 91, 1000, 1001, 7, 8, 9], dtype=torch.int32)
    slots = torch.tensor([3, 0, 35, 12, 13, 14, 15, 20, 21, 22, -1, 30, 31], dtype=torch.int32)
    f = plain.rotary_frequencies(rot, 100.0, None).float() if rot else torch.empty(0)
    x = qkv[:, : (nh + nkv) * dk].double().view(n, nh + nkv, dk)
    if not rot:
        turned = x
    elif interleaved:
        turned = plain.rotate_interleaved(x, pos, f.double())
    else:
        ang = pos.double()[:, None] * f.double()[None]
        c, s = ang.cos()[:, None], ang.sin()[:, None]
        a, b = x[..., : rot // 2], x[..., rot // 2 : rot]
        turned = torch.cat([a * c - b * s, b * c + a * s, x[..., rot:]], dim=-1)
    kc = torch.zeros(blocks, nkv, bs, dk, device=dev, dtype=dt)
    vc = torch.zeros(blocks, nkv, bs, dv, device=dev, dtype=dt)
    buf = qkv.to(dev, dt)
    ops.rope_cache_general(buf, pos.to(dev), f.to(dev), interleaved, slots.to(dev), kc, vc, nh, nkv, dk, dv, bs)
    tol = 5e-4 if dtype == "float32" else 3e-2  # angles of a thousand radians in 32-bit
    assert torch.allclose(buf[:, : nh * dk].float().cpu().double().view(n, nh, dk), turned[:, :nh], atol=tol, rtol=tol)
    v = qkv[:, (nh + nkv) * dk :].view(n, nkv, dv)
    for i in range(n):
        sl = int(slots[i])
        if sl < 0:
            continue
        assert torch.allclose(kc[sl // bs, :, sl % bs].float().cpu().double(), turned[i, nh:], atol=tol, rtol=tol)
        assert torch.equal(vc[sl // bs, :, sl % bs].float().cpu(), v[i])
    assert float(kc.float().abs().sum(-1).gt(0).sum()) == 12 * nkv
