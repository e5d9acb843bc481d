"""Reravik on the device against its plain implementation (tests/plain/reravik_plain.py), on small configurations
with random weights made here (tests/reravik_cases.py), in both precisions:

* every mechanism alone, on its kernel: layer norm, token shift with its carried row, the joined norm-add-norm,
  the gated recurrence (walked and tile-parallel), the sinusoidal embedding, the tanh-GELU gate, the per-head maps,
  and the latent attention with crafted scores at the edges of its window and of the cache's pages;
* whole prompts; a prompt followed by token-by-token decoding across page borders and window edges; prompts cut
  into portions of many sizes down to two tokens; batches of unequal requests against each alone; slots, pages
  and per-sequence state that are freed and used again; long decoding with a windowed cache that gives pages back;
* greedy generation through ``LLM`` and its scheduler with and without CUDA graphs, the command line, and the
  replay program.
"""
import json
import math
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from tests import reravik_cases as cases
from tests.plain import reravik_plain as plain

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
DTYPES = ["float32", "bfloat16"]


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    made = {}

    def get(name: str, seed: int = 11):
        key = (name, seed)
        if key not in made:
            cfg = cases.CONFIGS[name]()
            w = cases.random_weights(cfg, seed)
            made[key] = (cases.write_folder(cfg, w, str(tmp_path_factory.mktemp(f"reravik-{name}-{seed}"))), cfg, w)
        return made[key]
    return get


_plain = {}


def plain_logits(cfg, w, ids, key):
    k = (key, tuple(ids))
    if k not in _plain:
        _plain[k] = plain.forward(cfg, w, ids)
    return _plain[k]


def make_stepper(folder, dtype, max_tokens=64 * 40, chunk_tokens=2048, n_slots=None):
    from cpmcu_b200.cache import Cache
    from cpmcu_b200.engine.step import Stepper
    from cpmcu_b200.loading import load_model

    _, _, model = load_model(folder, dtype)
    cache = Cache(model.cache_needs(), max_tokens=max_tokens, dtype=DT[dtype], device="cuda:0", n_slots=n_slots,
                  max_step_tokens=chunk_tokens)
    return Stepper(model, cache, chunk_tokens=chunk_tokens)


def run_portions(stepper, requests, portions):
    """Feeds request r its tokens in portions[r] (a list of sizes that add up to its length), step k taking the k-th
    portion of every request that still has one, all as one batch; returns the logits of every position."""
    from cpmcu_b200.engine.step import SequenceStep

    slots = stepper.open(len(requests))
    at = [0] * len(requests)
    out = [[] for _ in requests]
    for k in range(max(len(p) for p in portions)):
        batch, who = [], []
        for r, ids in enumerate(requests):
            if k < len(portions[r]):
                n = portions[r][k]
                batch.append(SequenceStep(slots[r], ids[at[r]:at[r] + n], list(range(n))))
                who.append((r, n))
                at[r] += n
        logits = stepper.step(batch)
        o = 0
        for r, n in who:
            out[r].append(logits[o:o + n].clone())
            o += n
        for r, _ in who:
            if at[r] == len(requests[r]) and slots[r] is not None:
                stepper.close(slots[r])
                slots[r] = None
    stepper.ops.raise_on_kernel_error()
    stepper.cache.check_consistent()
    return [torch.cat(x) for x in out]


def check(got, want, dtype, what=""):
    e = cases.row_errors(got, want)
    worst = int(e.argmax())
    assert float(e.max()) <= cases.TOL[dtype], f"{what}: row {worst} differs by {float(e.max()):.3e} (allowed {cases.TOL[dtype]})"


# ---------------------------------------------------------------------------
# whole models
# ---------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["a", "b", "c", "d"])
def test_whole_prompt(folders, name, dtype):
    folder, cfg, w = folders(name)
    ids = cases.random_ids(cfg["vocab"], 150, 1)
    st = make_stepper(folder, dtype)
    got = run_portions(st, [ids], [[150]])[0]
    check(got, plain_logits(cfg, w, ids, name), dtype, "whole prompt")
    # the first tokens of a sequence, alone: positions 0, 1, 2 with nothing before them
    for n in (1, 2, 3):
        check(run_portions(st, [ids[:n]], [[n]])[0], plain_logits(cfg, w, ids, name)[:n], dtype, f"first {n} tokens")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["a", "b", "d"])
def test_prompt_then_token_by_token_across_pages_and_windows(folders, name, dtype):
    """A prompt of 50 tokens, then 150 single tokens: the decoded tokens cross the page borders at 64, 128 and 192
    and, in configuration a, the edges of windows of 37 and 70 keys, inside a page and across one."""
    folder, cfg, w = folders(name)
    ids = cases.random_ids(cfg["vocab"], 200, 2)
    st = make_stepper(folder, dtype)
    got = run_portions(st, [ids], [[50] + [1] * 150])[0]
    check(got, plain_logits(cfg, w, ids, name), dtype, "prompt then decode")


@pytest.mark.parametrize("dtype", DTYPES)
def test_token_by_token_from_the_first_token(folders, dtype):
    folder, cfg, w = folders("a")
    ids = cases.random_ids(cfg["vocab"], 90, 3)
    got = run_portions(make_stepper(folder, dtype), [ids], [[1] * 90])[0]
    check(got, plain_logits(cfg, w, ids, "a"), dtype, "decode from the first token")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("cuts", [[2] * 40 + [70], [63, 1, 64, 2, 20], [33, 32, 31, 3, 51], [64, 64, 22], [149, 1]])
def test_portions_of_a_prompt(folders, dtype, cuts):
    folder, cfg, w = folders("a")
    ids = cases.random_ids(cfg["vocab"], 150, 4)
    assert sum(cuts) == 150
    got = run_portions(make_stepper(folder, dtype), [ids], [cuts])[0]
    check(got, plain_logits(cfg, w, ids, "a"), dtype, f"portions {cuts[:5]}")


@pytest.mark.parametrize("dtype", DTYPES)
def test_step_function_cuts_long_steps_into_chunks(folders, dtype):
    """One step of 150 tokens through a step function whose forward passes take at most 48 packed tokens: a sequence
    continues in the next chunk, and the windowed lanes give pages back between the chunks."""
    folder, cfg, w = folders("a")
    reqs = [cases.random_ids(cfg["vocab"], n, 40 + n) for n in (150, 20, 77)]
    st = make_stepper(folder, dtype, chunk_tokens=48)
    got = run_portions(st, reqs, [[150], [20], [77]])
    for ids, g in zip(reqs, got):
        check(g, plain_logits(cfg, w, ids, "a"), dtype, "chunks of 48")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["a", "b"])
def test_batches_of_unequal_requests(folders, name, dtype):
    """Requests of 1, 2, 65, 130 and 40 tokens start together (the last 4 tokens of each decoded one by one, so the
    batch shrinks as the shorter ones end) and give what each gives alone."""
    folder, cfg, w = folders(name)
    lens = [5, 6, 69, 134, 44]
    reqs = [cases.random_ids(cfg["vocab"], n, 10 + n) for n in lens]
    st = make_stepper(folder, dtype)
    together = run_portions(st, reqs, [[n - 4, 1, 1, 1, 1] for n in lens])
    for ids, g in zip(reqs, together):
        check(g, plain_logits(cfg, w, ids, name), dtype, "in a batch")
    alone = [run_portions(st, [ids], [[len(ids) - 4, 1, 1, 1, 1]])[0] for ids in reqs]
    for g, a in zip(together, alone):
        assert float(cases.row_errors(g, a).max()) <= cases.TOL[dtype] / 3       # a batch changes nothing but rounding


@pytest.mark.parametrize("dtype", DTYPES)
def test_slots_pages_and_state_are_used_again(folders, dtype):
    """A cache of two slots and few pages serves nine requests one after another and in pairs: every slot, every
    page and every per-sequence state tensor is used again with what the last sequence left in it."""
    folder, cfg, w = folders("a")
    st = make_stepper(folder, dtype, max_tokens=64 * 6, n_slots=2)
    for round_no in range(3):
        reqs = [cases.random_ids(cfg["vocab"], n, 100 + 7 * round_no + n) for n in (130, 9, 70)]
        got = run_portions(st, reqs[:2], [[100] + [1] * 30, [9]])
        got.append(run_portions(st, [reqs[2]], [[3, 67]])[0])
        for ids, g in zip(reqs, got):
            check(g, plain_logits(cfg, w, ids, "a"), dtype, "reused slot")
        assert st.cache.slots.n_held == 0 and all(g.pages.n_held == 0 for g in st.cache.groups)


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding_in_a_small_windowed_cache(folders, dtype):
    """400 decoded tokens: the windowed lanes hold at most their window's pages and hand the others back on the way."""
    folder, cfg, w = folders("a")
    ids = cases.random_ids(cfg["vocab"], 420, 5)
    st = make_stepper(folder, dtype, max_tokens=64 * 8)
    from cpmcu_b200.engine.step import SequenceStep
    slot = st.open(1)[0]
    rows = [st.step([SequenceStep(slot, ids[:20], list(range(20)))])]
    for t in range(20, 420):
        rows.append(st.step([SequenceStep(slot, [ids[t]], [0])]))
    windowed = [g for g in st.cache.groups if g.needs.window]
    assert windowed and all(g.pages_held(slot) <= 3 for g in windowed)
    st.close(slot)
    check(torch.cat(rows), plain_logits(cfg, w, ids, "a"), dtype, "long decode")


# ---------------------------------------------------------------------------
# through the library's own entry points
# ---------------------------------------------------------------------------

@pytest.mark.parametrize("graph", [False, True])
def test_greedy_generation_through_llm(folders, graph):
    """fp32: the tokens of the plain implementation for a batch of unequal prompts (positions where the two best
    logits nearly tie are where a comparison stops), twice in a row so that slots and state are used again; prompts
    go through chunks of 16 tokens, which the graph variant records and replays."""
    from cpmcu_b200 import LLM

    folder, cfg, w = folders("a")
    llm = LLM(folder, dtype="float32", cuda_graph=graph, max_tokens=64 * 16, chunk_length=16)
    prompts = [cases.random_ids(cfg["vocab"], n, 60 + n) for n in (41, 3, 70)]
    want = [plain.greedy(cfg, w, p, 12) for p in prompts]
    for _ in range(2):
        res = llm.generate_batch(prompts, generation_length=12)
        compared = 0
        for r, (tokens, gaps) in zip(res, want):
            firm = next((i for i, g in enumerate(gaps) if g < 1e-3), len(tokens))
            assert r.tokens[:firm] == tokens[:firm]
            compared += firm
        assert compared >= 30


def test_bfloat16_generation_with_graphs_matches_eager(folders):
    from cpmcu_b200 import LLM

    folder, cfg, w = folders("a")
    prompts = [cases.random_ids(cfg["vocab"], n, 80 + n) for n in (33, 90)]
    outs = []
    for graph in (False, True):
        llm = LLM(folder, dtype="bfloat16", cuda_graph=graph, max_tokens=64 * 16, chunk_length=32)
        outs.append([r.tokens for r in llm.generate_batch(prompts, generation_length=10)])
    want = [plain.greedy(cfg, w, p, 10) for p in prompts]
    for eager, graphed, (tokens, gaps) in zip(outs[0], outs[1], want):
        firm = next((i for i, g in enumerate(gaps) if g < 0.05), len(tokens))
        assert eager[:firm] == tokens[:firm] and graphed[:firm] == tokens[:firm]


def test_command_line_and_replay(folders, tmp_path):
    folder, cfg, w = folders("b")
    ids = cases.random_ids(cfg["vocab"], 30, 9)
    env = dict(os.environ, PYTHONPATH=ROOT)
    p = subprocess.run([sys.executable, "-m", "cpmcu_b200.cli", "--model-path", folder, "--dtype", "float32",
                        "--prompt-ids", ",".join(map(str, ids)), "--num-generate", "6", "--max-tokens", "512"],
                       capture_output=True, text=True, env=env, cwd=ROOT, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    tokens, gaps = plain.greedy(cfg, w, ids, 6)
    firm = next((i for i, g in enumerate(gaps) if g < 1e-3), 6)
    assert firm >= 1 and " ".join(map(str, tokens[:firm])) in p.stdout.replace(",", " ").replace("  ", " ")
    # replay: a prompt in two portions, then a single token, logits at chosen places
    out = tmp_path / "out"
    steps = [{"step": 0, "entries": [{"id": "r", "tokens": ids[:17], "want": [0, 16]}], "end": []},
             {"step": 1, "entries": [{"id": "r", "tokens": ids[17:29], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "r", "tokens": ids[29:], "want": [0]}], "end": ["r"]}]
    p = subprocess.run([os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", "float32", "--out", str(out),
                        "--max-tokens", "256"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                       capture_output=True, text=True, env=env, cwd=ROOT, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [l for l in p.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2"]
    want = plain_logits(cfg, w, ids, "b")
    got0 = torch.from_numpy(np.fromfile(out / "0.f32", dtype="<f4")).view(2, -1)
    got2 = torch.from_numpy(np.fromfile(out / "2.f32", dtype="<f4")).view(1, -1)
    assert not (out / "1.f32").exists()
    check(got0, want[[0, 16]], "float32", "replay")
    check(got2, want[[29]], "float32", "replay")


def test_replay_of_many_short_requests_in_a_cache_sized_by_their_tokens(folders, tmp_path):
    """Twenty requests of three and four tokens in one batch, then one more token each, with ``--max-tokens`` set to the
    tokens they hold together: every request fills a small part of a page of its own."""
    folder, cfg, w = folders("c")
    reqs = [cases.random_ids(cfg["vocab"], 4 + (i % 2), 200 + i) for i in range(20)]
    steps = [{"step": 0, "entries": [{"id": f"q{i}", "tokens": r[:-1], "want": [len(r) - 2]} for i, r in enumerate(reqs)], "end": []},
             {"step": 1, "entries": [{"id": f"q{i}", "tokens": r[-1:], "want": [0]} for i, r in enumerate(reqs)],
              "end": [f"q{i}" for i in range(20)]}]
    out = tmp_path / "out"
    p = subprocess.run([os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", "bfloat16", "--out", str(out),
                        "--max-tokens", str(sum(len(r) for r in reqs))], input="\n".join(json.dumps(s) for s in steps) + "\n",
                       capture_output=True, text=True, env=dict(os.environ, PYTHONPATH=ROOT), cwd=ROOT, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    for step, at in ((0, -2), (1, -1)):
        got = torch.from_numpy(np.fromfile(out / f"{step}.f32", dtype="<f4")).view(20, -1)
        want = torch.stack([plain_logits(cfg, w, r, "c")[at] for r in reqs])
        check(got, want, "bfloat16", f"replay step {step}")


# ---------------------------------------------------------------------------
# mechanisms alone
# ---------------------------------------------------------------------------

def _ctx(q_lens, starts, slots, tiles=True):
    """A step's description on the device for sequences that bring ``q_lens`` tokens from positions ``starts``."""
    from cpmcu_b200.parts.base import QUERY_TILE_TOKENS, StepContext

    i32 = dict(dtype=torch.int32, device="cuda")
    pos = torch.cat([torch.arange(s, s + n) for n, s in zip(q_lens, starts)]).to(**i32)
    seq = torch.cat([torch.full((n,), i) for i, n in enumerate(q_lens)]).to(**i32)
    cu = torch.tensor([0] + list(np.cumsum(q_lens)), **i32)
    ctx = StepContext(n_tokens=sum(q_lens), n_seqs=len(q_lens), is_decode=all(n == 1 for n in q_lens), captured=False,
                      q_lens=list(q_lens), kv_lens=[s + n for n, s in zip(q_lens, starts)], slots=list(slots),
                      max_q_len=max(q_lens), max_kv_len=max(s + n for n, s in zip(q_lens, starts)),
                      token_ids=torch.zeros(sum(q_lens), **i32), positions=pos, token_seq=seq, cu_q=cu,
                      kv_len_dev=torch.tensor([s + n for n, s in zip(q_lens, starts)], **i32),
                      slot_dev=torch.tensor(list(slots), **i32))
    if tiles:
        ts = [i for i, n in enumerate(q_lens) for _ in range(0, n, QUERY_TILE_TOKENS)]
        trow = [r for n in q_lens for r in range(0, n, QUERY_TILE_TOKENS)]
        ctx.q_tiles = (torch.tensor(ts, **i32), torch.tensor(trow, **i32), len(ts))
    return ctx


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden", [96, 50, 1030])
def test_layer_norm_kernels(dtype, hidden):
    from cpmcu_b200.ops.ops import Ops

    ops = Ops(DT[dtype])
    g = torch.Generator().manual_seed(hidden)
    x = (torch.randn(21, hidden, generator=g) * 3 + 1.5).cuda()
    w, b, w2, b2, mix = [(torch.randn(hidden, generator=g) * s + o).cuda() for s, o in ((0.3, 1), (0.3, 0), (0.3, 1), (0.3, 0), (0.4, 0.5))]
    tol = 1e-5 if dtype == "float32" else 2e-2
    want = plain.layer_norm(x.double().cpu(), w.double().cpu(), b.double().cpu(), 1e-5)
    rows = torch.tensor([20, 0, 7], dtype=torch.int32, device="cuda")
    assert (ops.layernorm(x, w, b, 1e-5).double().cpu() - want).abs().max() < tol * 4
    assert (ops.layernorm(x, w, b, 1e-5, rows).double().cpu() - want[[20, 0, 7]]).abs().max() < tol * 4
    # token shift: three sequences (one continues from a carried row, one starts at position 0 in a slot that still
    # holds another sequence's row, one brings a single token), state of 5 slots
    q_lens, starts, slots = [9, 11, 1], [4, 0, 6], [3, 1, 0]
    ctx = _ctx(q_lens, starts, slots)
    state = torch.randn(5, hidden, generator=g).cuda()
    before = state.clone()
    y = ops.layernorm_shift(ctx, x, w, b, 1e-5, mix, state).double().cpu()
    h, o = want, 0
    for n, s0, slot in zip(q_lens, starts, slots):
        prev = torch.cat([(before[slot].double().cpu() if s0 > 0 else torch.zeros(hidden, dtype=torch.float64))[None], h[o:o + n - 1]])
        assert (y[o:o + n] - (h[o:o + n] + (prev - h[o:o + n]) * mix.double().cpu())).abs().max() < tol * 6
        assert (state[slot].double().cpu() - h[o + n - 1]).abs().max() < 1e-5
        o += n
    assert torch.equal(state[[2, 4]], before[[2, 4]])
    # x += norm(a), then another norm of the new x
    a = (torch.randn(21, hidden, generator=g) * 2).cuda().to(DT[dtype])
    x2 = x.clone()
    y2 = ops.post_norm_add(x2, a, w, b, 1e-5, (w2, b2))
    nx = x.double().cpu() + plain.layer_norm(a.double().cpu(), w.double().cpu(), b.double().cpu(), 1e-5)
    assert (x2.double().cpu() - nx).abs().max() < 1e-5 * 4
    assert (y2.double().cpu() - plain.layer_norm(nx, w2.double().cpu(), b2.double().cpu(), 1e-5)).abs().max() < tol * 4
    x3 = x.clone()
    assert ops.post_norm_add(x3, a, w, b, 1e-5) is None and torch.equal(x3, x2)
    ops.stream_inject(x3, x, w)
    assert torch.allclose(x3, x2 + x + w)


@pytest.mark.parametrize("dtype", DTYPES)
def test_recurrence_walked_and_tile_parallel(dtype):
    """Both forms of the scan against the plain recurrence: sequences of 1 to 300 tokens, one of them continuing from
    a carried state, one starting at position 0 in a slot that holds another sequence's state."""
    from cpmcu_b200.ops.ops import Ops

    ops = Ops(DT[dtype])
    width = 72
    g = torch.Generator().manual_seed(1)
    q_lens, starts, slots = [300, 1, 65, 64, 130], [0, 5, 7, 0, 64], [2, 0, 4, 1, 3]
    n = sum(q_lens)
    proj = (torch.randn(n, 3 * width, generator=g) * 2).cuda()
    bz, bx = torch.randn(width, generator=g).cuda(), torch.randn(width, generator=g).cuda()
    state0 = torch.rand(6, width, generator=g).cuda()
    outs = []
    for tiles in (False, True):
        ctx = _ctx(q_lens, starts, slots, tiles=tiles)
        state = state0.clone()
        outs.append((ops.mingru_scan(ctx, proj, bz, bx, state, width).double().cpu(), state.double().cpu()))
    P = proj.double().cpu()
    o = 0
    for ln, s0, slot in zip(q_lens, starts, slots):
        S = state0[slot].double().cpu() if s0 > 0 else torch.zeros(width, dtype=torch.float64)
        for t in range(o, o + ln):
            z = torch.sigmoid(P[t, :width] + bz.double().cpu())
            u = P[t, width:2 * width] + bx.double().cpu()
            S = (1 - z) * S + z * torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
            gate = P[t, 2 * width:]
            want = S * gate * torch.sigmoid(gate)
            for out, _ in outs:
                assert ((out[t] - want).abs() / (1 + want.abs())).max() < (1e-5 if dtype == "float32" else 1e-2)
        for _, st in outs:
            assert (st[slot] - S).abs().max() < 1e-5
        o += ln
    assert torch.equal(outs[0][1][5], state0[5].double().cpu()) and torch.equal(outs[1][1][5], state0[5].double().cpu())


@pytest.mark.parametrize("dtype", DTYPES)
def test_embedding_gate_and_head_maps(dtype):
    from cpmcu_b200.ops.ops import Ops

    ops = Ops(DT[dtype])
    g = torch.Generator().manual_seed(2)
    table = torch.randn(50, 40, generator=g).to(DT[dtype]).cuda()
    ids = torch.tensor([3, 49, 0, 3], dtype=torch.int32, device="cuda")
    pos = torch.tensor([0, 1, 777, 4095], dtype=torch.int32, device="cuda")
    freq = torch.pow(torch.tensor(10000.0), -2.0 * torch.arange(20, dtype=torch.float32) / 40).cuda()
    got = ops.embed_sinusoid(ids, pos, table, freq, 2.5).double().cpu()
    want = table.double().cpu()[ids.cpu().long()] * 2.5
    pv = torch.stack([plain.position_vectors(1, 40, first=int(p))[0] for p in pos.cpu()])
    assert (got - (want + pv)).abs().max() < 5e-4                        # fp32 angles of thousands of radians
    gu = (torch.randn(9, 2 * 24, generator=g) * 2).to(DT[dtype]).cuda()
    z, u = gu.double().cpu()[:, :24], gu.double().cpu()[:, 24:]
    tol = 1e-5 if dtype == "float32" else 1e-2

    def close(got, want):
        return float(((got.double().cpu() - want).abs() / (1 + want.abs())).max()) < tol

    assert close(ops.act_mul(gu, 0, 1), plain.gelu_tanh(z) * u)
    assert close(ops.act_mul(gu, 0, 0), z * torch.sigmoid(z) * u)
    il = gu.view(9, 2, 3, 8).transpose(1, 2).reshape(9, 48).contiguous()          # blocks of 8 gate, 8 up
    assert torch.equal(ops.act_mul(il, 8, 1), ops.act_mul(gu, 0, 1))
    x = torch.randn(11, 3, 20, generator=g).cuda()
    wm = torch.randn(3, 20, 13, generator=g).to(DT[dtype]).cuda()
    ref = torch.einsum("thk,hkn->thn", x.double().cpu(), wm.double().cpu())
    assert (ops.head_project(x, wm, 3, out_f32=True).double().cpu() - ref).abs().max() < 1e-4
    xt = x.to(DT[dtype]).contiguous()
    ref = torch.einsum("thk,hkn->thn", xt.double().cpu(), wm.double().cpu())
    assert close(ops.head_project(xt.view(11, 60), wm, 3, out_f32=False), ref)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rank,window", [(48, 37), (72, 64), (160, 65), (512, 0), (600, 130)])
def test_latent_attention_sees_exactly_its_window(dtype, rank, window):
    """Crafted latents: all rows are small but one, whose score towers over the others.  Placed just inside the
    window (the oldest visible key), just outside it, far back, at the first and last row of a page and at the
    query's own place, it either takes the whole output or leaves no trace, for a query in a prompt and for the
    same query decoded alone, with the sequence's pages scattered over the cache."""
    from cpmcu_b200.cache import Cache
    from cpmcu_b200.ops.ops import Ops
    from cpmcu_b200.parts.base import CacheNeeds

    ops = Ops(DT[dtype])
    H, n, p = 3, 200, 199
    g = torch.Generator().manual_seed(rank)
    cache = Cache([CacheNeeds(kv_heads=1, head_dim=rank, window=None, values=False)], max_tokens=64 * 12, dtype=DT[dtype], device="cuda")
    spare = cache.open_sequence(); cache.reserve(spare, 70)
    slot = cache.open_sequence(); cache.reserve(slot, 64)
    other = cache.open_sequence(); cache.reserve(other, 130)
    cache.reserve(slot, n); cache.sync()                       # the sequence's pages are not neighbours
    lane = cache.lane(0)
    table = lane.page_table[slot].cpu()
    lo = max(0, p - window + 1) if window else 0
    spots = {"oldest visible": lo, "own": p, "page start": 128, "page end": 191, "first": 0}
    if window:
        spots["just outside"] = lo - 1
        spots["far back"] = 3
    q = torch.randn(H, rank, generator=g) * 0.05
    q[:, 0] = 4.0
    for what, j in spots.items():
        lat = torch.randn(n, rank, generator=g) * 0.05
        lat[j, 0] = 50.0                                           # score 200 * scale against about 0 elsewhere
        lat = lat.to(DT[dtype])
        for t in range(n):
            lane.k[int(table[t // 64]), 0, t % 64] = lat[t].cuda()
        seen = lo <= j <= p
        vis = lat.double()[lo:p + 1]
        pr = torch.softmax((q.double() @ vis.T) * 0.5, dim=-1)
        want = pr @ vis
        if seen:
            assert float(pr[:, j - lo].min()) > 0.999
        for q_len in (1, 70):                                      # decoded alone; the last of 70 prompt tokens
            ctx = _ctx([q_len], [p + 1 - q_len], [slot])
            ql = torch.zeros(q_len, H, rank); ql[-1] = q
            ways = [dict(tensor_cores=False)]
            if dtype == "bfloat16" and rank % 16 == 0:
                ways += [dict(tensor_cores=True, n_splits=1), dict(tensor_cores=True, n_splits=3), dict()]
            for way in ways:
                out = ops.latent_attention(ctx, ql.cuda().contiguous(), lane, 0.5, window, **way)[-1].double().cpu()
                # the tensor-core kernel rounds the query and the softmax weights to bfloat16
                assert (out - want).abs().max() < (2e-3 if not way.get("tensor_cores", way == {}) else 0.3), (what, q_len, way)
                assert (out[:, 0] > 40).all() if seen else (out[:, 0].abs() < 1).all(), (what, q_len, way)


@pytest.mark.parametrize("rank,heads,window", [(48, 3, 37), (256, 16, 0), (512, 20, 300), (160, 33, 129)])
def test_latent_attention_on_tensor_cores_against_the_fp32_kernel(rank, heads, window):
    """Random latents and queries; sequences whose queries sit at the start, across page borders and deep inside;
    the keys of a token in one block and shared out over 2, 5 and 16 blocks."""
    from cpmcu_b200.cache import Cache
    from cpmcu_b200.ops.ops import Ops
    from cpmcu_b200.parts.base import CacheNeeds

    ops = Ops(torch.bfloat16)
    g = torch.Generator().manual_seed(rank + heads)
    cache = Cache([CacheNeeds(kv_heads=1, head_dim=rank, window=None, values=False)], max_tokens=64 * 20, dtype=torch.bfloat16, device="cuda")
    q_lens, starts = [70, 1, 5, 1], [0, 0, 190, 500]
    slots = []
    for n, s0 in zip(q_lens, starts):
        slot = cache.open_sequence()
        cache.reserve(slot, s0 + n)
        slots.append(slot)
    cache.sync()
    lane = cache.lane(0)
    lane.k.copy_((torch.randn(lane.k.shape, generator=g) * 0.7).to(torch.bfloat16))
    ctx = _ctx(q_lens, starts, slots)
    q = torch.randn(sum(q_lens), heads, rank, generator=g).cuda()
    want = ops.latent_attention(ctx, q, lane, 0.11, window, tensor_cores=False)
    for n_splits in (1, 2, 5, 16, None):
        got = ops.latent_attention(ctx, q, lane, 0.11, window, n_splits=n_splits, tensor_cores=True)
        err = (got - want).abs().max() / want.abs().max()
        assert float(err) < 2e-2, (n_splits, float(err))


@pytest.mark.parametrize("rows", [3, 8, 12, 40, 300])
def test_gated_products_with_tanh_gelu(rows):
    """The gate_up product with the tanh form of GELU through every path the row count selects (the weight-streaming
    kernel, the tcgen05 kernel, the library product followed by the activation kernel) against fp64."""
    from cpmcu_b200.ops.ops import Ops

    ops = Ops(torch.bfloat16)
    g = torch.Generator().manual_seed(rows)
    K, inter = 128, 160 * 128                          # enough tiles for the tcgen05 path at 300 rows
    gate = (torch.randn(inter, K, generator=g) * 0.2).bfloat16()
    up = (torch.randn(inter, K, generator=g) * 0.2).bfloat16()
    w = torch.stack([gate.view(inter // 8, 8, K), up.view(inter // 8, 8, K)], dim=1).reshape(2 * inter, K).contiguous().cuda()
    a = torch.randn(rows, K, generator=g).bfloat16().cuda()
    want = plain.gelu_tanh(a.double().cpu() @ gate.double().T) * (a.double().cpu() @ up.double().T)
    got = ops.gated_linear(a, w, 8, 1).double().cpu()
    assert float(((got - want).abs() / (1 + want.abs())).max()) < 2e-2
    ops.raise_on_kernel_error()
