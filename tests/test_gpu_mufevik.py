"""Mufevik on the GPU against the plain implementation (tests/plain/mufevik_plain.py): every mechanism's kernels alone,
then whole models through the step function, the cache and state manager, the generation loop, the command line and
replay, in both precisions.

Schedules: whole prompts; a prompt, then token by token across page borders; decoding from the first token; prompts in
portions down to two tokens; steps cut into chunks; batches of unequal requests; slots, pages and state used again;
long decoding.  Mechanisms: a score that towers over the others at the first key, far back, on both sides of a page
border and at the query itself, with a larger one just after the query that must not be seen; head mixing; matrix
recurrences in one piece and in pieces; convolutions whose inputs come from the state; routing with negative choice
scores and groups; the experts' grouped products.
"""
from __future__ import annotations

import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from tests import mufevik_cases as cases
from tests.plain import mufevik_plain as plain

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
            made[key] = (cases.write_folder(cfg, w, str(tmp_path_factory.mktemp(f"mufevik-{name}-{seed}"))), cfg, w)
        return made[key]
    return get


def make_stepper(folder, dtype, max_tokens=64 * 40, chunk_tokens=2048, n_slots=None):
    from cpmcu_b200.cache import Cache
    from cpmcu_b200.engine.step import Stepper
    from cpmcu_b200.loading import load_model

    _, _, model = load_model(folder, dtype)
    cache = Cache(model.cache_needs(), max_tokens=max_tokens, dtype=DT[dtype], device="cuda:0", n_slots=n_slots,
                  max_step_tokens=chunk_tokens)
    return Stepper(model, cache, chunk_tokens=chunk_tokens)


def run_portions(stepper, requests, portions, n_moe=0):
    """Feeds request r its tokens in portions[r] (sizes that add up to its length), step k taking the k-th portion of
    every request that still has one, all as one batch.  Returns (logits of every position per request, the experts
    the engine chose per request: a list over the layers with experts of [tokens, top], when ``n_moe`` is given)."""
    from cpmcu_b200.engine.step import SequenceStep

    slots = stepper.open(len(requests))
    at = [0] * len(requests)
    out = [[] for _ in requests]
    chosen = [[[] for _ in range(n_moe)] for _ in requests]
    for k in range(max(len(p) for p in portions)):
        batch, who = [], []
        for r, ids in enumerate(requests):
            if k < len(portions[r]):
                n = portions[r][k]
                batch.append(SequenceStep(slots[r], ids[at[r]:at[r] + n], list(range(n))))
                who.append((r, n))
                at[r] += n
        stepper.taps = {"experts": []} if n_moe else None
        logits = stepper.step(batch)
        if n_moe:
            taps = stepper.taps["experts"]                   # chunk by chunk, layer by layer
            per_layer = [torch.cat(taps[i::n_moe]).cpu() for i in range(n_moe)]
        stepper.taps = None
        o = 0
        for r, n in who:
            out[r].append(logits[o:o + n].clone())
            for i in range(n_moe):
                chosen[r][i].append(per_layer[i][o:o + n])
            o += n
        for r, _ in who:
            if at[r] == len(requests[r]) and slots[r] is not None:
                stepper.close(slots[r])
                slots[r] = None
    stepper.ops.raise_on_kernel_error()
    stepper.cache.check_consistent()
    return [torch.cat(x) for x in out], [[torch.cat(c) for c in per] for per in chosen]


_plain = {}


def plain_logits(cfg, w, ids, key):
    k = (key, tuple(ids))
    if k not in _plain:
        _plain[k] = plain.forward(cfg, w, ids)
    return _plain[k]


def check(got, want, dtype, what=""):
    e = cases.row_errors(got, want)
    worst = int(e.argmax())
    assert float(e.max()) <= cases.TOL[dtype], f"{what}: row {worst} differs by {float(e.max()):.3e} (allowed {cases.TOL[dtype]})"
    if e.numel() >= 20:
        assert float(e.median()) <= cases.MEDIAN_TOL[dtype], f"{what}: the median row differs by {float(e.median()):.3e}"


def run_and_check(stepper, cfg, w, key, requests, portions, dtype, what):
    """The plain implementation uses the experts the engine chose, which must lie within a small slack of the rule's
    cut-off (float32: a rounding error's worth) and differ from the rule's own choice for few tokens."""
    n_moe = cases.moe_layers(cfg)
    got, chosen = run_portions(stepper, requests, portions, n_moe)
    for r, ids in enumerate(requests):
        if n_moe:
            slack = []
            want = plain.forward(cfg, w, ids, forced=chosen[r], slack=slack)
            assert max(slack) <= cases.CHOICE_SLACK[dtype], f"{what}: a chosen expert lies {max(slack):.3e} below the cut-off"
            assert sum(1 for s in slack if s > 0) <= (0.1 if dtype == "bfloat16" else 0.01) * len(slack) + 1
        else:
            want = plain_logits(cfg, w, ids, key)
        check(got[r], want, dtype, f"{what}, request {r}")


# ---------------------------------------------------------------------------
# whole models
# ---------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["a", "b", "c", "d"])
def test_whole_prompt_and_first_tokens(folders, name, dtype):
    folder, cfg, w = folders(name)
    st = make_stepper(folder, dtype)
    reqs = [cases.random_ids(cfg["vocab"], n, 40 + n) for n in (150, 1, 2, 67)]
    for ids in reqs:
        run_and_check(st, cfg, w, name, [ids], [[len(ids)]], dtype, f"whole prompt of {len(ids)}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["a", "b", "d"])
def test_prompt_then_token_by_token_across_pages(folders, name, dtype):
    folder, cfg, w = folders(name)
    ids = cases.random_ids(cfg["vocab"], 210, 3)
    run_and_check(make_stepper(folder, dtype), cfg, w, name, [ids], [[60] + [1] * 150], dtype, "prompt then decode")


@pytest.mark.parametrize("dtype", DTYPES)
def test_token_by_token_from_the_first_token(folders, dtype):
    folder, cfg, w = folders("c")
    ids = cases.random_ids(cfg["vocab"], 70, 4)
    run_and_check(make_stepper(folder, dtype), cfg, w, "c", [ids], [[1] * 70], dtype, "decode from the start")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("cuts", [[2] * 40 + [70], [63, 1, 64, 2, 20], [33, 32, 31, 3, 51], [64, 64, 22], [149, 1], [1, 2, 147]])
def test_portions_of_a_prompt(folders, dtype, cuts):
    folder, cfg, w = folders("a")
    ids = cases.random_ids(cfg["vocab"], 150, 6)
    run_and_check(make_stepper(folder, dtype), cfg, w, "a", [ids], [cuts], dtype, f"portions {cuts[:4]}")


@pytest.mark.parametrize("dtype", DTYPES)
def test_step_function_cuts_long_steps_into_chunks(folders, dtype):
    folder, cfg, w = folders("d")
    reqs = [cases.random_ids(cfg["vocab"], n, 70 + n) for n in (130, 50, 3)]
    st = make_stepper(folder, dtype, chunk_tokens=48)
    run_and_check(st, cfg, w, "d", reqs, [[130], [50], [3]], dtype, "chunks of 48")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["a", "b", "d"])
def test_batches_of_unequal_requests(folders, name, dtype):
    folder, cfg, w = folders(name)
    reqs = [cases.random_ids(cfg["vocab"], n, 90 + n) for n in (100, 31, 66, 5)]
    portions = [[70] + [1] * 30, [21] + [1] * 10, [64, 2], [2] + [1] * 3]
    run_and_check(make_stepper(folder, dtype), cfg, w, name, reqs, portions, dtype, "batch")


@pytest.mark.parametrize("dtype", DTYPES)
def test_slots_pages_and_state_are_used_again(folders, dtype):
    """A cache of two slots and few pages serves nine requests one after another and in pairs: every slot, every page,
    every matrix state and every convolution state is used again with what the last sequence left in it."""
    folder, cfg, w = folders("a")
    st = make_stepper(folder, dtype, max_tokens=64 * 6, n_slots=2)
    for round_no in range(3):
        reqs = [cases.random_ids(cfg["vocab"], n, 100 + 7 * round_no + n) for n in (130, 9, 70)]
        run_and_check(st, cfg, w, "a", reqs[:2], [[100] + [1] * 30, [9]], dtype, "reused slots")
        run_and_check(st, cfg, w, "a", reqs[2:], [[3, 67]], dtype, "reused slots")
        assert st.cache.slots.n_held == 0 and all(g.pages.n_held == 0 for g in st.cache.groups)


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding(folders, dtype):
    folder, cfg, w = folders("b")
    ids = cases.random_ids(cfg["vocab"], 330, 5)
    run_and_check(make_stepper(folder, dtype, max_tokens=64 * 8), cfg, w, "b", [ids], [[10] + [1] * 320], dtype, "long decode")


# ---------------------------------------------------------------------------
# through the library's own entry points
# ---------------------------------------------------------------------------

@pytest.mark.parametrize("graph", [False, True])
def test_greedy_generation_through_llm(folders, graph):
    """fp32: the tokens of the plain implementation for a batch of unequal prompts (a comparison stops where the two
    best logits nearly tie), twice in a row so that slots and state are used again; prompts go through chunks of 16
    tokens, which the graph variant records and replays, and decoding through the decode runner."""
    from cpmcu_b200 import LLM

    folder, cfg, w = folders("a")
    llm = LLM(folder, dtype="float32", cuda_graph=graph, max_tokens=64 * 16, chunk_length=16)
    prompts = [cases.random_ids(cfg["vocab"], n, 60 + n) for n in (41, 3, 70)]
    want = [plain.greedy(cfg, w, p, 10) for p in prompts]
    for _ in range(2):
        res = llm.generate_batch(prompts, generation_length=10)
        compared = 0
        for r, (tokens, gaps) in zip(res, want):
            firm = next((i for i, g in enumerate(gaps) if g < 1e-3), len(tokens))
            assert r.tokens[:firm] == tokens[:firm]
            compared += firm
        assert compared >= 24


def test_bfloat16_generation_with_graphs_matches_eager(folders):
    from cpmcu_b200 import LLM

    folder, cfg, w = folders("d")
    prompts = [cases.random_ids(cfg["vocab"], n, 80 + n) for n in (33, 90)]
    outs = []
    for graph in (False, True):
        llm = LLM(folder, dtype="bfloat16", cuda_graph=graph, max_tokens=64 * 16, chunk_length=32)
        outs.append([r.tokens for r in llm.generate_batch(prompts, generation_length=10)])
    assert outs[0] == outs[1]


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


# ---------------------------------------------------------------------------
# mechanisms alone
# ---------------------------------------------------------------------------

def _ctx(q_lens, starts, slots):
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
    ts = [i for i, n in enumerate(q_lens) for _ in range(0, n, QUERY_TILE_TOKENS)]
    trow = [r for n in q_lens for r in range(0, n, QUERY_TILE_TOKENS)]
    ctx.q_tiles = (torch.tensor(ts, **i32), torch.tensor(trow, **i32), len(ts))
    return ctx


def _close(got, want, dtype, tol32=2e-5, tol16=2e-2):
    got, want = got.double().cpu(), want.double().cpu()
    err = float((got - want).abs().max() / want.abs().max().clamp_min(1e-30))
    assert err <= (tol32 if dtype == "float32" else tol16), err


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("S,W", [(1, 50), (3, 96), (16, 1030)])
def test_hyper_connection_kernel(dtype, S, W):
    from cpmcu_b200.ops.ops import Ops

    ops = Ops(DT[dtype])
    g = torch.Generator().manual_seed(S * W)
    T = 37
    x = torch.randn(T, S, W, generator=g)
    y = torch.randn(T, W, generator=g).to(DT[dtype])
    hw = {"in": torch.randn(S, generator=g), "out": torch.randn(S, generator=g), "mix": torch.randn(S, S, generator=g)}
    gain = torch.tensor([1.3])
    X = x.cuda().clone()
    dev = {k: v.cuda() for k, v in hw.items()}
    # read alone, write + read, write + sum
    h = ops.hyper_step(X, read=(dev["in"], gain.cuda()), eps=1e-5)
    want_h = plain.scalar_rms_norm(plain.hyper_read(x.double(), {k: v.double() for k, v in hw.items()}, ""), 1.3, 1e-5)
    _close(h, want_h, dtype, tol16=1e-2)
    assert torch.equal(X.cpu(), x)
    h2 = ops.hyper_step(X, write=(y.cuda(), dev["mix"], dev["out"]), read=(dev["in"], gain.cuda()), eps=1e-5)
    x2 = plain.hyper_write(x.double(), y.double(), {k: v.double() for k, v in hw.items()}, "")
    _close(X, x2, "float32")
    _close(h2, plain.scalar_rms_norm(plain.hyper_read(x2, {k: v.double() for k, v in hw.items()}, ""), 1.3, 1e-5), dtype, tol16=1e-2)
    total = torch.empty(T, W, device="cuda")
    ops.hyper_step(X, write=(y.cuda(), dev["mix"], dev["out"]), total=total)
    x3 = plain.hyper_write(x2, y.double(), {k: v.double() for k, v in hw.items()}, "")
    _close(total, x3.sum(1), "float32")
    _close(ops.hyper_fan_out(total, S), total[:, None, :].expand(T, S, W), "float32", tol32=0.0)


def _attention_reference(q, k, v, temp, talk, scale, rot):
    """q [T, H, d], k [T, G, d], v [T, G, dv] (float64) -> [T, H * dv], by the plain mixer with identity projections."""
    T, H, d = q.shape
    G, dv = k.shape[1], v.shape[2]
    W = max(H * d, G * d, G * dv)
    h = torch.zeros(T, 3 * W, dtype=torch.float64)
    h[:, :H * d], h[:, W:W + G * d], h[:, 2 * W:2 * W + G * dv] = q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1)
    eye = torch.eye(3 * W, dtype=torch.float64)
    w = {"q": eye[:H * d], "k": eye[W:W + G * d], "v": eye[2 * W:2 * W + G * dv], "o": torch.eye(H * dv, dtype=torch.float64),
         "temp": temp.double(), "talk": talk.double()}
    m = {"heads": H, "kv_heads": G, "dim": d, "vdim": dv, "scale": scale}
    if rot:
        m["rot"] = {"dims": rot[0], "base": rot[1]}
    return plain.talking_softmax_attention(h, w, "", m)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("generic", [True, False])
@pytest.mark.parametrize("H,G,d,dv,rot", [(4, 2, 24, 40, (16, 5000.0)), (5, 5, 12, 36, (6, 777.0)), (1, 1, 64, 64, (64, 10000.0)),
                                          (6, 3, 8, 12, None), (32, 8, 128, 128, (64, 1e6)), (8, 4, 64, 64, (32, 1e4)),
                                          (6, 3, 96, 96, None), (3, 3, 32, 32, (32, 50.0)), (40, 10, 16, 24, (8, 300.0)), (66, 66, 8, 8, None)])
def test_talking_attention_sees_every_key_up_to_the_query_and_mixes_heads(dtype, H, G, d, dv, rot, generic):
    """For chosen (query, key) pairs one score towers over the others: the first key, a key far back, the keys on both
    sides of a page border and the query itself; right after the query stands a still larger key that must stay
    unseen.  The towering part lies in dimensions that are not rotated where there are any.  Run as one prompt and as a
    prompt followed by single tokens, in slots and pages that are not the first; by the kernel that forms the mixed
    weights itself, and by the choice the library makes (runs of the tensor-core attention and a mix, where they fit)."""
    from cpmcu_b200.cache import Cache
    from cpmcu_b200.ops.ops import Ops
    from cpmcu_b200.parts.base import CacheNeeds
    from cpmcu_b200.parts.position import Rotary

    ops = Ops(DT[dtype])
    g = torch.Generator().manual_seed(H * d + dv)
    T = 200
    q = torch.randn(T, H, d, generator=g) * 0.5
    k = torch.randn(T, G, d, generator=g) * 0.5
    v = torch.randn(T, G, dv, generator=g)
    spike = d - 1                                            # not rotated unless the whole head is
    for qi, kj in ((199, 0), (198, 5), (150, 63), (151, 64), (130, 65), (190, 190), (64, 63), (63, 63)):
        q[qi, :, spike] = 9.0
        k[kj, :, spike] = 9.0
        if qi + 1 < T and qi + 1 not in (199, 198, 150, 151, 130, 190, 64, 63):
            k[qi + 1, :, spike] = 30.0                       # just outside: later than the query
    if rot and rot[0] == d:
        q[:, :, spike] = q[:, :, spike].clamp(-1, 1)         # a fully rotated head: keep the plain random case
        k[:, :, spike] = k[:, :, spike].clamp(-1, 1)
    temp = 1.0 + 0.3 * torch.randn(H, generator=g)
    talk = torch.eye(H) + 0.4 * torch.randn(H, H, generator=g)
    scale = 0.3
    rnd = lambda t: t.to(DT[dtype]).double()
    want = _attention_reference(rnd(q), rnd(k), rnd(v), temp, talk, scale, rot)
    qkv = torch.cat([q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1)], dim=1).to(DT[dtype]).cuda()
    inv_freq = Rotary(ops, d, rot[1], rot[0]).inv_freq if rot else None
    needs = CacheNeeds(kv_heads=G, head_dim=d, value_dim=dv if dv != d else 0)
    for pieces in ([T], [T - 9] + [1] * 9, [70, 2, 61] + [1] * 67):
        cache = Cache([needs], max_tokens=64 * 12, dtype=DT[dtype], device="cuda:0", n_slots=3)
        cache.open_sequence()
        other = cache.open_sequence()
        cache.reserve(other, 130)                            # the sequence under test gets neither slot 0 nor the first pages
        slot = cache.open_sequence()
        lane = cache.lane(0)
        outs, at = [], 0
        for n in pieces:
            cache.reserve(slot, at + n)
            cache.sync()
            ctx = _ctx([n], [at], [slot])
            qr = ops.rope_store_dv(ctx, qkv[at:at + n].contiguous(), lane, H, G, d, dv, inv_freq, rot[0] if rot else 0)
            fn = ops.talking_attention_generic if generic else ops.talking_attention
            outs.append(fn(ctx, qr, lane, G, dv, scale, temp.cuda(), talk.cuda()))
            at += n
        got = torch.cat(outs)
        _close(got, want, dtype, tol32=3e-5, tol16=3e-2)
        for qi in (199, 198, 150, 151, 130, 190, 64, 63):    # the rows with a towering score, one by one
            _close(got[qi], want[qi], dtype, tol32=3e-5, tol16=3e-2)


@pytest.mark.parametrize("delta", [False, True])
@pytest.mark.parametrize("H,G,d,dv", [(3, 3, 20, 24), (4, 2, 24, 16), (1, 1, 72, 16), (6, 3, 8, 8), (2, 1, 128, 130), (2, 2, 200, 33)])
def test_matrix_recurrence_in_one_piece_and_in_pieces(delta, H, G, d, dv):
    from cpmcu_b200.ops.ops import Ops

    ops = Ops(torch.float32)
    g = torch.Generator().manual_seed(d * dv + H)
    lens = [90, 1, 37]
    outs_want, ins = [], []
    for n in lens:
        q = torch.randn(n, G, d, generator=g) * d ** -0.5
        k = torch.randn(n, G, d, generator=g)
        k = k / k.norm(dim=-1, keepdim=True)
        v = torch.randn(n, H, dv, generator=g)
        decay = torch.rand(n, H, generator=g) * 0.5 + 0.5 if delta else torch.rand(n, H, d, generator=g) * 0.3 + 0.7
        beta = torch.rand(n, H, generator=g) if delta else None
        rep = H // G
        o, _ = plain.matrix_recurrence(q.double().repeat_interleave(rep, 1), k.double().repeat_interleave(rep, 1), v.double(),
                                       decay.double()[:, :, None] if delta else decay.double(), beta.double() if delta else None)
        outs_want.append(o * 0.7)
        ins.append((q, k, v, decay, beta))
    for cuts in ([1.0], [0.5, 1.0], [0.1, 0.2, 0.6, 1.0]):
        state = torch.full((5, H, d, dv), 7.0, device="cuda")          # rubbish that position 0 must not read
        slots = [4, 0, 2]
        got = [[] for _ in lens]
        done = [0] * len(lens)
        for c in cuts:
            upto = [max(done[i] + (1 if done[i] < n else 0), int(round(n * c))) if done[i] < n else n for i, n in enumerate(lens)]
            live = [i for i in range(len(lens)) if upto[i] > done[i]]
            if not live:
                continue
            ctx = _ctx([upto[i] - done[i] for i in live], [done[i] for i in live], [slots[i] for i in live])
            cat = lambda j: torch.cat([ins[i][j][done[i]:upto[i]].reshape(upto[i] - done[i], -1) for i in live]).cuda().contiguous()
            o = ops.linear_recurrence(ctx, cat(0), cat(1), cat(2), cat(3), cat(4) if delta else None, state, H, G, d, dv, 0.7,
                                      vector_decay=not delta)
            at = 0
            for i in live:
                got[i].append(o[at:at + upto[i] - done[i]])
                at += upto[i] - done[i]
                done[i] = upto[i]
        for i in range(len(lens)):
            _close(torch.cat(got[i]), outs_want[i], "float32", tol32=3e-5)


@pytest.mark.parametrize("K", [1, 2, 4, 8])
def test_convolution_reads_the_state_and_leaves_the_last_inputs(K):
    from cpmcu_b200.ops.ops import Ops

    ops = Ops(torch.float32)
    g = torch.Generator().manual_seed(K)
    H, G, d, dv = 3, 1, 20, 44
    C = 2 * G * d + H * dv
    N = C + H * dv + 2 * H
    lens = [50, 2, 9]
    taps = torch.randn(C, K, generator=g) * 0.6
    a_log, dt_bias = torch.randn(H, generator=g) * 0.5, torch.randn(H, generator=g)
    projs = [torch.randn(n, N, generator=g) for n in lens]
    want = []
    for p in projs:
        x = plain.silu(plain.short_convolution(p[:, :C].double(), taps.double()))
        q, k, v = x[:, :G * d].view(-1, G, d), x[:, G * d:2 * G * d].view(-1, G, d), x[:, 2 * G * d:]
        q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6)
        k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
        beta = torch.sigmoid(p[:, C + H * dv:C + H * dv + H].double())
        decay = torch.exp(-torch.exp(a_log.double()) * torch.nn.functional.softplus(p[:, C + H * dv + H:].double() + dt_bias.double()))
        want.append([q.reshape(len(p), -1), k.reshape(len(p), -1), v, beta, decay])
    for cuts in ([[50], [2], [9]], [[1, 1, 1, 2, 45], [1, 1], [3, 6]], [[25, 25], [2], [8, 1]]):
        state = torch.full((4, max(K - 1, 1), C), 5.0, device="cuda")
        slots = [3, 1, 0]
        got = [[] for _ in lens]
        done = [0] * 3
        for step in range(max(len(c) for c in cuts)):
            live = [i for i in range(3) if step < len(cuts[i])]
            ns = [cuts[i][step] for i in live]
            ctx = _ctx(ns, [done[i] for i in live], [slots[i] for i in live])
            proj = torch.cat([projs[i][done[i]:done[i] + n] for i, n in zip(live, ns)]).cuda()
            res = ops.conv_prepare(ctx, proj, taps.cuda(), state, a_log.cuda(), dt_bias.cuda(), C + H * dv, C + H * dv + H, H, G, d, dv, 1e-6)
            at = 0
            for i, n in zip(live, ns):
                got[i].append([r[at:at + n] for r in res])
                at += n
                done[i] += n
        for i in range(3):
            for j in range(5):
                _close(torch.cat([piece[j] for piece in got[i]]), want[i][j], "float32", tol32=2e-5)


@pytest.mark.parametrize("E,top,groups,keep", [(10, 3, 2, 1), (8, 2, 4, 2), (9, 4, 3, 2), (6, 6, 1, 1), (64, 6, 8, 3), (300, 8, 1, 1)])
def test_routing_follows_the_rule(E, top, groups, keep):
    from cpmcu_b200.ops.ops import Ops

    ops = Ops(torch.float32)
    g = torch.Generator().manual_seed(E + top)
    T = 400
    z = torch.randn(T, E + 1, generator=g) * 3.0
    corr = torch.randn(E, generator=g) * 0.1 - 0.3           # all choice scores negative: a masked 0 would win
    chosen, weights, gate = ops.moe_route(z.cuda(), corr.cuda(), E, top, groups, keep, gate_col=E)
    r = {"experts": E, "top": top, "groups": {"count": groups, "keep": keep}}
    s, choice = plain.route_scores(z[:, :E].double(), corr.double(), r)
    want = choice.topk(top, dim=-1)
    gap = (want.values[:, -1] - choice.masked_fill(torch.zeros_like(choice, dtype=torch.bool).scatter_(1, want.indices, True),
                                                    float("-inf")).max(-1).values) if top < E else torch.ones(T)
    firm = gap > 1e-6
    assert int(firm.sum()) > 0.95 * T
    got = chosen.cpu().long()
    assert torch.equal(got[firm].sort(-1).values, want.indices[firm].sort(-1).values)
    _close(weights.cpu()[firm], torch.gather(s, 1, got)[firm], "float32", tol32=1e-5)
    _close(gate, torch.sigmoid(z[:, E].double()), "float32", tol32=1e-6)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T,E,top,W,ff", [(1, 4, 1, 64, 24), (7, 6, 3, 96, 40), (130, 9, 4, 100, 20), (600, 5, 2, 256, 136)])
def test_experts_products_over_pairs_grouped_by_expert(dtype, T, E, top, W, ff):
    from cpmcu_b200.ops.ops import Ops

    ops = Ops(DT[dtype])
    g = torch.Generator().manual_seed(T + E)
    x = torch.randn(T, W, generator=g).to(DT[dtype])
    wg, wu = (torch.randn(E, ff, W, generator=g) / W ** 0.5).to(DT[dtype]), (torch.randn(E, ff, W, generator=g) / W ** 0.5).to(DT[dtype])
    wd = (torch.randn(E, W, ff, generator=g) / ff ** 0.5).to(DT[dtype])
    chosen = torch.stack([torch.randperm(E, generator=g)[:top] for _ in range(T)]).int()
    if T > 100:
        chosen[:, 0] = 1                                    # one expert with many tokens, some with none
        chosen[:, 1:] = torch.where(chosen[:, 1:] == 1, 0, chosen[:, 1:])
    weights = torch.rand(T, top, generator=g)
    shared = torch.randn(T, W, generator=g).to(DT[dtype])
    gate = torch.rand(T, generator=g)
    pairs = ops.moe_experts(x.cuda(), chosen.cuda(), wg.cuda(), wu.cuda(), wd.cuda())
    out = ops.moe_combine(pairs, weights.cuda(), shared.cuda(), gate.cuda())
    want = torch.zeros(T, W, dtype=torch.float64)
    for t in range(T):
        for j in range(top):
            e = int(chosen[t, j])
            w = {"gate": wg[e].double(), "up": wu[e].double(), "down": wd[e].double()}
            want[t] += weights[t, j].double() * plain.gated_expert(x[t:t + 1].double(), w, "")[0]
    want += gate.double()[:, None] * shared.double()
    _close(out, want, dtype, tol32=2e-5, tol16=2e-2)
    _close(ops.moe_combine(pairs, weights.cuda(), None, None), want - gate.double()[:, None] * shared.double(), dtype, tol32=2e-5, tol16=3e-2)


@pytest.mark.parametrize("dtype", DTYPES)
def test_head_norm_with_gate_and_the_join_of_two_mixers(dtype):
    from cpmcu_b200.ops.ops import Ops

    ops = Ops(DT[dtype])
    g = torch.Generator().manual_seed(1)
    T, H, dv, W = 33, 5, 36, 100
    o = torch.randn(T, H, dv, generator=g)
    wide = torch.randn(T, 3 * H * dv, generator=g)
    w = 1 + 0.2 * torch.randn(dv, generator=g)
    got = ops.gated_head_norm(o.cuda(), wide.cuda()[:, H * dv:2 * H * dv], w.cuda(), 1e-5)
    want = plain.rms_norm(o.double(), w.double(), 1e-5).reshape(T, -1) * plain.silu(wide[:, H * dv:2 * H * dv].double())
    _close(got, want, dtype, tol16=1e-2)
    a, b = torch.randn(T, W, generator=g).to(DT[dtype]), (3 * torch.randn(T, W, generator=g)).to(DT[dtype])
    wa, wb = 1 + 0.2 * torch.randn(W, generator=g), 1 + 0.2 * torch.randn(W, generator=g)
    got = ops.dual_rmsnorm_mean(a.cuda(), b.cuda(), wa.cuda(), wb.cuda(), 1e-5)
    want = 0.5 * (plain.rms_norm(a.double(), wa.double(), 1e-5) + plain.rms_norm(b.double(), wb.double(), 1e-5))
    _close(got, want, dtype, tol16=1e-2)
    z = torch.randn(T, H * dv, generator=g) * 4
    bias = torch.randn(H * dv, generator=g)
    got = ops.sigmoid_power(z.cuda().clone(), bias.cuda(), 7.0)
    _close(got, torch.sigmoid(z.double() + bias.double()) ** (1 / 7.0), "float32", tol32=1e-6)
