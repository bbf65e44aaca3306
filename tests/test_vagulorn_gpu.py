"""Vagulorn on the GPU against the plain implementation (``tests/plain/vagulorn.py``, float64).

Whole models of several small configurations, replayed whole, with a decoded tail, in portions down to
two tokens, and mixed with other requests in a pool so small that pages and state slots are used
again; every mechanism alone (a one-layer model, or its kernel with inputs made so that one key or a
mask's edge decides the result); long decoding; greedy generation through the public entry point and
the scheduler.

Errors are relative: the root mean square over the vocabulary of the difference of the logits (mean
taken off) over the standard deviation of the plain model's logits.
"""

import math

import numpy as np
import pytest
import torch

from acorninfer_b200.config.model_config import StateSpaceConfig, VagulornConfig
from tests import traces
from tests.paged import rows_layout, scatter_to_pages
from tests.plain import vagulorn as plain
from tests.tiny import random_tokens
from tests.vagulorn_tiny import VAGU_LONG, VAGUS, L, att, beside, make_model_dir, random_config, read_weights

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL = {"float32": 4e-5, "bfloat16": 0.1}
LENGTHS = [45, 38, 61, 50, 33, 29]


def rel_err(got, ref):
    d = np.asarray(got, np.float64) - np.asarray(ref, np.float64)
    d = d - d.mean()
    return math.sqrt((d ** 2).mean()) / float(np.std(ref))


@pytest.fixture(scope="module", params=list(VAGUS))
def case(request, tmp_path_factory):
    tiny = VAGUS[request.param]
    d = make_model_dir(tmp_path_factory.mktemp(request.param), tiny)
    w = read_weights(d)
    reqs = {f"r{i}": random_tokens(n, tiny["cfg"].vocab_size, 3000 + i) for i, n in enumerate(LENGTHS)}
    ref = {rid: plain.forward(tiny["cfg"].to_dict(), w, toks).numpy() for rid, toks in reqs.items()}
    return tiny, d, reqs, ref


def run_cut(tiny, model_dir, steps, dtype, max_requests=4, watch=None):
    from acorninfer_b200.engine.runner import ModelRunner
    from acorninfer_b200.replay import TraceSession

    pool = traces.max_live_tokens(steps)
    runner = ModelRunner.from_model_dir(model_dir, dtype=dtype, num_blocks=-(-pool // tiny["page_size"]),
                                        page_size=tiny["page_size"], max_requests=max_requests, max_step_tokens=4096)
    session = TraceSession(runner)

    def step(msg):
        if watch is None:
            return session.step(msg)
        out = session.step(dict(msg, end=[]))
        watch(session, msg)
        session.step({"entries": [], "end": msg["end"]})
        return out

    got = traces.collect(step, steps)
    runner.manager.assert_balanced()
    return got, runner


def check(got, ref, dtype, what, tol=None):
    errs = {key: rel_err(row, ref[key[0]][key[1]]) for key, row in got.items()}
    worst = max(errs, key=errs.get)
    assert errs[worst] < (tol or TOL[dtype]), f"{what}: {worst}: {errs[worst]:.3e}"


CUTS = {
    "whole": traces.whole,
    "decode_tail": lambda r: traces.decode_tail(r, tail=24),
    "portions": lambda r: traces.portions(r, sizes=(7, 2, 5, 3, 16, 2, 11, 4)),
    "mixed": lambda r: traces.mixed(r, max_live=4, seed=3, stagger=2),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("cut", list(CUTS))
def test_cut_matches_plain(case, cut, dtype):
    tiny, d, reqs, ref = case
    got, runner = run_cut(tiny, d, CUTS[cut](reqs), dtype)
    assert len(got) == sum(len(t) for t in reqs.values())
    check(got, ref, dtype, cut)
    if cut == "decode_tail":
        assert runner.graph_replays >= len(reqs) * 10        # single-token steps replay captured graphs


def test_cuts_agree_with_each_other_float32(case):
    """The logits at a position do not depend on how the tokens were cut into steps, on what else was
    in the batch or on which pages and slots held them, beyond rounding."""
    tiny, d, reqs, _ = case
    base, _ = run_cut(tiny, d, traces.whole(reqs), "float32")
    for cut in ("decode_tail", "portions", "mixed"):
        other, _ = run_cut(tiny, d, CUTS[cut](reqs), "float32")
        for key, row in base.items():
            assert rel_err(other[key], row) < 1e-5, f"{cut}: {key}"


def test_mixed_trace_uses_pages_and_slots_again(case):
    tiny, d, reqs, _ = case
    steps = CUTS["mixed"](reqs)
    pages: dict = {}
    slots: dict = {}

    def watch(session, msg):
        for rid, rc in session.live.items():
            slots.setdefault(rc.slot, set()).add(rid)
            for table in rc.tables:
                for page in table:
                    pages.setdefault(page, set()).add(rid)

    run_cut(tiny, d, steps, "float32", watch=watch)
    assert len(slots) <= 4 and sum(1 for users in slots.values() if len(users) >= 2) >= 1, slots
    assert sum(1 for users in pages.values() if len(users) >= 2) >= 2, pages


def test_first_step_of_one_token_and_requests_left_out(case):
    """A request whose first step is a single token (the convolution's zeros before the start, a state
    that starts at zero, a block or window that holds one key), then portions beside another request
    that decodes and is left out of some steps."""
    tiny, d, reqs, ref = case
    a, b = reqs["r0"], reqs["r1"]
    steps = [{"entries": [{"id": "r0", "tokens": a[:1], "want": [0]}], "end": []},
             {"entries": [{"id": "r0", "tokens": a[1:3], "want": [0, 1]}, {"id": "r1", "tokens": b[:9], "want": list(range(9))}], "end": []},
             {"entries": [{"id": "r1", "tokens": b[9:10], "want": [0]}], "end": []},
             {"entries": [{"id": "r0", "tokens": a[3:20], "want": list(range(17))}, {"id": "r1", "tokens": b[10:11], "want": [0]}], "end": []},
             {"entries": [{"id": "r0", "tokens": a[20:], "want": list(range(len(a) - 20))}], "end": ["r0"]},
             {"entries": [{"id": "r1", "tokens": b[11:], "want": list(range(len(b) - 11))}], "end": ["r1"]}]
    for i, s in enumerate(steps):
        s["step"] = i
    for dtype in ("float32", "bfloat16"):
        got, _ = run_cut(tiny, d, steps, dtype)
        check(got, ref, dtype, "first token alone")


def test_long_decoding_float32(case):
    """A short prompt and 170 decoded tokens: blocks and windows pass over decoded tokens many times, pages
    of a cache in blocks are given back and taken again, the recurrent state is carried all the way."""
    tiny, d, _, _ = case
    toks = random_tokens(190, tiny["cfg"].vocab_size, 77)
    ref = {"long": plain.forward(tiny["cfg"].to_dict(), read_weights(d), toks).numpy()}
    steps = traces.decode_tail({"long": toks}, tail=170)
    got, _ = run_cut(tiny, d, steps, "float32")
    check(got, ref, "float32", "long decoding")


def test_long_requests_blocks_and_windows_over_pages(tmp_path):
    """Requests of a few hundred tokens through blocks of 70 and a window of 130 with 20 kept keys over pages
    of 16: the tensor-core attention walks several chunks of keys whose first and last are cut by the mask,
    the kept keys ride in front of the window's, the group in blocks gives pages back while a request is
    still fed, and the states are carried over hundreds of tokens."""
    tiny = VAGU_LONG
    reqs = {f"L{i}": random_tokens(n, tiny["cfg"].vocab_size, 600 + i) for i, n in enumerate([330, 260, 150])}
    cuts = {"whole": traces.whole, "decode_tail": lambda r: traces.decode_tail(r, tail=90),
            "portions": lambda r: traces.portions(r, sizes=(64, 3, 2, 128, 29, 16, 2, 70)),
            "mixed": lambda r: traces.mixed(r, max_live=3, seed=5, max_portion=80, stagger=1)}
    d = make_model_dir(tmp_path, tiny)
    w = read_weights(d)
    ref = {rid: plain.forward(tiny["cfg"].to_dict(), w, toks).numpy() for rid, toks in reqs.items()}
    for dtype in ("float32", "bfloat16"):
        for cut, build in cuts.items():
            got, runner = run_cut(tiny, d, build(reqs), dtype)
            assert len(got) == sum(len(t) for t in reqs.values())
            check(got, ref, dtype, f"long, {cut}")


@pytest.mark.parametrize("seed", [1, 4, 9, 13, 16])
def test_configurations_drawn_at_random(seed, tmp_path):
    """Models whose sizes are drawn from what real models have (heads of 32 to 128, also with the whole head
    rotated; states up to 128; values wider than keys; windows of 32 to 256), requests of up to 600 tokens, whole
    and mixed in a small pool, float32 and bfloat16."""
    import random
    tiny = dict(cfg=random_config(seed), page_size=16, seed=seed)
    d = make_model_dir(tmp_path, tiny, sigma=0.06, sigma_norm=0.1)
    w = read_weights(d)
    rng = random.Random(seed)
    lengths = [rng.randint(300, 600), rng.randint(100, 300), rng.randint(2, 60), 1, rng.randint(60, 200)]
    reqs = {f"q{i}": random_tokens(n, tiny["cfg"].vocab_size, seed * 10 + i) for i, n in enumerate(lengths)}
    ref = {rid: plain.forward(tiny["cfg"].to_dict(), w, toks).numpy() for rid, toks in reqs.items()}
    for dtype, tol in (("float32", 6e-5), ("bfloat16", 0.15)):
        for cut, steps in (("whole", traces.whole(reqs)), ("decode_tail", traces.decode_tail(reqs, tail=40)),
                           ("mixed", traces.mixed(reqs, max_live=4, seed=seed, max_portion=90, stagger=1))):
            got, _ = run_cut(tiny, d, steps, dtype)
            check(got, ref, dtype, f"seed {seed}, {cut}", tol=tol)


def follows_plain(cfg, w, prompt, ids, slack):
    logits = plain.forward(cfg.to_dict(), w, ids[:-1])
    return all(float(logits[i - 1].max() - logits[i - 1][ids[i]]) <= slack for i in range(len(prompt), len(ids)))


@pytest.mark.parametrize("dtype,slack", [("float32", 1e-4), ("bfloat16", 0.15)])
def test_greedy_generation_through_the_engine(case, dtype, slack):
    """``generate``: the scheduler with a token budget (prompts cut into portions beside decoding
    requests), sampling on the device, a step ahead of the host."""
    from acorninfer_b200 import generate
    tiny, d, _, _ = case
    cfg = tiny["cfg"]
    w = read_weights(d)
    prompts = [random_tokens(n, cfg.vocab_size, 900 + n) for n in (1, 14, 23, 6, 31)]
    outs = generate(d, prompts, max_new_tokens=12, temperature=0.0, dtype=dtype, page_size=tiny["page_size"],
                    num_blocks=64, max_running=3, chunked_budget=10, watermark_blocks=0, eos_ids=())
    for p, ids in zip(prompts, outs):
        assert len(ids) == len(p) + 12 and follows_plain(cfg, w, p, ids, slack), (dtype, len(p))


def test_preemption_recomputes_state_float32(case):
    """So few pages that requests are preempted and recomputed from their first token: the recurrent
    states and the convolution's memory start over with the slot."""
    from acorninfer_b200.generation import build_engine, generate_with_engine
    tiny, d, _, _ = case
    cfg = tiny["cfg"]
    prompts = [random_tokens(n, cfg.vocab_size, 40 + n) for n in (20, 18, 13)]
    pages = -(-36 // tiny["page_size"]) * 2 + 1
    tight = build_engine(d, dtype="float32", page_size=tiny["page_size"], num_blocks=pages, watermark_blocks=0, max_running=3)
    got = generate_with_engine(tight, prompts, max_new_tokens=16, eos_ids=())
    w = read_weights(d)
    for p, a in zip(prompts, got):
        assert len(a) == len(p) + 16 and follows_plain(cfg, w, p, a, 1e-4)


# ------------------------------------------------------------------ one mechanism at a time


def _solo(mixer, ff=None, width=48, vocab=90, scale=2.0):
    return VagulornConfig(vocab_size=vocab, hidden_size=width, norm_eps=1e-5, embedding_scale=scale, layers=(L(mixer, ff),))


_SMALL_SSM = StateSpaceConfig(heads=1, vdim=4, state=3, groups=1, conv=1, norm_groups=1)
SOLOS = {
    "state space, heads in groups, 4 taps, 5 norm parts": _solo(StateSpaceConfig(heads=10, vdim=6, state=9, groups=5, conv=4, norm_groups=5)),
    "state space, one head, state of 70": _solo(StateSpaceConfig(heads=1, vdim=20, state=70, groups=1, conv=2, norm_groups=4)),
    "state space, state of 300, one tap": _solo(StateSpaceConfig(heads=2, vdim=3, state=300, groups=2, conv=1, norm_groups=1)),
    "attention in blocks of 5, values wider than keys": _solo(att(heads=4, kv_heads=2, dim=6, vdim=22, scale=0.4, rot_dims=4, rot_base=100.0, mask_size=5)),
    "attention, no mask, no rotation, values narrower": _solo(att(heads=3, kv_heads=3, dim=18, vdim=4, scale=0.3)),
    "attention in blocks of 1": _solo(att(heads=2, kv_heads=1, dim=8, vdim=8, scale=0.3, rot_dims=8, mask_size=1)),
    "window 4 with 7 kept keys beside decays": _solo(beside(att(heads=2, kv_heads=1, dim=14, vdim=14, scale=0.3, rot_dims=6, rot_base=50.0, mask_size=4, keep_first=7),
                                                            heads=4, dim=5, vdim=9, decay=(0.3, 0.9, 0.99, 1.0), left_scale=1.5, right_scale=0.25)),
    "window 9, nothing kept, beside one head of 130 key entries": _solo(beside(att(heads=6, kv_heads=2, dim=4, vdim=4, scale=0.5, rot_dims=2, mask_size=9),
                                                                               heads=1, dim=130, vdim=6, decay=(0.95,), left_scale=0.5, right_scale=2.0)),
    "gated feed-forward, widths no multiple of 8": _solo(_SMALL_SSM, ff=37, width=44),
    "embedding scale of 1, wide feed-forward": _solo(_SMALL_SSM, ff=200, scale=1.0),
}


@pytest.mark.parametrize("name", list(SOLOS))
def test_mechanism_alone(name, tmp_path):
    tiny = dict(cfg=SOLOS[name], page_size=4, seed=5)
    d = make_model_dir(tmp_path, tiny, sigma=0.3)
    w = read_weights(d)
    reqs = {f"s{i}": random_tokens(n, tiny["cfg"].vocab_size, 50 + i) for i, n in enumerate([26, 17, 9])}
    ref = {rid: plain.forward(tiny["cfg"].to_dict(), w, toks).numpy() for rid, toks in reqs.items()}
    for cut in ("whole", "portions", "mixed", "decode_tail"):
        steps = {"portions": traces.portions(reqs, sizes=(3, 2, 6, 2)), "decode_tail": traces.decode_tail(reqs, tail=8)}.get(cut) \
            or CUTS[cut](reqs)
        got, _ = run_cut(tiny, d, steps, "float32")
        check(got, ref, "float32", f"{name}, {cut}")
    got, _ = run_cut(tiny, d, CUTS["mixed"](reqs), "bfloat16")
    check(got, ref, "bfloat16", f"{name}, mixed, bfloat16", tol=0.2)


def ops():
    from acorninfer_b200.kernels import ops as o
    return o


def _attention_case(befores, qlens, P, d, dv, nq, nkv, rule, size, keep, spikes, dtype, kernel, seed=0):
    """Cache pages and queries for the attention kernels.  ``spikes``: (row, key position): that key and all
    queries of the row get a large component along one direction, so its score stands out wherever it is seen
    and the row's result is (nearly) that key's value."""
    o = ops()
    g = torch.Generator().manual_seed(seed)
    NP = sum(-(-(b + q) // P) for b, q in zip(befores, qlens)) + 5
    lay = rows_layout(befores, qlens, P, NP, seed=seed)
    k_pages = torch.zeros(NP, nkv, P, d, dtype=dtype, device=DEV)
    v_pages = torch.zeros(NP, nkv, P, dv, dtype=dtype, device=DEV)
    full = []
    for r, (b, q) in enumerate(zip(befores, qlens)):
        S = b + q
        k = torch.randn(S, nkv, d, generator=g) * 0.3
        v = torch.randn(S, nkv, dv, generator=g)
        qq = torch.randn(S, nq, d, generator=g) * 0.3
        for (rr, j) in spikes:
            if rr == r:
                k[j, :, d - 1] = 6.0
                qq[:, :, d - 1] = 4.0
        k, v, qq = k.to(dtype), v.to(dtype), qq.to(dtype)
        scatter_to_pages(k_pages, lay["tables"][r], k, P)
        scatter_to_pages(v_pages, lay["tables"][r], v, P)
        full.append((qq.double(), k.double(), v.double()))
    q_new = torch.cat([f[0][b:] for f, b in zip(full, befores)]).to(dtype).to(DEV).contiguous().view(-1, nq * d)
    scale = 0.5
    window, chunk = (size if rule == "window" else None), (size if rule == "blocks" else None)
    common = (k_pages, v_pages, lay["block_table"], lay["page_base"])
    if kernel == "plain":
        out = o.attention_plain(q_new, nq * d, *common, lay["token_row"], lay["positions"], lay["num_tokens"], nq, nkv,
                                d, scale, window, value_dim=dv, chunk=chunk, keep_first=keep)
    else:
        i32 = dict(dtype=torch.int32, device=DEV)
        starts = np.cumsum([0] + qlens)
        out = torch.zeros((lay["num_tokens"], nq * d), dtype=dtype, device=DEV)
        big = 32 if kernel.startswith("tc") else 10 ** 9          # rows from 32 tokens on go to the tcgen05 kernel
        tiles = torch.tensor([(r, q0) for r, n in enumerate(qlens) if n >= big for q0 in range(0, n, 128)], **i32).view(-1, 2)
        if tiles.shape[0]:
            o.attention_prefill_tc(q_new, nq * d, *common, torch.tensor(starts, **i32), torch.tensor(befores, **i32), tiles,
                                   lay["num_tokens"], nq, nkv, d, scale, window, out=out, chunk=chunk, keep_first=keep)
        tiles = torch.tensor([(r, q0) for r, n in enumerate(qlens) if 1 < n < big for q0 in range(0, n, 64)], **i32).view(-1, 2)
        if tiles.shape[0]:
            o.attention_prefill(q_new, nq * d, *common, torch.tensor(starts, **i32), torch.tensor(befores, **i32), tiles,
                                lay["num_tokens"], nq, nkv, d, scale, window, out=out, chunk=chunk, keep_first=keep)
        singles = torch.tensor([int(starts[r]) for r, n in enumerate(qlens) if n == 1], **i32)
        if singles.numel():
            o.attention_decode(q_new, nq * d, *common, lay["token_row"], lay["positions"], lay["num_tokens"], nq, nkv, d,
                               scale, window, int(kernel[-1]), token_list=singles, out=out, use_tma=False, chunk=chunk,
                               keep_first=keep)
    want = []
    for (fq, fk, fv), b in zip(full, befores):
        ok = plain.visible(fq.shape[0], rule, size, keep)
        want.append(plain.softmax_attention(fq, fk, fv, scale, ok)[b:])
    return out.float().cpu().view(-1, nq, dv), torch.cat(want)


KERNELS = [(torch.float32, 2e-5, "plain", 24, 40, 6, 3), (torch.bfloat16, 2e-2, "plain", 24, 16, 3, 1),
           (torch.bfloat16, 2e-2, "mma1", 32, 32, 4, 2), (torch.bfloat16, 2e-2, "mma3", 96, 96, 6, 3),
           (torch.bfloat16, 2e-2, "mma2", 128, 128, 8, 1)]


@pytest.mark.parametrize("dtype,tol,kernel,d,dv,nq,nkv", KERNELS + [(torch.bfloat16, 2e-2, "tc2", 128, 128, 8, 2)])
def test_attention_window_with_kept_first_keys(dtype, tol, kernel, d, dv, nq, nkv):
    """A key that outweighs all others is seen up to the query window - 1 tokens after it and no longer, in a
    prompt's rows and in single decoded tokens, at page borders; the first ``keep`` keys are seen from
    anywhere and the next one is not."""
    P, W, keep = 16, 64, 5
    # row 0: a whole prompt; row 1: a portion after 130 cached tokens; rows 2-5: single tokens whose window's
    # first key (2, 4) or the key just before it (3, 5) is the spiked one, at a page's border or not; rows 6, 7:
    # single tokens far away whose spiked key is the last kept one (6) or the first that is not kept (7)
    befores = [0, 130, 15 + W - 1, 15 + W, 16 + W - 1, 16 + W, 500, 500, 3]
    qlens = [300, 90, 1, 1, 1, 1, 1, 1, 2]
    spikes = [(0, 3), (0, 15), (0, 16), (0, 200), (1, 100), (1, 131), (1, 5), (2, 15), (3, 15), (4, 16), (5, 16),
              (6, keep - 1), (7, keep)]
    got, want = _attention_case(befores, qlens, P, d, dv, nq, nkv, "window", W, keep, spikes, dtype, kernel)
    assert (got - want).abs().max() < tol
    at = np.cumsum([0] + qlens)
    assert (got[at[2]] - got[at[3]]).abs().max() > 0.05 and (got[at[6]] - got[at[7]]).abs().max() > 0.05
    # more kept keys than a page holds and than the window is wide; a window of one
    for W2, keep2 in ((8, 21), (1, 0), (1, 2)):
        got, want = _attention_case([0, 99, 40], [70, 1, 3], P, d, dv, nq, nkv, "window", W2, keep2, [(0, 20), (1, 20), (2, 20)],
                                    dtype, kernel, seed=W2)
        assert (got - want).abs().max() < tol, (W2, keep2)
    # kept keys that fill more than one block of 128 keys, far in front of the window
    got, want = _attention_case([0, 400], [700, 200], P, d, dv, nq, nkv, "window", 40, 150, [(0, 149), (0, 150), (1, 10), (1, 140)],
                                dtype, kernel, seed=9)
    assert (got - want).abs().max() < tol


@pytest.mark.parametrize("dtype,tol,kernel,d,dv,nq,nkv", KERNELS + [(torch.bfloat16, 2e-2, "tc2", 128, 128, 8, 2)])
def test_attention_in_blocks_of_positions(dtype, tol, kernel, d, dv, nq, nkv):
    """Blocks are counted from position 0 of the request, wherever a portion starts: a spiked key is seen by the
    queries of its own block after it and by no other; far keys are never seen; no mask at all finds key 3 of 700."""
    P, C = 16, 48
    befores = [0, 100, 2 * C - 1, 2 * C, 3 * C - 1, 3 * C - 1, C]
    qlens = [200, 70, 1, 1, 1, 1, 2]
    spikes = [(0, 0), (0, C - 1), (0, C), (0, 130), (1, 2 * C), (1, 2 * C + 5), (1, 3 * C - 1), (2, C), (3, 2 * C - 1),
              (4, 2 * C), (5, 2 * C - 1), (6, C - 1)]
    got, want = _attention_case(befores, qlens, P, d, dv, nq, nkv, "blocks", C, 0, spikes, dtype, kernel)
    assert (got - want).abs().max() < tol
    at = np.cumsum([0] + qlens)
    assert (got[at[4]] - got[at[5]]).abs().max() > 0.05
    for C2 in (1, 7, 64, 1000):
        got, want = _attention_case([0, 99, 40], [70, 1, 3], P, d, dv, nq, nkv, "blocks", C2, 0, [(0, 20), (1, 98), (2, 41)],
                                    dtype, kernel, seed=C2)
        assert (got - want).abs().max() < tol, C2
    got, want = _attention_case([0, 699], [40, 1], P, d, dv, nq, nkv, None, 0, 0, [(1, 3)], dtype, kernel)
    assert (got - want).abs().max() < tol


@pytest.mark.parametrize("long", [False, True])
@pytest.mark.parametrize("H,G,N,V", [(4, 2, 7, 10), (1, 1, 70, 20), (3, 3, 300, 3), (2, 1, 16, 130), (6, 6, 32, 32)])
def test_linear_scan_carries_state_across_steps_and_slots(H, G, N, V, long):
    """The recurrence over rows of unequal length from states in scattered slots, in two steps (the second
    continues the first), against the loop; a slot that is zeroed starts over.  ``long``: rows of hundreds of
    tokens, which are run in segments side by side (rows shorter than a segment, and of one token, beside them)."""
    o = ops()
    g = torch.Generator().manual_seed(N)
    slots, lens1, lens2 = ([3, 0, 5], [700, 1, 130], [3, 400, 64]) if long else ([3, 0, 5], [9, 1, 17], [1, 12, 2])
    if long:
        assert o.scan_segments(700, 3, H, N, V)[1] >= 4
    state = torch.zeros(7, H * N * V + 11, device=DEV)
    state[:, :] = 123.0                       # what lies in a slot before its request starts must not matter ...
    state[slots] = 0                          # ... once the slot is zeroed
    seqs = []
    for n1, n2 in zip(lens1, lens2):
        T = n1 + n2
        seqs.append(dict(a=torch.rand(T, H, generator=g).double() * (0.1 if long else 0.5) + (0.9 if long else 0.5),
                         dt=torch.rand(T, H, generator=g).double(),
                         B=torch.randn(T, G, N, generator=g).double(), C=torch.randn(T, G, N, generator=g).double(),
                         x=torch.randn(T, H, V, generator=g).double(), D=torch.randn(H, generator=g).double()))
    D = seqs[0]["D"]
    hg = torch.arange(H) // (H // G)
    want = [plain.selective_recurrence(s["a"], s["dt"], s["B"][:, hg], s["C"][:, hg], s["x"], D) for s in seqs]
    i32 = dict(dtype=torch.int32, device=DEV)
    at = [0, 0, 0]
    for lens in (lens1, lens2):
        cat = lambda key, shape: torch.cat([s[key][a:a + n] for s, a, n in zip(seqs, at, lens)]).float().reshape(*shape).to(DEV)
        T = sum(lens)
        # B and C as column slices of one wider buffer, as the mixer passes them
        bc = torch.cat([cat("B", (T, G * N)), cat("C", (T, G * N))], dim=1).contiguous()
        y = o.linear_scan(bc[:, :G * N], bc[:, G * N:], cat("x", (T, H * V)), cat("a", (T, H)), cat("dt", (T, H)),
                          D.float().to(DEV), state, 5, torch.tensor(np.cumsum([0] + lens), **i32),
                          torch.tensor(slots, **i32), 3, H, G, N, V, longest_row=max(lens)).cpu().double().view(T, H, V)
        t0 = 0
        for r, n in enumerate(lens):
            ref = want[r][at[r]:at[r] + n]
            assert (y[t0:t0 + n] - ref).abs().max() < 2e-4 * max(1.0, float(ref.abs().max())), (r, lens)
            t0 += n
            at[r] += n
    assert float(state[1].min()) == 123.0 and float(state[3, :5].abs().max()) == 0.0      # other slots and the vector's head untouched


def test_linear_scan_with_one_decay_per_head_and_no_step_sizes():
    o = ops()
    g = torch.Generator().manual_seed(1)
    H, N, V, T = 3, 9, 5, 40
    k, q, v = (torch.randn(T, H, n, generator=g).double() for n in (N, N, V))
    decay = torch.tensor([1.0, 0.0, 0.9], dtype=torch.float64)
    want = plain.decay_recurrence(decay, k, v, q)
    state = torch.zeros(2, H * N * V, device=DEV)
    i32 = dict(dtype=torch.int32, device=DEV)
    f = lambda t: t.float().reshape(T, -1).to(DEV)
    y = o.linear_scan(f(k), f(q), f(v), decay.float().to(DEV), None, None, state, 0, torch.tensor([0, T], **i32),
                      torch.tensor([1], **i32), 1, H, H, N, V).cpu().double().view(T, H, V)
    assert (y - want).abs().max() < 1e-4 * float(want.abs().max())


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 2e-2)])
def test_gated_norm_layernorm_glu_and_head_gate(dtype, tol):
    o = ops()
    g = torch.Generator().manual_seed(3)
    T, W = 13, 60
    y, z = torch.randn(T, W, generator=g), torch.randn(T, W + 4, generator=g).to(dtype)
    w = torch.rand(W, generator=g) + 0.5
    zz = z[:, 4:].double()
    for groups in (1, 3, 5):
        for gate_first in (True, False):
            out = torch.zeros(T, W + 8, dtype=dtype, device=DEV)
            o.gated_norm(y.to(DEV), z.to(DEV)[:, 4:], w.to(DEV), 1e-5, groups, gate_first, out[:, 8:], 0.75)
            u = y.double() * plain.silu(zz) if gate_first else y.double()
            u = plain.rms_norm(u.view(T, groups, W // groups), 1e-5).reshape(T, W) * w.double()
            want = 0.75 * (u if gate_first else u * torch.sigmoid(zz))
            assert (out[:, 8:].double().cpu() - want).abs().max() < tol * 4 and float(out[:, :8].abs().max()) == 0.0
    # layer norm of the stream plus two pending results; the stream takes both
    x = torch.randn(T, W, generator=g) * 3 + 1
    a, b = torch.randn(T, W, generator=g).to(dtype), torch.randn(T, W, generator=g).to(dtype)
    bias = torch.randn(W, generator=g)
    resid = x.clone().to(DEV)
    out = o.add_layernorm(resid, o.DeltaPair(a.to(DEV), b.to(DEV)), w.to(DEV), bias.to(DEV), 1e-5, dtype)
    s = x.double() + a.double() + b.double()
    assert (resid.cpu().double() - s).abs().max() < 1e-5
    assert (out.cpu().double() - plain.layer_norm(s, w.double(), bias.double(), 1e-5)).abs().max() < tol * 4
    rows = torch.tensor([5, 0, 5], dtype=torch.int32, device=DEV)
    part = o.add_layernorm(resid, None, w.to(DEV), bias.to(DEV), 1e-5, dtype, row_idx=rows)
    assert (part.cpu().double() - plain.layer_norm(s[[5, 0, 5]], w.double(), bias.double(), 1e-5)).abs().max() < tol * 4
    # gelu-gated unit, in the plain layout and in blocks of 4
    gu = torch.randn(T, 2 * 24, generator=g).to(dtype)
    want = plain.gelu_tanh(gu[:, :24].double()) * gu[:, 24:].double()
    assert (o.swiglu(gu.to(DEV), activation="gelu_tanh").cpu().double() - want).abs().max() < tol * 4
    blocked = torch.stack([gu[:, :24].view(T, 6, 4), gu[:, 24:].view(T, 6, 4)], dim=2).reshape(T, 48)
    assert (o.swiglu(blocked.to(DEV), block=4, activation="gelu_tanh").cpu().double() - want).abs().max() < tol * 4
    # a gate per head, written into rows of a wider buffer
    heads, d = 5, 12
    xh, gate = torch.randn(T, heads * d, generator=g).to(dtype), torch.randn(T, heads + 3, generator=g).to(dtype)
    wide = torch.zeros(T, heads * d + 16, dtype=dtype, device=DEV)
    o.head_gate(xh.to(DEV), gate.to(DEV), heads, 0.8, out=wide[:, 16:])
    want = xh.double().view(T, heads, d) * (0.8 * torch.sigmoid(gate[:, :heads].double()))[:, :, None]
    assert (wide[:, 16:].cpu().double().view(T, heads, d) - want).abs().max() < tol * 4


@pytest.mark.parametrize("M", [5, 32, 700])
def test_gelu_gate_as_the_epilogue_of_the_tensor_core_products(M):
    """gate and up rows in blocks of 64: the product's own epilogue applies the tanh form of gelu to the gate
    (the one-CTA kernel for few rows, the paired kernel for many)."""
    o = ops()
    g = torch.Generator().manual_seed(M)
    K, I = 96, 192
    x = (torch.randn(M, K, generator=g) * 0.5).to(torch.bfloat16)
    wg, wu = (torch.randn(I, K, generator=g) * 0.2).to(torch.bfloat16), (torch.randn(I, K, generator=g) * 0.2).to(torch.bfloat16)
    w = torch.stack([wg.view(I // 64, 64, K), wu.view(I // 64, 64, K)], dim=1).reshape(2 * I, K).contiguous()
    got = o.linear(x.to(DEV), w.to(DEV), out_dtype=torch.bfloat16, swiglu=True, activation="gelu_tanh").float().cpu()
    want = plain.gelu_tanh(x.double() @ wg.double().T) * (x.double() @ wu.double().T)
    assert got.shape == (M, I) and (got.double() - want).abs().max() < 3e-2 * float(want.abs().max())
    silu = o.linear(x.to(DEV), w.to(DEV), out_dtype=torch.bfloat16, swiglu=True).float().cpu()
    assert (silu.double() - plain.silu(x.double() @ wg.double().T) * (x.double() @ wu.double().T)).abs().max() < 3e-2 * float(want.abs().max())
