"""Kogonex on the GPU against the plain implementation (``tests/plain/kogonex.py``, float64).

Whole models of several small configurations, replayed whole, with a decoded tail, in portions down to
two tokens, and mixed with other requests in a pool so small that pages and state slots are used
again; every mechanism alone (a one-layer model, or its kernel with inputs made so that one key, a
sink or a window's edge decides the result); long decoding; greedy generation through the public
entry point and the scheduler.

Errors are relative: the root mean square over the vocabulary of the difference of the logits (mean
taken off) over the standard deviation of the plain model's logits.  float32 differs from float64 by
1e-6 .. 1e-5 (summation order); bfloat16 by 5e-3 .. 9e-2 (bfloat16 activations between the products; the
largest at single positions of these small random models where a sublayer's output is small before its norm).
"""

import math

import numpy as np
import pytest
import torch

from acorninfer_b200.config.model_config import (ChannelDeltaConfig, KogonexConfig, KogonexLayer, LatentAttentionConfig,
                                                 RotaryScaling, RoutedExpertsConfig)
from tests import traces
from tests.kogonex_tiny import KOGOS, make_model_dir, read_weights
from tests.paged import rows_layout, scatter_to_pages
from tests.plain import kogonex as plain
from tests.tiny import random_tokens

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL = {"float32": 4e-5, "bfloat16": 0.12}
LENGTHS = [45, 38, 61, 50, 33, 29]


def rel_err(got, ref):
    d = np.asarray(got, np.float64) - np.asarray(ref, np.float64)
    d = d - d.mean()
    return math.sqrt((d ** 2).mean()) / float(np.std(ref))


@pytest.fixture(scope="module", params=list(KOGOS))
def case(request, tmp_path_factory):
    tiny = KOGOS[request.param]
    d = make_model_dir(tmp_path_factory.mktemp(request.param), tiny)
    w = read_weights(d)
    reqs = {f"r{i}": random_tokens(n, tiny["cfg"].vocab_size, 3000 + i) for i, n in enumerate(LENGTHS)}
    ref = {rid: plain.forward(tiny["cfg"].to_dict(), w, toks).numpy() for rid, toks in reqs.items()}
    return tiny, d, reqs, ref


@pytest.fixture(scope="module")
def case16(case, tmp_path_factory):
    """The same configuration with corrections that decide the experts alone: what bfloat16 runs are
    compared on (see ``make_model_dir``)."""
    tiny, _, reqs, _ = case
    d = make_model_dir(tmp_path_factory.mktemp("decisive"), tiny, decisive=True)
    w = read_weights(d)
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


def check(got, ref, dtype, what):
    errs = {key: rel_err(row, ref[key[0]][key[1]]) for key, row in got.items()}
    worst = max(errs, key=errs.get)
    assert errs[worst] < TOL[dtype], f"{what}: {worst}: {errs[worst]:.3e}"


CUTS = {
    "whole": traces.whole,
    "decode_tail": lambda r: traces.decode_tail(r, tail=24),
    "portions": lambda r: traces.portions(r, sizes=(7, 2, 5, 3, 16, 2, 11, 4)),
    "mixed": lambda r: traces.mixed(r, max_live=4, seed=3, stagger=2),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("cut", list(CUTS))
def test_cut_matches_plain(case, case16, cut, dtype):
    tiny, d, reqs, ref = case if dtype == "float32" else case16
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
    if pages:
        assert sum(1 for users in pages.values() if len(users) >= 2) >= 2, pages


def test_first_step_of_one_token_and_requests_left_out(case):
    """A request whose first step is a single token (the bigram row of a first token, the convolution's
    zeros before the start, a window that holds one key), then portions beside another request that
    decodes and is left out of some steps."""
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
    got, _ = run_cut(tiny, d, steps, "float32")
    check(got, ref, "float32", "first token alone")


def test_long_decoding_float32(case):
    """A short prompt and 170 decoded tokens: windows pass over decoded tokens many times, pages of a
    windowed cache are given back and taken again, the recurrent state is carried all the way."""
    tiny, d, _, _ = case
    toks = random_tokens(190, tiny["cfg"].vocab_size, 77)
    ref = {"long": plain.forward(tiny["cfg"].to_dict(), read_weights(d), toks).numpy()}
    steps = traces.decode_tail({"long": toks}, tail=170)
    got, _ = run_cut(tiny, d, steps, "float32")
    check(got, ref, "float32", "long decoding")


def test_long_requests_wide_windows_over_pages(tmp_path):
    """Requests of a few hundred tokens through windows of 70 and 130 over pages of 16: the tensor-core
    attention walks several blocks of keys whose first and last are cut by the window, the windowed
    group gives pages back while a request is still fed, and the reader of the shared cache looks
    further back than the layer that writes it."""
    from tests.kogonex_tiny import KOGO_LONG
    tiny = KOGO_LONG
    reqs = {f"L{i}": random_tokens(n, tiny["cfg"].vocab_size, 600 + i) for i, n in enumerate([330, 260, 150])}
    cuts = {"whole": traces.whole, "decode_tail": lambda r: traces.decode_tail(r, tail=90),
            "portions": lambda r: traces.portions(r, sizes=(64, 3, 2, 128, 29, 16, 2, 70)),
            "mixed": lambda r: traces.mixed(r, max_live=3, seed=5, max_portion=80, stagger=1)}
    for dtype, decisive in (("float32", False), ("bfloat16", True)):
        d = make_model_dir(tmp_path / dtype, tiny, decisive=decisive)
        w = read_weights(d)
        ref = {rid: plain.forward(tiny["cfg"].to_dict(), w, toks).numpy() for rid, toks in reqs.items()}
        for cut, build in cuts.items():
            got, runner = run_cut(tiny, d, build(reqs), dtype)
            assert len(got) == sum(len(t) for t in reqs.values())
            check(got, ref, dtype, f"long, {cut}")


def follows_plain(cfg, w, prompt, ids, slack):
    logits = plain.forward(cfg.to_dict(), w, ids[:-1])
    return all(float(logits[i - 1].max() - logits[i - 1][ids[i]]) <= slack for i in range(len(prompt), len(ids)))


@pytest.mark.parametrize("dtype,slack", [("float32", 1e-4), ("bfloat16", 0.15)])
def test_greedy_generation_through_the_engine(case, case16, dtype, slack):
    """``generate``: the scheduler with a token budget (prompts cut into portions beside decoding
    requests), sampling on the device, a step ahead of the host."""
    from acorninfer_b200 import generate
    tiny, d, _, _ = case if dtype == "float32" else case16
    cfg = tiny["cfg"]
    w = read_weights(d)
    prompts = [random_tokens(n, cfg.vocab_size, 900 + n) for n in (1, 14, 23, 6, 31)]
    outs = generate(d, prompts, max_new_tokens=12, temperature=0.0, dtype=dtype, page_size=tiny["page_size"],
                    num_blocks=64, max_running=3, chunked_budget=10, watermark_blocks=0, eos_ids=())
    for p, ids in zip(prompts, outs):
        assert len(ids) == len(p) + 12 and follows_plain(cfg, w, p, ids, slack), (dtype, len(p))


def test_preemption_recomputes_state_float32(case):
    """So few pages that requests are preempted and recomputed from their first token: the recurrent
    state and the bigram's previous token start over with the slot."""
    from acorninfer_b200.generation import build_engine, generate_with_engine
    tiny, d, _, _ = case
    cfg = tiny["cfg"]
    prompts = [random_tokens(n, cfg.vocab_size, 40 + n) for n in (20, 18, 13)]
    roomy = build_engine(d, dtype="float32", page_size=tiny["page_size"], num_blocks=64, watermark_blocks=0, max_running=3)
    want = generate_with_engine(roomy, prompts, max_new_tokens=16, eos_ids=())
    pages = -(-36 // tiny["page_size"]) * 2 + 1
    tight = build_engine(d, dtype="float32", page_size=tiny["page_size"], num_blocks=pages, watermark_blocks=0, max_running=3)
    got = generate_with_engine(tight, prompts, max_new_tokens=16, eos_ids=())
    w = read_weights(d)
    for p, a, b in zip(prompts, got, want):
        assert follows_plain(cfg, w, p, a, 1e-4) and follows_plain(cfg, w, p, b, 1e-4)


# ------------------------------------------------------------------ one mechanism at a time


def _solo(mixer, mlp=None, width=48, vocab=90, bigram=False):
    return KogonexConfig(vocab_size=vocab, hidden_size=width, norm_eps=1e-5, layers=(KogonexLayer(mixer, mlp),),
                         bigram_buckets=13 if bigram else None, bigram_mul_prev=9 if bigram else 0,
                         bigram_mul_cur=4 if bigram else 0)


_TINY_DELTA = ChannelDeltaConfig(heads=1, kv_heads=1, dim=4, vdim=4, conv=1, decay_rank=2, gate_rank=2)
SOLOS = {
    "delta rule, grouped heads, 4 taps": _solo(ChannelDeltaConfig(heads=6, kv_heads=2, dim=10, vdim=28, conv=4, decay_rank=3, gate_rank=5)),
    "delta rule, heads of 72 key channels": _solo(ChannelDeltaConfig(heads=1, kv_heads=1, dim=72, vdim=8, conv=2, decay_rank=4, gate_rank=4)),
    "delta rule, heads of 136 key channels": _solo(ChannelDeltaConfig(heads=2, kv_heads=1, dim=136, vdim=20, conv=3, decay_rank=4, gate_rank=4)),
    "latent attention, window 5, scaled positions": _solo(LatentAttentionConfig(
        heads=3, dim=8, rot_dim=6, vdim=10, kv_rank=12, scale=0.4, rot_dims=6, rot_base=100.0,
        scaling=RotaryScaling(3.0, 8, 2.0, 0.5), window=5)),
    "latent attention, no window, no rotated part": _solo(LatentAttentionConfig(
        heads=2, dim=16, rot_dim=0, vdim=8, kv_rank=24, scale=0.3, rot_dims=0, rot_base=1e4, window=None)),
    "experts in groups with identity experts": _solo(_TINY_DELTA, RoutedExpertsConfig(ff=20, experts=9, identity=3, top=4, groups=6, keep=3)),
    "one expert of one": _solo(_TINY_DELTA, RoutedExpertsConfig(ff=12, experts=1, identity=0, top=1)),
    "identity experts only": _solo(_TINY_DELTA, RoutedExpertsConfig(ff=12, experts=0, identity=4, top=2, groups=2, keep=2)),
    "bigram rows": _solo(_TINY_DELTA, None, bigram=True),
}


@pytest.mark.parametrize("name", list(SOLOS))
def test_mechanism_alone(name, tmp_path):
    tiny = dict(cfg=SOLOS[name], page_size=4, seed=5)
    d = make_model_dir(tmp_path, tiny, sigma=0.3)
    w = read_weights(d)
    reqs = {f"s{i}": random_tokens(n, tiny["cfg"].vocab_size, 50 + i) for i, n in enumerate([26, 17, 9])}
    ref = {rid: plain.forward(tiny["cfg"].to_dict(), w, toks).numpy() for rid, toks in reqs.items()}
    for cut in ("whole", "portions", "mixed"):
        got, _ = run_cut(tiny, d, CUTS[cut](reqs) if cut != "portions" else traces.portions(reqs, sizes=(3, 2, 6, 2)), "float32")
        check(got, ref, "float32", f"{name}, {cut}")


def ops():
    from acorninfer_b200.kernels import ops as o
    return o


@pytest.mark.parametrize("N,top,groups,keep", [(16, 3, 2, 1), (12, 2, 4, 2), (7, 7, 1, 1), (64, 6, 8, 3), (33, 1, 3, 3), (5, 2, 5, 2)])
def test_router_choice_matches_plain(N, top, groups, keep):
    g = torch.Generator().manual_seed(N * 100 + top)
    z = torch.randn(200, N, generator=g) * 2
    corr = torch.randn(N, generator=g) * 0.05
    idx, wts = ops().moe_route(z.to(DEV), corr.to(DEV), top, groups, keep)
    idx, wts = idx.cpu(), wts.cpu()
    r = {"top": top, "groups": {"count": groups, "keep": keep}}
    for t in range(z.shape[0]):
        want = plain.route(r, z[t].double(), corr.double())
        assert [e for e, _ in want] == idx[t].tolist(), t
        assert max(abs(float(a) - float(b)) for (_, a), b in zip(want, wts[t])) < 1e-6


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-4), (torch.bfloat16, 0.15)])
@pytest.mark.parametrize("E,T,top,min_rows", [(7, 90, 2, None), (2, 300, 2, None), (12, 5, 2, None), (3, 400, 2, 10 ** 9)])
def test_grouped_products_take_each_experts_own_rows(dtype, tol, E, T, top, min_rows, monkeypatch):
    """Rows scattered over experts, some experts with no rows and some with more than a tile: every
    row against its own expert's matrix.  In bfloat16 the second shape has enough rows an expert for the
    tcgen05 kernel (tiles of 128 rows, an expert's last tile partly another's rows); the others, and the
    last with that kernel switched off, take the three tile heights of the mma.sync kernel (64, 16, 128)."""
    o = ops()
    if min_rows is not None:
        monkeypatch.setattr(o, "GROUPED_TCGEN05_MIN_ROWS", min_rows)
    g = torch.Generator().manual_seed(2)
    N, K = 50, 40
    idx = torch.randint(0, E + 2, (T, top), generator=g, dtype=torch.int32)       # two more outputs: identity experts
    idx[idx == 1] = 0                                                              # expert 1 gets nothing
    x = torch.randn(T, K, generator=g).to(dtype)
    w = torch.randn(E, N, K, generator=g).to(dtype)
    offsets, slot_of, slot_token = o.moe_plan(idx.to(DEV), E + 2)
    out = o.grouped_gemm(x.to(DEV), slot_token, w.to(DEV), offsets, T * top).float().cpu()
    off = offsets.cpu().tolist()
    assert off[-1] == T * top and off[2] == off[1]
    so = slot_of.cpu()
    for t in range(T):
        for k in range(top):
            e, s = int(idx[t, k]), int(so[t, k])
            assert off[e] <= s < off[e + 1]
            if e < E:
                assert (out[s] - x[t].float() @ w[e].float().T).abs().max() < tol
    # gate and up rows in turns: silu(gate) * up from the product's own epilogue (bfloat16) or the kernel after it
    act = o.grouped_gemm(x.to(DEV), slot_token, w.to(DEV), offsets, T * top, swiglu_pairs=True).float().cpu()
    assert act.shape == (T * top, N // 2)
    for t in range(0, T, 7):
        e, s = int(idx[t, 0]), int(so[t, 0])
        if e < E:
            gu = x[t].float() @ w[e].float().T
            want = torch.nn.functional.silu(gu[0::2]) * gu[1::2]
            assert (act[s] - want).abs().max() < tol * 4, (t, e)


def _latent_case(befores, qlens, P, d, dv, nq, window, spikes, dtype, sink_value=None, seed=0, kernel="plain"):
    """Cache rows and queries for ``attention_plain`` in the latent layout (one kv head, values = the
    first dv entries of the key rows).  ``spikes``: (row, key position): that key and all queries of the
    row get a large component along one direction, so its score stands out wherever it is seen."""
    g = torch.Generator().manual_seed(seed)
    NP = sum(-(-(b + q) // P) for b, q in zip(befores, qlens)) + 5
    lay = rows_layout(befores, qlens, P, NP, seed=seed)
    pages = torch.zeros(NP, 1, P, d, dtype=dtype, device=DEV)
    full_q, full_k = [], []
    for r, (b, q) in enumerate(zip(befores, qlens)):
        S = b + q
        k = torch.randn(S, 1, d, generator=g) * 0.3
        qq = torch.randn(S, nq, d, generator=g) * 0.3
        for (rr, j) in spikes:
            if rr == r:
                k[j, 0, d - 1] = 6.0
                qq[:, :, d - 1] = 4.0
        k = k.to(dtype).double()
        qq = qq.to(dtype).double()
        scatter_to_pages(pages, lay["tables"][r], k.to(dtype), P)
        full_q.append(qq)
        full_k.append(k)
    q_new = torch.cat([fq[b:] for fq, b in zip(full_q, befores)]).to(dtype).to(DEV).contiguous()
    sink = None if sink_value is None else torch.full((nq,), float(sink_value)) + torch.arange(nq) * 0.5
    scale = 0.5
    if kernel == "tc":
        o = ops()
        assert o.latent_attention_tc_supported(dtype, nq, d, dv, P)
        n = o.LATENT_TILE_ROWS // nq
        i32 = dict(dtype=torch.int32, device=DEV)
        tiles = torch.tensor([(r, q0) for r, length in enumerate(qlens) for q0 in range(0, length, n)], **i32)
        args = (q_new, pages, lay["block_table"], lay["page_base"], torch.tensor(np.cumsum([0] + qlens), **i32),
                torch.tensor(befores, **i32), tiles, None if sink is None else sink.to(DEV), scale, window, dv)
        out = o.latent_attention_tc(*args).float().cpu()
        for splits in (1, 3, 7):              # a tile's key blocks shared out over several blocks and merged
            again = o.latent_attention_tc(*args, splits=splits).float().cpu()
            assert (again - out).abs().max() < 2e-2, splits
    else:
        out = ops().attention_plain(q_new.view(-1, nq * d), nq * d, pages, pages, lay["block_table"], lay["page_base"],
                                    lay["token_row"], lay["positions"], lay["num_tokens"], nq, 1, d, scale, window,
                                    value_dim=dv, sink32=None if sink is None else sink.to(DEV)).float().cpu()
    want = []
    for fq, fk, b in zip(full_q, full_k, befores):
        heads = []
        for h in range(nq):
            s = fq[:, h] @ fk[:, 0].T * scale
            p = plain.windowed_sink_softmax(s, torch.tensor(-1e30, dtype=torch.float64) if sink is None else sink[h].double(), window)
            heads.append(p @ fk[:, 0, :dv])
        want.append(torch.stack(heads, 1)[b:])
    return out.view(-1, nq, dv), torch.cat(want)


@pytest.mark.parametrize("dtype,tol,kernel,d,dv,nq", [(torch.float32, 2e-5, "plain", 24, 16, 3), (torch.bfloat16, 2e-2, "plain", 24, 16, 3),
                                                      (torch.bfloat16, 2e-2, "tc", 32, 16, 3), (torch.bfloat16, 2e-2, "tc", 112, 96, 8),
                                                      (torch.bfloat16, 2e-2, "tc", 160, 144, 16)])
def test_latent_layout_attention_window_edges_far_keys_and_sink(dtype, tol, kernel, d, dv, nq):
    """A key that outweighs all others is seen up to the query window - 1 tokens after it and no
    longer, in a prompt's rows and in single decoded tokens, at page borders; a far key among hundreds
    is found without a window; a sink takes its share of every row."""
    P, W = 16, 64
    # row 0: a whole prompt; row 1: a portion after 130 cached tokens; rows 2-5: single tokens whose
    # window's first key (2, 4) or the key just before it (3, 5) is the spiked one, at a page's border or not
    befores = [0, 130, 15 + W - 1, 15 + W, 16 + W - 1, 16 + W]
    qlens = [300, 90, 1, 1, 1, 1]
    spikes = [(0, 15), (0, 16), (0, 200), (1, 100), (1, 131), (2, 15), (3, 15), (4, 16), (5, 16)]
    got, want = _latent_case(befores, qlens, P, d, dv, nq, W, spikes, dtype, sink_value=0.5, kernel=kernel)
    assert (got - want).abs().max() < tol
    # the spiked key decides the rows that see it: the decoded token of row 2 returns (nearly) its
    # value, the one of row 3, one position later, does not
    lay_tokens = np.cumsum([0] + qlens)
    assert (got[lay_tokens[2]] - got[lay_tokens[3]]).abs().max() > 0.05
    # no window: key 3 of 700 decides a decoded token's result
    got, want = _latent_case([0, 699], [40, 1], P, d, dv, nq, None, [(1, 3)], dtype, kernel=kernel)
    assert (got - want).abs().max() < tol
    # a sink that outweighs the keys leaves almost nothing
    got, want = _latent_case([5], [20], P, d, dv, nq, 8, [], dtype, sink_value=12.0, kernel=kernel)
    assert (got - want).abs().max() < tol and got.abs().max() < 0.05


def test_bigram_rows_carry_the_previous_token_between_steps():
    o = ops()
    buckets, mp, mc, H = 11, 7, 3, 8
    table = torch.arange((buckets + 1) * H, dtype=torch.float32).view(buckets + 1, H).to(DEV)
    state = torch.zeros(3, dtype=torch.int32, device=DEV)
    seqs = {0: [5, 9, 2, 2, 7, 1], 2: [3, 3, 8, 0]}                 # by state slot
    want = {s: plain.bigram_rows(t, buckets, mp, mc) for s, t in seqs.items()}
    cuts = [{0: (0, 2), 2: (0, 1)}, {0: (2, 3)}, {2: (1, 4), 0: (3, 6)}]
    i32 = dict(dtype=torch.int32, device=DEV)
    for cut in cuts:
        ids, row, start, pos, slot = [], [], [0], [], []
        for r, (s, (a, b)) in enumerate(cut.items()):
            ids += seqs[s][a:b]
            row += [r] * (b - a)
            start.append(len(ids))
            pos.append(a)
            slot.append(s)
        x = torch.zeros(len(ids), H, device=DEV)
        o.bigram_add(x, torch.tensor(ids, **i32), torch.tensor(row, **i32), torch.tensor(start, **i32),
                     torch.tensor(pos, **i32), torch.tensor(slot, **i32), state, table, buckets, mp, mc)
        got = (x[:, 0] / H).round().int().tolist()
        t = 0
        for s, (a, b) in cut.items():
            assert got[t:t + b - a] == want[s][a:b], (cut, s)
            t += b - a
