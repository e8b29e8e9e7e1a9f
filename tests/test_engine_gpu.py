"""The engine against the plain implementation: whole, decoded tail, portions,
mixed batches with page reuse; in float32 and bfloat16; two (three) tiny
configurations that differ in every size and option."""


import pytest
import torch

import replay_driver as rd
import tiny
from plain_model import PlainModel

pytestmark = pytest.mark.gpu

LENGTHS = {"A": [5, 9, 17, 70], "B": [1, 6, 13, 31, 80], "C": [3, 40, 66, 90, 21], "D": [2, 35, 77],
           "E": [2, 140, 300, 70], "F": [4, 50, 27]}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for which in tiny.TINY:
        folder = str(tmp_path_factory.mktemp(f"tiny{which}"))
        tiny.write_tiny(folder, which)
        out[which] = folder
    return out


@pytest.fixture(scope="module")
def expected(models):
    """Whole-sequence logits of the plain implementation, per model, dtype, request."""
    cache = {}

    def get(which, dtype):
        key = (which, dtype)
        if key not in cache:
            plain = PlainModel(models[which], dtype)
            cache[key] = {rid: plain.forward(toks) for rid, toks in requests_of(which).items()}
        return cache[key]
    return get


def requests_of(which):
    vocab = tiny.TINY[which]["vocab_size"]
    return {f"r{i}": tiny.tokens(100 * i + len(which), n, vocab) for i, n in enumerate(LENGTHS[which])}


def make_engine(folder, dtype, page, max_tokens, live=4, poison=False):
    from freetoken_b200.engine import Engine, EngineArgs
    return Engine.from_folder(folder, EngineArgs(dtype=dtype, page_size=page,
                                                 num_pages=-(-max_tokens // page),
                                                 max_running_requests=live, poison_freed_pages=poison))


# In bfloat16 the discrete choice of experts may differ between two correct
# implementations where two experts' scores lie within rounding of each other.
# The bfloat16 comparisons therefore hand the engine's choice to the plain
# implementation (everything else is still computed by it) and check separately
# that the two choices differ only where the plain implementation's own margin
# is small.  float32 comparisons use the plain implementation's own choice.
MARGIN = 5e-3


def plain_logits(models, which, dtype, reqs, routing=None):
    plain = PlainModel(models[which], dtype)
    out = {}
    for rid, toks in reqs.items():
        forced = None if routing is None else routing[rid]
        out[rid] = plain.forward(toks, forced)
        if routing is not None:
            for layer, (own, margin) in enumerate(plain.routing):
                differ = (own.sort(-1).values != forced[layer].long().sort(-1).values).any(-1)
                assert (margin[differ] < MARGIN).all(), (
                    f"{which} request {rid} layer {layer}: the engine chose other experts at "
                    f"positions {differ.nonzero().flatten().tolist()} with margins {margin[differ].tolist()}")
                assert differ.float().mean() <= 0.25, f"too many routing differences in layer {layer}"
    return out


def compare(got, want, dtype, what):
    for rid in want:
        g, w = got[rid], want[rid]
        assert not torch.isnan(g).any(), f"{what}: request {rid} has positions without logits"
        bad = ~torch.isclose(g, w, **tiny.TOL[dtype])
        if bad.any():
            pos = int(bad.any(dim=1).nonzero()[0])
            err = (g - w).abs().max().item()
            raise AssertionError(
                f"{what} [{dtype}] request {rid}: first wrong position {pos} of {len(w)}, "
                f"max abs error {err:.3e}")


CUTS = {"whole": rd.whole, "decode_tail": rd.decode_tail, "portions": rd.portions, "mixed": rd.mixed}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", ["A", "B", "C", "D", "F"])
@pytest.mark.parametrize("cut", list(CUTS))
def test_cut_matches_plain(models, expected, which, dtype, cut):
    reqs = requests_of(which)
    schedule = CUTS[cut](reqs)
    page = tiny.PAGE[which]
    # exactly as many pages as the schedule's peak needs: pages are reused
    engine = make_engine(models[which], dtype, page, rd.peak_tokens(schedule, page))
    if dtype == "float32":
        got = rd.run_engine(engine, reqs, schedule)
        want = expected(which, dtype)
    else:
        routing = {}
        got = rd.run_engine(engine, reqs, schedule, routing)
        want = plain_logits(models, which, dtype, reqs, routing)
    compare(got, want, dtype, cut)
    assert engine.cache.free_pages() == engine.cache.total_pages()


@pytest.mark.parametrize("cut", list(CUTS))
def test_tcgen05_prefill_attention_in_the_engine(models, cut, monkeypatch):
    """Head size 64, pages of 64: every prompt portion, however short, goes
    through the tcgen05 / TMA attention kernel (its size threshold set to 0)."""
    from freetoken_b200.csrc import ops
    calls = []
    real = ops.attn_prefill_tc
    monkeypatch.setattr(ops, "PREFILL_TC_MIN_SCORES", 0)
    monkeypatch.setattr(ops, "MOE_SORT_CHUNKED_FROM", 1)      # and the chunked route sort
    monkeypatch.setattr(ops, "attn_prefill_tc", lambda *a, **k: (calls.append(1), real(*a, **k))[1])
    which, dtype = "E", "bfloat16"
    reqs = requests_of(which)
    schedule = CUTS[cut](reqs)
    page = tiny.PAGE[which]
    engine = make_engine(models[which], dtype, page, rd.peak_tokens(schedule, page))
    routing = {}
    got = rd.run_engine(engine, reqs, schedule, routing)
    ops.check_tc_status(engine.device)
    assert calls, "the tcgen05 attention kernel never ran"
    compare(got, plain_logits(models, which, dtype, reqs, routing), dtype, cut)
    assert engine.cache.free_pages() == engine.cache.total_pages()


@pytest.mark.parametrize("which,dtype", [("A", "float32"), ("C", "bfloat16"), ("E", "bfloat16"), ("E", "float32")])
def test_stale_pages_are_never_read(models, expected, which, dtype, monkeypatch):
    """The mixed schedule again (pages reused while requests come and go), with
    every free page filled with NaN: whenever it is free, a page is unreadable,
    so any read of stale data - a masked key's V row times a zero weight
    included - would turn logits into NaN.  tiny-E goes through the TMA-fed
    attention kernels, which fetch whole 64-key boxes of a page."""
    from freetoken_b200.csrc import ops
    if which == "E":
        monkeypatch.setattr(ops, "PREFILL_TC_MIN_SCORES", 0)
    reqs = requests_of(which)
    schedule = rd.mixed(reqs)
    page = tiny.PAGE[which]
    engine = make_engine(models[which], dtype, page, rd.peak_tokens(schedule, page), poison=True)
    if dtype == "float32":
        got = rd.run_engine(engine, reqs, schedule)
        want = expected(which, dtype)
    else:
        routing = {}
        got = rd.run_engine(engine, reqs, schedule, routing)
        want = plain_logits(models, which, dtype, reqs, routing)
    compare(got, want, dtype, "mixed, free pages poisoned")
    pool = engine.storage.paged[0]
    assert torch.isnan(pool[:, :, 1:].float()).all(), "a page that was given back is not poisoned"


@pytest.mark.parametrize("which", ["A", "B"])
def test_float32_cuts_agree_bitwise(models, which):
    """In float32 the logits at a position do not depend on the cut at all."""
    reqs = requests_of(which)
    page = tiny.PAGE[which]
    results = {}
    for cut, fn in CUTS.items():
        schedule = fn(reqs)
        engine = make_engine(models[which], "float32", page, rd.peak_tokens(schedule, page))
        results[cut] = rd.run_engine(engine, reqs, schedule)
    for cut in ("decode_tail", "portions", "mixed"):
        for rid in reqs:
            assert torch.equal(results[cut][rid], results["whole"][rid]), (cut, rid)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_tool(models, expected, tmp_path, dtype):
    """bin/trace_run as a child process: mixed schedule, scarce pages."""
    which = "B"
    reqs = requests_of(which)
    schedule = rd.mixed(reqs)
    page = 16
    got = rd.run_trace_tool(models[which], dtype, reqs, schedule, str(tmp_path / "out"),
                            rd.peak_tokens(schedule, page), page, tiny.TINY[which]["vocab_size"])
    if dtype == "float32":
        want = expected(which, dtype)
    else:
        # the same schedule in this process gives the experts the tool's run chose
        routing = {}
        engine = make_engine(models[which], dtype, page, rd.peak_tokens(schedule, page))
        same = rd.run_engine(engine, reqs, schedule, routing)
        for rid in reqs:
            assert torch.equal(same[rid], got[rid]), "the tool and the in-process engine differ"
        want = plain_logits(models, which, dtype, reqs, routing)
    compare(got, want, dtype, "trace_run mixed")


def test_decode_batch_on_the_tcgen05_experts_replays_like_it_runs(models, monkeypatch):
    """Twelve requests decoding together on tiny-A: more than four routes per expert, so the
    experts run on the tcgen05 grouped GEMM (tile list, gather and both products inside the
    captured graph).  The replayed steps must give the bits of the eagerly run ones."""
    from freetoken_b200.csrc import ops
    from freetoken_b200.engine import Engine, EngineArgs, StepEntry
    calls = []
    real = ops.moe_experts_tc
    monkeypatch.setattr(ops, "moe_experts_tc", lambda *a, **k: (calls.append(1), real(*a, **k))[1])
    vocab = tiny.TINY_A["vocab_size"]
    ids = [f"r{i}" for i in range(12)]
    prompts = [tiny.tokens(20 + i, 3 + i, vocab) for i in range(12)]
    steps = [[int(t) for t in tiny.tokens(40 + s, 12, vocab)] for s in range(6)]

    def run(max_bs):
        engine = Engine.from_folder(models["A"], EngineArgs(dtype="bfloat16", page_size=4, num_pages=128,
                                                            max_running_requests=12, cuda_graph_max_bs=max_bs))
        engine.step([StepEntry(r, p, []) for r, p in zip(ids, prompts)])
        out = [engine.step([StepEntry(r, [tok], [0]) for r, tok in zip(ids, toks)]).float().cpu() for toks in steps]
        ops.check_tc_status(engine.device)
        return out, engine.graph_replays

    eager, none = run(0)
    assert none == 0 and calls, "the grouped GEMM never ran"
    replayed, replays = run(64)
    assert replays >= 4
    for a, b in zip(eager, replayed):
        assert torch.equal(a, b)
