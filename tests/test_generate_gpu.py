"""Generation through the Python entry point: greedy tokens equal to the plain
implementation's greedy loop, long decoding (graph replay included), sampling."""

import pytest
import torch

import tiny
from generation_check import check_generation
from plain_model import PlainModel

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def folder_a(tmp_path_factory):
    return tiny.write_tiny(str(tmp_path_factory.mktemp("genA")), "A")


@pytest.fixture(scope="module")
def folder_c(tmp_path_factory):
    return tiny.write_tiny(str(tmp_path_factory.mktemp("genC")), "C")


@pytest.fixture(scope="module")
def folder_b(tmp_path_factory):
    return tiny.write_tiny(str(tmp_path_factory.mktemp("genB")), "B")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_tiny_b_workload_against_a_plain_sampling_loop(folder_b, dtype):
    """tiny-B (tied head, softmax routing, 3 KV heads of 24): four requests with
    prompts of 1/6/13/31 tokens in portions of at most 7, temperature 0.8 at seed 3,
    6 new tokens each, pages of 8.  The test draws the same uniform numbers from the
    request's generator and requires the tokens of a plain softmax(logits/T) +
    inverse-CDF loop over the plain model."""
    from freetoken_b200 import LLM, SamplingParams
    from freetoken_b200.sampling.sampler import RequestRng
    vocab = tiny.TINY_B["vocab_size"]
    prompts = [tiny.tokens(s, n, vocab) for s, n in ((1, 1), (2, 6), (3, 13), (4, 31))]
    params = SamplingParams(temperature=0.8, max_tokens=6, ignore_eos=True, seed=3)
    llm = LLM(folder_b, dtype, page_size=8, num_token_override=160, max_running_req=4,
              max_extend_tokens=7)
    out = llm.generate(prompts, params)
    plain = PlainModel(folder_b, dtype)
    ties = 0
    for prompt, result in zip(prompts, out):
        rng = RequestRng(3)
        uniforms = [rng.next_uniform() for _ in range(6)]
        assert len(result["token_ids"]) == 6
        ties += check_generation(plain, prompt, result["token_ids"], dtype, 0.8, uniforms)
    # a vocabulary of 384 near-uniform tokens puts a boundary within about 1e-3 of most
    # draws, so bfloat16 may land next door often; float32 may not at all
    assert dtype == "bfloat16" or ties == 0, f"{ties} of 24 tokens were decided by a tie"
    llm.scheduler.check_integrity()
    assert llm.engine.cache.free_pages() == llm.engine.cache.total_pages()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", ["B", "C"])
def test_greedy_generation_against_the_plain_model(folder_b, folder_c, which, dtype):
    from freetoken_b200 import LLM, SamplingParams
    folder = {"B": folder_b, "C": folder_c}[which]
    vocab = tiny.TINY[which]["vocab_size"]
    prompts = [tiny.tokens(s, n, vocab) for s, n in ((5, 3), (6, 11), (7, 26))]
    llm = LLM(folder, dtype, page_size=tiny.PAGE[which], num_token_override=192, max_running_req=3,
              max_extend_tokens=9)
    out = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True))
    plain = PlainModel(folder, dtype)
    ties = sum(check_generation(plain, p, r["token_ids"], dtype) for p, r in zip(prompts, out))
    assert ties == 0 if dtype == "float32" else ties < 12, f"{ties} of 24 tokens were decided by a tie"


def test_greedy_generation_float32(folder_a):
    """tiny-A workload: prompts of 5/9/17 tokens, 8 new tokens each, page size 4."""
    from freetoken_b200 import LLM, SamplingParams
    vocab = tiny.TINY_A["vocab_size"]
    prompts = [tiny.tokens(s, n, vocab) for s, n in ((1, 5), (2, 9), (3, 17))]
    llm = LLM(folder_a, "float32", page_size=4, num_token_override=96, max_running_req=3)
    out = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True))
    plain = PlainModel(folder_a, "float32")
    for prompt, result in zip(prompts, out):
        assert result["token_ids"] == plain.greedy(prompt, 8)
        assert result["finish_reason"] == "length"
    llm.scheduler.check_integrity()
    assert llm.engine.cache.free_pages() == llm.engine.cache.total_pages()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_matches_whole_sequence(folder_c, dtype):
    """Decode 150 tokens one by one (graph replay in bfloat16), then run prompt +
    generated tokens whole through a fresh engine: the logits that chose every
    token must agree, and so must the greedy choice unless two logits tie."""
    from freetoken_b200 import LLM, SamplingParams
    from freetoken_b200.engine import Engine, EngineArgs, StepEntry
    vocab = tiny.TINY_C["vocab_size"]
    prompts = [tiny.tokens(5, 33, vocab), tiny.tokens(6, 7, vocab)]
    llm = LLM(folder_c, dtype, page_size=16, num_token_override=512, max_running_req=2)
    out = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=150, ignore_eos=True))
    if dtype == "bfloat16":
        assert llm.engine.graph_replays > 100
    engine = Engine.from_folder(folder_c, EngineArgs(dtype=dtype, page_size=16, max_tokens=512,
                                                     max_running_requests=2))
    for prompt, result in zip(prompts, out):
        gen = result["token_ids"]
        assert len(gen) == 150
        seq = prompt + gen
        logits = engine.step([StepEntry("w", seq[:-1], list(range(len(prompt) - 1, len(seq) - 1)))])
        engine.end_request("w")
        logits = logits.float().cpu()
        top2 = logits.topk(2, dim=-1).values
        clear = (top2[:, 0] - top2[:, 1]) > (1e-4 if dtype == "float32" else 5e-2)
        greedy = logits.argmax(-1)
        agree = greedy == torch.tensor(gen)
        assert agree[clear].all(), f"decoded tokens differ from whole-sequence greedy at {(~agree & clear).nonzero().flatten().tolist()}"


def test_first_tokens_of_a_sequence(folder_a):
    """Positions 0 and 1: one key, no history, first slot of the first page."""
    from freetoken_b200.engine import Engine, EngineArgs, StepEntry
    plain = PlainModel(folder_a, "float32")
    engine = Engine.from_folder(folder_a, EngineArgs(dtype="float32", page_size=4, max_tokens=16,
                                                     max_running_requests=2))
    toks = tiny.tokens(9, 3, tiny.TINY_A["vocab_size"])
    want = plain.forward(toks)
    got0 = engine.step([StepEntry("a", toks[:1], [0])]).cpu().clone()
    got1 = engine.step([StepEntry("a", toks[1:2], [0])]).cpu().clone()
    got2 = engine.step([StepEntry("a", toks[2:3], [0])]).cpu().clone()
    assert torch.allclose(torch.cat([got0, got1, got2]), want, **tiny.TOL["float32"])


def test_temperature_sampling_is_reproducible_and_batch_independent(folder_a):
    """tiny-B style workload: temperature 0.8, seeds per request; a request's
    tokens do not depend on what else is in the batch."""
    from freetoken_b200 import LLM, SamplingParams
    vocab = tiny.TINY_A["vocab_size"]
    prompts = [tiny.tokens(s, n, vocab) for s, n in ((1, 1), (2, 6), (3, 13), (4, 31))]
    params = [SamplingParams(temperature=0.8, max_tokens=6, ignore_eos=True, seed=3 + i) for i in range(4)]
    llm = LLM(folder_a, "float32", page_size=8, num_token_override=256, max_running_req=4,
              max_extend_tokens=7)
    together = llm.generate(prompts, params)
    again = llm.generate(prompts, params)
    assert [r["token_ids"] for r in together] == [r["token_ids"] for r in again]
    alone = [llm.generate([p], [sp])[0] for p, sp in zip(prompts, params)]
    assert [r["token_ids"] for r in together] == [r["token_ids"] for r in alone]
    assert any(r["token_ids"] != llm.generate([p], SamplingParams(max_tokens=6, ignore_eos=True))[0]["token_ids"]
               for r, p in zip(together, prompts)), "temperature sampling never left the greedy path"


def test_eos_stops_generation(folder_a):
    from freetoken_b200 import LLM, SamplingParams
    vocab = tiny.TINY_A["vocab_size"]
    prompt = tiny.tokens(1, 5, vocab)
    llm = LLM(folder_a, "float32", page_size=4, num_token_override=64, max_running_req=1)
    free = llm.generate([prompt], SamplingParams(max_tokens=8, ignore_eos=True))[0]["token_ids"]
    stop_at = free[3]
    if stop_at in free[:3]:
        pytest.skip("the chosen stop token appears earlier")
    # a stop token that is no EOS ends the request and stays in the answer
    # (python/freetoken/llm/llm.py:101-103 drops EOS ids only)
    out = llm.generate([prompt], SamplingParams(max_tokens=8, stop_token_ids=[stop_at]))[0]
    assert out["token_ids"] == free[:4] and out["finish_reason"] == "stop"
    # the same token as the model's EOS: dropped
    llm.eos_token_ids = [stop_at]
    llm.scheduler.eos = {stop_at}
    out = llm.generate([prompt], SamplingParams(max_tokens=8))[0]
    assert out["token_ids"] == free[:3] and out["finish_reason"] == "stop"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_overlapped_scheduling_gives_the_same_tokens(folder_c, dtype, monkeypatch):
    """Steps launched before the previous step's tokens are read (inputs handed on
    on the device, results read one step late) against the synchronous loop:
    greedy and seeded sampling, stops on a token in mid-flight, more requests
    than slots so that pages and slots are reused."""
    from freetoken_b200 import LLM, SamplingParams
    vocab = tiny.TINY_C["vocab_size"]
    prompts = [tiny.tokens(20 + i, n, vocab) for i, n in enumerate((3, 18, 40, 9, 27, 5))]
    llm = LLM(folder_c, dtype, page_size=16, num_token_override=256, max_running_req=3,
              max_extend_tokens=24)

    def both(params):
        monkeypatch.setenv("FREETOKEN_DISABLE_OVERLAP_SCHEDULING", "1")
        sync = llm.generate(prompts, params)
        monkeypatch.setenv("FREETOKEN_DISABLE_OVERLAP_SCHEDULING", "0")
        replays = llm.engine.graph_replays
        over = llm.generate(prompts, params)
        llm.scheduler.check_integrity()
        assert llm.engine.cache.free_pages() == llm.engine.cache.total_pages()
        return sync, over, llm.engine.graph_replays - replays

    greedy = [SamplingParams(max_tokens=12 + 3 * i, ignore_eos=True) for i in range(len(prompts))]
    sync, over, replays = both(greedy)
    assert [r["token_ids"] for r in sync] == [r["token_ids"] for r in over]
    if dtype == "bfloat16":
        assert replays > 0, "decode-only steps of the overlapped loop did not replay a graph"
    # stop on a token that the free run produced in the middle of two requests
    stops = []
    for r in sync:
        t = r["token_ids"]
        stops.append([t[5]] if len(t) > 5 else [])
    stopping = [SamplingParams(max_tokens=p.max_tokens, stop_token_ids=s) for p, s in zip(greedy, stops)]
    sync2, over2, _ = both(stopping)
    assert [(r["token_ids"], r["finish_reason"]) for r in sync2] == \
        [(r["token_ids"], r["finish_reason"]) for r in over2]
    assert any(r["finish_reason"] == "stop" for r in sync2)
    sampled = [SamplingParams(temperature=0.9, top_p=0.95, max_tokens=10, ignore_eos=True, seed=7 + i)
               for i in range(len(prompts))]
    sync3, over3, _ = both(sampled)
    assert [r["token_ids"] for r in sync3] == [r["token_ids"] for r in over3]


def test_status_lines_nvtx_ranges_and_the_default_pool(folder_a):
    """The scheduler's throughput lines reach the caller's log function, NVTX ranges
    change no token, and an engine that is given no pool size takes one from the free
    memory: enough pages for every running request at the longest sequence, no more."""
    from freetoken_b200 import LLM, SamplingParams
    vocab = tiny.TINY_A["vocab_size"]
    prompts = [tiny.tokens(s, n, vocab) for s, n in ((1, 5), (2, 19))]
    params = SamplingParams(max_tokens=9, ignore_eos=True)
    lines = []
    plain = LLM(folder_a, "float32", page_size=4, num_token_override=128, max_running_req=2,
                max_extend_tokens=8).generate(prompts, params)
    llm = LLM(folder_a, "float32", page_size=4, max_running_req=2, max_extend_tokens=8,
              log_status=lines.append, decode_log_interval=2, nvtx=True)
    out = llm.generate(prompts, params)
    assert [r["token_ids"] for r in out] == [r["token_ids"] for r in plain]
    assert sum(l.startswith("Prefill batch, #new-seq:") for l in lines) >= 3      # 24 prompt tokens, 8 a step
    assert any(l.startswith("Decode batch, #running-req:") for l in lines)
    cache = llm.engine.cache
    per_request = -(-tiny.TINY_A["max_position_embeddings"] // 4)
    assert cache.total_pages() == [2 * per_request]
    assert llm.engine.max_seq_len == tiny.TINY_A["max_position_embeddings"]
    assert cache.free_pages() == cache.total_pages()
