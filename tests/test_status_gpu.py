"""The failure path of the kernels' bounded waits: a wait that runs out leaves a
code in a device status word, the host turns it into a KernelError that names
kernel and role, and the word is cleared.  Nothing here faults, traps or hangs
the device: the status is written from the host, or a one-block kernel waits a
millisecond on a barrier nobody arrives at and returns.

The reference's counterpart is ``raise_if_unhealthy()`` after every step
(python/freetoken/engine/engine.py:922-925)."""

import time

import pytest
import torch

import tiny

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


@pytest.fixture(autouse=True)
def clean_status():
    from freetoken_b200.csrc import ops
    ops.tc_status(DEV).zero_()
    yield
    ops.tc_status(DEV).zero_()


@pytest.fixture(scope="module")
def folder_a(tmp_path_factory):
    return tiny.write_tiny(str(tmp_path_factory.mktemp("statusA")), "A")


@pytest.mark.parametrize("code,kernel,role", [(2, "moe_gemm_tc", "MMA issuer"), (13, "attn_prefill_tc", "K tile"),
                                              (22, "attn_decode_tma", "consumer"), (77, "a kernel", "a role")])
def test_a_recorded_failure_raises_and_is_cleared(folder_a, code, kernel, role):
    from freetoken_b200.csrc import ops
    from freetoken_b200.engine import Engine, EngineArgs
    engine = Engine.from_folder(folder_a, EngineArgs(dtype="float32", page_size=4, max_tokens=16))
    engine.check_status()                      # nothing recorded: no error
    ops.tc_status(engine.device).fill_(code)
    with pytest.raises(ops.KernelError) as err:
        engine.check_status()
    assert kernel in str(err.value) and role in str(err.value) and f"code {code}" in str(err.value)
    assert int(ops.tc_status(engine.device).item()) == 0
    engine.check_status()


def test_generate_notices_a_failure_in_the_step_that_recorded_it(folder_a):
    """The status word is read with every step's sampled tokens."""
    from freetoken_b200 import LLM, SamplingParams
    from freetoken_b200.csrc import ops
    llm = LLM(folder_a, "float32", page_size=4, num_token_override=64, max_running_req=1)
    prompt = tiny.tokens(1, 5, tiny.TINY_A["vocab_size"])
    llm.generate([prompt], SamplingParams(max_tokens=3, ignore_eos=True))
    steps = llm.engine.steps
    ops.tc_status(llm.engine.device).fill_(3)
    with pytest.raises(ops.KernelError, match="epilogue"):
        llm.generate([prompt], SamplingParams(max_tokens=50, ignore_eos=True))
    # at most the step in flight ran beyond the one whose status was read
    assert llm.engine.steps - steps <= 2
    assert int(ops.tc_status(llm.engine.device).item()) == 0


def test_a_wait_that_runs_out_returns_and_records_its_code():
    from freetoken_b200.csrc import ops
    status = ops.tc_status(DEV)
    # somebody arrives: the wait succeeds, nothing is recorded
    ops.wait_selftest(DEV, 1_000_000, arrive=True)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    # nobody arrives: the wait gives up after its millisecond and the kernel returns
    start = time.time()
    ops.wait_selftest(DEV, 1_000_000, arrive=False)
    torch.cuda.synchronize()
    assert time.time() - start < 1.0
    assert int(status.item()) == 31
    with pytest.raises(ops.KernelError, match="wait_selftest"):
        ops.check_tc_status(DEV)
    assert int(status.item()) == 0
    # the first failure is the one that is kept
    status.fill_(11)
    ops.wait_selftest(DEV, 100_000, arrive=False)
    torch.cuda.synchronize()
    assert int(status.item()) == 11
    # the device is as usable as before
    assert float((torch.ones(8, device=DEV) * 2).sum()) == 16.0
