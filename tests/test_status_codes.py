"""The table of status codes: one header the kernels and the host both read."""

import os
import re

from freetoken_b200.csrc import ops

CSRC = os.path.dirname(os.path.abspath(ops.__file__))


def test_every_code_a_kernel_records_has_a_message():
    header = open(os.path.join(CSRC, "status_codes.h")).read()
    names = dict(re.findall(r"X\((\w+),\s*(\d+),", header))
    assert len(set(names.values())) == len(names), "two roles share a code"
    table = ops._status_table()
    assert sorted(table) == sorted(int(c) for c in names.values())
    used = set()
    for f in os.listdir(CSRC):
        if f.endswith(".cu"):
            text = open(os.path.join(CSRC, f)).read()
            assert not re.search(r"atomicCAS\(a\.status, 0, \d", text), f"{f} records a bare number"
            used |= set(re.findall(r"FT_ST_(\w+)", text))
    assert used and used <= set(names), used - set(names)


def test_messages_name_kernel_and_role():
    assert "attn_decode_tma" in ops.status_message(21) and "producer" in ops.status_message(21)
    assert "moe_gemm_tc" in ops.status_message(4)
    assert "code 99" in ops.status_message(99)
