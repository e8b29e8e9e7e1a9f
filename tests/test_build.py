"""The library builder's housekeeping (no compiler needed)."""

import os

from freetoken_b200.csrc import build


def test_dropping_older_binaries_leaves_libraries_with_longer_names_alone(tmp_path):
    names = ["libft_attention_decode_0123456789abcdef.so", "libft_attention_decode_fedcba9876543210.so",
             "libft_attention_decode_tma_0123456789abcdef.so", "libft_attention_decoder_0123456789abcdef.so",
             "notes.txt"]
    for n in names:
        (tmp_path / n).write_bytes(b"")
    keep = str(tmp_path / names[1])
    removed = build.drop_stale(str(tmp_path), "attention_decode", keep)
    assert removed == [names[0]]
    assert sorted(os.listdir(tmp_path)) == sorted(names[1:])


def test_every_library_has_its_source_and_a_digest():
    for name, src in build.LIBRARIES.items():
        assert os.path.exists(os.path.join(build.HERE, src)), name
        assert len(build._digest(name)) == 16
    for header in build.HEADERS:
        assert os.path.exists(os.path.join(build.HERE, header)), header
