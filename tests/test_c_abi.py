"""The C ABI without a GPU: the shared library loads, exports every function that
include/sah_b200.h declares, the ctypes table covers the same set, and entry points refuse
bad arguments with a status and a message instead of launching anything."""

import ctypes
import re
from pathlib import Path

import pytest

from sparse_attention_hub import _native

HEADER = Path(__file__).resolve().parent.parent / "include" / "sah_b200.h"


def _declared():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(sah_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_function():
    lib = _native.load()
    names = _declared()
    assert len(names) > 40
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing


def test_ctypes_table_matches_the_header():
    assert sorted(_native.EXPORTED_SYMBOLS) == _declared()


def test_version_and_launch_counter():
    lib = _native.load()
    assert lib.sah_version().decode().startswith("sah_b200")
    assert _native.launch_count() >= 0


def test_bad_arguments_return_a_status_and_a_message():
    lib = _native.load()
    # null pointers: nothing is launched, so this is safe without a device
    assert lib.sah_mask_fill_band(None, 1, 1, 32, 1, 0, 0, 1, 0, 1, None) == 1
    assert b"null" in lib.sah_last_error()
    assert lib.sah_hash_topk(None, 0, None, 32, None, 1, 0, 0, 0, 1, 1, 1, 32, 1, None, 1, None, None) == 1
    assert lib.sah_lsh_match(None, 32, None, 1, 4, 1, 4, 5, 4, 32, 1, None, None, None) == 1
    with pytest.raises(_native.NativeLibraryError):
        _native.check(1, "sah_lsh_match")
    with pytest.raises(NotImplementedError):
        _native.check(2, "anything")


def test_workspace_size_queries():
    lib = _native.load()
    assert lib.sah_topk_select_ws_bytes(32, 4096) > 32 * 4096 // 256 * 1024
    assert lib.sah_pq_scores_ws_bytes(1, 32, 8, 1, 16, 256) == 8 * 16 * 256 * 4 * 4
    sizes = _native.AttnSizes()
    assert lib.sah_attn_query_sizes(8, 32, 8, 1, 32768, 128, 0, 148, ctypes.byref(sizes)) == 0
    assert sizes.groups == 64 and sizes.ucols_bytes > 0


def test_plan_refuses_sizes_of_another_key_count():
    """The counter block is laid out by the key count: a plan call whose `sizes` came from a
    query for fewer keys (too few chunk counters) is refused before anything is launched, and
    a bitmap row stride W padded beyond ceil(S/32) does not change the layout."""
    lib = _native.load()
    small, big = _native.AttnSizes(), _native.AttnSizes()
    assert lib.sah_attn_query_sizes(1, 8, 2, 1, 40000, 128, 0, 148, ctypes.byref(small)) == 0
    assert lib.sah_attn_query_sizes(1, 8, 2, 1, 80000, 128, 0, 148, ctypes.byref(big)) == 0
    assert big.ucount_bytes > small.ucount_bytes
    one = ctypes.c_void_p(16)  # never dereferenced: the call is refused first
    status = lib.sah_attn_plan(one, None, None, None, _native.SAH_BF16, 1, 8, 2, 1, 80000, 2500,
                               ctypes.byref(small), one, one, None, one, None)
    assert status == 1 and b"key count" in lib.sah_last_error()
    # W too small for S is refused as before
    assert lib.sah_attn_plan(one, None, None, None, _native.SAH_BF16, 1, 8, 2, 1, 80000, 100,
                             ctypes.byref(big), one, one, None, one, None) == 1
    # the in-kernel MagicPig weights need their own size query (has_data = 2) ...
    assert lib.sah_attn_plan_lsh(one, None, one, 80000, one, 1, 8, 2, 1, 80000, 2500,
                                 ctypes.byref(big), one, one, one, one, None) == 1
    assert b"MagicPig" in lib.sah_last_error()
    # ... and at most four mask rows per KV group
    wide = _native.AttnSizes()
    assert lib.sah_attn_query_sizes(1, 16, 2, 1, 4096, 128, 2, 148, ctypes.byref(wide)) == 0
    assert lib.sah_attn_plan_lsh(one, None, one, 4096, one, 1, 16, 2, 1, 4096, 128,
                                 ctypes.byref(wide), one, one, one, one, None) == 2


def test_every_chained_launch_names_a_kernel_that_waits_for_its_predecessors():
    """`sah_launch_chain` sets the programmatic-stream-serialization attribute, which lets a grid
    start before the kernel in front of it has finished; that is only sound when the kernel's
    first statement is `sah_pdl_entry()` (the hardware wait for the predecessors).  Read from the
    sources: every kernel that is launched that way begins with it."""
    csrc = HEADER.parent.parent / "sparse-attention-hub_b200" / "csrc"
    text = "\n".join(p.read_text() for p in sorted(csrc.glob("*.cu*")))
    launched = set(re.findall(r"sah_launch_chain\(\s*([A-Za-z0-9_]+)\s*[<,]", text))
    launched.discard("kernel")  # the helper's own parameter
    assert len(launched) > 40
    for name in sorted(launched):
        m = re.search(r"__global__[^;{]*?\b" + name + r"\s*\(", text)
        assert m, name
        depth, i = 1, m.end()
        while depth:
            depth += {"(": 1, ")": -1}.get(text[i], 0)
            i += 1
        body = text[text.index("{", i) + 1:]
        assert body.lstrip().startswith(("sah_pdl_entry();", "sah_pdl_entry_early();")), name
    # and nothing else sets the attribute
    assert text.count("cudaLaunchAttributeProgrammaticStreamSerialization") == 1
