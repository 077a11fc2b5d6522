"""The C-ABI library loads and exports exactly what include/jointqk_b200.h declares.
No compute call is made (this runs without a GPU)."""

import ctypes
import re
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]


def _declared_functions():
    text = (ROOT / "include" / "jointqk_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(jqk_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from jointqk_b200 import _native

    names = _declared_functions()
    assert "jqk_decode_attend" in names and "jqk_compress_paged" in names and "jqk_moments_accumulate" in names
    lib = ctypes.CDLL(str(ROOT / "jointqk_b200" / "libjointqk_b200.so"))
    for n in names:
        assert hasattr(lib, n), f"{n} declared in the header but not exported"
    assert sorted(_native.SIGNATURES) == names, "binding table and header disagree"


def test_version_and_argument_errors_without_gpu():
    from jointqk_b200 import _native

    assert _native.lib.jqk_version() == _native.ABI_VERSION == 2
    assert _native.lib.jqk_head_tables_bytes() == ctypes.sizeof(_native.JqkHeadTables)
    rc = _native.lib.jqk_moments_accumulate(None, None, 1, 10, 1280, 1280, 3, 2, 128, None, None, None, None, None, 0, None, 0, None)
    assert rc == -1 and b"GQA mismatch" in _native.lib.jqk_last_error()
    rc = _native.lib.jqk_compress_paged(None, None, 0, 0, 0, 0, 1, None, None, 1, None, 1, 1, None, None, None)
    assert rc == -1 and b"null head tables" in _native.lib.jqk_last_error()
    assert _native.lib.jqk_decode_workspace_bytes(1, 32, 8, 37) > 37 * 32 * 128 * 4
    assert _native.lib.jqk_decode_default_split(1, 32, 8, 32768) % 32 == 0


def test_decode_split_fits_waves_of_148_blocks():
    """Host-only helpers: the split is a multiple of 384 keys (one 32-key tile per warp), keeps one
    short batch inside a single wave of 148 blocks, and gives large batches blocks of several
    thousand keys with the block count at or under a multiple of 148."""
    from jointqk_b200 import paged

    tps = paged.default_split(1, 32, 8, 32768)
    assert tps % 384 == 0 and 8 * -(-32768 // tps) <= 148 and tps == paged.split_for_lengths([32768], 32, 8)
    lens = [64850, 48381, 47953, 40224, 35138, 25021, 21352, 6227]
    tps = paged.split_for_lengths(lens, 32, 8)
    blocks = 8 * sum(-(-n // tps) for n in lens)
    assert tps % 384 == 0 and 4096 <= tps <= 16384 and blocks % 148 > 148 // 2 or blocks % 148 == 0
    assert paged.split_for_lengths([0, 0], 8, 8) == 384 and paged.split_for_lengths([100], 8, 8) == 384
    assert -(-1_000_000 // paged.default_split(1, 32, 8, 1_000_000)) <= 4096   # the merge's split limit
