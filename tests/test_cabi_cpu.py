"""CPU-side checks of the boundary: the library builds, loads and exports every symbol include/kda_b200.h declares,
the ctypes structs match the compiled layout, and argument errors surface as the reference's ValueError contract.
No compute call is made here (there is no GPU on the CPU runner)."""
import ctypes
import re

import pytest
import torch

import __graft_entry__ as entry


@pytest.fixture(scope="module")
def lib():
    entry.build()
    from kda_b200 import _cabi
    return _cabi.lib()


def test_exports_every_declared_symbol(lib):
    header = (entry.ROOT / "include" / "kda_b200.h").read_text()
    body = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    declared = set(re.findall(r"\b(kda_[a-z_0-9]+)\s*\(", body))
    assert {"kda_prefill_launch", "kda_prefill_workspace_bytes", "kda_segment_launch", "kda_scan_launch",
            "kda_fixup_launch", "kda_state_rows_copy"} <= declared
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in include/kda_b200.h but not exported"


def test_struct_layout_matches(lib):
    from kda_b200 import _cabi
    assert lib.kda_abi_struct_bytes(0) == ctypes.sizeof(_cabi.KdaPrefillArgs)
    assert lib.kda_abi_struct_bytes(1) == ctypes.sizeof(_cabi.KdaSegmentArgs)


def test_workspace_size_and_error_strings(lib):
    a = lib.kda_prefill_workspace_bytes(1, 4)
    b = lib.kda_prefill_workspace_bytes(512, 64)
    assert 0 < a < b and b >= 64 * 65536
    assert lib.kda_prefill_workspace_bytes(-1, 4) == 0
    assert b"ok" == lib.kda_error_string(0)
    assert b"workspace" in lib.kda_error_string(-2)
    assert lib.kda_version().startswith(b"kda_b200")


def test_null_arguments_are_rejected_without_a_device(lib):
    from kda_b200 import _cabi
    assert lib.kda_prefill_launch(None, None) == -1
    a = _cabi.KdaPrefillArgs()
    a.H, a.N, a.T = 4, 1, 0
    assert lib.kda_prefill_launch(ctypes.byref(a), None) == -1        # no workspace / status
    assert lib.kda_scan_launch(None, None, None, None, None, 1, 1, None) == -1
    assert lib.kda_scan_strided_launch(None, None, None, None, None, 1, 1, 0, None) == -1
    assert lib.kda_state_rows_copy(None, 0, 0, None, 0, None, 1, 1, None) == -1
    assert lib.kda_fixup_tiles_launch(None, None, 0, 0, None, None, None, None, 1, 1, 0, None) == -1


def test_segment_tiles_counts_tiles_of_32_tokens_per_segment(lib):
    """Host helper that sizes the tile-major scratch of a segment launch: every segment rounds up on its own, tables
    are clamped to [0, T] as the device planner clamps them."""
    def tiles(t0, t1, T):
        a = (ctypes.c_int64 * len(t0))(*t0)
        b = (ctypes.c_int64 * len(t1))(*t1)
        return lib.kda_segment_tiles(a, b, len(t0), T)
    assert tiles([0, 33, 64], [33, 64, 1000], 1000) == 2 + 1 + 30
    assert tiles([0], [131072], 131072) == 4096
    assert tiles([-5, 10], [10, 99], 40) == 1 + 1          # clamped: [0, 10) and [10, 40)
    assert tiles([7], [7], 100) == 0
    assert lib.kda_segment_tiles(None, None, 3, 10) == 0


def test_host_argument_contract():
    import kda_b200
    q = torch.zeros(1, 8, 2, 128, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="CUDA tensor"):
        kda_b200.run(q, q, q, q, torch.zeros(1, 8, 2, dtype=torch.bfloat16), torch.zeros(2), torch.zeros(256), 0.1,
                     torch.zeros(1, 2, 128, 128))
    with pytest.raises(ValueError):
        kda_b200.prepare(q, q, q, q, None, None, None, 0.1, None)


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from kda_b200 import _cabi
    monkeypatch.setattr(_cabi, "_lib", None)
    monkeypatch.setattr(_cabi, "LIB_PATH", tmp_path / "nope.so")
    with pytest.raises(RuntimeError, match="missing"):
        _cabi.lib()
