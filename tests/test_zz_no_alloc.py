"""kda_prefill_launch_noalloc: the prefill call for callers that cannot allocate device memory (code inside an
allocator callback, a process whose device memory a serving engine has reserved up front, a thread that may be under
stream capture).  Its scratch is a fixed array inside the library instead of a caller workspace.  The test drives it
through the C ABI and checks, on two calls in a row (the array keeps the previous call's contents), that output and
final state equal those of kda_prefill_launch bit for bit, and that sizes beyond the stated limits are refused.
Collected last on purpose: a run that stops at the first failure has then already run every other test."""
import ctypes as C

import pytest
import torch

import kda_oracle as ko
from kda_testlib import DEV, D, to_dev

pytestmark = pytest.mark.gpu


def test_noalloc_entry_point_matches_the_workspace_entry_point():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    import kda_b200
    from kda_b200 import _cabi
    lib = _cabi.lib()
    stream = lambda: C.c_void_p(torch.cuda.current_stream().cuda_stream)  # noqa: E731
    for call, (H, lens, seed) in enumerate([(4, [100, 33, 1, 257], 31), (16, [64] * 5 + [700], 32)]):
        d = to_dev(ko.make_inputs_raw(H, lens, seed))
        launch = kda_b200.prepare(*d)                       # builds the argument block; owns out / final-state tensors
        out_ref, fin_ref = launch()                         # existing entry point (caller workspace)
        torch.cuda.synchronize()
        out_ref, fin_ref = out_ref.clone(), fin_ref.clone()
        launch._result[0].zero_()
        launch._result[1].zero_()
        args = launch._args
        saved = (args.workspace, args.workspace_bytes)
        args.workspace, args.workspace_bytes = None, 0      # the new entry point must not need them
        rc = lib.kda_prefill_launch_noalloc(C.byref(args), stream())
        args.workspace, args.workspace_bytes = saved
        assert rc == 0, lib.kda_error_string(rc).decode()
        torch.cuda.synchronize()
        assert kda_b200.status_bits(launch) == 0 and kda_b200.kernel_error(launch) == 0
        assert torch.equal(launch._result[0], out_ref), f"call {call}: output differs"
        assert torch.equal(launch._result[1], fin_ref), f"call {call}: final state differs"
    # limits: more heads or sequences than the fixed array was sized for
    big = kda_b200.prepare(*to_dev(ko.make_inputs_raw(_cabi.NOALLOC_MAX_HEADS + 1, [40], 33)))
    assert lib.kda_prefill_launch_noalloc(C.byref(big._args), stream()) == -4
    many = kda_b200.prepare(*to_dev(ko.make_inputs_raw(1, [2] * (_cabi.NOALLOC_MAX_SEQS + 1), 34)))
    assert lib.kda_prefill_launch_noalloc(C.byref(many._args), stream()) == -4
    assert b"maximum" in lib.kda_error_string(-4)
