"""GPU tests of the paths that exist for robustness rather than speed: a wait inside the kernel that runs out (the
kernel must finish by itself, report a code and leave the context usable), decays beyond the range of the clamped
intra-chunk exponents (reported, never silent), the checkpoint-overlap policy on a chain of overlapping sequences, and
beta read in place for head counts that are not multiples of eight."""
import ctypes as C

import pytest
import torch

import c_oracle
import kda_oracle as ko
from kda_testlib import DEV, D, cu_of, gold_raw, to_dev

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def kda():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    import kda_b200
    return kda_b200


def test_bounded_wait_gives_up_and_the_next_launch_is_correct(kda):
    """The kernel's hand-offs are bounded waits.  With the diagnostic switch under which the arrival of the v tiles is
    never signalled, the first waiter on a v tile runs into the (shortened) bound: the kernel must still end by itself,
    free its tensor memory, report a nonzero code in status[2] and leave the device usable.  Nothing faults or hangs:
    the flag that would end the wait is simply never set."""
    from kda_b200 import _cabi
    lib = _cabi.lib()
    lens = [300, 64, 1000]
    inputs = ko.make_inputs_raw(4, lens, 77)
    gold_o, gold_s, _ = gold_raw(inputs, lens)
    d = to_dev(inputs)
    launch = kda.prepare(*d)
    assert lib.kda_debug_configure(200, 1, None) == 0          # 200 us bound, v tiles never signalled
    try:
        launch()
        torch.cuda.synchronize()                               # returns: every CTA gave up and left
        code = kda.kernel_error(launch)
    finally:
        assert lib.kda_debug_configure(0, 0, None) == 0
    assert code != 0, "a wait that can never be satisfied must be reported in status[2]"
    # the same prepared launch, now undisturbed, gives the right answer (tensor memory was freed, no stale state)
    out, fin = launch()
    torch.cuda.synchronize()
    assert kda.kernel_error(launch) == 0 and kda.status_bits(launch) == 0
    ko.check_close(out.cpu(), gold_o, "launch after a give-up: output")
    ko.check_close(fin.cpu(), gold_s, "launch after a give-up: final state")


def test_plain_call_decay_range(kda):
    """Plain-call log-decays are unbounded.  At the raw front-end's bound (-5 per token) the intra-chunk exponents stay
    inside fp32 and the result is exact; at -12 per token a key channel decays by more than 2^126 within 16 tokens, the
    exponents are clamped and the call must say so (status bit 16) instead of returning silently inexact numbers."""
    H, T = 2, 96
    q, k, v, g, beta, scale, init, cu = ko.make_inputs_plain(H, [T], 5)
    for per_token, expect_bit in ((-5.0, 0), (-12.0, 16)):
        gg = torch.full_like(g, per_token)
        launch = kda.prepare_plain(q.to(DEV), k.to(DEV), v.to(DEV), gg.to(DEV), beta.to(DEV), scale, init.to(DEV), True, cu.to(DEV))
        o, fin = launch()
        torch.cuda.synchronize()
        assert kda.status_bits(launch) == expect_bit, f"g = {per_token} per token"
        assert bool(torch.isfinite(o.float()).all()) and bool(torch.isfinite(fin).all())
        if not expect_bit:
            gold_o, gold_s = c_oracle.recurrence_plain(q, k, v, gg, beta, scale, init, cu)
            ko.check_close(o.float().cpu(), gold_o, "decay at the -5 bound: output")
            ko.check_close(fin.cpu(), gold_s, "decay at the -5 bound: final state")


def test_checkpoint_overlap_chain_follows_final_decisions(kda):
    """Sequences A, B, C with B's rows overlapping A's and C's rows overlapping only B's: B loses its rows, and because
    B wrote none, C keeps its own (the reference resolves overlaps against final decisions,
    kda/b200/csrc/w3/validate_dev.cuh:124-142)."""
    H, lens, every = 2, [64, 64, 64], 32               # two rows per sequence
    inputs = ko.make_inputs_raw(H, lens, 91)
    q, k, v, g, beta, A_log, dt_bias, scale = to_dev(inputs[:8])
    pool = to_dev([inputs[8]])[0].clone()
    pool0 = pool.clone()
    ck = torch.full((8, H, D, D), float("nan"), device=DEV)
    ccs = torch.tensor([0, 1, 2, 0], dtype=torch.int64, device=DEV)     # A rows 0-1, B rows 1-2, C rows 2-3
    idx = torch.arange(3, dtype=torch.int32, device=DEV)
    launch = kda.prepare(q, k, v, g, beta, A_log, dt_bias, scale, pool, cu_of(lens), dynamic_layout=True, ssm_state_indices=idx,
                         state_checkpoints=ck, checkpoint_cu_starts=ccs, checkpoint_every_n_tokens=every)
    launch()
    torch.cuda.synchronize()
    assert kda.status_bits(launch) == 8
    assert torch.equal(ck[0], pool0[0]), "A's row 0 is its initial state"
    assert torch.equal(ck[2], pool0[2]), "C kept its rows: row 2 is C's initial state"
    assert bool(torch.isfinite(ck[:4]).all()) and bool(torch.isnan(ck[4:]).all())
    gold = gold_raw(inputs, lens, every=every)[2]                       # rows A0 A1 B0 B1 C0 C1
    ko.check_close(ck[1].cpu(), gold[1], "A's second row (not overwritten by B)")
    ko.check_close(ck[3].cpu(), gold[5], "C's second row")


def test_beta_is_read_in_place_for_any_head_count(kda):
    """beta [1, T, H] is read with scalar loads, so a head slice of a wider beta needs no private copy whatever H is
    (H = 12 and H = 3 are not multiples of eight)."""
    for H, Hs in ((24, 12), (5, 3)):
        lens = [130, 77]
        d = to_dev(ko.make_inputs_raw(H, lens, 600 + H))
        q, k, v, g, beta, A_log, dt_bias, scale, init, cu = d
        sl = slice(1, 1 + Hs)
        view = [q[:, :, sl], k[:, :, sl], v[:, :, sl], g[:, :, sl], beta[:, :, sl], A_log[sl].contiguous(),
                dt_bias.view(H, D)[sl].reshape(-1), scale, init[:, sl].contiguous(), cu]
        launch = kda.prepare(*view)
        assert launch._copies == [], f"H = {Hs}: an operand was copied although its layout can be read in place"
        a = launch()
        a = (a[0].clone(), a[1].clone())
        b = kda.run(*[t.contiguous() if torch.is_tensor(t) else t for t in view])
        assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])


def test_host_latency_of_run_is_within_the_reference_limits(kda):
    """The reference states host-side limits for run(): <= 1 ms + 0.01 ms per sequence for a repeated layout and
    <= 2 ms + 0.025 ms per sequence for a new one (kda/b200/README.md:39-41).  Nothing is planned on the host here (the
    schedule is made on the device at every launch), so every layout counts as new and must meet the tighter limit."""
    import time
    H, T = 8, 4096
    inputs = ko.make_inputs_raw(H, [T], 41)
    q, k, v, g, beta, A_log, dt_bias, scale = to_dev(inputs[:8])
    for n_seq in (1, 32, 512):
        lens = [T // n_seq] * n_seq
        pool = torch.zeros(n_seq, H, D, D, device=DEV)
        idx = torch.arange(n_seq, dtype=torch.int32, device=DEV)
        cu = cu_of(lens)
        call = lambda: kda.run(q, k, v, g, beta, A_log, dt_bias, scale, pool, cu, ssm_state_indices=idx)  # noqa: E731
        call()
        times = []
        for _ in range(9):
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            call()
            times.append(time.perf_counter() - t0)
        torch.cuda.synchronize()
        med_ms = sorted(times)[len(times) // 2] * 1e3
        assert med_ms <= 1.0 + 0.01 * n_seq, f"run() with {n_seq} sequences took {med_ms:.3f} ms on the host"
