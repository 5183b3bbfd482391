"""The oracle against the reference's own outputs (tests/golden/*.npz, written by tests/golden/make_golden.py from
kda/b200/reference.py) and against itself across front-ends and implementations (torch and C)."""
import numpy as np
import pytest
import torch

import c_oracle
import kda_oracle as ko

CASES = ["raw_h2_t70", "raw_h2_varlen", "raw_h1_slow_t96", "raw_h2_t40_fp32"]


def load(golden_dir, name):
    z = np.load(golden_dir / f"{name}.npz")
    bf = lambda a: torch.from_numpy(a.copy()).view(torch.bfloat16)  # noqa: E731
    d = dict(q=bf(z["q"]), k=bf(z["k"]), v=bf(z["v"]), g=bf(z["g"]), beta=bf(z["beta"]),
             A_log=torch.from_numpy(z["A_log"]), dt_bias=torch.from_numpy(z["dt_bias"]), scale=float(z["scale"]),
             init=torch.from_numpy(z["init"]), cu=torch.from_numpy(z["cu"]), out=bf(z["out"]),
             final=torch.from_numpy(z["final"]), ref_dtype=str(z["ref_dtype"]))
    return d


@pytest.mark.parametrize("name", CASES)
def test_torch_oracle_matches_reference_output(golden_dir, name):
    d = load(golden_dir, name)
    dt = torch.float32 if "float32" in d["ref_dtype"] else torch.float64
    out, fin = ko.kda_recurrence(d["q"], d["k"], d["v"], d["g"], d["beta"], d["A_log"], d["dt_bias"], d["scale"],
                                 d["init"], d["cu"], dtype=dt)
    # same arithmetic in the same order and precision: bf16 outputs must agree to the last bit up to rare rounding ties
    diff = (out.float() - d["out"].float()).abs()
    assert float(diff.max()) <= 2.0 ** -8 * float(d["out"].float().abs().max())
    assert float((diff > 0).float().mean()) < 1e-3
    tol = 1e-4 if dt == torch.float32 else 1e-6
    assert torch.allclose(fin, d["final"], rtol=tol, atol=tol)


@pytest.mark.parametrize("name", CASES[:3])
def test_c_oracle_matches_reference_output(golden_dir, name):
    d = load(golden_dir, name)
    out, fin = c_oracle.recurrence_raw(d["q"], d["k"], d["v"], d["g"], d["beta"], d["A_log"], d["dt_bias"], d["scale"],
                                       d["init"], d["cu"])
    diff = (out.float() - d["out"].float()).abs()
    assert float(diff.max()) <= 2.0 ** -8 * float(d["out"].float().abs().max())
    assert float((diff > 0).float().mean()) < 1e-3
    assert torch.allclose(fin, d["final"], rtol=1e-6, atol=1e-6)
    o32, f32 = c_oracle.recurrence_raw(d["q"], d["k"], d["v"], d["g"], d["beta"], d["A_log"], d["dt_bias"], d["scale"],
                                       d["init"], d["cu"], precision="f32")
    ko.check_close(o32, d["out"], "C fp32 out", 1e-3)
    ko.check_close(f32, d["final"], "C fp32 final", 1e-4)


def test_plain_frontend_equals_raw_frontend_on_activated_inputs(golden_dir):
    """The pre-activated call is the same loop fed with the activated tensors, state transposed."""
    d = load(golden_dir, "raw_h2_varlen")
    qn, kn, a, b = ko.activate_raw(d["q"][0], d["k"][0], d["g"][0], d["beta"][0], d["A_log"], d["dt_bias"])
    out, fin = ko.kda_recurrence_plain(qn[None], kn[None], d["v"].double(), a[None], b[None], d["scale"],
                                       d["init"].transpose(-1, -2), d["cu"])
    assert float((out.to(torch.bfloat16).float() - d["out"].float()).abs().max()) <= 2.0 ** -8 * float(d["out"].float().abs().max())
    assert torch.allclose(fin.transpose(-1, -2), d["final"], rtol=1e-6, atol=1e-6)
    oc, fc = c_oracle.recurrence_plain(qn[None], kn[None], d["v"], a[None], b[None], d["scale"],
                                       d["init"].transpose(-1, -2).contiguous(), d["cu"])
    ko.check_close(oc, out, "C plain out", 1e-4)   # the C entry takes fp32 inputs: activated tensors are rounded
    ko.check_close(fc.transpose(-1, -2), d["final"], "C plain final", 1e-4)


def test_checkpoint_rows_and_chaining(golden_dir):
    d = load(golden_dir, "raw_h2_varlen")
    lens = (d["cu"][1:] - d["cu"][:-1]).tolist()
    out, fin, rows = ko.kda_checkpoints(d["q"], d["k"], d["v"], d["g"], d["beta"], d["A_log"], d["dt_bias"], d["scale"],
                                        d["init"], lens, every=32)
    assert rows.shape[0] == sum(-(-n // 32) for n in lens)
    # chaining over segments must not change results (state hand-off is exact in fp64 up to the fp32 cast)
    ko.check_close(out, d["out"], "chained out", 1e-3)
    ko.check_close(fin, d["final"], "chained final", 1e-5)
    assert torch.equal(rows[0], d["init"][0])          # row 0 of a sequence is its initial state
    assert torch.equal(rows[1], d["init"][1])          # sequence 0 has 5 tokens -> exactly one row


def test_segment_map_composes(golden_dir):
    """S_end = S_in @ P + S_loc and o = o_loc + S_in applied to Qt, on a 2-piece split of a sequence."""
    d = load(golden_dir, "raw_h1_slow_t96")
    qn, kn, a, b = ko.activate_raw(d["q"][0], d["k"][0], d["g"][0], d["beta"][0], d["A_log"], d["dt_bias"])
    v = d["v"][0].double()
    cut, T = 32, 96
    S0 = d["init"].double().transpose(-1, -2)                                # key-first
    o_full, fin_full = ko._recur(qn, kn, v, a, b, d["scale"], S0, [0, T])
    o_head, S_A = ko._recur(qn[:cut], kn[:cut], v[:cut], a[:cut], b[:cut], d["scale"], S0, [0, cut])
    zero = torch.zeros_like(S0)
    o_loc, S_loc = ko._recur(qn[cut:], kn[cut:], v[cut:], a[cut:], b[cut:], d["scale"], zero, [0, T - cut])
    P, Qt = ko.segment_map(qn[cut:], kn[cut:], a[cut:], b[cut:], d["scale"])
    St_in = S_A[0].transpose(-1, -2)                                         # value-first [H,V,K]
    St_end = St_in @ P + S_loc[0].transpose(-1, -2)
    assert torch.allclose(St_end, fin_full[0].transpose(-1, -2), rtol=1e-9, atol=1e-9)
    o_fix = o_loc + torch.einsum("hvk,thk->thv", St_in, Qt)
    assert torch.allclose(o_fix, o_full[cut:], rtol=1e-9, atol=1e-9)


def test_acceptance_criterion():
    g = torch.randn(1000)
    ko.check_close(g + 1e-3 * torch.randn(1000), g, "small noise")
    with pytest.raises(AssertionError):
        ko.check_close(g + 0.1 * torch.randn(1000), g, "large noise")
    with pytest.raises(AssertionError):
        bad = g.clone(); bad[3] = float("nan")
        ko.check_close(bad, g, "nan")
