"""GPU parity of the CUDA path (through the C ABI) against the CPU oracle and the reference's golden outputs.

Cases follow the reference's own test file kda/b200/test_kda_b200.py (shapes :79-110, serving contract :114-160,
graph replay :163-210, bf16 checkpoints :213-240, wrapper :243-249, API errors :252-268), at sizes the CPU oracle
finishes in seconds.  Tolerance (kda/b200/test_kda_b200.py:28-35): every element within half the gold tensor's RMS or
5 % of its own magnitude, relative L2 < 1e-2; pool slots that must not change are compared bit for bit."""
import random

import numpy as np
import pytest
import torch

import kda_oracle as ko
from kda_testlib import DEV, D, ck_meta, cu_of, gold_raw, partition, slow_gates_, to_dev

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def kda():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    import kda_b200
    from kda_b200 import _cabi
    _cabi.lib()      # a missing library must fail here, loudly
    return kda_b200


def _plain_case(kda, H, lens, seed, slow=False, static=False):
    inputs = ko.make_inputs_raw(H, lens, seed)
    if slow:
        slow_gates_(inputs, seed)
    gold_o, gold_s, _ = gold_raw(inputs, lens)
    d = to_dev(inputs)
    if len(lens) == 1 and seed % 2:
        d[9] = None
    res = kda.prepare(*d)() if static else kda.run(*d)
    torch.cuda.synchronize()
    tag = f"H={H} lens={lens[:8]} slow={slow}"
    ko.check_close(res[0].cpu(), gold_o, tag + " output")
    ko.check_close(res[1].cpu(), gold_s, tag + " final_state")


# ----------------------------------------------------------------------------------------------- golden fixtures
@pytest.mark.parametrize("name", ["raw_h2_t70", "raw_h2_varlen", "raw_h1_slow_t96", "raw_h2_t40_fp32"])
def test_reference_golden_vectors(kda, golden_dir, name):
    """Inputs and outputs written by the reference's reference.py (tests/golden/make_golden.py)."""
    z = np.load(golden_dir / f"{name}.npz")
    bf = lambda a: torch.from_numpy(a.copy()).view(torch.bfloat16).to(DEV)  # noqa: E731
    out, fin = kda.run(bf(z["q"]), bf(z["k"]), bf(z["v"]), bf(z["g"]), bf(z["beta"]), torch.from_numpy(z["A_log"]).to(DEV),
                       torch.from_numpy(z["dt_bias"]).to(DEV), float(z["scale"]), torch.from_numpy(z["init"]).to(DEV),
                       torch.from_numpy(z["cu"]).to(DEV))
    torch.cuda.synchronize()
    ko.check_close(out.cpu(), torch.from_numpy(z["out"].copy()).view(torch.bfloat16), name + " output")
    ko.check_close(fin.cpu(), torch.from_numpy(z["final"]), name + " final_state")


# ----------------------------------------------------------------------------------------------- plain calls
@pytest.mark.parametrize("H,lens", [(64, [1024]), (96, [300, 547, 271]), (64, [256] * 4)])
def test_many_heads(kda, H, lens):
    _plain_case(kda, H, lens, 100 + H, static=True)
    _plain_case(kda, H, lens, 200 + H, static=False)


@pytest.mark.parametrize("H,lens", [(12, [2048]), (16, [700, 1348]), (12, [256, 512, 900, 100, 160, 240, 400, 87]),
                                    (16, [64] * 16), (12, [random.Random(3).randint(17, 255) for _ in range(16)])])
def test_serving_head_counts_varlen(kda, H, lens):
    _plain_case(kda, H, lens, 300 + len(lens))


def test_slow_decay(kda):
    _plain_case(kda, 4, [6144], 400, slow=True)
    _plain_case(kda, 16, [3000, 1, 2048, 777, 64, 33], 401, slow=True)


@pytest.mark.parametrize("H,lens", [(1, [4096]), (4, list(range(1, 16))), (8, [37]), (32, [700, 1300, 45]), (96, [1]),
                                    (128, [300]), (12, [1, 17, 33, 1, 1023, 64, 1, 2])])
def test_other_heads_and_tiny(kda, H, lens):
    _plain_case(kda, H, lens, 500 + H)


@pytest.mark.parametrize("H,lens", [(4, [64] * 512), (2, [random.Random(7).randint(1, 300) for _ in range(200)]),
                                    (3, [1] * 70 + [2048] + [1] * 70)])
def test_many_short_sequences(kda, H, lens):
    """Layouts with far more (sequence, head) tasks than SMs, most of them one or two chunks long (the 512 x 64 layout
    of the single-graph configuration), and single-token runs next to a long one."""
    _plain_case(kda, H, lens, 600 + H)


@pytest.mark.parametrize("seed", [11, 12, 13])
def test_random_layout_sweep(kda, seed):
    """Randomised layouts against the fp64 recurrence: head counts, sequence counts and lengths drawn per case (short and
    partial chunks, odd / even chunk counts, single tokens), slow gates in a third of the cases."""
    rng = random.Random(seed)
    for case in range(12):
        H = rng.choice([1, 2, 3, 5, 8])
        n = rng.randint(1, 10)
        lens = [rng.choice([1, 31, 32, 33, 64, 65]) if rng.random() < 0.3 else rng.randint(1, 400) for _ in range(n)]
        _plain_case(kda, H, lens, 1000 * seed + case, slow=(case % 3 == 2), static=bool(case & 1))


def test_single_sequence_no_cu(kda):
    inputs = ko.make_inputs_raw(16, [1500], 600)
    gold_o, gold_s, _ = gold_raw(inputs, [1500])
    d = to_dev(inputs)
    d[9] = None
    out, fin = kda.run(*d)
    ko.check_close(out.cpu(), gold_o, "cu_seqlens=None output")
    ko.check_close(fin.cpu(), gold_s, "cu_seqlens=None final_state")


def test_deterministic(kda):
    d = to_dev(ko.make_inputs_raw(8, [700, 33, 1], 601))
    a = kda.run(*d)
    a = (a[0].clone(), a[1].clone())
    b = kda.run(*d)
    assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])


@pytest.mark.parametrize("kernel", [0, 1])
def test_repeated_runs_are_bit_identical(kda, kernel):
    """Many CTAs with different run lengths, several launches: any hand-off race between the warp roles shows up as a
    run-to-run difference."""
    lens = [256, 512, 900, 100, 160, 240, 400, 87, 1300, 33]
    inputs = ko.make_inputs_raw(12, lens, 603)
    gold_o, gold_s, _ = gold_raw(inputs, lens)
    d = to_dev(inputs)
    first = None
    for rep in range(6):
        out, fin = kda.prepare(*d, kernel=kernel)()
        torch.cuda.synchronize()
        if first is None:
            first = (out.clone(), fin.clone())
            ko.check_close(out.cpu(), gold_o, "repeat output")
            ko.check_close(fin.cpu(), gold_s, "repeat final_state")
        else:
            assert torch.equal(out, first[0]) and torch.equal(fin, first[1]), f"run {rep} differs from run 0"


def test_strided_head_slice_is_read_in_place(kda):
    """A head slice of wider tensors (the head-parallel layout) gives the same bits as a contiguous copy."""
    H, Hs, lens = 8, 4, [200, 77]
    d = to_dev(ko.make_inputs_raw(H, lens, 602))
    q, k, v, g, beta, A_log, dt_bias, scale, init, cu = d
    sl = slice(2, 2 + Hs)
    args_view = [q[:, :, sl], k[:, :, sl], v[:, :, sl], g[:, :, sl], beta[:, :, sl], A_log[sl],
                 dt_bias.view(H, D)[sl].reshape(-1), scale, init[:, sl].contiguous(), cu]
    args_copy = [t.contiguous() if torch.is_tensor(t) else t for t in args_view]
    a = kda.run(*args_view)
    b = kda.run(*args_copy)
    assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])


# ----------------------------------------------------------------------------------------------- serving contract
def _serving(kda, H, lens, seed, every=64, use_source=False, pad=0, ck_dtype=torch.float32):
    gen = torch.Generator().manual_seed(seed)
    inputs = ko.make_inputs_raw(H, lens, seed)
    q, k, v, g, beta, A_log, dt_bias, scale = to_dev(inputs[:8])
    cu = cu_of(lens)
    N, P = len(lens), len(lens) + 5
    slot = H * D * D
    pool = (torch.randn(P, slot + pad, generator=gen) * 0.25).to(DEV).as_strided((P, H, D, D), (slot + pad, D * D, D, 1))
    idx = torch.randperm(P, generator=gen)[:N].to(torch.int32).to(DEV)
    start = pool[idx.long()].clone()
    kw = dict(ssm_state_indices=idx)
    src = None
    if use_source:
        src = (torch.randn(P + 3, H, D, D, generator=gen) * 0.25).to(DEV)
        sidx = torch.randperm(P + 3, generator=gen)[:N].to(torch.int32).to(DEV)
        kw.update(initial_state_source=src, initial_state_indices=sidx)
        start = src[sidx.long()].clone()
    src_before = None if src is None else src.clone()
    ck = None
    if every:
        ccs, C = ck_meta(lens, every)
        ck = torch.full((C, H, D, D), float("nan"), device=DEV, dtype=ck_dtype)
        kw.update(state_checkpoints=ck, checkpoint_cu_starts=ccs, checkpoint_every_n_tokens=every)
    pool_before = pool.clone()
    res = kda.kda_prefill(q, k, v, g, beta, A_log, dt_bias, pool, cu, scale, **kw)
    torch.cuda.synchronize()
    gold_o, gold_s, gold_ck = gold_raw(inputs, lens, init=start.cpu(), every=every)
    tag = f"H={H} lens={lens[:8]} every={every} source={use_source} pad={pad}"
    ko.check_close(res[0].cpu(), gold_o, tag + " output")
    ko.check_close(pool[idx.long()].cpu(), gold_s, tag + " pool slots")
    keep = torch.ones(P, dtype=torch.bool, device=DEV)
    keep[idx.long()] = False
    assert torch.equal(pool[keep], pool_before[keep]), tag + ": other pool slots modified"
    if src is not None:
        assert torch.equal(src, src_before), tag + ": source pool modified"
    if every:
        assert len(res) == 3 and res[2] is ck
        ko.check_close(ck.float().cpu(), gold_ck, tag + " checkpoints")
    return res, pool, ck


def test_pool_checkpoints(kda):
    _serving(kda, 12, [300, 64, 1, 1000, 77], 700)
    _serving(kda, 16, [1024] * 4, 701)
    _serving(kda, 12, [2048], 702, every=256)
    _serving(kda, 16, [2048, 513, 77], 703, use_source=True, pad=64)
    _serving(kda, 12, [1000, 200, 3], 704, every=0)
    _serving(kda, 8, [1500, 31, 32, 33], 705, every=32)


def test_bf16_checkpoints(kda):
    """bf16 rows are the fp32 rows rounded to nearest even; output and pool do not depend on the checkpoint dtype
    (kda/b200/test_kda_b200.py:213-240)."""
    for H, lens, every in ((12, [300, 64, 1, 1000, 77], 64), (16, [1024] * 4, 64), (12, [2048], 256)):
        got = {}
        for dt in (torch.float32, torch.bfloat16):
            res, pool, ck = _serving(kda, H, lens, 1000 + H + len(lens), every=every, ck_dtype=dt)
            got[dt] = (res[0].clone(), pool.clone(), ck.clone())
        tag = f"bf16 checkpoints H={H} lens={lens[:6]} every={every}"
        assert torch.equal(got[torch.float32][0], got[torch.bfloat16][0]), tag + ": output differs"
        assert torch.equal(got[torch.float32][1], got[torch.bfloat16][1]), tag + ": pool differs"
        assert torch.equal(got[torch.float32][2].to(torch.bfloat16), got[torch.bfloat16][2]), tag + ": rows != rounded fp32 rows"


def test_dynamic_layout_graph_replay(kda):
    """Capture once, replay after the tables and inputs change in place (kda/b200/test_kda_b200.py:163-210)."""
    for H, T, N, every in ((12, 1024, 6, 64), (16, 1536, 3, 64), (12, 512, 16, 0)):
        rng = random.Random(H * T + N)
        gen = torch.Generator().manual_seed(H + T + N)
        lens0 = partition(rng, T, N)
        inputs = ko.make_inputs_raw(H, lens0, 800 + H + N)
        q, k, v, g, beta, A_log, dt_bias, scale = to_dev(inputs[:8])
        cu = cu_of(lens0)
        P = N + 4
        pool0 = (torch.randn(P, H, D, D, generator=gen) * 0.25).to(DEV)
        pool = pool0.clone()
        idx = torch.randperm(P, generator=gen)[:N].to(torch.int32).to(DEV)
        kw = dict(dynamic_layout=True, ssm_state_indices=idx)
        ck = ccs = None
        if every:
            ccs, _ = ck_meta(lens0, every)
            ck = torch.full((T // every + N, H, D, D), float("nan"), device=DEV)
            kw.update(state_checkpoints=ck, checkpoint_cu_starts=ccs, checkpoint_every_n_tokens=every)
        launch = kda.prepare(q, k, v, g, beta, A_log, dt_bias, scale, pool, cu, **kw)
        launch()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            res = launch()
        for r, lens in enumerate([partition(rng, T, N), partition(rng, T, N), [T - (N - 1)] + [1] * (N - 1)]):
            cu.copy_(cu_of(lens))
            host = []
            for t in (q, k, v, g, beta):
                h = (torch.randn(t.shape, generator=gen) * 0.5).to(torch.bfloat16)
                host.append(h)
                t.copy_(h)
            pool.copy_(pool0)
            idx.copy_(torch.randperm(P, generator=gen)[:N].to(torch.int32))
            if every:
                new_ccs, C = ck_meta(lens, every)
                ccs.copy_(new_ccs)
                ck.fill_(float("nan"))
            graph.replay()
            torch.cuda.synchronize()
            assert kda.status_bits(launch) == 0
            gold_o, gold_s, gold_ck = gold_raw(host + [inputs[5], inputs[6], scale], lens, init=pool0[idx.long()].cpu(), every=every)
            tag = f"replay {r} H={H} T={T} N={N}"
            ko.check_close(res[0].cpu(), gold_o, tag + " output")
            ko.check_close(pool[idx.long()].cpu(), gold_s, tag + " pool slots")
            if every:
                ko.check_close(ck[:C].cpu(), gold_ck, tag + " checkpoints")


@pytest.mark.parametrize("H,lens,every,ck_dtype", [(2, [8192, 300, 64, 4000, 33], 256, torch.float32), (1, [16384], 1024, torch.bfloat16),
                                                   (4, [6000, 6000, 100], 0, None), (8, [2048, 9000, 1, 700, 5000, 31], 64, torch.bfloat16)])
def test_serving_call_cuts_long_requests(kda, H, lens, every, ck_dtype):
    """With few heads a long request is a serial chain that bounds the whole launch, so the device planner cuts it into
    pieces (affine state maps for the entering states, then the pieces as ordinary tasks).  Output, pool slots and
    checkpoint rows must be those of the fp64 recurrence and of the same call with cutting switched off; untouched slots
    stay bit-identical; a captured graph keeps working when the lengths change."""
    gen = torch.Generator().manual_seed(len(lens) + H)
    inputs = ko.make_inputs_raw(H, lens, 1200 + H)
    q, k, v, g, beta, A_log, dt_bias, scale = to_dev(inputs[:8])
    N, P = len(lens), len(lens) + 3
    pool0 = (torch.randn(P, H, D, D, generator=gen) * 0.25).to(DEV)
    idx = torch.randperm(P, generator=gen)[:N].to(torch.int32).to(DEV)
    cu = cu_of(lens)
    got = {}
    for cuts in (None, 0):
        pool = pool0.clone()
        kw = dict(dynamic_layout=True, ssm_state_indices=idx, max_cut_pieces=cuts)
        ck = None
        if every:
            ccs, rows = ck_meta(lens, every)
            ck = torch.full((rows, H, D, D), float("nan"), device=DEV, dtype=ck_dtype)
            kw.update(state_checkpoints=ck, checkpoint_cu_starts=ccs, checkpoint_every_n_tokens=every)
        launch = kda.prepare(q, k, v, g, beta, A_log, dt_bias, scale, pool, cu, **kw)
        out = launch()[0]
        torch.cuda.synchronize()
        assert kda.status_bits(launch) == 0 and kda.kernel_error(launch) == 0
        na, nb, ncut = launch.plan_counts()
        if cuts == 0:
            assert (na, nb, ncut) == (N, 0, 0)
        else:
            assert ncut >= 1 and nb >= 1, f"the planner was expected to cut the long request(s): counts {(na, nb, ncut)}"
        got[cuts] = (out.clone(), pool.clone(), None if ck is None else ck.clone())
    gold_o, gold_s, gold_ck = gold_raw(inputs[:8], lens, init=pool0[idx.long()].cpu(), every=every)
    tag = f"cut serving call H={H} lens={lens} every={every}"
    ko.check_close(got[None][0].cpu(), gold_o, tag + " output")
    ko.check_close(got[None][1][idx.long()].cpu(), gold_s, tag + " pool slots")
    ko.check_close(got[None][0].float().cpu(), got[0][0].float().cpu(), tag + " output vs uncut call")
    ko.check_close(got[None][1][idx.long()].cpu(), got[0][1][idx.long()].cpu(), tag + " pool slots vs uncut call")
    keep = torch.ones(P, dtype=torch.bool, device=DEV)
    keep[idx.long()] = False
    assert torch.equal(got[None][1][keep], pool0[keep]), tag + ": other pool slots modified"
    if every:
        assert not torch.isnan(got[None][2].float()).any(), tag + ": a checkpoint row was left unwritten"
        ko.check_close(got[None][2].float().cpu(), gold_ck, tag + " checkpoint rows")
        ko.check_close(got[None][2].float().cpu(), got[0][2].float().cpu(), tag + " checkpoint rows vs uncut call")


def test_cut_plan_follows_the_layout_under_one_graph(kda):
    """One captured graph: the planner cuts when a replay's layout has a dominating long sequence and does not when the
    same tokens come as many short ones."""
    H, T, N = 2, 8192, 16
    inputs = ko.make_inputs_raw(H, [T], 1300)
    q, k, v, g, beta, A_log, dt_bias, scale = to_dev(inputs[:8])
    pool0 = (torch.randn(N + 2, H, D, D, generator=torch.Generator().manual_seed(9)) * 0.25).to(DEV)
    pool = pool0.clone()
    idx = torch.arange(N, dtype=torch.int32, device=DEV)
    layouts = [[T - (N - 1)] + [1] * (N - 1), [T // N] * N, [5000, 3000] + [16] * 12 + [0, 0]]
    cu = cu_of(layouts[0])
    launch = kda.prepare(q, k, v, g, beta, A_log, dt_bias, scale, pool, cu, dynamic_layout=True, ssm_state_indices=idx)
    launch()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        res = launch()
    for lens, expect_cut in zip(layouts, (True, False, True)):
        cu.copy_(cu_of(lens))
        pool.copy_(pool0)
        graph.replay()
        torch.cuda.synchronize()
        assert kda.status_bits(launch) == 0 and kda.kernel_error(launch) == 0
        assert (launch.plan_counts()[2] > 0) == expect_cut, f"lens {lens[:4]}..: counts {launch.plan_counts()}"
        gold_o, gold_s, _ = gold_raw(inputs[:8], lens, init=pool0[:N].cpu())
        ko.check_close(res[0].cpu(), gold_o, f"graph replay with cuts, lens {lens[:4]}.. output")
        ko.check_close(pool[:N].cpu(), gold_s, f"graph replay with cuts, lens {lens[:4]}.. pool slots")
        assert torch.equal(pool[N:], pool0[N:])


def test_wrapper_matches_run(kda):
    d = to_dev(ko.make_inputs_raw(12, [1000, 300, 17], 900))
    q, k, v, g, beta, A_log, dt_bias, scale, init, cu = d
    a = kda.run(*d)
    a = (a[0].clone(), a[1].clone())
    b = kda.kda_prefill(q, k, v, g, beta, A_log, dt_bias, init, cu)
    assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])


def test_api_errors(kda):
    d = to_dev(ko.make_inputs_raw(12, [100, 200, 300, 400], 950))
    q, k, v, g, beta, A_log, dt_bias, scale, _, cu = d
    pool = torch.zeros(8, 12, D, D, device=DEV)
    idx = torch.arange(8, dtype=torch.int32, device=DEV)[::2]     # non-contiguous slot table
    with pytest.raises(ValueError):
        kda.run(q, k, v, g, beta, A_log, dt_bias, scale, pool, cu, ssm_state_indices=idx)
    with pytest.raises(ValueError):
        kda.run(q, k, v, g, beta, A_log[:6], dt_bias, scale, pool[:4], cu)
    with pytest.raises(ValueError):
        kda.run(q, k, v, g, beta, A_log, dt_bias, scale, pool[:4].double(), cu)
    with pytest.raises(ValueError):      # written pool aliases the source pool
        kda.run(q, k, v, g, beta, A_log, dt_bias, scale, pool, cu, ssm_state_indices=idx.contiguous(),
                initial_state_source=pool, initial_state_indices=idx.contiguous())
    with pytest.raises(ValueError):      # checkpoint interval not a multiple of the chunk
        kda.run(q, k, v, g, beta, A_log, dt_bias, scale, pool, cu, ssm_state_indices=idx.contiguous(),
                state_checkpoints=torch.zeros(40, 12, D, D, device=DEV),
                checkpoint_cu_starts=torch.zeros(5, dtype=torch.int64, device=DEV), checkpoint_every_n_tokens=48)


# ----------------------------------------------------------------------------------------------- table validation
def test_status_bits_neutralise_bad_tables(kda):
    H, lens = 4, [100, 60, 33]
    inputs = ko.make_inputs_raw(H, lens, 960)
    q, k, v, g, beta, A_log, dt_bias, scale = to_dev(inputs[:8])
    N, P = 3, 6
    gen = torch.Generator().manual_seed(1)
    pool0 = (torch.randn(P, H, D, D, generator=gen) * 0.25).to(DEV)

    # repeated slot: the first claim keeps it, the second sequence's state goes to scratch, bit 2
    pool = pool0.clone()
    idx = torch.tensor([2, 2, 9], dtype=torch.int32, device=DEV)       # 9 is out of range as well
    launch = kda.prepare(q, k, v, g, beta, A_log, dt_bias, scale, pool, cu_of(lens), dynamic_layout=True, ssm_state_indices=idx)
    out, _ = launch()
    assert kda.status_bits(launch) == 2
    gold_o, gold_s, _ = gold_raw(inputs, lens[:1], init=pool0[2:3].cpu())
    ko.check_close(pool[2:3].cpu(), gold_s, "first claimant's slot")
    ko.check_close(out[:, :100].cpu(), gold_o[:, :100], "first claimant's output")
    keep = [0, 1, 3, 4, 5]
    assert torch.equal(pool[keep], pool0[keep])
    assert bool(torch.isfinite(out.float()).all())

    # rejected cu_seqlens: every sequence empty, states untouched, output zero-filled, bit 1
    pool = pool0.clone()
    idx = torch.tensor([0, 1, 2], dtype=torch.int32, device=DEV)
    bad_cu = torch.tensor([0, 100, 90, 193], dtype=torch.int64, device=DEV)
    launch = kda.prepare(q, k, v, g, beta, A_log, dt_bias, scale, pool, bad_cu, dynamic_layout=True, ssm_state_indices=idx)
    out, _ = launch()
    assert kda.status_bits(launch) == 1
    assert torch.equal(pool, pool0)
    assert float(out.float().abs().max()) == 0.0

    # checkpoint rows outside the buffer / overlapping an earlier sequence: those sequences write none, bit 8
    pool = pool0.clone()
    ck = torch.full((5, H, D, D), float("nan"), device=DEV)
    ccs = torch.tensor([0, 1, 4, 0], dtype=torch.int64, device=DEV)     # seq 0 rows 0-3 (100/32 -> 4): seq 1 at row 1 overlaps
    launch = kda.prepare(q, k, v, g, beta, A_log, dt_bias, scale, pool, cu_of(lens), dynamic_layout=True, ssm_state_indices=idx,
                         state_checkpoints=ck, checkpoint_cu_starts=ccs, checkpoint_every_n_tokens=32)
    launch()
    assert kda.status_bits(launch) == 8
    assert bool(torch.isfinite(ck[:4]).all()) and bool(torch.isnan(ck[4]).all())
    assert torch.equal(ck[0], pool0[0])


# ----------------------------------------------------------------------------------------------- pre-activated call
def test_chunk_kda_plain_config0(kda):
    """BASELINE config 0: T=512, H=4, zero initial state, pre-activated fp32 inputs (q/k/v cast to bf16 by the call)."""
    q, k, v, g, beta, scale, init, cu = ko.make_inputs_plain(4, [512], 0, qkv_dtype=torch.float32, init_std=0.0)
    import c_oracle
    qb, kb, vb = (t.to(torch.bfloat16) for t in (q, k, v))
    gold_o, gold_s = c_oracle.recurrence_plain(qb, kb, vb, g, beta, scale, None, None)
    o, fin = kda.chunk_kda(q.to(DEV), k.to(DEV), v.to(DEV), g.to(DEV), beta.to(DEV), scale=scale, output_final_state=True)
    assert o.dtype == torch.float32 and tuple(fin.shape) == (1, 4, D, D)
    ko.check_close(o.cpu(), gold_o, "config 0 output")
    ko.check_close(fin.cpu(), gold_s, "config 0 final state")
    o2, none = kda.chunk_kda(q.to(DEV), k.to(DEV), v.to(DEV), g.to(DEV), beta.to(DEV))
    assert none is None and torch.equal(o2, o)


@pytest.mark.parametrize("g_mean", [0.0, 2.0])
def test_chunk_kda_plain_varlen(kda, g_mean):
    """BASELINE config 1 shape family at reduced size: varlen, bf16 q/k/v, fp32 g/beta, N(0, 0.05) initial states."""
    import c_oracle
    lens = [128, 1000, 333, 2047, 17]
    q, k, v, g, beta, scale, init, cu = ko.make_inputs_plain(8, lens, 11, g_mean=g_mean)
    gold_o, gold_s = c_oracle.recurrence_plain(q, k, v, g, beta, scale, init, cu)
    o, fin = kda.chunk_kda(q.to(DEV), k.to(DEV), v.to(DEV), g.to(DEV), beta.to(DEV), scale, init.to(DEV), True, cu.to(DEV))
    ko.check_close(o.cpu(), gold_o, "plain varlen output")
    ko.check_close(fin.cpu(), gold_s, "plain varlen final state")


def test_chunk_kda_batched(kda):
    import c_oracle
    q, k, v, g, beta, scale, init, cu = ko.make_inputs_plain(2, [96, 96, 96], 12)
    gold_o, gold_s = c_oracle.recurrence_plain(q, k, v, g, beta, scale, init, cu)
    rs = lambda t: t.reshape(3, 96, *t.shape[2:]).to(DEV)  # noqa: E731
    o, fin = kda.chunk_kda(rs(q), rs(k), rs(v), rs(g), rs(beta), scale, init.to(DEV), True)
    assert tuple(o.shape) == (3, 96, 2, D)
    ko.check_close(o.reshape(1, 288, 2, D).cpu(), gold_o, "batched output")
    ko.check_close(fin.cpu(), gold_s, "batched final state")


def test_zero_token_call_passes_states_through(kda):
    H = 4
    q = torch.zeros(1, 0, H, D, dtype=torch.bfloat16, device=DEV)
    beta = torch.zeros(1, 0, H, dtype=torch.bfloat16, device=DEV)
    pool = torch.randn(3, H, D, D, device=DEV)
    before = pool.clone()
    src = torch.randn(2, H, D, D, device=DEV)
    cu = torch.zeros(3, dtype=torch.int64, device=DEV)
    out, p = kda.run(q, q, q, q, beta, torch.zeros(H, device=DEV), torch.zeros(H * D, device=DEV), 0.1, pool, cu,
                     ssm_state_indices=torch.tensor([2, 0], dtype=torch.int32, device=DEV),
                     initial_state_source=src, initial_state_indices=torch.tensor([1, 0], dtype=torch.int32, device=DEV))
    torch.cuda.synchronize()
    assert out.shape[1] == 0
    assert torch.equal(pool[2], src[1]) and torch.equal(pool[0], src[0]) and torch.equal(pool[1], before[1])
