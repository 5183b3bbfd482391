"""GPU parity of the context-parallel path (segment maps, scan, fix-up) and the state row copies, through the C ABI.
Single GPU: the pieces are segments of one chain, the same algebra that runs across ranks (the multi-rank
orchestration is covered on CPU ranks by tests/test_parallel_cpu.py)."""
import ctypes as C

import pytest
import torch

import kda_oracle as ko
from kda_testlib import DEV, D, gold_raw, slow_gates_, to_dev

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def kda():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    import kda_b200
    return kda_b200


@pytest.mark.parametrize("H,T,pieces,slow,kernel", [(4, 1000, 4, False, 0), (2, 2048, 3, True, 0), (8, 333, 8, False, 0),
                                                    (4, 1000, 4, False, 1), (3, 97, 2, False, 0), (2, 40, 5, False, 0),
                                                    (96, 4096, 0, False, 0), (5, 777, 0, True, 0)])   # 0: planned boundaries
def test_context_parallel_single_gpu(kda, H, T, pieces, slow, kernel):
    from kda_b200 import parallel
    inputs = ko.make_inputs_raw(H, [T], 40 + H + pieces)
    if slow:
        slow_gates_(inputs, 40)
    gold_o, gold_s, _ = gold_raw(inputs, [T])
    q, k, v, g, beta, A_log, dt_bias, scale, init, _ = to_dev(inputs)
    out, fin = parallel.context_parallel_prefill(q, k, v, g, beta, A_log, dt_bias, scale, init, pieces=pieces,
                                                 backend=parallel.CudaBackend(kernel=kernel))
    torch.cuda.synchronize()
    tag = f"cp H={H} T={T} pieces={pieces} slow={slow} kernel={kernel}"
    ko.check_close(out.cpu(), gold_o, tag + " output")
    ko.check_close(fin.cpu(), gold_s, tag + " final_state")
    # and against the ordinary single-chain call on the same device
    o2, f2 = kda.run(q, k, v, g, beta, A_log, dt_bias, scale, init)
    ko.check_close(out.cpu(), o2.cpu(), tag + " vs plain call (output)", 6e-3)
    ko.check_close(fin.cpu(), f2.cpu(), tag + " vs plain call (state)", 6e-3)


@pytest.mark.parametrize("H,bounds,slow,plain_first", [(4, [0, 500, 1000], False, False), (2, [0, 33, 64, 1000, 2047], True, False),
                                                       (148, [0, 4096], False, False), (3, [0, 1, 40], False, False),
                                                       (5, [0, 640, 900, 1500], False, True), (150, [0, 2048, 2560], True, True)])
def test_dual_chain_segments_match_two_task_segments(kda, H, bounds, slow, plain_first):
    """A mapped segment as ONE dual-chain task (both chains over one operand preparation) gives the outputs, Qt rows and
    state maps of the two-task scheme (chain L and chain Tr as separate tasks): the same products in the same order, so
    bit for bit; and the maps reproduce the plain chain's final state.  `plain_first`: the launch mixes a plain first
    piece (from the caller's state) with dual-chain tasks, as the first rank of a context-parallel call does."""
    from kda_b200 import parallel
    T = bounds[-1]
    inputs = ko.make_inputs_raw(H, [T], 50 + H)
    if slow:
        slow_gates_(inputs, 50)
    q, k, v, g, beta, A_log, dt_bias, scale, init, _ = to_dev(inputs)
    need = [1] * (len(bounds) - 1)
    if plain_first:
        need[0] = 0
    res = {}
    for dual in (True, False):
        be = parallel.CudaBackend(dual=dual)
        out, qt, P, S_loc = be.segment_maps(q, k, v, g, beta, A_log, dt_bias, scale, True, bounds, need,
                                            init if plain_first else None)
        o_rows, q_rows = be.rows_of(out, qt, bounds, need)       # the dual-chain tasks write tiles: bring them to rows
        res[dual] = [t.clone() for t in (o_rows, q_rows, P, S_loc)]
        torch.cuda.synchronize()
        assert be.kernel_error() == 0
    t_map = bounds[1] if plain_first else 0          # Qt rows exist for mapped tokens only
    for name, a, b in zip(("o_loc", "Qt", "P", "S_loc"), res[True], res[False]):
        if name == "Qt":
            a, b = a[:, t_map:], b[:, t_map:]
        assert torch.equal(a, b), f"dual-chain {name} differs from the two-task scheme (H={H}, bounds={bounds})"
    # compose the maps from the initial state and compare with the plain call's final state
    S = init[0].double().cpu()
    for i in range(len(need)):
        S = S @ res[True][2][i].double().cpu() + res[True][3][i].double().cpu()
    _, fin = kda.run(q, k, v, g, beta, A_log, dt_bias, scale, init, max_cut_pieces=0)
    ko.check_close(S.float()[None], fin.cpu(), f"state through the dual-chain maps (H={H}, bounds={bounds})", 6e-3)


@pytest.mark.parametrize("H,bounds", [(3, [0, 33, 64, 1000, 2047]), (5, [0, 1, 40, 41]), (8, [0, 512, 1024])])
def test_fixup_over_tiles_matches_fixup_over_rows(kda, H, bounds):
    """The two forms of the fix-up (tile-major scratch of dual-chain tasks, rows of the two-task scheme) give the same
    output rows bit for bit, also for pieces that do not start on a multiple of 32 tokens, and they match the plain
    call within the tolerance."""
    from kda_b200 import parallel
    T = bounds[-1]
    inputs = ko.make_inputs_raw(H, [T], 90 + H)
    q, k, v, g, beta, A_log, dt_bias, scale, init, _ = to_dev(inputs)
    need = [0] + [1] * (len(bounds) - 2)
    outs = {}
    for dual in (True, False):
        be = parallel.CudaBackend(dual=dual)
        out, qt, P, S_loc = be.segment_maps(q, k, v, g, beta, A_log, dt_bias, scale, True, bounds, need, init)
        S_in, _ = be.scan(P, S_loc, None)
        outs[dual] = be.fixup(out, qt, S_in, bounds, need).clone()
        torch.cuda.synchronize()
        assert be.kernel_error() == 0
    assert torch.equal(outs[True], outs[False]), f"tile and row forms of the fix-up differ (H={H}, bounds={bounds})"
    o2, _ = kda.run(q, k, v, g, beta, A_log, dt_bias, scale, init, max_cut_pieces=0)
    ko.check_close(outs[True].cpu(), o2.cpu(), f"fix-up over tiles vs the plain call (H={H}, bounds={bounds})", 6e-3)


def test_context_parallel_call_replays_under_a_cuda_graph(kda):
    """With a reusing backend the context-parallel call allocates nothing after its first run, synchronises nowhere and
    reads its inputs where they lie: captured once, replayed after the inputs were refilled in place, it gives the
    result of the refilled inputs."""
    from kda_b200 import parallel
    H, T = 6, 4096
    be = parallel.CudaBackend(reuse=True)
    data = [to_dev(ko.make_inputs_raw(H, [T], seed)) for seed in (61, 62)]
    q, k, v, g, beta, A_log, dt_bias, scale, init, _ = [t.clone() if torch.is_tensor(t) else t for t in data[0]]

    def call():
        return parallel.context_parallel_prefill(q, k, v, g, beta, A_log, dt_bias, scale, init, pieces=4, backend=be)

    for _ in range(2):
        call()                                    # warm-up: buffers, tables, plan
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out, fin = call()
    for src in (data[1], data[0]):
        for dst, t in zip((q, k, v, g, beta, A_log, dt_bias, init), (*src[:7], src[8])):
            dst.copy_(t)
        graph.replay()
        torch.cuda.synchronize()
        assert be.kernel_error() == 0
        o2, f2 = kda.run(q, k, v, g, beta, A_log, dt_bias, scale, init, max_cut_pieces=0)
        ko.check_close(out.cpu(), o2.cpu(), "graph replay of the context-parallel call (output)", 6e-3)
        ko.check_close(fin.cpu(), f2.cpu(), "graph replay of the context-parallel call (state)", 6e-3)


def test_scan_matches_fp64(kda):
    from kda_b200 import parallel
    be = parallel.CudaBackend()
    gen = torch.Generator().manual_seed(5)
    n, H = 5, 3
    P = (torch.randn(n, H, D, D, generator=gen) * 0.08)
    L = torch.randn(n, H, D, D, generator=gen)
    S0 = torch.randn(H, D, D, generator=gen)
    S_in, S_end = be.scan(P.to(DEV), L.to(DEV), S0.to(DEV))
    cur = S0.double()
    for i in range(n):
        assert torch.allclose(S_in[i].cpu().double(), cur, rtol=1e-4, atol=1e-4)
        cur = cur @ P[i].double() + L[i].double()
    assert torch.allclose(S_end.cpu().double(), cur, rtol=1e-4, atol=1e-4)


def test_scan_over_one_gathered_buffer_matches_the_packed_scan(kda):
    """Maps that lie apart (the two halves of one [n][2][H][128][128] buffer, as one all-gather of (P, S_loc) pairs
    delivers them) scan to the same bits as packed maps."""
    from kda_b200 import parallel
    be = parallel.CudaBackend()
    gen = torch.Generator().manual_seed(6)
    n, H = 4, 5
    both = torch.randn(n, 2, H, D, D, generator=gen).to(DEV)
    both[:, 0] *= 0.08
    S0 = torch.randn(H, D, D, generator=gen).to(DEV)
    a_in, a_end = [t.clone() for t in be.scan(both[:, 0].contiguous(), both[:, 1].contiguous(), S0)]
    b_in, b_end = be.scan(both[:, 0], both[:, 1], S0)
    torch.cuda.synchronize()
    assert torch.equal(a_in, b_in) and torch.equal(a_end, b_end)


def test_state_rows_copy(kda):
    from kda_b200 import _cabi
    lib = _cabi.lib()
    H = 3
    src = torch.randn(6, H, D, D, device=DEV)
    idx = torch.tensor([4, 0, 5], dtype=torch.int32, device=DEV)
    dst = torch.zeros(3, H, D, D, device=DEV)
    st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert lib.kda_state_rows_copy(dst.data_ptr(), H * D * D, 0, src.data_ptr(), H * D * D, idx.data_ptr(), 3, H, st) == 0
    torch.cuda.synchronize()
    assert torch.equal(dst, src[idx.long()])
    dstb = torch.zeros(3, H, D, D, device=DEV, dtype=torch.bfloat16)
    assert lib.kda_state_rows_copy(dstb.data_ptr(), H * D * D, 1, src.data_ptr(), H * D * D, idx.data_ptr(), 3, H, st) == 0
    torch.cuda.synchronize()
    assert torch.equal(dstb, src[idx.long()].to(torch.bfloat16))       # round to nearest even


@pytest.mark.parametrize("H,T,every,pieces,ck_dtype", [(4, 2048, 64, 4, torch.float32), (3, 1000, 64, 3, torch.bfloat16),
                                                       (2, 4096, 0, 5, None), (16, 8192, 256, 0, torch.bfloat16)])
def test_cut_sequence_matches_the_serving_call(kda, H, T, every, pieces, ck_dtype):
    """One long sequence cut into pieces (two passes: affine maps + scan for the entering states, then the ordinary
    launch over the pieces) gives the output, pool slot and checkpoint rows of the uncut serving call and of the fp64
    recurrence."""
    from kda_b200 import parallel
    inputs = ko.make_inputs_raw(H, [T], 70 + H)
    q, k, v, g, beta, A_log, dt_bias, scale, init, _ = to_dev(inputs)
    gen = torch.Generator().manual_seed(5)
    pool0 = (torch.randn(6, H, D, D, generator=gen) * 0.25).to(DEV)
    slot, row0 = 4, 3
    rows = -(-T // every) if every else 0
    res = {}
    for mode in ("plain", "cut"):
        pool = pool0.clone()
        ck = torch.full((rows + row0 + 2, H, D, D), float("nan"), dtype=ck_dtype, device=DEV) if every else None
        if mode == "plain":
            kw = dict(dynamic_layout=True, ssm_state_indices=torch.tensor([slot], dtype=torch.int32, device=DEV))
            if every:
                kw.update(state_checkpoints=ck, checkpoint_every_n_tokens=every,
                          checkpoint_cu_starts=torch.tensor([row0, row0 + rows], dtype=torch.int64, device=DEV))
            launch = kda.prepare(q, k, v, g, beta, A_log, dt_bias, scale, pool, None, **kw)
        else:
            launch = parallel.prepare_cut_sequence(q, k, v, g, beta, A_log, dt_bias, scale, pool, slot, state_checkpoints=ck,
                                                   checkpoint_row0=row0, checkpoint_every_n_tokens=every, pieces=pieces)
            assert launch.pieces >= 2
        out = launch()[0]
        launch()                                   # a second call on the updated pool must not depend on leftovers
        pool.copy_(pool0)
        out = launch()[0]
        torch.cuda.synchronize()
        assert kda.status_bits(launch) == 0 and kda.kernel_error(launch) == 0
        res[mode] = (out.clone(), pool.clone(), None if ck is None else ck.clone())
    gold_o, gold_s, gold_ck = gold_raw(inputs[:8] + [pool0[slot:slot + 1].cpu()], [T], every=every)
    tag = f"cut sequence H={H} T={T} every={every} pieces={pieces}"
    ko.check_close(res["cut"][0].cpu(), gold_o, tag + " output")
    ko.check_close(res["cut"][1][slot].cpu(), gold_s[0], tag + " pool slot")
    ko.check_close(res["cut"][0].cpu().float(), res["plain"][0].cpu().float(), tag + " output vs uncut call")
    ko.check_close(res["cut"][1][slot].cpu(), res["plain"][1][slot].cpu(), tag + " pool slot vs uncut call")
    others = [i for i in range(6) if i != slot]
    assert torch.equal(res["cut"][1][others], pool0[others]), tag + ": other pool slots changed"
    if every:
        ko.check_close(res["cut"][2][row0:row0 + rows].float().cpu(), res["plain"][2][row0:row0 + rows].float().cpu(), tag + " checkpoint rows")
        assert torch.isnan(res["cut"][2][:row0].float()).all() and torch.isnan(res["cut"][2][row0 + rows:].float()).all(), tag + ": rows outside the range written"
