"""Host-side logic of the multi-GPU paths on CPU ranks (gloo, world size 2): token sharding, piece boundaries,
the all-gather layout and the scan order of context parallelism, and head sharding.  The three compute steps are
supplied by a stand-in backend built on the CPU oracle, so what is under test is the orchestration in
kda_b200/parallel.py; the CUDA backend's numerics are covered by the GPU tests."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import kda_oracle as ko

D = 128


class OracleBackend:
    """The three context-parallel steps restated with the CPU oracle (test infrastructure)."""

    def segment_maps(self, q, k, v, g, beta, A_log, dt_bias, scale, raw, bounds, need_map, first_state):
        assert raw
        qn, kn, a, b = ko.activate_raw(q[0], k[0], g[0], beta[0], A_log, dt_bias)
        vf = v[0].double()
        T, H = q.shape[1], q.shape[2]
        n = len(bounds) - 1
        out = torch.zeros(1, T, H, D, dtype=torch.float64)
        qt = torch.zeros(1, T, H, D, dtype=torch.float64)
        P = torch.zeros(n, H, D, D, dtype=torch.float64)
        S_loc = torch.zeros(n, H, D, D, dtype=torch.float64)
        for i in range(n):
            sl = slice(bounds[i], bounds[i + 1])
            L = bounds[i + 1] - bounds[i]
            S0 = torch.zeros(1, H, D, D, dtype=torch.float64)
            if not need_map[i] and first_state is not None:
                S0 = first_state[i:i + 1].double().transpose(-1, -2)
            o, fin = ko._recur(qn[sl], kn[sl], vf[sl], a[sl], b[sl], scale, S0, [0, L])
            out[0, sl] = o
            S_loc[i] = fin[0].transpose(-1, -2)
            if need_map[i]:
                P[i], qt[0, sl] = ko.segment_map(qn[sl], kn[sl], a[sl], b[sl], scale)
        return out, qt, P, S_loc

    def scan(self, P, S_loc, S0):
        n, H = P.shape[0], P.shape[1]
        cur = torch.zeros(H, D, D, dtype=P.dtype) if S0 is None else S0.clone()
        S_in = torch.zeros_like(S_loc)
        for i in range(n):
            S_in[i] = cur
            cur = cur @ P[i] + S_loc[i]
        return S_in, cur

    def fixup(self, out, qt, S_in, bounds, need_map):
        for i in range(len(bounds) - 1):
            if need_map[i]:
                sl = slice(bounds[i], bounds[i + 1])
                out[0, sl] += torch.einsum("hvk,thk->thv", S_in[i], qt[0, sl])
        return out


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _cp_worker(rank, world, port, pieces, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from kda_b200 import parallel
        H, T = 2, 160
        q, k, v, g, beta, A_log, dt_bias, scale, init, cu = ko.make_inputs_raw(H, [T], 21)
        cuts = [0, 96, T] if world == 2 else [0, T]
        sl = slice(cuts[rank], cuts[rank + 1])
        out, fin = parallel.context_parallel_prefill(q[:, sl], k[:, sl], v[:, sl], g[:, sl], beta[:, sl], A_log, dt_bias, scale,
                                                     init if rank == 0 else None, pieces=pieces, backend=OracleBackend())
        gold_o, gold_f = ko.kda_recurrence(q, k, v, g, beta, A_log, dt_bias, scale, init, cu)
        ok_o = torch.allclose(out[0].float(), gold_o[0, sl].float(), atol=2e-3, rtol=2e-2)
        ok_f = torch.allclose(fin.float(), gold_f, atol=1e-5, rtol=1e-5)
        ret[rank] = (bool(ok_o), bool(ok_f), float((out[0].float() - gold_o[0, sl].float()).abs().max()))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("pieces", [1, 3])
def test_context_parallel_orchestration_two_ranks(pieces):
    world, port = 2, _free_port()
    ret = mp.Manager().dict()
    mp.spawn(_cp_worker, args=(world, port, pieces, ret), nprocs=world, join=True)
    for r in range(world):
        assert ret[r][0] and ret[r][1], f"rank {r}: {ret[r]}"


def test_split_pieces_and_head_slice():
    from kda_b200 import parallel
    assert parallel.split_pieces(160, 2) == [0, 96, 160]
    assert parallel.split_pieces(100, 8) == [0, 32, 64, 96, 100]
    assert parallel.split_pieces(1, 4) == [0, 1]
    b = parallel.split_pieces(131072 // 8, 3)
    assert b[0] == 0 and b[-1] == 16384 and all(x % 32 == 0 for x in b)
    t = torch.arange(2 * 3 * 8 * 4).reshape(2, 3, 8, 4)
    (s,) = parallel.head_slice(1, 4, t)
    assert s.shape == (2, 3, 2, 4) and torch.equal(s, t[:, :, 2:4])
    with pytest.raises(ValueError):
        parallel.head_slice(0, 3, t)
    # wave model: rank 0 of a long H=96 sequence keeps one plain chain (96 CTAs, one wave); mapped ranks cut into
    # three pieces (576 CTAs in four waves of a third of the chunks beat 192 CTAs in two waves of all of them)
    assert parallel.choose_pieces(16384, 96, True) == 1
    assert parallel.choose_pieces(16384, 96, False) == 3
    assert parallel.choose_pieces(32, 4, False) == 1
    # cost-balanced shards: chunk-aligned, in order, sum to T, and a smaller makespan than the equal split
    for world in (2, 4, 8):
        sh = parallel.balanced_shards(131072, world, 96)
        assert sum(sh) == 131072 and all(x % 32 == 0 and x > 0 for x in sh) and sh[0] > sh[1]
        bal = max(parallel.segment_cost(t, 96, i == 0) for i, t in enumerate(sh))
        eq = max(parallel.segment_cost(131072 // world, 96, i == 0) for i in range(world))
        assert bal < eq
    # planned piece boundaries: start at 0, end at T, strictly increasing, chunk-aligned inside; with H = 96 on 148
    # SMs the first rank keeps a long plain piece next to shorter mapped ones, and the plan beats a single piece
    for T, H, first in ((131072, 96, True), (131072, 96, False), (1000, 4, True), (40, 2, True), (33, 2, False), (1, 1, True), (32, 3, False)):
        b = parallel.plan_bounds(T, H, first)
        assert b[0] == 0 and b[-1] == T and all(x < y for x, y in zip(b[:-1], b[1:])) and all(x % 32 == 0 for x in b[:-1])
    b = parallel.plan_bounds(131072, 96, True)
    assert len(b) >= 3 and b[1] - b[0] > b[2] - b[1]
    assert parallel.segment_cost(131072, 96, True) < 4096
    assert parallel.balanced_shards(1000, 1, 4) == [1000]
    sh = parallel.balanced_shards(1000, 3, 4)
    assert sum(sh) == 1000 and all(x % 32 == 0 for x in sh[:-1])


def _hp_worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from kda_b200 import parallel
        H, lens = 4, [40, 9]
        q, k, v, g, beta, A_log, dt_bias, scale, init, cu = ko.make_inputs_raw(H, lens, 22)
        qs, ks, vs, gs, bs = parallel.head_slice(rank, world, q, k, v, g, beta)
        (ins,) = parallel.head_slice(rank, world, init, heads_dim=1)
        hs = H // world
        o, f = ko.kda_recurrence(qs, ks, vs, gs, bs, A_log[rank * hs:(rank + 1) * hs], dt_bias.view(H, D)[rank * hs:(rank + 1) * hs].reshape(-1),
                                 scale, ins, cu)
        of = o.float().contiguous()
        parts = [torch.zeros_like(of) for _ in range(world)]
        dist.all_gather(parts, of)
        gold_o, _ = ko.kda_recurrence(q, k, v, g, beta, A_log, dt_bias, scale, init, cu)
        ret[rank] = bool(torch.equal(torch.cat(parts, 2), gold_o.float()))
    finally:
        dist.destroy_process_group()


def test_head_parallel_shards_reassemble():
    world, port = 2, _free_port()
    ret = mp.Manager().dict()
    mp.spawn(_hp_worker, args=(world, port, ret), nprocs=world, join=True)
    assert all(ret[r] for r in range(world))
