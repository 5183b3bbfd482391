"""Multi-GPU execution of KDA prefill: head parallelism and context parallelism (one process per GPU).

Head parallelism needs no communication: heads are independent, so rank r runs the ordinary call on its head slice
(`head_slice`), reading strided views of wider tensors in place.

Context parallelism splits ONE long sequence over tokens.  The recurrence is affine in the state, so a token segment
that does not know its entering state yet can still be processed (value-first orientation, as
kda/b200/csrc/w3/kernel.py:22-38 and kda/b200/csrc/w3/cp_fix.cu:4-21 of the reference do inside one GPU):

    chain L  (S0 = 0, real v)   ->  o_loc, S_loc            chain Tr (S0 = I, v = 0)   ->  Qt, P
    S_end = S_in @ P + S_loc            out_t = o_loc_t + S_in applied to Qt_t

Every rank cuts its token shard into `pieces` chunk-aligned pieces (more pieces = more CTAs to fill 148 SMs), runs both
chains per piece in one launch, composes its pieces into one map per head, all-gathers the per-rank maps
(2 x H x 64 KB fp32 per rank) over NCCL, scans them to get its entering state, scans its own pieces from there and
fixes the outputs up.  The first piece of rank 0 knows its entering state (the caller's initial state), runs the plain
chain and contributes the map (P = 0, S_loc = its true end state), which keeps the algebra uniform.

The three compute steps go through the C ABI (kda_segment_launch, kda_scan_launch, kda_fixup_tiles_launch or
kda_fixup_launch).  They are
grouped in a backend object so that the orchestration (piece boundaries, gather layout, scan order) can be exercised
on CPU ranks with a stand-in backend supplied by the tests; the package itself ships only the CUDA backend.
"""
from __future__ import annotations

import ctypes as C
import functools

import torch

from . import _cabi

D = 128
CHUNK = 32


def head_slice(rank, world, *tensors, heads_dim=2):
    """Views of the heads owned by `rank` (contiguous block of H/world heads) of [1,T,H,...] token tensors."""
    out = []
    for t in tensors:
        H = t.shape[heads_dim]
        if H % world:
            raise ValueError(f"KDA kernel: {H} heads do not shard evenly over {world} ranks")
        hs = H // world
        out.append(t.narrow(heads_dim, rank * hs, hs))
    return out


def split_pieces(T, pieces):
    """Chunk-aligned piece boundaries of a shard of T tokens: `pieces` near-equal runs (fewer when T is short)."""
    nchunks = -(-T // CHUNK)
    pieces = max(1, min(pieces, nchunks))
    base, extra = divmod(nchunks, pieces)
    bounds, c = [0], 0
    for i in range(pieces):
        c += base + (1 if i < extra else 0)
        bounds.append(min(T, c * CHUNK))
    return bounds


def choose_pieces(T, H, first_rank, n_sms=148, max_pieces=8):
    """Pieces per rank that minimise the makespan of the segment launch in chunk steps: a mapped piece costs two CTAs
    per head (chains L and Tr), the unmapped first piece of rank 0 one; CTAs run in waves of `n_sms`."""
    nchunks = -(-T // CHUNK)
    best, best_cost = 1, None
    for p in range(1, max(1, min(max_pieces, nchunks)) + 1):
        ctas = H * (2 * p - (1 if first_rank else 0))
        cost = -(-ctas // n_sms) * -(-nchunks // p)
        if best_cost is None or cost < best_cost:
            best, best_cost = p, cost
    return best


def _makespan(costs, n_sms):
    """Longest-first list scheduling of task costs on n_sms workers (what the hardware block scheduler does with a
    grid whose CTAs are ordered by decreasing length)."""
    import heapq
    heap = [0.0] * n_sms
    for c in sorted(costs, reverse=True):
        heapq.heapreplace(heap, heap[0] + c)
    return max(heap)


def plan_bounds(T, H, first_rank, n_sms=148, max_pieces=8, task_overhead=3.0, fixup_steps_per_chunk_head=0.0025):
    """Piece boundaries of one rank's shard (see `_plan`, which also returns the simulated cost)."""
    return list(_plan(T, H, first_rank, n_sms, max_pieces, task_overhead, fixup_steps_per_chunk_head)[0])


DUAL_COST = 1.40     # a dual-chain chunk step (with its two output tiles) in units of a single-chain one (measured inside the
                     # 131072-token segment launches: 3.44 us against 2.47 us per chunk at 1.97 GHz)


@functools.lru_cache(maxsize=256)        # the search costs milliseconds on the host; layouts repeat call after call
def _plan(T, H, first_rank, n_sms=148, max_pieces=8, task_overhead=3.0, fixup_steps_per_chunk_head=0.0025):
    """Piece boundaries (chunk-aligned token offsets, first 0, last T) of one rank's shard, chosen by simulating the
    segment launch: the first piece of the first rank is one plain task per head, every mapped piece ONE dual-chain task
    per head (`DUAL_COST`; with `CudaBackend(dual=False)` or the cross-check kernel it is two plain tasks, which this
    model does not follow); a task costs its chunks plus `task_overhead` chunk steps, and mapped tokens cost a fix-up
    pass.  On the first rank the plain first piece may be LONGER than the mapped pieces: while its H CTAs run, the
    remaining SMs work through the dual chains of the shorter pieces (with H = 96 on 148 SMs the plain chain alone
    would leave a third of the GPU idle)."""
    nch = -(-T // CHUNK)
    if nch <= 1:
        return [0, T], (float(nch) + task_overhead, 0.0)
    best, best_cost = [0, nch], None
    firsts = sorted({nch} | {max(1, int(nch * f / 32)) for f in range(1, 32)}) if first_rank else [0]
    for c_first in firsts:
        rest = nch - c_first
        for m in range(0, max_pieces + 1):
            if (m == 0) != (rest == 0) or m > rest:      # m mapped pieces share the `rest` chunks (none when rest = 0)
                continue
            base, extra = divmod(rest, m) if m else (0, 0)
            pieces = [base + (1 if i < extra else 0) for i in range(m)]
            costs = [c_first + task_overhead] * H if c_first else []
            for c in pieces:
                # a mapped piece runs as one dual-chain task per head
                costs += [DUAL_COST * c + task_overhead] * H
            seg = _makespan(costs, n_sms)
            fix = fixup_steps_per_chunk_head * rest * H
            if best_cost is None or seg + fix < sum(best_cost) - 1e-9:
                cuts, acc = [0], 0
                for c in ([c_first] if c_first else []) + pieces:
                    acc += c
                    cuts.append(acc)
                best, best_cost = cuts, (seg, fix)
    return [min(T, c * CHUNK) for c in best], best_cost


def segment_cost(T, H, first_rank, n_sms=148, max_pieces=8):
    """Simulated makespan of a rank's segment launch plus its fix-up pass, in chunk steps (see `plan_bounds`)."""
    return sum(phase_costs(T, H, first_rank, n_sms, max_pieces))


def phase_costs(T, H, first_rank, n_sms=148, max_pieces=8):
    """(segment launch, fix-up pass) of a rank's shard in chunk steps."""
    if T <= 0:
        return 0.0, 0.0
    return _plan(T, H, first_rank, n_sms, max_pieces)[1]


def balanced_shards(T, world, H, n_sms=148, max_pieces=8):
    """Token counts per rank for a context-parallel call over `world` ranks (see `_balanced_shards`)."""
    return list(_balanced_shards(T, world, H, n_sms, max_pieces))


@functools.lru_cache(maxsize=64)         # about a second of host search for a new (T, world, H); layouts repeat
def _balanced_shards(T, world, H, n_sms, max_pieces):
    """Token counts per rank (chunk-aligned, in rank order, summing to T) for context parallelism.  Rank 0 runs the plain
    chain on its first piece while every other piece runs two chains, so equal shards leave rank 0 idle (the reference
    cuts unequal segments for the same reason, kda/b200/csrc/w3/kernel.py:22-38).  The exchange of the maps stands
    between the segment launches and the fix-up passes of all ranks, so the call lasts
    max over ranks (segments) + max over ranks (fix-up); the first shard is the one that minimises that sum in the wave
    model, the other ranks share the rest equally."""
    nch = -(-T // CHUNK)
    if world <= 1 or nch < world:
        return (T,) + (0,) * (world - 1)

    def split(c0):
        rest = nch - c0
        base, extra = divmod(rest, world - 1)
        return [c0] + [base + (1 if i < extra else 0) for i in range(world - 1)]

    def cost(c0):
        ch = split(c0)
        ph = [phase_costs(ch[0] * CHUNK, H, True, n_sms, max_pieces), phase_costs(ch[1] * CHUNK, H, False, n_sms, max_pieces)]
        return max(x[0] for x in ph) + max(x[1] for x in ph)

    # coarse scan of the first shard between the equal share and the whole sequence, then a local refinement
    lo, hi = nch // world, nch - (world - 1)
    step = max(1, (hi - lo) // 48)
    best = min(range(lo, hi + 1, step), key=cost)
    while step > 1:
        step = max(1, step // 4)
        best = min(range(max(lo, best - 4 * step), min(hi, best + 4 * step) + 1, step), key=cost)
    chunks = split(best)
    shards = [c * CHUNK for c in chunks]
    shards[-1] -= nch * CHUNK - T          # the last chunk of the sequence may be partial
    return tuple(shards)


class CudaBackend:
    """The shipped backend: the three context-parallel steps on the current CUDA device through the C ABI."""

    def __init__(self, kernel=None, dual=True, reuse=False):
        from . import default_kernel
        self.lib = _cabi.lib()
        self.kernel = default_kernel() if kernel is None else int(kernel)
        self.dual = bool(dual)      # a mapped segment is one dual-chain task (False: two tasks, chains L and Tr)
        # reuse=True: every result and scratch tensor is allocated once per shape and handed out again at the next call
        # (a serving loop over one layout then allocates nothing after its first step; results of a call are only
        # valid until the next one)
        self.reuse = bool(reuse)
        self._bufs = {}
        self._table_cache = {}
        self._tiled = (False, 0, 0)
        self.status = None          # int32[4] of the most recent segment launch: [2] != 0 means a wait inside it gave up

    def _buf(self, key, shape, dtype, dev, zero=False):
        if not self.reuse:
            return (torch.zeros if zero else torch.empty)(shape, dtype=dtype, device=dev)
        k = (key, tuple(shape), dtype, str(dev))
        t = self._bufs.get(k)
        if t is None:
            t = self._bufs[k] = (torch.zeros if zero else torch.empty)(shape, dtype=dtype, device=dev)
        elif zero:
            t.zero_()
        return t

    def kernel_error(self):
        """Device-side error code of the most recent segment launch (0 = none); synchronises."""
        return 0 if self.status is None else int(self.status[2].item())

    def _tables(self, bounds, need_map, dev):
        """Device copies of the piece tables, kept per layout: a repeated call uploads nothing."""
        key = (tuple(bounds), tuple(need_map), str(dev))
        t = self._table_cache.get(key)
        if t is None:
            if len(self._table_cache) > 64:
                self._table_cache.clear()
            t = (torch.tensor(bounds[:-1], dtype=torch.int64, device=dev), torch.tensor(bounds[1:], dtype=torch.int64, device=dev),
                 torch.tensor(need_map, dtype=torch.int32, device=dev))
            self._table_cache[key] = t
        return t

    @staticmethod
    def _stream(dev):
        return C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)

    def segment_maps(self, q, k, v, g, beta, A_log, dt_bias, scale, raw, bounds, need_map, first_state):
        """Runs chain L (and chain Tr where need_map) for the pieces [bounds[i], bounds[i+1]) in one launch.
        Returns (out, qt, P, S_loc): P, S_loc [n,H,128,128] fp32 (value-first); out [1,T,H,128] bf16; qt the handle that
        `fixup` takes.  On the tcgen05 kernel a mapped piece is ONE dual-chain task per head (both chains over one operand
        preparation) next to the plain tasks of unmapped pieces; its o_loc and Qt go TILE-MAJOR into a scratch
        (`qt` is that scratch; `out` then holds rows only for unmapped pieces until `fixup` has run; `rows_of` gives the
        row form for inspection).  `dual=False` keeps two tasks per mapped piece with o_loc rows in `out` and Qt rows in
        `qt` [1,T,H,128]."""
        dev = q.device
        T, H = q.shape[1], q.shape[2]
        n = len(bounds) - 1
        tiled = self.dual and self.kernel == _cabi.KERNEL_TCGEN05 and any(need_map)
        out = self._buf("out", (1, T, H, D), torch.bfloat16, dev)
        n_tiles = sum(-(-(bounds[i + 1] - bounds[i]) // CHUNK) for i in range(n))
        if tiled:
            qt = self._buf("tiles", (2, n_tiles, H, D, CHUNK), torch.bfloat16, dev)      # [0] Qt tiles, [1] o_loc tiles
        else:
            qt = self._buf("qt", (1, T, H, D), torch.bfloat16, dev)
        self._tiled = (tiled, n_tiles, T)
        # (the P of an unmapped piece must read as the zero map; mapped pieces overwrite theirs)
        P = self._buf("P", (n, H, D, D), torch.float32, dev, zero=not all(need_map))
        S_loc = self._buf("S_loc", (n, H, D, D), torch.float32, dev)
        t0, t1, nm = self._tables(bounds, need_map, dev)
        ws_bytes = self.lib.kda_prefill_workspace_bytes(2 * n, H)
        ws = self._buf("ws", (ws_bytes + 256,), torch.uint8, dev)
        status = self._buf("status", (4,), torch.int32, dev)
        self.status = status
        s = _cabi.KdaSegmentArgs()
        a = s.base
        a.q, a.k, a.v, a.g, a.beta, a.out = q.data_ptr(), k.data_ptr(), v.data_ptr(), g.data_ptr(), beta.data_ptr(), out.data_ptr()
        a.ldq, a.ldk, a.ldv, a.ldg = (t.stride(1) if T > 1 else H * D for t in (q, k, v, g))
        a.ldbeta = beta.stride(1) if T > 1 else H
        a.ldo = H * D
        a.A_log = A_log.data_ptr() if raw else None
        a.dt_bias = dt_bias.data_ptr() if raw else None
        a.scale, a.lower_bound = float(scale), -5.0
        a.frontend = _cabi.FRONTEND_RAW if raw else _cabi.FRONTEND_PLAIN
        a.state_layout = _cabi.STATE_VALUE_FIRST
        a.H, a.N, a.T = H, n, T
        if first_state is not None:
            a.src_base, a.src_slot_stride, a.src_slots = first_state.data_ptr(), first_state.stride(0), first_state.shape[0]
        a.workspace, a.workspace_bytes = (ws.data_ptr() + 255) // 256 * 256, ws_bytes
        a.status = status.data_ptr()
        a.kernel = _cabi.KERNEL_TCGEN05_TWO_TASK if (self.kernel == _cabi.KERNEL_TCGEN05 and not self.dual) else self.kernel
        s.n_seg = n
        s.seg_t0, s.seg_t1, s.seg_need_map = t0.data_ptr(), t1.data_ptr(), nm.data_ptr()
        s.qt, s.P, s.S_loc = qt.data_ptr(), P.data_ptr(), S_loc.data_ptr()
        if tiled:
            s.tiles, s.n_tiles = qt.data_ptr(), n_tiles
        _cabi.check(self.lib.kda_segment_launch(C.byref(s), self._stream(dev)), "kda_segment_launch")
        self._keep = (t0, t1, nm, ws, status)       # alive until the stream has consumed them
        return out, qt, P, S_loc

    def rows_of(self, out, qt, bounds, need_map):
        """(o_loc rows, Qt rows) [1,T,H,128] of the most recent `segment_maps` call, whichever form it wrote (tests)."""
        if not self._tiled[0]:
            return out, qt
        T, H = out.shape[1], out.shape[2]
        o_rows, q_rows = out.clone(), torch.zeros_like(out)
        tile = 0
        for i in range(len(bounds) - 1):
            t0, t1 = bounds[i], bounds[i + 1]
            nt = -(-(t1 - t0) // CHUNK)
            if need_map[i] and nt:
                for dst, src in ((q_rows, qt[0]), (o_rows, qt[1])):
                    rows = src[tile:tile + nt].permute(0, 3, 1, 2).reshape(nt * CHUNK, H, D)     # [tile][tok][h][v] -> rows
                    dst[0, t0:t1] = rows[:t1 - t0]
            tile += nt
        return o_rows, q_rows

    def scan(self, P, S_loc, S0):
        """S_in[0] = S0 (or 0), S_in[i+1] = S_in[i] @ P[i] + S_loc[i]; returns (S_in [n,H,128,128], S_end [H,128,128])."""
        n, H = P.shape[0], P.shape[1]
        S_in = self._buf(("S_in", P.data_ptr()), tuple(S_loc.shape), torch.float32, P.device)
        S_end = self._buf(("S_end", P.data_ptr()), (H, D, D), torch.float32, P.device)
        s0 = None if S0 is None else S0.data_ptr()
        if n > 1 and P.stride(0) != H * D * D:
            # maps that lie apart (the two halves of one gathered [rank][2][H][128][128] buffer)
            assert P.stride(0) == S_loc.stride(0) and P[0].is_contiguous() and S_loc[0].is_contiguous()
            _cabi.check(self.lib.kda_scan_strided_launch(P.data_ptr(), S_loc.data_ptr(), s0, S_in.data_ptr(), S_end.data_ptr(), n, H,
                                                         P.stride(0), self._stream(P.device)), "kda_scan_strided_launch")
        else:
            _cabi.check(self.lib.kda_scan_launch(P.data_ptr(), S_loc.data_ptr(), s0, S_in.data_ptr(), S_end.data_ptr(), n, H,
                                                 self._stream(P.device)), "kda_scan_launch")
        return S_in, S_end

    def fixup(self, out, qt, S_in, bounds, need_map):
        dev = out.device
        n, H = len(bounds) - 1, out.shape[2]
        t0, t1, nm = self._tables(bounds, need_map, dev)
        tiled, n_tiles, T = getattr(self, "_tiled", (False, 0, 0))
        if tiled:
            _cabi.check(self.lib.kda_fixup_tiles_launch(out.data_ptr(), qt.data_ptr(), n_tiles, H * D, S_in.data_ptr(), t0.data_ptr(),
                                                        t1.data_ptr(), nm.data_ptr(), n, H, T, self._stream(dev)), "kda_fixup_tiles_launch")
        else:
            _cabi.check(self.lib.kda_fixup_launch(out.data_ptr(), qt.data_ptr(), H * D, S_in.data_ptr(), t0.data_ptr(), t1.data_ptr(),
                                                  nm.data_ptr(), n, H, self._stream(dev)), "kda_fixup_launch")
        self._keep2 = (t0, t1, nm)
        return out


def plan_cut(T, H, every, n_sms=148, max_pieces=24, task_overhead=3.0):
    """Number of equal pieces (aligned to the checkpoint interval) for `prepare_cut_sequence`, or 1 when cutting does
    not pay.  Cost of p pieces in chunk steps: pass 1 runs the plain chain on piece 0 and both chains on pieces
    1..p-2 (the last piece's map is not needed), pass 2 runs every piece once from its true entering state."""
    align = max(CHUNK, int(every or CHUNK))
    nch = -(-T // CHUNK)
    best_p, best = 1, _makespan([nch + task_overhead] * H, n_sms)
    for p in range(2, max_pieces + 1):
        L = -(-(-(-T // p)) // align) * align
        pe = -(-T // L)
        if pe < 2:
            continue
        c = L // CHUNK + task_overhead
        cost = _makespan([c] * (H * (1 + 2 * max(0, pe - 2))), n_sms) + _makespan([c] * (H * pe), n_sms)
        if cost < best * 0.9:
            best_p, best = pe, cost
    return best_p


def prepare_cut_sequence(q, k, v, g, beta, A_log, dt_bias, scale, pool, slot, *, state_checkpoints=None, checkpoint_row0=0,
                         checkpoint_every_n_tokens=0, pieces=0):
    """Serving prefill of ONE long sequence on few heads, cut into pieces so that all SMs work, WITH checkpoint rows.

    q, k, v, g [1, T, H, 128] bf16 and beta [1, T, H] bf16 (the reference front-end), pool [P, H, 128, 128] fp32
    value-first updated in place at `slot`; `state_checkpoints` [C, H, 128, 128] (fp32 or bf16) receives the state
    before every `checkpoint_every_n_tokens`-th token in rows `checkpoint_row0 ...`, exactly as the ordinary call.

    Two passes, because checkpoint rows need true states: pass 1 gets every piece's entering state from the affine
    maps (plain chain on piece 0, chains L and Tr on the middle pieces, nothing on the last) and one scan; pass 2 is the
    ordinary serving launch over the pieces as if they were sequences, each starting from its entering state through
    the source-pool arguments, emitting outputs and checkpoint rows.  Three piece-chains of work instead of one, on up
    to 148 SMs instead of H (the reference cuts long requests inside its planner, kda/b200/csrc/w3/base/kernel.py:362-593).
    Returns launch() -> (out [1, T, H, 128] bf16, pool, state_checkpoints); everything is allocated here, the launch
    only enqueues kernels and device copies on the current stream (no host synchronisation)."""
    import kda_b200
    dev = q.device
    T, H = q.shape[1], q.shape[2]
    every = int(checkpoint_every_n_tokens or 0)
    lib = _cabi.lib()
    p = pieces if pieces > 0 else plan_cut(T, H, every)
    align = max(CHUNK, every or CHUNK)
    L = -(-(-(-T // max(p, 1))) // align) * align
    p = -(-T // L)
    ck_kw = {}
    if every:
        ck_kw = dict(state_checkpoints=state_checkpoints, checkpoint_every_n_tokens=every)
    if p < 2:
        starts = torch.tensor([checkpoint_row0, checkpoint_row0 + -(-T // every)], dtype=torch.int64, device=dev) if every else None
        return kda_b200.prepare(q, k, v, g, beta, A_log, dt_bias, scale, pool, None, dynamic_layout=True,
                                ssm_state_indices=torch.tensor([slot], dtype=torch.int32, device=dev),
                                **(dict(ck_kw, checkpoint_cu_starts=starts) if every else {}))
    bounds = [min(T, i * L) for i in range(p + 1)]
    n1 = p - 1                                   # pieces whose end state pass 1 has to deliver
    T1 = bounds[n1]
    # ---- pass 1: maps of pieces 0 .. p-2
    P = torch.zeros(n1, H, D, D, dtype=torch.float32, device=dev)
    S_loc = torch.empty(n1, H, D, D, dtype=torch.float32, device=dev)
    t0 = torch.tensor(bounds[:n1], dtype=torch.int64, device=dev)
    t1 = torch.tensor(bounds[1:n1 + 1], dtype=torch.int64, device=dev)
    nm = torch.tensor([0] + [1] * (n1 - 1), dtype=torch.int32, device=dev)
    ws_bytes = lib.kda_prefill_workspace_bytes(2 * n1, H)
    ws = torch.zeros(ws_bytes + 256, dtype=torch.uint8, device=dev)
    status1 = torch.zeros(4, dtype=torch.int32, device=dev)
    first = pool[slot:slot + 1]
    seg = _cabi.KdaSegmentArgs()
    a = seg.base
    a.q, a.k, a.v, a.g, a.beta = q.data_ptr(), k.data_ptr(), v.data_ptr(), g.data_ptr(), beta.data_ptr()
    a.out = None                                 # maps only: pass 1 writes no output rows
    a.ldq, a.ldk, a.ldv, a.ldg = (t.stride(1) for t in (q, k, v, g))
    a.ldbeta, a.ldo = beta.stride(1), H * D
    a.A_log, a.dt_bias = A_log.data_ptr(), dt_bias.data_ptr()
    a.scale, a.lower_bound = float(scale), -5.0
    a.frontend, a.state_layout = _cabi.FRONTEND_RAW, _cabi.STATE_VALUE_FIRST
    a.H, a.N, a.T = H, n1, T1
    a.src_base, a.src_slot_stride, a.src_slots = first.data_ptr(), first.stride(0), 1
    a.workspace, a.workspace_bytes = (ws.data_ptr() + 255) // 256 * 256, ws_bytes
    a.status = status1.data_ptr()
    a.kernel = kda_b200.default_kernel()
    seg.n_seg = n1
    seg.seg_t0, seg.seg_t1, seg.seg_need_map = t0.data_ptr(), t1.data_ptr(), nm.data_ptr()
    seg.qt, seg.P, seg.S_loc = None, P.data_ptr(), S_loc.data_ptr()
    # ---- scan: entering states of all p pieces, laid out as the source pool of pass 2
    src = torch.empty(p, H, D, D, dtype=torch.float32, device=dev)
    # ---- pass 2: the ordinary serving launch over the pieces
    dstpool = torch.empty(p, H, D, D, dtype=torch.float32, device=dev)
    ids = torch.arange(p, dtype=torch.int32, device=dev)
    cu2 = torch.tensor(bounds, dtype=torch.int64, device=dev)
    kw = dict(dynamic_layout=True, ssm_state_indices=ids, initial_state_source=src, initial_state_indices=ids)
    if every:
        rows = [0]
        for i in range(p):
            rows.append(rows[-1] + -(-(bounds[i + 1] - bounds[i]) // every))
        kw.update(state_checkpoints=state_checkpoints, checkpoint_every_n_tokens=every,
                  checkpoint_cu_starts=torch.tensor([checkpoint_row0 + r for r in rows], dtype=torch.int64, device=dev))
    launch2 = kda_b200.prepare(q, k, v, g, beta, A_log, dt_bias, scale, dstpool, cu2, **kw)
    keep = (P, S_loc, t0, t1, nm, ws, status1, first, src, dstpool, ids, cu2)

    def launch():
        stream = C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
        _cabi.check(lib.kda_segment_launch(C.byref(seg), stream), "kda_segment_launch")
        _cabi.check(lib.kda_scan_launch(P.data_ptr(), S_loc.data_ptr(), first.data_ptr(), src.data_ptr(),
                                        src[n1].data_ptr(), n1, H, stream), "kda_scan_launch")
        res = launch2()
        pool[slot].copy_(dstpool[p - 1])
        return (res[0], pool, state_checkpoints) if every else (res[0], pool)

    launch.keepalive = keep
    launch.pieces = p
    launch.status = launch2.status
    launch.status_pass1 = status1
    return launch


def compose_rank_map(backend, P, S_loc, first_is_zero=False):
    """Total map of a rank's pieces per head: P_rank = P_0 @ P_1 @ ..., L_rank = (..(S_loc_0 @ P_1 + S_loc_1) @ P_2 ..).
    `first_is_zero`: P_0 is the zero map (a plain first piece, which starts from a known state), so is the product."""
    n = P.shape[0]
    _, L_rank = backend.scan(P, S_loc, None)
    if n == 1 or first_is_zero:
        return P[0], L_rank
    zeros = backend._buf("zeros", tuple(S_loc[1:].shape), torch.float32, P.device, zero=True) if hasattr(backend, "_buf") \
        else torch.zeros_like(S_loc[1:])
    _, P_rank = backend.scan(P[1:], zeros, P[0])
    return P_rank, L_rank


def context_parallel_prefill(q, k, v, g, beta, A_log, dt_bias, scale, initial_state=None, *, group=None, pieces=0,
                             raw=True, backend=None, events=None):
    """Context-parallel prefill of ONE sequence whose tokens are sharded over the ranks of `group` in rank order.

    q, k, v, g [1, T_local, H, 128] and beta [1, T_local, H] are this rank's shard (contiguous token rows);
    initial_state [1, H, 128, 128] fp32 value-first is read on rank 0 (zeros when None).  With `group=None` (or a
    single rank) this is intra-GPU context parallelism: the pieces only serve to fill the SMs.  `pieces=0` plans the
    piece boundaries by simulating the segment launch (`plan_bounds`); `pieces=n` cuts n equal pieces.
    `events`, when a list, receives (phase name, CUDA event) pairs recorded on the current stream at the phase
    boundaries ("start", "segments", "maps", "exchange", "scan", "fixup"), for callers that time the phases.
    Returns (out [1, T_local, H, 128] bf16 for the local tokens, final_state [1, H, 128, 128] fp32 on every rank).
    Nothing here synchronises; `backend.kernel_error()` afterwards tells whether a bounded wait inside the segment
    kernel gave up (the maps, and with them every rank's result, are then invalid).  With `CudaBackend(reuse=True)`
    repeated calls over one layout allocate nothing after the first."""
    import torch.distributed as dist

    def mark(name):
        if events is not None:
            e = torch.cuda.Event(enable_timing=True)
            e.record()
            events.append((name, e))

    world = dist.get_world_size(group) if (group is not None or (dist.is_available() and dist.is_initialized())) else 1
    rank = dist.get_rank(group) if world > 1 else 0
    backend = backend or CudaBackend()
    T, H = q.shape[1], q.shape[2]
    bounds = plan_bounds(T, H, rank == 0) if pieces <= 0 else split_pieces(T, pieces)
    n = len(bounds) - 1
    need_map = [1] * n
    first = None
    if rank == 0:
        need_map[0] = 0            # the first piece of the sequence starts from the caller's state: plain chain
        first = initial_state if initial_state is not None else torch.zeros(1, H, D, D, dtype=torch.float32, device=q.device)
    mark("start")
    out, qt, P, S_loc = backend.segment_maps(q, k, v, g, beta, A_log, dt_bias, scale, raw, bounds, need_map, first)
    mark("segments")
    # P of an unmapped piece is the zero map (its S_loc is the true end state): segment_maps leaves it zero-filled
    if world == 1:
        # one rank: a single scan yields both the entering states of the pieces and the final state
        mark("maps")
        mark("exchange")
        S_in, S_final = backend.scan(P, S_loc, None)
        mark("scan")
        out = backend.fixup(out, qt, S_in, bounds, need_map)
        mark("fixup")
        return out, S_final[None]
    P_rank, L_rank = compose_rank_map(backend, P, S_loc, first_is_zero=not need_map[0])
    mark("maps")
    if world > 1:
        # ONE gather of the (P, S_loc) pair of every rank; the scan reads the two halves of the gathered buffer in place
        mk = backend._buf if hasattr(backend, "_buf") else (lambda key, shape, dt, dev, zero=False: torch.empty(shape, dtype=dt, device=dev))
        pair = mk("pair", (2, H, D, D), P_rank.dtype, P_rank.device)
        pair[0].copy_(P_rank)
        pair[1].copy_(L_rank)
        gathered = mk("gather", (world, 2, H, D, D), P_rank.dtype, P_rank.device)
        dist.all_gather_into_tensor(gathered.view(world * 2 * H, D, D), pair.view(2 * H, D, D), group=group)
        S_in_ranks, S_final = backend.scan(gathered[:, 0], gathered[:, 1], None)
        S_enter = S_in_ranks[rank]
    else:
        S_enter = None
        S_final = L_rank
    mark("exchange")
    S_in, _ = backend.scan(P, S_loc, S_enter)
    mark("scan")
    out = backend.fixup(out, qt, S_in, bounds, need_map)
    mark("fixup")
    return out, S_final[None]
