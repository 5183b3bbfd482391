"""Helpers shared by the GPU parity tests: seeded inputs, gold results from the CPU oracle, comparison."""
import random

import numpy as np
import torch

import c_oracle
import kda_oracle as ko

D = 128
DEV = "cuda:0"


def cu_of(lens, device=DEV):
    return torch.tensor([0, *np.cumsum(lens).tolist()], dtype=torch.int64, device=device)


def ck_meta(lens, every, device=DEV):
    counts = [-(-n // every) for n in lens]
    return torch.tensor([0, *np.cumsum(counts).tolist()], dtype=torch.int64, device=device), sum(counts)


def slow_gates_(inputs, seed):
    """Slow decay (long memory) as kda/b200/test_kda_b200.py:58-62: A_log = 0, dt_bias uniform in [-12, -6]."""
    gen = torch.Generator().manual_seed(seed)
    H = inputs[5].numel()
    inputs[5].fill_(0.0)
    inputs[6].copy_(torch.rand(H * D, generator=gen) * 6.0 - 12.0)


def gold_raw(inputs, lens, init=None, every=0):
    """fp64 recurrence on the CPU (C oracle), with checkpoint rows chained over segments when every > 0."""
    q, k, v, g, beta, A_log, dt_bias, scale = inputs[:8]
    init = inputs[8] if init is None else init
    if not every:
        o, f = c_oracle.recurrence_raw(q, k, v, g, beta, A_log, dt_bias, scale, init, [0, *np.cumsum(lens).tolist()])
        return o, f, None
    # chain over checkpoint segments: each segment is its own "sequence" starting from the previous end state
    outs, finals, rows, t0 = [], [], [], 0
    for n, L in enumerate(lens):
        S = init[n:n + 1].clone()
        for s in range(0, L, every):
            e = min(L, s + every)
            rows.append(S[0].clone())
            sl = slice(t0 + s, t0 + e)
            o, S = c_oracle.recurrence_raw(q[:, sl], k[:, sl], v[:, sl], g[:, sl], beta[:, sl], A_log, dt_bias, scale, S,
                                           [0, e - s])
            outs.append(o)
        finals.append(S[0])
        t0 += L
    return torch.cat(outs, 1), torch.stack(finals), (torch.stack(rows) if rows else None)


def to_dev(inputs, device=DEV):
    return [t.to(device) if torch.is_tensor(t) else t for t in inputs]


def partition(rng: random.Random, T, N):
    cuts = sorted(rng.sample(range(1, T), N - 1))
    return [b - a for a, b in zip([0, *cuts], [*cuts, T])]


def plain_on_device(H, T, seed, g_mean=0.0, device=DEV):
    """Pre-activated inputs of the benchmark configurations, drawn on the device: q, k ~ N(0,1) L2-normalised per head
    then bf16, v ~ N(0,1) bf16, g = logsigmoid(N(g_mean, 1)) fp32, beta = sigmoid(N(0,1)) fp32."""
    gen = torch.Generator(device=device).manual_seed(seed)
    q = torch.nn.functional.normalize(torch.randn(1, T, H, D, generator=gen, device=device), dim=-1).to(torch.bfloat16)
    k = torch.nn.functional.normalize(torch.randn(1, T, H, D, generator=gen, device=device), dim=-1).to(torch.bfloat16)
    v = torch.randn(1, T, H, D, generator=gen, device=device).to(torch.bfloat16)
    g = torch.nn.functional.logsigmoid(torch.randn(1, T, H, D, generator=gen, device=device) + g_mean)
    beta = torch.sigmoid(torch.randn(1, T, H, generator=gen, device=device))
    return q, k, v, g, beta


def gold_plain(q, k, v, g, beta, scale, init, lens, every=0):
    """fp64 recurrence of the pre-activated call on the CPU (C oracle; state key-first), with checkpoint rows chained
    over segments when every > 0: returns (out, final states, rows or None)."""
    if not every:
        o, f = c_oracle.recurrence_plain(q, k, v, g, beta, scale, init, [0, *np.cumsum(lens).tolist()])
        return o, f, None
    # one oracle call per checkpoint interval "wave": segment j of every sequence that still has one
    outs = torch.zeros(q.shape, dtype=torch.float32)
    S = init.clone()
    rows = [[] for _ in lens]
    starts = [0, *np.cumsum(lens).tolist()]
    for j in range(-(-max(lens) // every)):
        segs = [(n, starts[n] + j * every, starts[n] + min(lens[n], (j + 1) * every)) for n in range(len(lens)) if j * every < lens[n]]
        for n, _, _ in segs:
            rows[n].append(S[n].clone())
        tok = torch.cat([torch.arange(a, b) for _, a, b in segs])
        cu = [0, *np.cumsum([b - a for _, a, b in segs]).tolist()]
        ids = [n for n, _, _ in segs]
        o, f = c_oracle.recurrence_plain(q[:, tok], k[:, tok], v[:, tok], g[:, tok], beta[:, tok], scale, S[ids], cu)
        outs[:, tok] = o
        S[ids] = f
    return outs, S, torch.stack([r for rs in rows for r in rs])
