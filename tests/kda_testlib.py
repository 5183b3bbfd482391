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
