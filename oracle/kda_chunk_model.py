"""Chunked CPU model of the CUDA kernel's arithmetic (test infrastructure; never imported by the product path).

Follows the chunked form of the recurrence (derived from kda/b200/reference.py:30-37; the same algebra the reference
states in kda/b200/csrc/w3/base/tiny/kda_tiny.cu:5-11) with the roundings of the GPU path: 32-token chunks, one
reference exponent per chunk half (the cumulative log-decay after token 15), bf16 MMA operands, fp32 accumulation,
fp32 state.  Used to check the algorithm and its tolerance on the CPU and to localise GPU mismatches stage by stage.
"""
from __future__ import annotations

import torch

C = 32
HALF = 16
D = 128


def bf(x):
    return x.to(torch.bfloat16).to(torch.float32)


@torch.no_grad()
def chunk_forward(qn, kn, v, a, b, scale, St0, want_stages=False, v_zero=False):
    """One (sequence, head).  qn, kn, v, a: [L, D] fp32 (activated), b: [L]; St0 value-first [V, K] fp32.
    Returns out [L, V] (bf16-rounded fp32), final St [V, K] fp32 and, optionally, per-chunk stage tensors."""
    L = qn.shape[0]
    St = St0.clone().float()
    out = torch.zeros(L, D)
    stages = []
    for c0 in range(0, L, C):
        n = min(C, L - c0)
        pad = lambda x: torch.cat([x[c0:c0 + n].float(), torch.zeros(C - n, *x.shape[1:])])  # noqa: E731
        q_, k_, v_, a_, b_ = pad(qn), pad(kn), pad(v), pad(a), pad(b)
        if v_zero:
            v_ = torch.zeros_like(v_)
        G = torch.cumsum(a_, 0)
        r, last = G[HALF - 1], G[C - 1]
        E, Ei = torch.exp(G - r), torch.exp(r - G)
        kd_s, qd_s, ki_s = bf(k_ * E), bf(scale * q_ * E), bf(k_ * Ei)
        er, elr = torch.exp(r), torch.exp(last - r)
        kd_t, qd_t, kr = bf(k_ * E * er), bf(scale * q_ * E * er), bf(k_ * Ei * elr)
        A = torch.tril(kd_s @ ki_s.T, -1) * b_[:, None]
        M = torch.tril(qd_s @ ki_s.T, 0)
        T = torch.zeros(C, C)
        for i in range(C):                       # forward substitution, row by row, fp32
            T[i] = -(A[i, :i] @ T[:i]) if i else 0
            T[i, i] = 1.0
        Tb, Mb = bf(T * b_[None, :]), bf(M)
        Sb = bf(St)
        Wt = Sb @ kd_t.T
        Ot = Sb @ qd_t.T
        Rt = bf(bf(v_).T - Wt)
        U2 = bf(Rt @ Tb.T)
        Ot = Ot + U2 @ Mb.T
        St = St * torch.exp(last)[None, :] + U2 @ kr
        out[c0:c0 + n] = bf(Ot.T)[:n]
        if want_stages:
            stages.append(dict(G=G, kd_t=kd_t, qd_t=qd_t, kr=kr, A=A, M=M, T=T, Wt=Wt, U2=U2, St=St.clone()))
    return (out, St, stages) if want_stages else (out, St)


@torch.no_grad()
def forward(qn, kn, v, a, b, scale, St0, cu):
    """All (sequence, head) pairs.  qn.. [T,H,D], b [T,H]; St0 [N,H,V,K].  Returns out [T,H,V], final [N,H,V,K]."""
    T, H, _ = qn.shape
    out = torch.zeros(T, H, D)
    fin = torch.zeros(len(cu) - 1, H, D, D)
    for n in range(len(cu) - 1):
        s, e = cu[n], cu[n + 1]
        for h in range(H):
            o, S = chunk_forward(qn[s:e, h], kn[s:e, h], v[s:e, h], a[s:e, h], b[s:e, h], scale, St0[n, h])
            out[s:e, h], fin[n, h] = o, S
    return out, fin
