"""CPU oracle for KDA prefill.  TEST INFRASTRUCTURE ONLY: nothing in the product path imports this module.

It restates, in plain torch on the CPU, the operator definition that the CUDA path must reproduce:

* `kda_recurrence`       the raw-gate front-end, token by token, following kda/b200/reference.py:17-38 of the
                         reference (L2-normalised q/k with eps 1e-6, lines 21-22; gate line 24; sigmoid beta line 26;
                         decay-then-update order lines 33-35; output from the UPDATED state line 36; value-first
                         state, transposed on the way in and out, lines 31 and 37).
* `kda_recurrence_plain` the pre-activated front-end (`chunk_kda`-style call): the same loop
                         (reference.py:30-37) with lines 21-26 replaced by the identity, state kept key-first.
* `kda_checkpoints`      checkpoint rows (state before token j*n) obtained by chaining the recurrence over
                         checkpoint segments, as kda/b200/test_kda_b200.py:38-55 does.
* `segment_map`          the affine state map of a token segment (kda/b200/csrc/w3/kernel.py:22-38 and
                         kda/b200/csrc/w3/cp_fix.cu:4-21): S_end = S_in @ P + S_loc, o = o_loc + S_in applied to Qt.
* `close` / `check_close` the acceptance criterion of kda/b200/test_kda_b200.py:28-35.

Parity is pinned: tests/golden/*.npz hold outputs of the reference's own reference.py on seeded inputs (written by
tests/golden/make_golden.py, which imports the reference), and tests/test_oracle.py checks this module against them.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

D = 128
REL_L2_MAX = 1e-2      # kda/b200/test_kda_b200.py:24
ELEM_RMS_FRAC = 0.5    # kda/b200/test_kda_b200.py:31
ELEM_REL_FRAC = 0.05   # kda/b200/test_kda_b200.py:31


# ----------------------------------------------------------------------------------------------- activation
def activate_raw(q, k, g, beta, A_log, dt_bias, lower_bound=-5.0, dtype=torch.float64):
    """Raw-gate front-end (reference.py:21-26): returns q_hat, k_hat [T,H,D], log-decay a [T,H,D] (<= 0), beta [T,H]."""
    H = q.shape[-2]
    qn = F.normalize(q.reshape(-1, H, D).to(dtype), dim=-1, eps=1e-6)
    kn = F.normalize(k.reshape(-1, H, D).to(dtype), dim=-1, eps=1e-6)
    a = lower_bound * torch.sigmoid(A_log.to(dtype).exp().view(H, 1)
                                    * (g.reshape(-1, H, D).to(dtype) + dt_bias.to(dtype).view(H, D)))
    b = torch.sigmoid(beta.reshape(-1, H).to(dtype))
    return qn, kn, a, b


def _cu_list(cu_seqlens, T):
    if cu_seqlens is None:
        return [0, T]
    return [int(c) for c in (cu_seqlens.tolist() if torch.is_tensor(cu_seqlens) else cu_seqlens)]


def _recur(qn, kn, vf, a, b, scale, S0_kv, cu):
    """Token loop shared by both front-ends.  S0_kv: [N,H,K,V] key-first.  Returns out [T,H,V], final [N,H,K,V]."""
    dtype = qn.dtype
    T, H, _ = qn.shape
    decay = a.exp()
    out = torch.zeros(T, H, D, dtype=dtype)
    final = torch.empty(len(cu) - 1, H, D, D, dtype=dtype)
    for n in range(len(cu) - 1):
        S = S0_kv[n].to(dtype).clone()
        for t in range(cu[n], cu[n + 1]):
            S = S * decay[t][:, :, None]                                    # reference.py:33
            kS = torch.einsum("hk,hkv->hv", kn[t], S)                       # reference.py:34
            S = S + kn[t][:, :, None] * (b[t][:, None] * (vf[t] - kS))[:, None, :]   # reference.py:35
            out[t] = scale * torch.einsum("hk,hkv->hv", qn[t], S)           # reference.py:36
        final[n] = S
    return out, final


@torch.no_grad()
def kda_recurrence(q, k, v, g, beta, A_log, dt_bias, scale, initial_state, cu_seqlens, lower_bound=-5.0,
                   dtype=torch.float64):
    """Raw front-end, value-first state.  Shapes as kda/b200/reference.py:3-6.
    Returns (out [1,T,H,128] bf16, final_state [N,H,128(V),128(K)] fp32)."""
    T, H = q.shape[1], q.shape[2]
    qn, kn, a, b = activate_raw(q[0], k[0], g[0], beta[0], A_log, dt_bias, lower_bound, dtype)
    cu = _cu_list(cu_seqlens, T)
    out, fin = _recur(qn, kn, v[0].to(dtype), a, b, scale, initial_state.to(dtype).transpose(-1, -2), cu)
    return out[None].to(torch.bfloat16), fin.transpose(-1, -2).float().contiguous()


@torch.no_grad()
def kda_recurrence_plain(q, k, v, g, beta, scale=None, initial_state=None, cu_seqlens=None, dtype=torch.float64):
    """Pre-activated front-end: q, k already L2-normalised, g the log-decay (<= 0) per channel, beta in (0, 1);
    state key-first [N,H,K,V].  Returns (out [1,T,H,V] in `dtype`, final_state [N,H,K,V] fp32)."""
    T, H = q.shape[1], q.shape[2]
    if scale is None:
        scale = D ** -0.5
    cu = _cu_list(cu_seqlens, T)
    N = len(cu) - 1
    S0 = torch.zeros(N, H, D, D, dtype=dtype) if initial_state is None else initial_state.to(dtype)
    out, fin = _recur(q[0].to(dtype), k[0].to(dtype), v[0].to(dtype), g[0].to(dtype), beta[0].to(dtype), scale, S0, cu)
    return out[None], fin.float()


@torch.no_grad()
def kda_checkpoints(q, k, v, g, beta, A_log, dt_bias, scale, init, lens, every=0, lower_bound=-5.0,
                    dtype=torch.float64):
    """Raw front-end over sequences `lens` with checkpoint rows every `every` tokens (0 = none):
    row (sequence n, j) = state before token j*every, j = 0 .. ceil(len/every)-1; there is no row for the final state
    (kda/b200/kda_b200.py:19-22, kda/b200/test_kda_b200.py:38-55).  Returns out, finals [N,H,V,K], rows or None."""
    outs, finals, rows, t0 = [], [], [], 0
    H = q.shape[2]
    for n, L in enumerate(lens):
        S = init[n:n + 1].clone()
        seg = every if every else max(L, 1)
        for s in range(0, L, seg):
            e = min(L, s + seg)
            if every:
                rows.append(S[0].clone())
            sl = slice(t0 + s, t0 + e)
            o, S = kda_recurrence(q[:, sl], k[:, sl], v[:, sl], g[:, sl], beta[:, sl], A_log, dt_bias, scale, S,
                                  [0, e - s], lower_bound, dtype)
            outs.append(o)
        finals.append(S[0])
        t0 += L
    out = torch.cat(outs, 1) if outs else torch.zeros(1, 0, H, D, dtype=torch.bfloat16)
    return out, torch.stack(finals), (torch.stack(rows) if (every and rows) else None)


@torch.no_grad()
def segment_map(qn, kn, a, b, scale, dtype=torch.float64):
    """Affine map of one token segment, value-first orientation (kda/b200/csrc/w3/cp_fix.cu:8-10):
    St_end = St_in @ P + St_loc and o_t = o_loc_t + St_in @ Qt_t, hence the two chains of the reference's dual kernel:
    chain Tr (v = 0, S0 = I) gives P [H,K,K] and Qt [T,H,K]; chain L (S0 = 0) is the ordinary recurrence.
    Inputs are activated ([T,H,D], [T,H]).  Returns P [H,K',K], Qt [T,H,K']."""
    T, H, _ = qn.shape
    eye = torch.eye(D, dtype=dtype).expand(1, H, D, D)      # key-first [K, V=K']: row k, "value" column k'
    zero_v = torch.zeros(T, H, D, dtype=dtype)
    Qt, fin = _recur(qn.to(dtype), kn.to(dtype), zero_v, a.to(dtype), b.to(dtype), scale, eye, [0, T])
    # fin[0] is key-first [K, K']; value-first P[k', k] = fin[k, k']
    return fin[0].transpose(-1, -2).contiguous(), Qt


def compose_maps(P1, L1, P2, L2):
    """(P2,L2) after (P1,L1), value-first: S -> (S @ P1 + L1) @ P2 + L2."""
    return P1 @ P2, L1 @ P2 + L2


# ----------------------------------------------------------------------------------------------- acceptance
def close_stats(got, gold):
    """(worst element ratio, relative L2, finite) under the criterion of kda/b200/test_kda_b200.py:28-35: an element
    passes when its error is within half the RMS of the gold tensor OR within 5 % of the gold element's magnitude."""
    x, y = got.detach().double().cpu(), gold.detach().double().cpu()
    if y.numel() == 0:
        return 0.0, 0.0, True
    err = (x - y).abs()
    rms = y.pow(2).mean().sqrt()
    ratio = torch.minimum(err / (ELEM_RMS_FRAC * rms), err / (ELEM_REL_FRAC * y.abs() + 1e-30))
    worst = float(torch.nan_to_num(ratio, nan=float("inf")).max())
    l2 = float(torch.linalg.vector_norm(x - y) / torch.linalg.vector_norm(y).clamp_min(1e-30))
    return worst, l2, bool(torch.isfinite(x).all())


def check_close(got, gold, what, rel_l2_max=REL_L2_MAX):
    worst, l2, finite = close_stats(got, gold)
    assert finite, f"{what}: non-finite values"
    assert worst <= 1.0 and l2 < rel_l2_max, f"{what}: worst element ratio {worst:.2f}, relative L2 {l2:.2e}"
    return worst, l2


# ----------------------------------------------------------------------------------------------- seeded inputs
def make_inputs_raw(H, lens, seed, device="cpu"):
    """Inputs with the distributions of the reference's generator (kda/b200/bench.py:66-83): bf16 N(0, 0.5) q/k/v/g and
    beta logits, A_log = log U(1,16), dt_bias from dt log-uniform in [1e-3, 1e-1], fp32 N(0, 0.25) initial states.
    Drawn on the CPU generator (the reference draws on CUDA; only the distributions are reproduced)."""
    gen = torch.Generator().manual_seed(seed)
    T = sum(lens)

    def randn(shape, s, dt=torch.bfloat16):
        return (torch.randn(shape, generator=gen) * s).to(dt)

    A_log = torch.log(torch.empty(H).uniform_(1.0, 16.0, generator=gen))
    dt = torch.exp(torch.rand(H * D, generator=gen) * (math.log(0.1) - math.log(0.001)) + math.log(0.001)).clamp_(min=1e-4)
    dt_bias = dt + torch.log(-torch.expm1(-dt))
    q, k, v, g = (randn((1, T, H, D), 0.5) for _ in range(4))
    beta = randn((1, T, H), 0.5)
    init = randn((len(lens), H, D, D), 0.25, torch.float32)
    cu = torch.tensor([0, *torch.tensor(lens).cumsum(0).tolist()], dtype=torch.int64)
    res = [q, k, v, g, beta, A_log, dt_bias, 1.0 / math.sqrt(D), init, cu]
    return [t.to(device) if torch.is_tensor(t) else t for t in res]


def make_inputs_plain(H, lens, seed, qkv_dtype=torch.bfloat16, g_mean=0.0, init_std=0.05, device="cpu"):
    """Pre-activated inputs as the benchmark configurations describe them: q, k ~ N(0,1) L2-normalised per head (then
    cast), v ~ N(0,1), g = logsigmoid(N(g_mean,1)) fp32, beta = sigmoid(N(0,1)) fp32, initial state N(0, init_std)
    key-first [N,H,K,V] (zeros when init_std == 0)."""
    gen = torch.Generator().manual_seed(seed)
    T = sum(lens)
    q = F.normalize(torch.randn(1, T, H, D, generator=gen), dim=-1).to(qkv_dtype)
    k = F.normalize(torch.randn(1, T, H, D, generator=gen), dim=-1).to(qkv_dtype)
    v = torch.randn(1, T, H, D, generator=gen).to(qkv_dtype)
    g = F.logsigmoid(torch.randn(1, T, H, D, generator=gen) + g_mean)
    beta = torch.sigmoid(torch.randn(1, T, H, generator=gen))
    init = torch.randn(len(lens), H, D, D, generator=gen) * init_std
    cu = torch.tensor([0, *torch.tensor(lens).cumsum(0).tolist()], dtype=torch.int64)
    res = [q, k, v, g, beta, D ** -0.5, init, cu]
    return [t.to(device) if torch.is_tensor(t) else t for t in res]
