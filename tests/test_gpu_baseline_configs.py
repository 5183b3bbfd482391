"""GPU parity at the FULL sizes of the benchmark configurations (configs[1]..configs[4]): the CUDA path runs the whole
shape, the fp64 C oracle checks a subset of heads (heads are independent, so a head slice of the inputs is a complete
problem for the oracle).  Tolerance as everywhere (kda/b200/test_kda_b200.py:28-35): every element within half the gold
tensor's RMS or 5 % of its own magnitude, relative L2 < 1e-2; untouched pool slots bit for bit.  Inputs are seeded
synthetic draws with the configurations' distributions, generated on the device."""
import math
import random

import numpy as np
import pytest
import torch

import c_oracle
import kda_oracle as ko
from kda_testlib import DEV, D, ck_meta, cu_of, plain_on_device, gold_plain

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def kda():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    import kda_b200
    return kda_b200


def _heads_cpu(tensors, heads):
    """Head subset of [1,T,H,...] / [N,H,...] device tensors, on the CPU."""
    return [t[:, :, heads].cpu() if t.dim() >= 3 and t.shape[0] == 1 else t[:, heads].cpu() for t in tensors]


def test_config1_varlen_plain_call_full_size(kda):
    """configs[1]: 16 sequences, lengths uniform in [128, 4096], H = 32, bf16 q/k/v, fp32 g/beta, N(0, 0.05) initial
    states, final state requested."""
    H, heads = 32, [0, 13, 31]
    rng = random.Random(1)
    lens = [rng.randint(128, 4096) for _ in range(16)]
    q, k, v, g, beta = plain_on_device(H, sum(lens), 101)
    init = torch.randn(len(lens), H, D, D, generator=torch.Generator(device=DEV).manual_seed(102), device=DEV) * 0.05
    cu = cu_of(lens)
    o, fin = kda.chunk_kda(q, k, v, g, beta, D ** -0.5, init, True, cu)
    torch.cuda.synchronize()
    qs, ks, vs, gs, bs = _heads_cpu([q, k, v, g, beta], heads)
    gold_o, gold_s = c_oracle.recurrence_plain(qs, ks, vs, gs, bs, D ** -0.5, init[:, heads].cpu(), cu.cpu())
    ko.check_close(o[:, :, heads].cpu(), gold_o, "configs[1] output")
    ko.check_close(fin[:, heads].cpu(), gold_s, "configs[1] final state")


def test_config2_serving_call_full_size(kda):
    """configs[2]: H = 64, 48 requests on random distinct slots of a 256-slot fp32 pool ~ N(0, 0.05), lengths
    lognormal(ln 1024, 0.8) clipped to [16, 8192], bf16 checkpoints every 1024 tokens."""
    H, heads, every, slots = 64, [0, 37, 63], 1024, 256
    gen = torch.Generator().manual_seed(2)
    lens = [int(x) for x in torch.exp(torch.randn(48, generator=gen) * 0.8 + math.log(1024.0)).clamp(16, 8192).round().tolist()]
    N = len(lens)
    q, k, v, g, beta = plain_on_device(H, sum(lens), 201)
    pool = torch.randn(slots, H, D, D, generator=torch.Generator(device=DEV).manual_seed(202), device=DEV) * 0.05
    pool0 = pool.clone()
    idx = torch.randperm(slots, generator=gen)[:N].to(torch.int32).to(DEV)
    cu = cu_of(lens)
    ccs, rows = ck_meta(lens, every)
    ck = torch.full((rows, H, D, D), float("nan"), dtype=torch.bfloat16, device=DEV)
    launch = kda.prepare_plain(q, k, v, g, beta, D ** -0.5, pool, False, cu, dynamic_layout=True, ssm_state_indices=idx,
                               state_checkpoints=ck, checkpoint_cu_starts=ccs, checkpoint_every_n_tokens=every)
    out = launch()[0]
    torch.cuda.synchronize()
    assert kda.status_bits(launch) == 0 and kda.kernel_error(launch) == 0
    qs, ks, vs, gs, bs = _heads_cpu([q, k, v, g, beta], heads)
    gold_o, gold_s, gold_ck = gold_plain(qs, ks, vs, gs, bs, D ** -0.5, pool0[idx.long()][:, heads].cpu(), lens, every)
    ko.check_close(out[:, :, heads].cpu(), gold_o, "configs[2] output")
    ko.check_close(pool[idx.long()][:, heads].cpu(), gold_s, "configs[2] pool slots")
    ko.check_close(ck[:, heads].float().cpu(), gold_ck, "configs[2] bf16 checkpoint rows")
    assert not torch.isnan(ck.float()).any(), "a checkpoint row of another head was left unwritten"
    keep = torch.ones(slots, dtype=torch.bool, device=DEV)
    keep[idx.long()] = False
    assert torch.equal(pool[keep], pool0[keep]), "configs[2]: other pool slots modified"


def test_config3_long_context_full_size(kda):
    """configs[3] on one GPU: T = 131072, H = 96, g = logsigmoid(N(2,1)) (slow decay), zero initial state, through the
    context-parallel call (pieces planned by the library); two heads against the fp64 recurrence."""
    from kda_b200 import parallel
    H, T, heads = 96, 131072, [5, 95]
    q, k, v, g, beta = plain_on_device(H, T, 301, g_mean=2.0)
    out, fin = parallel.context_parallel_prefill(q, k, v, g, beta, None, None, D ** -0.5, None, raw=False)
    torch.cuda.synchronize()
    qs, ks, vs, gs, bs = _heads_cpu([q, k, v, g, beta], heads)
    gold_o, gold_s = c_oracle.recurrence_plain(qs, ks, vs, gs, bs, D ** -0.5, None, None)
    ko.check_close(out[:, :, heads].cpu(), gold_o, "configs[3] output")
    # the context-parallel call works value-first; the plain oracle returns key-first states
    ko.check_close(fin[:, heads].transpose(-1, -2).cpu(), gold_s, "configs[3] final state")


def test_config4_one_graph_over_batch_layouts(kda):
    """configs[4]: ONE captured graph (token capacity 32768, H = 64, 512 sequence slots, pool of 1024 slots) replayed
    over the layouts 1 x 32768, 32 x 1024, 512 x 64 and a random mix by rewriting cu_seqlens in place; the number of
    live sequences changes from replay to replay (trailing table entries describe empty sequences, whose slots must
    stay bit-identical like every other untouched slot)."""
    T, H, N_CAP, SLOTS, heads = 32768, 64, 512, 1024, [0, 63]
    q, k, v, g, beta = plain_on_device(H, T, 401, g_mean=2.0)
    pool0 = torch.randn(SLOTS, H, D, D, generator=torch.Generator(device=DEV).manual_seed(402), device=DEV) * 0.05
    pool = pool0.clone()
    slots = torch.randperm(SLOTS, generator=torch.Generator().manual_seed(3))[:N_CAP].to(torch.int32).to(DEV)
    rng = random.Random(5)
    mix, left = [], T
    while left > 0:
        n = min(left, rng.randint(1, 4096))
        mix.append(n)
        left -= n
    layouts = {"1x32768": [T], "32x1024": [1024] * 32, "512x64": [64] * 512, "mix": mix}

    def cu_full(lens):
        c = [0, *np.cumsum(lens).tolist()]
        return torch.tensor(c + [T] * (N_CAP + 1 - len(c)), dtype=torch.int64, device=DEV)

    cu = cu_full(layouts["32x1024"])
    launch = kda.prepare_plain(q, k, v, g, beta, D ** -0.5, pool, False, cu, dynamic_layout=True, ssm_state_indices=slots)
    launch()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        res = launch()
    qs, ks, vs, gs, bs = _heads_cpu([q, k, v, g, beta], heads)
    for name, lens in layouts.items():
        n = len(lens)
        cu.copy_(cu_full(lens))
        pool.copy_(pool0)
        graph.replay()
        torch.cuda.synchronize()
        assert kda.status_bits(launch) == 0 and kda.kernel_error(launch) == 0, name
        live = slots[:n].long()
        gold_o, gold_s = c_oracle.recurrence_plain(qs, ks, vs, gs, bs, D ** -0.5, pool0[live][:, heads].cpu(),
                                                   torch.tensor([0, *np.cumsum(lens).tolist()]))
        ko.check_close(res[0][:, :, heads].cpu(), gold_o, f"configs[4] {name} output")
        ko.check_close(pool[live][:, heads].cpu(), gold_s, f"configs[4] {name} touched pool slots")
        keep = torch.ones(SLOTS, dtype=torch.bool, device=DEV)
        keep[live] = False
        assert torch.equal(pool[keep], pool0[keep]), f"configs[4] {name}: untouched pool slots modified"
