"""Kimi Delta Attention (KDA) chunked prefill for NVIDIA B200 (sm_100a), host side.

Same calling conventions as the reference's `kda/b200/kda_b200.py` (lines 44-76 there):

    out, final_state = kda_prefill(q, k, v, g, beta, A_log, dt_bias, initial_state, cu_seqlens)
    launch = prepare(q, k, v, g, beta, A_log, dt_bias, scale, pool, cu_seqlens, dynamic_layout=True,
                     ssm_state_indices=slots, state_checkpoints=ckpt, checkpoint_cu_starts=starts,
                     checkpoint_every_n_tokens=64)
    out, pool, ckpt = launch()          # zero-argument, re-reads every buffer, CUDA-graph capturable
    status_bits(launch)                 # 0 = every caller table was valid

Shapes: q, k, v, g [1, T, H, 128] bf16; beta [1, T, H] bf16 logits; A_log [H] fp32; dt_bias [H*128] fp32;
initial_state [N, H, 128 (V), 128 (K)] fp32 value-first, or a pool [P, H, 128, 128] with `ssm_state_indices`;
cu_seqlens [N+1] int32/int64 or None (one sequence).  Gate, beta sigmoid and q/k L2 norm are computed in the kernel.

`chunk_kda` is the plain, pre-activated call (g = fp32 log-decay, beta in (0,1), q/k already normalised, state
key-first [N, H, K, V]).

All compute goes through the C ABI of libkda_b200.so (include/kda_b200.h); this module only checks arguments,
owns output / workspace tensors and passes raw device pointers.  There is no CPU or eager fallback.
"""
from __future__ import annotations

import ctypes as C
import os

import torch

from . import _cabi

D = 128
CHUNK = 32
LOWER_BOUND = -5.0   # the reference fixes the gate's lower bound (kda/b200/csrc/w3/base/kernel.py:723)

__all__ = ["kda_prefill", "run", "prepare", "status_bits", "chunk_kda", "prepare_plain"]


def default_kernel():
    """Kernel used by new launches: the tcgen05 kernel, unless KDA_B200_KERNEL=mma_sync selects the warp-level
    cross-check kernel (read when a launch is prepared, not on the hot path)."""
    return _cabi.KERNEL_MMA_SYNC if os.environ.get("KDA_B200_KERNEL", "") == "mma_sync" else _cabi.KERNEL_TCGEN05


def _err(msg):
    return ValueError("KDA kernel: " + msg)


def _byte_interval(t):
    """[lo, hi) of the bytes a tensor's elements can touch (its extreme elements under its strides), or None when empty."""
    if t is None or not torch.is_tensor(t) or t.numel() == 0:
        return None
    reach = 0
    for extent, stride in zip(t.shape, t.stride()):
        reach += (extent - 1) * abs(stride)
    return t.data_ptr(), t.data_ptr() + (reach + 1) * t.element_size()


def _reject_aliasing(written, read_only):
    """Buffers the launch writes (state pool, checkpoint rows) may not share bytes with one another or with anything it
    reads: sequences are processed in an order the caller does not control, so the result would depend on it.  The
    reference refuses such calls as well (kda/b200/csrc/w3/kernel.py:1016-1026).  One sweep over the intervals sorted by
    start address: an overlap exists exactly when some interval starts before the furthest end seen so far."""
    ivs = []
    for is_written, group in ((True, written), (False, read_only)):
        for name, t in group:
            iv = _byte_interval(t)
            if iv is not None:
                ivs.append((iv[0], iv[1], is_written, name))
    ivs.sort(key=lambda r: r[0])
    # furthest-reaching written and read-only interval seen so far: (end, name)
    far = {True: (0, None), False: (0, None)}
    for lo, hi, is_written, name in ivs:
        clash = far[True] if far[True][0] > lo else (far[False] if is_written and far[False][0] > lo else None)
        if clash is not None:
            w, o = (name, clash[1]) if is_written else (clash[1], name)
            raise _err(f"{w} overlaps the memory of {o}: written buffers must not alias any other operand")
        if hi > far[is_written][0]:
            far[is_written] = (hi, name)


def _token_view_ok(t, width):
    """True when the kernel can read `t` in place.  [1,T,H,width] tiles go through the copy engine: unit inner stride,
    heads `width` apart, token stride a multiple of 8 elements, 16-byte aligned base.  beta [1,T,H] is read with scalar
    loads: unit head stride and a token stride of at least H are enough (any H, any alignment)."""
    T, H = t.shape[1], t.shape[2]
    if t.dim() == 3:
        return (H == 1 or t.stride(2) == 1) and (T <= 1 or t.stride(1) >= H)
    if t.stride(3) != 1 or (H > 1 and t.stride(2) != width) or t.data_ptr() % 16:
        return False
    return T <= 1 or (t.stride(1) % 8 == 0 and t.stride(1) >= H * width)


def _table(t, name, n, live):
    if t is None:
        return None
    if not torch.is_tensor(t) or t.dtype not in (torch.int32, torch.int64) or t.dim() != 1 or t.numel() != n or not t.is_cuda:
        got = (tuple(t.shape), t.dtype) if torch.is_tensor(t) else type(t)
        raise _err(f"{name} must be a 1-D CUDA int32 / int64 tensor with {n} entries, got {got}")
    if not t.is_contiguous():
        if live:
            raise _err(f"{name} must be contiguous with dynamic_layout=True (the launch reads it in place at every replay)")
        raise _err(f"{name} must be contiguous")
    return t


def _check_args(q, k, v, g, beta, A_log, dt_bias, initial_state, cu_seqlens, dynamic_layout, raw):
    """Shape / dtype / device contract of the call (the conditions of kda/b200/csrc/w3/kernel.py:1255-1281; a violation
    raises ValueError).  Returns cu_seqlens, moved to q's device when the static path allows that."""
    operands = {"q": q, "k": k, "v": v, "g": g, "beta": beta}
    if raw:
        operands.update(A_log=A_log, dt_bias=dt_bias)
    bad = [n for n, t in operands.items() if not (torch.is_tensor(t) and t.is_cuda)]
    if bad:
        raise _err(f"{bad[0]} must be a CUDA tensor")
    if q.dim() != 4 or q.shape[0] != 1 or q.shape[3] != D:
        raise _err(f"expected q of shape [1, T, H, 128], got {tuple(q.shape)}")
    _, T, H, _ = q.shape
    # (name, tensor, what it must look like, does it?)
    rules = [(n, operands[n], f"the shape of q {tuple(q.shape)}", tuple(operands[n].shape) == tuple(q.shape)) for n in "kvg"]
    rules.append(("beta", beta, f"[1, T, H] = [1, {T}, {H}]",
                  beta.dim() >= 2 and beta.shape[0] == 1 and beta.shape[1] == T and beta.numel() == T * H))
    if raw:
        rules.append(("A_log", A_log, f"H = {H} entries", A_log.numel() == H))
        rules.append(("dt_bias", dt_bias, f"H * 128 = {H * D} entries", dt_bias.numel() == H * D))
    for name, t, want, ok in rules:
        if not ok:
            raise _err(f"{name} must have {want}, got {tuple(t.shape)}")
    if initial_state is not None and initial_state.dtype != torch.float32:
        raise _err(f"initial_state / the state pool must be fp32, got {initial_state.dtype}")
    for t in (*operands.values(), initial_state, cu_seqlens):
        if torch.is_tensor(t) and t.is_cuda and t.device != q.device:
            raise _err(f"all CUDA tensors must be on the device of q ({q.device}), got one on {t.device}")
    if cu_seqlens is None:
        return None
    if not (torch.is_tensor(cu_seqlens) and cu_seqlens.dim() == 1 and cu_seqlens.dtype in (torch.int32, torch.int64)):
        raise _err("cu_seqlens must be a 1-D int32 / int64 tensor")
    if cu_seqlens.numel() < 2:
        raise _err("cu_seqlens must describe at least one sequence")
    if cu_seqlens.device == q.device and cu_seqlens.is_contiguous():
        return cu_seqlens
    if dynamic_layout:
        raise _err("cu_seqlens must be a contiguous tensor on q's device with dynamic_layout=True "
                   "(it is read in place at every replay)")
    return cu_seqlens.to(q.device).contiguous()


class _Launch:
    """Zero-argument launch closure.  Owns the output, workspace and status tensors; every call re-reads the caller's
    buffers (same addresses) and enqueues two kernels on the current stream."""

    def __init__(self, args, keep, copies, result, status, device):
        self._args = args
        self._keep = keep          # tensors whose storage the argument block points into
        self._copies = copies      # (private contiguous copy, caller tensor) pairs refreshed at every call
        self._result = result
        self.status = status
        self._device = device
        self._lib = _cabi.lib()

    def __call__(self):
        for c, t in self._copies:
            c.copy_(t)
        with torch.cuda.device(self._device):
            stream = torch.cuda.current_stream(self._device).cuda_stream
            rc = self._lib.kda_prefill_launch(C.byref(self._args), C.c_void_p(stream))
        _cabi.check(rc, "kda_prefill_launch")
        return self._result

    def plan_counts(self):
        """(tasks of the first launch, tasks of the second launch, cut sequences) as the device planner decided them at
        the most recent call; the second and third are 0 when no sequence was cut.  Synchronises."""
        counts = (C.c_int32 * 3)()
        with torch.cuda.device(self._device):
            stream = torch.cuda.current_stream(self._device).cuda_stream
            _cabi.check(self._lib.kda_prefill_plan_counts(C.byref(self._args), counts, C.c_void_p(stream)), "kda_prefill_plan_counts")
        return tuple(int(c) for c in counts)


def cut_capacity(T, H, n_sms=148):
    """Pieces the device planner may cut long sequences into, over the whole call (the workspace holds three 64 KB state
    maps per piece and head).  Cutting only pays while (sequence, head) chains are too few or too uneven to fill the
    SMs, so about two pieces per SM-and-head are plenty; calls too short to have a long chain get none."""
    if T < 64 * CHUNK or H >= 2 * n_sms:
        return 0
    return int(min(_cabi.MAX_CUT_PIECES, max(2, -(-2 * n_sms // H))))


def status_bits(launch):
    """Table-validation bits of the most recent call of a launch (0 = every caller table was valid; synchronises):
    1 = rejected cu_seqlens (every sequence treated as empty, output zero-filled), 2 = bad / repeated
    ssm_state_indices entry, 4 = bad initial_state_indices entry, 8 = checkpoint rows outside state_checkpoints or
    overlapping (kda/b200/kda_b200.py:56-62)."""
    status = getattr(launch, "status", None)
    return 0 if status is None else int(status[0].item())


def kernel_error(launch):
    """Device-side error code of the most recent call (0 = none); synchronises."""
    status = getattr(launch, "status", None)
    return 0 if status is None else int(status[2].item())


def _prepare(q, k, v, g, beta, A_log, dt_bias, scale, initial_state, cu_seqlens, *, raw, key_first,
             ssm_state_indices=None, state_checkpoints=None, checkpoint_cu_starts=None, checkpoint_every_n_tokens=0,
             initial_state_source=None, initial_state_indices=None, dynamic_layout=False, want_final=True, kernel=None,
             max_cut_pieces=None):
    cu_seqlens = _check_args(q, k, v, g, beta, A_log, dt_bias, initial_state, cu_seqlens, dynamic_layout, raw)
    dev = q.device
    T, H = q.shape[1], q.shape[2]
    N = 1 if cu_seqlens is None else cu_seqlens.numel() - 1
    pool = ssm_state_indices is not None
    every = int(checkpoint_every_n_tokens or 0)

    # ---- token tensors: read in place when the layout allows, else through a private copy refreshed per launch
    copies, keep = [], []
    tok_dt = torch.bfloat16
    g_dt = torch.bfloat16 if raw else torch.float32
    b_dt = torch.bfloat16 if raw else torch.float32

    def norm(t, dt, width):
        if t.dtype == dt and _token_view_ok(t, width):
            return t
        c = torch.empty(t.shape, dtype=dt, device=dev)
        copies.append((c, t))
        return c

    if beta.dim() != 3:
        beta = beta.reshape(1, T, H)
    q_, k_, v_ = norm(q, tok_dt, D), norm(k, tok_dt, D), norm(v, tok_dt, D)
    g_, beta_ = norm(g, g_dt, D), norm(beta, b_dt, 1)
    if raw:
        A_ = A_log if (A_log.dtype == torch.float32 and A_log.is_contiguous()) else None
        if A_ is None:
            A_ = torch.empty(H, dtype=torch.float32, device=dev)
            copies.append((A_, A_log.reshape(H)))
        dtb_ = dt_bias if (dt_bias.dtype == torch.float32 and dt_bias.is_contiguous()) else None
        if dtb_ is None:
            dtb_ = torch.empty(H * D, dtype=torch.float32, device=dev)
            copies.append((dtb_, dt_bias.reshape(H * D)))
    else:
        A_ = dtb_ = None

    # ---- state
    _reject_aliasing([("the state pool", initial_state if pool else None),
                      ("state_checkpoints", state_checkpoints if every else None)],
                     [("initial_state_source", initial_state_source), ("initial_state", None if pool else initial_state)]
                     + [(n, t) for n, t in zip("q k v g beta A_log dt_bias".split(), (q, k, v, g, beta, A_log, dt_bias))
                        if torch.is_tensor(t)])
    if initial_state is None and pool:
        raise _err("initial_state (the pool) is required with ssm_state_indices")
    if pool:
        if not (initial_state.dim() == 4 and tuple(initial_state.shape[1:]) == (H, D, D)):
            raise _err(f"the state pool must be fp32 [P, {H}, 128, 128], got {tuple(initial_state.shape)} {initial_state.dtype}")
        if not (initial_state.stride()[1:] == (D * D, D, 1) and initial_state.stride(0) >= H * D * D
                and initial_state.stride(0) % 4 == 0 and initial_state.data_ptr() % 16 == 0):
            raise _err("pool slots must be dense [H, 128, 128] blocks, slot stride >= H*128*128 and a multiple of 4 floats, "
                       "16-byte aligned")
    elif initial_state is not None:
        if tuple(initial_state.shape) != (N, H, D, D):
            raise _err(f"initial_state must be [N, H, 128, 128] with N = {N}, got {tuple(initial_state.shape)}")
        if not initial_state.is_contiguous():
            raise _err("initial_state must be contiguous without ssm_state_indices")
        if initial_state.data_ptr() % 16:
            c = torch.empty_like(initial_state)
            copies.append((c, initial_state))
            initial_state = c
    d_idx = _table(ssm_state_indices, "ssm_state_indices", N, dynamic_layout)
    s_idx = _table(initial_state_indices, "initial_state_indices", N, dynamic_layout)
    src = initial_state
    if initial_state_source is not None:
        src = initial_state_source
        if not (src.dtype == torch.float32 and src.dim() == 4 and tuple(src.shape[1:]) == (H, D, D)
                and src.stride()[1:] == (D * D, D, 1) and src.stride(0) > 0 and src.stride(0) % 4 == 0
                and src.data_ptr() % 16 == 0):
            raise _err("initial_state_source must be fp32 [P0, H, 128, 128] with dense, 16-byte aligned slots")
        if s_idx is None:
            raise _err("initial_state_source needs initial_state_indices")
    elif s_idx is not None:
        raise _err("initial_state_indices without initial_state_source")
    if pool:
        dst = initial_state
    elif want_final:
        dst = torch.empty(N, H, D, D, dtype=torch.float32, device=dev)
    else:
        dst = None

    # ---- checkpoints
    ck = ck_starts = None
    ck_copy_back = None
    if every:
        if every < CHUNK or every % CHUNK:
            raise _err(f"checkpoint_every_n_tokens must be a multiple of {CHUNK} (chunk size), got {every}")
        if state_checkpoints is None or checkpoint_cu_starts is None:
            raise _err("checkpoint_every_n_tokens needs state_checkpoints and checkpoint_cu_starts")
        if not (torch.is_tensor(state_checkpoints) and state_checkpoints.dtype in (torch.float32, torch.bfloat16)
                and state_checkpoints.is_contiguous() and state_checkpoints.dim() == 4
                and tuple(state_checkpoints.shape[1:]) == (H, D, D) and state_checkpoints.device == dev):
            raise _err("state_checkpoints must be a contiguous fp32 or bf16 [C, H, 128, 128] CUDA tensor")
        ck = state_checkpoints
        if ck.data_ptr() % 16:
            raise _err("state_checkpoints must be 16-byte aligned")
        ck_starts = _table(checkpoint_cu_starts, "checkpoint_cu_starts", N + 1, dynamic_layout)

    lib = _cabi.lib()
    pieces = cut_capacity(T, H) if max_cut_pieces is None else int(max_cut_pieces)
    ws_bytes = lib.kda_prefill_workspace_bytes_cuts(N, H, pieces)
    workspace = torch.zeros(ws_bytes + 256, dtype=torch.uint8, device=dev)
    ws_ptr = (workspace.data_ptr() + 255) // 256 * 256
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    out = torch.empty(1, T, H, D, dtype=torch.bfloat16, device=dev)

    a = _cabi.KdaPrefillArgs()
    a.q, a.k, a.v, a.g, a.beta, a.out = (q_.data_ptr(), k_.data_ptr(), v_.data_ptr(), g_.data_ptr(), beta_.data_ptr(),
                                         out.data_ptr())
    a.ldq, a.ldk, a.ldv, a.ldg = (t.stride(1) if T > 1 else H * D for t in (q_, k_, v_, g_))
    a.ldbeta = beta_.stride(1) if T > 1 else H
    a.ldo = H * D
    a.A_log = A_.data_ptr() if raw else None
    a.dt_bias = dtb_.data_ptr() if raw else None
    a.scale, a.lower_bound = float(scale), LOWER_BOUND
    a.frontend = _cabi.FRONTEND_RAW if raw else _cabi.FRONTEND_PLAIN
    a.state_layout = _cabi.STATE_KEY_FIRST if key_first else _cabi.STATE_VALUE_FIRST
    a.H, a.N, a.T = H, N, T
    a.cu_seqlens = cu_seqlens.data_ptr() if cu_seqlens is not None else None
    a.cu_is64 = int(cu_seqlens is not None and cu_seqlens.dtype == torch.int64)
    if src is not None:
        a.src_base, a.src_slot_stride, a.src_slots = src.data_ptr(), src.stride(0), src.shape[0]
    a.src_idx = s_idx.data_ptr() if s_idx is not None else None
    a.src_idx_is64 = int(s_idx is not None and s_idx.dtype == torch.int64)
    if dst is not None:
        a.dst_base, a.dst_slot_stride, a.dst_slots = dst.data_ptr(), dst.stride(0), dst.shape[0]
    a.dst_idx = d_idx.data_ptr() if d_idx is not None else None
    a.dst_idx_is64 = int(d_idx is not None and d_idx.dtype == torch.int64)
    if every:
        a.ck_base, a.ck_is_bf16, a.ck_every, a.ck_rows = ck.data_ptr(), int(ck.dtype == torch.bfloat16), every, ck.shape[0]
        a.ck_starts, a.ck_starts_is64 = ck_starts.data_ptr(), int(ck_starts.dtype == torch.int64)
    a.workspace, a.workspace_bytes = ws_ptr, ws_bytes
    a.status = status.data_ptr()
    a.kernel = default_kernel() if kernel is None else int(kernel)
    a.max_cut_pieces = pieces

    keep += [q_, k_, v_, g_, beta_, A_, dtb_, cu_seqlens, src, dst, d_idx, s_idx, ck, ck_starts, workspace, status, out]
    result = (out, dst) if not every else (out, dst, state_checkpoints)
    return _Launch(a, keep, copies, result, status, dev)


def prepare(q, k, v, g, beta, A_log, dt_bias, scale, initial_state, cu_seqlens=None, *, dynamic_layout=False, **serving):
    """prepare(...) -> launch.  Same arguments as `run` plus `dynamic_layout`; `launch()` re-reads the current contents of
    every input buffer.  The schedule is always derived on the device from cu_seqlens, so both settings are CUDA-graph
    safe; `dynamic_layout=True` additionally insists that the tables are contiguous device tensors read in place
    (kda/b200/kda_b200.py:49-53).  Without a pool, `initial_state` is read-only and the final state is a new tensor."""
    if initial_state is None and serving.get("initial_state_source") is None:
        raise _err("initial_state is required unless only initial_state_source is given")
    return _prepare(q, k, v, g, beta, A_log, dt_bias, scale, initial_state, cu_seqlens, raw=True, key_first=False,
                    dynamic_layout=dynamic_layout, **serving)


def run(q, k, v, g, beta, A_log, dt_bias, scale, initial_state, cu_seqlens=None, **serving):
    """run(...) -> (output, final_state[, state_checkpoints]); the serving entry point (kda/b200/kda_b200.py:44-47)."""
    return prepare(q, k, v, g, beta, A_log, dt_bias, scale, initial_state, cu_seqlens, dynamic_layout=True, **serving)()


def kda_prefill(q, k, v, g, beta, A_log, dt_bias, initial_state, cu_seqlens=None, scale=None, *,
                ssm_state_indices=None, state_checkpoints=None, checkpoint_cu_starts=None, checkpoint_every_n_tokens=0,
                initial_state_source=None, initial_state_indices=None):
    """Keyword-friendly wrapper of `run`; scale defaults to 1/sqrt(128) (kda/b200/kda_b200.py:65-76)."""
    if scale is None:
        scale = q.shape[-1] ** -0.5
    return run(q, k, v, g, beta, A_log, dt_bias, scale, initial_state, cu_seqlens,
               ssm_state_indices=ssm_state_indices, state_checkpoints=state_checkpoints,
               checkpoint_cu_starts=checkpoint_cu_starts, checkpoint_every_n_tokens=checkpoint_every_n_tokens,
               initial_state_source=initial_state_source, initial_state_indices=initial_state_indices)


def prepare_plain(q, k, v, g, beta, scale=None, initial_state=None, output_final_state=False, cu_seqlens=None, **serving):
    """Launch closure of the pre-activated call (see chunk_kda)."""
    if q.dim() == 4 and q.shape[0] > 1:
        if cu_seqlens is not None:
            raise _err("cu_seqlens needs batch size 1 (packed varlen layout)")
        B, T = q.shape[0], q.shape[1]
        q, k, v, g = (t.reshape(1, B * T, *t.shape[2:]) for t in (q, k, v, g))
        beta = beta.reshape(1, B * T, -1)
        cu_seqlens = torch.arange(0, (B + 1) * T, T, dtype=torch.int64, device=q.device)
    if scale is None:
        scale = q.shape[-1] ** -0.5
    return _prepare(q, k, v, g, beta, None, None, scale, initial_state, cu_seqlens, raw=False, key_first=True,
                    want_final=output_final_state or "ssm_state_indices" in serving, **serving)


def chunk_kda(q, k, v, g, beta, scale=None, initial_state=None, output_final_state=False, cu_seqlens=None, **serving):
    """Plain `chunk_kda`-style call with PRE-ACTIVATED inputs: q, k already L2-normalised, g the fp32 log-decay (<= 0)
    per token / head / key channel, beta fp32 in (0, 1); state key-first [N, H, K, V] fp32.  q, k, v are read as bf16
    (other dtypes are cast).  Returns (o [B, T, H, 128] in q's dtype, final_state or None)."""
    shape, dt = q.shape, q.dtype
    res = prepare_plain(q, k, v, g, beta, scale, initial_state, output_final_state, cu_seqlens, **serving)()
    o = res[0].reshape(shape)
    return (o if dt == torch.bfloat16 else o.to(dt), *res[1:])
