"""ctypes front of oracle/kda_oracle.c (test infrastructure; the product path never imports this)."""
from __future__ import annotations

import ctypes
import subprocess
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
_libs = {}


def build():
    subprocess.run(["make", "-C", str(HERE), "-s"], check=True)


def lib(precision="f64"):
    if precision not in _libs:
        path = HERE / "_build" / f"libkda_oracle_{precision}.so"
        if not path.exists():
            build()
        L = ctypes.CDLL(str(path))
        fp, i64p = ctypes.POINTER(ctypes.c_float), ctypes.POINTER(ctypes.c_int64)
        L.kda_oracle_plain.argtypes = [fp, fp, fp, fp, fp, ctypes.c_double, fp, i64p, ctypes.c_int, ctypes.c_int, fp, fp]
        L.kda_oracle_raw.argtypes = [fp, fp, fp, fp, fp, fp, fp, ctypes.c_double, ctypes.c_double, fp, i64p,
                                     ctypes.c_int, ctypes.c_int, fp, fp]
        L.kda_oracle_plain.restype = L.kda_oracle_raw.restype = ctypes.c_int
        _libs[precision] = L
    return _libs[precision]


def _f32(t):
    return np.ascontiguousarray(t.detach().float().cpu().numpy())


def _p(a):
    return None if a is None else a.ctypes.data_as(ctypes.POINTER(ctypes.c_float))


def threads(precision="f64"):
    return lib(precision).kda_oracle_threads()


def set_threads(n=0, precision="f64"):
    """OpenMP threads of later calls of this precision's library (0 = every host CPU, whatever OMP_NUM_THREADS says)."""
    return lib(precision).kda_oracle_set_threads(int(n))


def recurrence_raw(q, k, v, g, beta, A_log, dt_bias, scale, initial_state, cu_seqlens, lower_bound=-5.0,
                   precision="f64"):
    """Same contract as kda_oracle.kda_recurrence: returns (out bf16 [1,T,H,128], final fp32 value-first)."""
    T, H = q.shape[1], q.shape[2]
    cu = np.asarray([0, T] if cu_seqlens is None else [int(c) for c in cu_seqlens], dtype=np.int64)
    N = len(cu) - 1
    a = [_f32(x[0]) for x in (q, k, v, g, beta)]
    init = None if initial_state is None else _f32(initial_state)
    out = np.zeros((T, H, 128), np.float32)
    fin = np.zeros((N, H, 128, 128), np.float32)
    rc = lib(precision).kda_oracle_raw(*[_p(x) for x in a], _p(_f32(A_log)), _p(_f32(dt_bias)), float(scale),
                                       float(lower_bound), _p(init), cu.ctypes.data_as(ctypes.POINTER(ctypes.c_int64)),
                                       N, H, _p(out), _p(fin))
    assert rc == 0
    return torch.from_numpy(out)[None].to(torch.bfloat16), torch.from_numpy(fin)


def recurrence_plain(q, k, v, g, beta, scale, initial_state, cu_seqlens, precision="f64"):
    """Same contract as kda_oracle.kda_recurrence_plain: returns (out fp32 [1,T,H,128], final fp32 key-first)."""
    T, H = q.shape[1], q.shape[2]
    cu = np.asarray([0, T] if cu_seqlens is None else [int(c) for c in cu_seqlens], dtype=np.int64)
    N = len(cu) - 1
    a = [_f32(x[0]) for x in (q, k, v, g, beta)]
    init = None if initial_state is None else _f32(initial_state)
    out = np.zeros((T, H, 128), np.float32)
    fin = np.zeros((N, H, 128, 128), np.float32)
    rc = lib(precision).kda_oracle_plain(*[_p(x) for x in a], float(scale), _p(init),
                                         cu.ctypes.data_as(ctypes.POINTER(ctypes.c_int64)), N, H, _p(out), _p(fin))
    assert rc == 0
    return torch.from_numpy(out)[None], torch.from_numpy(fin)
