"""Writes tests/golden/*.npz: outputs of the reference's OWN token-by-token definition (kda/b200/reference.py,
imported from the reference checkout given on the command line) on small seeded inputs.

    python tests/golden/make_golden.py /path/to/eat-kernels

The reference checkout is only needed to (re)generate the fixtures; the tests read the committed .npz files.
bf16 tensors are stored as their int16 bit patterns.
"""
import importlib.util
import math
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent / "oracle"))
from kda_oracle import make_inputs_raw  # noqa: E402  (seeded input generator only; outputs come from the reference)

CASES = {
    # name: (H, lens, seed, slow_decay, dtype of the reference run)
    "raw_h2_t70": (2, [70], 11, False, torch.float64),
    "raw_h2_varlen": (2, [5, 33, 64, 1], 12, False, torch.float64),
    "raw_h1_slow_t96": (1, [96], 13, True, torch.float64),
    "raw_h2_t40_fp32": (2, [40], 14, False, torch.float32),
}


def bits(t):
    return t.contiguous().view(torch.int16).numpy()


def main(ref_root):
    spec = importlib.util.spec_from_file_location("ref_reference", Path(ref_root) / "kda" / "b200" / "reference.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    for name, (H, lens, seed, slow, dtype) in CASES.items():
        q, k, v, g, beta, A_log, dt_bias, scale, init, cu = make_inputs_raw(H, lens, seed)
        if slow:   # slow decay as kda/b200/test_kda_b200.py:58-62: A_log = 0, dt_bias uniform in [-12, -6]
            gen = torch.Generator().manual_seed(seed)
            A_log.fill_(0.0)
            dt_bias.copy_(torch.rand(H * 128, generator=gen) * 6.0 - 12.0)
        out, fin = mod.kda_reference(q, k, v, g, beta, A_log, dt_bias, scale, init, cu, dtype=dtype)
        np.savez_compressed(HERE / f"{name}.npz", q=bits(q), k=bits(k), v=bits(v), g=bits(g), beta=bits(beta),
                            A_log=A_log.numpy(), dt_bias=dt_bias.numpy(), scale=np.float64(scale), init=init.numpy(),
                            cu=cu.numpy(), out=bits(out), final=fin.numpy(),
                            ref_dtype=np.array(str(dtype)))
        print(name, "T", sum(lens), "H", H, "out rms", float(out.float().pow(2).mean().sqrt()))


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: make_golden.py <path of a checkout of the reference repository>")
    main(sys.argv[1])
