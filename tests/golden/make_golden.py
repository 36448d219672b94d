"""Generate the golden vectors in this directory from the reference modules.

Run in a container where the reference checkout is mounted::

    python tests/golden/make_golden.py --reference <path of the BGU-CS-VIL/WTConv checkout>

The reference package ``wtconv`` is imported UNCHANGED from that path (only the
table-only ``pywt`` stand-in in ``oracle/pywt_stub`` is put in front of it,
because PyWavelets cannot be installed offline).  Every case stores the seeded
input, all parameters (by their reference ``state_dict`` key) and the output of
the reference module's own ``forward`` -- so the committed ``.npz`` files pin
both oracles and the CUDA path to the reference's arithmetic.  The files are
small (a few hundred KB in total); the full BASELINE config 1 is stored as
summary statistics plus a slice (see ``cfg1`` below).
"""
from __future__ import annotations

import argparse
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))

# (name, ndim, C, K, L, stride, bias, shape, dtype)
CASES = [
    ("2d_c4_k5_l3_even", 2, 4, 5, 3, 1, True, (2, 4, 16, 24), "float32"),
    ("2d_c3_k5_l3_odd", 2, 3, 5, 3, 1, True, (2, 3, 13, 9), "float32"),
    ("2d_c2_k3_l2_odd", 2, 2, 3, 2, 1, False, (1, 2, 7, 7), "float32"),
    ("2d_c2_k7_l4_deep", 2, 2, 7, 4, 1, True, (1, 2, 5, 6), "float32"),
    ("2d_c2_k1_l2", 2, 2, 1, 2, 1, True, (1, 2, 6, 5), "float32"),
    ("2d_c4_k5_l2_stride2", 2, 4, 5, 2, 2, True, (2, 4, 11, 14), "float32"),
    ("2d_c8_k5_l5_56", 2, 8, 5, 5, 1, True, (1, 8, 56, 56), "float32"),
    ("2d_c8_k5_l2_7", 2, 8, 5, 2, 1, True, (2, 8, 7, 7), "float32"),
    ("2d_c4_k5_l1_1x1", 2, 4, 5, 1, 1, True, (1, 4, 1, 1), "float32"),
    ("2d_c8_k5_l3_bf16", 2, 8, 5, 3, 1, True, (2, 8, 14, 14), "bfloat16"),
    ("2d_c8_k5_l3_f16", 2, 8, 5, 3, 1, True, (2, 8, 14, 14), "float16"),
    ("1d_c4_k5_l4_even", 1, 4, 5, 4, 1, True, (2, 4, 256), "float32"),
    ("1d_c3_k5_l4_odd", 1, 3, 5, 4, 1, True, (2, 3, 257), "float32"),
    ("1d_c2_k3_l3_stride3", 1, 2, 3, 3, 3, False, (1, 2, 100), "float32"),
    ("1d_c2_k7_l5_short", 1, 2, 7, 5, 1, True, (1, 2, 9), "float32"),
]


def build(ref_mod, ndim, c, k, levels, stride, bias, seed):
    torch.manual_seed(seed)
    cls = ref_mod["WTConv2d"] if ndim == 2 else ref_mod["WTConv1d"]
    m = cls(c, c, kernel_size=k, stride=stride, bias=bias, wt_levels=levels, wt_type="db1")
    g = torch.Generator().manual_seed(seed + 1)
    with torch.no_grad():
        for i in range(levels):
            m.wavelet_scale[i].weight.copy_(
                torch.rand(m.wavelet_scale[i].weight.shape, generator=g) * 0.15 + 0.05)
        m.base_scale.weight.copy_(torch.rand(m.base_scale.weight.shape, generator=g) + 0.5)
    return m.eval()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of the reference checkout (read only)")
    args = ap.parse_args()
    sys.path.insert(0, os.path.join(ROOT, "oracle", "pywt_stub"))
    sys.path.insert(0, args.reference)
    from wtconv.wtconv2d import WTConv2d          # the reference, unchanged
    from wtconv.wtconv1d import WTConv1d
    ref_mod = {"WTConv2d": WTConv2d, "WTConv1d": WTConv1d}
    torch.set_num_threads(1)

    for idx, (name, ndim, c, k, levels, stride, bias, shape, dtype) in enumerate(CASES):
        seed = 1000 + idx
        m = build(ref_mod, ndim, c, k, levels, stride, bias, seed)
        g = torch.Generator().manual_seed(seed + 2)
        x = torch.randn(shape, generator=g)
        tdt = getattr(torch, dtype)
        m = m.to(tdt)
        x = x.to(tdt)
        with torch.no_grad():
            y = m(x)
        out = {"x": x.float().numpy(), "y": y.float().numpy(),
               "meta": np.array([ndim, c, k, levels, stride, int(bias)], dtype=np.int64),
               "dtype": np.array(dtype)}
        for key, val in m.state_dict().items():
            out["p:" + key] = val.float().numpy()
        np.savez_compressed(os.path.join(HERE, name + ".npz"), **out)
        print(f"{name}: x{tuple(x.shape)} -> y{tuple(y.shape)} {dtype}")

    # BASELINE config 1, verbatim recipe: seed 0, default init, randn input.
    torch.manual_seed(0)
    m = WTConv2d(32, 32, kernel_size=5, wt_levels=3, bias=True).eval()
    x = torch.randn(8, 32, 56, 56)
    with torch.no_grad():
        y = m(x)
        y64 = m.double()(x.double())
    out = {"x_stats": np.array([x.double().sum().item(), x.double().pow(2).sum().item()]),
           "y_stats": np.array([y.double().sum().item(), y.double().pow(2).sum().item(),
                                y.abs().max().item()]),
           "y_slice": y[0, :4].numpy(), "y64_slice": y64[0, :4].numpy(),
           "y_rows": y[:, :, 17, :].numpy()}
    for key, val in m.float().state_dict().items():
        if "filter" not in key:
            out["p:" + key] = val.numpy()
    np.savez_compressed(os.path.join(HERE, "cfg1.npz"), **out)
    print("cfg1 written; fp32 vs fp64 err", float((y.double() - y64).abs().max() / y64.abs().max()))


if __name__ == "__main__":
    main()
