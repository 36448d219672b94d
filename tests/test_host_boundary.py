"""CPU checks of the drop-in boundary: exported symbols, module API, state_dict layout."""
import ctypes
import os
import re

import numpy as np
import pytest
import torch

from conftest import ROOT, golden_names, load_golden


def _lib():
    from wtconv_b200 import _lib as L
    if not os.path.exists(L.LIB_PATH):
        from wtconv_b200 import build
        build.build()
    return L


def test_library_exports_every_declared_symbol():
    L = _lib()
    header = open(os.path.join(ROOT, "include", "wtconv_b200.h")).read()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    declared = set(re.findall(r"\b(wtconv\w*)\s*\(", header))
    assert declared == set(L.SYMBOLS), "header and ctypes table disagree"
    lib = ctypes.CDLL(L.LIB_PATH)
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared in include/wtconv_b200.h but not exported"


def test_host_only_entry_points():
    L = _lib()
    lib = L.load()
    assert lib.wtconv_query(0) == 1 and lib.wtconv_query(1) == 29 and lib.wtconv_query(3) == 100
    # 2-D: per-channel block (28 floats per tap set, 1 + 4*5 sets) + channels-last copy (26 x 16 per set and group)
    assert lib.wtconv_packed_param_floats(2, 96, 5, 5) == 96 * 28 * 21 + 6 * 21 * 26 * 16
    assert lib.wtconv_packed_param_floats(1, 64, 5, 4) == 64 * 8 * 9
    assert "odd" in L.status_string(-2)
    nbytes = ctypes.c_size_t(123)
    assert lib.wtconv2d_workspace_bytes(128, 192, 28, 28, 5, 4, 1, None, None, ctypes.byref(nbytes)) == 0
    assert nbytes.value == 0                        # NCHW, small planes: the whole cascade stays on chip
    cl = (ctypes.c_longlong * 4)(192 * 28 * 28, 1, 28 * 192, 192)
    assert lib.wtconv2d_workspace_bytes(128, 192, 28, 28, 5, 4, 1, cl, cl, ctypes.byref(nbytes)) == 0
    # channels-last: fp32 reconstruction of level 2 (14 x 14) + the four bf16 sub-bands of level 2 (7 x 7)
    # when the tensors start on 16-byte boundaries; the chain of unaligned tensors (low-pass planes and
    # reconstructions of levels 1 and 2 in fp32) needs more, and the larger figure is reported
    aligned = 128 * 192 * (14 * 14 * 4 + 4 * 7 * 7 * 2)
    unaligned = 128 * 192 * (2 * 14 * 14 + 2 * 7 * 7) * 4
    assert nbytes.value == max(aligned, unaligned)
    assert lib.wtconv2d_workspace_bytes(2, 256, 512, 512, 5, 5, 1, None, None, ctypes.byref(nbytes)) == 0
    assert 0 < nbytes.value <= 2 * 256 * 512 * 512 * 4 // 3
    assert lib.wtconv2d_workspace_bytes(2, 8, 16, 16, 4, 5, 1, None, None, ctypes.byref(nbytes)) == -2


def test_launch_chains_of_the_benchmark_shapes():
    """Planner through the C ABI (host only): large channels-last planes take the channels-last
    chain (pyramid, deep stage, level stage), small ones the register-level kernels, NCHW and other
    kernel sizes the CTA-tile stages."""
    L = _lib()
    lib = L.load()

    def count(B, C, H, K, Lv, code, channels_last, stride=1):
        st = (ctypes.c_longlong * 4)(*((C * H * H, 1, H * C, C) if channels_last else (C * H * H, H * H, H, 1)))
        n = ctypes.c_int(-1)
        assert lib.wtconv2d_launch_count(B, C, H, H, K, Lv, stride, code, st, st, ctypes.byref(n)) == 0
        return n.value

    # bf16 channels-last: regplane | reduce, regplane, quad | pyramid, deep, level | the same
    assert [count(128, C, H, 5, Lv, 1, True) for C, H, Lv in
            ((768, 7, 2), (384, 14, 3), (192, 28, 4), (96, 56, 5))] == [1, 3, 3, 3]
    assert count(128, 96, 56, 5, 1, 1, True) == 1           # one level: the level stage alone
    assert count(128, 768, 7, 5, 2, 1, False) == 1          # NCHW: one whole-plane CTA-tile stage
    assert count(128, 96, 56, 5, 5, 1, False) == 1          # NCHW: the 56x56 pyramid still fits on chip
    assert count(2, 256, 512, 5, 5, 1, False) >= 4          # 512x512: reductions and a chain of tiled stages
    # channels-last 512x512: two low-pass launches, pyramid, deep stage (level 5), level stages 4, 3, 2, 1
    assert count(2, 256, 512, 5, 5, 1, True) == 8
    assert count(128, 768, 7, 3, 2, 1, True) == 1           # K = 3 has no register-level instance
    assert count(4, 16, 7, 5, 2, 0, True, stride=2) == 1    # strided output: CTA-tile stage
    n = ctypes.c_int(0)
    assert lib.wtconv2d_launch_count(1, 8, 8, 8, 4, 1, 1, 0, None, None, ctypes.byref(n)) == -2   # even K


@pytest.mark.parametrize("name", golden_names())
def test_state_dict_matches_reference_layout(name):
    import wtconv_b200
    x, params, y, meta = load_golden(name)
    cls = wtconv_b200.WTConv2d if meta["ndim"] == 2 else wtconv_b200.WTConv1d
    m = cls(meta["C"], meta["C"], kernel_size=meta["K"], stride=meta["stride"], bias=meta["bias"], wt_levels=meta["L"])
    sd = m.state_dict()
    assert list(sd.keys()) == list(params.keys())            # same names in the same order
    for k, v in params.items():
        assert tuple(sd[k].shape) == v.shape, k
    if meta["dtype"] == "float32":
        assert np.array_equal(sd["wt_filter"].numpy(), params["wt_filter"])
        assert np.array_equal(sd["iwt_filter"].numpy(), params["iwt_filter"])
    m.load_state_dict({k: torch.from_numpy(v) for k, v in params.items()}, strict=True)
    assert not m.wt_filter.requires_grad and not m.iwt_filter.requires_grad
    assert sum(p.numel() for p in m.parameters()) == sum(v.size for v in params.values())


def test_module_api_and_errors():
    import wtconv_b200
    m = wtconv_b200.WTConv2d(8, 8, 5, 2, False, 3, 'db1')         # positional order of the reference ctor
    assert (m.in_channels, m.wt_levels, m.stride, m.dilation) == (8, 3, 2, 1)
    assert m.base_conv.bias is None and isinstance(m.do_stride, torch.nn.AvgPool2d)
    with pytest.raises(AssertionError):
        wtconv_b200.WTConv2d(8, 16)
    with pytest.raises(NotImplementedError):
        wtconv_b200.WTConv2d(8, 8, wt_type='db2')
    with pytest.raises(RuntimeError, match="CUDA"):
        with torch.no_grad():
            m(torch.zeros(1, 8, 4, 4))
    # substrings the reference optimiser setup keys on (wtconvnext/wtconvnext.py:372-377)
    names = [n for n, _ in m.named_parameters()]
    assert any("wavelet_scale" in n for n in names) and any("base_scale" in n for n in names)
    # nn.Conv2d children are visible to the reference's _init_weights (wtconvnext/wtconvnext.py:483-487)
    assert sum(isinstance(c, torch.nn.Conv2d) for c in m.modules()) == 4
