"""Kernel logic on the CPU: the CTA bodies of the CUDA kernels, compiled for the host.

tests/emu/emu.cu compiles the same kernel bodies and planners as the product
library with the phase macro turned into a loop over thread ids, so tiling,
halos, odd-size zero extension, cropping, strides and the multi-stage chain are
checked here against the golden vectors of the reference without a GPU.
"""
import numpy as np
import pytest
import torch

import emu_lib
from conftest import golden_names, load_golden, max_err

TOL = {"float32": 1e-5, "bfloat16": 2e-2, "float16": 2e-2}


def _params(params):
    return {k: torch.from_numpy(v) for k, v in params.items() if "filter" not in k}


def _run(name, layout="nchw", force=(0, 0, 0)):
    x, params, y, meta = load_golden(name)
    dt = getattr(torch, meta["dtype"])
    packed = emu_lib.pack(_params(params), meta["ndim"], meta["C"], meta["K"], meta["L"],
                          param_dtype=dt, filter_dtype=dt)
    xt = torch.from_numpy(x).to(dt)
    if meta["ndim"] == 2:
        if layout == "cl":
            xt = xt.contiguous(memory_format=torch.channels_last)
        out, info = emu_lib.forward2d(xt, packed, meta["K"], meta["L"], meta["stride"], force)
    else:
        out, info = emu_lib.forward1d(xt, packed, meta["K"], meta["L"], meta["stride"], force)
    assert tuple(out.shape) == y.shape
    assert not torch.isnan(out.float()).any(), "kernel left output elements unwritten"
    return max_err(out.float().numpy(), y), TOL[meta["dtype"]], info


@pytest.mark.parametrize("layout", ["nchw", "cl"])
@pytest.mark.parametrize("name", golden_names())
def test_emulated_kernel_matches_reference(name, layout):
    if name.startswith("1d") and layout == "cl":
        pytest.skip("1-D has a single layout")
    err, tol, _ = _run(name, layout)
    assert err <= tol, f"{name}: err {err:.3e} > {tol}"


@pytest.mark.parametrize("force", [(8, 1, 1), (8, 2, 2), (16, 2, 4), (16, 3, 3), (8, 1, 2, 2), (16, 2, 1, 2)])
@pytest.mark.parametrize("name", [n for n in golden_names() if n.startswith("2d") and "1x1" not in n])
def test_emulated_tiled_multistage_chain(name, force):
    err, tol, info = _run(name, "cl", force)
    assert err <= tol, f"{name} force={force}: err {err:.3e} > {tol} (stages={info[0]})"
    if len(force) == 4 and force[3] == 2 and name == "2d_c8_k5_l5_56":
        assert info[0] >= 3 and info[1] >= 2      # chain with materialised low-pass planes


@pytest.mark.parametrize("force", [(64, 0, 1), (128, 0, 2)])
@pytest.mark.parametrize("name", [n for n in golden_names() if n.startswith("1d") and "short" not in n])
def test_emulated_1d_tiles(name, force):
    x, params, y, meta = load_golden(name)
    unit = (1 << meta["L"]) * 8 * meta["stride"]
    edge = max(force[0] // unit, 1) * unit
    err, tol, info = _run(name, "nchw", (edge, 0, force[2]))
    assert err <= tol, f"{name}: err {err:.3e} (tiles={info[0]})"


# Register-resident small-plane kernel: whole 7x7 layers and the bottom of pyramids whose planes
# reach 7x7 (channels-last tensors); odd channel and batch counts exercise the lane / warp masks.
@pytest.mark.parametrize("B,C,H,W,L,dtype", [
    (3, 40, 7, 7, 2, torch.float32), (5, 33, 7, 7, 1, torch.float32), (2, 64, 7, 7, 3, torch.float32),
    (9, 8, 7, 7, 2, torch.bfloat16), (2, 16, 14, 14, 3, torch.float32), (2, 9, 13, 14, 3, torch.float32),
    (1, 12, 28, 27, 4, torch.float32), (1, 8, 56, 56, 5, torch.float16), (1, 8, 55, 53, 4, torch.float32),
])
def test_emulated_register_resident_bottom(B, C, H, W, L, dtype):
    from oracle import wtconv_torch
    torch.manual_seed(B * 1000 + C * 10 + L)
    params = wtconv_torch.random_params(C, 5, L, ndim=2, bias=True)
    x = torch.randn(B, C, H, W).to(dtype).contiguous(memory_format=torch.channels_last)
    ref = wtconv_torch.wtconv2d_forward(x.double(), {k: v.double() for k, v in params.items()}).numpy()
    packed = emu_lib.pack(params, 2, C, 5, L)
    y, info = emu_lib.forward2d(x, packed, 5, L)
    assert info[4] == 1, f"the register-resident stage was not planned: {info}"
    assert info[5] == (1 if max(H, W) > 7 else 0), f"four-warp 14x14 stage: {info}"
    assert not torch.isnan(y.float()).any()
    tol = TOL[str(dtype).split(".")[1]]
    assert max_err(y.double().numpy(), ref) <= tol
    y2, info2 = emu_lib.forward2d(x, packed, 5, L, regplane=-1)
    assert info2[4] == 0
    assert max_err(y2.double().numpy(), ref) <= tol


# The adjoint parameter block (flipped taps, no bias) turns the forward kernels into the gradient
# of the input; checked against autograd through the oracle.
@pytest.mark.parametrize("ndim,shape,L,K", [(2, (2, 8, 14, 13), 3, 5), (2, (1, 4, 30, 17), 2, 3), (2, (1, 8, 56, 56), 5, 5),
                                            (1, (2, 4, 133), 3, 5)])
def test_emulated_input_gradient(ndim, shape, L, K):
    from oracle import wtconv_torch
    torch.manual_seed(sum(shape))
    C = shape[1]
    params = wtconv_torch.random_params(C, K, L, ndim=ndim, bias=True)
    x = torch.randn(shape, dtype=torch.float64, requires_grad=True)
    fn = wtconv_torch.wtconv2d_forward if ndim == 2 else wtconv_torch.wtconv1d_forward
    y = fn(x, {k: v.double() for k, v in params.items()})
    gy = torch.randn_like(y)
    (gx,) = torch.autograd.grad(y, x, gy)
    packed = emu_lib.pack(params, ndim, C, K, L, adjoint=True)
    g32 = gy.float()
    if ndim == 2:
        g32 = g32.contiguous(memory_format=torch.channels_last)
        out, _ = emu_lib.forward2d(g32, packed, K, L)
    else:
        out, _ = emu_lib.forward1d(g32, packed, K, L)
    assert max_err(out.double().numpy(), gx.numpy()) <= 1e-5


# Parameter gradients: pyramid, correlation-sum and per-parameter scaling kernels (emulated) against
# autograd through the oracle.
@pytest.mark.parametrize("shape,L,K,bias,layout", [((2, 5, 14, 13), 3, 5, True, "cl"), ((1, 4, 30, 17), 2, 3, False, "nchw"),
                                                    ((2, 33, 7, 7), 2, 5, True, "cl"), ((1, 3, 9, 20), 4, 7, True, "nchw")])
def test_emulated_parameter_gradients(shape, L, K, bias, layout):
    from oracle import wtconv_torch
    torch.manual_seed(sum(shape) + K)
    C = shape[1]
    params = wtconv_torch.random_params(C, K, L, ndim=2, bias=bias)
    for i in range(L):
        params[f"wavelet_scale.{i}.weight"].uniform_(0.05, 0.3)
    params["base_scale.weight"].uniform_(0.5, 1.5)
    pd = {k: v.double().requires_grad_(True) for k, v in params.items()}
    x = torch.randn(shape)
    y = wtconv_torch.wtconv2d_forward(x.double(), pd)
    gy = torch.randn(y.shape)
    names = ["base_conv.weight", "base_conv.bias", "base_scale.weight"]
    for i in range(L):
        names += [f"wavelet_convs.{i}.weight", f"wavelet_scale.{i}.weight"]
    have = [n for n in names if n in pd]
    ref = dict(zip(have, torch.autograd.grad(y, [pd[n] for n in have], gy.double())))
    xt, gt = x, gy
    if layout == "cl":
        xt = xt.contiguous(memory_format=torch.channels_last)
        gt = gt.contiguous(memory_format=torch.channels_last)
    stats = emu_lib.weight_grad_stats(xt, gt, K, L)
    assert not torch.isnan(stats).any()
    grads = emu_lib.param_grads(stats, params, names, 2, C, K, L)
    for n, gr in zip(names, grads):
        if n not in ref:
            assert gr is None
            continue
        err = float((gr.double() - ref[n]).abs().max() / ref[n].abs().max())
        assert err <= 1e-5, f"{n}: {err:.3e}"


def test_emulated_parameter_gradients_1d():
    """1-D layers reuse the 2-D kernels on the signal viewed as a one-row image."""
    from oracle import wtconv_torch
    torch.manual_seed(5)
    C, K, L = 6, 5, 3
    params = wtconv_torch.random_params(C, K, L, ndim=1, bias=True)
    pd = {k: v.double().requires_grad_(True) for k, v in params.items()}
    x = torch.randn(2, C, 133)
    y = wtconv_torch.wtconv1d_forward(x.double(), pd)
    gy = torch.randn(y.shape)
    names = ["base_conv.weight", "base_conv.bias", "base_scale.weight"]
    for i in range(L):
        names += [f"wavelet_convs.{i}.weight", f"wavelet_scale.{i}.weight"]
    ref = torch.autograd.grad(y, [pd[n] for n in names], gy.double())
    stats = emu_lib.weight_grad_stats(x.unsqueeze(2), gy.unsqueeze(2), K, L)
    grads = emu_lib.param_grads(stats, params, names, 1, C, K, L)
    for n, gr, r in zip(names, grads, ref):
        assert tuple(gr.shape) == tuple(r.shape), n
        err = float((gr.double() - r).abs().max() / r.abs().max())
        assert err <= 1e-5, f"{n}: {err:.3e}"


@pytest.mark.parametrize("seed", [11, 12, 13])
def test_emulated_random_configurations(seed):
    """Seeded sweep over kernel sizes, level counts, odd plane sizes, channel counts that do not fill a
    channel group, strides and the three input layouts, against the float64 evaluation of the oracle
    (fp32: normalised max error <= 1e-5).  The planner decides the chain, so the sweep reaches the
    whole-plane, tiled, direct-store, register-resident and four-warp stages."""
    import random
    from oracle import wtconv_torch
    rnd = random.Random(seed)
    chains = set()
    for it in range(120):
        K = rnd.choice([1, 3, 5, 5, 5, 7])
        L = rnd.choice([0, 1, 2, 3, 4, 5])
        kind = rnd.random()
        if kind < 0.4:
            base = rnd.choice([7, 14, 13, 27, 28, 55, 56])
            H, W = base - rnd.choice([0, 0, 1]), base - rnd.choice([0, 0, 1])
        elif kind < 0.92:
            H, W = rnd.randint(1, 70), rnd.randint(1, 70)
        else:
            H, W = rnd.randint(60, 160), rnd.randint(60, 160)
        C = rnd.choice([1, 3, 8, 9, 16, 24, 33, 40])
        B = rnd.choice([1, 2, 3])
        if B * C * H * W > 3e5:
            B, C = 1, min(C, 9)
        stride = rnd.choice([1, 1, 1, 2, 3])
        bias = rnd.random() < 0.8
        layout = rnd.choice(["nchw", "cl", "cl", "strided"])
        params = wtconv_torch.random_params(C, K, L, bias=bias, seed=seed * 1000 + it)
        x = torch.randn(B, C, H, W, generator=torch.Generator().manual_seed(seed * 1000 + it))
        xt = x
        if layout == "cl":
            xt = x.contiguous(memory_format=torch.channels_last)
        elif layout == "strided":
            big = torch.zeros(B, C, H + 3, W + 2)
            big[:, :, 1:H + 1, 2:W + 2] = x
            xt = big[:, :, 1:H + 1, 2:W + 2]
        packed = emu_lib.pack(params, 2, C, K, L)
        out, info = emu_lib.forward2d(xt, packed, K, L, stride=stride)
        ref = wtconv_torch.wtconv2d_forward(
            x.double(), {k: v.double() for k, v in params.items()}, stride=stride,
            filters=tuple(f.double() for f in wtconv_torch.haar_filters_2d(C))).float()
        case = (B, C, H, W, K, L, stride, bias, layout)
        assert tuple(out.shape) == tuple(ref.shape), case
        assert not torch.isnan(out).any(), case
        assert max_err(out.numpy(), ref.numpy()) <= 1e-5, case
        chains.add((info[0], info[1], info[4], info[5]))
    assert len(chains) >= 3          # more than one kind of launch chain was exercised


# Kernel sizes beyond the unrolled instances (1, 3, 5, 7) take the run-time-size instance of the
# CTA-tile kernels; the reference's CUDA backend accepts odd sizes up to 29
# (fast_wtconv/cuda_haar/haar_common.cuh:24-50), the pure-PyTorch reference any size.
@pytest.mark.parametrize("case", [
    (2, 3, 9, 2, (2, 3, 20, 17), 1, "nchw"), (2, 2, 11, 3, (1, 2, 40, 33), 1, "cl"), (2, 2, 29, 1, (1, 2, 30, 31), 1, "nchw"),
    (2, 4, 9, 2, (1, 4, 16, 16), 2, "cl"), (2, 2, 15, 3, (1, 2, 90, 70), 1, "nchw"),
    (1, 3, 9, 3, (2, 3, 100), 1, ""), (1, 2, 29, 2, (1, 2, 300), 3, ""), (1, 2, 13, 4, (1, 2, 257), 1, ""),
], ids=lambda c: f"{c[0]}d-K{c[2]}-L{c[3]}-s{c[5]}{c[6]}")
def test_emulated_run_time_kernel_size(case):
    from oracle import wtconv_torch
    nd, C, K, L, shape, stride, layout = case
    params = wtconv_torch.random_params(C, K, L, ndim=nd, seed=K + L)
    x = torch.randn(*shape, generator=torch.Generator().manual_seed(K))
    packed = emu_lib.pack(params, nd, C, K, L)
    p64 = {k: v.double() for k, v in params.items()}
    if nd == 2:
        xin = x.contiguous(memory_format=torch.channels_last) if layout == "cl" else x
        y, _ = emu_lib.forward2d(xin, packed, K, L, stride=stride)
        ref = wtconv_torch.wtconv2d_forward(x.double(), p64, stride=stride)
    else:
        y, _ = emu_lib.forward1d(x, packed, K, L, stride=stride)
        ref = wtconv_torch.wtconv1d_forward(x.double(), p64, stride=stride)
    assert tuple(y.shape) == tuple(ref.shape) and not torch.isnan(y).any()
    assert max_err(y.numpy(), ref.numpy()) <= 1e-5
