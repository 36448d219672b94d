"""Loader of the host emulation library (TEST INFRASTRUCTURE, see tests/emu/emu.cu).

Builds ``tests/emu/libwtconv_emu.so`` with nvcc (host code only) when it is
missing or older than the kernel sources, and wraps its entry points for torch
CPU tensors.  Nothing in the package imports this module.
"""
from __future__ import annotations

import ctypes
import glob
import os
import subprocess

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
SRC = os.path.join(HERE, "emu", "emu.cu")
LIB = os.path.join(HERE, "emu", "libwtconv_emu.so")
DTYPE_CODE = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}

_lib = None


def _stale():
    if not os.path.exists(LIB):
        return True
    deps = [SRC] + glob.glob(os.path.join(ROOT, "wtconv_b200", "csrc", "*.h")) \
        + glob.glob(os.path.join(ROOT, "wtconv_b200", "csrc", "*.cuh")) \
        + glob.glob(os.path.join(ROOT, "include", "*.h"))
    t = os.path.getmtime(LIB)
    return any(os.path.getmtime(d) > t for d in deps)


def build(force=False):
    """Builds under a file lock into a temporary name and renames it into place, so that test
    workers running side by side never load a half-written library."""
    if force or _stale():
        import fcntl
        with open(LIB + ".lock", "w") as lock:
            fcntl.flock(lock, fcntl.LOCK_EX)
            if force or _stale():
                tmp = f"{LIB}.{os.getpid()}.tmp"
                cmd = ["nvcc", "-O2", "-std=c++17", "-Wno-deprecated-gpu-targets", "-Xcompiler", "-fPIC", "-shared",
                       "-o", tmp, SRC]
                subprocess.run(cmd, check=True, cwd=os.path.dirname(SRC))
                os.replace(tmp, LIB)
    return LIB


def lib():
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(build())
        for name in ("emu_pack_params", "emu_wtconv2d_forward", "emu_wtconv1d_forward", "emu_force", "emu_regplane",
                     "emu_wtconv2d_pyramid", "emu_wtconv2d_weight_grad_stats", "emu_param_grads"):
            getattr(_lib, name).restype = ctypes.c_int
    return _lib


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else ctypes.c_void_p(0)


def taps(ndim, dtype):
    """Magnitude of one analysis / synthesis tap as a reference module of `dtype` holds it."""
    s = torch.tensor(2.0 ** -0.5, dtype=torch.float64).to(torch.float32)
    t = (s * s) if ndim == 2 else s
    t = t.to(dtype)
    return float(t), float(t)


def pack(params, ndim, C, K, L, param_dtype=torch.float32, filter_dtype=None, adjoint=False):
    p = {k: v.to(param_dtype).contiguous() for k, v in params.items()}
    sub = 4 if ndim == 2 else 2
    n = C * ((K ** ndim + 1 + 3) // 4 * 4) * (1 + sub * L)
    packed = torch.empty(n, dtype=torch.float32)
    ww = (ctypes.c_void_p * max(L, 1))(*[p[f"wavelet_convs.{i}.weight"].data_ptr() for i in range(L)])
    ws = (ctypes.c_void_p * max(L, 1))(*[p[f"wavelet_scale.{i}.weight"].data_ptr() for i in range(L)])
    ana, syn = taps(ndim, filter_dtype or param_dtype)
    st = lib().emu_pack_params(ndim, C, K, L, DTYPE_CODE[param_dtype], ctypes.c_double(ana), ctypes.c_double(syn),
                               _ptr(p["base_conv.weight"]), _ptr(p.get("base_conv.bias")),
                               _ptr(p["base_scale.weight"]), ww, ws, _ptr(packed), int(adjoint))
    assert st == 0
    return packed


def forward2d(x, packed, K, L, stride=1, force=(0, 0, 0), channels_last_out=None, regplane=0):
    """x: CPU tensor (B,C,H,W) in any strides; returns (y, info).  info = [stages, reductions,
    channel group and shared memory of the last stage, register-resident stages, ...];
    regplane=-1 plans without the register-resident small-plane kernel."""
    B, C, H, W = x.shape
    Ho, Wo = -(-H // stride), -(-W // stride)
    cl = x.stride(1) == 1 and C > 1 if channels_last_out is None else channels_last_out
    y = torch.full((B, C, Ho, Wo), float("nan"), dtype=x.dtype)
    if cl:
        y = y.contiguous(memory_format=torch.channels_last)
    xs = (ctypes.c_longlong * 4)(*x.stride())
    ys = (ctypes.c_longlong * 4)(*y.stride())
    info = (ctypes.c_int * 8)()
    lib().emu_force(*(tuple(force) + (0,) * (4 - len(force))))
    lib().emu_regplane(regplane)
    st = lib().emu_wtconv2d_forward(_ptr(x), _ptr(y), _ptr(packed), B, C, H, W, K, L, stride, DTYPE_CODE[x.dtype],
                                    xs, ys, info)
    lib().emu_force(0, 0, 0, 0)
    lib().emu_regplane(0)
    assert st == 0, f"emulation status {st}"
    return y, list(info)


def forward1d(x, packed, K, L, stride=1, force=(0, 0, 0)):
    B, C, N = x.shape
    y = torch.full((B, C, N // stride), float("nan"), dtype=x.dtype)
    xs = (ctypes.c_longlong * 3)(*x.stride())
    ys = (ctypes.c_longlong * 3)(*y.stride())
    info = (ctypes.c_int * 8)()
    lib().emu_force(*(tuple(force) + (0,) * (4 - len(force))))
    st = lib().emu_wtconv1d_forward(_ptr(x), _ptr(y), _ptr(packed), B, C, N, K, L, stride, DTYPE_CODE[x.dtype],
                                    xs, ys, info)
    lib().emu_force(0, 0, 0, 0)
    assert st == 0, f"emulation status {st}"
    return y, list(info)


def weight_grad_stats(x, gy, K, L, nsplit=2):
    """Correlation sums of the parameter gradients (emulated kernels): tensor (1+4L, K*K+1, C)."""
    B, C, H, W = x.shape
    n = 0
    h, w = H, W
    for _ in range(L):
        h, w = (h + 1) // 2, (w + 1) // 2
        n += B * h * w * 4 * C
    xp = torch.full((max(n, 1),), float("nan"), dtype=torch.float32)
    gp = torch.full((max(n, 1),), float("nan"), dtype=torch.float32)
    xs = (ctypes.c_longlong * 4)(*x.stride())
    gs = (ctypes.c_longlong * 4)(*gy.stride())
    code = DTYPE_CODE[x.dtype]
    assert lib().emu_wtconv2d_pyramid(_ptr(x), _ptr(xp), B, C, H, W, L, code, xs) == 0
    assert lib().emu_wtconv2d_pyramid(_ptr(gy), _ptr(gp), B, C, H, W, L, code, gs) == 0
    stats = torch.full((1 + 4 * L, K * K + 1, C), float("nan"), dtype=torch.float32)
    assert lib().emu_wtconv2d_weight_grad_stats(_ptr(x), _ptr(gy), _ptr(xp), _ptr(gp), _ptr(stats), B, C, H, W, K, L,
                                                code, xs, gs, nsplit) == 0
    return stats


def param_grads(stats, params, names, ndim, C, K, L):
    """Parameter gradients from the correlation sums (emulated wtconv_param_grads, fp32 parameters)."""
    p = [params[n].float().contiguous() if n in params else None for n in names]
    g = [torch.full_like(t, float("nan")) if t is not None else None for t in p]
    arr_t = ctypes.c_void_p * max(L, 1)
    ptrs = lambda ts, first: arr_t(*[ts[first + 2 * i].data_ptr() for i in range(L)])
    ana, syn = taps(ndim, torch.float32)
    st = lib().emu_param_grads(ndim, C, K, L, ctypes.c_double(ana), ctypes.c_double(syn), _ptr(stats),
                               _ptr(p[0]), _ptr(p[1]), _ptr(p[2]), ptrs(p, 3), ptrs(p, 4),
                               _ptr(g[0]), _ptr(g[1]), _ptr(g[2]), ptrs(g, 3), ptrs(g, 4))
    assert st == 0
    return g
