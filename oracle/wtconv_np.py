"""Closed-form float64 numpy restatement of the reference WTConv forward.

TEST INFRASTRUCTURE -- see ``oracle/__init__.py``.

Independent of ``oracle.wtconv_torch``: no convolution library call, only the
2x2 (resp. 2-tap) Haar butterflies and explicit shifted-add depthwise stencils
on arrays that are treated as zero outside their support.  This is the "truth"
run against which fp32 / bf16 error budgets are measured.

Reference anchors: wtconv/wtconv2d.py:38-87, wtconv/wtconv1d.py:38-87,
wtconv/util/wavelet.py:23-43 (sub-band order LL, LH, HL, HH and signs).
The taps are the exact 1/2 (2-D) and 1/sqrt(2) (1-D); the reference's fp32
filter bank holds 0.49999997 / 0.70710677, a relative difference of 6e-8 per
transform that is far inside the 1e-5 parity budget.
"""
from __future__ import annotations

import numpy as np


def _as64(t):
    if hasattr(t, "detach"):
        t = t.detach().to("cpu").double().numpy()
    return np.asarray(t, dtype=np.float64)


def _levels(params) -> int:
    n = 0
    while f"wavelet_convs.{n}.weight" in params:
        n += 1
    return n


def _dwconv2d(x, w):
    """Depthwise 'same' cross-correlation, zero outside: x (B,C,H,W), w (C,K,K)."""
    k = w.shape[-1]
    r = k // 2
    h, wd = x.shape[2], x.shape[3]
    xp = np.pad(x, ((0, 0), (0, 0), (r, r), (r, r)))
    out = np.zeros_like(x)
    for i in range(k):
        for j in range(k):
            out += w[None, :, i, j, None, None] * xp[:, :, i:i + h, j:j + wd]
    return out


def _dwconv1d(x, w):
    k = w.shape[-1]
    r = k // 2
    n = x.shape[2]
    xp = np.pad(x, ((0, 0), (0, 0), (r, r)))
    out = np.zeros_like(x)
    for j in range(k):
        out += w[None, :, j, None] * xp[:, :, j:j + n]
    return out


def wtconv2d_forward(x, params, stride: int = 1):
    """y = base_scale*(base_conv(x)+b) + sum over levels (wtconv2d.py:38-87)."""
    x = _as64(x)
    b, c, h, w = x.shape
    levels = _levels(params)
    low = x
    stash = []
    for i in range(levels):                                   # wtconv2d.py:46-62
        hh, ww = low.shape[2], low.shape[3]
        lp = np.pad(low, ((0, 0), (0, 0), (0, hh % 2), (0, ww % 2)))
        a, bq = lp[:, :, 0::2, 0::2], lp[:, :, 0::2, 1::2]
        cq, d = lp[:, :, 1::2, 0::2], lp[:, :, 1::2, 1::2]
        sub = [0.5 * (a + bq + cq + d), 0.5 * (a + bq - cq - d),
               0.5 * (a - bq + cq - d), 0.5 * (a - bq - cq + d)]
        wt = _as64(params[f"wavelet_convs.{i}.weight"])
        k = wt.shape[-1]
        wt = wt.reshape(c, 4, k, k)
        sc = _as64(params[f"wavelet_scale.{i}.weight"]).reshape(c, 4)
        filt = [sc[None, :, s, None, None] * _dwconv2d(sub[s], wt[:, s]) for s in range(4)]
        stash.append((filt, (hh, ww)))
        low = sub[0]                                           # raw LL goes down
    up = 0.0
    for filt, (hh, ww) in reversed(stash):                     # wtconv2d.py:64-78
        ll = filt[0] + up
        lh, hl, hhb = filt[1], filt[2], filt[3]
        rec = np.zeros(ll.shape[:2] + (2 * ll.shape[2], 2 * ll.shape[3]))
        rec[:, :, 0::2, 0::2] = 0.5 * (ll + lh + hl + hhb)
        rec[:, :, 0::2, 1::2] = 0.5 * (ll + lh - hl - hhb)
        rec[:, :, 1::2, 0::2] = 0.5 * (ll - lh + hl - hhb)
        rec[:, :, 1::2, 1::2] = 0.5 * (ll - lh - hl + hhb)
        up = rec[:, :, :hh, :ww]
    bw = _as64(params["base_conv.weight"]).reshape(c, *params["base_conv.weight"].shape[-2:])
    base = _dwconv2d(x, bw)
    if params.get("base_conv.bias") is not None:
        base = base + _as64(params["base_conv.bias"])[None, :, None, None]
    y = _as64(params["base_scale.weight"]).reshape(1, c, 1, 1) * base + up   # wtconv2d.py:81-82
    if stride > 1:
        y = y[:, :, ::stride, ::stride]
    return y


def wtconv1d_forward(x, params, stride: int = 1):
    """1-D twin (wtconv1d.py:38-87); stride is a true average pool (:34)."""
    x = _as64(x)
    b, c, n = x.shape
    levels = _levels(params)
    s2 = 1.0 / np.sqrt(2.0)
    low = x
    stash = []
    for i in range(levels):
        m = low.shape[2]
        lp = np.pad(low, ((0, 0), (0, 0), (0, m % 2)))
        a, bq = lp[:, :, 0::2], lp[:, :, 1::2]
        sub = [s2 * (a + bq), s2 * (a - bq)]
        wt = _as64(params[f"wavelet_convs.{i}.weight"])
        k = wt.shape[-1]
        wt = wt.reshape(c, 2, k)
        sc = _as64(params[f"wavelet_scale.{i}.weight"]).reshape(c, 2)
        filt = [sc[None, :, s, None] * _dwconv1d(sub[s], wt[:, s]) for s in range(2)]
        stash.append((filt, m))
        low = sub[0]
    up = 0.0
    for filt, m in reversed(stash):
        lo, hi = filt[0] + up, filt[1]
        rec = np.zeros(lo.shape[:2] + (2 * lo.shape[2],))
        rec[:, :, 0::2] = s2 * (lo + hi)
        rec[:, :, 1::2] = s2 * (lo - hi)
        up = rec[:, :, :m]
    bw = _as64(params["base_conv.weight"]).reshape(c, -1)
    base = _dwconv1d(x, bw)
    if params.get("base_conv.bias") is not None:
        base = base + _as64(params["base_conv.bias"])[None, :, None]
    y = _as64(params["base_scale.weight"]).reshape(1, c, 1) * base + up
    if stride > 1:
        nout = y.shape[2] // stride
        y = y[:, :, :nout * stride].reshape(b, c, nout, stride).mean(axis=3)
    return y
