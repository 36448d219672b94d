"""Op-for-op torch restatement of the reference WTConv forward (CPU oracle).

TEST INFRASTRUCTURE -- see ``oracle/__init__.py``.

The functions take a plain ``dict`` of tensors keyed exactly like the
reference ``state_dict`` (``base_conv.weight``, ``base_conv.bias``,
``base_scale.weight``, ``wavelet_convs.<i>.weight``, ``wavelet_scale.<i>.weight``)
and run the same ATen operator sequence as the reference modules, so the
rounding points in reduced precision are the same as the reference's.

Reference anchors (paths inside the reference project):
  * filter bank ............ wtconv/util/wavelet.py:6-20 (1-D), :23-43 (2-D)
  * analysis / synthesis ... wtconv/util/wavelet.py:46-59 (1-D), :62-75 (2-D)
  * 2-D forward ............ wtconv/wtconv2d.py:38-87
  * 1-D forward ............ wtconv/wtconv1d.py:38-87
  * scale module ........... wtconv/wtconv2d.py:89-97
"""
from __future__ import annotations

import math
from typing import Dict, Optional

import torch
import torch.nn.functional as F

# db1 decomposition / reconstruction taps as PyWavelets 1.6.0 tabulates them
# (the reference reads them through ``pywt.Wavelet('db1')``,
# wtconv/util/wavelet.py:7,24).
_S = 1.0 / math.sqrt(2.0)
DB1 = dict(dec_lo=[_S, _S], dec_hi=[-_S, _S], rec_lo=[_S, _S], rec_hi=[_S, -_S])


def haar_filters_1d(channels: int, dtype=torch.float32):
    """(2C,1,2) analysis and synthesis banks, wtconv/util/wavelet.py:6-20."""
    lo_a = torch.tensor(DB1["dec_lo"][::-1], dtype=dtype)
    hi_a = torch.tensor(DB1["dec_hi"][::-1], dtype=dtype)
    lo_s = torch.tensor(DB1["rec_lo"], dtype=dtype)
    hi_s = torch.tensor(DB1["rec_hi"], dtype=dtype)
    ana = torch.stack([lo_a, hi_a])[:, None].repeat(channels, 1, 1)
    syn = torch.stack([lo_s, hi_s])[:, None].repeat(channels, 1, 1)
    return ana, syn


def haar_filters_2d(channels: int, dtype=torch.float32):
    """(4C,1,2,2) analysis and synthesis banks, wtconv/util/wavelet.py:23-43.

    Sub-band order LL, LH, HL, HH; the outer products are evaluated in
    ``dtype`` exactly like the reference does (fp32 taps come out as
    0.49999997, bf16 taps as 0.5).
    """
    lo_a = torch.tensor(DB1["dec_lo"][::-1], dtype=dtype)
    hi_a = torch.tensor(DB1["dec_hi"][::-1], dtype=dtype)
    lo_s = torch.tensor(DB1["rec_lo"], dtype=dtype)
    hi_s = torch.tensor(DB1["rec_hi"], dtype=dtype)

    def bank(lo, hi):
        rows = [lo[None, :] * lo[:, None], lo[None, :] * hi[:, None],
                hi[None, :] * lo[:, None], hi[None, :] * hi[:, None]]
        return torch.stack(rows)[:, None].repeat(channels, 1, 1, 1)

    return bank(lo_a, hi_a), bank(lo_s, hi_s)


def _levels(params: Dict[str, torch.Tensor]) -> int:
    n = 0
    while f"wavelet_convs.{n}.weight" in params:
        n += 1
    return n


def wtconv2d_forward(x: torch.Tensor, params: Dict[str, torch.Tensor], stride: int = 1,
                     filters: Optional[tuple] = None) -> torch.Tensor:
    """Reference 2-D forward, wtconv/wtconv2d.py:38-87, as a pure function."""
    c = x.shape[1]
    levels = _levels(params)
    if filters is None:
        ana, syn = haar_filters_2d(c, torch.float32)
        ana, syn = ana.to(x.device, x.dtype), syn.to(x.device, x.dtype)
    else:
        ana, syn = filters
    ksz = params["base_conv.weight"].shape[-1]

    low = x
    stash = []
    for i in range(levels):                                     # wtconv2d.py:46-62
        h, w = low.shape[2], low.shape[3]
        if (h % 2) or (w % 2):
            low = F.pad(low, (0, w % 2, 0, h % 2))              # right/bottom zeros
        sub = F.conv2d(low, ana, stride=2, groups=c)            # wavelet.py:62-67
        b, _, hh, ww = sub.shape
        low = sub.reshape(b, c, 4, hh, ww)[:, :, 0]             # raw LL goes down
        wt = params[f"wavelet_convs.{i}.weight"]
        sc = params[f"wavelet_scale.{i}.weight"]
        filt = F.conv2d(sub, wt, padding=ksz // 2, groups=4 * c)
        filt = torch.mul(sc, filt).reshape(b, c, 4, hh, ww)
        stash.append((filt, (h, w)))

    up = 0
    for filt, (h, w) in reversed(stash):                        # wtconv2d.py:64-78
        b, _, _, hh, ww = filt.shape
        merged = torch.cat([(filt[:, :, 0] + up).unsqueeze(2), filt[:, :, 1:4]], dim=2)
        up = F.conv_transpose2d(merged.reshape(b, 4 * c, hh, ww), syn, stride=2, groups=c)
        up = up[:, :, :h, :w]

    base = F.conv2d(x, params["base_conv.weight"], params.get("base_conv.bias"),
                    padding=ksz // 2, groups=c)
    y = torch.mul(params["base_scale.weight"], base) + up       # wtconv2d.py:81-82
    if stride > 1:                                              # AvgPool2d(kernel_size=1, stride)
        y = y[:, :, ::stride, ::stride]
    return y


def wtconv1d_forward(x: torch.Tensor, params: Dict[str, torch.Tensor], stride: int = 1,
                     filters: Optional[tuple] = None) -> torch.Tensor:
    """Reference 1-D forward, wtconv/wtconv1d.py:38-87, as a pure function."""
    c = x.shape[1]
    levels = _levels(params)
    if filters is None:
        ana, syn = haar_filters_1d(c, torch.float32)
        ana, syn = ana.to(x.device, x.dtype), syn.to(x.device, x.dtype)
    else:
        ana, syn = filters
    ksz = params["base_conv.weight"].shape[-1]

    low = x
    stash = []
    for i in range(levels):                                     # wtconv1d.py:46-62
        n = low.shape[2]
        if n % 2:
            low = F.pad(low, (0, 1))
        sub = F.conv1d(low, ana, stride=2, groups=c)            # wavelet.py:46-51
        b, _, half = sub.shape
        low = sub.reshape(b, c, 2, half)[:, :, 0]
        wt = params[f"wavelet_convs.{i}.weight"]
        sc = params[f"wavelet_scale.{i}.weight"]
        filt = torch.mul(sc, F.conv1d(sub, wt, padding=ksz // 2, groups=2 * c))
        stash.append((filt.reshape(b, c, 2, half), n))

    up = 0
    for filt, n in reversed(stash):                             # wtconv1d.py:64-78
        b, _, _, half = filt.shape
        merged = torch.cat([(filt[:, :, 0] + up).unsqueeze(2), filt[:, :, 1:2]], dim=2)
        up = F.conv_transpose1d(merged.reshape(b, 2 * c, half), syn, stride=2, groups=c)
        up = up[:, :, :n]

    base = F.conv1d(x, params["base_conv.weight"], params.get("base_conv.bias"),
                    padding=ksz // 2, groups=c)
    y = torch.mul(params["base_scale.weight"], base) + up
    if stride > 1:                                              # AvgPool1d(kernel=stride, stride)
        y = F.avg_pool1d(y, kernel_size=stride, stride=stride)
    return y


def random_params(channels: int, ksz: int, levels: int, ndim: int = 2, bias: bool = True,
                  seed: int = 0, dtype=torch.float32, scale_range=(0.05, 0.2)) -> Dict[str, torch.Tensor]:
    """Seeded synthetic parameters with the reference's shapes (wtconv2d.py:23-31)."""
    g = torch.Generator().manual_seed(seed)
    sub = 4 if ndim == 2 else 2
    kshape = (ksz, ksz) if ndim == 2 else (ksz,)
    ones = (1,) * ndim
    bound = 1.0 / math.sqrt(ksz ** ndim)

    def u(shape, lo, hi):
        return (torch.rand(shape, generator=g, dtype=torch.float32) * (hi - lo) + lo).to(dtype)

    p = {"base_conv.weight": u((channels, 1) + kshape, -bound, bound),
         "base_scale.weight": u((1, channels) + ones, 0.5, 1.5)}
    if bias:
        p["base_conv.bias"] = u((channels,), -bound, bound)
    for i in range(levels):
        p[f"wavelet_convs.{i}.weight"] = u((sub * channels, 1) + kshape, -bound, bound)
        p[f"wavelet_scale.{i}.weight"] = u((1, sub * channels) + ones, *scale_range)
    return p
