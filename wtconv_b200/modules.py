"""``WTConv2d`` / ``WTConv1d`` modules backed by the sm_100a kernels.

Drop-in replacements for the reference layers ``wtconv/wtconv2d.py:8-87`` and
``wtconv/wtconv1d.py:8-87``: same constructor signature and positional order,
same sub-module / parameter names and shapes (so ``state_dict`` round-trips with
``strict=True`` in both directions, ``wt_filter`` / ``iwt_filter`` included),
same seeded initialisation stream.  They plug into the reference model zoo
through its ``wtconv_class=`` hook (``wtconvnext/wtconvnext.py:76,105-114``).

Everything runs on CUDA only, in the kernels of ``libwtconv_b200.so``: there is no
PyTorch-op or CPU path.  ``WTConv2d`` is one autograd node (input gradient: the forward
kernels on the adjoint parameter block; parameter gradients: correlation sums between
sub-band pyramids, scaled per parameter by one more small kernel);
``WTConv1d`` uses the same kernels on the signal viewed as a one-row image.
"""
from __future__ import annotations

import ctypes
import math

import torch
import torch.nn as nn

from . import _lib

_DTYPE_CODE = {torch.float32: _lib.F32, torch.bfloat16: _lib.BF16, torch.float16: _lib.F16}
_SQRT_HALF = 1.0 / math.sqrt(2.0)
_EMPTY = object()   # call record of an input without elements
# db1 taps as PyWavelets tabulates them; the reference reads them through
# pywt.Wavelet (wtconv/util/wavelet.py:7,24) and supports nothing the table lacks.
_DB1 = dict(dec_lo=[_SQRT_HALF, _SQRT_HALF], dec_hi=[-_SQRT_HALF, _SQRT_HALF],
            rec_lo=[_SQRT_HALF, _SQRT_HALF], rec_hi=[_SQRT_HALF, -_SQRT_HALF])


def _filter_bank(ndim: int, channels: int):
    """Analysis / synthesis banks with the reference's values and shapes
    (wtconv/util/wavelet.py:6-20 for 1-D, :23-43 for 2-D).  They are kept only for
    ``state_dict`` compatibility; the kernels apply the Haar butterflies directly."""
    lo_a = torch.tensor(_DB1["dec_lo"][::-1], dtype=torch.float)
    hi_a = torch.tensor(_DB1["dec_hi"][::-1], dtype=torch.float)
    lo_s = torch.tensor(_DB1["rec_lo"], dtype=torch.float)
    hi_s = torch.tensor(_DB1["rec_hi"], dtype=torch.float)
    if ndim == 1:
        ana = torch.stack([lo_a, hi_a])[:, None].repeat(channels, 1, 1)
        syn = torch.stack([lo_s, hi_s])[:, None].repeat(channels, 1, 1)
        return ana, syn

    def bank(lo, hi):
        sub = [lo.unsqueeze(0) * lo.unsqueeze(1), lo.unsqueeze(0) * hi.unsqueeze(1),
               hi.unsqueeze(0) * lo.unsqueeze(1), hi.unsqueeze(0) * hi.unsqueeze(1)]
        return torch.stack(sub)[:, None].repeat(channels, 1, 1, 1)

    return bank(lo_a, hi_a), bank(lo_s, hi_s)


class _ScaleModule(nn.Module):
    """Per-channel scale, same state as the reference's (wtconv/wtconv2d.py:89-97).
    Its multiplication is folded into the packed kernel parameters."""

    def __init__(self, dims, init_scale=1.0, init_bias=0):
        super().__init__()
        self.dims = dims
        self.weight = nn.Parameter(torch.ones(*dims) * init_scale)
        self.bias = None

    def forward(self, x):
        return torch.mul(self.weight, x)


class _WTConvNd(nn.Module):
    _ndim = 2

    def __init__(self, in_channels, out_channels, kernel_size=5, stride=1, bias=True, wt_levels=1, wt_type='db1'):
        super().__init__()
        assert in_channels == out_channels
        if wt_type not in ('db1', 'haar'):
            raise NotImplementedError(f"only the db1/haar wavelet is implemented, got {wt_type!r}")
        nd = self._ndim
        conv = nn.Conv2d if nd == 2 else nn.Conv1d
        sub = 4 if nd == 2 else 2
        ones = [1] * nd

        self.in_channels = in_channels
        self.wt_levels = wt_levels
        self.stride = stride
        self.dilation = 1
        self.kernel_size = kernel_size

        ana, syn = _filter_bank(nd, in_channels)
        self.wt_filter = nn.Parameter(ana, requires_grad=False)
        self.iwt_filter = nn.Parameter(syn, requires_grad=False)

        self.base_conv = conv(in_channels, in_channels, kernel_size, padding='same', stride=1, dilation=1,
                              groups=in_channels, bias=bias)
        self.base_scale = _ScaleModule([1, in_channels] + ones)
        self.wavelet_convs = nn.ModuleList(
            [conv(in_channels * sub, in_channels * sub, kernel_size, padding='same', stride=1, dilation=1,
                  groups=in_channels * sub, bias=False) for _ in range(wt_levels)])
        self.wavelet_scale = nn.ModuleList(
            [_ScaleModule([1, in_channels * sub] + ones, init_scale=0.1) for _ in range(wt_levels)])

        if stride > 1:   # kept for attribute parity; the kernels apply the stride themselves
            self.do_stride = (nn.AvgPool2d(kernel_size=1, stride=stride) if nd == 2
                              else nn.AvgPool1d(kernel_size=stride, stride=stride))
        else:
            self.do_stride = None

        self._packed = {}
        self._packed_key = {}
        self._call_cache = {}

    # -- parameter folding -------------------------------------------------
    def _kernel_params(self):
        ps = [self.base_conv.weight, self.base_conv.bias, self.base_scale.weight]
        for conv, sc in zip(self.wavelet_convs, self.wavelet_scale):
            ps += [conv.weight, sc.weight]
        return ps

    def _param_key(self):
        """Identity of the parameter values: storage, address, in-place version, dtype."""
        ps = self._kernel_params()
        return tuple((p.untyped_storage()._cdata, p.data_ptr(), p._version) if p is not None else None for p in ps) \
            + (ps[0].dtype, self.wt_filter.dtype)

    def _replicate_for_data_parallel(self):
        # nn.DataParallel rebuilds its replicas on every forward: their parameters are fresh copies
        # (new addresses each time) of the master's.  A replica therefore keys its folded block on
        # the master's parameters; the cache dicts are shared with the master and hold one block
        # per device, so a device re-packs only after the master's parameters changed.
        replica = super()._replicate_for_data_parallel()
        replica._master_key = self._param_key()
        return replica

    def _packed_params(self, device, adjoint=False):
        """fp32 block of folded parameters (or of the adjoint layer: flipped taps, no bias), one per
        device, rebuilt only when a parameter changed (storage, address, in-place version or dtype)."""
        ps = self._kernel_params()
        key = getattr(self, "_master_key", None) or self._param_key()
        slot = (adjoint, device)
        cached = self._packed.get(slot)
        if cached is not None and key == self._packed_key.get(slot):
            packed, event, waited = cached
            # the block was written on the stream that was current at the time: other streams wait once
            sid = torch.cuda.current_stream(device).cuda_stream
            if sid not in waited and not torch.cuda.is_current_stream_capturing():
                torch.cuda.current_stream(device).wait_event(event)
                waited.add(sid)
            return packed
        lib = _lib.load()
        real = [p for p in ps if p is not None]
        pdt = real[0].dtype
        if pdt not in _DTYPE_CODE or any(p.dtype != pdt for p in real):
            raise TypeError("WTConv parameters must share one dtype out of float32 / bfloat16 / float16")
        if any(p.device != device for p in real):
            raise RuntimeError("WTConv parameters and input must live on the same CUDA device")
        nd, C, K, L = self._ndim, self.in_channels, self.kernel_size, self.wt_levels
        # keep contiguous views alive until the launch below has been enqueued
        hold = [p.detach().contiguous() if p is not None else None for p in ps]
        n = lib.wtconv_packed_param_floats(nd, C, K, L)
        packed = torch.empty(n, dtype=torch.float32, device=device)
        # tap magnitude exactly as a reference module of this dtype stores it in
        # wt_filter / iwt_filter (computed on the host: no device sync)
        s = torch.tensor(_SQRT_HALF, dtype=torch.float32)
        tap = float(((s * s) if nd == 2 else s).to(self.wt_filter.dtype))
        arr_t = ctypes.c_void_p * max(L, 1)
        ww = arr_t(*[hold[3 + 2 * i].data_ptr() for i in range(L)])
        ws = arr_t(*[hold[4 + 2 * i].data_ptr() for i in range(L)])
        with torch.cuda.device(device):
            cur = torch.cuda.current_stream(device)
            pack = lib.wtconv_pack_params_adjoint if adjoint else lib.wtconv_pack_params
            st = pack(nd, C, K, L, _DTYPE_CODE[pdt], tap, tap,
                      hold[0].data_ptr(), hold[1].data_ptr() if hold[1] is not None else None,
                      hold[2].data_ptr(), ww, ws, packed.data_ptr(), cur.cuda_stream)
            _lib.check(st, "wtconv_pack_params")
            event = torch.cuda.Event()
            event.record(cur)
        self._packed[slot], self._packed_key[slot] = (packed, event, {cur.cuda_stream}), key
        return packed

    def _check_input(self, x):
        if not x.is_cuda:
            raise RuntimeError("wtconv_b200 layers run only on CUDA tensors (sm_100a kernels, no CPU path)")
        if x.dtype not in _DTYPE_CODE:
            raise TypeError(f"unsupported activation dtype {x.dtype}; use float32, bfloat16 or float16")
        if x.dim() != self._ndim + 2 or x.shape[1] != self.in_channels:
            raise ValueError(f"expected a {self._ndim + 2}-D input with {self.in_channels} channels, got {tuple(x.shape)}")

    def forward(self, x):
        self._check_input(x)
        if torch.is_grad_enabled():
            ps = self._kernel_params()
            trainable = any(p is not None and p.requires_grad for p in ps)
            if trainable or x.requires_grad:
                return _WTConvFunction.apply(x, self, *[p for p in ps if p is not None])
        return self._run(x)

    def _param_grads(self, x, g):
        """Gradients of all parameters for input x and output gradient g (full resolution).  A 1-D
        signal is handed to the 2-D kernels as a one-row image."""
        lib = _lib.load()
        dev = x.device
        K, L, code = self.kernel_size, self.wt_levels, _DTYPE_CODE[x.dtype]
        if g.dtype != x.dtype:
            g = g.to(x.dtype)
        if self._ndim == 2:
            B, C, H, W = x.shape
            xstr, gstr = x.stride(), g.stride()
        else:
            B, C, W = x.shape
            H = 1
            xstr = (x.stride(0), x.stride(1), 0, x.stride(2))
            gstr = (g.stride(0), g.stride(1), 0, g.stride(2))
        n = lib.wtconv2d_pyramid_floats(B, C, H, W, L)
        xp = torch.empty(max(n, 1), dtype=torch.float32, device=dev)
        gp = torch.empty(max(n, 1), dtype=torch.float32, device=dev)
        stats = torch.empty((1 + 4 * L, K * K + 1, C), dtype=torch.float32, device=dev)
        xs = (ctypes.c_longlong * 4)(*xstr)
        gs = (ctypes.c_longlong * 4)(*gstr)
        with torch.cuda.device(dev):
            stream = torch.cuda.current_stream(dev).cuda_stream
            _lib.check(lib.wtconv2d_pyramid(x.data_ptr(), xp.data_ptr(), B, C, H, W, L, code, xs, stream),
                       "wtconv2d_pyramid")
            _lib.check(lib.wtconv2d_pyramid(g.data_ptr(), gp.data_ptr(), B, C, H, W, L, code, gs, stream),
                       "wtconv2d_pyramid")
            _lib.check(lib.wtconv2d_weight_grad_stats(x.data_ptr(), g.data_ptr(), xp.data_ptr(), gp.data_ptr(),
                                                      stats.data_ptr(), B, C, H, W, K, L, code, xs, gs, stream),
                       "wtconv2d_weight_grad_stats")
            ps = self._kernel_params()
            hold = [p.detach().contiguous() if p is not None else None for p in ps]
            grads = [torch.empty_like(h) if h is not None else None for h in hold]
            s = torch.tensor(_SQRT_HALF, dtype=torch.float32)
            tap = float(((s * s) if self._ndim == 2 else s).to(self.wt_filter.dtype))
            arr_t = ctypes.c_void_p * max(L, 1)
            ptrs = lambda ts, first: arr_t(*[ts[first + 2 * i].data_ptr() for i in range(L)])
            _lib.check(lib.wtconv_param_grads(
                self._ndim, C, K, L, _DTYPE_CODE[hold[0].dtype], tap, tap, stats.data_ptr(),
                hold[0].data_ptr(), hold[1].data_ptr() if hold[1] is not None else None, hold[2].data_ptr(),
                ptrs(hold, 3), ptrs(hold, 4),
                grads[0].data_ptr(), grads[1].data_ptr() if grads[1] is not None else None, grads[2].data_ptr(),
                ptrs(grads, 3), ptrs(grads, 4), stream), "wtconv_param_grads")
        return grads

    def _grad_to_full_resolution(self, gy, in_shape):
        """Adjoint of the output stride: the gradient of the layer output before the stride."""
        s = self.stride
        if s == 1:
            return gy
        full = gy.new_zeros(in_shape)
        if self._ndim == 2:
            full[..., ::s, ::s] = gy                       # wtconv2d.py:33-34: AvgPool2d(1, s) picks samples
        else:
            n = gy.shape[-1] * s                            # wtconv1d.py:34: AvgPool1d(s, s) averages s samples
            full[..., :n] = gy.repeat_interleave(s, dim=-1) / s
        return full


class _WTConvFunction(torch.autograd.Function):
    """The layer as one autograd node.  Input gradient: the Haar transform is orthogonal and odd sizes
    are padded and cropped at the same places, so the adjoint of the layer is the layer itself with
    every kernel flipped and the bias dropped -- one more forward call on the gradient, with the
    adjoint parameter block.  Parameter gradients: correlation sums between the sub-band
    pyramids of the input and of the output gradient (wtconv2d_weight_grad_stats), scaled per
    parameter by wtconv_param_grads."""

    @staticmethod
    def forward(ctx, x, module, *params):
        ctx.module = module
        ctx.in_shape = x.shape
        ctx.save_for_backward(x)
        return module._run(x)

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, gy):
        m = ctx.module
        (x,) = ctx.saved_tensors
        g = m._grad_to_full_resolution(gy, ctx.in_shape)
        gx = m._run(g, adjoint=True, stride=1) if ctx.needs_input_grad[0] else None
        nparam = len(ctx.needs_input_grad) - 2
        if not any(ctx.needs_input_grad[2:]):
            return (gx, None) + (None,) * nparam
        grads = m._param_grads(x, g)
        present = [gr for gr, p in zip(grads, m._kernel_params()) if p is not None]
        present = [gr if need else None for gr, need in zip(present, ctx.needs_input_grad[2:])]
        return (gx, None) + tuple(present)


class WTConv2d(_WTConvNd):
    """Wavelet convolution layer, forward on B200 (reference: wtconv/wtconv2d.py:8-87)."""
    _ndim = 2

    def _run(self, x, adjoint=False, stride=None):
        lib = _lib.load()
        dev = x.device
        s = self.stride if stride is None else stride
        # everything that depends only on the geometry of the call is computed once per
        # (shape, strides, dtype, stride): output layout, ctypes stride arrays, scratch size
        key = (tuple(x.shape), x.stride(), x.dtype, s)
        rec = self._call_cache.get(key)
        if rec is None:
            rec = self._call_cache[key] = self._plan_call(lib, x, s)
        if rec is _EMPTY:
            B, C, H, W = x.shape
            return x.new_empty((B, C, -(-H // s), -(-W // s)))
        make_contiguous, out_shape, out_format, xs, ys, nbytes, dims = rec
        if make_contiguous:
            x = x.contiguous()
        y = torch.empty(out_shape, dtype=x.dtype, device=dev, memory_format=out_format)
        packed = self._packed_params(dev, adjoint)
        ws = torch.empty(nbytes, dtype=torch.uint8, device=dev) if nbytes else None
        if torch.cuda.current_device() == dev.index:
            st = lib.wtconv2d_forward(x.data_ptr(), y.data_ptr(), packed.data_ptr(),
                                      ws.data_ptr() if ws is not None else None, nbytes, *dims, xs, ys,
                                      torch.cuda.current_stream(dev).cuda_stream)
        else:
            with torch.cuda.device(dev):
                st = lib.wtconv2d_forward(x.data_ptr(), y.data_ptr(), packed.data_ptr(),
                                          ws.data_ptr() if ws is not None else None, nbytes, *dims, xs, ys,
                                          torch.cuda.current_stream(dev).cuda_stream)
        if st:
            _lib.check(st, "wtconv2d_forward")
        return y

    def _plan_call(self, lib, x, s):
        B, C, H, W = x.shape
        if x.numel() == 0:
            return _EMPTY
        channels_last = x.is_contiguous(memory_format=torch.channels_last) and not x.is_contiguous()
        make_contiguous = not channels_last and not x.is_contiguous()
        if make_contiguous:
            x = x.contiguous()
        out_shape = (B, C, -(-H // s), -(-W // s))
        out_format = torch.channels_last if channels_last else torch.contiguous_format
        y = torch.empty(out_shape, dtype=x.dtype, device="meta", memory_format=out_format)
        K, L, code = self.kernel_size, self.wt_levels, _DTYPE_CODE[x.dtype]
        xs = (ctypes.c_longlong * 4)(*x.stride())
        ys = (ctypes.c_longlong * 4)(*y.stride())
        out = ctypes.c_size_t(0)
        _lib.check(lib.wtconv2d_workspace_bytes(B, C, H, W, K, L, code, xs, ys, ctypes.byref(out)),
                   "wtconv2d_workspace_bytes")
        if len(self._call_cache) > 64:
            self._call_cache.clear()
        return (make_contiguous, out_shape, out_format, xs, ys, int(out.value), (B, C, H, W, K, L, s, code))


class WTConv1d(_WTConvNd):
    """1-D wavelet convolution layer, forward on B200 (reference: wtconv/wtconv1d.py:8-87)."""
    _ndim = 1

    def _run(self, x, adjoint=False, stride=None):
        lib = _lib.load()
        B, C, N = x.shape
        s = self.stride if stride is None else stride
        y = torch.empty((B, C, N // s), dtype=x.dtype, device=x.device)
        if y.numel() == 0:
            return y
        if x.stride(2) != 1:
            x = x.contiguous()
        packed = self._packed_params(x.device, adjoint)
        xs = (ctypes.c_longlong * 3)(*x.stride())
        ys = (ctypes.c_longlong * 3)(*y.stride())
        with torch.cuda.device(x.device):
            stream = torch.cuda.current_stream(x.device).cuda_stream
            st = lib.wtconv1d_forward(x.data_ptr(), y.data_ptr(), packed.data_ptr(), B, C, N, self.kernel_size,
                                      self.wt_levels, s, _DTYPE_CODE[x.dtype], xs, ys, stream)
        _lib.check(st, "wtconv1d_forward")
        return y
