"""Parity at the full benchmark sizes: the launches the benchmark times are the launches checked.

The CUDA path runs the whole problem (all samples, all channels); the CPU oracle is run on a
subset small enough to finish in seconds -- whole samples for the stage layers and the 1-D layer,
a channel slice for the 512 x 512 layer (every operator of the layer is depthwise, so a channel
slice of the output depends on the same slice of the input and of the parameters only).

Tolerances (normalised max error): 1e-5 for fp32 against the float64 oracle; 2e-2 for bf16 against
the oracle run in bf16 (the reference's own rounding), and 5e-3 against the float64 oracle on the
bf16-rounded inputs and parameters (fp32 arithmetic on 16-bit storage).
"""
import numpy as np
import pytest
import torch

from conftest import max_err
from oracle import wtconv_np, wtconv_torch

pytestmark = pytest.mark.gpu

STAGES = [(96, 56, 5), (192, 28, 4), (384, 14, 3), (768, 7, 2)]   # WTConvNeXt-T (C, H=W, wt_levels)


def _cuda():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    return torch.device("cuda:0")


def _module(ndim, C, L, params, dtype, dev):
    import wtconv_b200
    cls = wtconv_b200.WTConv2d if ndim == 2 else wtconv_b200.WTConv1d
    m = cls(C, C, kernel_size=5, wt_levels=L, bias=True)
    sd = m.state_dict()
    for k, v in params.items():
        sd[k] = v.reshape(sd[k].shape).float()
    m.load_state_dict(sd, strict=True)
    return m.to(dev).to(dtype).eval()


def _check(out, x, params, dtype, ndim=2):
    """out, x: CPU tensors of the same samples / channels; params: fp32 parameters of those channels."""
    np_fwd = wtconv_np.wtconv2d_forward if ndim == 2 else wtconv_np.wtconv1d_forward
    th_fwd = wtconv_torch.wtconv2d_forward if ndim == 2 else wtconv_torch.wtconv1d_forward
    p_dt = {k: v.to(dtype) for k, v in params.items()}
    truth = np_fwd(x.to(dtype).double(), {k: v.double() for k, v in p_dt.items()})
    got = out.float().numpy()
    if dtype == torch.float32:
        assert max_err(got, truth) <= 1e-5
        return
    with torch.no_grad():
        ref = th_fwd(x.to(dtype), p_dt).float().numpy()
    assert max_err(got, ref) <= 2e-2
    assert max_err(got, truth) <= 5e-3


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32], ids=["bf16", "f32"])
@pytest.mark.parametrize("stage", range(4))
def test_stage_layers_at_batch_128(stage, dtype):
    """The four benchmark launches (B=128, channels-last): samples 0, 1, 77 and 127, every channel,
    against the oracle; the other samples through the batch independence of the layer (the two
    halves of the batch, run as launches of their own, must reproduce the whole bit for bit)."""
    dev = _cuda()
    C, H, L = STAGES[stage]
    params = wtconv_torch.random_params(C, 5, L, seed=100 + stage)
    g = torch.Generator().manual_seed(900 + stage)
    x = torch.randn(128, C, H, H, generator=g)
    m = _module(2, C, L, params, dtype, dev)
    xd = x.to(dev).to(dtype).contiguous(memory_format=torch.channels_last)
    with torch.no_grad():
        y = m(xd)
        halves = torch.cat([m(xd[:64]), m(xd[64:])])
    assert y.shape == xd.shape and y.dtype == dtype and y.is_contiguous(memory_format=torch.channels_last)
    assert torch.isfinite(y.float()).all()
    assert torch.equal(y, halves)
    idx = [0, 1, 77, 127]
    _check(y[idx].cpu(), x[idx], params, dtype)


def test_odd_batch_with_two_slots_per_cta():
    """Stage-2 shape at batch 129: the deep stage packs two samples per CTA, so its last CTA owns a
    sample slot beyond the batch (its sub-band box is all out-of-bounds fill and nothing is stored)."""
    dev = _cuda()
    C, H, L = STAGES[1]
    params = wtconv_torch.random_params(C, 5, L, seed=101)
    x = torch.randn(129, C, H, H, generator=torch.Generator().manual_seed(77))
    m = _module(2, C, L, params, torch.bfloat16, dev)
    with torch.no_grad():
        y = m(x.to(dev).to(torch.bfloat16).contiguous(memory_format=torch.channels_last))
    assert torch.isfinite(y.float()).all()
    idx = [0, 127, 128]
    _check(y[idx].cpu(), x[idx], params, torch.bfloat16)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("shape,L", [((1, 16, 300, 261), 6), ((2, 8, 130, 257), 4), ((1, 32, 224, 224), 5), ((1, 24, 97, 140), 3)])
def test_large_channels_last_planes(shape, L, dtype):
    """Planes whose deeper sub-bands do not fit on chip: low-pass plane kernel, one level stage per
    level, deep stage for the rest (odd sizes at every level, channel counts that do not fill a group)."""
    dev = _cuda()
    B, C, H, W = shape
    params = wtconv_torch.random_params(C, 5, L, seed=H + L)
    x = torch.randn(*shape, generator=torch.Generator().manual_seed(W))
    m = _module(2, C, L, params, dtype, dev)
    with torch.no_grad():
        y = m(x.to(dev).to(dtype).contiguous(memory_format=torch.channels_last))
    assert y.shape == x.shape and y.is_contiguous(memory_format=torch.channels_last)
    _check(y.cpu(), x, params, dtype)


@pytest.mark.parametrize("layout", ["cl", "nchw"])
def test_segmentation_layer_512(layout):
    """BASELINE config 4: WTConv2d(256,256,5,wt_levels=5) on (2,256,512,512) bf16, both layouts; the
    oracle runs on the eight channels 0-3 and 252-255 of both samples."""
    dev = _cuda()
    C, L = 256, 5
    params = wtconv_torch.random_params(C, 5, L, seed=400)
    g = torch.Generator().manual_seed(401)
    x = torch.randn(2, C, 512, 512, generator=g)
    m = _module(2, C, L, params, torch.bfloat16, dev)
    xd = x.to(dev).to(torch.bfloat16)
    if layout == "cl":
        xd = xd.contiguous(memory_format=torch.channels_last)
    with torch.no_grad():
        y = m(xd)
    assert y.shape == xd.shape
    if layout == "cl":
        assert y.is_contiguous(memory_format=torch.channels_last)
    assert torch.isfinite(y.float()).all()
    ch = torch.tensor([0, 1, 2, 3, 252, 253, 254, 255])

    def cut(name, v):          # the slice of a parameter that belongs to channels `ch`
        if name.startswith("wavelet"):      # (4C, ...) or (1, 4C, ...): sub-bands of channel c are 4c..4c+3
            sub = (ch[:, None] * 4 + torch.arange(4)[None, :]).reshape(-1)
            return v.index_select(1 if v.shape[0] == 1 else 0, sub)
        return v.index_select(1 if (v.dim() > 1 and v.shape[0] == 1) else 0, ch)
    p8 = {k: cut(k, v) for k, v in params.items()}
    _check(y.index_select(1, ch.to(dev)).cpu(), x.index_select(1, ch), p8, torch.bfloat16)


@pytest.mark.parametrize("N", [4096, 4097])
def test_wtconv1d_at_batch_512(N):
    """BASELINE config 5: WTConv1d(64,64,5,wt_levels=4) on (512,64,N) fp32, sums of sinusoids plus
    noise; samples 0, 1, 255 and 511 against the float64 oracle, the rest through batch independence."""
    dev = _cuda()
    C, L, B = 64, 4, 512
    params = wtconv_torch.random_params(C, 5, L, ndim=1, seed=500)
    g = torch.Generator().manual_seed(502)
    t = torch.arange(N, dtype=torch.float32)
    amp = torch.rand(B, C, 4, generator=g) + 0.5
    frq = torch.rand(B, C, 4, generator=g) * 63 + 1
    phs = torch.rand(B, C, 4, generator=g) * 2 * np.pi
    x = torch.zeros(B, C, N)
    for j in range(4):
        x += amp[:, :, j:j + 1] * torch.sin(2 * np.pi * frq[:, :, j:j + 1] * t / N + phs[:, :, j:j + 1])
    x += 0.1 * torch.randn(B, C, N, generator=g)
    m = _module(1, C, L, params, torch.float32, dev)
    xd = x.to(dev)
    with torch.no_grad():
        y = m(xd)
        halves = torch.cat([m(xd[:256]), m(xd[256:])])
    assert y.shape == xd.shape and torch.isfinite(y).all()
    assert torch.equal(y, halves)
    idx = [0, 1, 255, 511]
    _check(y[idx].cpu(), x[idx], params, torch.float32, ndim=1)


def test_device_status_word_is_clear_after_the_tma_fed_kernels():
    """The bounded waits of the TMA-fed kernels report through wtconv_device_status; after ordinary
    launches of the channels-last chain the word must read zero."""
    dev = _cuda()
    from wtconv_b200 import _lib
    lib = _lib.load()
    params = wtconv_torch.random_params(96, 5, 5, seed=100)
    m = _module(2, 96, 5, params, torch.bfloat16, dev)
    x = torch.randn(8, 96, 56, 56, device=dev, dtype=torch.bfloat16).contiguous(memory_format=torch.channels_last)
    with torch.no_grad():
        m(x)
    assert lib.wtconv_device_status(torch.cuda.current_stream().cuda_stream) == 0
