"""GPU parity of the CUDA path (through the Python modules, i.e. through the C ABI)
against the CPU oracles and the golden vectors of the reference.

Tolerances (normalised max error max|y-ref|/max|ref|): 1e-5 for fp32, 2e-2 for
bf16 / fp16 -- the bounds the layer's specification states.
"""
import numpy as np
import pytest
import torch

from conftest import GOLDEN_DIR, golden_names, load_golden, max_err
from oracle import wtconv_np, wtconv_torch

pytestmark = pytest.mark.gpu

TOL = {torch.float32: 1e-5, torch.bfloat16: 2e-2, torch.float16: 2e-2}


def _cuda():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    return torch.device("cuda:0")


def _module(ndim, C, K, L, stride, bias, params, dtype, dev):
    import wtconv_b200
    cls = wtconv_b200.WTConv2d if ndim == 2 else wtconv_b200.WTConv1d
    m = cls(C, C, kernel_size=K, stride=stride, bias=bias, wt_levels=L)
    sd = m.state_dict()
    for k, v in params.items():
        if "filter" in k:
            continue
        sd[k] = torch.as_tensor(v).reshape(sd[k].shape).float()
    m.load_state_dict(sd, strict=True)
    return m.to(dev).to(dtype).eval()


def _oracle(ndim, x, params, stride, dtype=torch.float32):
    fn = wtconv_torch.wtconv2d_forward if ndim == 2 else wtconv_torch.wtconv1d_forward
    p = {k: torch.as_tensor(v).to(dtype) for k, v in params.items() if "filter" not in k}
    with torch.no_grad():
        return fn(x.to(dtype), p, stride=stride)


@pytest.mark.parametrize("layout", ["nchw", "cl"])
@pytest.mark.parametrize("name", golden_names())
def test_golden_vectors(name, layout):
    dev = _cuda()
    x, params, y, meta = load_golden(name)
    if meta["ndim"] == 1 and layout == "cl":
        pytest.skip("1-D has a single layout")
    dt = getattr(torch, meta["dtype"])
    m = _module(meta["ndim"], meta["C"], meta["K"], meta["L"], meta["stride"], meta["bias"], params, dt, dev)
    xt = torch.from_numpy(x).to(dev).to(dt)
    if layout == "cl":
        xt = xt.contiguous(memory_format=torch.channels_last)
    with torch.no_grad():
        out = m(xt)
    assert tuple(out.shape) == y.shape and out.dtype == dt
    if layout == "cl" and meta["C"] > 1 and min(y.shape[2:]) > 1:
        assert out.is_contiguous(memory_format=torch.channels_last)
    assert max_err(out.float().cpu().numpy(), y) <= TOL[dt]


def test_config1_exact_recipe():
    """BASELINE config 1: WTConv2d(32,32,5,wt_levels=3), seed 0, x (8,32,56,56) fp32, NCHW."""
    dev = _cuda()
    import wtconv_b200
    z = np.load(f"{GOLDEN_DIR}/cfg1.npz")
    torch.manual_seed(0)
    m = wtconv_b200.WTConv2d(32, 32, kernel_size=5, wt_levels=3, bias=True)   # same init stream as the reference
    x = torch.randn(8, 32, 56, 56)
    for k in z.files:
        if k.startswith("p:"):
            assert np.array_equal(m.state_dict()[k[2:]].numpy(), z[k]), f"init stream differs at {k}"
    with torch.no_grad():
        y = m.to(dev)(x.to(dev)).cpu()
    assert max_err(y[0, :4].numpy(), z["y_slice"]) <= 1e-5
    assert max_err(y[:, :, 17, :].numpy(), z["y_rows"]) <= 1e-5
    assert max_err(y[0, :4].numpy(), z["y64_slice"]) <= 1e-5
    ys = np.array([y.double().sum().item(), y.double().pow(2).sum().item(), y.abs().max().item()])
    assert np.allclose(ys, z["y_stats"], rtol=1e-5)


STAGES = [(96, 56, 5), (192, 28, 4), (384, 14, 3), (768, 7, 2)]   # WTConvNeXt-T (C, H=W, wt_levels)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("stage", range(4))
def test_config2_stage_shapes(stage, dtype):
    """BASELINE config 2 shapes at batch 2, channels-last; bf16/fp16 are checked against the
    same-dtype oracle (reference rounding) and against the float64 truth."""
    dev = _cuda()
    C, H, L = STAGES[stage]
    params = wtconv_torch.random_params(C, 5, L, seed=100 + stage)
    g = torch.Generator().manual_seed(200 + stage)
    x = torch.randn(2, C, H, H, generator=g)
    m = _module(2, C, 5, L, 1, True, params, dtype, dev)
    xt = x.to(dev).to(dtype).contiguous(memory_format=torch.channels_last)
    with torch.no_grad():
        out = m(xt).float().cpu()
    p_dt = {k: v.to(dtype) for k, v in params.items()}
    truth = wtconv_np.wtconv2d_forward(x.to(dtype).double(), {k: v.double() for k, v in p_dt.items()})
    if dtype == torch.float32:
        assert max_err(out.numpy(), truth) <= 1e-5
    else:
        ref = _oracle(2, x, params, 1, dtype).float()
        assert max_err(out.numpy(), ref.numpy()) <= TOL[dtype]
        # fp32 math on low-precision storage: closer to the truth than the same-dtype reference is
        assert max_err(out.numpy(), truth) <= max(max_err(ref.numpy(), truth), 5e-3)


def _rand_cases(n, seed):
    rng = np.random.RandomState(seed)
    cases = []
    for _ in range(n):
        K = int(rng.choice([1, 3, 5, 5, 5, 7]))
        L = int(rng.randint(0, 6))
        C = int(rng.choice([1, 2, 3, 4, 5, 8, 12, 16, 24]))
        H, W = int(rng.randint(1, 41)), int(rng.randint(1, 41))
        B = int(rng.randint(1, 4))
        stride = int(rng.choice([1, 1, 1, 2, 3]))
        bias = bool(rng.randint(0, 2))
        layout = str(rng.choice(["nchw", "cl", "strided"]))
        dtype = [torch.float32, torch.float32, torch.bfloat16, torch.float16][int(rng.randint(0, 4))]
        cases.append((B, C, H, W, K, L, stride, bias, layout, dtype))
    return cases


@pytest.mark.parametrize("case", _rand_cases(48, 7), ids=lambda c: "-".join(str(v).replace("torch.", "") for v in c))
def test_random_shapes_2d(case):
    dev = _cuda()
    B, C, H, W, K, L, stride, bias, layout, dtype = case
    params = wtconv_torch.random_params(C, K, L, bias=bias, seed=B * 1000 + H * 10 + W)
    g = torch.Generator().manual_seed(H * 100 + W)
    x = torch.randn(B, C, H, W, generator=g)
    m = _module(2, C, K, L, stride, bias, params, dtype, dev)
    xt = x.to(dev).to(dtype)
    if layout == "cl":
        xt = xt.contiguous(memory_format=torch.channels_last)
    elif layout == "strided":
        big = torch.zeros(B, C, H + 3, W + 2, device=dev, dtype=dtype)
        big[:, :, 1:H + 1, 2:W + 2] = xt
        xt = big[:, :, 1:H + 1, 2:W + 2]
    with torch.no_grad():
        out = m(xt)
    ref = _oracle(2, x, params, stride, dtype if dtype != torch.float32 else torch.float64).float()
    assert tuple(out.shape) == tuple(ref.shape)
    assert max_err(out.float().cpu().numpy(), ref.numpy()) <= TOL[dtype]


# Pyramids whose planes reach 7x7 take the register-resident kernel at the bottom (channels-last):
# odd channel counts and batch sizes exercise its lane and warp masks, stride 2 its fallback.
@pytest.mark.parametrize("B,C,H,W,L,stride,dtype", [
    (5, 40, 7, 7, 2, 1, torch.float32), (131, 33, 7, 7, 1, 1, torch.float32), (2, 64, 7, 7, 3, 1, torch.bfloat16),
    (3, 72, 14, 14, 3, 1, torch.float32), (2, 9, 13, 14, 3, 1, torch.float16), (3, 100, 28, 27, 4, 1, torch.float32),
    (2, 24, 56, 56, 5, 1, torch.bfloat16), (4, 16, 7, 7, 2, 2, torch.float32), (2, 8, 55, 53, 4, 2, torch.float32),
])
def test_register_resident_bottom(B, C, H, W, L, stride, dtype):
    dev = _cuda()
    params = wtconv_torch.random_params(C, 5, L, bias=True, seed=B + C + H)
    g = torch.Generator().manual_seed(C * 100 + W)
    x = torch.randn(B, C, H, W, generator=g)
    m = _module(2, C, 5, L, stride, True, params, dtype, dev)
    xt = x.to(dev).to(dtype).contiguous(memory_format=torch.channels_last)
    with torch.no_grad():
        out = m(xt)
    ref = _oracle(2, x, params, stride, dtype if dtype != torch.float32 else torch.float64).float()
    assert tuple(out.shape) == tuple(ref.shape)
    assert not torch.isnan(out.float()).any()
    assert max_err(out.float().cpu().numpy(), ref.numpy()) <= TOL[dtype]


@pytest.mark.parametrize("shape,L", [((1, 8, 200, 264), 5), ((2, 4, 131, 77), 4), ((1, 16, 96, 300), 6)])
@pytest.mark.parametrize("layout", ["nchw", "cl"])
def test_large_planes_use_the_tiled_chain(shape, L, layout):
    """Planes that do not fit on chip run as a chain of tiled stages through scratch memory."""
    dev = _cuda()
    B, C, H, W = shape
    params = wtconv_torch.random_params(C, 5, L, seed=H + W)
    g = torch.Generator().manual_seed(H * W)
    x = torch.randn(shape, generator=g)
    m = _module(2, C, 5, L, 1, True, params, torch.float32, dev)
    xt = x.to(dev)
    if layout == "cl":
        xt = xt.contiguous(memory_format=torch.channels_last)
    with torch.no_grad():
        out = m(xt).cpu()
    ref = _oracle(2, x, params, 1, torch.float64)
    assert max_err(out.numpy(), ref.numpy()) <= 1e-5


@pytest.mark.parametrize("N", [4096, 4097, 1000, 37])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_config5_1d(N, dtype):
    """BASELINE config 5 shapes (C=64, K=5, 4 levels, even and odd length) at batch 4, sinusoid input."""
    dev = _cuda()
    C, L = 64, 4
    params = wtconv_torch.random_params(C, 5, L, ndim=1, seed=500)
    g = torch.Generator().manual_seed(501)
    t = torch.arange(N, dtype=torch.float64)
    amp = torch.rand(4, C, 4, generator=g, dtype=torch.float64) + 0.5
    frq = torch.rand(4, C, 4, generator=g, dtype=torch.float64) * 63 + 1
    phs = torch.rand(4, C, 4, generator=g, dtype=torch.float64) * 2 * np.pi
    x = (amp[..., None] * torch.sin(2 * np.pi * frq[..., None] * t / N + phs[..., None])).sum(2)
    x = (x + 0.1 * torch.randn(4, C, N, generator=g, dtype=torch.float64)).float()
    m = _module(1, C, 5, L, 1, True, params, dtype, dev)
    with torch.no_grad():
        out = m(x.to(dev).to(dtype)).float().cpu()
    ref = _oracle(1, x, params, 1, dtype if dtype != torch.float32 else torch.float64).float()
    assert max_err(out.numpy(), ref.numpy()) <= TOL[dtype]


@pytest.mark.parametrize("case", [(3, 5, 100, 3, 3, 3), (2, 7, 513, 7, 5, 2), (1, 1, 9, 5, 6, 1), (2, 16, 2500, 5, 8, 4)])
def test_random_shapes_1d(case):
    dev = _cuda()
    B, C, N, K, L, stride = case
    params = wtconv_torch.random_params(C, K, L, ndim=1, seed=N)
    x = torch.randn(B, C, N, generator=torch.Generator().manual_seed(N + 1))
    m = _module(1, C, K, L, stride, True, params, torch.float32, dev)
    with torch.no_grad():
        out = m(x.to(dev)).cpu()
    ref = _oracle(1, x, params, stride, torch.float64)
    assert tuple(out.shape) == tuple(ref.shape)
    assert max_err(out.numpy(), ref.numpy()) <= 1e-5


# ---------------------------------------------------------------------------
# size-independent properties at the full BASELINE sizes
# ---------------------------------------------------------------------------

def _stage1_module(dev, dtype):
    params = wtconv_torch.random_params(96, 5, 5, seed=101)
    return _module(2, 96, 5, 5, 1, True, params, dtype, dev), params


def test_full_size_shards_equal_whole_and_deterministic():
    """Batch shards are independent (depthwise everywhere): running 128 samples at once,
    twice, and as four shards of 32 must give bit-identical outputs."""
    dev = _cuda()
    m, _ = _stage1_module(dev, torch.bfloat16)
    x = torch.randn(128, 96, 56, 56, device=dev, dtype=torch.bfloat16).contiguous(memory_format=torch.channels_last)
    with torch.no_grad():
        whole = m(x)
        again = m(x)
        parts = torch.cat([m(x[i:i + 32]) for i in range(0, 128, 32)])
    assert torch.equal(whole, again)
    assert torch.equal(whole, parts)


def test_full_size_sample_against_oracle():
    """Full config-2 stage-1 launch (B=128, bf16, channels-last); two samples checked on the CPU."""
    dev = _cuda()
    m, params = _stage1_module(dev, torch.bfloat16)
    g = torch.Generator().manual_seed(9)
    x = torch.randn(128, 96, 56, 56, generator=g).to(torch.bfloat16)
    with torch.no_grad():
        y = m(x.to(dev).contiguous(memory_format=torch.channels_last)).float().cpu()
    for n in (0, 127):
        ref = _oracle(2, x[n:n + 1].float(), params, 1, torch.bfloat16).float()
        assert max_err(y[n:n + 1].numpy(), ref.numpy()) <= 2e-2


def test_full_size_linearity_fp32():
    """The layer is affine in x: f(a*x1 + x2) - f(0) == a*(f(x1)-f(0)) + (f(x2)-f(0))."""
    dev = _cuda()
    m, _ = _stage1_module(dev, torch.float32)
    x1 = torch.randn(32, 96, 56, 56, device=dev).contiguous(memory_format=torch.channels_last)
    x2 = torch.randn_like(x1)
    with torch.no_grad():
        f0 = m(torch.zeros_like(x1))
        lhs = m(0.5 * x1 + x2) - f0
        rhs = 0.5 * (m(x1) - f0) + (m(x2) - f0)
    assert max_err(lhs.cpu().numpy(), rhs.cpu().numpy()) <= 1e-5


@pytest.mark.parametrize("shape,L", [((4, 96, 56, 56), 5), ((3, 8, 57, 33), 4), ((2, 4, 7, 7), 2), ((1, 2, 300, 130), 5)])
def test_perfect_reconstruction(shape, L):
    """base_scale = 0 and identity (delta) sub-band kernels with unit scale: the cascade is
    analysis followed by synthesis and must return x, odd sizes included."""
    dev = _cuda()
    B, C, H, W = shape
    import wtconv_b200
    m = wtconv_b200.WTConv2d(C, C, kernel_size=5, wt_levels=L).to(dev).eval()
    with torch.no_grad():
        m.base_scale.weight.zero_()
        for conv, sc in zip(m.wavelet_convs, m.wavelet_scale):
            conv.weight.zero_()
            conv.weight[:, 0, 2, 2] = 1.0
            sc.weight.fill_(1.0)
            # only the deepest level passes its low band on unchanged; shallower low bands
            # are replaced by the reconstruction coming from below
        for i in range(L - 1):
            m.wavelet_convs[i].weight[0::4] = 0.0
        x = torch.randn(shape, device=dev)
        y = m(x)
    assert max_err(y.cpu().numpy(), x.cpu().numpy()) <= 1e-5


def test_zero_wavelet_scale_leaves_base_path():
    """wavelet_scale = 0  =>  y = base_scale * (depthwise conv(x) + bias); checked against cuDNN."""
    dev = _cuda()
    import wtconv_b200
    m = wtconv_b200.WTConv2d(24, 24, kernel_size=7, wt_levels=3).to(dev).eval()
    with torch.no_grad():
        for sc in m.wavelet_scale:
            sc.weight.zero_()
        m.base_scale.weight.uniform_(0.5, 1.5)
        x = torch.randn(3, 24, 29, 31, device=dev)
        y = m(x)
        ref = m.base_scale.weight * torch.nn.functional.conv2d(x.double(), m.base_conv.weight.double(),
                                                               m.base_conv.bias.double(), padding=3, groups=24)
    assert max_err(y.cpu().numpy(), ref.cpu().numpy()) <= 1e-5


def test_impulse_footprint():
    """A single impulse spreads at most (K//2)*2^l + 2^l - 1 pixels at level l."""
    dev = _cuda()
    params = wtconv_torch.random_params(2, 5, 3, bias=False, seed=5)
    m = _module(2, 2, 5, 3, 1, False, params, torch.float32, dev)
    x = torch.zeros(1, 2, 64, 64)
    x[0, :, 32, 32] = 1.0
    with torch.no_grad():
        y = m(x.to(dev)).cpu()
    ref = _oracle(2, x, params, 1, torch.float64)
    assert max_err(y.numpy(), ref.numpy()) <= 1e-5
    reach = 2 * 8 + 7
    mask = torch.ones(64, 64, dtype=torch.bool)
    mask[32 - reach:32 + reach + 1, 32 - reach:32 + reach + 1] = False
    assert float(y[0, :, mask].abs().max()) == 0.0


def test_autocast_mixed_dtypes_and_repack():
    """fp32 parameters with bf16 activations, and re-folding after an in-place parameter update."""
    dev = _cuda()
    params = wtconv_torch.random_params(16, 5, 3, seed=11)
    m = _module(2, 16, 5, 3, 1, True, params, torch.float32, dev)
    x = torch.randn(2, 16, 20, 20)
    with torch.no_grad():
        y = m(x.to(dev).to(torch.bfloat16)).float().cpu()
        ref = _oracle(2, x.to(torch.bfloat16).float(), params, 1, torch.float64)
        assert max_err(y.numpy(), ref.numpy()) <= 1e-2          # only the output rounding is bf16
        m.wavelet_scale[0].weight.mul_(2.0)
        y2 = m(x.to(dev)).cpu()
    params2 = dict(params)
    params2["wavelet_scale.0.weight"] = params["wavelet_scale.0.weight"] * 2.0
    assert max_err(y2.numpy(), _oracle(2, x, params2, 1, torch.float64).numpy()) <= 1e-5


def test_c_abi_error_codes():
    """Argument errors come back as negative statuses and python exceptions, never as a fault."""
    dev = _cuda()
    import ctypes
    import wtconv_b200
    from wtconv_b200 import _lib
    lib = _lib.load()
    x = torch.zeros(1, 4, 8, 8, device=dev)
    y = torch.zeros_like(x)
    packed = torch.zeros(lib.wtconv_packed_param_floats(2, 4, 5, 1), device=dev)
    xs = (ctypes.c_longlong * 4)(*x.stride())
    args = lambda K, L, dt: (x.data_ptr(), y.data_ptr(), packed.data_ptr(), None, 0, 1, 4, 8, 8, K, L, 1, dt, xs, xs, None)
    assert lib.wtconv2d_forward(*args(4, 1, 0)) == -2
    assert lib.wtconv2d_forward(*args(31, 1, 0)) == -2      # beyond the accepted range (odd sizes up to 29)
    assert lib.wtconv2d_forward(*args(5, -1, 0)) == -3
    assert lib.wtconv2d_forward(*args(5, 1, 7)) == -1
    assert lib.wtconv2d_forward(None, y.data_ptr(), packed.data_ptr(), None, 0, 1, 4, 8, 8, 5, 1, 1, 0, xs, xs, None) == -1
    assert lib.wtconv2d_forward(*args(5, 1, 0)) == 0
    m = wtconv_b200.WTConv2d(4, 4, kernel_size=31, wt_levels=1).to(dev)
    with torch.no_grad(), pytest.raises(ValueError):
        m(x)
    torch.cuda.synchronize()


# Gradient of the input (frozen parameters): the adjoint of the layer is the layer with flipped
# kernels and no bias, run by the same CUDA kernels; checked against autograd through the oracle.
@pytest.mark.parametrize("ndim,shape,L,K,stride,layout,dtype", [
    (2, (2, 8, 56, 56), 5, 5, 1, "cl", torch.float32), (2, (3, 40, 14, 13), 3, 5, 1, "cl", torch.float32),
    (2, (2, 6, 21, 30), 3, 3, 1, "nchw", torch.float32), (2, (2, 4, 17, 16), 2, 5, 2, "nchw", torch.float32),
    (2, (2, 16, 7, 7), 2, 5, 1, "cl", torch.bfloat16), (2, (1, 4, 150, 90), 4, 7, 1, "cl", torch.float32),
    (1, (2, 6, 515), 4, 5, 1, "nchw", torch.float32), (1, (2, 4, 100), 3, 3, 2, "nchw", torch.float32),
])
def test_input_gradient(ndim, shape, L, K, stride, layout, dtype):
    dev = _cuda()
    C = shape[1]
    params = wtconv_torch.random_params(C, K, L, ndim=ndim, bias=True, seed=sum(shape))
    g = torch.Generator().manual_seed(shape[-1])
    x = torch.randn(shape, generator=g)
    m = _module(ndim, C, K, L, stride, True, params, dtype, dev)
    for p in m.parameters():
        p.requires_grad_(False)
    xt = x.to(dev).to(dtype)
    if layout == "cl":
        xt = xt.contiguous(memory_format=torch.channels_last)
    xt.requires_grad_(True)
    y = m(xt)
    gy = torch.randn(y.shape, generator=g)
    (gx,) = torch.autograd.grad(y, xt, gy.to(dev).to(dtype))
    # oracle: autograd through the reference operator sequence in fp64
    xr = x.to(dtype).double().requires_grad_(True)
    fn = wtconv_torch.wtconv2d_forward if ndim == 2 else wtconv_torch.wtconv1d_forward
    yr = fn(xr, {k: torch.as_tensor(v).to(dtype).double() for k, v in params.items() if "filter" not in k}, stride=stride)
    (gr,) = torch.autograd.grad(yr, xr, gy.to(dtype).double())
    assert tuple(gx.shape) == tuple(x.shape)
    assert max_err(y.detach().float().cpu().numpy(), yr.detach().numpy()) <= TOL[dtype]
    assert max_err(gx.float().cpu().numpy(), gr.numpy()) <= TOL[dtype]


# Full backward of the 2-D layer (input and every parameter) against autograd through the oracle.
@pytest.mark.parametrize("shape,L,K,stride,bias,layout,dtype", [
    ((4, 24, 56, 56), 5, 5, 1, True, "cl", torch.float32), ((3, 40, 14, 13), 3, 5, 1, True, "cl", torch.float32),
    ((2, 6, 21, 30), 3, 3, 1, False, "nchw", torch.float32), ((2, 4, 17, 16), 2, 5, 2, True, "nchw", torch.float32),
    ((8, 64, 7, 7), 2, 5, 1, True, "cl", torch.bfloat16), ((1, 4, 90, 50), 4, 7, 1, True, "cl", torch.float32),
])
def test_parameter_gradients(shape, L, K, stride, bias, layout, dtype):
    dev = _cuda()
    C = shape[1]
    params = wtconv_torch.random_params(C, K, L, ndim=2, bias=bias, seed=sum(shape))
    g = torch.Generator().manual_seed(shape[-1])
    for i in range(L):
        params[f"wavelet_scale.{i}.weight"] = torch.empty_like(torch.as_tensor(params[f"wavelet_scale.{i}.weight"])).uniform_(0.05, 0.3, generator=g)
    x = torch.randn(shape, generator=g)
    m = _module(2, C, K, L, stride, bias, params, dtype, dev).train()
    xt = x.to(dev).to(dtype)
    if layout == "cl":
        xt = xt.contiguous(memory_format=torch.channels_last)
    xt.requires_grad_(True)
    y = m(xt)
    gy = torch.randn(y.shape, generator=g)
    y.backward(gy.to(dev).to(dtype))
    # oracle in fp64 on the parameter values the module holds
    names = [n for n, _ in m.named_parameters() if "filter" not in n]
    pd = {n: p.detach().cpu().double().requires_grad_(True) for n, p in m.named_parameters() if "filter" not in n}
    xr = x.to(dtype).double().requires_grad_(True)
    yr = wtconv_torch.wtconv2d_forward(xr, pd, stride=stride)
    refs = torch.autograd.grad(yr, [xr] + [pd[n] for n in names], gy.to(dtype).double())
    tol = 1e-4 if dtype == torch.float32 else 3e-2      # sums over B*H*W terms in fp32 / results rounded to bf16
    assert max_err(xt.grad.float().cpu().numpy(), refs[0].numpy()) <= TOL[dtype]
    got = dict(m.named_parameters())
    for n, r in zip(names, refs[1:]):
        assert got[n].grad is not None, n
        err = max_err(got[n].grad.float().cpu().numpy(), r.numpy())
        assert err <= tol, f"{n}: {err:.3e}"
    assert m.wt_filter.grad is None and m.iwt_filter.grad is None


@pytest.mark.parametrize("shape,L,K,stride", [((3, 8, 515), 4, 5, 1), ((2, 4, 100), 3, 3, 2), ((4, 64, 4096), 4, 5, 1)])
def test_parameter_gradients_1d(shape, L, K, stride):
    dev = _cuda()
    C = shape[1]
    params = wtconv_torch.random_params(C, K, L, ndim=1, bias=True, seed=sum(shape))
    g = torch.Generator().manual_seed(shape[-1])
    x = torch.randn(shape, generator=g)
    m = _module(1, C, K, L, stride, True, params, torch.float32, dev).train()
    xt = x.to(dev).requires_grad_(True)
    y = m(xt)
    gy = torch.randn(y.shape, generator=g)
    y.backward(gy.to(dev))
    names = [n for n, _ in m.named_parameters() if "filter" not in n]
    pd = {n: p.detach().cpu().double().requires_grad_(True) for n, p in m.named_parameters() if "filter" not in n}
    xr = x.double().requires_grad_(True)
    yr = wtconv_torch.wtconv1d_forward(xr, pd, stride=stride)
    refs = torch.autograd.grad(yr, [xr] + [pd[n] for n in names], gy.double())
    assert max_err(xt.grad.cpu().numpy(), refs[0].numpy()) <= 1e-5
    got = dict(m.named_parameters())
    for n, r in zip(names, refs[1:]):
        err = max_err(got[n].grad.cpu().numpy(), r.numpy())
        assert err <= 1e-4, f"{n}: {err:.3e}"


# Kernel sizes without an unrolled instance (odd, 9 .. 29): the run-time-size CTA-tile kernels.
@pytest.mark.parametrize("case", [
    (2, 8, 9, 3, (2, 8, 40, 37), 1, "cl", torch.float32), (2, 6, 11, 2, (2, 6, 56, 56), 1, "nchw", torch.float32),
    (2, 4, 29, 1, (1, 4, 64, 48), 1, "cl", torch.float32), (2, 16, 9, 2, (2, 16, 28, 28), 2, "cl", torch.bfloat16),
    (2, 4, 13, 4, (1, 4, 150, 120), 1, "nchw", torch.float32),
    (1, 6, 9, 3, (2, 6, 1000), 1, "", torch.float32), (1, 4, 29, 2, (2, 4, 4097), 2, "", torch.float32),
    (1, 8, 15, 4, (2, 8, 4096), 1, "", torch.bfloat16),
], ids=lambda c: f"{c[0]}d-K{c[2]}-L{c[3]}-s{c[5]}{c[6]}-{str(c[7])[6:]}")
def test_run_time_kernel_size(case):
    dev = _cuda()
    nd, C, K, L, shape, stride, layout, dtype = case
    params = wtconv_torch.random_params(C, K, L, ndim=nd, seed=K + L)
    x = torch.randn(*shape, generator=torch.Generator().manual_seed(K))
    m = _module(nd, C, K, L, stride, True, params, dtype, dev)
    xt = x.to(dev).to(dtype)
    if layout == "cl":
        xt = xt.contiguous(memory_format=torch.channels_last)
    with torch.no_grad():
        out = m(xt).float().cpu()
    ref = _oracle(nd, x, params, stride, torch.float64 if dtype == torch.float32 else dtype).float()
    assert tuple(out.shape) == tuple(ref.shape)
    assert max_err(out.numpy(), ref.numpy()) <= TOL[dtype]
