"""The allocation-free entry point `wtconv2d_forward_noalloc`.

Some hosts of these kernels cannot allocate device memory when they call them: a
CUDA-graph capture or latency-critical serving loop (an allocation would synchronise
the device), an inference-runtime plug-in that is handed fixed buffers and owns no
allocator, an embedder whose memory budget is frozen after start-up.  For them the
library carries its scratch planes as a built-in 16 MiB array.  This test calls that
entry point through the C ABI, twice in a row, and checks it against the CPU oracle
and against the regular `wtconv2d_forward` (caller-provided workspace) on problems
that do use scratch; the size pre-check is exercised with the chain that the very
pointers of the call get.

The file name sorts last on purpose: a run that stops at the first failure has then
already executed every other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

LIMIT = 16 << 20


def _setup(B, C, H, W, K, L, dtype, channels_last, seed):
    from oracle import wtconv_torch
    from wtconv_b200 import _lib, modules
    dev = torch.device("cuda:0")
    lib = _lib.load()
    m = modules.WTConv2d(C, C, kernel_size=K, wt_levels=L)
    sd = m.state_dict()
    for k, v in wtconv_torch.random_params(C, K, L, seed=seed).items():
        sd[k] = v.reshape(sd[k].shape)
    m.load_state_dict(sd)
    m = m.to(dev).to(dtype).eval()
    packed = m._packed_params(dev)
    x = torch.randn(B, C, H, W, generator=torch.Generator().manual_seed(seed + 1)).to(dev).to(dtype)
    if channels_last:
        x = x.contiguous(memory_format=torch.channels_last)
    return lib, packed, x


def _oracle(x, C, K, L, seed):
    """Float64 oracle on the (rounded) inputs and parameters the kernels saw."""
    from oracle import wtconv_np, wtconv_torch
    params = {k: v.to(x.dtype).double() for k, v in wtconv_torch.random_params(C, K, L, seed=seed).items()}
    return torch.as_tensor(wtconv_np.wtconv2d_forward(x.double().cpu().contiguous(), params))


def _norm_err(y, ref):
    return float((y.double().cpu() - ref.double().cpu()).abs().max() / ref.double().abs().max())


def _call_pair(lib, packed, x, K, L):
    B, C, H, W = x.shape
    code = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}[x.dtype]
    xs = (ctypes.c_longlong * 4)(*x.stride())
    need = ctypes.c_size_t(0)
    assert lib.wtconv2d_workspace_bytes(B, C, H, W, K, L, code, xs, xs, ctypes.byref(need)) == 0
    stream = torch.cuda.current_stream().cuda_stream
    # regular entry point, caller-provided workspace
    y_ref = torch.full_like(x, float("nan"))
    ws = torch.empty(max(int(need.value), 16), dtype=torch.uint8, device=x.device)
    st = lib.wtconv2d_forward(x.data_ptr(), y_ref.data_ptr(), packed.data_ptr(), ws.data_ptr(), int(need.value),
                              B, C, H, W, K, L, 1, code, xs, xs, stream)
    assert st == 0
    # allocation-free entry point: no workspace argument at all
    y = torch.full_like(x, float("nan"))
    st = lib.wtconv2d_forward_noalloc(x.data_ptr(), y.data_ptr(), packed.data_ptr(), B, C, H, W, K, L, 1, code,
                                      xs, xs, stream)
    torch.cuda.synchronize()
    return st, y, y_ref, int(need.value)


@pytest.mark.parametrize("case", [
    (8, 32, 56, 56, 5, 5, torch.bfloat16, True),     # TMA-fed chain: scratch holds level-2 sub-bands and R_1
    (1, 8, 200, 136, 5, 5, torch.float32, False),    # three-stage chain with materialised low-pass planes
    (4, 16, 28, 28, 5, 4, torch.float32, True),      # fits on chip: needs no scratch, must still work
])
def test_noalloc_matches_workspace_entry_point_twice(case):
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    B, C, H, W, K, L, dtype, cl = case
    lib, packed, x = _setup(B, C, H, W, K, L, dtype, cl, seed=H + W)
    for attempt in range(2):                          # second call reuses the array with stale contents
        st, y, y_ref, need = _call_pair(lib, packed, x, K, L)
        assert st == 0, f"call {attempt}: status {st}"
        assert need <= LIMIT
        assert not torch.isnan(y.float()).any()
        assert torch.equal(y, y_ref), f"call {attempt}: differs from the workspace entry point"
        err = _norm_err(y, _oracle(x, C, K, L, seed=H + W))
        tol = 1e-5 if dtype == torch.float32 else 5e-3      # fp32 arithmetic, one rounding of the output
        assert err <= tol, f"call {attempt}: normalised max error {err:.3e} against the oracle"
        x = x.roll(1, dims=0).contiguous(memory_format=torch.channels_last if cl else torch.contiguous_format)


def test_noalloc_rejects_problems_beyond_the_built_in_array():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from wtconv_b200 import _lib
    lib, packed, x = _setup(2, 96, 56, 56, 5, 5, torch.bfloat16, True, seed=3)
    xs = (ctypes.c_longlong * 4)(*x.stride())
    y = torch.zeros_like(x)
    # same layer at batch 128 needs 128*96*4704 bytes = 57.8 MB of scratch: over the limit.
    # Only sizes are checked before the rejection, so the small tensors above are never touched.
    st = lib.wtconv2d_forward_noalloc(x.data_ptr(), y.data_ptr(), packed.data_ptr(), 128, 96, 56, 56, 5, 5, 1, 1,
                                      xs, xs, None)
    assert st == -8
    assert "scratch" in _lib.status_string(st)
    torch.cuda.synchronize()


def test_noalloc_size_check_uses_the_chain_of_the_actual_pointers():
    """bf16 channels-last 28x28 planes, 4 levels, B*C = 64*192: tensors on 16-byte boundaries take the
    TMA-fed chain (1176 bytes of scratch per plane, 14.4 MB: fits); the same strides from an address
    that is only element-aligned take the CTA-tile chain (1960 bytes per plane, 24 MB: over the limit).
    The first call must succeed and match the oracle, the second must be rejected with
    WTCONV_ERR_SCRATCH_LIMIT (not with a workspace error from the inner call)."""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    B, C, H, K, L = 64, 192, 28, 5, 4
    lib, packed, x = _setup(B, C, H, H, K, L, torch.bfloat16, True, seed=11)
    xs = (ctypes.c_longlong * 4)(*x.stride())
    stream = torch.cuda.current_stream().cuda_stream
    y = torch.full_like(x, float("nan"))
    st = lib.wtconv2d_forward_noalloc(x.data_ptr(), y.data_ptr(), packed.data_ptr(), B, C, H, H, K, L, 1, 1, xs, xs, stream)
    torch.cuda.synchronize()
    assert st == 0
    idx = [0, 31, 63]
    assert _norm_err(y[idx], _oracle(x[idx], C, K, L, seed=11)) <= 5e-3
    # same data one element further: aligned to the element size only
    flat = torch.empty(x.numel() + 8, dtype=x.dtype, device=x.device)
    x_off = flat[1:1 + x.numel()].view(B, H, H, C).permute(0, 3, 1, 2)
    x_off.copy_(x)
    assert x_off.data_ptr() % 16 == 2 and x_off.stride() == x.stride()
    st = lib.wtconv2d_forward_noalloc(x_off.data_ptr(), y.data_ptr(), packed.data_ptr(), B, C, H, H, K, L, 1, 1, xs, xs,
                                      stream)
    torch.cuda.synchronize()
    assert st == -8
    # the regular entry point accepts those pointers with the workspace size the library reports
    need = ctypes.c_size_t(0)
    assert lib.wtconv2d_workspace_bytes(B, C, H, H, K, L, 1, xs, xs, ctypes.byref(need)) == 0
    ws = torch.empty(int(need.value), dtype=torch.uint8, device=x.device)
    y2 = torch.full_like(x, float("nan"))
    st = lib.wtconv2d_forward(x_off.data_ptr(), y2.data_ptr(), packed.data_ptr(), ws.data_ptr(), int(need.value),
                              B, C, H, H, K, L, 1, 1, xs, xs, stream)
    torch.cuda.synchronize()
    assert st == 0
    assert _norm_err(y2[idx], _oracle(x[idx], C, K, L, seed=11)) <= 5e-3
