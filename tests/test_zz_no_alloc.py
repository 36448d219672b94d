"""The allocation-free entry point `wtconv2d_forward_noalloc`.

Some hosts of these kernels cannot allocate device memory when they call them: a
CUDA-graph capture or latency-critical serving loop (an allocation would synchronise
the device), an inference-runtime plug-in that is handed fixed buffers and owns no
allocator, an embedder whose memory budget is frozen after start-up.  For them the
library carries its scratch planes as a built-in 16 MiB array.  This test calls that
entry point through the C ABI, twice in a row, and checks it against the regular
`wtconv2d_forward` (caller-provided workspace) on problems that do use scratch.

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
    (8, 32, 56, 56, 5, 5, torch.bfloat16, True),     # split into two launches: scratch holds R_1 planes
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
        err = float((y.float() - y_ref.float()).abs().max() / y_ref.float().abs().max())
        tol = 1e-5 if dtype == torch.float32 else 2e-2
        assert err <= tol, f"call {attempt}: normalised max error {err:.3e}"
        x = x.roll(1, dims=0).contiguous(memory_format=torch.channels_last if cl else torch.contiguous_format)


def test_noalloc_rejects_problems_beyond_the_built_in_array():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from wtconv_b200 import _lib
    lib, packed, x = _setup(2, 96, 56, 56, 5, 5, torch.bfloat16, True, seed=3)
    xs = (ctypes.c_longlong * 4)(*x.stride())
    y = torch.zeros_like(x)
    # same layer at batch 128 needs 128*96*28*28*4 bytes = 38.5 MB of scratch: over the limit.
    # Only sizes are checked before the rejection, so the small tensors above are never touched.
    st = lib.wtconv2d_forward_noalloc(x.data_ptr(), y.data_ptr(), packed.data_ptr(), 128, 96, 56, 56, 5, 5, 1, 1,
                                      xs, xs, None)
    assert st == -8
    assert "scratch" in _lib.status_string(st)
    torch.cuda.synchronize()
