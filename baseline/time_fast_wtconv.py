"""Informational comparator: the reference's own fused CUDA backend on the same GPU.

``fast_wtconv/wtconv_cuda.py`` of BGU-CS-VIL/WTConv (JIT-built CUDA kernels, NCHW only, its own
constructor and parameter names) is timed next to this library on the WTConvNeXt-T stage shapes,
with the weights of one copied into the other so that the outputs can be compared as well.

The reference is not part of this repository.  Install a copy first (in a container where its
checkout is readable; the build needs nvcc but no GPU)::

    python baseline/time_fast_wtconv.py --install <path of the reference checkout>

which copies ``fast_wtconv/`` and ``wtconv/`` to ``baseline/_ref/src`` (ignored by git) and JIT-builds the
CUDA extension for sm_100 into ``baseline/_ref/torch_ext``.  Then, on a B200::

    python baseline/time_fast_wtconv.py

bench.py uses the same copies: ``wtconv/`` for its CPU reference arm and ``fast_wtconv/`` for the
secondary GPU comparison in its JSON line.
"""
import argparse
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")
os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0")
os.environ.setdefault("TORCH_EXTENSIONS_DIR", os.path.join(REF, "torch_ext"))
os.environ.setdefault("HAAR_MAX_K", "5")
sys.path.insert(0, os.path.join(REF, "src"))
sys.path.insert(0, os.path.dirname(HERE))

STAGES = [(96, 56, 5), (192, 28, 4), (384, 14, 3), (768, 7, 2)]   # (C, H=W, wt_levels), batch 128, K=5


def install(checkout):
    # fast_wtconv: the reference's CUDA backend (GPU comparator); wtconv: its pure-PyTorch layer, which
    # bench.py --impl reference runs unchanged on the host cores
    for pkg in ("fast_wtconv", "wtconv"):
        dst = os.path.join(REF, "src", pkg)
        if os.path.isdir(dst):
            shutil.rmtree(dst)
        shutil.copytree(os.path.join(checkout, pkg), dst)
    from fast_wtconv.cuda_haar import haar_cuda
    print("built", haar_cuda._get_module())


def event_ms(fn, reps=10):
    import torch
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        out = fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / reps, out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--install", metavar="CHECKOUT", help="copy and build the reference backend, then exit")
    ap.add_argument("--batch", type=int, default=128)
    ap.add_argument("--backward", action="store_true", help="time forward + backward (input and parameter gradients)")
    args = ap.parse_args()
    if args.install:
        return install(args.install)
    import torch
    import wtconv_b200
    from fast_wtconv.wtconv_cuda import WTConv2d as FastWTConv2d
    dev = torch.device("cuda:0")
    for dtype in (torch.bfloat16, torch.float32):
        for C, H, L in STAGES:
            torch.manual_seed(C)
            ours = wtconv_b200.WTConv2d(C, C, kernel_size=5, wt_levels=L).to(dev).to(dtype).eval()
            ref = FastWTConv2d(C, C, 5, 1, L, True).to(dev).to(dtype).eval()
            sd = ours.state_dict()
            with torch.no_grad():
                ref.base_weight.copy_(sd["base_conv.weight"])
                ref.base_bias.copy_(sd["base_conv.bias"])
                ref.base_scale.copy_(sd["base_scale.weight"])
                for i in range(L):
                    ref.wt_weights[i].copy_(sd[f"wavelet_convs.{i}.weight"])
                    ref.wt_scales[i].copy_(sd[f"wavelet_scale.{i}.weight"])
                x = torch.randn(args.batch, C, H, H, device=dev, dtype=dtype)
                xcl = x.contiguous(memory_format=torch.channels_last)
                if not args.backward:
                    ms_ref, yr = event_ms(lambda: ref(x))
                    ms_ours, yo = event_ms(lambda: ours(xcl))
            if args.backward:
                gy = torch.randn_like(x)
                gycl = gy.contiguous(memory_format=torch.channels_last)
                xr, xo = x.clone().requires_grad_(True), xcl.clone().requires_grad_(True)

                def step(m, xin, g):
                    m.zero_grad(set_to_none=True)
                    xin.grad = None
                    y = m(xin)
                    y.backward(g)
                    return xin.grad

                ms_ref, yr = event_ms(lambda: step(ref, xr, gy))
                ms_ours, yo = event_ms(lambda: step(ours, xo, gycl))
            diff = float((yo.float() - yr.float()).abs().max() / yr.float().abs().max())
            print(f"{str(dtype)[6:]:9s} C={C:4d} H={H:3d} L={L}: fast_wtconv CUDA (NCHW) {ms_ref * 1e3:8.1f} us | "
                  f"this library (channels-last) {ms_ours * 1e3:8.1f} us | ratio {ms_ref / ms_ours:5.2f} | "
                  f"normalised max difference {diff:.2e}", flush=True)


if __name__ == "__main__":
    main()
