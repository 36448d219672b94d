"""WTConvNeXt-T harness: parameter-count pin (CPU) and model-level parity on the GPU between
the harness built with the B200 layer and the same harness built with an oracle-backed layer."""
import pytest
import torch
import torch.nn as nn


def test_parameter_count_matches_reference_log():
    import wtconv_b200
    from wtconv_b200.wtconvnext_harness import WTConvNeXtTiny
    m = WTConvNeXtTiny(wtconv_b200.WTConv2d)
    assert sum(p.numel() for p in m.parameters()) == 30595624      # logs/val_tiny.out:4 of the reference
    assert sum(isinstance(c, wtconv_b200.WTConv2d) for c in m.modules()) == 18


class _OracleWTConv2d(nn.Module):
    """Same parameters as the layer under test, forward through the CPU oracle's operator sequence
    (runs on whatever device the tensors are on) -- test infrastructure only."""

    def __init__(self, c_in, c_out, kernel_size=5, stride=1, bias=True, wt_levels=1):
        super().__init__()
        import wtconv_b200
        self.inner = wtconv_b200.WTConv2d(c_in, c_out, kernel_size=kernel_size, stride=stride, bias=bias,
                                          wt_levels=wt_levels)
        self.stride = stride

    def forward(self, x):
        from oracle import wtconv_torch
        params = {k: v for k, v in self.inner.state_dict().items() if "filter" not in k}
        return wtconv_torch.wtconv2d_forward(x, params, stride=self.stride)


@pytest.mark.gpu
def test_model_logits_match_oracle_layers():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    import wtconv_b200
    from wtconv_b200.wtconvnext_harness import WTConvNeXtTiny
    dev = torch.device("cuda:0")
    torch.manual_seed(0)
    ours = WTConvNeXtTiny(wtconv_b200.WTConv2d)
    with torch.no_grad():
        for m in ours.modules():                       # make the layers matter: default layer scale is 1e-6
            if hasattr(m, "gamma"):
                m.gamma.fill_(0.5)
    ref = WTConvNeXtTiny(_OracleWTConv2d)
    sd = ours.state_dict()
    ref.load_state_dict({k.replace("conv_dw.", "conv_dw.inner."): v for k, v in sd.items()})
    ours, ref = ours.to(dev).eval(), ref.to(dev).eval()
    x = torch.randn(2, 3, 224, 224, device=dev)
    tf32 = torch.backends.cudnn.allow_tf32
    torch.backends.cudnn.allow_tf32 = False            # the stem / downsampling convs stay true fp32
    try:
        with torch.no_grad():
            a = ours(x.contiguous(memory_format=torch.channels_last))
            b32 = ref(x)
            b64 = ref.double()(x.double())
    finally:
        torch.backends.cudnn.allow_tf32 = tf32

    def nerr(u, v):
        return float((u.double() - v.double()).abs().max() / v.double().abs().max())

    # 18 blocks of fp32 round-off compound through the LayerNorms, so the yardstick is the fp64
    # evaluation of the same network: the B200 layers must sit as close to it as the fp32 oracle does.
    e_ours, e_oracle = nerr(a, b64), nerr(b32, b64)
    assert e_ours <= max(2.0 * e_oracle, 2e-5), f"vs fp64: ours {e_ours:.3e}, fp32 oracle {e_oracle:.3e}"
    assert nerr(a, b32) <= 5e-4, f"logit mismatch {nerr(a, b32):.3e}"


@pytest.mark.gpu
def test_model_training_step_matches_oracle_layers():
    """One forward + backward of the harness: gradients through the 18 B200 layers (input and
    parameters) against the same network with oracle layers under autograd, both in fp32."""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    import wtconv_b200
    from wtconv_b200.wtconvnext_harness import WTConvNeXtTiny
    dev = torch.device("cuda:0")
    torch.manual_seed(1)
    ours = WTConvNeXtTiny(wtconv_b200.WTConv2d)
    with torch.no_grad():
        for m in ours.modules():
            if hasattr(m, "gamma"):
                m.gamma.fill_(0.5)
    ref = WTConvNeXtTiny(_OracleWTConv2d)
    ref.load_state_dict({k.replace("conv_dw.", "conv_dw.inner."): v for k, v in ours.state_dict().items()})
    ours, ref = ours.to(dev).train(), ref.to(dev).double().train()
    x = torch.randn(2, 3, 224, 224, device=dev)
    target = torch.randint(0, 1000, (2,), device=dev)
    tf32 = torch.backends.cudnn.allow_tf32
    torch.backends.cudnn.allow_tf32 = False
    try:
        loss_a = torch.nn.functional.cross_entropy(ours(x.contiguous(memory_format=torch.channels_last)), target)
        loss_a.backward()
        loss_b = torch.nn.functional.cross_entropy(ref(x.double()), target)
        loss_b.backward()
    finally:
        torch.backends.cudnn.allow_tf32 = tf32
    assert abs(float(loss_a.detach()) - float(loss_b.detach())) <= 1e-4 * abs(float(loss_b.detach()))
    ga = dict(ours.named_parameters())
    checked = 0
    for name, pb in ref.named_parameters():
        if "filter" in name or pb.grad is None:
            continue
        pa = ga[name.replace("conv_dw.inner.", "conv_dw.")]
        assert pa.grad is not None, name
        err = float((pa.grad.double() - pb.grad).abs().max() / (pb.grad.abs().max() + 1e-30))
        assert err <= 2e-3, f"{name}: {err:.3e}"        # fp32 network against its fp64 evaluation
        checked += 1
    assert checked >= 140


@pytest.mark.gpu
def test_captured_forward_replays_eager_result():
    """The CUDA-graph replay of the whole model gives the logits of the eager forward (bf16: normalised
    max error <= 2e-2; the library GEMMs may pick another algorithm under capture), for more than one
    batch through the same graph, and rejects another shape."""
    import wtconv_b200
    from wtconv_b200.wtconvnext_harness import CapturedForward, WTConvNeXtTiny
    dev = torch.device("cuda", 0)
    torch.manual_seed(5)
    model = WTConvNeXtTiny(wtconv_b200.WTConv2d).to(dev).to(torch.bfloat16).eval()
    model = model.to(memory_format=torch.channels_last)
    xs = [torch.randn(2, 3, 224, 224, device=dev, dtype=torch.bfloat16).contiguous(memory_format=torch.channels_last)
          for _ in range(2)]
    fwd = CapturedForward(model, xs[0])
    with torch.no_grad():
        for x in (xs[1], xs[0], xs[1]):
            want = model(x)
            got = fwd(x).clone()
            err = float((got.float() - want.float()).abs().max() / want.float().abs().max())
            assert err <= 2e-2, err
    with pytest.raises(ValueError):
        fwd(xs[0][:1])
