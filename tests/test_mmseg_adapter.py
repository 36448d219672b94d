"""Segmentation-backbone adapter: state_dict layout of the shim layer, rebinding, in-place swap of a
built model and the classification -> mmseg checkpoint key map
(semantic_segmentation/mmseg/models/backbones/wtconvnext.py:66,425-457,
semantic_segmentation/translate_model_to_mmseg.py:8-40).  mmseg itself is not needed."""
import types

import pytest
import torch
import torch.nn as nn

import wtconv_b200
from wtconv_b200 import mmseg_adapter as mm
from oracle import wtconv_torch as oracle


def _expected_layer_keys(levels, bias=True, stride=1):
    keys = ["wt_filter", "iwt_filter", "base_conv.weight"] + (["base_conv.bias"] if bias else []) + ["base_scale.weight"]
    keys += [f"wavelet_convs.{l}.weight" for l in range(levels)]
    keys += [f"wavelet_scale.{l}.weight" for l in range(levels)]
    if stride > 1:
        keys.append("stride_filter")
    return keys


@pytest.mark.parametrize("stride", [1, 2])
def test_shim_state_dict_layout(stride):
    layer = mm.MMSegWTConv2d(8, 8, kernel_size=5, stride=stride, wt_levels=3)
    sd = layer.state_dict()
    assert sorted(sd.keys()) == sorted(_expected_layer_keys(3, stride=stride))
    if stride > 1:
        assert sd["stride_filter"].shape == (8, 1, 1, 1)
        assert not layer.stride_filter.requires_grad
        assert bool((sd["stride_filter"] == 1).all())
    # strict loading of a checkpoint of the reference copy: same keys, same shapes
    ref_like = {k: torch.randn_like(v) if k != "stride_filter" else v.clone() for k, v in sd.items()}
    layer.load_state_dict(ref_like, strict=True)
    # the classification layer has no stride_filter: a segmentation checkpoint must not load strictly into it
    if stride > 1:
        plain = wtconv_b200.WTConv2d(8, 8, kernel_size=5, stride=stride, wt_levels=3)
        with pytest.raises(RuntimeError):
            plain.load_state_dict(ref_like, strict=True)


def test_install_rebinds_module_name():
    class _WTConv2d(nn.Module):
        pass

    backbone = types.ModuleType("fake_backbone")
    backbone._WTConv2d = _WTConv2d
    # the block constructor of the reference resolves the name at call time
    exec("def build(c, **cfg):\n    return _WTConv2d(c, c, **cfg)\n", backbone.__dict__)
    prev = mm.install(backbone)
    assert prev is _WTConv2d
    layer = backbone.build(16, kernel_size=5, wt_levels=2)
    assert isinstance(layer, mm.MMSegWTConv2d) and layer.wt_levels == 2
    with pytest.raises(AttributeError):
        mm.install(types.ModuleType("empty"))


class _WTConv2d(nn.Module):
    """Stand-in with the attribute layout of the reference copy (no forward of its own)."""

    def __init__(self, C, K, L, stride):
        super().__init__()
        self.wt_levels, self.stride = L, stride
        ana, syn = oracle.haar_filters_2d(C)
        self.wt_filter = nn.Parameter(ana, requires_grad=False)
        self.iwt_filter = nn.Parameter(syn, requires_grad=False)
        self.base_conv = nn.Conv2d(C, C, K, padding="same", groups=C)
        self.base_scale = nn.Module()
        self.base_scale.weight = nn.Parameter(torch.rand(1, C, 1, 1) + 0.5)
        self.wavelet_convs = nn.ModuleList([nn.Conv2d(4 * C, 4 * C, K, padding="same", groups=4 * C, bias=False)
                                            for _ in range(L)])
        self.wavelet_scale = nn.ModuleList()
        for _ in range(L):
            m = nn.Module()
            m.weight = nn.Parameter(torch.rand(1, 4 * C, 1, 1) * 0.2)
            self.wavelet_scale.append(m)
        if stride > 1:
            self.stride_filter = nn.Parameter(torch.ones(C, 1, 1, 1), requires_grad=False)


def _model(stride=2):
    torch.manual_seed(3)
    return nn.Sequential(nn.Conv2d(3, 8, 1), nn.Sequential(_WTConv2d(8, 5, 2, 1), nn.GELU()), _WTConv2d(8, 3, 1, stride))


def test_swap_layers_keeps_parameters_and_keys():
    model = _model()
    before = {k: v for k, v in model.state_dict().items()}
    ids = {k: id(p) for k, p in model.named_parameters()}
    assert mm.swap_layers(model) == 2
    assert isinstance(model[1][0], mm.MMSegWTConv2d) and isinstance(model[2], mm.MMSegWTConv2d)
    assert model[2].stride == 2 and model[2].kernel_size == 3 and model[1][0].wt_levels == 2
    after = model.state_dict()
    assert list(after.keys()) == list(before.keys()) or sorted(after.keys()) == sorted(before.keys())
    for k in before:
        assert torch.equal(before[k], after[k]), k
    for k, p in model.named_parameters():
        if not k.endswith("wt_filter"):          # the filter banks are re-wrapped, everything else is the same object
            assert ids[k] == id(p), k
    assert mm.swap_layers(model) == 0           # idempotent


def _classification_checkpoint():
    """Key layout of the classification model (timm ConvNeXt naming with the WTConv layer as conv_dw)."""
    layer = wtconv_b200.WTConv2d(4, 4, kernel_size=5, wt_levels=2).state_dict()
    sd = {"stem.0.weight": torch.zeros(1), "stem.0.bias": torch.zeros(1), "stem.1.weight": torch.zeros(1),
          "stem.1.bias": torch.zeros(1)}
    for s in range(4):
        if s > 0:
            for i in (0, 1):
                for p in ("weight", "bias"):
                    sd[f"stages.{s}.downsample.{i}.{p}"] = torch.zeros(1)
        for b in range(2):
            root = f"stages.{s}.blocks.{b}"
            sd[f"{root}.gamma"] = torch.zeros(1)
            for k, v in layer.items():
                sd[f"{root}.conv_dw.{k}"] = v
            for p in ("weight", "bias"):
                sd[f"{root}.norm.{p}"] = torch.zeros(1)
                sd[f"{root}.mlp.fc1.{p}"] = torch.zeros(1)
                sd[f"{root}.mlp.fc2.{p}"] = torch.zeros(1)
    sd["head.norm.weight"] = torch.zeros(1)
    sd["head.fc.weight"] = torch.zeros(1)
    return sd


def test_translate_to_mmseg_key_map():
    sd = _classification_checkpoint()
    out = mm.translate_to_mmseg(sd)
    assert all(k.startswith("backbone.") for k in out)
    assert len(out) == len(sd) - 2                                   # the classification head is left out
    assert out["backbone.downsample_layers.0.1.bias"] is sd["stem.1.bias"]
    assert out["backbone.downsample_layers.2.0.weight"] is sd["stages.2.downsample.0.weight"]
    assert out["backbone.stages.1.0.gamma"] is sd["stages.1.blocks.0.gamma"]
    assert out["backbone.stages.3.1.pointwise_conv1.weight"] is sd["stages.3.blocks.1.mlp.fc1.weight"]
    assert out["backbone.stages.3.1.pointwise_conv2.bias"] is sd["stages.3.blocks.1.mlp.fc2.bias"]
    assert out["backbone.stages.0.1.norm.weight"] is sd["stages.0.blocks.1.norm.weight"]
    assert out["backbone.stages.2.1.depthwise_conv.wavelet_convs.1.weight"] is \
        sd["stages.2.blocks.1.conv_dw.wavelet_convs.1.weight"]
    assert out["backbone.stages.2.1.depthwise_conv.base_scale.weight"] is \
        sd["stages.2.blocks.1.conv_dw.base_scale.weight"]
    # the translated depthwise_conv entries load strictly into the shim layer
    sub = {k[len("backbone.stages.0.0.depthwise_conv."):]: v for k, v in out.items()
           if k.startswith("backbone.stages.0.0.depthwise_conv.")}
    mm.MMSegWTConv2d(4, 4, kernel_size=5, wt_levels=2).load_state_dict(sub, strict=True)
    assert list(mm.translate_to_mmseg(sd, prefix="").keys())[0] == "downsample_layers.0.0.weight"
    bad = dict(sd)
    bad["stages.0.blocks.0.grn.weight"] = torch.zeros(1)
    with pytest.raises(KeyError):
        mm.translate_to_mmseg(bad)


@pytest.mark.gpu
def test_swapped_model_matches_reference_layout_forward():
    """A built model with reference-layout layers, swapped in place, gives the oracle's outputs
    (stride 2 through stride_filter == strided store).  fp32: normalised max error <= 1e-5."""
    model = _model().cuda()
    x = torch.randn(4, 3, 30, 27, device="cuda")

    def ref_forward(m, t):
        t = m[0](t)
        l1 = m[1][0]
        t = torch.nn.functional.gelu(oracle.wtconv2d_forward(t, oracle_params(l1), stride=l1.stride))
        l2 = m[2]
        return oracle.wtconv2d_forward(t, oracle_params(l2), stride=l2.stride)

    def oracle_params(l):
        p = {"base_conv.weight": l.base_conv.weight, "base_conv.bias": l.base_conv.bias,
             "base_scale.weight": l.base_scale.weight}
        for i in range(l.wt_levels):
            p[f"wavelet_convs.{i}.weight"] = l.wavelet_convs[i].weight
            p[f"wavelet_scale.{i}.weight"] = l.wavelet_scale[i].weight
        return p

    prev = torch.backends.cudnn.allow_tf32
    torch.backends.cudnn.allow_tf32 = False
    try:
        with torch.no_grad():
            want = ref_forward(model, x)
            assert mm.swap_layers(model) == 2
            got = model(x)
    finally:
        torch.backends.cudnn.allow_tf32 = prev
    assert got.shape == want.shape == (4, 8, 15, 14)
    err = (got - want).abs().max() / want.abs().max()
    assert err <= 1e-5, float(err)
    # a stride_filter that is not all ones cannot be honoured by the strided store: loud error
    model[2].stride_filter.data[0] = 2.0
    model[2]._stride_filter_checked = None
    with pytest.raises(ValueError):
        model(x)
