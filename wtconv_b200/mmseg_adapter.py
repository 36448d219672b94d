"""Adapter for the reference's segmentation backbone and its checkpoint formats.

The mmseg backbone of the reference does not import ``wtconv.WTConv2d``: it carries a private copy,
``_WTConv2d`` (semantic_segmentation/mmseg/models/backbones/wtconvnext.py:425-457), that its block
builds as ``self.depthwise_conv = _WTConv2d(in_channels, in_channels, **dw_conv_cfg)`` (:66).  The copy
differs from the classification layer in one ``state_dict`` entry: with ``stride > 1`` it owns a
frozen ``stride_filter`` of ones, shape (C, 1, 1, 1), used as a 1x1 strided depthwise convolution
(:451-453) -- the same sub-sampling ``y[..., ::s, ::s]`` the classification layer gets from
``AvgPool2d(kernel_size=1, stride=s)`` (wtconv/wtconv2d.py:33-36).

Three pieces, none of which needs mmseg itself:

* ``MMSegWTConv2d`` -- the B200 layer with that ``state_dict`` (strict loading of a segmentation
  checkpoint works);
* ``install(backbone_module)`` rebinds the module-level name ``_WTConv2d`` of the reference's backbone
  file, so models built afterwards use the B200 layer; ``swap_layers(model)`` does the same for a model
  that is already built (parameters are carried over, not copied);
* ``translate_to_mmseg(state_dict)`` -- the key map of
  semantic_segmentation/translate_model_to_mmseg.py:8-40 as a function: classification checkpoint keys
  (timm ConvNeXt layout) to the ``backbone.*`` keys of the mmseg model.
"""
from __future__ import annotations

from collections import OrderedDict

import torch
import torch.nn as nn

from .modules import WTConv2d

__all__ = ["MMSegWTConv2d", "install", "swap_layers", "translate_to_mmseg"]


class MMSegWTConv2d(WTConv2d):
    """``_WTConv2d`` of the segmentation backbone on the B200 kernels.

    Same constructor as the reference copy (wtconvnext.py:426).  The sub-sampling itself is done by the
    kernels' strided store; ``stride_filter`` exists for the ``state_dict`` only and must stay all ones
    (the reference never trains it: ``requires_grad=False``), which ``forward`` checks once per value.
    """

    def __init__(self, in_channels, out_channels, kernel_size=5, stride=1, bias=True, wt_levels=1, wt_type='db1'):
        super().__init__(in_channels, out_channels, kernel_size=kernel_size, stride=stride, bias=bias,
                         wt_levels=wt_levels, wt_type=wt_type)
        self._stride_filter_checked = None
        if stride > 1:
            self.stride_filter = nn.Parameter(torch.ones(in_channels, 1, 1, 1), requires_grad=False)

    def forward(self, x):
        f = getattr(self, "stride_filter", None)
        if f is not None:
            key = (f.data_ptr(), f._version)
            if key != self._stride_filter_checked:
                if not bool((f == 1).all()):
                    raise ValueError("stride_filter must be all ones: the kernels sub-sample without a filter")
                self._stride_filter_checked = key
        return super().forward(x)


def install(backbone_module):
    """Rebinds ``_WTConv2d`` in the reference's backbone module (the imported
    ``mmseg.models.backbones.wtconvnext``) and returns the class it replaced.  The block constructor
    looks the name up in its module globals at call time (wtconvnext.py:66), so every backbone built
    after this call holds B200 layers."""
    if not hasattr(backbone_module, "_WTConv2d"):
        raise AttributeError(f"{getattr(backbone_module, '__name__', backbone_module)!r} defines no _WTConv2d")
    previous = backbone_module._WTConv2d
    backbone_module._WTConv2d = MMSegWTConv2d
    return previous


_LAYER_NAMES = ("WTConv2d", "_WTConv2d")


def _is_reference_layer(m: nn.Module) -> bool:
    if isinstance(m, WTConv2d):
        return False
    return type(m).__name__ in _LAYER_NAMES and all(
        hasattr(m, a) for a in ("base_conv", "base_scale", "wavelet_convs", "wavelet_scale", "wt_levels"))


def _convert(old: nn.Module) -> WTConv2d:
    C = old.base_conv.in_channels
    K = old.base_conv.kernel_size[0]
    cls = MMSegWTConv2d if (type(old).__name__ == "_WTConv2d" or hasattr(old, "stride_filter")) else WTConv2d
    new = cls(C, C, kernel_size=K, stride=old.stride, bias=old.base_conv.bias is not None,
              wt_levels=old.wt_levels)
    # the reference layer's parameters become the new layer's parameters (same objects: an optimizer
    # or an EMA that already holds them keeps working)
    new.base_conv.weight = old.base_conv.weight
    if old.base_conv.bias is not None:
        new.base_conv.bias = old.base_conv.bias
    new.base_scale.weight = old.base_scale.weight
    for l in range(old.wt_levels):
        new.wavelet_convs[l].weight = old.wavelet_convs[l].weight
        new.wavelet_scale[l].weight = old.wavelet_scale[l].weight
    new.wt_filter = nn.Parameter(old.wt_filter.detach(), requires_grad=False)
    new.iwt_filter = nn.Parameter(old.iwt_filter.detach(), requires_grad=False)
    if hasattr(old, "stride_filter") and hasattr(new, "stride_filter"):
        new.stride_filter = old.stride_filter
    new.train(old.training)
    return new


def swap_layers(model: nn.Module) -> int:
    """Replaces, in place, every reference ``WTConv2d`` / ``_WTConv2d`` inside `model` by the B200
    layer holding the same parameter tensors.  Returns the number of layers replaced."""
    n = 0
    for parent in list(model.modules()):
        for name, child in list(parent.named_children()):
            if _is_reference_layer(child):
                setattr(parent, name, _convert(child))
                n += 1
    return n


def translate_to_mmseg(state_dict, prefix: str = "backbone."):
    """Classification checkpoint keys -> mmseg backbone keys
    (semantic_segmentation/translate_model_to_mmseg.py:8-40):

    ``stem.i.p``                          -> ``downsample_layers.0.i.p``
    ``stages.s.downsample.i.p``           -> ``downsample_layers.s.i.p``
    ``stages.s.blocks.b.gamma``           -> ``stages.s.b.gamma``
    ``stages.s.blocks.b.mlp.fc1|fc2.p``   -> ``stages.s.b.pointwise_conv1|2.p``
    ``stages.s.blocks.b.norm.p``          -> ``stages.s.b.norm.p``
    ``stages.s.blocks.b.conv_dw.<rest>``  -> ``stages.s.b.depthwise_conv.<rest>``

    everything under `prefix`.  Like the reference script, keys outside these groups (the
    classification head and its norm) are left out; unlike it, an unknown entry of a block raises
    instead of being printed, so a changed checkpoint layout cannot pass silently.  Values are the same
    tensor objects.
    """
    out = OrderedDict()
    for key, value in state_dict.items():
        sp = key.split(".")
        if sp[0] == "stem" and len(sp) >= 3:
            new = f"downsample_layers.0.{sp[1]}.{sp[2]}"
        elif sp[0] == "stages" and len(sp) >= 5 and sp[2] == "downsample":
            new = f"downsample_layers.{sp[1]}.{sp[3]}.{sp[4]}"
        elif sp[0] == "stages" and len(sp) >= 5 and sp[2] == "blocks":
            s, b, what = sp[1], sp[3], sp[4]
            if what == "gamma":
                new = f"stages.{s}.{b}.gamma"
            elif what == "mlp" and len(sp) >= 7 and sp[5] in ("fc1", "fc2"):
                new = f"stages.{s}.{b}.pointwise_conv{1 if sp[5] == 'fc1' else 2}.{sp[6]}"
            elif what == "norm" and len(sp) >= 6:
                new = f"stages.{s}.{b}.norm.{sp[5]}"
            elif what == "conv_dw":
                new = f"stages.{s}.{b}.depthwise_conv.{'.'.join(sp[5:])}"
            else:
                raise KeyError(f"unknown block entry in checkpoint key {key!r}")
        else:
            continue
        out[prefix + new] = value
    return out
