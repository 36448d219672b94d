"""Inference-only WTConvNeXt-T harness (timm-free) around the WTConv2d layers.

This is NOT a re-implementation of the reference model zoo: timm is not
installable offline, so `wtconvnext/wtconvnext.py` cannot be imported on either
machine.  The harness restates just the inference forward of the tiny variant
with plain `torch.nn` so that 18 WTConv2d layers sit between the standard
PyTorch ops they sit between in the reference, for the images/sec measurement
and for a model-level parity check (same harness with two different layer
classes, so any restatement difference cancels).

Structure followed (reference file wtconvnext/wtconvnext.py):
  stem ............ Conv2d 4x4 stride 4 + channel LayerNorm          :292-297
  downsample ...... channel LayerNorm + Conv2d 2x2 stride 2           :167-181
  block ........... conv_dw -> NHWC LayerNorm -> Linear 4x -> GELU -> Linear
                    -> layer scale gamma -> + shortcut                :125-140
  head ............ global average pool -> LayerNorm -> Linear        :360-368
  init ............ trunc_normal(0.02) weights, zero biases           :483-493
  tiny variant .... depths (3,3,9,3), dims (96,192,384,768), kernel 5,
                    wt_levels (5,4,3,2)                                :227-244,570-574
Parameter count pin: 30 595 624 (logs/val_tiny.out:4).
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

DEPTHS = (3, 3, 9, 3)
DIMS = (96, 192, 384, 768)
WT_LEVELS = (5, 4, 3, 2)


class _ChannelNorm(nn.LayerNorm):
    """LayerNorm over the channel dimension of an NCHW tensor."""

    def forward(self, x):
        x = x.permute(0, 2, 3, 1)
        x = F.layer_norm(x, self.normalized_shape, self.weight, self.bias, self.eps)
        return x.permute(0, 3, 1, 2)


class _Block(nn.Module):
    def __init__(self, dim, wt_levels, conv_cls):
        super().__init__()
        self.conv_dw = conv_cls(dim, dim, kernel_size=5, stride=1, bias=True, wt_levels=wt_levels)
        self.norm = nn.LayerNorm(dim, eps=1e-6)
        self.fc1 = nn.Linear(dim, 4 * dim)
        self.fc2 = nn.Linear(4 * dim, dim)
        self.gamma = nn.Parameter(1e-6 * torch.ones(dim))

    def forward(self, x):
        y = self.conv_dw(x).permute(0, 2, 3, 1)
        y = self.fc2(F.gelu(self.fc1(self.norm(y))))
        return (y * self.gamma).permute(0, 3, 1, 2) + x


class WTConvNeXtTiny(nn.Module):
    def __init__(self, conv_cls, num_classes=1000):
        super().__init__()
        self.stem = nn.Sequential(nn.Conv2d(3, DIMS[0], 4, stride=4), _ChannelNorm(DIMS[0], eps=1e-6))
        stages, prev = [], DIMS[0]
        for dim, depth, lv in zip(DIMS, DEPTHS, WT_LEVELS):
            layers = []
            if dim != prev:
                layers += [_ChannelNorm(prev, eps=1e-6), nn.Conv2d(prev, dim, 2, stride=2)]
            layers += [_Block(dim, lv, conv_cls) for _ in range(depth)]
            stages.append(nn.Sequential(*layers))
            prev = dim
        self.stages = nn.Sequential(*stages)
        self.head_norm = nn.LayerNorm(prev, eps=1e-6)
        self.head_fc = nn.Linear(prev, num_classes)
        for m in self.modules():
            if isinstance(m, (nn.Conv2d, nn.Linear)):
                nn.init.trunc_normal_(m.weight, std=0.02)
                if m.bias is not None:
                    nn.init.zeros_(m.bias)

    def forward(self, x):
        x = self.stages(self.stem(x))
        return self.head_fc(self.head_norm(x.mean((2, 3))))


class CapturedForward:
    """Whole-model inference forward captured once into a CUDA graph and replayed per batch.

    The WTConv2d layers plan their launch chain on the host for every call; at small batches that
    planning and the 18 x (3..6) launches cost more than the kernels.  Capturing the forward of a fixed
    input shape removes all of it: `__call__` copies the batch into the graph's input buffer, replays,
    and returns the graph's output buffer (valid until the next call).  Parameters are read in place
    by the replay; the folded parameter blocks of the WTConv2d layers are NOT refreshed by it, so
    capture again after changing weights.
    """

    def __init__(self, model: nn.Module, example: torch.Tensor, warmup: int = 3):
        if not example.is_cuda:
            raise ValueError("CapturedForward needs a CUDA example input")
        self.model = model
        self.static_in = example.clone(memory_format=torch.preserve_format)
        side = torch.cuda.Stream(device=example.device)
        side.wait_stream(torch.cuda.current_stream(example.device))
        with torch.no_grad(), torch.cuda.stream(side):
            for _ in range(max(1, warmup)):       # packs parameters, plans chains, sets kernel attributes
                model(self.static_in)
        torch.cuda.current_stream(example.device).wait_stream(side)
        torch.cuda.synchronize(example.device)
        self.graph = torch.cuda.CUDAGraph()
        with torch.no_grad(), torch.cuda.graph(self.graph):
            self.static_out = model(self.static_in)

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        if x.shape != self.static_in.shape or x.dtype != self.static_in.dtype:
            raise ValueError(f"captured for {tuple(self.static_in.shape)} {self.static_in.dtype}, "
                             f"got {tuple(x.shape)} {x.dtype}")
        self.static_in.copy_(x, non_blocking=True)
        self.graph.replay()
        return self.static_out
