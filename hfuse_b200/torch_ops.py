"""Loads the PyTorch extension so that `torch.ops.hfuse_b200.*` exists.

    from hfuse_b200 import torch_ops          # registers the operators
    col, out, idx = torch.ops.hfuse_b200.im2col_maxpool(x, [3, 3], [1, 1], [1, 1], [1, 1], y, [2, 2], [2, 2], [0, 0], [1, 1])

The extension is a thin C++ layer over the C ABI (csrc/torch_ext.cpp); it must have been built
with `python -m hfuse_b200.build --torch-ext`.  Loading fails loudly when it is missing.
"""
import os

import torch

from . import _lib
from .build import TORCH_EXT

if not os.path.exists(TORCH_EXT):
    raise ImportError(f"{TORCH_EXT} is missing: build it with `python -m hfuse_b200.build --torch-ext`")
_lib.lib()                       # libhfuse_b200.so first, so the extension's dependency resolves
torch.ops.load_library(TORCH_EXT)
ops = torch.ops.hfuse_b200
