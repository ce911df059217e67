"""tdc_b200 — B200-native core convolution of Tucker-factorised conv layers.

The package is a thin host layer over libtdc_b200.so (hand-written sm_100a CUDA behind a
C ABI, see include/tdc_b200.h).  It mirrors the reference's operator surface for this
path: TKConv2dC (inference/TKConv.py:23-141) as TKConv2dC_B200, the (TH, TW, TC) tiling
parameters of its code generators as Tile, and its analytical tile selector
(A100-evaluation/TDC-LAYERS-MODELING/model.py) as select_tile.
"""
from ._lib import B200, EPI_NONE, EPI_RELU, LIB_PATH, W_CRSK, W_KCRS, DevInfo, LaunchInfo, TdcError, Tile, lib
from .ops import (affine_relu, conv2d, conv2d_epi, pool2d, tk_block_epi, core_conv2d, out_hw, permute_weights, query_device, select_tile, tile_cost, tile_info,
                  tk_block, tk_block_workspace_bytes)
from .tiles import best_tile, load_tables, table_tile
from .resnet import HalfRanks, HalfRanksBottleneck, TKBasicBlock, TKBottleneck, TKResNet, fill_deterministic, tkc_resnet18, tkc_resnet50
from .tc import TcConv
from .graph import GraphedForward
from .densenet import Growth32Ranks, TKDenseBlock, TKDenseLayer, TKDenseNet, TKDenseTransition, tkc_densenet121, tkc_densenet201, tkc_densenet264
from .svdconv import SVDConv2dC_B200, SVDConv2dM_B200, SVDConv2dR_B200, svd_factors
from .tkconv import TKConv2dC_B200
from .tkconv_variants import TKConv2dM_B200, TKConv2dR_B200
from .tucker import partial_tucker_hosvd, tucker_to_dense
from .vgg import HalfRanksVGG, TKVGG, tkc_vgg16

__all__ = [
    "affine_relu", "GraphedForward", "Growth32Ranks", "TKDenseBlock", "TKDenseLayer", "TKDenseNet", "TKDenseTransition", "tkc_densenet121", "tkc_densenet201",
    "tkc_densenet264", "SVDConv2dC_B200", "SVDConv2dM_B200", "SVDConv2dR_B200", "svd_factors",
    "B200", "DevInfo", "EPI_NONE", "EPI_RELU", "LIB_PATH", "LaunchInfo", "TKConv2dC_B200", "TKConv2dM_B200", "TKConv2dR_B200", "TKVGG", "HalfRanksVGG", "tkc_vgg16", "partial_tucker_hosvd",
    "tucker_to_dense", "TcConv", "TdcError", "Tile",
    "W_CRSK", "W_KCRS", "best_tile", "conv2d", "conv2d_epi", "pool2d", "tk_block_epi", "HalfRanks", "TKBasicBlock", "TKResNet",
    "fill_deterministic", "tkc_resnet18", "tkc_resnet50", "TKBottleneck", "HalfRanksBottleneck", "core_conv2d", "lib", "out_hw", "permute_weights", "query_device",
    "select_tile", "table_tile", "load_tables", "tile_cost", "tile_info", "tk_block", "tk_block_workspace_bytes",
]
from . import torch_ops  # registers torch.ops.tdc.core_conv2d / tk_block
