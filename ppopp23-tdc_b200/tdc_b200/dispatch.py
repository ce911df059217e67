"""Which kernel runs one convolution: shared by the network assemblies and the Tucker module.

`precision`: "fp32" = the fp32 FMA kernel always (bit-reproducible); "fp16x3" / "tf32x3" / "tf32" = tensor cores
wherever a plan exists (operands split into two fp16 or two TF32 parts: fp32-level results; plain TF32);
"auto" = tensor cores with split operands (AUTO_MODE) where the layer has enough work to fill the GPU, the fp32 FMA
kernel with its measured-table tile otherwise.
"""
from . import ops, tiles
from ._lib import W_CRSK

# tensor-core mode of each precision name (tdc_tc_plan.mode)
MODES = {"tf32": 1, "tf32x3": 3, "fp16x3": 4}
AUTO_MODE = 4          # what "auto" runs on tensor cores: split fp16 operands (twice the MMA rate of split TF32, half the
                       # accumulations per output, inputs must lie within fp16's range of +-65504)


def one_conv(owner, name, x, w_kcrs, w_crsk, scale, shift, residual, relu, stride, padding, precision):
    """One convolution with its epilogue on the kernel that suits it: tensor cores (3xTF32) for
    stride-1 3x3 and any 1x1 layers with enough work to fill the GPU when `precision` allows, the fp32
    kernel with a table tile otherwise."""
    from . import tc
    B, Cc, H, W = x.shape
    K, _, R, S = w_kcrs.shape
    one_pass = tc.supported(R, S, stride, padding, W)
    if precision != "fp32" and one_pass and \
            (precision != "auto" or tc.worthwhile(B, Cc, (H - 1) // stride + 1, (W - 1) // stride + 1, K, R)):
        return tc.cached(owner, name, w_kcrs, MODES.get(precision, AUTO_MODE))(x, scale, shift, residual, relu, stride=stride)
    Ho, Wo = (H + 2 * padding - R) // stride + 1, (W + 2 * padding - S) // stride + 1
    if precision != "fp32" and not one_pass and tc.general_supported(R, S, stride, padding, Wo) and \
            (precision != "auto" or (2.0 * B * Ho * Wo * Cc * K * R * S >= 0.5e9 and B * Ho * Wo >= 256 * 128)):
        # strided 3x3 cores, the 7x7 stem: the gathering plan (under "auto" only with at least 256 position tiles:
        # it pays per channel block and tile, and with few tiles the fp32 kernel's slices and clusters win)
        return tc.cached(owner, name, w_kcrs, MODES.get(precision, AUTO_MODE), general=True)(
            x, scale, shift, residual, relu, stride=stride, padding=padding)
    tile = tiles.table_tile(B, Cc, H, W, K, R, S, padding, stride)
    if w_crsk is not None:
        if callable(w_crsk):          # made (and cached by the owner) only when this path is taken
            w_crsk = w_crsk()
        return ops.conv2d_epi(x, w_crsk, scale, shift, residual, relu, stride, padding, w_layout=W_CRSK, tile=tile)
    return ops.conv2d_epi(x, w_kcrs.detach(), scale, shift, residual, relu, stride, padding, tile=tile)
