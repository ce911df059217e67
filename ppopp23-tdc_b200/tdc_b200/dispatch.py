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
    """One convolution with its epilogue on the kernel that suits it: tensor cores for every layer a plan exists for
    when `precision` names them, under "auto" only where `_on_tensor_cores` says the layer has the work for them; the
    fp32 FMA kernel with a table tile otherwise."""
    from . import tc
    B, Cc, H, W = x.shape
    K, _, R, S = w_kcrs.shape
    one_pass = tc.supported(R, S, stride, padding, W)
    Ho, Wo = (H + 2 * padding - R) // stride + 1, (W + 2 * padding - S) // stride + 1
    if precision != "fp32" and (one_pass or tc.general_supported(R, S, stride, padding, Wo)) and \
            (precision != "auto" or _auto_path(owner, name, B, Cc, K, H, W, R, S, stride, padding)):
        mode = MODES.get(precision, AUTO_MODE)
        if one_pass and not _thin_and_wide(Cc, W, R, stride):
            return tc.cached(owner, name, w_kcrs, mode)(x, scale, shift, residual, relu, stride=stride)
        return tc.cached(owner, name, w_kcrs, mode, general=True)(x, scale, shift, residual, relu, stride=stride, padding=padding)
    tile = tiles.table_tile(B, Cc, H, W, K, R, S, padding, stride)
    if w_crsk is not None:
        if callable(w_crsk):          # made (and cached by the owner) only when this path is taken
            w_crsk = w_crsk()
        return ops.conv2d_epi(x, w_crsk, scale, shift, residual, relu, stride, padding, w_layout=W_CRSK, tile=tile)
    return ops.conv2d_epi(x, w_kcrs.detach(), scale, shift, residual, relu, stride, padding, tile=tile)


def _auto_path(owner, name, *shape):
    """`_on_tensor_cores` for this layer and shape, remembered on the module that owns the weight: the answer depends on
    shapes only, and a batch-1 forward would otherwise spend more host time on it than the launch costs."""
    memo = owner.__dict__.setdefault("_auto_paths", {})
    hit = memo.get((name, shape))
    if hit is None:
        hit = memo[(name, shape)] = _on_tensor_cores(*shape)
    return hit


def _thin_and_wide(Cc, W, R, stride):
    """A 3x3 layer with very few input channels on a wide image (the first layer of a VGG: 3 -> 64 at 224x224): the one-pass
    plan stages whole 16-channel blocks and, with two image rows of halo per 128-position tile, 4.5 times the rows it
    needs; gathering the 9*C values of each position instead is the cheaper load (batch 64: C = 3: 308 against 820 us,
    C = 8: 588 against 820, C = 16: 942 against 821; cuDNN 686 / 1321 / 2148)."""
    return R == 3 and stride == 1 and Cc <= 8 and W >= 128


def _on_tensor_cores(B, Cc, K, H, W, R, S, stride, padding):
    """Whether "auto" sends this convolution to tensor cores."""
    from . import tc
    Ho, Wo = (H + 2 * padding - R) // stride + 1, (W + 2 * padding - S) // stride + 1
    if tc.supported(R, S, stride, padding, W):
        if _thin_and_wide(Cc, W, R, stride):
            return B * H * W >= 64 * 128
        # the measured crossovers of the one-pass plans against the fp32 kernel
        return tc.worthwhile(B, Cc, (H - 1) // stride + 1, (W - 1) // stride + 1, K, R)
    if not tc.general_supported(R, S, stride, padding, Wo):
        return False
    flops, positions = 2.0 * B * Ho * Wo * Cc * K * R * S, B * Ho * Wo
    if tc.strided_rows(S, stride):
        # stride 2 with a 3- or 7-wide filter: the plan that gathers (channel, filter row, column phase) and takes the
        # column steps as MMA taps.  Measured against the fp32 kernel at batch 256 / 32: stem 485 / 76 us against
        # 1794 / 250 (batch 1: 16 against 20); 32->64 at 56: 93 / 39 against 257 / 49; 128->256 at 14: 126 / 64
        # against 258 / 59
        return flops >= 0.2e9 and positions >= 64 * 128
    # every (channel, filter row, filter column) gathered: it pays per channel block and tile, and with few tiles the
    # fp32 kernel's slices and clusters win
    return flops >= 0.5e9 and positions >= 256 * 128


def _conv_us(B, Cc, K, Ho, Wo, R, stride=1, on_tc=True):
    """Rough time of one convolution in microseconds: a fixed part per launch plus the slower of arithmetic (on the
    tensor-core path at the rates the sweep shapes reach: they rise with the output channels per MMA; on the fp32 FMA
    kernel at its measured 30 TFLOP/s) and the memory passes over input and output.  Only good for comparing ways to
    run the same layer."""
    flops = 2.0 * B * Ho * Wo * Cc * K * R * R
    nbytes = 4.0 * B * (Cc * Ho * Wo * stride * stride + K * Ho * Wo)
    # what the memory passes reach: 2.5 TB/s on layers of ~150 MB, rising to 3.7 TB/s on the very large ones
    # (128 -> 64 1x1 at 28x28, batch 256: 154 MB in 55 us; at 112x112, batch 64: 616 MB in ~160 us)
    mem_rate = 2.5e12 * min(1.5, max(1.0, (nbytes / 150e6) ** 0.25))
    if not on_tc:
        return 8.0 + max(flops / 30e12 * 1e6, nbytes / mem_rate * 1e6)
    if stride > 1 and R > 1:
        rate = 150e12                                  # the gathering plans are bound by their loaders
    elif R > 1:
        rate = 330e12 if K >= 128 else (240e12 if K >= 64 else 110e12)
    else:
        rate = 200e12 if K >= 128 else (150e12 if K >= 64 else 80e12)
    # a CTA walks the channel blocks of a tile one after the other, about 0.1 us per (16 channels x tap) with blocks of
    # 128 output channels (half that with smaller ones): with few tiles this chain, not the arithmetic, is the time
    nt = 128 if K > 64 else 64
    tiles = -(-(B * (Ho + (R > 1)) * (Wo + (R > 1))) // 256) * -(-K // nt)
    # (a one-tap filter pays per block what a 3x3 pays for its nine taps: the hand-over of the stage, not the MMAs)
    serial = -(-tiles // 148) * (Cc / 16.0) * (R * R if R > 1 else 8) * (0.1 if nt == 128 else 0.05)
    return 12.0 + max(flops / rate * 1e6, nbytes / mem_rate * 1e6, serial)


def tucker_strategy(conv, x, precision):
    """"dense" or "chain" for a Tucker conv (first 1x1, core, last 1x1).  The dense form (one conv with the factors
    multiplied into one filter, `TKConv2dC_B200._dense_weight`) does 9CK multiply-adds per pixel where the chain does
    C*R1 + 9*R1*R2 + R2*K, but it is one launch with no intermediate: measured on the bottleneck middles C = K = 64..512,
    R = C/2, batch 32: 39 / 38 / 35 / 59 us against 71 / 63 / 57 / 97 us for the chain (batch 1: 16 / 18 / 27 / 57 against
    36 / 40 / 48 / 91).  Taken under "auto" only (the named precisions run the factored form as written), when the
    estimate says it is faster by a twentieth at least.  Each form is priced on the kernel `one_conv` would run it on:
    a strided layer with few positions stays on the fp32 FMA kernel, where the merged filter is no bargain (256 -> 512 at
    14x14, stride 2, batch 32: 341 us merged, 107 us as the chain)."""
    if precision != "auto":
        return "chain"
    memo = conv.__dict__.setdefault("_strategies", {})     # the choice depends on shapes only
    hit = memo.get(tuple(x.shape))
    if hit is None:
        hit = memo[tuple(x.shape)] = _tucker_strategy(conv, x)
    return hit


def _tucker_strategy(conv, x):
    from . import tc
    B, Cc, H, W = x.shape
    R, S = conv.kernel_size
    stride, pad = conv.stride[0], conv.padding[0]
    if R != S or conv.stride[0] != conv.stride[1] or conv.padding[0] != conv.padding[1]:
        return "chain"
    Ho, Wo = (H + 2 * pad - R) // stride + 1, (W + 2 * pad - S) // stride + 1
    K, R1, R2 = conv.out_channels, conv.in_rank, conv.out_rank
    if not (tc.supported(R, S, stride, pad, W) or tc.general_supported(R, S, stride, pad, Wo)):
        return "chain"
    # each form at the speed of the kernel `one_conv` would give it: a strided layer with few positions, for one, stays on
    # the fp32 FMA kernel, where the merged filter's 9*C*K multiply-adds per pixel cost their full price
    dense = _conv_us(B, Cc, K, Ho, Wo, R, stride, _on_tensor_cores(B, Cc, K, H, W, R, S, stride, pad))
    chain = _conv_us(B, Cc, R1, H, W, 1, 1, _on_tensor_cores(B, Cc, R1, H, W, 1, 1, 1, 0)) + \
        _conv_us(B, R1, R2, Ho, Wo, R, stride, _on_tensor_cores(B, R1, R2, H, W, R, S, stride, pad)) + \
        _conv_us(B, R2, K, Ho, Wo, 1, 1, _on_tensor_cores(B, R2, K, Ho, Wo, 1, 1, 1, 0))
    return "dense" if dense <= 0.95 * chain else "chain"
