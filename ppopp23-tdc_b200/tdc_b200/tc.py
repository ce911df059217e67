"""Tensor-core variant of the core convolution (tcgen05, TF32 or fp16 operands) — host side.

`TcConv` holds what the C ABI needs per layer: the plan (tdc_tc_plan_make) and the filter
pre-arranged for the kernel (tdc_tc_prepare_weights).  mode 3 ("3xTF32") and mode 4 ("3xFP16")
give fp32-level results; mode 1 is plain TF32.  Mode 4 scales its input into fp16's range and needs
the input's largest magnitude for that: every mode-4 output carries the partial maxima of its own
magnitudes as the attribute `_tdc_absmax`, and a mode-4 call whose input carries one skips the pass
over the input that would otherwise find it (the three steps of a Tucker conv chain this way).  The default plan serves "same" convolutions with 1x1 or 3x3 filters
and stride 1 (1x1 filters also strided) and reads the input once; `general=True` makes the plan that
takes any filter size, stride and padding by gathering (channel, row, column) triples.
"""
import ctypes as C

import torch

from . import _lib
from ._lib import TcPlan, TdcError, lib
from .ops import _dev_f32, _epilogue, _on_device, _stream


ABSMAX_FLOATS = 1024      # TDC_TC_ABSMAX_FLOATS


def _check(code):
    if code != _lib.OK:
        raise TdcError(code, lib.tdc_tc_last_error_string().decode())


class TcConv:
    def __init__(self, weight, mode=3, w_layout=_lib.W_KCRS, general=False, exact_range=False, unbiased=False):
        """weight: [K][C][R][S] (or [C][R][S][K] with w_layout=W_CRSK), fp32 CUDA tensor.  `exact_range` (mode 4): take
        the input's scale from its true maximum (a pass over the input per call) instead of from a sample.  `unbiased`
        (modes 3, 4): put back the expected loss of the tensor core's truncating accumulation (TDC_TC_UNBIASED); sums of
        small integers are then no longer exact."""
        self.exact_range, self.unbiased = bool(exact_range), bool(unbiased)
        if w_layout == _lib.W_KCRS:
            K, Cc, R, S = weight.shape
        else:
            Cc, R, S, K = weight.shape
        self.plan = TcPlan()
        _check((lib.tdc_tc_plan_make_general if general else lib.tdc_tc_plan_make)(Cc, K, R, S, mode, C.byref(self.plan)))
        self.C, self.K, self.R, self.S, self.mode, self.general = Cc, K, R, S, mode, bool(general)
        self._weight, self._w_layout = weight, w_layout
        self.wt = self._prepare(self.plan)
        self._by_nt = {(self.plan.nt, None): (self.plan, self.wt)}  # (output-channel block size, strided-row (stride, padding parity)) -> (plan, prepared filter)
        self._sms = torch.cuda.get_device_properties(weight.device).multi_processor_count
        self._nt_of = {}                                         # (batch, image, flags) -> block size (the rules are library calls)

    def _prepare(self, plan):
        wt = torch.empty(plan.weights_bytes, dtype=torch.uint8, device=self._weight.device)
        with torch.cuda.device(self._weight.device):
            _check(lib.tdc_tc_prepare_weights(C.byref(plan), _dev_f32(self._weight, "weight"), self._w_layout,
                                              wt.data_ptr(), _stream()))
        return wt

    def _make_plan(self, nt, rows):
        plan = TcPlan()
        if rows:
            _check(lib.tdc_tc_plan_make_strided(self.C, self.K, self.R, self.S, rows[0], rows[1], self.mode, nt, C.byref(plan)))
        else:
            _check(lib.tdc_tc_plan_make_nt(self.C, self.K, self.R, self.S, self.mode, int(self.general), nt, C.byref(plan)))
        return plan

    def _for_image(self, B, H, W, Ho, Wo, flags, rows=None):
        """(plan, prepared filter) with the output-channel block size that suits this layer: the default for layers with
        many position tiles, smaller blocks (more CTAs) for few, and smaller again while the block does not leave room
        for two stages beside the patch of a wide image; prepared on first use.  `rows` = (stride, parity of the padding):
        the strided-row plan for them instead of the triple-gathering one."""
        halo = 0 if self.general else (self.R - 1) // 2
        key = (B, H, W, flags, rows)
        nt = self._nt_of.get(key)
        if nt is None:
            nt = lib.tdc_tc_pick_nt(self.K, self.mode, B * (Ho + halo) * (Wo + halo), self._sms)
            while nt > 32:
                plan = self._make_plan(nt, rows)
                if lib.tdc_tc_check_launch(C.byref(plan), B, H, W, flags & 0xFF) != _lib.ERR_SMEM:
                    break
                nt //= 2
            self._nt_of[key] = nt
        hit = self._by_nt.get((nt, rows))
        if hit is None:
            plan = self._make_plan(nt, rows)
            hit = self._by_nt[(nt, rows)] = (plan, self._prepare(plan))
        return hit

    def __call__(self, x, scale=None, bias=None, residual=None, relu=False, out=None, stride=1, padding=None):
        """`stride` > 1 is taken for 1x1 filters (the down-sampling shortcut of a residual stage) and by general
        plans, which also take any `padding` (the others pad (R-1)/2)."""
        B, Cc, H, W = x.shape
        if Cc != self.C:
            raise TdcError(_lib.ERR_SHAPE, "x has %d channels, the filter expects %d" % (Cc, self.C))
        if not 1 <= stride <= 16:
            raise TdcError(_lib.ERR_UNSUPPORTED, "stride %d" % stride)
        flags = stride - 1
        if self.general:
            padding = 0 if padding is None else padding
            if not 0 <= padding <= 15:
                raise TdcError(_lib.ERR_UNSUPPORTED, "padding %d" % padding)
            flags |= padding << 4
            Ho, Wo = (H + 2 * padding - self.R) // stride + 1, (W + 2 * padding - self.S) // stride + 1
        else:
            if padding is not None and padding != (self.R - 1) // 2:
                raise TdcError(_lib.ERR_UNSUPPORTED, "this plan pads (R-1)/2; make it with general=True for padding %d" % padding)
            Ho, Wo = (H - 1) // stride + 1, (W - 1) // stride + 1
        if out is None:
            out = torch.empty((B, self.K, Ho, Wo), device=x.device, dtype=torch.float32)
        e = _epilogue(scale, bias, residual, relu)
        # strided filters 2 or 4 strides wide (the 3x3 stride-2 cores, the 7x7 stride-2 stem): the strided-row plan, whose
        # loaders gather C*R*stride values per position instead of C*R*S
        rows = (stride, padding & 1) if (self.general and self.mode == 4 and strided_rows(self.S, stride)) else None
        plan, wt = self._for_image(B, H, W, Ho, Wo, flags, rows)
        if self.unbiased and self.mode != 1:
            flags |= 0x200                        # TDC_TC_UNBIASED
        if self.mode != 4:
            with _on_device(x.device):
                _check(lib.tdc_conv2d_tc(C.byref(plan), _dev_f32(x, "x"), wt.data_ptr(), _dev_f32(out, "out"),
                                         B, H, W, C.byref(e), flags, _stream()))
            return out
        xmax = getattr(x, "_tdc_absmax", None)
        if xmax is None and self.exact_range:
            flags |= 0x100                        # TDC_TC_EXACT_RANGE
        ymax = torch.empty(ABSMAX_FLOATS, device=x.device, dtype=torch.float32)
        with _on_device(x.device):
            _check(lib.tdc_conv2d_tc_ranged(C.byref(plan), _dev_f32(x, "x"), wt.data_ptr(), _dev_f32(out, "out"),
                                            B, H, W, C.byref(e), flags, xmax.data_ptr() if xmax is not None else None,
                                            ymax.data_ptr(), _stream()))
        out._tdc_absmax = ymax
        return out


def supported(R, S, stride, padding, W):
    """True when the tensor-core variant is built for this convolution."""
    return R == S and R in (1, 3) and (stride == 1 or (R == 1 and 1 <= stride <= 16)) and padding == (R - 1) // 2 and W <= 256 * stride


def general_supported(R, S, stride, padding, Wo):
    """True when a general plan (any filter, stride, padding) can run this convolution."""
    return 1 <= R <= 15 and 1 <= S <= 15 and 1 <= stride <= 16 and 0 <= padding <= 15 and Wo <= 256


def strided_rows(S, stride):
    """True when a strided convolution takes the plan that gathers (channel, filter row, column phase) and runs the
    column steps as 2 or 4 MMA taps (fp16 parts only): 3-wide to 8-wide filters at stride 2, for instance."""
    return stride >= 2 and -(-S // stride) in (2, 4)


def worthwhile(B, C, H, W, K, R):
    """The tensor-core kernel works on tiles of 128 positions x up to 128 channels; with too few position tiles or too
    little arithmetic the fp32 kernel with its channel slices and clusters is the faster one.  The thresholds are a fit
    to 420 layers (3x3 and 1x1, 32..2048 channels, 7..56 pixels, batch 1..64) timed on both paths in one run
    (tests/golden/tc_vs_fp32_times_b200.json, which a CPU test holds the rule to).  A 3x3
    layer wants 3 position tiles and 0.1 GFLOP: 0.2 % from always taking the faster path.  A 1x1 layer with few tiles
    is one CTA walking all input channels, about 12 us + 0.085 us per channel whatever the tile count, while the fp32
    kernel's time follows the arithmetic; the three cases below are 1.2 % from the faster path (the thresholds they
    replace, which asked for 12..24 tiles: 4.3 %), and on CUDA-graphed forwards at batch 1..16 they are never slower
    and up to 23 % faster (TK-ResNet-50 at batch 4: 2.50 -> 1.91 ms; TK-DenseNet-121 at batch 8: 4.70 -> 3.65 ms)."""
    pad = (R - 1) // 2
    flops, positions = 2.0 * B * H * W * C * K * R * R, B * (H + pad) * (W + pad)
    if R == 1:
        tiles = positions / 128.0
        return (tiles >= 4 and flops >= 0.02e9) or (C <= 512 and flops >= 0.2e9) or \
               (tiles >= 3 and K >= 2 * C and flops >= 0.1e9)
    return flops >= 0.1e9 and positions >= 3 * 128


def cached(owner, name, weight, mode, w_layout=_lib.W_KCRS, general=False):
    """TcConv for `weight`, kept on the module that owns the weight (`owner`) under `name`, and
    rebuilt when the tensor is written to or replaced (version / storage check).  Keeping it on the
    owner — not in a table keyed by address — means a freed network's entries can never be taken
    for those of a new network whose weights happen to land on the same addresses.  These are the convolutions of the
    modules and networks, which chain many layers: they run with `unbiased` set."""
    store = owner.__dict__.setdefault("_tc_convs", {})
    key = (weight._version, weight.data_ptr(), tuple(weight.shape))
    hit = store.get((name, mode, w_layout, general))
    if hit is None or hit[0] != key:
        hit = store[(name, mode, w_layout, general)] = (key, TcConv(weight.detach(), mode, w_layout, general, unbiased=True))
    return hit[1]


def status():
    """Device status word of the tensor-core kernels (synchronises): 0 = no bounded wait ran out."""
    s = C.c_int(-1)
    _check(lib.tdc_tc_status(C.byref(s)))
    return s.value
