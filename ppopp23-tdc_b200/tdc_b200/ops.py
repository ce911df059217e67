"""Torch-facing operators over the C ABI.  Tensors only lend their device pointers and the
current stream; all arithmetic happens in libtdc_b200.so.  Inputs must be CUDA, fp32 and
contiguous — anything else raises (there is no fallback path)."""
import ctypes as C

import torch

from . import _lib
from ._lib import EPI_NONE, EPI_RELU, W_CRSK, W_KCRS, DevInfo, LaunchInfo, TdcError, Tile, check, lib


def _pair(v):
    if isinstance(v, (tuple, list)):
        if len(v) != 2 or v[0] != v[1]:
            raise TdcError(_lib.ERR_UNSUPPORTED, "only equal vertical/horizontal %r is built" % (v,))
        return int(v[0])
    return int(v)


def _dev_f32(t, name):
    if not isinstance(t, torch.Tensor) or not t.is_cuda or t.dtype != torch.float32 or not t.is_contiguous():
        raise TdcError(_lib.ERR_UNSUPPORTED, "%s must be a contiguous fp32 CUDA tensor" % name)
    return t.data_ptr()


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream():
    """The current CUDA stream of the current device as the integer the C ABI takes (the raw query where this torch has
    it: a tenth of the host time of building a Stream object, and a batch-1 forward asks some twenty times)."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


class _on_device:
    """`with _on_device(t.device):` — torch.cuda.device() only when the tensor's GPU is not the current one (the
    context manager costs more host time than a small launch)."""
    __slots__ = ("ctx",)

    def __init__(self, device):
        idx = device.index
        self.ctx = None if idx is None or idx == torch.cuda.current_device() else torch.cuda.device(device)

    def __enter__(self):
        if self.ctx is not None:
            self.ctx.__enter__()

    def __exit__(self, *exc):
        if self.ctx is not None:
            return self.ctx.__exit__(*exc)
        return False


def out_hw(H, W, R, S, pad, stride):
    return (H + 2 * pad - R) // stride + 1, (W + 2 * pad - S) // stride + 1


def permute_weights(w_kcrs):
    """[K][C][R][S] -> [C][R][S][K], the layout the kernel stages with 16-byte copies
    (the reference kernel's own k[c][r][s][n],
    A100-evaluation/TDC-LAYERS-ORACLE/template_benchmark_cudnn.template:396)."""
    K, Cc, R, S = w_kcrs.shape
    out = torch.empty((Cc, R, S, K), device=w_kcrs.device, dtype=torch.float32)
    with torch.cuda.device(w_kcrs.device):
        check(lib.tdc_permute_weights(_dev_f32(w_kcrs, "w"), out.data_ptr(), K, Cc, R, S, _stream()))
    return out


def conv2d(x, w, bias=None, stride=1, padding=0, w_layout=W_KCRS, relu=False, tile=None, out=None):
    """y = conv2d(x, w) (+bias)(ReLU). The core step of TKConv2dC.forward
    (inference/TKConv.py:92-93) when bias is None; with R=S=1 its first/last step (:91,:94)."""
    stride, padding = _pair(stride), _pair(padding)
    B, Cc, H, W = x.shape
    if w_layout == W_KCRS:
        K, Cw, R, S = w.shape
    else:
        Cw, R, S, K = w.shape
    if Cw != Cc:
        raise TdcError(_lib.ERR_SHAPE, "x has %d channels, w expects %d" % (Cc, Cw))
    Ho, Wo = out_hw(H, W, R, S, padding, stride)
    if out is None:
        out = torch.empty((B, K, max(Ho, 0), max(Wo, 0)), device=x.device, dtype=torch.float32)
    tp = C.byref(tile) if tile is not None else None
    with _on_device(x.device):
        check(lib.tdc_conv2d_f32(_dev_f32(x, "x"), _dev_f32(w, "w"),
                                 _dev_f32(bias, "bias") if bias is not None else None, _dev_f32(out, "out"),
                                 B, Cc, H, W, K, R, S, padding, stride, w_layout,
                                 EPI_RELU if relu else EPI_NONE, tp, _stream()))
    return out


def core_conv2d(x, w, stride=1, padding=0, w_layout=W_KCRS, tile=None, out=None):
    """The hot path through tdc_core_conv2d_f32 (no bias, no activation)."""
    stride, padding = _pair(stride), _pair(padding)
    B, Cc, H, W = x.shape
    if w_layout == W_KCRS:
        K, Cw, R, S = w.shape
    else:
        Cw, R, S, K = w.shape
    if Cw != Cc:
        raise TdcError(_lib.ERR_SHAPE, "x has %d channels, w expects %d" % (Cc, Cw))
    Ho, Wo = out_hw(H, W, R, S, padding, stride)
    if out is None:
        out = torch.empty((B, K, max(Ho, 0), max(Wo, 0)), device=x.device, dtype=torch.float32)
    tp = C.byref(tile) if tile is not None else None
    with _on_device(x.device):
        check(lib.tdc_core_conv2d_f32(_dev_f32(x, "x"), _dev_f32(w, "w"), _dev_f32(out, "out"),
                                      B, Cc, H, W, K, R, S, padding, stride, w_layout, tp, _stream()))
    return out


def tk_block_workspace_bytes(B, Cc, H, W, R1, R2, K, R, S, pad, stride):
    return lib.tdc_tk_block_workspace_bytes(B, Cc, H, W, R1, R2, K, R, S, pad, stride)


def tk_block(x, first, core, last, bias=None, stride=1, padding=0, core_layout=W_KCRS, relu=False,
             workspace=None, out=None, core_tile=None):
    """TKConv2dC.forward (inference/TKConv.py:90-95): 1x1 C->R1, core R1->R2, 1x1 R2->K + bias.
    `first` is [R1][C][1][1] (or [R1][C]), `last` is [K][R2][1][1] (or [K][R2])."""
    stride, padding = _pair(stride), _pair(padding)
    B, Cc, H, W = x.shape
    R1, K = first.shape[0], last.shape[0]
    if core_layout == W_KCRS:
        R2, R1c, R, S = core.shape
    else:
        R1c, R, S, R2 = core.shape
    if first.shape[1] != Cc or R1c != R1 or last.shape[1] != R2:
        raise TdcError(_lib.ERR_SHAPE, "Tucker factors do not chain: first %s core %s last %s" %
                       (tuple(first.shape), tuple(core.shape), tuple(last.shape)))
    Ho, Wo = out_hw(H, W, R, S, padding, stride)
    need = tk_block_workspace_bytes(B, Cc, H, W, R1, R2, K, R, S, padding, stride)
    if workspace is None:
        workspace = torch.empty(need, device=x.device, dtype=torch.uint8)
    if out is None:
        out = torch.empty((B, K, Ho, Wo), device=x.device, dtype=torch.float32)
    with _on_device(x.device):
        check(lib.tdc_tk_block_f32(_dev_f32(x, "x"), _dev_f32(first, "first"), _dev_f32(core, "core"),
                                   _dev_f32(last, "last"), _dev_f32(bias, "bias") if bias is not None else None,
                                   _dev_f32(out, "out"), B, Cc, H, W, R1, R2, K, R, S, padding, stride,
                                   core_layout, EPI_RELU if relu else EPI_NONE,
                                   C.byref(core_tile) if core_tile is not None else None, workspace.data_ptr(), workspace.numel() * workspace.element_size(), _stream()))
    return out


def _epilogue(scale, bias, residual, relu):
    e = _lib.Epilogue()
    e.scale = _dev_f32(scale, "scale") if scale is not None else None
    e.bias = _dev_f32(bias, "bias") if bias is not None else None
    e.residual = _dev_f32(residual, "residual") if residual is not None else None
    e.relu = 1 if relu else 0
    return e


POOL_MAX, POOL_AVG_INCLUDE_PAD, POOL_AVG_EXCLUDE_PAD = 0, 1, 2


def pool2d(x, kernel_size, stride=None, padding=0, mode=POOL_MAX, out=None):
    """The pooling layer of the end-to-end skeleton (Pool::initialize / Pool::forward,
    A100-evaluation/EndToEnd/resnet18-tk/src/Pool.cu:8-48; nn.MaxPool2d(3, 2, 1) in
    inference/resnet_inet_tt.py:323): x [B][C][H][W] -> [B][C][Ho][Wo]."""
    kh, kw = (int(v) for v in kernel_size) if isinstance(kernel_size, (tuple, list)) else (int(kernel_size),) * 2
    stride = kh if stride is None else _pair(stride)
    padding = _pair(padding)
    B, Cc, H, W = x.shape
    Ho, Wo = (H - kh + 2 * padding) // stride + 1, (W - kw + 2 * padding) // stride + 1
    if out is None:
        out = torch.empty((B, Cc, Ho, Wo), device=x.device, dtype=torch.float32)
    with _on_device(x.device):
        code = lib.tdc_pool2d_f32(_dev_f32(x, "x"), _dev_f32(out, "out"), B, Cc, H, W, kh, kw, padding, stride, mode, _stream())
    if code != _lib.OK:
        raise TdcError(code, "tdc_pool2d_f32: window %dx%d stride %d padding %d on %dx%d" % (kh, kw, stride, padding, H, W))
    bound = getattr(x, "_tdc_absmax", None)
    if bound is not None:      # no pooling mode raises the largest magnitude: the input's bound holds for the output
        out._tdc_absmax = bound
    return out


def _image_view(t, name):
    """(pointer, image stride) of a [B][C][H][W] fp32 CUDA tensor whose images are dense [C][H][W] blocks that may be
    spaced apart — a channel slice `buf[:, :C]` of a larger NCHW buffer."""
    B, Cc, H, W = t.shape
    if t.dtype != torch.float32 or not t.is_cuda:
        raise TdcError(_lib.ERR_UNSUPPORTED, "%s must be a float32 CUDA tensor" % name)
    sb, sc, sh, sw = t.stride()
    if (sc, sh, sw) != (H * W, W, 1) or (B > 1 and sb < Cc * H * W):
        raise TdcError(_lib.ERR_UNSUPPORTED, "%s: images must be dense [C][H][W] blocks (strides %s)" % (name, t.stride()))
    return t.data_ptr(), (sb if B > 1 else Cc * H * W)


def affine_relu(x, scale=None, shift=None, relu=True, out=None):
    """y = relu?(x*scale[c] + shift[c]) per channel — inference BatchNorm + ReLU ahead of a conv (norm1 / norm2 of a
    dense layer, inference/densenet_inet_tt.py:36-60; BatchNorm::forward + Activation::forward of the end-to-end
    skeleton).  `x` and `out` may be channel slices of larger NCHW buffers; with no scale, shift or ReLU this is the
    copy that appends new features to a dense block's feature buffer."""
    B, Cc, H, W = x.shape
    if out is None:
        out = torch.empty((B, Cc, H, W), device=x.device, dtype=torch.float32)
    elif tuple(out.shape) != (B, Cc, H, W):
        raise TdcError(_lib.ERR_SHAPE, "out has shape %s, expected %s" % (tuple(out.shape), (B, Cc, H, W)))
    xp, xs = _image_view(x, "x")
    yp, ys = _image_view(out, "out")
    with _on_device(x.device):
        code = lib.tdc_affine_relu_f32(xp, yp, _dev_f32(scale, "scale") if scale is not None else None,
                                       _dev_f32(shift, "shift") if shift is not None else None, B, Cc, H * W, xs, ys,
                                       1 if relu else 0, _stream())
    if code != _lib.OK:
        raise TdcError(code, "tdc_affine_relu_f32")
    return out


def conv2d_epi(x, w, scale=None, bias=None, residual=None, relu=False, stride=1, padding=0, w_layout=W_KCRS,
               tile=None, out=None):
    """y = relu?(conv(x, w) * scale[k] + bias[k] + residual): a conv with a folded inference-mode
    BatchNorm, the residual add and the ReLU of the reference's blocks
    (inference/resnet_inet_tt.py:102-117) in one launch."""
    stride, padding = _pair(stride), _pair(padding)
    B, Cc, H, W = x.shape
    if w_layout == W_KCRS:
        K, Cw, R, S = w.shape
    else:
        Cw, R, S, K = w.shape
    if Cw != Cc:
        raise TdcError(_lib.ERR_SHAPE, "x has %d channels, w expects %d" % (Cc, Cw))
    Ho, Wo = out_hw(H, W, R, S, padding, stride)
    if out is None:
        out = torch.empty((B, K, Ho, Wo), device=x.device, dtype=torch.float32)
    if residual is not None and tuple(residual.shape) != tuple(out.shape):
        raise TdcError(_lib.ERR_SHAPE, "residual %s does not match the output %s" % (tuple(residual.shape), tuple(out.shape)))
    e = _epilogue(scale, bias, residual, relu)
    with _on_device(x.device):
        check(lib.tdc_conv2d_epi_f32(_dev_f32(x, "x"), _dev_f32(w, "w"), _dev_f32(out, "out"), B, Cc, H, W, K, R, S,
                                     padding, stride, w_layout, C.byref(e), C.byref(tile) if tile is not None else None,
                                     _stream()))
    return out


def tk_block_epi(x, first, core, last, scale=None, bias=None, residual=None, relu=False, stride=1, padding=0,
                 core_layout=W_KCRS, workspace=None, out=None, core_tile=None):
    """tk_block with the full epilogue on its last 1x1 step."""
    stride, padding = _pair(stride), _pair(padding)
    B, Cc, H, W = x.shape
    R1, K = first.shape[0], last.shape[0]
    if core_layout == W_KCRS:
        R2, R1c, R, S = core.shape
    else:
        R1c, R, S, R2 = core.shape
    if first.shape[1] != Cc or R1c != R1 or last.shape[1] != R2:
        raise TdcError(_lib.ERR_SHAPE, "Tucker factors do not chain: first %s core %s last %s" %
                       (tuple(first.shape), tuple(core.shape), tuple(last.shape)))
    Ho, Wo = out_hw(H, W, R, S, padding, stride)
    need = tk_block_workspace_bytes(B, Cc, H, W, R1, R2, K, R, S, padding, stride)
    if workspace is None:
        workspace = torch.empty(need, device=x.device, dtype=torch.uint8)
    if out is None:
        out = torch.empty((B, K, Ho, Wo), device=x.device, dtype=torch.float32)
    if residual is not None and tuple(residual.shape) != tuple(out.shape):
        raise TdcError(_lib.ERR_SHAPE, "residual %s does not match the output %s" % (tuple(residual.shape), tuple(out.shape)))
    e = _epilogue(scale, bias, residual, relu)
    with _on_device(x.device):
        check(lib.tdc_tk_block_epi_f32(_dev_f32(x, "x"), _dev_f32(first, "first"), _dev_f32(core, "core"),
                                       _dev_f32(last, "last"), _dev_f32(out, "out"), B, Cc, H, W, R1, R2, K, R, S,
                                       padding, stride, core_layout, C.byref(e),
                                       C.byref(core_tile) if core_tile is not None else None, workspace.data_ptr(),
                                       workspace.numel() * workspace.element_size(), _stream()))
    return out


def select_tile(B, Cc, H, W, K, R=3, S=3, pad=1, stride=1, dev=None):
    """Analytical tile choice (tdc_select_tile). `dev=None` queries the current GPU; pass
    `_lib.B200` to model a B200 without one."""
    t = Tile()
    check(lib.tdc_select_tile(B, Cc, H, W, K, R, S, pad, stride, C.byref(dev) if dev is not None else None,
                              C.byref(t)))
    return t


def tile_cost(shape, tile, dev=None):
    """(cycles, [filter volume, input volume, output volume, flops*waves]) of a complete tile."""
    cost = C.c_double()
    vols = (C.c_double * 4)()
    check(lib.tdc_tile_cost(*shape, C.byref(tile), C.byref(dev) if dev is not None else None, C.byref(cost), vols))
    return cost.value, list(vols)


def tile_info(shape, tile):
    """Completes `tile` in place and returns the launch facts (needs a GPU)."""
    info = LaunchInfo()
    check(lib.tdc_tile_info(*shape, C.byref(tile), C.byref(info)))
    return info


def query_device(device=-1):
    d = DevInfo()
    check(lib.tdc_query_device(device, C.byref(d)))
    return d
