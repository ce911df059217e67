"""CPU oracle for the Tucker core convolution — TEST INFRASTRUCTURE ONLY.

Only tests, the smoke check and the benchmark's CPU-baseline leg may import this module;
the product (ppopp23-tdc_b200/) never does.

Two restatements of the reference's algorithm live here:

* `conv2d_*` / `tk_block` / `ref_tiled`: numpy front ends of conv_oracle.c (plain C; built
  by `make -C oracle`).  They restate the definition of the convolution the reference calls
  at inference/TKConv.py:90-95 and the block/thread walk of its CUDA kernel
  (A100-evaluation/TDC-LAYERS-ORACLE/template_benchmark_cudnn.template:365-402).
* `TKConv2dCRef`: the reference module's forward written out with the same torch calls in
  the same order (inference/TKConv.py:85-106).  On a machine without the reference tree
  this is what "the reference's CPU PyTorch path" means: its arithmetic lives in
  torch.nn.functional.conv2d, a third-party dependency of the reference (README.md:16,
  "torch >= 1.4"; 2.11.0 here), not in the reference's own files.

Pinning: conv_oracle.c and TKConv2dCRef are checked against outputs of the reference's own
TKConv2dC (imported unmodified from the reference tree, with stub modules for the absent
tensorly) that are committed as tests/golden/*.npz together with the script that made them,
and against the reference drivers' own exactness property (integer inputs, all-ones
weights).  The reference ships no golden tensors of its own for this path.
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = os.path.join(_HERE, "liboracle.so")
W_KCRS, W_CRSK = 0, 1


def build(force=False):
    src = os.path.join(_HERE, "conv_oracle.c")
    if force or not os.path.exists(_LIB) or os.path.getmtime(_LIB) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "-B" if force else "-s", "liboracle.so"], check=True,
                       capture_output=True)
    return _LIB


_lib = None


def lib():
    global _lib
    if _lib is None:
        build()
        _lib = C.CDLL(_LIB)
        _lib.tdc_oracle_conv2d_ref_tiled.restype = C.c_int
        _lib.tdc_oracle_threads.restype = C.c_int
    return _lib


def threads():
    return lib().tdc_oracle_threads()


def _f(a):
    a = np.ascontiguousarray(a, dtype=np.float32)
    return a, a.ctypes.data_as(C.c_void_p)


def _dims(x, w, w_layout):
    B, Cc, H, W = x.shape
    if w_layout == W_KCRS:
        K, Cw, R, S = w.shape
    else:
        Cw, R, S, K = w.shape
    assert Cw == Cc, (x.shape, w.shape)
    return B, Cc, H, W, K, R, S


def out_hw(H, W, R, S, pad, stride):
    return (H + 2 * pad - R) // stride + 1, (W + 2 * pad - S) // stride + 1


def conv2d_f32(x, w, bias=None, pad=0, stride=1, w_layout=W_KCRS, use_fma=True, relu=False):
    x, xp = _f(x); w, wp = _f(w)
    B, Cc, H, W, K, R, S = _dims(x, w, w_layout)
    Ho, Wo = out_hw(H, W, R, S, pad, stride)
    y = np.empty((B, K, Ho, Wo), np.float32)
    bp = None
    if bias is not None:
        bias, bp = _f(bias)
    lib().tdc_oracle_conv2d_f32(xp, wp, bp, y.ctypes.data_as(C.c_void_p), B, Cc, H, W, K, R, S, pad, stride,
                                w_layout, int(use_fma), int(relu))
    return y


def conv2d_f32_sliced(x, w, tc, ks, bias=None, pad=0, stride=1, w_layout=W_KCRS, relu=False, kc=1):
    """Bit-exact twin of the device kernel for channel chunk `tc` split over `ks` slices of a CTA
    and `kc` CTAs of a cluster."""
    x, xp = _f(x); w, wp = _f(w)
    B, Cc, H, W, K, R, S = _dims(x, w, w_layout)
    Ho, Wo = out_hw(H, W, R, S, pad, stride)
    y = np.empty((B, K, Ho, Wo), np.float32)
    bp = None
    if bias is not None:
        bias, bp = _f(bias)
    lib().tdc_oracle_conv2d_f32_sliced(xp, wp, bp, y.ctypes.data_as(C.c_void_p), B, Cc, H, W, K, R, S, pad, stride,
                                       w_layout, tc, ks, kc, int(relu))
    return y


def conv2d_f64(x, w, bias=None, pad=0, stride=1, w_layout=W_KCRS, relu=False):
    """The arbiter: double accumulation, one rounding to fp32."""
    x, xp = _f(x); w, wp = _f(w)
    B, Cc, H, W, K, R, S = _dims(x, w, w_layout)
    Ho, Wo = out_hw(H, W, R, S, pad, stride)
    y = np.empty((B, K, Ho, Wo), np.float32)
    bp = None
    if bias is not None:
        bias, bp = _f(bias)
    lib().tdc_oracle_conv2d_f64(xp, wp, bp, y.ctypes.data_as(C.c_void_p), B, Cc, H, W, K, R, S, pad, stride,
                                w_layout, int(relu))
    return y


def ref_tiled(inp, kernel_crsk, TH, TW, TC):
    """The reference CUDA kernel's walk (one image, 3x3, pad 1, stride 1) on the CPU.
    inp [C][H][W], kernel [C][3][3][N] -> [N][H][W]."""
    inp, ip = _f(inp); kernel_crsk, kp = _f(kernel_crsk)
    Cc, H, W = inp.shape
    N = kernel_crsk.shape[3]
    out = np.zeros((N, H, W), np.float32)
    rc = lib().tdc_oracle_conv2d_ref_tiled(ip, kp, out.ctypes.data_as(C.c_void_p), Cc, N, H, W, TH, TW, TC)
    if rc:
        raise ValueError("ref_tiled: C %% TC != 0 or out of memory (rc=%d)" % rc)
    return out


def tk_block(x, first, core, last, bias=None, pad=0, stride=1, core_layout=W_KCRS, f64=False):
    """TKConv2dC.forward (inference/TKConv.py:90-95) on the C oracle. Returns (y, z1, z2)."""
    x, xp = _f(x)
    first, fp_ = _f(np.asarray(first).reshape(first.shape[0], first.shape[1]))
    last, lp = _f(np.asarray(last).reshape(last.shape[0], last.shape[1]))
    core, cp = _f(core)
    B, Cc, H, W = x.shape
    R1, K = first.shape[0], last.shape[0]
    if core_layout == W_KCRS:
        R2, _, R, S = core.shape
    else:
        _, R, S, R2 = core.shape
    Ho, Wo = out_hw(H, W, R, S, pad, stride)
    z1 = np.empty((B, R1, H, W), np.float32)
    z2 = np.empty((B, R2, Ho, Wo), np.float32)
    y = np.empty((B, K, Ho, Wo), np.float32)
    bp = None
    if bias is not None:
        bias, bp = _f(bias)
    vp = lambda a: a.ctypes.data_as(C.c_void_p)
    lib().tdc_oracle_tk_block(xp, fp_, cp, lp, bp, vp(y), vp(z1), vp(z2), B, Cc, H, W, R1, R2, K, R, S, pad, stride,
                              core_layout, int(f64))
    return y, z1, z2


# ---- the reference module's forward, call for call (torch on CPU) -----------------------
def _torch():
    import torch
    import torch.nn.functional as F
    return torch, F


class TKConv2dCRef:
    """inference/TKConv.py:23-106 without the parts that need tensorly: holds the three
    kernels and the bias, and runs forward / forward_features exactly as the reference does
    (F.conv2d x3, :90-95 and :97-106).  Parameters are plain tensors the caller sets."""

    def __init__(self, first_kernel, core_kernel, last_kernel, bias=None, stride=1, padding=0, dilation=1):
        self.first_kernel, self.core_kernel, self.last_kernel, self.bias = first_kernel, core_kernel, last_kernel, bias
        self.stride, self.padding, self.dilation, self.groups = stride, padding, dilation, 1

    def forward(self, x):
        _, F = _torch()
        out = F.conv2d(x, self.first_kernel)
        out = F.conv2d(out, self.core_kernel, None, self.stride, self.padding, self.dilation, self.groups)
        out = F.conv2d(out, self.last_kernel, self.bias)
        return out

    def forward_features(self, x):
        _, F = _torch()
        features = []
        out = F.conv2d(x, self.first_kernel)
        features.append(out)
        out = F.conv2d(out, self.core_kernel, None, self.stride, self.padding, self.dilation, self.groups)
        features.append(out)
        out = F.conv2d(out, self.last_kernel, self.bias)
        features.append(out)
        return out, features

    def core(self, z1):
        """Only the hot step, inference/TKConv.py:92-93."""
        _, F = _torch()
        return F.conv2d(z1, self.core_kernel, None, self.stride, self.padding, self.dilation, self.groups)
