"""ctypes front-end of the CPU oracle (``oracle/_build/libtenmo_ref.so``).

TEST INFRASTRUCTURE ONLY.  The oracle restates tenmo's CPU path (see ``tenmo_ref.h``) and is what the
CUDA library is checked against.  Only tests, the smoke check and the benchmark's CPU-baseline leg
import this module; the ``tenmo_b200`` package never does.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "_build", "libtenmo_ref.so")


class Opts(C.Structure):
    _fields_ = [("simd_width", C.c_int32), ("contract_scalar", C.c_int32), ("threads", C.c_int32)]


class Mat(C.Structure):
    _fields_ = [
        ("ptr", C.c_void_p),
        ("offset", C.c_int64),
        ("row_stride", C.c_int64),
        ("col_stride", C.c_int64),
        ("batch_rank", C.c_int32),
        ("batch_shape", C.c_int64 * 6),
        ("batch_stride", C.c_int64 * 6),
    ]


def build(force: bool = False) -> str:
    """Compile the oracle with its Makefile if the shared object is missing or stale."""
    src = [os.path.join(_HERE, f) for f in ("tenmo_ref.cpp", "tenmo_ref.h", "Makefile")]
    stale = force or not os.path.exists(_LIB_PATH) or any(
        os.path.getmtime(s) > os.path.getmtime(_LIB_PATH) for s in src
    )
    if stale:
        subprocess.run(["make", "-C", _HERE], check=True, capture_output=True)
    return _LIB_PATH


_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        L = C.CDLL(_LIB_PATH)
        P, I64, F = C.c_void_p, C.c_int64, C.c_float
        L.tenmo_ref_matmul_2d.argtypes = [C.POINTER(Mat), C.POINTER(Mat), P, I64, I64, I64, C.POINTER(Opts)]
        L.tenmo_ref_matmul_2d.restype = None
        L.tenmo_ref_matmul_nd.argtypes = L.tenmo_ref_matmul_2d.argtypes
        L.tenmo_ref_matmul_nd.restype = I64
        L.tenmo_ref_matmul_naive.argtypes = [C.POINTER(Mat), C.POINTER(Mat), P, I64, I64, I64]
        L.tenmo_ref_matmul_naive.restype = None
        L.tenmo_ref_add_bias.argtypes = [P, P, P, I64, I64]
        L.tenmo_ref_add_inplace.argtypes = [P, P, I64]
        L.tenmo_ref_relu_fwd.argtypes = [P, P, P, I64]
        L.tenmo_ref_relu_bwd.argtypes = [P, P, P, I64]
        L.tenmo_ref_sigmoid_fwd.argtypes = [P, P, I64]
        L.tenmo_ref_sigmoid_bwd.argtypes = [P, P, P, I64]
        L.tenmo_ref_colsum.argtypes = [P, P, I64, I64]
        L.tenmo_ref_ce_fwd.argtypes = [P, I64, I64, P, I64, I64, I64, F, C.c_int, P, P]
        L.tenmo_ref_ce_fwd.restype = I64
        L.tenmo_ref_ce_bwd.argtypes = [P, P, I64, I64, I64, F, C.c_int, P, I64, P]
        L.tenmo_ref_sgd_step.argtypes = [P, P, P, I64, F, F, F]
        L.tenmo_ref_accuracy.argtypes = [P, I64, I64, P, I64, I64]
        L.tenmo_ref_accuracy.restype = I64
        PP = C.POINTER(C.c_void_p)
        L.tenmo_ref_mlp_step.argtypes = [C.c_int, P, PP, PP, PP, PP, PP, PP, P, P, I64, F, F, F, F, C.c_int, P,
                                         C.POINTER(Opts)]
        L.tenmo_ref_mlp_step.restype = F
        L.tenmo_ref_softmax_fwd.argtypes = [P, P, I64, I64, C.c_int]
        L.tenmo_ref_softmax_bwd.argtypes = [P, P, P, I64, I64, C.c_int]
        L.tenmo_ref_mv.argtypes = [P, I64, I64, P, I64, P, I64, I64, C.c_int]
        L.tenmo_ref_vm.argtypes = [P, I64, P, I64, I64, P, I64, I64, C.c_int]
        _lib = L
    return _lib


def _ptr(a: np.ndarray) -> int:
    return a.ctypes.data


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


class View:
    """An NDBuffer-like strided view: a flat fp32 base array + shape, element strides, element offset."""

    def __init__(self, base: np.ndarray, shape, strides=None, offset: int = 0):
        self.base = _f32(base).reshape(-1)
        self.shape = tuple(int(s) for s in shape)
        if strides is None:
            strides, acc = [], 1
            for s in reversed(self.shape):
                strides.append(acc)
                acc *= s
            strides = tuple(reversed(strides))
        self.strides = tuple(int(s) for s in strides)
        self.offset = int(offset)

    @staticmethod
    def of(a) -> "View":
        a = _f32(a)
        return View(a.reshape(-1), a.shape)

    def t(self) -> "View":
        """transpose(-1,-2) as a stride view (what matmul.mojo:37,47 does)."""
        sh, st = list(self.shape), list(self.strides)
        sh[-1], sh[-2] = sh[-2], sh[-1]
        st[-1], st[-2] = st[-2], st[-1]
        return View(self.base, sh, st, self.offset)

    def numpy(self) -> np.ndarray:
        it = np.lib.stride_tricks.as_strided(
            self.base[self.offset:], shape=self.shape, strides=tuple(4 * s for s in self.strides), writeable=False
        )
        return np.array(it)

    def mat(self) -> Mat:
        m = Mat()
        m.ptr = _ptr(self.base)
        m.offset = self.offset
        m.row_stride, m.col_stride = self.strides[-2], self.strides[-1]
        br = len(self.shape) - 2
        m.batch_rank = br
        for d in range(br):
            m.batch_shape[d] = self.shape[d]
            m.batch_stride[d] = self.strides[d]
        return m


def make_opts(simd_width=8, contract_scalar=1, threads=1) -> Opts:
    return Opts(simd_width, contract_scalar, threads)


def matmul(A, B, simd_width=8, contract_scalar=1, threads=1) -> np.ndarray:
    """Tensor.matmul for rank >= 2 operands: 2D goes to MmCpu2d, everything else to MmCpuNd."""
    A = A if isinstance(A, View) else View.of(A)
    B = B if isinstance(B, View) else View.of(B)
    m, n = A.shape[-2:]
    n2, p = B.shape[-2:]
    if n != n2:
        raise ValueError(f"inner dims must match, got {n} and {n2}")
    o = make_opts(simd_width, contract_scalar, threads)
    ma, mb = A.mat(), B.mat()
    if len(A.shape) == 2 and len(B.shape) == 2:
        out = np.empty((m, p), np.float32)
        lib().tenmo_ref_matmul_2d(C.byref(ma), C.byref(mb), _ptr(out), m, n, p, C.byref(o))
        return out
    bshape = np.broadcast_shapes(A.shape[:-2], B.shape[:-2])
    out = np.empty(tuple(bshape) + (m, p), np.float32)
    r = lib().tenmo_ref_matmul_nd(C.byref(ma), C.byref(mb), _ptr(out), m, n, p, C.byref(o))
    if r < 0:
        raise ValueError("batch shapes not broadcastable")
    return out


def matmul_naive(A, B) -> np.ndarray:
    A = A if isinstance(A, View) else View.of(A)
    B = B if isinstance(B, View) else View.of(B)
    m, n = A.shape
    _, p = B.shape
    out = np.empty((m, p), np.float32)
    ma, mb = A.mat(), B.mat()
    lib().tenmo_ref_matmul_naive(C.byref(ma), C.byref(mb), _ptr(out), m, n, p)
    return out


def add_bias(a, b) -> np.ndarray:
    a, b = _f32(a), _f32(b)
    out = np.empty_like(a)
    lib().tenmo_ref_add_bias(_ptr(a), _ptr(b), _ptr(out), a.shape[0], a.shape[1])
    return out


def relu_fwd(x):
    x = _f32(x)
    out, mask = np.empty_like(x), np.empty_like(x)
    lib().tenmo_ref_relu_fwd(_ptr(x), _ptr(out), _ptr(mask), x.size)
    return out, mask


def relu_bwd(g, mask) -> np.ndarray:
    g, mask = _f32(g), _f32(mask)
    dx = np.empty_like(g)
    lib().tenmo_ref_relu_bwd(_ptr(g), _ptr(mask), _ptr(dx), g.size)
    return dx


def sigmoid_fwd(x) -> np.ndarray:
    x = _f32(x)
    y = np.empty_like(x)
    lib().tenmo_ref_sigmoid_fwd(_ptr(x), _ptr(y), x.size)
    return y


def sigmoid_bwd(g, y) -> np.ndarray:
    g, y = _f32(g), _f32(y)
    dx = np.empty_like(g)
    lib().tenmo_ref_sigmoid_bwd(_ptr(g), _ptr(y), _ptr(dx), g.size)
    return dx


def _conv_sig():
    L = lib()
    if not hasattr(L, "_conv_bound"):
        P, I64, I = C.c_void_p, C.c_int64, C.c_int
        L.tenmo_ref_conv2d_fwd.argtypes = [P, P, P, P, I64, I64, I64, I64, I64, I, I, I, I, I]
        L.tenmo_ref_conv2d_fwd.restype = None
        L.tenmo_ref_conv2d_bwd.argtypes = [P, P, P, P, P, P, I64, I64, I64, I64, I64, I, I, I, I]
        L.tenmo_ref_conv2d_bwd.restype = None
        L.tenmo_ref_maxpool2d_fwd.argtypes = [P, P, P, I64, I64, I64, I, I, I]
        L.tenmo_ref_maxpool2d_fwd.restype = None
        L.tenmo_ref_maxpool2d_bwd.argtypes = [P, P, P, I64, I64, I64, I64, I64]
        L.tenmo_ref_maxpool2d_bwd.restype = None
        L._conv_bound = True
    return L


def pad_nchw(x, pad: int) -> np.ndarray:
    """Constant zero padding of the two spatial dims, what the reference's Conv2D applies before the fused
    convolution (pad.mojo)."""
    x = _f32(x)
    return np.ascontiguousarray(np.pad(x, ((0, 0), (0, 0), (pad, pad), (pad, pad)))) if pad else x


def conv2d_fwd(x, kernel, bias, stride=1, dilation=1, pad=0, contract=1) -> np.ndarray:
    xp, kernel = pad_nchw(x, pad), _f32(kernel)
    N, Cin, Hp, Wp = xp.shape
    Cout, _, KH, KW = kernel.shape
    Ho = (Hp - ((KH - 1) * dilation + 1)) // stride + 1
    Wo = (Wp - ((KW - 1) * dilation + 1)) // stride + 1
    out = np.empty((N, Cout, Ho, Wo), np.float32)
    b = _f32(bias) if bias is not None else None
    _conv_sig().tenmo_ref_conv2d_fwd(_ptr(xp), _ptr(kernel), _ptr(b) if b is not None else None, _ptr(out), N, Cin, Hp, Wp,
                                     Cout, KH, KW, stride, dilation, contract)
    return out


def conv2d_bwd(grad, x, kernel, stride=1, dilation=1, pad=0):
    """Returns (dx, d_kernel, d_bias); dx is cropped back to the unpadded image (the Pad op's backward)."""
    xp, kernel, grad = pad_nchw(x, pad), _f32(kernel), _f32(grad)
    N, Cin, Hp, Wp = xp.shape
    Cout, _, KH, KW = kernel.shape
    dxp, dk, db = np.empty_like(xp), np.empty_like(kernel), np.empty(Cout, np.float32)
    _conv_sig().tenmo_ref_conv2d_bwd(_ptr(grad), _ptr(xp), _ptr(kernel), _ptr(dxp), _ptr(dk), _ptr(db), N, Cin, Hp, Wp, Cout,
                                     KH, KW, stride, dilation)
    dx = dxp[:, :, pad:Hp - pad, pad:Wp - pad] if pad else dxp
    return np.ascontiguousarray(dx), dk, db


def maxpool2d_fwd(x, k=2, stride=2, pad=0):
    x = _f32(x)
    N, Cn, H, W = x.shape
    Ho, Wo = (H + 2 * pad - k) // stride + 1, (W + 2 * pad - k) // stride + 1
    out, arg = np.empty((N, Cn, Ho, Wo), np.float32), np.empty((N, Cn, Ho, Wo), np.int64)
    _conv_sig().tenmo_ref_maxpool2d_fwd(_ptr(x), _ptr(out), _ptr(arg), N * Cn, H, W, k, stride, pad)
    return out, arg


def maxpool2d_bwd(g, argmax, in_shape) -> np.ndarray:
    g, argmax = _f32(g), np.ascontiguousarray(argmax, dtype=np.int64)
    N, Cn, H, W = in_shape
    dx = np.empty(in_shape, np.float32)
    _conv_sig().tenmo_ref_maxpool2d_bwd(_ptr(g), _ptr(argmax), _ptr(dx), N * Cn, H, W, g.shape[2], g.shape[3])
    return dx


def softmax_fwd(x, simd_width: int = 8) -> np.ndarray:
    """SoftmaxNdBuffer.softmax over the last axis (softmax.mojo:30-48) through the C restatement: row max, exp,
    the chunked Buffer.sum (buffers.mojo:1304-1333) and a division, all in fp32."""
    x = _f32(x)
    flat = x.reshape(-1, x.shape[-1])
    y = np.empty_like(flat)
    lib().tenmo_ref_softmax_fwd(_ptr(flat), _ptr(y), flat.shape[0], flat.shape[1], simd_width)
    return y.reshape(x.shape)


def softmax_bwd(g, y, simd_width: int = 8) -> np.ndarray:
    """SoftmaxBackwardDelegate (softmax.mojo:206-213): y * (g - sum(g * y))."""
    g, y = _f32(g), _f32(y)
    gf, yf = g.reshape(-1, g.shape[-1]), y.reshape(-1, y.shape[-1])
    dx = np.empty_like(gf)
    lib().tenmo_ref_softmax_bwd(_ptr(gf), _ptr(yf), _ptr(dx), gf.shape[0], gf.shape[1], simd_width)
    return dx.reshape(g.shape)


def mv(M, v, contract_scalar: int = 1) -> np.ndarray:
    """M[..., m, k] @ v[k] (matrixvector.mojo:205-285), a 1-D vector shared by every batch of M."""
    M, v = _f32(M), _f32(v)
    flat = M.reshape(-1, M.shape[-2], M.shape[-1])
    out = np.empty(flat.shape[:2], np.float32)
    m, k = flat.shape[1:]
    for b in range(flat.shape[0]):
        lib().tenmo_ref_mv(_ptr(flat[b]), k, 1, _ptr(v), 1, _ptr(out[b]), m, k, contract_scalar)
    return out.reshape(M.shape[:-1])


def vm(v, M, contract_scalar: int = 1) -> np.ndarray:
    """v[k] @ M[k, n] (vectormatrix.mojo:210-340)."""
    M, v = _f32(M), _f32(v)
    k, n = M.shape
    out = np.empty(n, np.float32)
    lib().tenmo_ref_vm(_ptr(v), 1, _ptr(M), n, 1, _ptr(out), k, n, contract_scalar)
    return out


def colsum(x) -> np.ndarray:
    x = _f32(x)
    out = np.empty(x.shape[1], np.float32)
    lib().tenmo_ref_colsum(_ptr(x), _ptr(out), x.shape[0], x.shape[1])
    return out


_RED = {"mean": 0, "sum": 1, "none": 2}


def ce_fwd(logits, labels, reduction="mean", ignore_index=-100, label_smoothing=0.0):
    """Returns (loss, softmax, valid_count)."""
    logits = _f32(logits)
    labels = np.ascontiguousarray(labels, dtype=np.int64)
    M, Cc = logits.shape
    sm = np.empty_like(logits)
    red = _RED[reduction]
    loss = np.zeros(M if red == 2 else 1, np.float32)
    valid = lib().tenmo_ref_ce_fwd(_ptr(logits), Cc, 1, _ptr(labels), M, Cc, ignore_index, label_smoothing, red,
                                   _ptr(sm), _ptr(loss))
    return (loss if red == 2 else loss[0]), sm, int(valid)


def ce_bwd(softmax, labels, valid_count, reduction="mean", ignore_index=-100, label_smoothing=0.0, upstream=None):
    softmax = _f32(softmax)
    labels = np.ascontiguousarray(labels, dtype=np.int64)
    M, Cc = softmax.shape
    red = _RED[reduction]
    if upstream is None:
        upstream = np.ones(M if red == 2 else 1, np.float32)
    upstream = _f32(upstream).reshape(-1)
    out = np.empty_like(softmax)
    lib().tenmo_ref_ce_bwd(_ptr(softmax), _ptr(labels), M, Cc, ignore_index, label_smoothing, red, _ptr(upstream),
                           valid_count, _ptr(out))
    return out


def sgd_step(p, g, v, lr, momentum=0.0, weight_decay=0.0):
    """In place on p and v (both contiguous fp32 arrays)."""
    assert p.dtype == np.float32 and v.dtype == np.float32 and p.flags.c_contiguous and v.flags.c_contiguous
    g = _f32(g)
    lib().tenmo_ref_sgd_step(_ptr(p), _ptr(g), _ptr(v), p.size, lr, momentum, weight_decay)


def accuracy(logits, labels) -> int:
    logits = _f32(logits)
    labels = np.ascontiguousarray(labels, dtype=np.int64)
    M, Cc = logits.shape
    return int(lib().tenmo_ref_accuracy(_ptr(logits), Cc, 1, _ptr(labels), M, Cc))


class MLP:
    """Parameters + SGD state of a Linear/ReLU stack, stepped through the oracle."""

    def __init__(self, weights, biases):
        self.W = [_f32(w).copy() for w in weights]
        self.b = [_f32(x).copy() for x in biases]
        self.vW = [np.zeros_like(w) for w in self.W]
        self.vb = [np.zeros_like(x) for x in self.b]
        self.dW = [np.zeros_like(w) for w in self.W]
        self.db = [np.zeros_like(x) for x in self.b]
        self.dims = np.array([self.W[0].shape[0]] + [w.shape[1] for w in self.W], np.int64)

    def _pp(self, arrs):
        arr = (C.c_void_p * len(arrs))(*[_ptr(a) for a in arrs])
        return C.cast(arr, C.POINTER(C.c_void_p)), arr

    def step(self, X, labels, lr=0.01, momentum=0.9, weight_decay=0.0, grad_scale=1.0, update=True, threads=1,
             contract_scalar=1):
        """One forward/backward(/SGD) step; returns (mean loss, logits)."""
        X = _f32(X)
        labels = np.ascontiguousarray(labels, dtype=np.int64)
        batch = X.shape[0]
        logits = np.empty((batch, int(self.dims[-1])), np.float32)
        o = make_opts(8, contract_scalar, threads)
        keep = []
        ptrs = []
        for group in (self.W, self.b, self.vW, self.vb, self.dW, self.db):
            pp, arr = self._pp(group)
            keep.append(arr)
            ptrs.append(pp)
        loss = lib().tenmo_ref_mlp_step(len(self.W), _ptr(self.dims), *ptrs, _ptr(X), _ptr(labels), batch, lr,
                                        momentum, weight_decay, grad_scale, 1 if update else 0, _ptr(logits),
                                        C.byref(o))
        return float(loss), logits
