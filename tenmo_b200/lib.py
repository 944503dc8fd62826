"""ctypes binding of ``libtenmo_cuda.so`` -- the C ABI declared in ``include/tenmo_cuda.h``.

Plays the role ``BLASHandle`` plays in the reference (tenmo/blashandle.mojo:176-251): the shared
library is opened once, a failure to load is kept as an error string (``is_initialized()`` false)
and any call on an uninitialised handle raises.  There is no CPU fallback: without the CUDA
library nothing on this path runs.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("TENMO_CUDA_PATH", os.path.join(_HERE, "libtenmo_cuda.so"))

MAX_BATCH_RANK = 6
ALGO_AUTO, ALGO_SIMT_FP32, ALGO_TC_3XTF32 = -1, 0, 1
DP_P2P_HANDLE_BYTES = 128
ACT_NONE, ACT_RELU, ACT_SIGMOID = 0, 1, 2
REDUCTION = {"mean": 0, "sum": 1, "none": 2}  # shared/__init__.mojo:4-40
DP_ID_BYTES = 128

# every symbol include/tenmo_cuda.h declares
EXPORTS = [
    "tenmo_cuda_init", "tenmo_cuda_destroy", "tenmo_cuda_last_error", "tenmo_cuda_version", "tenmo_cuda_set_stream",
    "tenmo_cuda_synchronize", "tenmo_cuda_device_info", "tenmo_cuda_check_device_status", "tenmo_cuda_launch_count",
    "tenmo_cuda_profile_begin", "tenmo_cuda_profile_end", "tenmo_cuda_reserve_sms",
    "tenmo_gemm_f32", "tenmo_gemm_f32_ex", "tenmo_gemv_f32", "tenmo_vecmat_f32", "tenmo_split_lo_f32", "tenmo_gemm_last_algo", "tenmo_gemm_last_kernel", "tenmo_gemm_last_stream_k", "tenmo_gemm_last_pair", "tenmo_cuda_wait_probe", "tenmo_add_bias_f32", "tenmo_add_inplace_f32", "tenmo_fill_f32",
    "tenmo_relu_fwd_f32", "tenmo_relu_bwd_f32", "tenmo_sigmoid_fwd_f32", "tenmo_sigmoid_bwd_f32", "tenmo_colsum_f32",
    "tenmo_conv_out_size", "tenmo_conv2d_fwd_f32", "tenmo_conv2d_bwd_input_f32", "tenmo_conv2d_bwd_weight_f32", "tenmo_im2col_f32", "tenmo_col2im_f32", "tenmo_channel_sum_f32", "tenmo_maxpool2d_fwd_f32",
    "tenmo_maxpool2d_bwd_f32",
    "tenmo_colsum_f32_static", "tenmo_softmax_fwd_f32", "tenmo_softmax_bwd_f32", "tenmo_ce_fwd_f32", "tenmo_ce_bwd_f32", "tenmo_ce_fwd_bwd_f32", "tenmo_sgd_step_f32", "tenmo_sgd_step_lo_f32", "tenmo_accuracy_f32", "tenmo_dp_get_unique_id",
    "tenmo_dp_init", "tenmo_dp_allreduce_sum_f32", "tenmo_dp_finalize",
    "tenmo_dp_p2p_alloc", "tenmo_dp_p2p_connect", "tenmo_dp_p2p_allreduce_sum_f32", "tenmo_dp_p2p_sgd_step_f32", "tenmo_dp_p2p_set_coresident", "tenmo_dp_p2p_close",
]


class TenmoError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"tenmo_cuda status {status}: {message}")
        self.status = status


class Mat(C.Structure):
    """``tenmo_mat``: a strided, possibly batched fp32 matrix view in device memory."""

    _fields_ = [
        ("ptr", C.c_void_p),
        ("offset", C.c_int64),
        ("row_stride", C.c_int64),
        ("col_stride", C.c_int64),
        ("batch_rank", C.c_int32),
        ("batch_shape", C.c_int64 * MAX_BATCH_RANK),
        ("batch_stride", C.c_int64 * MAX_BATCH_RANK),
    ]


class GemmOpts(C.Structure):
    """``tenmo_gemm_opts``."""

    _fields_ = [
        ("beta", C.c_float),
        ("bias", C.c_void_p),
        ("act", C.c_int),
        ("aux", C.c_void_p),
        ("colsum", C.c_void_p),
        ("a_lo", C.c_void_p),
        ("b_lo", C.c_void_p),
        ("c_lo", C.c_void_p),
        ("mul_mask", C.c_void_p),
        ("bias_m", C.c_void_p),
    ]


def make_mat(ptr: int, shape, strides, offset: int = 0) -> Mat:
    if len(shape) < 2 or len(shape) != len(strides):
        raise ValueError("make_mat needs rank >= 2 and one stride per dim")
    if len(shape) - 2 > MAX_BATCH_RANK:
        raise ValueError(f"at most {MAX_BATCH_RANK} batch dims")
    m = Mat()
    m.ptr = ptr
    m.offset = offset
    m.row_stride, m.col_stride = strides[-2], strides[-1]
    m.batch_rank = len(shape) - 2
    for d in range(m.batch_rank):
        m.batch_shape[d] = shape[d]
        m.batch_stride[d] = strides[d]
    return m


def _bind(lib):
    P, I, I64, F = C.c_void_p, C.c_int, C.c_int64, C.c_float
    sig = {
        "tenmo_cuda_init": (I, [I, C.POINTER(P)]),
        "tenmo_cuda_destroy": (None, [P]),
        "tenmo_cuda_last_error": (C.c_char_p, [P]),
        "tenmo_cuda_version": (C.c_char_p, []),
        "tenmo_cuda_set_stream": (I, [P, P]),
        "tenmo_cuda_synchronize": (I, [P]),
        "tenmo_cuda_device_info": (I, [P, C.POINTER(I), C.POINTER(I), C.POINTER(I), C.POINTER(I)]),
        "tenmo_cuda_check_device_status": (I, [P]),
        "tenmo_cuda_launch_count": (I64, [P, I]),
        "tenmo_cuda_reserve_sms": (I, [P, I]),
        "tenmo_cuda_profile_begin": (I, [P]),
        "tenmo_cuda_profile_end": (I, [P, C.POINTER(I64), C.POINTER(C.c_double)]),
        "tenmo_gemm_f32": (I, [P, I, I64, I64, I64, C.POINTER(Mat), C.POINTER(Mat), P, F, P, I, P, P]),
        "tenmo_gemm_f32_ex": (I, [P, I, I64, I64, I64, C.POINTER(Mat), C.POINTER(Mat), P, C.POINTER(GemmOpts)]),
        "tenmo_gemv_f32": (I, [P, I64, I64, C.POINTER(Mat), P, I64, P, F]),
        "tenmo_vecmat_f32": (I, [P, I64, I64, P, I64, C.POINTER(Mat), P, F]),
        "tenmo_split_lo_f32": (I, [P, C.POINTER(Mat), I64, I64, P, I64]),
        "tenmo_gemm_last_algo": (I, [P]),
        "tenmo_gemm_last_kernel": (C.c_char_p, [P]),
        "tenmo_gemm_last_stream_k": (I, [P]),
        "tenmo_gemm_last_pair": (I, [P]),
        "tenmo_cuda_wait_probe": (I, [P, C.c_int]),
        "tenmo_add_bias_f32": (I, [P, P, P, P, I64, I64]),
        "tenmo_add_inplace_f32": (I, [P, P, P, I64]),
        "tenmo_fill_f32": (I, [P, P, F, I64]),
        "tenmo_relu_fwd_f32": (I, [P, P, P, P, I64]),
        "tenmo_relu_bwd_f32": (I, [P, P, P, P, F, I64]),
        "tenmo_sigmoid_fwd_f32": (I, [P, P, P, I64]),
        "tenmo_sigmoid_bwd_f32": (I, [P, P, P, P, F, I64]),
        "tenmo_colsum_f32": (I, [P, P, I64, I64, I64, P, F]),
        "tenmo_colsum_f32_static": (I, [P, I64, I64, I64, P, F, P]),
        "tenmo_conv_out_size": (I, [I64, I, I, I, I, C.POINTER(I64)]),
        "tenmo_conv2d_fwd_f32": (I, [P, P, I64, I64, I64, I64, P, P, I64, I, I, I, I, I, I, P, P]),
        "tenmo_conv2d_bwd_input_f32": (I, [P, P, P, P, I64, I64, I64, I64, I64, I, I, I, I, I, P, F]),
        "tenmo_conv2d_bwd_weight_f32": (I, [P, P, P, P, I64, I64, I64, I64, I64, I, I, I, I, I, P, P, F]),
        "tenmo_im2col_f32": (I, [P, P, I64, I64, I64, I64, I, I, I, I, I, P]),
        "tenmo_col2im_f32": (I, [P, P, I64, I64, I64, I64, I, I, I, I, I, P, F]),
        "tenmo_channel_sum_f32": (I, [P, P, I64, I64, I64, P, F]),
        "tenmo_maxpool2d_fwd_f32": (I, [P, P, I64, I64, I64, I64, I, I, I, P, P]),
        "tenmo_maxpool2d_bwd_f32": (I, [P, P, P, I64, I64, I64, I64, I64, I64, P]),
        "tenmo_softmax_fwd_f32": (I, [P, P, I64, P, I64, I64]),
        "tenmo_softmax_bwd_f32": (I, [P, P, P, P, F, I64, I64]),
        "tenmo_ce_fwd_f32": (I, [P, P, I64, P, I, I64, I64, I64, F, I, P, P, P]),
        "tenmo_ce_bwd_f32": (I, [P, P, P, I, I64, I64, I64, F, I, P, P, P, F]),
        "tenmo_ce_fwd_bwd_f32": (I, [P, P, I64, P, I, I64, I64, I64, F, I, P, P, P, P, P]),
        "tenmo_sgd_step_f32": (I, [P, I, P, P, P, P, F, F, F, F]),
        "tenmo_sgd_step_lo_f32": (I, [P, I, P, P, P, P, P, P, F, F, F, F]),
        "tenmo_accuracy_f32": (I, [P, P, I64, P, I, I64, I64, P, P]),
        "tenmo_dp_get_unique_id": (I, [P, P, C.c_size_t]),
        "tenmo_dp_init": (I, [P, I, I, P, C.c_size_t]),
        "tenmo_dp_allreduce_sum_f32": (I, [P, P, I64]),
        "tenmo_dp_finalize": (I, [P]),
        "tenmo_dp_p2p_alloc": (I, [P, I64, C.POINTER(C.c_void_p), P, C.c_size_t]),
        "tenmo_dp_p2p_connect": (I, [P, I, I, P, C.c_size_t]),
        "tenmo_dp_p2p_allreduce_sum_f32": (I, [P, I64, I64]),
        "tenmo_dp_p2p_sgd_step_f32": (I, [P, I64, I64, I64, P, P, I64, F, F, F, F]),
        "tenmo_dp_p2p_set_coresident": (I, [P, I]),
        "tenmo_dp_p2p_close": (I, [P]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args


class TenmoCuda:
    """One context on one device.  ``TenmoCuda(device)`` never raises on load failure; check
    ``is_initialized()`` / ``get_error()`` like the reference's BLAS handle, or use ``require()``."""

    def __init__(self, device: int = 0, path: str | None = None):
        self._lib = None
        self._ctx = C.c_void_p()
        self._error = ""
        self.path = path or LIB_PATH
        try:
            self._lib = C.CDLL(self.path)
            _bind(self._lib)
        except (OSError, AttributeError) as e:
            self._lib = None
            self._error = f"Failed to load tenmo CUDA library {self.path}: {e}"
            return
        st = self._lib.tenmo_cuda_init(device, C.byref(self._ctx))
        if st != 0:
            self._error = self._lib.tenmo_cuda_last_error(None).decode()
            self._ctx = C.c_void_p()

    # -- handle state -------------------------------------------------------------------------------
    def is_initialized(self) -> bool:
        return self._lib is not None and bool(self._ctx)

    def get_error(self) -> str:
        return self._error

    def require(self) -> "TenmoCuda":
        if not self.is_initialized():
            raise TenmoError(-2, self._error or "tenmo CUDA library not initialised")
        return self

    def close(self):
        if self.is_initialized():
            self._lib.tenmo_cuda_destroy(self._ctx)
            self._ctx = C.c_void_p()

    def _ck(self, st: int):
        if st != 0:
            raise TenmoError(st, self._lib.tenmo_cuda_last_error(self._ctx).decode())

    def _call(self, name: str, *args):
        if not self.is_initialized():
            raise TenmoError(-2, self._error or "tenmo CUDA library not initialised")
        self._ck(getattr(self._lib, name)(self._ctx, *args))

    # -- context ------------------------------------------------------------------------------------
    def version(self) -> str:
        return self.require()._lib.tenmo_cuda_version().decode()

    def set_stream(self, cuda_stream: int | None):
        """``cuda_stream`` is a raw cudaStream_t (0 = CUDA's default stream); ``None`` = the context's own."""
        self._call("tenmo_cuda_set_stream", C.c_void_p(-1 if cuda_stream is None else cuda_stream))

    def synchronize(self):
        self._call("tenmo_cuda_synchronize")

    def device_info(self) -> dict:
        v = [C.c_int() for _ in range(4)]
        self._call("tenmo_cuda_device_info", *[C.byref(x) for x in v])
        return dict(sm_count=v[0].value, cc_major=v[1].value, cc_minor=v[2].value, sm_clock_khz=v[3].value)

    def check_device_status(self):
        self._call("tenmo_cuda_check_device_status")

    def launch_count(self, reset: bool = False) -> int:
        return int(self.require()._lib.tenmo_cuda_launch_count(self._ctx, 1 if reset else 0))

    def reserve_sms(self, n: int):
        """Leave ``n`` SMs out of the persistent GEMM grid (for a collective running on another stream)."""
        self._call("tenmo_cuda_reserve_sms", n)

    def profile_begin(self):
        self._call("tenmo_cuda_profile_begin")

    def profile_end(self):
        """Returns (launches, total_ms) of the GEMM main kernels since profile_begin."""
        n, ms = C.c_int64(0), C.c_double(0.0)
        self._call("tenmo_cuda_profile_end", C.byref(n), C.byref(ms))
        return int(n.value), float(ms.value)

    # -- ops (raw device pointers as ints) ------------------------------------------------------------
    def gemm(self, M, N, K, A: Mat, B: Mat, c_ptr, *, algo=ALGO_AUTO, beta=0.0, bias=0, act=ACT_NONE, aux=0, colsum=0):
        self._call("tenmo_gemm_f32", algo, M, N, K, C.byref(A), C.byref(B), c_ptr, beta, bias or None, act,
                   aux or None, colsum or None)

    def gemm_ex(self, M, N, K, A: Mat, B: Mat, c_ptr, *, algo=ALGO_AUTO, beta=0.0, bias=0, act=ACT_NONE, aux=0, colsum=0,
                a_lo=0, b_lo=0, c_lo=0, mul_mask=0, bias_m=0):
        """tenmo_gemm_f32_ex: the GEMM with precomputed / produced lo planes and a fused mask multiply."""
        o = GemmOpts(beta, bias or None, act, aux or None, colsum or None, a_lo or None, b_lo or None, c_lo or None,
                     mul_mask or None, bias_m or None)
        self._call("tenmo_gemm_f32_ex", algo, M, N, K, C.byref(A), C.byref(B), c_ptr, C.byref(o))

    def gemv(self, M, K, A: Mat, x, incx, y, beta=0.0):
        """y[i] = sum_k A[i,k] x[k]: the HBM-bound matrix @ vector kernel (one matrix per call)."""
        self._call("tenmo_gemv_f32", M, K, C.byref(A), x, incx, y, beta)

    def vecmat(self, K, N, x, incx, A: Mat, y, beta=0.0):
        """y[j] = sum_k x[k] A[k,j]: the HBM-bound vector @ matrix kernel (one matrix per call)."""
        self._call("tenmo_vecmat_f32", K, N, x, incx, C.byref(A), y, beta)

    def split_lo(self, X: Mat, rows, cols, lo_out, capacity):
        self._call("tenmo_split_lo_f32", C.byref(X), rows, cols, lo_out, capacity)

    def gemm_last_algo(self) -> int:
        return int(self.require()._lib.tenmo_gemm_last_algo(self._ctx))

    def wait_probe(self, limit_us: int):
        """A kernel whose bounded wait runs out after limit_us; check_device_status() then raises TenmoError."""
        self._call("tenmo_cuda_wait_probe", int(limit_us))

    def gemm_last_kernel(self) -> str:
        return self.require()._lib.tenmo_gemm_last_kernel(self._ctx).decode()

    def gemm_last_stream_k(self) -> int:
        """Pieces of the stream-K tail of the last tensor-core GEMM launch (0: every tile computed whole)."""
        return int(self.require()._lib.tenmo_gemm_last_stream_k(self._ctx))

    def gemm_last_pair(self) -> bool:
        """True when the last tensor-core GEMM ran as CTA pairs (tcgen05 cta_group::2)."""
        return bool(self.require()._lib.tenmo_gemm_last_pair(self._ctx))

    def add_bias(self, x, bias, out, M, N):
        self._call("tenmo_add_bias_f32", x, bias, out, M, N)

    def add_inplace(self, out, inp, n):
        self._call("tenmo_add_inplace_f32", out, inp, n)

    def fill(self, x, value, n):
        self._call("tenmo_fill_f32", x, value, n)

    def relu_fwd(self, x, out, mask, n):
        self._call("tenmo_relu_fwd_f32", x, out, mask or None, n)

    def relu_bwd(self, g, mask, dx, n, beta=0.0):
        self._call("tenmo_relu_bwd_f32", g, mask, dx, beta, n)

    def sigmoid_fwd(self, x, y, n):
        self._call("tenmo_sigmoid_fwd_f32", x, y, n)

    def sigmoid_bwd(self, g, y, dx, n, beta=0.0):
        self._call("tenmo_sigmoid_bwd_f32", g, y, dx, beta, n)

    def colsum(self, x, M, N, ldx, out, beta=0.0):
        self._call("tenmo_colsum_f32", x, M, N, ldx, out, beta)

    def colsum_static(self, x, M, N, ldx, out, beta=0.0, stream=0):
        """Column sum through the entry point that allocates nothing (fixed in-module scratch, N <= 16384).
        Needs no context: it runs on the current device and on ``stream`` (a raw cudaStream_t)."""
        if self._lib is None:
            raise TenmoError(-2, self._error or "tenmo CUDA library not loaded")
        st = self._lib.tenmo_colsum_f32_static(x, M, N, ldx, out, beta, C.c_void_p(stream))
        if st != 0:
            raise TenmoError(st, self._lib.tenmo_cuda_last_error(None).decode())

    def conv2d_fwd(self, x, N, Cn, H, W, weight, bias, Cout, KH, KW, stride, dilation, pad, act, out, mask=0):
        """Convolution forward as an implicit GEMM (bias-initialised accumulators, optional ReLU + mask)."""
        self._call("tenmo_conv2d_fwd_f32", x, N, Cn, H, W, weight, bias or None, Cout, KH, KW, stride, dilation, pad, act, out,
                   mask or None)

    def conv2d_bwd_input(self, g, g_mask, weight, N, Cn, H, W, Cout, KH, KW, stride, dilation, pad, dx, beta=0.0):
        self._call("tenmo_conv2d_bwd_input_f32", g, g_mask or None, weight, N, Cn, H, W, Cout, KH, KW, stride, dilation, pad, dx,
                   beta)

    def conv2d_bwd_weight(self, x, g, g_mask, N, Cn, H, W, Cout, KH, KW, stride, dilation, pad, dW, db, beta=0.0):
        self._call("tenmo_conv2d_bwd_weight_f32", x, g, g_mask or None, N, Cn, H, W, Cout, KH, KW, stride, dilation, pad, dW, db,
                   beta)

    def im2col(self, x, N, Cn, H, W, KH, KW, stride, dilation, pad, patches):
        self._call("tenmo_im2col_f32", x, N, Cn, H, W, KH, KW, stride, dilation, pad, patches)

    def col2im(self, dpatches, N, Cn, H, W, KH, KW, stride, dilation, pad, dx, beta=0.0):
        self._call("tenmo_col2im_f32", dpatches, N, Cn, H, W, KH, KW, stride, dilation, pad, dx, beta)

    def channel_sum(self, g, N, Cn, S, out, beta=0.0):
        self._call("tenmo_channel_sum_f32", g, N, Cn, S, out, beta)

    def maxpool2d_fwd(self, x, N, Cn, H, W, k, stride, pad, out, argmax):
        self._call("tenmo_maxpool2d_fwd_f32", x, N, Cn, H, W, k, stride, pad, out, argmax)

    def maxpool2d_bwd(self, g, argmax, N, Cn, H, W, Ho, Wo, dx):
        self._call("tenmo_maxpool2d_bwd_f32", g, argmax, N, Cn, H, W, Ho, Wo, dx)

    def softmax_fwd(self, x, ldx, y, M, Cn):
        self._call("tenmo_softmax_fwd_f32", x, ldx, y, M, Cn)

    def softmax_bwd(self, y, g, dx, M, Cn, beta=0.0):
        self._call("tenmo_softmax_bwd_f32", y, g, dx, beta, M, Cn)

    def ce_fwd(self, logits, ld, labels, label_is_i64, M, Cn, ignore_index, label_smoothing, reduction, softmax,
               loss, valid_count):
        self._call("tenmo_ce_fwd_f32", logits, ld, labels, 1 if label_is_i64 else 0, M, Cn, ignore_index,
                   label_smoothing, reduction, softmax or None, loss, valid_count)

    def ce_fwd_bwd(self, logits, ld, labels, label_is_i64, M, Cn, ignore_index, label_smoothing, reduction, softmax,
                   loss, valid_count, upstream, dlogits):
        """Loss and its gradient in one call (one launch for a small batch); same bits as ce_fwd then ce_bwd."""
        self._call("tenmo_ce_fwd_bwd_f32", logits, ld, labels, 1 if label_is_i64 else 0, M, Cn, ignore_index,
                   label_smoothing, reduction, softmax, loss, valid_count, upstream or None, dlogits)

    def ce_bwd(self, softmax, labels, label_is_i64, M, Cn, ignore_index, label_smoothing, reduction, upstream,
               valid_count, dlogits, beta=0.0):
        self._call("tenmo_ce_bwd_f32", softmax, labels, 1 if label_is_i64 else 0, M, Cn, ignore_index,
                   label_smoothing, reduction, upstream or None, valid_count or None, dlogits, beta)

    def sgd_step(self, p_ptrs, g_ptrs, v_ptrs, numels, lr, momentum=0.0, weight_decay=0.0, grad_scale=1.0, lo_ptrs=None,
                 lo_numels=None):
        """lo_ptrs / lo_numels: optional per-tensor lo planes of the updated parameters (tenmo_sgd_step_lo_f32)."""
        n = len(p_ptrs)
        arr = lambda xs: (C.c_void_p * n)(*xs)
        pa, ga = arr(p_ptrs), arr(g_ptrs)
        va = arr(v_ptrs) if v_ptrs is not None else None
        na = (C.c_int64 * n)(*numels)
        if lo_ptrs is None:
            self._call("tenmo_sgd_step_f32", n, pa, ga, va, na, lr, momentum, weight_decay, grad_scale)
        else:
            la, ln = arr([x or None for x in lo_ptrs]), (C.c_int64 * n)(*lo_numels)
            self._call("tenmo_sgd_step_lo_f32", n, pa, ga, va, na, la, ln, lr, momentum, weight_decay, grad_scale)

    def accuracy(self, logits, ld, labels, label_is_i64, M, Cn, correct_dev) -> int:
        host = C.c_int64(0)
        self._call("tenmo_accuracy_f32", logits, ld, labels, 1 if label_is_i64 else 0, M, Cn, correct_dev,
                   C.byref(host))
        return int(host.value)

    def accuracy_async(self, logits, ld, labels, label_is_i64, M, Cn, correct_dev):
        self._call("tenmo_accuracy_f32", logits, ld, labels, 1 if label_is_i64 else 0, M, Cn, correct_dev, None)

    # -- data parallel ---------------------------------------------------------------------------------
    def dp_get_unique_id(self) -> bytes:
        buf = C.create_string_buffer(DP_ID_BYTES)
        self._call("tenmo_dp_get_unique_id", buf, DP_ID_BYTES)
        return buf.raw

    def dp_init(self, rank: int, world: int, uid: bytes | None):
        buf = C.create_string_buffer(uid, DP_ID_BYTES) if uid else None
        self._call("tenmo_dp_init", rank, world, buf, DP_ID_BYTES if uid else 0)

    def dp_allreduce_sum(self, buf, count):
        self._call("tenmo_dp_allreduce_sum_f32", buf, count)

    def dp_finalize(self):
        self._call("tenmo_dp_finalize")

    # -- data parallel over peer memory (one kernel of this library instead of NCCL) --------------------
    def dp_p2p_alloc(self, count: int):
        """The gradient bucket (count floats, zeroed, owned by the library): (device pointer, IPC handle bytes)."""
        ptr = C.c_void_p()
        handles = C.create_string_buffer(DP_P2P_HANDLE_BYTES)
        self._call("tenmo_dp_p2p_alloc", count, C.byref(ptr), handles, DP_P2P_HANDLE_BYTES)
        return int(ptr.value), handles.raw

    def dp_p2p_connect(self, rank: int, world: int, all_handles: bytes):
        buf = C.create_string_buffer(all_handles, len(all_handles))
        self._call("tenmo_dp_p2p_connect", rank, world, buf, len(all_handles))

    def dp_p2p_allreduce_sum(self, offset: int, count: int):
        self._call("tenmo_dp_p2p_allreduce_sum_f32", offset, count)

    def dp_p2p_sgd_step(self, grad_offset: int, param_offset: int, count: int, v, p_lo, lo_count: int, lr, momentum=0.0,
                        weight_decay=0.0, grad_scale=1.0):
        """Exchange + SGD with the optimiser sharded over the ranks (gradients and parameters both live in the bucket)."""
        self._call("tenmo_dp_p2p_sgd_step_f32", grad_offset, param_offset, count, v or None, p_lo or None, lo_count, lr,
                   momentum, weight_decay, grad_scale)

    def dp_p2p_set_coresident(self, on: bool):
        """Small exchange CTAs that fit beside the persistent GEMM CTA (for an overlapped exchange) instead of large ones."""
        self._call("tenmo_dp_p2p_set_coresident", 1 if on else 0)

    def dp_p2p_close(self):
        self._call("tenmo_dp_p2p_close")
