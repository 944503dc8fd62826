"""Host-side mirror of tenmo's data model for the dense fp32 training path.

``NDBuffer`` = shape + element strides + element offset over a device allocation
(tenmo/ndbuffer.mojo:66-74); ``Tensor`` = NDBuffer + requires_grad + gradbox + ancestry
(tenmo/tensor.mojo); ``Tensor.backward`` = DFS topological order + fan-in counted ready queue
(tenmo/tensor.mojo:3154-3247) with the integer-tag dispatch of ``Backward.invoke``
(tenmo/backpropagation.mojo:278-519).  Every device operation goes through the C ABI of
libtenmo_cuda.so; torch only owns the device allocations.  Names, argument meaning and error
behaviour follow the reference so that the parity tests read like the reference's own tests.
"""
from __future__ import annotations

from collections import deque

import numpy as np
import torch

from . import lib as _lib
from .lib import TenmoCuda, make_mat

# op tags, values as in tenmo/backpropagation.mojo:30-96
BACKWARD_RELU = 2
BACKWARD_MATMUL_ND = 3
BACKWARD_MATMUL_2D = 4
BACKWARD_TRANSPOSE = 5
BACKWARD_SIGMOID = 7
BACKWARD_SOFTMAX = 8
BACKWARD_CE_CLASS_INDICES_INT32 = 9
BACKWARD_SUM = 16
BACKWARD_MATRIX_VECTOR_MUL = 20
BACKWARD_VECTOR_MATMUL = 21
BACKWARD_ADD_BROADCAST = 23
BACKWARD_DOT = 30
BACKWARD_CE_CLASS_INDICES_INT64 = 66

_handles: dict[int, TenmoCuda] = {}
_gemm_algo = _lib.ALGO_AUTO


def handle(device: int | None = None) -> TenmoCuda:
    """The process-wide context of a device, bound to torch's current stream.  Raises if the CUDA
    library or the GPU is missing -- there is no CPU path behind it."""
    dev = torch.cuda.current_device() if device is None else device
    h = _handles.get(dev)
    if h is None:
        h = TenmoCuda(dev).require()
        _handles[dev] = h
    h.set_stream(torch.cuda.current_stream(dev).cuda_stream)
    return h


def set_gemm_algo(name: str):
    """'auto' | 'simt' (strict fp32) | '3xtf32' (tcgen05): the run-time switch TENMO_CUDA_GEMM."""
    global _gemm_algo
    _gemm_algo = {"auto": _lib.ALGO_AUTO, "simt": _lib.ALGO_SIMT_FP32, "3xtf32": _lib.ALGO_TC_3XTF32}[name]


def panic(*parts):
    """tenmo/common_utils.mojo:97-106 aborts; here a host error that tests can catch."""
    raise RuntimeError(" ".join(str(p) for p in parts))


def _contig_strides(shape):
    st, acc = [], 1
    for s in reversed(shape):
        st.append(acc)
        acc *= s
    return tuple(reversed(st))


class NDBuffer:
    """A strided fp32 (or integer label) view of a flat device allocation."""

    def __init__(self, storage: torch.Tensor, shape, strides=None, offset: int = 0):
        self.storage = storage
        self.shape = tuple(int(s) for s in shape)
        self.strides = tuple(int(s) for s in (strides if strides is not None else _contig_strides(self.shape)))
        self.offset = int(offset)

    # -- construction ------------------------------------------------------------------------------
    @staticmethod
    def zeros(shape, dtype=torch.float32) -> "NDBuffer":
        n = int(np.prod(shape)) if len(shape) else 1
        return NDBuffer(torch.zeros(max(n, 1), dtype=dtype, device="cuda"), shape)

    @staticmethod
    def empty(shape) -> "NDBuffer":
        n = int(np.prod(shape)) if len(shape) else 1
        return NDBuffer(torch.empty(max(n, 1), dtype=torch.float32, device="cuda"), shape)

    @staticmethod
    def from_numpy(a, dtype=np.float32) -> "NDBuffer":
        a = np.ascontiguousarray(a, dtype=dtype)
        return NDBuffer(torch.from_numpy(a.reshape(-1).copy()).cuda(), a.shape)

    # -- queries -------------------------------------------------------------------------------------
    def numels(self) -> int:
        return int(np.prod(self.shape)) if self.shape else 1

    def rank(self) -> int:
        return len(self.shape)

    def is_contiguous(self) -> bool:
        # strides.mojo:239-264: C-order strides for every dim of size > 1
        expect = 1
        for s, st in zip(reversed(self.shape), reversed(self.strides)):
            if s > 1 and st != expect:
                return False
            expect *= s
        return True

    def data_ptr(self) -> int:
        return self.storage.data_ptr() + self.offset * self.storage.element_size()

    def mat(self):
        return make_mat(self.storage.data_ptr(), self.shape, self.strides, self.offset)

    def numpy(self) -> np.ndarray:
        flat = self.storage.detach().cpu().numpy()
        item = flat.dtype.itemsize
        view = np.lib.stride_tricks.as_strided(flat[self.offset:], shape=self.shape,
                                               strides=tuple(item * s for s in self.strides), writeable=False)
        return np.array(view)

    # -- views ---------------------------------------------------------------------------------------
    def transpose(self, axes=(-1, -2)) -> "NDBuffer":
        """Stride view, no copy (what matmul.mojo:37,47 passes to the backward GEMMs)."""
        a, b = (ax % len(self.shape) for ax in axes)
        sh, st = list(self.shape), list(self.strides)
        sh[a], sh[b] = sh[b], sh[a]
        st[a], st[b] = st[b], st[a]
        return NDBuffer(self.storage, sh, st, self.offset)

    def view(self, shape, strides, offset=0) -> "NDBuffer":
        return NDBuffer(self.storage, shape, strides, self.offset + offset)

    def unsqueeze(self, axis: int) -> "NDBuffer":
        """Insert a size-1 dim as a view (its stride is never used)."""
        sh, st = list(self.shape), list(self.strides)
        sh.insert(axis, 1)
        st.insert(axis, 1)
        return NDBuffer(self.storage, sh, st, self.offset)

    def reshape(self, shape) -> "NDBuffer":
        if not self.is_contiguous():
            return self.contiguous().reshape(shape)
        return NDBuffer(self.storage, shape, None, self.offset)

    def contiguous(self) -> "NDBuffer":
        if self.is_contiguous():
            return self
        t = torch.as_strided(self.storage, self.shape, self.strides, self.offset).contiguous()
        return NDBuffer(t.reshape(-1), self.shape)

    # -- the hot path ----------------------------------------------------------------------------------
    def matmul_2d(self, other: "NDBuffer") -> "NDBuffer":
        """NDBuffer.matmul_2d (ndbuffer.mojo:2404-2443)."""
        if self.rank() != 2 or other.rank() != 2:
            panic("NDBuffer -> matmul_2d: both operands must be rank 2, got", self.shape, "and", other.shape)
        return self.matmul_nd(other)

    def matmul_nd(self, other: "NDBuffer") -> "NDBuffer":
        """NDBuffer.matmul_nd (ndbuffer.mojo:2445-2501): batch dims broadcast NumPy-style."""
        if self.rank() < 2 or other.rank() < 2:
            panic("NDBuffer -> matmul_nd: operands must have rank >= 2")
        m, k = self.shape[-2:]
        k2, p = other.shape[-2:]
        if k != k2:
            panic("NDBuffer -> matmul_nd: inner dims must match, got", k, "and", k2)
        try:
            bshape = tuple(np.broadcast_shapes(self.shape[:-2], other.shape[:-2]))
        except ValueError:
            panic("NDBuffer -> matmul_nd: batch shapes not broadcastable:", self.shape[:-2], "vs", other.shape[:-2])
        out = NDBuffer.empty(bshape + (m, p))
        handle().gemm(m, p, k, self.mat(), other.mat(), out.data_ptr(), algo=_gemm_algo)
        return out

    def add_bias(self, bias: "NDBuffer") -> "NDBuffer":
        """arithmetic_ops[Add] with a trailing-dim broadcast right operand (ndbuffer.mojo:1856-1909)."""
        x = self.contiguous()
        n = bias.shape[-1]
        if x.shape[-1] != n or bias.numels() != n:
            panic("NDBuffer -> add: shapes not broadcastable:", self.shape, "and", bias.shape)
        out = NDBuffer.empty(x.shape)
        handle().add_bias(x.data_ptr(), bias.contiguous().data_ptr(), out.data_ptr(), x.numels() // n, n)
        return out

    def inplace_add(self, other: "NDBuffer"):
        """inplace_ops[Add]: the Gradbox accumulate (ndbuffer.mojo:1698-1732)."""
        if self.shape != other.shape or not self.is_contiguous():
            panic("NDBuffer -> inplace add: shape mismatch", self.shape, other.shape)
        handle().add_inplace(self.data_ptr(), other.contiguous().data_ptr(), self.numels())

    def fill(self, value: float):
        handle().fill(self.data_ptr(), value, self.numels())

    def sum_leading(self, target_shape) -> "NDBuffer":
        """sum_over_broadcasted_axes (sum_mean_reduction.mojo:184-211): sum the axes along which ``target_shape`` was
        broadcast -- extra leading dims and dims where the target has size 1 -- back to the target's shape.  Leading
        axes (bias gradient, broadcast batch) reduce in place as a column sum; interior size-1 axes (a batch such as
        (2,1,m,k) against (1,3,k,n)) are first moved to the front by a strided copy, then take the same kernel."""
        target_shape = tuple(int(d) for d in target_shape)
        if tuple(self.shape) == target_shape:
            return self
        rank = len(self.shape)
        if len(target_shape) > rank:
            panic("sum_over_broadcasted_axes: the target has more dims than the gradient:", self.shape, "->", target_shape)
        padded = (1,) * (rank - len(target_shape)) + target_shape
        summed = [d for d in range(rank) if padded[d] != self.shape[d]]
        if any(padded[d] != 1 for d in summed):
            panic("sum_over_broadcasted_axes: shapes are not a broadcast of one another:", self.shape, "->", target_shape)
        kept = [d for d in range(rank) if d not in summed]
        x = self
        if summed != list(range(len(summed))):  # an interior axis: bring the summed axes to the front
            order = summed + kept
            x = NDBuffer(self.storage, [self.shape[d] for d in order], [self.strides[d] for d in order], self.offset)
        x = x.contiguous()
        lead = int(np.prod([self.shape[d] for d in summed])) if summed else 1
        cols = x.numels() // lead if lead else 0
        out = NDBuffer.empty(target_shape)
        handle().colsum(x.data_ptr(), lead, cols, cols, out.data_ptr())
        return out


class Ancestry:
    """BackwardFnArg + parents (backpropagation.mojo:138-209, tensor.mojo:1007-1028)."""

    def __init__(self, op_code: int, parents, arg=None):
        self.op_code = op_code
        self.parents = list(parents)
        self.arg = arg


class Tensor:
    _next_id = 0

    def __init__(self, buffer: NDBuffer, requires_grad: bool = False):
        self.buffer = buffer
        self.requires_grad = requires_grad
        self.gradbox: NDBuffer | None = None
        self.ancestry: Ancestry | None = None
        Tensor._next_id += 1
        self._id = Tensor._next_id

    # -- construction ----------------------------------------------------------------------------------
    @staticmethod
    def from_numpy(a, requires_grad=False) -> "Tensor":
        return Tensor(NDBuffer.from_numpy(a), requires_grad)

    @staticmethod
    def d2(rows, requires_grad=False) -> "Tensor":
        return Tensor.from_numpy(np.asarray(rows, np.float32), requires_grad)

    d1 = d3 = d2

    @staticmethod
    def zeros(*shape, requires_grad=False) -> "Tensor":
        return Tensor(NDBuffer.zeros(shape), requires_grad)

    @staticmethod
    def ones(*shape, requires_grad=False) -> "Tensor":
        return Tensor.from_numpy(np.ones(shape, np.float32), requires_grad)

    @staticmethod
    def labels(values, dtype=np.int64) -> "Tensor":
        """Class-index targets; int64 is the reference's DEFAULT_INDEX_DTYPE (mnemonics.mojo:63)."""
        return Tensor(NDBuffer.from_numpy(values, dtype=dtype))

    # -- queries -----------------------------------------------------------------------------------------
    def shape(self):
        return self.buffer.shape

    def strides(self):
        return self.buffer.strides

    def numpy(self) -> np.ndarray:
        return self.buffer.numpy()

    def item(self) -> float:
        return float(self.buffer.numpy().reshape(-1)[0])

    def grad(self) -> "Tensor":
        if self.gradbox is None:
            panic("Tensor -> grad: requires_grad is False or no gradient has been accumulated")
        return Tensor(self.gradbox)

    def all_close(self, other, rtol=1e-5, atol=1e-8) -> bool:
        # buffers.mojo:1909-1946: |a - b| <= atol + rtol * |b|
        a = self.numpy().astype(np.float64)
        b = (other.numpy() if isinstance(other, Tensor) else np.asarray(other)).astype(np.float64)
        return a.shape == b.shape and bool(np.all(np.abs(a - b) <= atol + rtol * np.abs(b)))

    # -- views -------------------------------------------------------------------------------------------
    def transpose(self, axes=(-1, -2)) -> "Tensor":
        """A stride view; the gradient flows back through the same permutation (BACKWARD_TRANSPOSE)."""
        out = Tensor(self.buffer.transpose(axes), requires_grad=False)
        if self.requires_grad:
            out.requires_grad = True
            out.ancestry = Ancestry(BACKWARD_TRANSPOSE, [self], arg=tuple(axes))
        return out

    def view(self, shape, strides, offset=0) -> "Tensor":
        return Tensor(self.buffer.view(shape, strides, offset), requires_grad=False)

    # -- ops ---------------------------------------------------------------------------------------------
    def matmul(self, other: "Tensor", track_grad: bool = True, mode: str = "mm") -> "Tensor":
        """Tensor.matmul -> Matmul.forward (tensor.mojo:4141-4159, matmul.mojo:202-241).  ``mode`` mirrors the
        reference's compile-time ``mode`` parameter: "mm" classifies by rank, "mv" / "vm" / "dot" force it."""
        a, b = self.shape(), other.shape()
        if mode != "mm":
            return self._matmul_rank1(other, track_grad, mode)
        if len(a) <= 1 or len(b) <= 1:  # classify_matmul (matmul.mojo:258-272): dot / vm / mv
            return self._matmul_rank1(other, track_grad)
        if a[-1] != b[-2]:
            panic("Matmul: incompatible shapes", a, b)
        two_d = len(a) == 2 and len(b) == 2
        ndb = self.buffer.matmul_2d(other.buffer) if two_d else self.buffer.matmul_nd(other.buffer)
        out = Tensor(ndb)
        if track_grad and (self.requires_grad or other.requires_grad):
            out.requires_grad = True
            out.ancestry = Ancestry(BACKWARD_MATMUL_2D if two_d else BACKWARD_MATMUL_ND, [self, other])
        return out

    def _matmul_rank1(self, other: "Tensor", track_grad: bool, kind: str | None = None) -> "Tensor":
        """dot, vector @ matrix and matrix @ vector (dotproduct.mojo, vectormatrix.mojo:210-375,
        matrixvector.mojo:205-402) as GEMMs with a unit dimension: the vector becomes a (1,k) row or a (k,1)
        column view, batch dims broadcast as usual, and the unit dim is dropped from the result."""
        a, b = self.shape(), other.shape()
        if len(a) == 0 or len(b) == 0:
            panic("Matmul: scalar operands")
        if kind is None:
            kind = "dot" if (len(a) == 1 and len(b) == 1) else ("vm" if len(a) == 1 else "mv")
        if kind == "dot":
            code, la, lb, drop = BACKWARD_DOT, self.buffer.unsqueeze(0), other.buffer.unsqueeze(1), (-1, -2)
        elif kind == "vm":  # v[..., k] @ M[..., k, n] -> [..., n]
            code, la, lb, drop = BACKWARD_VECTOR_MATMUL, self.buffer.unsqueeze(len(a) - 1), other.buffer, (-2,)
        else:  # M[..., m, k] @ v[..., k] -> [..., m]
            code, la, lb, drop = BACKWARD_MATRIX_VECTOR_MUL, self.buffer, other.buffer.unsqueeze(len(b)), (-1,)
        if la.shape[-1] != lb.shape[-2]:
            panic("Matmul: incompatible shapes", a, b)
        fast = self._rank1_hbm_kernel(other, kind)
        if fast is not None:
            out = Tensor(fast)
            if track_grad and (self.requires_grad or other.requires_grad):
                out.requires_grad = True
                full_shape = tuple(la.shape[:-1]) + (lb.shape[-1],)
                out.ancestry = Ancestry(code, [self, other], arg=dict(la=la, lb=lb, full_shape=full_shape))
            return out
        full = la.matmul_nd(lb)
        shape = list(full.shape)
        for d in sorted((ax % len(shape) for ax in drop), reverse=True):
            del shape[d]
        out = Tensor(full.reshape(tuple(shape)))
        if track_grad and (self.requires_grad or other.requires_grad):
            out.requires_grad = True
            out.ancestry = Ancestry(code, [self, other], arg=dict(la=la, lb=lb, full_shape=full.shape))
        return out

    def _rank1_hbm_kernel(self, other: "Tensor", kind: str):
        """Large unbatched matrix @ vector / vector @ matrix products go to the bandwidth-bound kernels
        (tenmo_gemv_f32 / tenmo_vecmat_f32); small ones, batched ones and matrices without a unit-stride axis keep the
        GEMM with a unit dimension, whose k-ascending chain is bit-identical to the reference's loops."""
        if kind == "mv":
            M, v = self.buffer, other.buffer
        elif kind == "vm":
            v, M = self.buffer, other.buffer
        else:
            return None
        if len(M.shape) != 2 or len(v.shape) != 1 or M.numels() < (1 << 20) or 1 not in M.strides or v.strides[0] < 1:
            return None
        out = NDBuffer.empty((M.shape[0] if kind == "mv" else M.shape[1],))
        mat = make_mat(M.storage.data_ptr(), M.shape, M.strides, M.offset)
        vptr = v.storage.data_ptr() + 4 * v.offset
        if kind == "mv":
            handle().gemv(M.shape[0], M.shape[1], mat, vptr, v.strides[0], out.data_ptr())
        else:
            handle().vecmat(M.shape[0], M.shape[1], vptr, v.strides[0], mat, out.data_ptr())
        return out

    def __matmul__(self, other):
        return self.matmul(other)

    def add_bias(self, bias: "Tensor", track_grad: bool = True) -> "Tensor":
        """Adder.forward with differing shapes => BACKWARD_ADD_BROADCAST (addition.mojo:71-112)."""
        out = Tensor(self.buffer.add_bias(bias.buffer))
        if track_grad and (self.requires_grad or bias.requires_grad):
            out.requires_grad = True
            out.ancestry = Ancestry(BACKWARD_ADD_BROADCAST, [self, bias])
        return out

    def relu(self, track_grad: bool = True) -> "Tensor":
        """ReLU.forward: output and a float 0/1 mask kept for backward (relu.mojo:50-95)."""
        x = self.buffer.contiguous()
        out, mask = NDBuffer.empty(x.shape), NDBuffer.empty(x.shape)
        handle().relu_fwd(x.data_ptr(), out.data_ptr(), mask.data_ptr(), x.numels())
        t = Tensor(out)
        if track_grad and self.requires_grad:
            t.requires_grad = True
            t.ancestry = Ancestry(BACKWARD_RELU, [self], arg=mask)
        return t

    def sigmoid(self, track_grad: bool = True) -> "Tensor":
        """Sigmoid.forward; the output is kept for backward (sigmoid.mojo:32-53)."""
        x = self.buffer.contiguous()
        out = NDBuffer.empty(x.shape)
        handle().sigmoid_fwd(x.data_ptr(), out.data_ptr(), x.numels())
        t = Tensor(out)
        if track_grad and self.requires_grad:
            t.requires_grad = True
            t.ancestry = Ancestry(BACKWARD_SIGMOID, [self], arg=out)
        return t

    def softmax(self, track_grad: bool = True) -> "Tensor":
        """Softmax over the last axis (Softmax.forward, softmax.mojo:222-305); the output is kept for backward."""
        x = self.buffer.contiguous()
        C = x.shape[-1]
        M = x.numels() // C
        out = NDBuffer.empty(x.shape)
        handle().softmax_fwd(x.data_ptr(), C, out.data_ptr(), M, C)
        t = Tensor(out)
        if track_grad and self.requires_grad:
            t.requires_grad = True
            t.ancestry = Ancestry(BACKWARD_SOFTMAX, [self], arg=out)
        return t

    def sum(self) -> "Tensor":
        """Scalar sum of all elements (used by the reference's matmul gradient tests as the loss)."""
        x = self.buffer.contiguous()
        out = NDBuffer.empty(())
        handle().colsum(x.data_ptr(), x.numels(), 1, 1, out.data_ptr())
        t = Tensor(out)
        if self.requires_grad:
            t.requires_grad = True
            t.ancestry = Ancestry(BACKWARD_SUM, [self])
        return t

    # -- autograd ------------------------------------------------------------------------------------------
    def zero_grad(self):
        if self.gradbox is not None:
            self.gradbox.fill(0.0)

    def seed_grad(self, value: float):
        self.gradbox = NDBuffer.empty(self.shape())
        self.gradbox.fill(value)

    def update_grad(self, incoming: NDBuffer):
        """Ancestor.update_grad with AddTensor: gradbox += incoming (ancestry.mojo:72-105)."""
        if self.gradbox is None:
            self.gradbox = NDBuffer.zeros(self.shape())
        if tuple(incoming.shape) != tuple(self.shape()):
            incoming = incoming.reshape(self.shape())
        self.gradbox.inplace_add(incoming)

    def backward(self, start_grad=1.0, retain_graph: bool = False):
        """Tensor.backward (tensor.mojo:3132-3247)."""
        if not self.requires_grad:
            return
        if isinstance(start_grad, Tensor):
            self.gradbox = NDBuffer.zeros(self.shape())
            self.gradbox.inplace_add(start_grad.buffer.reshape(self.shape()))
        else:
            self.seed_grad(float(start_grad))
        # DFS: collect nodes, count fan-in (number of children that will send a gradient)
        fan_in: dict[int, int] = {}
        nodes: dict[int, Tensor] = {self._id: self}
        stack = [self]
        seen = {self._id}
        while stack:
            node = stack.pop()
            if node.ancestry is None:
                continue
            for par in node.ancestry.parents:
                if not par.requires_grad:
                    continue
                fan_in[par._id] = fan_in.get(par._id, 0) + 1
                if par._id not in seen:
                    seen.add(par._id)
                    nodes[par._id] = par
                    stack.append(par)
        ready = deque([self])
        while ready:
            node = ready.popleft()
            if node.ancestry is None:
                continue
            touched = Backward.invoke(node, retain_graph)
            for par in touched:
                fan_in[par._id] -= 1
                if fan_in[par._id] == 0:
                    ready.append(par)


class Backward:
    """Backward.invoke: if/elif dispatch on the integer tag (backpropagation.mojo:278-519)."""

    @staticmethod
    def invoke(output: Tensor, retain_graph: bool):
        code = output.ancestry.op_code
        if code == BACKWARD_MATMUL_2D or code == BACKWARD_MATMUL_ND:
            return Backward.matmul(output, retain_graph)
        elif code == BACKWARD_ADD_BROADCAST:
            return Backward.add_broadcast(output, retain_graph)
        elif code == BACKWARD_RELU:
            return Backward.relu(output, retain_graph)
        elif code == BACKWARD_SIGMOID:
            return Backward.sigmoid(output, retain_graph)
        elif code == BACKWARD_SUM:
            return Backward.sum(output, retain_graph)
        elif code == BACKWARD_TRANSPOSE:
            return Backward.transpose(output, retain_graph)
        elif code == BACKWARD_SOFTMAX:
            return Backward.softmax(output, retain_graph)
        elif code in (BACKWARD_MATRIX_VECTOR_MUL, BACKWARD_VECTOR_MATMUL, BACKWARD_DOT):
            return Backward.matmul_rank1(output, retain_graph)
        elif code in (BACKWARD_CE_CLASS_INDICES_INT64, BACKWARD_CE_CLASS_INDICES_INT32):
            from .crossentropy import ce_class_indices_backward

            return ce_class_indices_backward(output, retain_graph)
        panic("Backward.invoke: unknown op code", code)

    @staticmethod
    def matmul(output: Tensor, retain_graph: bool):
        """Matmul2dBackward / MatmulNdBackward (matmul.mojo:24-54,101-137): dA = dC.B^T, dB = A^T.dC on
        transposed stride views, each only if that parent requires grad; batched results are summed back
        over broadcast batch dims; `+=` into the parent's gradbox."""
        grad_out = output.gradbox
        A, B = output.ancestry.parents
        touched = []
        if A.requires_grad:
            ndb = grad_out.matmul_nd(B.buffer.transpose((-1, -2)))
            A.update_grad(ndb.sum_leading(A.shape()))
            touched.append(A)
        if B.requires_grad:
            ndb = A.buffer.transpose((-1, -2)).matmul_nd(grad_out)
            B.update_grad(ndb.sum_leading(B.shape()))
            touched.append(B)
        if not retain_graph:
            grad_out.fill(0.0)
        return touched

    @staticmethod
    def matmul_rank1(output: Tensor, retain_graph: bool):
        """MatrixVectorMulNdBackward / VectorMatmulNdBackward / dot backward (matrixvector.mojo:15-201,
        vectormatrix.mojo:14-206): the outer-product and gemv gradients are the two backward GEMMs of the
        unit-dimension matmul, summed over broadcast batch dims back to each parent's shape."""
        arg = output.ancestry.arg
        la, lb = arg["la"], arg["lb"]
        A, B = output.ancestry.parents
        g = output.gradbox.reshape(arg["full_shape"])
        touched = []
        if A.requires_grad:
            ndb = g.matmul_nd(lb.transpose((-1, -2)))
            A.update_grad(ndb.sum_leading(la.shape).reshape(A.shape()))
            touched.append(A)
        if B.requires_grad:
            ndb = la.transpose((-1, -2)).matmul_nd(g)
            B.update_grad(ndb.sum_leading(lb.shape).reshape(B.shape()))
            touched.append(B)
        if not retain_graph:
            output.gradbox.fill(0.0)
        return touched

    @staticmethod
    def add_broadcast(output: Tensor, retain_graph: bool):
        """BroadcastBackward[augment=False] (broadcast.mojo:17-88): the left parent gets the upstream
        unchanged, the bias gets the upstream summed over the broadcast axes."""
        grad_out = output.gradbox
        left, bias = output.ancestry.parents
        touched = []
        if left.requires_grad:
            left.update_grad(grad_out)
            touched.append(left)
        if bias.requires_grad:
            bias.update_grad(grad_out.sum_leading(bias.shape()))
            touched.append(bias)
        if not retain_graph:
            grad_out.fill(0.0)
        return touched

    @staticmethod
    def relu(output: Tensor, retain_graph: bool):
        """ReLUBackward: grad * mask (relu.mojo:19-46)."""
        (parent,) = output.ancestry.parents
        mask = output.ancestry.arg
        g = output.gradbox
        dx = NDBuffer.empty(g.shape)
        handle().relu_bwd(g.data_ptr(), mask.data_ptr(), dx.data_ptr(), g.numels())
        parent.update_grad(dx)
        if not retain_graph:
            g.fill(0.0)
        return [parent]

    @staticmethod
    def sigmoid(output: Tensor, retain_graph: bool):
        """SigmoidBackward: g * y * (1 - y) (sigmoid.mojo:9-29)."""
        (parent,) = output.ancestry.parents
        y = output.ancestry.arg
        g = output.gradbox
        dx = NDBuffer.empty(g.shape)
        handle().sigmoid_bwd(g.data_ptr(), y.data_ptr(), dx.data_ptr(), g.numels())
        parent.update_grad(dx)
        if not retain_graph:
            g.fill(0.0)
        return [parent]

    @staticmethod
    def softmax(output: Tensor, retain_graph: bool):
        """SoftmaxBackwardDelegate (softmax.mojo:206-213): y * (g - sum(g * y)) in one kernel."""
        (parent,) = output.ancestry.parents
        y = output.ancestry.arg
        g = output.gradbox
        C = y.shape[-1]
        dx = NDBuffer.empty(y.shape)
        handle().softmax_bwd(y.data_ptr(), g.data_ptr(), dx.data_ptr(), y.numels() // C, C)
        parent.update_grad(dx)
        if not retain_graph:
            g.fill(0.0)
        return [parent]

    @staticmethod
    def transpose(output: Tensor, retain_graph: bool):
        """The upstream gradient, permuted back, is added to the parent (a host-side layout step next to the
        path: the strided copy is torch's, not a kernel of this library)."""
        (parent,) = output.ancestry.parents
        parent.update_grad(output.gradbox.transpose(output.ancestry.arg).contiguous())
        if not retain_graph:
            output.gradbox.fill(0.0)
        return [parent]

    @staticmethod
    def sum(output: Tensor, retain_graph: bool):
        """The upstream scalar spread over the parent's shape, without a host round trip: a (numel, 1) column of ones
        times the (1, 1) upstream gradient, accumulated by the GEMM's epilogue."""
        (parent,) = output.ancestry.parents
        n = int(np.prod(parent.shape())) if parent.shape() else 1
        ones = NDBuffer(torch.ones(max(n, 1), dtype=torch.float32, device="cuda"), (n, 1))
        inc = NDBuffer.empty(parent.shape())
        g = output.gradbox.reshape((1, 1))
        handle().gemm(n, 1, 1, ones.mat(), g.mat(), inc.data_ptr(), algo=_lib.ALGO_SIMT_FP32)  # exact: 1.0 * g
        parent.update_grad(inc)
        if not retain_graph:
            output.gradbox.fill(0.0)
        return [parent]
