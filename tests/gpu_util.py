"""Helpers for the gpu-marked tests: device buffers come from torch, every op goes through the C ABI."""
import numpy as np
import torch

from tenmo_b200 import TenmoCuda, make_mat

_handle = None


def handle() -> TenmoCuda:
    """One context for the test session, bound to torch's current stream.  Fails loudly when the CUDA
    library is missing or the device is not a B200-class GPU."""
    global _handle
    if _handle is None:
        _handle = TenmoCuda(0).require()
    _handle.set_stream(torch.cuda.current_stream().cuda_stream)
    return _handle


def dev(a, dtype=np.float32) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(a, dtype=dtype)).cuda()


def empty(*shape) -> torch.Tensor:
    return torch.empty(*shape, dtype=torch.float32, device="cuda")


def host(t: torch.Tensor) -> np.ndarray:
    return t.detach().cpu().numpy()


def gpu_matmul(view_a, view_b, *, algo=0, beta=0.0, bias=None, act=0, want_aux=False, c_init=None, colsum=False):
    """Runs tenmo_gemm_f32 on two oracle-style views (flat base + shape/strides/offset).
    Returns (C, aux, colsum) as numpy arrays (aux/colsum None when not requested)."""
    h = handle()
    a_dev, b_dev = dev(view_a.base), dev(view_b.base)
    M, K = view_a.shape[-2:]
    K2, N = view_b.shape[-2:]
    assert K == K2
    bshape = tuple(np.broadcast_shapes(view_a.shape[:-2], view_b.shape[:-2]))
    out_shape = bshape + (M, N)
    if c_init is not None:
        c = dev(c_init)
    else:
        c = torch.full(out_shape, float("nan"), dtype=torch.float32, device="cuda")
    aux = torch.full(out_shape, float("nan"), dtype=torch.float32, device="cuda") if want_aux else None
    cs = torch.zeros(N, dtype=torch.float32, device="cuda") if colsum else None
    bias_dev = dev(bias) if bias is not None else None
    ma = make_mat(a_dev.data_ptr(), view_a.shape, view_a.strides, view_a.offset)
    mb = make_mat(b_dev.data_ptr(), view_b.shape, view_b.strides, view_b.offset)
    h.gemm(M, N, K, ma, mb, c.data_ptr(), algo=algo, beta=beta, bias=bias_dev.data_ptr() if bias is not None else 0,
           act=act, aux=aux.data_ptr() if want_aux else 0, colsum=cs.data_ptr() if colsum else 0)
    torch.cuda.synchronize()
    return host(c), (host(aux) if want_aux else None), (host(cs) if colsum else None)
