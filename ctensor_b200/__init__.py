"""ctensor_b200 — B200 (sm_100a) elementwise / broadcast / reduction operators behind a C ABI.

The product is ``libctb200.so`` (sources in ``ctensor_b200/csrc``, interface in
``include/ctb200.h``).  This module is the thin Python binding used by the tests and the
benchmark: it loads the library with ctypes, wraps device memory held by torch tensors in
``ctb_view`` structs and calls the C entry points on torch's current CUDA stream.  torch only
provides memory, streams and process groups; no torch operator computes a result here.

There is no CPU fallback: importing works anywhere, but every operator call needs the built
library and a CUDA device and raises otherwise.
"""
from __future__ import annotations

import ctypes
import os
from dataclasses import dataclass
from typing import Optional, Sequence

_PKG_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG_DIR, "libctb200.so")
MAX_DIMS = 8

# dtypes (reference DType numbering)
F32, I32, F64, U8, U16, U32, U64, I8, I16, I64, BOOL = range(11)        # the reference's DType numbering
# binary operators
ADD, SUB, MUL, DIV, LT, LE, GT, GE, EQ, NE, POW = range(11)
# unary operators
(ADD_S, SUB_S, RSUB_S, MUL_S, DIV_S, RDIV_S, POW_S, RPOW_S, LT_S, LE_S, GT_S, GE_S, EQ_S, NE_S,
 ABS, RELU, EXP, LOG, TANH, SIGMOID, SQRT, GELU_TANH,
 SIN, COS, TAN, ASIN, ACOS, ATAN, SINH, COSH, SOFTPLUS) = range(31)
# reductions
SUM, MEAN, MAX, MIN, VAR, ARGMAX = range(6)
DIM_FULL = -1

STATUS_NAMES = {0: "CTB_OK", 1: "CTB_ERR_NULL", 2: "CTB_ERR_SHAPE", 3: "CTB_ERR_DTYPE",
                4: "CTB_ERR_DIM", 5: "CTB_ERR_ARG", 6: "CTB_ERR_CUDA", 7: "CTB_ERR_WORKSPACE",
                8: "CTB_ERR_LIMIT"}

# every symbol include/ctb200.h declares
EXPORTED_SYMBOLS = [
    "ctb_abi_version", "ctb_last_error", "ctb_device_count", "ctb_alloc", "ctb_free", "ctb_sync",
    "ctb_alloc_managed", "ctb_free_managed", "ctb_set_device", "ctb_device_sync",
    "ctb_binary", "ctb_unary", "ctb_copy_strided", "ctb_reduce", "ctb_reduce_workspace_bytes",
    "ctb_reduce_ws", "ctb_reduce_dim_noalloc", "ctb_reduce_full_partial", "ctb_finalize_full", "ctb_softmax_lastdim",
    "ctb_layernorm_lastdim", "ctb_binary_host", "ctb_unary_host", "ctb_reduce_host",
    "ctb_log_softmax_lastdim", "ctb_gather", "ctb_accumulate_grad", "ctb_sgd_step", "ctb_adam_step",
    "ctb_copy_into", "ctb_cat", "ctb_channel_moments", "ctb_batchnorm_apply",
    "ctb_matmul", "ctb_optimizer_step",
    "ctb_pool_alloc_managed", "ctb_pool_free_managed", "ctb_pool_trim", "ctb_pool_set_limit", "ctb_pool_stats",
    "ctb_prefetch_managed",
    "ctb_div_backward", "ctb_tanh_backward", "ctb_cross_entropy", "ctb_cross_entropy_backward",
    "ctb_shard_range", "ctb_comm_init_all", "ctb_comm_size", "ctb_comm_device", "ctb_comm_stream", "ctb_comm_sync",
    "ctb_comm_destroy", "ctb_allreduce", "ctb_full_reduce_sharded", "ctb_matmul_tc",
]


class CtbError(RuntimeError):
    """A C-ABI call returned a non-zero status.  ``code`` is the ctb_status value; the message
    is the library's, which equals the reference's exception text for the same mistake."""

    def __init__(self, code: int, message: str):
        super().__init__(f"{STATUS_NAMES.get(code, code)}: {message}")
        self.code = code
        self.message = message


class OptimizerHyper(ctypes.Structure):
    """struct ctb_optimizer_hyper."""
    _fields_ = [(n, ctypes.c_double) for n in ("lr", "beta1", "beta2", "eps", "weight_decay", "alpha")]


(OPT_SGD, OPT_ADAM, OPT_ADAMW, OPT_ADAMAX, OPT_NADAM, OPT_RADAM, OPT_RMSPROP, OPT_ADAGRAD, OPT_LION) = range(9)


class PoolInfo(ctypes.Structure):
    """struct ctb_pool_info."""
    _fields_ = [("live_bytes", ctypes.c_size_t), ("cached_bytes", ctypes.c_size_t), ("cached_blocks", ctypes.c_size_t),
                ("hits", ctypes.c_uint64), ("misses", ctypes.c_uint64), ("trims", ctypes.c_uint64)]


class View(ctypes.Structure):
    """struct ctb_view."""
    _fields_ = [("base", ctypes.c_void_p), ("offset", ctypes.c_int64),
                ("dtype", ctypes.c_int32), ("ndim", ctypes.c_int32),
                ("shape", ctypes.c_int64 * MAX_DIMS), ("stride", ctypes.c_int64 * MAX_DIMS)]


def make_view(base: int, dtype: int, shape: Sequence[int], strides: Sequence[int], offset: int = 0) -> View:
    if len(shape) > MAX_DIMS:
        raise CtbError(5, f"ndim {len(shape)} not in 0..{MAX_DIMS}")
    v = View()
    v.base = base
    v.offset = offset
    v.dtype = dtype
    v.ndim = len(shape)
    for i, (s, st) in enumerate(zip(shape, strides)):
        v.shape[i] = s
        v.stride[i] = st
    return v


_lib = None


def lib() -> ctypes.CDLL:
    """Load libctb200.so (built in-tree by ``ctensor_b200.build``)."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it first (python -c 'import __graft_entry__ as g; g.build()' "
            "or python -m ctensor_b200.build).  There is no CPU fallback.")
    L = ctypes.CDLL(LIB_PATH)
    vp, vd, i32, i64 = ctypes.POINTER(View), ctypes.c_void_p, ctypes.c_int, ctypes.c_int64
    L.ctb_abi_version.restype = i32
    L.ctb_last_error.restype = ctypes.c_char_p
    L.ctb_device_count.restype = i32
    L.ctb_alloc.argtypes = [ctypes.POINTER(vd), ctypes.c_size_t, i32, vd]
    L.ctb_free.argtypes = [vd, vd]
    L.ctb_sync.argtypes = [vd]
    L.ctb_alloc_managed.argtypes = [ctypes.POINTER(vd), ctypes.c_size_t, i32]
    L.ctb_free_managed.argtypes = [vd]
    L.ctb_pool_alloc_managed.argtypes = [ctypes.POINTER(vd), ctypes.c_size_t, i32, i32, vd]
    L.ctb_pool_free_managed.argtypes = [vd]
    L.ctb_pool_trim.argtypes = [i32]
    L.ctb_pool_set_limit.argtypes = [i32, ctypes.c_size_t]
    L.ctb_pool_stats.argtypes = [i32, ctypes.POINTER(PoolInfo)]
    L.ctb_prefetch_managed.argtypes = [vd, ctypes.c_size_t, i32, vd]
    L.ctb_shard_range.argtypes = [i64, i32, i32, ctypes.POINTER(i64), ctypes.POINTER(i64)]
    L.ctb_comm_init_all.argtypes = [i32, ctypes.POINTER(i32)]
    L.ctb_comm_device.argtypes = [i32]
    L.ctb_comm_stream.argtypes = [i32]
    L.ctb_comm_stream.restype = vd
    L.ctb_allreduce.argtypes = [ctypes.POINTER(vd), ctypes.c_size_t, i32, i32]
    L.ctb_full_reduce_sharded.argtypes = [i32, ctypes.POINTER(vp), i64, ctypes.POINTER(vp)]
    L.ctb_div_backward.argtypes = [vp, vp, vp, vp, vp, i32, vd]
    L.ctb_tanh_backward.argtypes = [vp, vp, vp, i32, vd]
    L.ctb_cross_entropy.argtypes = [vp, vp, i32, vp, vd, vd]
    L.ctb_cross_entropy_backward.argtypes = [vp, vp, ctypes.c_double, vp, i32, vd, vd]
    L.ctb_binary.argtypes = [i32, vp, vp, vp, vd]
    L.ctb_unary.argtypes = [i32, vp, ctypes.c_double, vp, vd]
    L.ctb_copy_strided.argtypes = [vp, vp, vd]
    L.ctb_reduce.argtypes = [i32, vp, i32, vp, vd]
    L.ctb_reduce_workspace_bytes.restype = ctypes.c_size_t
    L.ctb_reduce_workspace_bytes.argtypes = [vp, i32]
    L.ctb_reduce_ws.argtypes = [i32, vp, i32, vp, vd, ctypes.c_size_t, vd]
    L.ctb_reduce_dim_noalloc.argtypes = [i32, vp, i32, vp, vd]
    L.ctb_reduce_full_partial.argtypes = [i32, vp, vd, vd]
    L.ctb_finalize_full.argtypes = [i32, vd, i64, vp, vd]
    L.ctb_softmax_lastdim.argtypes = [vp, vp, i32, vp, vd]
    L.ctb_layernorm_lastdim.argtypes = [vp, vp, vp, ctypes.c_double, vp, vd]
    L.ctb_log_softmax_lastdim.argtypes = [vp, vp, vp, vd]
    L.ctb_gather.argtypes = [vp, i32, vp, vp, vd, vd]
    L.ctb_accumulate_grad.argtypes = [vp, vp, vd]
    L.ctb_sgd_step.argtypes = [vp, vp, ctypes.c_double, vd]
    L.ctb_copy_into.argtypes = [vp, vp, vd]
    L.ctb_matmul.argtypes = [vp, vp, vp, vd]
    L.ctb_matmul_tc.argtypes = [vp, vp, vp, vd, vd]
    L.ctb_optimizer_step.argtypes = [i32, vp, vp, vd, vd, ctypes.POINTER(OptimizerHyper), i32, vd]
    L.ctb_channel_moments.argtypes = [vp, vp, vp, vd]
    L.ctb_batchnorm_apply.argtypes = [vp, vp, vp, vp, vp, ctypes.c_double, vp, vd]
    L.ctb_cat.argtypes = [ctypes.POINTER(vp), i32, i32, vp, vd]
    L.ctb_adam_step.argtypes = [vp, vp, vd, vd] + [ctypes.c_double] * 4 + [i32, ctypes.c_double, i32, vd]
    L.ctb_binary_host.argtypes = [i32, vp, vp, vp, i32]
    L.ctb_unary_host.argtypes = [i32, vp, ctypes.c_double, vp, i32]
    L.ctb_reduce_host.argtypes = [i32, vp, i32, vp, i32]
    for name in EXPORTED_SYMBOLS:      # AttributeError here = the library lacks a declared symbol
        getattr(L, name)
    _lib = L
    return L


def check(status: int) -> None:
    if status != 0:
        raise CtbError(status, lib().ctb_last_error().decode())


# ---- torch plumbing (device memory + streams) -------------------------------------------------------
def _torch():
    import torch
    return torch


def _dtype_code(t) -> int:
    torch = _torch()
    try:
        return _TORCH_CODES[t.dtype] if _TORCH_CODES else _torch_codes()[t.dtype]
    except KeyError:
        raise CtbError(3, f"unsupported dtype {t.dtype}")


_TORCH_CODES: dict = {}


def _torch_codes() -> dict:
    """torch dtype -> element-type code (the reference's DType numbering)."""
    torch = _torch()
    _TORCH_CODES.update({torch.float32: F32, torch.int32: I32, torch.float64: F64, torch.uint8: U8, torch.int8: I8,
                         torch.int16: I16, torch.int64: I64, torch.bool: BOOL})
    for name, code in (("uint16", U16), ("uint32", U32), ("uint64", U64)):      # copy-only types; newer torch has them
        if hasattr(torch, name):
            _TORCH_CODES[getattr(torch, name)] = code
    return _TORCH_CODES


def _torch_dtype(code: int):
    return {v: k for k, v in _torch_codes().items()}[code]


@dataclass
class DView:
    """A strided view of a torch storage buffer: the (Storage, offset, shape, strides) quadruple
    of the reference's Tensorimpl.  ``buf`` is a 1-d torch tensor (CUDA for the device entry
    points, CPU — ideally pinned — for the ``*_host`` ones)."""
    buf: "object"
    shape: tuple
    strides: tuple
    offset: int = 0

    @staticmethod
    def of(t) -> "DView":
        """View of a torch tensor as it is (its own strides; offset folded into data_ptr)."""
        if any(s < 0 for s in t.stride()):
            raise CtbError(5, "negative strides are not supported")
        return DView(t, tuple(t.shape), tuple(t.stride()), 0)

    @property
    def dtype(self) -> int:
        return _dtype_code(self.buf)

    @property
    def numel(self) -> int:
        n = 1
        for s in self.shape:
            n *= s
        return n

    def cview(self) -> View:
        """The C descriptor of this view; built once per DView (a view never changes), so a caller that
        keeps its DViews pays the ctypes marshalling once, not per call."""
        cv = self.__dict__.get("_cv")
        if cv is None:
            cv = make_view(self.buf.data_ptr(), self.dtype, self.shape, self.strides, self.offset)
            self.__dict__["_cv"] = cv
        return cv

    def permute(self, dims: Sequence[int]) -> "DView":
        return DView(self.buf, tuple(self.shape[d] for d in dims), tuple(self.strides[d] for d in dims), self.offset)


def _as_dview(x) -> DView:
    return x if isinstance(x, DView) else DView.of(x)


def _stream_ptr(x: DView) -> int:
    torch = _torch()
    if not x.buf.is_cuda:
        raise CtbError(6, "device entry point called with host memory (use the *_host functions)")
    return torch.cuda.current_stream(x.buf.device).cuda_stream


class _NoGuard:
    def __enter__(self):
        return None

    def __exit__(self, *exc):
        return False


_NO_GUARD = _NoGuard()


def _device_guard(x: DView):
    """Makes the tensor's device current for the call; free when it already is."""
    cuda = _torch().cuda
    dev = x.buf.device
    if dev.type == "cuda" and dev.index == cuda.current_device():
        return _NO_GUARD
    return cuda.device(dev)


def broadcast_shape(a: Sequence[int], b: Sequence[int]) -> tuple:
    nd = max(len(a), len(b))
    out = []
    for i in range(nd):
        da = 1 if i < nd - len(a) else a[i - (nd - len(a))]
        db = 1 if i < nd - len(b) else b[i - (nd - len(b))]
        if da != db and da != 1 and db != 1:
            raise CtbError(2, "Shape mismatch in binary op")
        out.append(db if da == 1 else da)
    return tuple(out)


def reduced_shape(shape: Sequence[int], dim: int) -> tuple:
    if dim == DIM_FULL:
        return (1,)
    s = tuple(x for i, x in enumerate(shape) if i != dim)
    return s if s else (1,)


def _new_out(like: DView, shape, dtype_code=None):
    torch = _torch()
    return torch.empty(shape, dtype=_torch_dtype(like.dtype if dtype_code is None else dtype_code),
                       device=like.buf.device)


# ---- operators (device memory) ------------------------------------------------------------------------
def binary(op: int, a, b, out=None):
    """out = a (op) b with broadcasting; a, b: torch CUDA tensors or DViews."""
    a, b = _as_dview(a), _as_dview(b)
    if out is None:
        out = _new_out(a, broadcast_shape(a.shape, b.shape))
    with _device_guard(a):
        check(lib().ctb_binary(op, a.cview(), b.cview(), _as_dview(out).cview(), _stream_ptr(a)))
    return out


def unary(op: int, a, scalar: float = 0.0, out=None):
    a = _as_dview(a)
    if out is None:
        out = _new_out(a, a.shape)
    with _device_guard(a):
        check(lib().ctb_unary(op, a.cview(), float(scalar), _as_dview(out).cview(), _stream_ptr(a)))
    return out


def contiguous(a, out=None):
    """Strided gather into fresh row-major storage (Tensor::contiguous / clone)."""
    a = _as_dview(a)
    if out is None:
        out = _new_out(a, a.shape)
    with _device_guard(a):
        check(lib().ctb_copy_strided(a.cview(), _as_dview(out).cview(), _stream_ptr(a)))
    return out


def reduce(op: int, a, dim: int = DIM_FULL, out=None, workspace=None):
    """sum/mean/max/min/var/argmax along ``dim`` (DIM_FULL = everything)."""
    a = _as_dview(a)
    if out is None:
        out = _new_out(a, reduced_shape(a.shape, dim), I32 if op == ARGMAX else None)
    with _device_guard(a):
        if workspace is None:
            check(lib().ctb_reduce(op, a.cview(), dim, _as_dview(out).cview(), _stream_ptr(a)))
        else:
            check(lib().ctb_reduce_ws(op, a.cview(), dim, _as_dview(out).cview(), workspace.data_ptr(),
                                      workspace.numel() * workspace.element_size(), _stream_ptr(a)))
    return out


NOALLOC_SCRATCH_BYTES = 4 * 1024 * 1024 + 64 * 1024


def reduce_dim_noalloc(op: int, a, dim: int, out):
    """ctb_reduce_dim_noalloc: the dim-wise reduction for callers that must not allocate device
    memory (allocator callbacks, fully budgeted or real-time processes).  Scratch comes from a
    fixed array inside the library; `out` must be provided; shapes that need more than
    NOALLOC_SCRATCH_BYTES of scratch raise CtbError(CTB_ERR_LIMIT).  Calls on one device share
    that array: keep them stream-ordered, and make the first call outside stream capture."""
    a = _as_dview(a)
    with _device_guard(a):
        check(lib().ctb_reduce_dim_noalloc(op, a.cview(), dim, _as_dview(out).cview(), _stream_ptr(a)))
    return out


def reduce_workspace_bytes(a, dim: int) -> int:
    return int(lib().ctb_reduce_workspace_bytes(_as_dview(a).cview(), dim))


def reduce_full_partial(op: int, a, partial=None):
    """fp64 partial of a full reduction over this shard (device tensor with one double)."""
    torch = _torch()
    a = _as_dview(a)
    if partial is None:
        partial = torch.empty(1, dtype=torch.float64, device=a.buf.device)
    with _device_guard(a):
        check(lib().ctb_reduce_full_partial(op, a.cview(), partial.data_ptr(), _stream_ptr(a)))
    return partial


def finalize_full(op: int, partial, total_count: int, out=None, dtype_code: int = F32):
    torch = _torch()
    if out is None:
        out = torch.empty(1, dtype=_torch_dtype(dtype_code), device=partial.device)
    with torch.cuda.device(partial.device):
        check(lib().ctb_finalize_full(op, partial.data_ptr(), int(total_count), _as_dview(out).cview(),
                                      torch.cuda.current_stream(partial.device).cuda_stream))
    return out


def softmax(x, mask=None, causal: bool = False, out=None):
    x = _as_dview(x)
    m = None if mask is None else _as_dview(mask)
    if out is None:
        out = _new_out(x, x.shape)
    with _device_guard(x):
        check(lib().ctb_softmax_lastdim(x.cview(), None if m is None else m.cview(), int(causal),
                                        _as_dview(out).cview(), _stream_ptr(x)))
    return out


def log_softmax(x, mask=None, out=None):
    """(t - max t) - ln(sum exp(t - max t)) over the last dim, t = x (+ mask)."""
    x = _as_dview(x)
    m = None if mask is None else _as_dview(mask)
    if out is None:
        out = _new_out(x, x.shape)
    with _device_guard(x):
        check(lib().ctb_log_softmax_lastdim(x.cview(), None if m is None else m.cview(),
                                            _as_dview(out).cview(), _stream_ptr(x)))
    return out


def gather(x, dim: int, index, out=None):
    """Tensor::gather: out[i] = x[i with coordinate ``dim`` replaced by index[i]]; the index may hold
    any integer dtype (src/core/tensor.cpp:352-356 of the reference refuses the floating ones: so does
    this binding; the library itself also takes them, as the first generation's gather does).
    Raises CtbError(CTB_ERR_DIM) with the reference's text when an index is out of bounds."""
    torch = _torch()
    x, idx = _as_dview(x), _as_dview(index)
    if idx.dtype in (F32, F64):
        raise CtbError(3, "Index tensor must be integer type")
    if out is None:
        out = _new_out(x, idx.shape)
    bad = torch.zeros(1, dtype=torch.int32, device=x.buf.device)
    with _device_guard(x):
        check(lib().ctb_gather(x.cview(), dim, idx.cview(), _as_dview(out).cview(), bad.data_ptr(),
                               _stream_ptr(x)))
    if int(bad.item()):
        raise CtbError(4, "Gather index out of bounds")
    return out


def accumulate_grad(grad, src):
    """grad += src with the broadcast dims of src summed first and non-finite values skipped
    (accumulate_grad of the reference's autograd); ``grad`` is updated in place."""
    g, s = _as_dview(grad), _as_dview(src)
    with _device_guard(g):
        check(lib().ctb_accumulate_grad(g.cview(), s.cview(), _stream_ptr(g)))
    return grad


def div_backward(grad, a, b, want_a=True, want_b=True, out_a=None, out_b=None, accumulate=False):
    """ctb_div_backward: (grad / b, -((grad * a) / ((b * b) + 1e-6))) over the broadcast shape; with
    ``accumulate`` the results are added into out_a / out_b (existing gradient buffers)."""
    g, a, b = _as_dview(grad), _as_dview(a), _as_dview(b)
    shape = broadcast_shape(g.shape, broadcast_shape(a.shape, b.shape))
    if want_a and out_a is None:
        out_a = _new_out(g, shape)
    if want_b and out_b is None:
        out_b = _new_out(g, shape)
    with _device_guard(g):
        check(lib().ctb_div_backward(g.cview(), a.cview(), b.cview(), _as_dview(out_a).cview() if want_a else None,
                                     _as_dview(out_b).cview() if want_b else None, int(accumulate), _stream_ptr(g)))
    return out_a, out_b


def tanh_backward(grad, t, out=None, accumulate=False):
    """ctb_tanh_backward: grad * (1 / (cosh t * cosh t))."""
    g, t = _as_dview(grad), _as_dview(t)
    if out is None:
        out = _new_out(g, broadcast_shape(g.shape, t.shape))
    with _device_guard(g):
        check(lib().ctb_tanh_backward(g.cview(), t.cview(), _as_dview(out).cview(), int(accumulate), _stream_ptr(g)))
    return out


def cross_entropy(logits, labels, mean=True, out=None, bad=None):
    """ctb_cross_entropy: mean | sum over the rows of -(log_softmax(logits)[row, label])."""
    x, lab = _as_dview(logits), _as_dview(labels)
    if out is None:
        out = _new_out(x, (1,))
    with _device_guard(x):
        check(lib().ctb_cross_entropy(x.cview(), lab.cview(), int(mean), _as_dview(out).cview(),
                                      None if bad is None else bad.data_ptr(), _stream_ptr(x)))
    return out


def cross_entropy_backward(logits, labels, grad_scale, out=None, accumulate=False, bad=None):
    """ctb_cross_entropy_backward: (softmax(logits) - onehot(labels)) * grad_scale."""
    x, lab = _as_dview(logits), _as_dview(labels)
    if out is None:
        out = _new_out(x, x.shape)
    with _device_guard(x):
        check(lib().ctb_cross_entropy_backward(x.cview(), lab.cview(), float(grad_scale), _as_dview(out).cview(),
                                               int(accumulate), None if bad is None else bad.data_ptr(), _stream_ptr(x)))
    return out


def matmul(a, b, out=None):
    """matmul_mp: 2-d operands, or 3-d with one leading batch dim."""
    av, bv = _as_dview(a), _as_dview(b)
    if out is None:
        batch = max(av.shape[0] if len(av.shape) == 3 else 1, bv.shape[0] if len(bv.shape) == 3 else 1)
        shape = (av.shape[-2], bv.shape[-1]) if len(av.shape) < 3 and len(bv.shape) < 3 else (batch, av.shape[-2], bv.shape[-1])
        out = _new_out(av, shape)
    with _device_guard(av):
        check(lib().ctb_matmul(av.cview(), bv.cview(), _as_dview(out).cview(), _stream_ptr(av)))
    return out


def matmul_tc(a, b, out=None, status=None):
    """ctb_matmul_tc: the product on the tensor cores (TF32 products, fp32 accumulation).  `status`: an
    int32 CUDA tensor of one element that is non-zero afterwards if the kernel gave up a wait."""
    a, b = _as_dview(a), _as_dview(b)
    if out is None:
        out = _new_out(a, tuple(a.shape[:-1]) + (b.shape[-1],))
    with _device_guard(a):
        check(lib().ctb_matmul_tc(a.cview(), b.cview(), _as_dview(out).cview(),
                                  None if status is None else status.data_ptr(), _stream_ptr(a)))
    return out


def channel_moments(x):
    """Per-channel (dim 1) mean and biased variance of a contiguous x[N, C, ...]: (mean, var)."""
    xv = _as_dview(x)
    c = xv.shape[1] if len(xv.shape) > 1 else 0
    mean, var = _new_out(xv, (c,)), _new_out(xv, (c,))
    with _device_guard(xv):
        check(lib().ctb_channel_moments(xv.cview(), DView.of(mean).cview(), DView.of(var).cview(), _stream_ptr(xv)))
    return mean, var


def batchnorm_apply(x, mean, var, gamma=None, beta=None, eps: float = 1e-5, out=None):
    """((x - mean[c]) * (var[c] + eps)^-0.5) * gamma[c] + beta[c] for a contiguous x[N, C, ...]."""
    xv = _as_dview(x)
    opt = lambda t: None if t is None else _as_dview(t).cview()
    if out is None:
        out = _new_out(xv, xv.shape)
    with _device_guard(xv):
        check(lib().ctb_batchnorm_apply(xv.cview(), _as_dview(mean).cview(), _as_dview(var).cview(),
                                        opt(gamma), opt(beta), float(eps), _as_dview(out).cview(), _stream_ptr(xv)))
    return out


def copy_into(src, dst):
    """dst[...] = src (broadcast allowed); dst may be any strided view."""
    s, d = _as_dview(src), _as_dview(dst)
    with _device_guard(d):
        check(lib().ctb_copy_into(s.cview(), d.cview(), _stream_ptr(d)))
    return dst


def cat(tensors, dim: int = 0, out=None):
    """cat_mp: concatenate along ``dim``."""
    vs = [_as_dview(t) for t in tensors]
    if out is None and vs:
        shape = list(vs[0].shape)
        if 0 <= dim < len(shape):
            shape[dim] = sum(v.shape[dim] if len(v.shape) == len(shape) else 0 for v in vs)
        out = _new_out(vs[0], tuple(shape))
    cviews = [v.cview() for v in vs]
    arr = (ctypes.POINTER(View) * max(1, len(cviews)))(*[ctypes.pointer(c) for c in cviews])
    if not vs:
        check(lib().ctb_cat(arr, 0, dim, None, None))       # raises "cat_mp: empty list"
        return None
    with _device_guard(vs[0]):
        check(lib().ctb_cat(arr, len(cviews), dim, _as_dview(out).cview(), _stream_ptr(vs[0])))
    return out


def sgd_step(param, grad, lr: float):
    """param -= lr * grad in place (SGD::step of the reference)."""
    p, g = _as_dview(param), _as_dview(grad)
    with _device_guard(p):
        check(lib().ctb_sgd_step(p.cview(), g.cview(), float(lr), _stream_ptr(p)))
    return param


def adam_step(param, grad, m, v, lr: float, step: int, beta1: float = 0.9, beta2: float = 0.999,
              eps: float = 1e-8, weight_decay=None):
    """One Adam step in place (AdamW when ``weight_decay`` is given); m, v: fp32 CUDA tensors."""
    p, g = _as_dview(param), _as_dview(grad)
    with _device_guard(p):
        check(lib().ctb_adam_step(p.cview(), g.cview(), m.data_ptr(), v.data_ptr(), float(lr), float(beta1),
                                  float(beta2), float(eps), int(step),
                                  0.0 if weight_decay is None else float(weight_decay),
                                  0 if weight_decay is None else 1, _stream_ptr(p)))
    return param


def optimizer_step(kind: int, param, grad, state1, state2, step: int, lr: float, beta1: float = 0.9,
                   beta2: float = 0.999, eps: float = 1e-8, weight_decay: float = 0.0, alpha: float = 0.99):
    """One in-place step of any of the reference's optimizers (OPT_* codes)."""
    p, g = _as_dview(param), _as_dview(grad)
    h = OptimizerHyper(lr, beta1, beta2, eps, weight_decay, alpha)
    with _device_guard(p):
        check(lib().ctb_optimizer_step(kind, p.cview(), g.cview(), None if state1 is None else state1.data_ptr(),
                                       None if state2 is None else state2.data_ptr(), ctypes.byref(h), int(step),
                                       _stream_ptr(p)))
    return param


def layernorm(x, gamma=None, beta=None, eps: float = 1e-5, out=None):
    x = _as_dview(x)
    g = None if gamma is None else _as_dview(gamma)
    b = None if beta is None else _as_dview(beta)
    if out is None:
        out = _new_out(x, x.shape)
    with _device_guard(x):
        check(lib().ctb_layernorm_lastdim(x.cview(), None if g is None else g.cview(),
                                          None if b is None else b.cview(), float(eps),
                                          _as_dview(out).cview(), _stream_ptr(x)))
    return out


# ---- operators (host memory in, host memory out) --------------------------------------------------------
def binary_host(op: int, a, b, out, device: int = 0):
    a, b, o = _as_dview(a), _as_dview(b), _as_dview(out)
    check(lib().ctb_binary_host(op, a.cview(), b.cview(), o.cview(), device))
    return out


def unary_host(op: int, a, out, scalar: float = 0.0, device: int = 0):
    a, o = _as_dview(a), _as_dview(out)
    check(lib().ctb_unary_host(op, a.cview(), float(scalar), o.cview(), device))
    return out


def reduce_host(op: int, a, dim: int, out, device: int = 0):
    a, o = _as_dview(a), _as_dview(out)
    check(lib().ctb_reduce_host(op, a.cview(), dim, o.cview(), device))
    return out
