"""ctypes bindings of the CPU checkers used by the tests (never by the product).

* ``Oracle``    — oracle/libctb_oracle.so, the plain-C restatement (oracle/ctb_oracle.c).
* ``Reference`` — oracle/_ref/libctensor_ref.so, the real reference compiled by
  oracle/build_ref.sh (present only where that build ran or was carried along).

Both take ``HostView`` operands: a 1-d numpy storage buffer plus (offset, shape, strides in
elements), i.e. the reference's (Storage, offset, shape, strides) quadruple.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from dataclasses import dataclass
from typing import Optional, Sequence

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ORACLE_DIR = os.path.join(ROOT, "oracle")
ORACLE_SO = os.path.join(ORACLE_DIR, "libctb_oracle.so")
REF_SO = os.path.join(ORACLE_DIR, "_ref", "libctensor_ref.so")

MAX_DIMS = 8
F32, I32, F64, U8, U16, U32, U64, I8, I16, I64, BOOL = range(11)       # the reference's DType numbering
NP_DTYPES = {F32: np.float32, I32: np.int32, F64: np.float64, U8: np.uint8, U16: np.uint16, U32: np.uint32,
             U64: np.uint64, I8: np.int8, I16: np.int16, I64: np.int64, BOOL: np.bool_}
DT_OF = {np.dtype(v): k for k, v in NP_DTYPES.items()}

# operator codes (include/ctb200.h)
ADD, SUB, MUL, DIV, LT, LE, GT, GE, EQ, NE, POW = range(11)
(ADD_S, SUB_S, RSUB_S, MUL_S, DIV_S, RDIV_S, POW_S, RPOW_S, LT_S, LE_S, GT_S, GE_S, EQ_S, NE_S,
 ABS, RELU, EXP, LOG, TANH, SIGMOID, SQRT, GELU_TANH,
 SIN, COS, TAN, ASIN, ACOS, ATAN, SINH, COSH, SOFTPLUS) = range(31)
SUM, MEAN, MAX, MIN, VAR, ARGMAX = range(6)
PATH_MP, PATH_AVX2, PATH_AVX512, PATH_DISPATCH = range(4)

BINARY_NAMES = ["add", "sub", "mul", "div", "lt", "le", "gt", "ge", "eq", "ne", "pow"]
UNARY_NAMES = ["add_s", "sub_s", "rsub_s", "mul_s", "div_s", "rdiv_s", "pow_s", "rpow_s",
               "lt_s", "le_s", "gt_s", "ge_s", "eq_s", "ne_s", "abs", "relu", "exp", "log",
               "tanh", "sigmoid", "sqrt", "gelu_tanh", "sin", "cos", "tan", "asin", "acos", "atan",
               "sinh", "cosh", "softplus"]
REDUCE_NAMES = ["sum", "mean", "max", "min", "var", "argmax"]


class CView(ctypes.Structure):
    _fields_ = [("base", ctypes.c_void_p), ("offset", ctypes.c_int64),
                ("dtype", ctypes.c_int32), ("ndim", ctypes.c_int32),
                ("shape", ctypes.c_int64 * MAX_DIMS), ("stride", ctypes.c_int64 * MAX_DIMS)]


@dataclass
class HostView:
    buf: np.ndarray                 # 1-d contiguous storage
    shape: tuple
    strides: tuple                  # elements
    offset: int = 0

    @staticmethod
    def contig(arr: np.ndarray) -> "HostView":
        arr = np.ascontiguousarray(arr)
        shape = tuple(int(s) for s in arr.shape)
        strides, st = [], 1
        for s in reversed(shape):
            strides.append(st)
            st *= s
        return HostView(arr.reshape(-1), shape, tuple(reversed(strides)), 0)

    @property
    def dtype(self) -> int:
        return DT_OF[self.buf.dtype]

    @property
    def ndim(self) -> int:
        return len(self.shape)

    @property
    def numel(self) -> int:
        n = 1
        for s in self.shape:
            n *= s
        return n

    def permute(self, dims: Sequence[int]) -> "HostView":
        return HostView(self.buf, tuple(self.shape[d] for d in dims),
                        tuple(self.strides[d] for d in dims), self.offset)

    def narrow(self, dim: int, start: int, length: int) -> "HostView":
        shape = list(self.shape)
        shape[dim] = length
        return HostView(self.buf, tuple(shape), self.strides, self.offset + start * self.strides[dim])

    def step(self, dim: int, k: int) -> "HostView":
        shape, strides = list(self.shape), list(self.strides)
        shape[dim] = (shape[dim] + k - 1) // k
        strides[dim] *= k
        return HostView(self.buf, tuple(shape), tuple(strides), self.offset)

    def expand(self, shape: Sequence[int]) -> "HostView":
        """Broadcast view (stride 0 on expanded dims), right-aligned."""
        shape = tuple(shape)
        pad = len(shape) - self.ndim
        st = []
        for i, s in enumerate(shape):
            j = i - pad
            if j < 0 or (self.shape[j] == 1 and s != 1):
                st.append(0)
            else:
                st.append(self.strides[j])
        return HostView(self.buf, shape, tuple(st), self.offset)

    def numpy(self) -> np.ndarray:
        """Materialise the logical tensor (numpy strided gather)."""
        es = self.buf.dtype.itemsize
        v = np.lib.stride_tricks.as_strided(self.buf[self.offset:], shape=self.shape,
                                            strides=tuple(s * es for s in self.strides))
        return np.array(v)

    def cview(self, base_ptr: Optional[int] = None) -> CView:
        v = CView()
        v.base = self.buf.ctypes.data if base_ptr is None else base_ptr
        v.offset = self.offset
        v.dtype = self.dtype
        v.ndim = self.ndim
        for i in range(self.ndim):
            v.shape[i] = self.shape[i]
            v.stride[i] = self.strides[i]
        return v


def broadcast_shape(a: Sequence[int], b: Sequence[int]) -> tuple:
    nd = max(len(a), len(b))
    out = []
    for i in range(nd):
        da = 1 if i < nd - len(a) else a[i - (nd - len(a))]
        db = 1 if i < nd - len(b) else b[i - (nd - len(b))]
        if da != db and da != 1 and db != 1:
            raise ValueError("Shape mismatch in binary op")
        out.append(max(da, db))
    return tuple(out)


def matmul_shape(a: Sequence[int], b: Sequence[int]) -> tuple:
    """Result shape of matmul_mp (the left operand's shape with the last extent replaced)."""
    return tuple(a[:-1]) + (b[-1],)


def reduced_shape(shape: Sequence[int], dim: int) -> tuple:
    if dim == -1:
        return (1,)
    s = tuple(x for i, x in enumerate(shape) if i != dim)
    return s if s else (1,)


def _ptr(v: Optional[HostView]):
    return None if v is None else ctypes.byref(v.cview())


def build_oracle() -> str:
    subprocess.check_call(["make", "-s", "-C", ORACLE_DIR])
    return ORACLE_SO


class Oracle:
    def __init__(self):
        if not os.path.exists(ORACLE_SO) or os.path.getmtime(ORACLE_SO) < os.path.getmtime(
                os.path.join(ORACLE_DIR, "ctb_oracle.c")):
            build_oracle()
        L = self.lib = ctypes.CDLL(ORACLE_SO)
        vp = ctypes.POINTER(CView)
        L.orc_binary.restype = ctypes.c_int64
        L.orc_binary.argtypes = [ctypes.c_int, vp, vp, ctypes.c_void_p]
        L.orc_unary.restype = ctypes.c_int64
        L.orc_unary.argtypes = [ctypes.c_int, vp, ctypes.c_double, ctypes.c_void_p]
        L.orc_reduce.restype = ctypes.c_int64
        L.orc_reduce.argtypes = [ctypes.c_int, vp, ctypes.c_int, ctypes.c_void_p]
        L.orc_contiguous.restype = ctypes.c_int64
        L.orc_contiguous.argtypes = [vp, ctypes.c_void_p]
        L.orc_softmax_lastdim.restype = ctypes.c_int64
        L.orc_softmax_lastdim.argtypes = [vp, vp, ctypes.c_int, ctypes.c_void_p]
        L.orc_layernorm_lastdim.restype = ctypes.c_int64
        L.orc_layernorm_lastdim.argtypes = [vp, vp, vp, ctypes.c_double, ctypes.c_void_p]
        L.orc_log_softmax_lastdim.restype = ctypes.c_int64
        L.orc_log_softmax_lastdim.argtypes = [vp, vp, ctypes.c_void_p]
        L.orc_gather.restype = ctypes.c_int64
        L.orc_gather.argtypes = [vp, ctypes.c_int, vp, ctypes.c_void_p]
        L.orc_accumulate_grad.restype = ctypes.c_int64
        L.orc_accumulate_grad.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_int64), ctypes.c_int, vp]
        L.orc_channel_moments.restype = None
        L.orc_channel_moments.argtypes = [ctypes.c_void_p] + [ctypes.c_int64] * 3 + [ctypes.c_void_p] * 2
        L.orc_batchnorm_apply.restype = None
        L.orc_batchnorm_apply.argtypes = ([ctypes.c_void_p] + [ctypes.c_int64] * 3 + [ctypes.c_void_p] * 4 +
                                          [ctypes.c_double, ctypes.c_void_p])
        L.orc_matmul.restype = ctypes.c_int64
        L.orc_matmul.argtypes = [vp, vp, ctypes.c_void_p]
        L.orc_cat.restype = ctypes.c_int64
        L.orc_cat.argtypes = [ctypes.POINTER(vp), ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
        L.orc_sgd_step.restype = None
        L.orc_sgd_step.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_double]
        L.orc_adam_step.restype = None
        L.orc_adam_step.argtypes = ([ctypes.c_void_p] * 4 + [ctypes.c_int64] + [ctypes.c_double] * 4 +
                                    [ctypes.c_int, ctypes.c_double, ctypes.c_int])
        L.orc_optimizer_step.restype = None
        L.orc_optimizer_step.argtypes = ([ctypes.c_int] + [ctypes.c_void_p] * 4 + [ctypes.c_int64] +
                                         [ctypes.c_double] * 6 + [ctypes.c_int])
        L.orc_cross_entropy_backward.restype = None
        L.orc_cross_entropy_backward.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64,
                                                 ctypes.c_int, ctypes.c_double, ctypes.c_void_p]
        L.orc_unary_sweep_f32.restype = None
        L.orc_unary_sweep_f32.argtypes = [ctypes.c_int, ctypes.c_uint32, ctypes.c_uint32,
                                          ctypes.c_int64, ctypes.c_double, ctypes.c_void_p,
                                          ctypes.c_void_p]

    def binary(self, op, a: HostView, b: HostView) -> np.ndarray:
        shape = broadcast_shape(a.shape, b.shape)
        out = np.empty(shape, NP_DTYPES[a.dtype])
        n = self.lib.orc_binary(op, a.cview(), b.cview(), out.ctypes.data)
        assert n == out.size, "oracle binary failed"
        return out

    def unary(self, op, a: HostView, scalar: float = 0.0) -> np.ndarray:
        out = np.empty(a.shape, NP_DTYPES[a.dtype])
        n = self.lib.orc_unary(op, a.cview(), float(scalar), out.ctypes.data)
        assert n == out.size, "oracle unary failed"
        return out

    def reduce(self, op, a: HostView, dim: int) -> np.ndarray:
        out = np.empty(reduced_shape(a.shape, dim), np.int32 if op == ARGMAX else NP_DTYPES[a.dtype])
        n = self.lib.orc_reduce(op, a.cview(), dim, out.ctypes.data)
        assert n == out.size, "oracle reduce failed"
        return out

    def contiguous(self, a: HostView) -> np.ndarray:
        out = np.empty(a.shape, NP_DTYPES[a.dtype])
        assert self.lib.orc_contiguous(a.cview(), out.ctypes.data) == out.size
        return out

    def softmax(self, x: HostView, mask: Optional[HostView] = None, causal: bool = False) -> np.ndarray:
        shape = x.shape if mask is None else broadcast_shape(x.shape, mask.shape)
        out = np.empty(shape, np.float32)
        n = self.lib.orc_softmax_lastdim(x.cview(), _ptr(mask), int(causal), out.ctypes.data)
        assert n == out.size, "oracle softmax failed"
        return out

    def layernorm(self, x: HostView, gamma: Optional[HostView], beta: Optional[HostView],
                  eps: float = 1e-5) -> np.ndarray:
        out = np.empty(x.shape, np.float32)
        n = self.lib.orc_layernorm_lastdim(x.cview(), _ptr(gamma), _ptr(beta), eps, out.ctypes.data)
        assert n == out.size, "oracle layernorm failed"
        return out

    def log_softmax(self, x: HostView, mask: Optional[HostView] = None) -> np.ndarray:
        shape = x.shape if mask is None else broadcast_shape(x.shape, mask.shape)
        out = np.empty(shape, np.float32)
        n = self.lib.orc_log_softmax_lastdim(x.cview(), _ptr(mask), out.ctypes.data)
        assert n == out.size, "oracle log_softmax failed"
        return out

    def gather(self, x: HostView, dim: int, index: HostView) -> np.ndarray:
        """Raises IndexError where the reference throws "Gather index out of bounds"."""
        out = np.empty(index.shape, NP_DTYPES[x.dtype])
        n = self.lib.orc_gather(x.cview(), dim, index.cview(), out.ctypes.data)
        if n == -2:
            raise IndexError("Gather index out of bounds")
        assert n == out.size, "oracle gather failed"
        return out

    def accumulate_grad(self, grad: np.ndarray, src: HostView) -> np.ndarray:
        """Returns grad + fold(src) (a new contiguous array of grad's shape)."""
        out = np.ascontiguousarray(grad).copy()
        shape = (ctypes.c_int64 * MAX_DIMS)(*out.shape)
        n = self.lib.orc_accumulate_grad(out.ctypes.data, shape, out.ndim, src.cview())
        assert n == out.size, "oracle accumulate_grad failed"
        return out

    def matmul(self, a: HostView, b: HostView) -> np.ndarray:
        out = np.empty(matmul_shape(a.shape, b.shape), NP_DTYPES[a.dtype])
        n = self.lib.orc_matmul(a.cview(), b.cview(), out.ctypes.data)
        assert n == out.size, "oracle matmul failed"
        return out

    @staticmethod
    def _ncs(x: np.ndarray):
        n, c = x.shape[0], x.shape[1]
        return n, c, int(np.prod(x.shape[2:], dtype=np.int64)) if x.ndim > 2 else 1

    def channel_moments(self, x: np.ndarray):
        """x: contiguous fp32 [N, C, ...] -> (mean[C], var[C])."""
        x = np.ascontiguousarray(x, np.float32)
        n, c, s = self._ncs(x)
        mean, var = np.empty(c, np.float32), np.empty(c, np.float32)
        self.lib.orc_channel_moments(x.ctypes.data, n, c, s, mean.ctypes.data, var.ctypes.data)
        return mean, var

    def batchnorm_apply(self, x: np.ndarray, mean, var, gamma=None, beta=None, eps=1e-5) -> np.ndarray:
        x = np.ascontiguousarray(x, np.float32)
        n, c, s = self._ncs(x)
        out = np.empty_like(x)
        ptr = lambda a: None if a is None else np.ascontiguousarray(a, np.float32).ctypes.data
        keep = [np.ascontiguousarray(a, np.float32) for a in (mean, var)]
        g = None if gamma is None else np.ascontiguousarray(gamma, np.float32)
        b = None if beta is None else np.ascontiguousarray(beta, np.float32)
        self.lib.orc_batchnorm_apply(x.ctypes.data, n, c, s, keep[0].ctypes.data, keep[1].ctypes.data,
                                     None if g is None else g.ctypes.data, None if b is None else b.ctypes.data,
                                     eps, out.ctypes.data)
        return out

    def cat(self, views, dim: int) -> np.ndarray:
        shape = list(views[0].shape)
        shape[dim] = sum(v.shape[dim] for v in views)
        out = np.empty(shape, NP_DTYPES[views[0].dtype])
        cv = [v.cview() for v in views]
        arr = (ctypes.POINTER(CView) * len(cv))(*[ctypes.pointer(c) for c in cv])
        n = self.lib.orc_cat(arr, len(cv), dim, out.ctypes.data)
        assert n == out.size, "oracle cat failed"
        return out

    def optimizer_steps(self, kind: int, param: np.ndarray, grad: np.ndarray, steps: int, lr: float,
                        beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.01) -> np.ndarray:
        """`steps` updates with the same gradient; kind 0 SGD, 1 Adam, 2 AdamW.  Returns the parameter."""
        p = np.ascontiguousarray(param).copy()
        g = np.ascontiguousarray(grad)
        if kind == 0:
            for _ in range(steps):
                self.lib.orc_sgd_step(DT_OF[p.dtype], p.ctypes.data, g.ctypes.data, p.size, lr)
            return p
        m = np.zeros(p.size, np.float32)
        v = np.zeros(p.size, np.float32)
        if kind >= 3:
            for t in range(1, steps + 1):
                self.lib.orc_optimizer_step(kind, p.ctypes.data, g.ctypes.data, m.ctypes.data, v.ctypes.data, p.size,
                                            lr, beta1, beta2, eps, weight_decay, beta2, t)
            return p
        for t in range(1, steps + 1):
            self.lib.orc_adam_step(p.ctypes.data, g.ctypes.data, m.ctypes.data, v.ctypes.data, p.size, lr,
                                   beta1, beta2, eps, t, weight_decay, 1 if kind == 2 else 0)
        return p

    # ---- backward bodies and the cross-entropy rows: the reference's operator chains, spelled with
    # ---- the primitives above (each pinned to the reference on its own) ----------------------------
    def div_backward(self, g: HostView, a: HostView, b: HostView):
        """GradDiv::backward, src/core/autograd.cpp:188-202 -> (g / b, -((g * a) / ((b * b) + 1e-6)))."""
        c = HostView.contig
        da = self.binary(DIV, g, b)
        num, den = self.binary(MUL, g, a), self.binary(MUL, b, b)
        den_safe = self.unary(ADD_S, c(den), 1e-6)
        res = self.binary(DIV, c(num), c(den_safe))
        return da, self.unary(MUL_S, c(res), -1.0)

    def tanh_backward(self, g: HostView, t: HostView):
        """GradTanh::backward, src/core/autograd.cpp:434-438: g * (1 / (cosh t * cosh t))."""
        c = HostView.contig
        ch = c(self.unary(COSH, t))
        inv = self.unary(RDIV_S, c(self.binary(MUL, ch, ch)), 1.0)
        return self.binary(MUL, g, c(inv))

    def cross_entropy(self, logits: HostView, labels: HostView, mean: bool = True):
        """Loss::CrossEntropy, src/neuralnet/loss.cpp:90-118: log-softmax chain, gather, * -1, mean | sum."""
        c = HostView.contig
        logp = c(self.log_softmax(logits))
        idx = c(labels.numpy().reshape(-1, 1))
        nll = self.unary(MUL_S, c(self.gather(logp, 1, idx)), -1.0)
        return self.reduce(MEAN if mean else SUM, c(nll.reshape(-1)), -1)

    def cross_entropy_backward(self, logits: HostView, labels: HostView, mean: bool = True, grad_out: float = 1.0):
        x = np.ascontiguousarray(logits.numpy(), np.float32)
        lab = np.ascontiguousarray(labels.numpy().reshape(-1), np.int32)
        out = np.empty_like(x)
        self.lib.orc_cross_entropy_backward(x.ctypes.data, lab.ctypes.data, x.shape[0], x.shape[1], int(mean),
                                            float(grad_out), out.ctypes.data)
        return out

    def sweep(self, op, start: int, step: int, count: int, scalar: float = 0.0):
        xin = np.empty(count, np.float32)
        out = np.empty(count, np.float32)
        self.lib.orc_unary_sweep_f32(op, start, step, count, scalar, xin.ctypes.data, out.ctypes.data)
        return xin, out


class Reference:
    """The real reference (when oracle/_ref/libctensor_ref.so exists and this CPU can run it)."""

    @staticmethod
    def available() -> bool:
        return os.path.exists(REF_SO)

    def __init__(self):
        L = self.lib = ctypes.CDLL(REF_SO)
        vp = ctypes.POINTER(CView)
        i64, vd = ctypes.c_int64, ctypes.c_void_p
        L.ref_last_error.restype = ctypes.c_char_p
        L.ref_cpu_features.restype = ctypes.c_int
        L.ref_max_threads.restype = ctypes.c_int
        L.ref_set_threads.argtypes = [ctypes.c_int]
        L.ref_binary.restype = i64
        L.ref_binary.argtypes = [ctypes.c_int, ctypes.c_int, vp, vp, vd, i64]
        L.ref_unary.restype = i64
        L.ref_unary.argtypes = [ctypes.c_int, ctypes.c_int, vp, ctypes.c_double, vd, i64]
        L.ref_reduce.restype = i64
        L.ref_reduce.argtypes = [ctypes.c_int, ctypes.c_int, vp, ctypes.c_int, vd, i64]
        L.ref_contiguous.restype = i64
        L.ref_contiguous.argtypes = [vp, vd, i64]
        L.ref_softmax_lastdim.restype = i64
        L.ref_softmax_lastdim.argtypes = [ctypes.c_int, vp, vp, vd, i64]
        L.ref_layernorm_lastdim.restype = i64
        L.ref_layernorm_lastdim.argtypes = [vp, vp, vp, ctypes.c_double, vd, i64]
        L.ref_log_softmax_lastdim.restype = i64
        L.ref_log_softmax_lastdim.argtypes = [ctypes.c_int, vp, vp, vd, i64]
        L.ref_gather.restype = i64
        L.ref_gather.argtypes = [vp, ctypes.c_int, vp, vd, i64]
        L.ref_accumulate_grad.restype = i64
        L.ref_accumulate_grad.argtypes = [vp, vd, vp, vd, i64]
        L.ref_channel_moments.restype = i64
        L.ref_channel_moments.argtypes = [vp, vd, vd]
        L.ref_batchnorm_apply.restype = i64
        L.ref_batchnorm_apply.argtypes = [vp, vp, vp, vp, vp, ctypes.c_double, vd, i64]
        L.ref_matmul.restype = i64
        L.ref_matmul.argtypes = [vp, vp, vd, i64]
        L.ref_cat.restype = i64
        L.ref_cat.argtypes = [ctypes.POINTER(vp), ctypes.c_int, ctypes.c_int, vd, i64]
        L.ref_optimizer_steps.restype = i64
        L.ref_optimizer_steps.argtypes = ([ctypes.c_int, vd, vd, i64, ctypes.c_int] + [ctypes.c_double] * 5 + [vd])
        L.ref_div_backward.restype = i64
        L.ref_div_backward.argtypes = [vp, vp, vp, vd, vd, i64]
        L.ref_tanh_backward.restype = i64
        L.ref_tanh_backward.argtypes = [vp, vp, vd, i64]
        L.ref_cross_entropy_backward.restype = i64
        L.ref_cross_entropy_backward.argtypes = [vp, vp, ctypes.c_int, ctypes.c_double, vd, i64]
        L.ref_bench_step.restype = ctypes.c_double
        L.ref_bench_step.argtypes = [ctypes.c_int, vd, vd, i64]
        feats = L.ref_cpu_features()
        self.has_avx2 = bool(feats & 1)
        self.has_avx512 = bool(feats & 2)

    def simd_path(self) -> int:
        """The SIMD back-end this host can execute (AVX-512 preferred, as the dispatcher does)."""
        if self.has_avx512:
            return PATH_AVX512
        if self.has_avx2:
            return PATH_AVX2
        raise RuntimeError("host CPU has neither AVX2 nor AVX-512")

    def _check(self, n, out):
        if n < 0:
            raise RuntimeError(self.lib.ref_last_error().decode())
        assert n == out.size, (n, out.size)
        return out

    def bench_step(self, path, x: np.ndarray, y: np.ndarray) -> float:
        """Seconds for add, mul, exp, relu, gelu-chain on contiguous fp32 arrays (timed in C++)."""
        t = self.lib.ref_bench_step(path, x.ctypes.data, y.ctypes.data, x.size)
        if t < 0:
            raise RuntimeError(self.lib.ref_last_error().decode())
        return t

    def bench_ops(self, path, x: np.ndarray, y: np.ndarray):
        """Seconds for each of add, mul, exp, relu, gelu-chain (timed in C++); None if this build of the
        reference library predates the entry point."""
        if not hasattr(self.lib, "ref_bench_ops"):
            return None
        sec = (ctypes.c_double * 5)()
        self.lib.ref_bench_ops.restype = ctypes.c_int
        self.lib.ref_bench_ops.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p]
        if self.lib.ref_bench_ops(path, x.ctypes.data, y.ctypes.data, x.size, ctypes.addressof(sec)) != 0:
            raise RuntimeError(self.lib.ref_last_error().decode())
        return list(sec)

    def binary(self, op, a, b, path=PATH_MP):
        out = np.empty(broadcast_shape(a.shape, b.shape), NP_DTYPES[a.dtype])
        return self._check(self.lib.ref_binary(path, op, a.cview(), b.cview(), out.ctypes.data, out.nbytes), out)

    def unary(self, op, a, scalar=0.0, path=PATH_MP):
        out = np.empty(a.shape, NP_DTYPES[a.dtype])
        return self._check(self.lib.ref_unary(path, op, a.cview(), float(scalar), out.ctypes.data, out.nbytes), out)

    def reduce(self, op, a, dim, path=PATH_MP):
        out = np.empty(reduced_shape(a.shape, dim), np.int32 if op == ARGMAX else NP_DTYPES[a.dtype])
        return self._check(self.lib.ref_reduce(path, op, a.cview(), dim, out.ctypes.data, out.nbytes), out)

    def contiguous(self, a):
        out = np.empty(a.shape, NP_DTYPES[a.dtype])
        return self._check(self.lib.ref_contiguous(a.cview(), out.ctypes.data, out.nbytes), out)

    def softmax(self, x, mask=None, exp_path=None):
        shape = x.shape if mask is None else broadcast_shape(x.shape, mask.shape)
        out = np.empty(shape, np.float32)
        p = self.simd_path() if exp_path is None else exp_path
        return self._check(self.lib.ref_softmax_lastdim(p, x.cview(), _ptr(mask), out.ctypes.data, out.nbytes), out)

    def log_softmax(self, x, mask=None, exp_path=None):
        shape = x.shape if mask is None else broadcast_shape(x.shape, mask.shape)
        out = np.empty(shape, np.float32)
        p = self.simd_path() if exp_path is None else exp_path
        return self._check(self.lib.ref_log_softmax_lastdim(p, x.cview(), _ptr(mask), out.ctypes.data, out.nbytes), out)

    def gather(self, x, dim, index):
        out = np.empty(index.shape, NP_DTYPES[x.dtype])
        return self._check(self.lib.ref_gather(x.cview(), dim, index.cview(), out.ctypes.data, out.nbytes), out)

    def accumulate_grad(self, grad: np.ndarray, src):
        """grad: contiguous array with the target's shape (the gradient buffer's start value)."""
        g = np.ascontiguousarray(grad)
        out = np.empty_like(g)
        target = HostView.contig(np.zeros(g.shape, g.dtype))
        return self._check(self.lib.ref_accumulate_grad(target.cview(), g.ctypes.data, src.cview(),
                                                        out.ctypes.data, out.nbytes), out)

    def matmul(self, a, b):
        out = np.empty(matmul_shape(a.shape, b.shape), NP_DTYPES[a.dtype])
        return self._check(self.lib.ref_matmul(a.cview(), b.cview(), out.ctypes.data, out.nbytes), out)

    def channel_moments(self, x: np.ndarray):
        hv = HostView.contig(np.ascontiguousarray(x, np.float32))
        c = hv.shape[1]
        mean, var = np.empty(c, np.float32), np.empty(c, np.float32)
        n = self.lib.ref_channel_moments(hv.cview(), mean.ctypes.data, var.ctypes.data)
        if n < 0:
            raise RuntimeError(self.lib.ref_last_error().decode())
        return mean, var

    def batchnorm_apply(self, x, mean, var, gamma=None, beta=None, eps=1e-5):
        hv = HostView.contig(np.ascontiguousarray(x, np.float32))
        hp = [None if a is None else HostView.contig(np.ascontiguousarray(a, np.float32)) for a in (mean, var, gamma, beta)]
        out = np.empty(hv.shape, np.float32)
        return self._check(self.lib.ref_batchnorm_apply(hv.cview(), _ptr(hp[0]), _ptr(hp[1]), _ptr(hp[2]), _ptr(hp[3]),
                                                        eps, out.ctypes.data, out.nbytes), out)

    def cat(self, views, dim):
        shape = list(views[0].shape)
        shape[dim] = sum(v.shape[dim] for v in views)
        out = np.empty(shape, NP_DTYPES[views[0].dtype])
        cv = [v.cview() for v in views]
        arr = (ctypes.POINTER(CView) * len(cv))(*[ctypes.pointer(c) for c in cv])
        return self._check(self.lib.ref_cat(arr, len(cv), dim, out.ctypes.data, out.nbytes), out)

    def optimizer_steps(self, kind, param, grad, steps, lr, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.01):
        p = np.ascontiguousarray(param, np.float32)
        g = np.ascontiguousarray(grad, np.float32)
        out = np.empty_like(p)
        return self._check(self.lib.ref_optimizer_steps(kind, p.ctypes.data, g.ctypes.data, p.size, steps, lr,
                                                        beta1, beta2, eps, weight_decay, out.ctypes.data), out)

    def div_backward(self, g, a, b):
        """The reference's own GradDiv node on same-shape operands -> (grad of a, grad of b)."""
        oa, ob = np.empty(a.shape, NP_DTYPES[a.dtype]), np.empty(b.shape, NP_DTYPES[b.dtype])
        self._check(self.lib.ref_div_backward(g.cview(), a.cview(), b.cview(), oa.ctypes.data, ob.ctypes.data, ob.nbytes), ob)
        return oa, ob

    def tanh_backward(self, g, t):
        out = np.empty(t.shape, NP_DTYPES[t.dtype])
        return self._check(self.lib.ref_tanh_backward(g.cview(), t.cview(), out.ctypes.data, out.nbytes), out)

    def cross_entropy(self, logits, labels, mean=True):
        """Loss::CrossEntropy's chain through the reference's own functions (its dispatcher throws
        for the dim-wise max/sum on AVX-512 hosts, so the back-end functions are called directly)."""
        c = HostView.contig
        logp = c(self.log_softmax(logits))
        nll = self.unary(MUL_S, c(self.gather(logp, 1, c(labels.numpy().reshape(-1, 1)))), -1.0)
        flat = c(nll.reshape(-1))
        total = self.reduce(SUM, flat, 0)
        return self.unary(MUL_S, c(total), 1.0 / flat.numel) if mean else total

    def cross_entropy_backward(self, logits, labels, mean=True, grad_out=1.0):
        """The reference's own GradCrossEntropy node."""
        out = np.empty(logits.shape, np.float32)
        lab = HostView.contig(np.ascontiguousarray(labels.numpy().reshape(-1, 1), np.int32))
        return self._check(self.lib.ref_cross_entropy_backward(logits.cview(), lab.cview(), int(mean), float(grad_out),
                                                               out.ctypes.data, out.nbytes), out)

    def layernorm(self, x, gamma, beta, eps=1e-5):
        out = np.empty(x.shape, np.float32)
        return self._check(self.lib.ref_layernorm_lastdim(x.cview(), _ptr(gamma), _ptr(beta), eps,
                                                          out.ctypes.data, out.nbytes), out)
