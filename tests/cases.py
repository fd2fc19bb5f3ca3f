"""The catalogue of small parity cases shared by the golden-vector generator, the oracle tests
and the GPU tests.  Every case is a dict:

    name, kind ('binary'|'unary'|'reduce'|'copy'|'softmax'|'layernorm'|'log_softmax'|'gather'|
    'accgrad'|'optim'|'cat'|'bn_moments'|'bn_apply'|'matmul'|'div_bwd'|'tanh_bwd'|'ce'|'ce_bwd'), op, views (HostViews),
    scalar, dim, causal, exact (bit-exact vs tolerance), path (reference back-end that defines it)

Inputs are seeded; the golden file stores them anyway so it does not depend on numpy's RNG.
"""
from __future__ import annotations

import hashlib

import numpy as np

import oracle_lib as ol
from oracle_lib import HostView

SPECIAL_F32 = np.array(
    [0.0, -0.0, 1.0, -1.0, 0.5, 0.75, 1.5, 3.0, 2.0, 10.0, -10.0, 88.0, 88.5, -88.0, -88.5, 100.0,
     -100.0, 1e-40, -1e-40, 1.17549435e-38, 3.4e38, -3.4e38, np.inf, -np.inf, np.nan, 1e-7, -1e-7,
     0.70710677, 0.707106, 0.70710683, 1e10, -1e10, 1e-20, 44.0, -44.5, 0.34657359, 6.0e-8,
     16777216.0, 0.1, -0.1, 7.0, -7.0, 1e18, -1e18, -1.5e18], dtype=np.float32)


def _rng(seed):
    return np.random.default_rng(seed)


def _u(seed, shape, lo=-1.0, hi=1.0):
    return _rng(seed).uniform(lo, hi, shape).astype(np.float32)


def _n(seed, shape, scale=1.0):
    return (_rng(seed).standard_normal(shape) * scale).astype(np.float32)


def _simd_path(op):
    """Reference back-end that defines each fp32 unary flavour."""
    if op == ol.LOG:
        return ol.PATH_AVX2
    if op in (ol.EXP, ol.TANH, ol.SIGMOID, ol.GELU_TANH):
        return ol.PATH_AVX512
    return ol.PATH_MP


def all_cases():
    cases = []

    def add(**kw):
        kw.setdefault("scalar", 0.0)
        kw.setdefault("dim", 0)
        kw.setdefault("causal", False)
        kw.setdefault("exact", True)
        kw.setdefault("path", ol.PATH_MP)
        cases.append(kw)

    # ---- binary, fp32 -------------------------------------------------------------------------
    A = HostView.contig(_u(0, (64, 48)))
    B = HostView.contig(_u(1, (1, 48)))
    C = HostView.contig(_u(2, (64, 1)))
    S1 = HostView.contig(_u(3, (1,)))
    V = HostView.contig(_u(4, (48,)))
    buf4 = HostView.contig(_n(5, (2, 5, 3, 16)))
    P4 = buf4.permute([0, 2, 1, 3])                    # scaled version of the permuted 4-d view
    M4 = HostView.contig(_u(6, (1, 3, 1, 16), -1.0, 0.0))
    T = A.permute([1, 0])                               # transposed: inner stride != 1
    big = HostView.contig(_n(7, (3, 2051)))             # ragged length (not a multiple of 4)
    off = HostView(_n(8, (5000,)), (37, 101), (101, 1), 3)      # odd offset -> misaligned base
    stepped = HostView(_n(9, (64 * 70,)), (64, 35), (70, 2), 0)  # inner stride 2
    for op in range(10):
        nm = ol.BINARY_NAMES[op]
        add(name=f"bin_{nm}_rowbcast", kind="binary", op=op, views=[A, B])
        add(name=f"bin_{nm}_colbcast", kind="binary", op=op, views=[A, C])
        add(name=f"bin_{nm}_same", kind="binary", op=op, views=[A, A.narrow(0, 0, 64)])
    for op in (ol.ADD, ol.SUB, ol.MUL, ol.DIV):
        nm = ol.BINARY_NAMES[op]
        add(name=f"bin_{nm}_bcast_a", kind="binary", op=op, views=[B, A])
        add(name=f"bin_{nm}_scalar_b", kind="binary", op=op, views=[A, S1])
        add(name=f"bin_{nm}_scalar_a", kind="binary", op=op, views=[S1, A])
        add(name=f"bin_{nm}_vec", kind="binary", op=op, views=[A, V])
        add(name=f"bin_{nm}_perm4d", kind="binary", op=op, views=[P4, M4])
        add(name=f"bin_{nm}_transposed", kind="binary", op=op, views=[T, HostView.contig(_u(10, (48, 64)))])
        add(name=f"bin_{nm}_outer", kind="binary", op=op, views=[C, B])        # [64,1] o [1,48]
        add(name=f"bin_{nm}_ragged", kind="binary", op=op, views=[big, big.narrow(0, 1, 1)])
        add(name=f"bin_{nm}_offset", kind="binary", op=op, views=[off, off])
        add(name=f"bin_{nm}_stepped", kind="binary", op=op, views=[stepped, stepped])
        sp = HostView.contig(SPECIAL_F32)
        add(name=f"bin_{nm}_special", kind="binary", op=op,
            views=[HostView.contig(np.repeat(SPECIAL_F32, SPECIAL_F32.size).reshape(SPECIAL_F32.size, -1)), sp])
    pw_e = HostView.contig(_u(28, (1, 53), -2.0, 3.0))
    add(name="bin_pow_rowbcast", kind="binary", op=ol.POW, views=[HostView.contig(np.abs(_n(17, (37, 53), 3.0)) + np.float32(1e-3)), pw_e],
        exact=False)
    # both operands single elements (the dispatcher's scalar short-circuit computes the same value)
    add(name="bin_add_1x1", kind="binary", op=ol.ADD, views=[S1, HostView.contig(_u(11, (1, 1)))])

    # ---- binary, int32 and fp64 ------------------------------------------------------------------
    Ai = HostView.contig(_rng(12).integers(-100, 100, (7, 9)).astype(np.int32))
    Bi = HostView.contig(_rng(13).integers(1, 9, (9,)).astype(np.int32))
    edge_a = HostView.contig(np.array([2000000000, -2000000000, 7, -7, 0, 5], np.int32))
    edge_b = HostView.contig(np.array([2000000000, 2000000000, 2, 2, 0, 0], np.int32))
    Ad = HostView.contig(_rng(14).standard_normal((5, 6)))
    Bd = HostView.contig(_rng(15).standard_normal((6,)))
    for op in range(10):
        nm = ol.BINARY_NAMES[op]
        add(name=f"bin_{nm}_i32", kind="binary", op=op, views=[Ai, Bi])
        add(name=f"bin_{nm}_i32_edge", kind="binary", op=op, views=[edge_a, edge_b])
        add(name=f"bin_{nm}_f64", kind="binary", op=op, views=[Ad, Bd])

    # ---- unary ---------------------------------------------------------------------------------------
    X = HostView.contig(_n(16, (37, 53), 3.0))
    Xp = HostView.contig(np.abs(_n(17, (37, 53), 3.0)) + np.float32(1e-3))
    sp = HostView.contig(SPECIAL_F32)
    U1 = HostView.contig(_u(27, (37, 53)))            # |x| <= 1 for asin/acos
    for op in range(31):
        nm = ol.UNARY_NAMES[op]
        path = _simd_path(op)
        # libm functions evaluated in double (pow, trig, hyperbolic, softplus): tolerance only
        exact = op not in (ol.POW_S, ol.RPOW_S) and op < ol.SIN
        for s in ((0.5, -3.0, 2.0) if op < ol.ABS else (0.0,)):
            tag = f"{nm}_{s}" if op < ol.ABS else nm
            src = Xp if op in (ol.POW_S, ol.RPOW_S, ol.LOG, ol.SQRT) else (U1 if op in (ol.ASIN, ol.ACOS) else X)
            if op == ol.RPOW_S and s < 0:
                continue
            add(name=f"un_{tag}", kind="unary", op=op, views=[src], scalar=s, exact=exact, path=path)
            if exact:
                add(name=f"un_{tag}_special", kind="unary", op=op, views=[sp], scalar=s, path=path)
        if path == ol.PATH_MP and op >= ol.ABS or op in (ol.MUL_S, ol.ADD_S):
            # strided inputs (the SIMD unary back-ends of the reference are stride-blind)
            add(name=f"un_{nm}_perm4d", kind="unary", op=op, views=[P4], scalar=1.5, path=ol.PATH_MP)
            add(name=f"un_{nm}_transposed", kind="unary", op=op, views=[T], scalar=1.5, path=ol.PATH_MP)
    for op in (ol.ADD_S, ol.MUL_S, ol.DIV_S, ol.RSUB_S, ol.GT_S, ol.ABS, ol.RELU, ol.SQRT):
        nm = ol.UNARY_NAMES[op]
        add(name=f"un_{nm}_i32", kind="unary", op=op, views=[Ai], scalar=2.5)
        add(name=f"un_{nm}_f64", kind="unary", op=op, views=[Ad], scalar=2.5)
    add(name="un_mul_s_i32_overflow", kind="unary", op=ol.MUL_S, views=[edge_a], scalar=3.0)

    # ---- the other integer types and Bool: served by the reference's scalar back-end through double
    # (read_scalar_at / write_scalar_at); results stored with x86's static_cast.  Values stay inside
    # the types' ranges except in the *_wrap cases (the low bits of the truncated 32-bit integer).
    narrow = {
        "u8": (np.uint8, _rng(101).integers(0, 200, (6, 11)), _rng(102).integers(1, 12, (11,))),
        "i8": (np.int8, _rng(103).integers(-60, 60, (6, 11)), _rng(104).integers(1, 9, (11,))),
        "i16": (np.int16, _rng(105).integers(-3000, 3000, (6, 11)), _rng(106).integers(1, 90, (11,))),
        "i64": (np.int64, _rng(107).integers(-10**12, 10**12, (6, 11)), _rng(108).integers(1, 10**6, (11,))),
        "bool": (np.bool_, _rng(109).integers(0, 2, (6, 11)), _rng(110).integers(0, 2, (11,))),
    }
    for tn, (npdt, av, bv) in narrow.items():
        An, Bn = HostView.contig(av.astype(npdt)), HostView.contig(bv.astype(npdt))
        bin_ops = (ol.ADD, ol.SUB, ol.MUL, ol.LT, ol.LE, ol.GT, ol.GE, ol.EQ, ol.NE) + (() if tn == "bool" else (ol.DIV,))
        for op in bin_ops:
            if tn in ("u8", "i8") and op == ol.MUL:
                continue                                    # products leave the range: see *_wrap below
            add(name=f"bin_{ol.BINARY_NAMES[op]}_{tn}", kind="binary", op=op, views=[An, Bn])
        for op in (ol.ADD_S, ol.MUL_S, ol.DIV_S, ol.RSUB_S, ol.GT_S, ol.ABS, ol.RELU):
            if tn == "bool" and op not in (ol.GT_S, ol.ABS, ol.RELU):
                continue
            add(name=f"un_{ol.UNARY_NAMES[op]}_{tn}", kind="unary", op=op, views=[An], scalar=0.5 if op == ol.MUL_S else 2.0)
        add(name=f"un_add_s_{tn}_transposed", kind="unary", op=ol.ADD_S, views=[An.permute([1, 0])], scalar=1.0)
        add(name=f"copy_{tn}_transposed", kind="copy", op=0, views=[An.permute([1, 0])])
        for op in (ol.SUM, ol.MEAN, ol.MAX, ol.MIN, ol.ARGMAX):
            if tn in ("u8", "i8") and op == ol.SUM:
                continue
            for dim in (0, 1) + (() if op == ol.ARGMAX else (-1,)):
                if tn in ("u8", "i8", "bool") and op in (ol.SUM, ol.MEAN) and dim == -1:
                    continue
                add(name=f"red_{ol.REDUCE_NAMES[op]}_{tn}_d{dim}", kind="reduce", op=op, views=[An], dim=dim)
    wrap_a = HostView.contig(np.array([200, 100, 255, 7, 0, 128], np.uint8))
    wrap_b = HostView.contig(np.array([100, 100, 255, 40, 0, 2], np.uint8))
    for op in (ol.ADD, ol.MUL, ol.SUB):
        add(name=f"bin_{ol.BINARY_NAMES[op]}_u8_wrap", kind="binary", op=op, views=[wrap_a, wrap_b])
    add(name="red_sum_u8_wrap_d0", kind="reduce", op=ol.SUM, dim=0, views=[HostView.contig(np.full((9, 4), 100, np.uint8))])
    add(name="un_mul_s_i64_out_of_range", kind="unary", op=ol.MUL_S, scalar=1e10,
        views=[HostView.contig(np.array([10**12, -10**12, 5, 0], np.int64))])
    for tn, npdt in (("u16", np.uint16), ("u32", np.uint32), ("u64", np.uint64)):      # copied, never computed
        add(name=f"copy_{tn}_transposed", kind="copy", op=0,
            views=[HostView.contig(_rng(111).integers(0, 60000, (5, 7)).astype(npdt)).permute([1, 0])])

    # ---- strided copy -----------------------------------------------------------------------------------
    for nm, v in (("perm4d", P4), ("transposed", T), ("offset", off), ("stepped", stepped),
                  ("i32", HostView.contig(Ai.numpy()).permute([1, 0])), ("f64", Ad.permute([1, 0])),
                  ("narrow", A.narrow(1, 5, 17))):
        add(name=f"copy_{nm}", kind="copy", op=0, views=[v])

    # ---- reductions ---------------------------------------------------------------------------------------
    R = HostView.contig(_n(18, (33, 70)))
    R3 = HostView.contig(_n(19, (6, 20, 36)))
    Rlong = HostView.contig(_n(20, (3, 5000)))
    Rtall = HostView.contig(_n(21, (700, 36)))
    nan_rows = HostView.contig(np.array(
        [[1, np.nan, 3, 2], [np.nan, 1, 3, 2], [np.nan] * 4, [-np.inf, -2e18, -1e18, -3e18],
         [5, 7, 7, 1], [-1.0, -1.0, -2.0, -1.0]], np.float32))
    for op in range(6):
        nm = ol.REDUCE_NAMES[op]
        exact = op in (ol.MAX, ol.MIN, ol.ARGMAX)
        for vn, v in (("2d", R), ("3d", R3), ("long", Rlong), ("tall", Rtall), ("perm4d", P4),
                      ("transposed", R.permute([1, 0])), ("stepped", stepped), ("i32", Ai), ("f64", Ad)):
            dims = list(range(v.ndim)) + ([] if op == ol.ARGMAX else [-1])
            if op == ol.VAR and v.dtype == ol.I32:
                continue                      # var is a float-only composite
            for dim in dims:
                add(name=f"red_{nm}_{vn}_d{dim}", kind="reduce", op=op, views=[v], dim=dim,
                    exact=exact or v.dtype == ol.I32)
        if op in (ol.MAX, ol.MIN, ol.ARGMAX):
            add(name=f"red_{nm}_nan_rows", kind="reduce", op=op, views=[nan_rows], dim=1)
    # zeros of both signs as the extreme value: the reference keeps the FIRST zero of a line in
    # index order (std::max/min never replace an equal value), so the sign of a zero result depends
    # on positions.  One input per kernel shape: short lines, long lines, column splits, very long
    # lines (the split kernel), strided / other dtypes (the generic kernels).
    def zeros_mix(seed, shape, sign):
        pick = np.array([-0.0, 0.0, -1.5, -3.0], np.float32) * np.float32(sign)
        return pick[_rng(seed).integers(0, 4, shape)]
    for op, sign in ((ol.MAX, 1.0), (ol.MIN, -1.0)):
        nm = ol.REDUCE_NAMES[op]
        z2 = HostView.contig(zeros_mix(71, (33, 70), sign))
        zlong = HostView.contig(zeros_mix(72, (3, 5000), sign))
        ztall = HostView.contig(zeros_mix(73, (700, 36), sign))
        zsplit = HostView.contig(zeros_mix(74, (2, 70000), sign))
        zd = HostView.contig(zeros_mix(75, (9, 40), sign).astype(np.float64))
        for vn, v, dims in (("2d", z2, (0, 1, -1)), ("long", zlong, (0, 1, -1)), ("tall", ztall, (0, 1, -1)),
                            ("split", zsplit, (1, -1)), ("transposed", z2.permute([1, 0]), (0, 1, -1)),
                            ("f64", zd, (0, 1, -1))):
            for dim in dims:
                add(name=f"red_{nm}_zeros_{vn}_d{dim}", kind="reduce", op=op, views=[v], dim=dim)
        # relu output (+0 where the input was negative) joined with raw -0 inputs
        add(name=f"red_{nm}_zeros_first_wins", kind="reduce", op=op, dim=1, views=[HostView.contig(np.array(
            [[-0.0, 0.0, 0.0], [0.0, -0.0, -0.0], [-1.0 * sign, -0.0, 0.0], [0.0, -2.0 * sign, -0.0]], np.float32))])
    one = HostView.contig(np.array([4.25], np.float32))
    for op in (ol.SUM, ol.MEAN, ol.MAX, ol.MIN, ol.VAR):
        add(name=f"red_{ol.REDUCE_NAMES[op]}_single", kind="reduce", op=op, views=[one], dim=0, exact=True)

    # ---- fused rows ---------------------------------------------------------------------------------------
    add(name="softmax_2d", kind="softmax", op=0, views=[R], exact=False, path=ol.PATH_AVX512)
    add(name="softmax_perm4d_mask", kind="softmax", op=0, views=[P4, M4], exact=False, path=ol.PATH_AVX512)
    add(name="softmax_long", kind="softmax", op=0, views=[Rlong], exact=False, path=ol.PATH_AVX512)
    sq = HostView.contig(_n(22, (2, 3, 24, 24)))
    cm = np.where(np.arange(24)[None, :] > np.arange(24)[:, None], np.float32(-1e9), np.float32(0)).astype(np.float32)
    add(name="softmax_causal_as_mask", kind="softmax", op=0, views=[sq, HostView.contig(cm.reshape(1, 1, 24, 24))],
        exact=False, path=ol.PATH_AVX512)
    g = HostView.contig((_n(23, (70,), 0.02) + 1).astype(np.float32))
    b = HostView.contig(_n(24, (70,), 0.02))
    add(name="layernorm_2d", kind="layernorm", op=0, views=[R, g, b], scalar=1e-5, exact=False)
    g36 = HostView.contig((_n(25, (36,), 0.02) + 1).astype(np.float32))
    b36 = HostView.contig(_n(26, (36,), 0.02))
    add(name="layernorm_3d", kind="layernorm", op=0, views=[R3, g36, b36], scalar=1e-5, exact=False)

    # ---- callers either side of the path: log-softmax rows, gather, accumulate_grad ------------------------
    logits = HostView.contig(_n(29, (33, 10), 3.0))           # [batch, classes] of Loss::CrossEntropy
    add(name="logsoftmax_2d", kind="log_softmax", op=0, views=[logits], exact=False, path=ol.PATH_AVX512)
    add(name="logsoftmax_wide", kind="log_softmax", op=0, views=[R], exact=False, path=ol.PATH_AVX512)
    add(name="logsoftmax_long", kind="log_softmax", op=0, views=[Rlong], exact=False, path=ol.PATH_AVX512)
    add(name="logsoftmax_perm4d_mask", kind="log_softmax", op=0, views=[P4, M4], exact=False, path=ol.PATH_AVX512)
    tgt = HostView.contig(_rng(30).integers(0, 10, (33, 1)).astype(np.int32))
    add(name="gather_targets", kind="gather", op=0, views=[logits, tgt], dim=1)
    idx0 = HostView.contig(_rng(31).integers(-33, 33, (5, 10)).astype(np.int32))     # negative = from the end
    add(name="gather_dim0_negative", kind="gather", op=0, views=[logits, idx0], dim=0)
    idx3 = HostView.contig(_rng(32).integers(0, 20, (6, 7, 36)).astype(np.int32))
    add(name="gather_3d_dim1", kind="gather", op=0, views=[R3, idx3], dim=1)
    idxp = HostView.contig(_rng(33).integers(0, 3, (2, 2, 5, 16)).astype(np.int32))
    add(name="gather_perm4d", kind="gather", op=0, views=[P4, idxp], dim=1)
    add(name="gather_i32", kind="gather", op=0, views=[Ai, HostView.contig(_rng(34).integers(0, 9, (7, 4)).astype(np.int32))], dim=1)
    add(name="gather_f64", kind="gather", op=0, views=[Ad, HostView.contig(_rng(35).integers(0, 5, (3, 6)).astype(np.int32))], dim=0)
    # accumulate_grad: views = [start value of the gradient buffer (target's shape), incoming gradient]
    gsrc = HostView.contig(_n(36, (64, 48)))
    add(name="accgrad_same", kind="accgrad", op=0, views=[HostView.contig(_n(37, (64, 48))), gsrc])
    add(name="accgrad_bias_row", kind="accgrad", op=0, views=[HostView.contig(_n(38, (1, 48))), gsrc], exact=False)
    add(name="accgrad_bias_vec", kind="accgrad", op=0, views=[HostView.contig(_n(39, (48,))), gsrc], exact=False)
    add(name="accgrad_col", kind="accgrad", op=0, views=[HostView.contig(_n(40, (64, 1))), gsrc], exact=False)
    add(name="accgrad_tall", kind="accgrad", op=0, views=[HostView.contig(_n(41, (36,))), Rtall], exact=False)
    add(name="accgrad_transposed_src", kind="accgrad", op=0, views=[HostView.contig(_n(42, (48, 64))), gsrc.permute([1, 0])])
    add(name="accgrad_src_broadcasts", kind="accgrad", op=0, views=[HostView.contig(_n(43, (64, 48))), B])
    nf = _n(44, (64, 48)).copy()
    nf[3, 5] = np.nan
    nf[7, 0] = np.inf
    nf[9, 47] = -np.inf
    add(name="accgrad_skips_nonfinite", kind="accgrad", op=0, views=[HostView.contig(_n(45, (64, 48))), HostView.contig(nf)])
    add(name="accgrad_bias_nonfinite", kind="accgrad", op=0, views=[HostView.contig(_n(46, (48,))), HostView.contig(nf)], exact=False)
    add(name="accgrad_i32", kind="accgrad", op=0, views=[HostView.contig(_rng(47).integers(-9, 9, (9,)).astype(np.int32)), Ai])
    add(name="accgrad_f64", kind="accgrad", op=0, views=[HostView.contig(_rng(48).standard_normal((6,))), Ad], exact=False)

    # ---- backward bodies: views = [incoming gradient, forward operands...]; op 0 -> grad of a, 1 -> grad of b.
    # Same-shape operands are pinned by the reference's own GradDiv / GradTanh nodes; the broadcast cases by
    # the same operator chain spelled with the reference's back-end functions.
    bg = HostView.contig(_n(76, (37, 53)))
    ba = HostView.contig(_n(77, (37, 53), 2.0))
    bb = HostView.contig(np.where(np.abs(_n(78, (37, 53))) < 0.05, np.float32(0.05), _n(78, (37, 53))).astype(np.float32))
    brow = HostView.contig(_u(79, (1, 53), 0.5, 2.0))
    bcol = HostView.contig(_u(80, (37, 1), -2.0, -0.5))
    for which in (0, 1):
        nm = "ab"[which]
        add(name=f"divbwd_{nm}_same", kind="div_bwd", op=which, views=[bg, ba, bb], exact=True)
        add(name=f"divbwd_{nm}_row_b", kind="div_bwd", op=which, views=[bg, ba, brow], exact=True)
        add(name=f"divbwd_{nm}_col_a", kind="div_bwd", op=which, views=[bg, bcol, bb], exact=True)
        add(name=f"divbwd_{nm}_transposed", kind="div_bwd", op=which,
            views=[HostView.contig(_n(81, (53, 37))).permute([1, 0]), ba, bb], exact=True)
        add(name=f"divbwd_{nm}_special", kind="div_bwd", op=which,
            views=[HostView.contig(np.repeat(SPECIAL_F32, SPECIAL_F32.size).reshape(SPECIAL_F32.size, -1)),
                   HostView.contig(SPECIAL_F32[::-1].copy()), HostView.contig(SPECIAL_F32)], exact=True)
        add(name=f"divbwd_{nm}_f64", kind="div_bwd", op=which,
            views=[HostView.contig(_rng(82).standard_normal((5, 6))), Ad, HostView.contig(_rng(83).standard_normal((6,)) + 3.0)], exact=True)
    add(name="tanhbwd_same", kind="tanh_bwd", op=0, views=[bg, ba], exact=False)
    add(name="tanhbwd_row", kind="tanh_bwd", op=0, views=[bg, brow], exact=False)
    add(name="tanhbwd_large_arguments", kind="tanh_bwd", op=0,
        views=[HostView.contig(np.ones(12, np.float32)), HostView.contig(np.array([0, 1e-3, 0.5, -0.5, 5, -5, 20, -20, 44, 60, 89, -100], np.float32))], exact=False)
    # ---- cross-entropy rows: views = [logits [B,C], labels int32 [B,1]]; op 1 = mean, 0 = sum --------------------
    ce_logits = HostView.contig(_n(84, (33, 10), 3.0))
    ce_labels = HostView.contig(_rng(85).integers(0, 10, (33, 1)).astype(np.int32))
    wide_logits = HostView.contig(_n(86, (7, 3000), 2.0))
    wide_labels = HostView.contig(_rng(87).integers(0, 3000, (7, 1)).astype(np.int32))
    for red, rn in ((1, "mean"), (0, "sum")):
        add(name=f"ce_{rn}", kind="ce", op=red, views=[ce_logits, ce_labels], exact=False, path=ol.PATH_AVX512)
        add(name=f"ce_{rn}_wide", kind="ce", op=red, views=[wide_logits, wide_labels], exact=False, path=ol.PATH_AVX512)
        add(name=f"cebwd_{rn}", kind="ce_bwd", op=red, views=[ce_logits, ce_labels], scalar=1.0, exact=False)
        add(name=f"cebwd_{rn}_wide", kind="ce_bwd", op=red, views=[wide_logits, wide_labels], scalar=0.37, exact=False)
    add(name="ce_mean_row_slice", kind="ce", op=1, views=[HostView.contig(_n(88, (33, 16))).narrow(1, 3, 10), ce_labels], exact=False,
        path=ol.PATH_AVX512)

    # ---- cat: views = the inputs, dim = the cat dim ------------------------------------------------------------
    add(name="cat_dim0", kind="cat", op=0, views=[A, A.narrow(0, 3, 11), B], dim=0)
    add(name="cat_dim1", kind="cat", op=0, views=[A, C, A.narrow(1, 1, 5)], dim=1)
    add(name="cat_transposed", kind="cat", op=0, views=[T, HostView.contig(_u(51, (48, 3)))], dim=1)
    add(name="cat_perm4d_dim2", kind="cat", op=0, views=[P4, P4.narrow(2, 1, 2)], dim=2)
    add(name="cat_i32", kind="cat", op=0, views=[Ai, Ai], dim=1)
    add(name="cat_f64_single", kind="cat", op=0, views=[Ad.permute([1, 0])], dim=0)
    add(name="cat_ragged_offset", kind="cat", op=0, views=[off, off.narrow(1, 2, 1), off.step(1, 3)], dim=1)

    # ---- matmul_mp (left operand carries the batch dim, as the reference's result shape does) ----------------------
    ma = HostView.contig(_n(59, (70, 45)))
    mb = HostView.contig(_n(60, (45, 33)))
    add(name="matmul_2d", kind="matmul", op=0, views=[ma, mb])
    add(name="matmul_2d_transposed_b", kind="matmul", op=0, views=[ma, HostView.contig(_n(61, (33, 45))).permute([1, 0])])
    add(name="matmul_2d_transposed_a", kind="matmul", op=0, views=[HostView.contig(_n(62, (45, 70))).permute([1, 0]), mb])
    add(name="matmul_3d", kind="matmul", op=0, views=[HostView.contig(_n(63, (5, 17, 130))), HostView.contig(_n(64, (5, 130, 9)))])
    add(name="matmul_3d_shared_b", kind="matmul", op=0, views=[HostView.contig(_n(65, (4, 64, 64))), HostView.contig(_n(66, (64, 64)))])
    add(name="matmul_long_k", kind="matmul", op=0, views=[HostView.contig(_n(67, (3, 1000))), HostView.contig(_n(68, (1000, 2)))])
    add(name="matmul_special", kind="matmul", op=0,
        views=[HostView.contig(SPECIAL_F32[:40].reshape(5, 8)), HostView.contig(SPECIAL_F32[5:45].reshape(8, 5))])
    add(name="matmul_i32", kind="matmul", op=0, views=[Ai, HostView.contig(_rng(69).integers(-9, 9, (9, 4)).astype(np.int32))])
    add(name="matmul_f64", kind="matmul", op=0, views=[Ad, HostView.contig(_rng(70).standard_normal((6, 7)))])

    # ---- BatchNorm forward: moments of x[N,C,...] (op 0 -> mean, 1 -> var) and the normalisation ------------------
    bn4 = HostView.contig(_n(52, (6, 5, 7, 8), 2.0) + np.float32(0.75))
    bn3 = HostView.contig(_n(53, (33, 12, 20)))
    bn2 = HostView.contig(_n(54, (257, 36), 3.0))
    for nm, v in (("4d", bn4), ("3d", bn3), ("2d", bn2)):
        c = v.shape[1]
        add(name=f"bn_mean_{nm}", kind="bn_moments", op=0, views=[v], exact=False)
        add(name=f"bn_var_{nm}", kind="bn_moments", op=1, views=[v], exact=False)
        mu = HostView.contig(_n(55, (c,), 0.3))
        vr = HostView.contig(np.abs(_n(56, (c,))) + np.float32(0.1))
        gm = HostView.contig((_n(57, (c,), 0.02) + 1).astype(np.float32))
        bt = HostView.contig(_n(58, (c,), 0.02))
        add(name=f"bn_apply_{nm}", kind="bn_apply", op=0, views=[v, mu, vr, gm, bt], scalar=1e-5)
    add(name="bn_apply_4d_no_affine", kind="bn_apply", op=0,
        views=[bn4, HostView.contig(_n(55, (5,), 0.3)), HostView.contig(np.abs(_n(56, (5,))) + np.float32(0.1))], scalar=1e-3)

    # ---- optimizer steps: views = [parameter, gradient]; op = optimizer (0 SGD ... 8 Lion); dim = number of steps ----
    w0 = HostView.contig(_n(49, (1003,), 0.5))
    gw = HostView.contig(_n(50, (1003,), 2.0))
    gsp = SPECIAL_F32[np.isfinite(SPECIAL_F32)]
    wsp = HostView.contig(np.linspace(-2, 2, gsp.size).astype(np.float32))
    for kind, nm in enumerate(("sgd", "adam", "adamw", "adamax", "nadam", "radam", "rmsprop", "adagrad", "lion")):
        add(name=f"optim_{nm}_1step", kind="optim", op=kind, views=[w0, gw], dim=1, scalar=0.01)
        add(name=f"optim_{nm}_7steps", kind="optim", op=kind, views=[w0, gw], dim=7, scalar=0.003)
        add(name=f"optim_{nm}_special_grads", kind="optim", op=kind, views=[wsp, HostView.contig(gsp)], dim=2, scalar=0.1)
    return cases


def run_case(impl, case):
    """Evaluate a case on an Oracle- or Reference-like object."""
    k, v = case["kind"], case["views"]
    is_ref = isinstance(impl, ol.Reference)
    if k == "binary":
        return impl.binary(case["op"], v[0], v[1], ol.PATH_MP) if is_ref else impl.binary(case["op"], v[0], v[1])
    if k == "unary":
        return (impl.unary(case["op"], v[0], case["scalar"], case["path"]) if is_ref
                else impl.unary(case["op"], v[0], case["scalar"]))
    if k == "copy":
        return impl.contiguous(v[0])
    if k == "reduce":
        return impl.reduce(case["op"], v[0], case["dim"], ol.PATH_MP) if is_ref else impl.reduce(case["op"], v[0], case["dim"])
    if k == "softmax":
        mask = v[1] if len(v) > 1 else None
        return impl.softmax(v[0], mask, case["path"]) if is_ref else impl.softmax(v[0], mask, case["causal"])
    if k == "layernorm":
        return impl.layernorm(v[0], v[1], v[2], case["scalar"])
    if k == "log_softmax":
        mask = v[1] if len(v) > 1 else None
        return impl.log_softmax(v[0], mask, case["path"]) if is_ref else impl.log_softmax(v[0], mask)
    if k == "gather":
        return impl.gather(v[0], case["dim"], v[1])
    if k == "accgrad":
        return impl.accumulate_grad(v[0].numpy(), v[1])
    if k == "matmul":
        return impl.matmul(v[0], v[1])
    if k == "bn_moments":
        return impl.channel_moments(v[0].numpy())[case["op"]]
    if k == "bn_apply":
        p = [t.numpy() for t in v[1:]] + [None] * (5 - len(v))
        return impl.batchnorm_apply(v[0].numpy(), p[0], p[1], p[2], p[3], case["scalar"])
    if k == "cat":
        return impl.cat(v, case["dim"])
    if k == "div_bwd":
        if is_ref:
            if v[0].shape == v[1].shape == v[2].shape and v[0].dtype == ol.F32:     # the reference's own node
                return impl.div_backward(v[0], v[1], v[2])[case["op"]]
            return ol.Oracle.div_backward(impl, v[0], v[1], v[2])[case["op"]]     # its back-end functions, same chain
        return impl.div_backward(v[0], v[1], v[2])[case["op"]]
    if k == "tanh_bwd":
        if is_ref and v[0].shape != v[1].shape:
            return ol.Oracle.tanh_backward(impl, v[0], v[1])
        return impl.tanh_backward(v[0], v[1])
    if k == "ce":
        return impl.cross_entropy(v[0], v[1], bool(case["op"]))
    if k == "ce_bwd":
        return impl.cross_entropy_backward(v[0], v[1], bool(case["op"]), case["scalar"])
    if k == "optim":
        return impl.optimizer_steps(case["op"], v[0].numpy(), v[1].numpy(), case["dim"], case["scalar"])
    raise ValueError(k)


def digest(arr: np.ndarray) -> str:
    """SHA-256 of an output's shape, dtype and bytes, with every NaN mapped to one canonical
    pattern (x86 and the GPU propagate different NaN payloads)."""
    a = np.ascontiguousarray(arr).copy()
    if a.dtype.kind == "f":
        a[np.isnan(a)] = np.nan
    h = hashlib.sha256()
    h.update(str(a.dtype).encode())
    h.update(str(a.shape).encode())
    h.update(a.tobytes())
    return h.hexdigest()


GOLDEN_PATH = __import__("os").path.join(__import__("os").path.dirname(__import__("os").path.abspath(__file__)),
                                         "golden", "golden_cases.npz")


def load_golden():
    """-> dict name -> {'views': [HostView...], 'digest': str | None, 'out': ndarray | None}"""
    z = np.load(GOLDEN_PATH, allow_pickle=False)
    res = {}
    for n in z["__names__"]:
        n = str(n)
        views = []
        i = 0
        while f"{n}/in{i}/meta" in z:
            meta = z[f"{n}/in{i}/meta"]
            nd = int(meta[1])
            buf = z["buf/" + str(z[f"{n}/in{i}/key"])]
            views.append(HostView(buf, tuple(int(x) for x in meta[2:2 + nd]),
                                  tuple(int(x) for x in meta[2 + nd:2 + 2 * nd]), int(meta[0])))
            i += 1
        res[n] = {"views": views,
                  "digest": str(z[f"{n}/digest"]) if f"{n}/digest" in z else None,
                  "out": z[f"{n}/out"] if f"{n}/out" in z else None}
    return res
