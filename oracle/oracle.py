"""TEST INFRASTRUCTURE - NOT PART OF THE PRODUCT.

numpy front end of the CPU restatement of the reference's training hot path (oracle/om_oracle_*.c), plus a small
reverse-mode tape that replays the reference engine's traversal and accumulation order
(src/OneModel/Tensors/Autograd/Engine.cs:124-344 of the reference: iterative DFS post-order over record inputs,
reverse sweep, first gradient adopted, later ones added in arrival order).

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline legs may import this module.
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None

f32p = np.ctypeslib.ndpointer(dtype=np.float32, flags="C_CONTIGUOUS")
i64p = np.ctypeslib.ndpointer(dtype=np.int64, flags="C_CONTIGUOUS")
i32p = np.ctypeslib.ndpointer(dtype=np.int32, flags="C_CONTIGUOUS")


def build():
    subprocess.check_call(["make", "-s", "-C", _HERE])


def lib():
    global _LIB
    if _LIB is None:
        path = os.path.join(_HERE, "libom_oracle.so")
        if not os.path.exists(path):
            build()
        _LIB = C.CDLL(path)
        _LIB.orc_sumsq.restype = C.c_double
    return _LIB


def set_threads(n=0):
    """Sets the OpenMP thread count of the checker's parallel loops (0 = leave as is); returns the count in effect."""
    return int(lib().orc_set_threads(int(n)))


def _f(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _i64(a):
    return np.ascontiguousarray(a, dtype=np.int64)


def _p(a):
    return a.ctypes.data_as(C.c_void_p) if a is not None else None


# ---- plain functions ---------------------------------------------------------------------------------------------------

def gemm(a, b, ta=False, tb=False, mode="fp32"):
    """op(a) @ op(b) with the reference's one-accumulator FMA order. mode 'tf32'/'bf16' rounds the operands first."""
    a, b = _f(a), _f(b)
    if mode == "tf32":
        a, b = round_tf32(a), round_tf32(b)
    elif mode == "bf16":
        a, b = round_bf16(a), round_bf16(b)
    m, k = (a.shape[1], a.shape[0]) if ta else a.shape
    n = b.shape[0] if tb else b.shape[1]
    c = np.empty((m, n), np.float32)
    lib().orc_gemm(int(ta), int(tb), m, n, k, _p(a), a.shape[1], _p(b), b.shape[1], _p(c), n, 0)
    return c


def round_bf16(x):
    x = _f(x)
    y = np.empty_like(x)
    lib().orc_round_bf16(_p(x), _p(y), C.c_int64(x.size))
    return y


def colsum_bf16(g):
    """The bias gradient g^T 1 of the bfloat16 tier in the order the device adds it (include/onemodel_b200.h,
    om_colsum_bf16): g [rows, cols] is rounded to bfloat16; in every chunk of 512 rows, lane l adds rows l, l + 32, ... in
    fp32 in increasing order; the 32 lane sums, then the chunks, are added in double in increasing order. (The reference
    sums a bias gradient in one fp32 pass, Ops.cs ReduceToShape; the order here is this library's own.)"""
    g = round_bf16(np.ascontiguousarray(g, np.float32)).reshape(-1, g.shape[-1])
    rows, cols = g.shape
    total = np.zeros(cols, np.float64)
    for r0 in range(0, rows, 512):
        chunk = np.zeros((512, cols), np.float32)
        n = min(512, rows - r0)
        chunk[:n] = g[r0:r0 + n]
        chunk = chunk.reshape(16, 32, cols)          # [round, lane, column]: row = lane + 32 * round
        lanes = np.zeros((32, cols), np.float32)
        for u in range(16):
            lanes = lanes + chunk[u]
        part = np.zeros(cols, np.float64)
        for lane in range(32):
            part += lanes[lane].astype(np.float64)
        total += part
    return total.astype(np.float32)


def round_tf32(x, nearest=True):
    x = _f(x)
    y = np.empty_like(x)
    lib().orc_round_tf32(_p(x), _p(y), C.c_int64(x.size), int(nearest))
    return y


UNARY = dict(none=0, relu=1, gelu_erf=2, gelu_tanh=3, sigmoid=4, tanh=5, neg=6, exp=7, sqrt=8, erf=9)


def unary(op, x):
    x = _f(x)
    y = np.empty_like(x)
    lib().orc_unary(UNARY[op], _p(x), _p(y), C.c_int64(x.size))
    return y


def unary_bwd(op, g, saved):
    g, saved = _f(g), _f(saved)
    dx = np.empty_like(saved)
    lib().orc_unary_bwd(UNARY[op], _p(g), _p(saved), _p(dx), C.c_int64(g.size))
    return dx


def sum_to(g, target_shape):
    """BackwardOps.SumTo: g summed down to target_shape (double accumulators)."""
    g = _f(g)
    target_shape = tuple(target_shape)
    if g.shape == target_shape:
        return g
    rank, lead = g.ndim, g.ndim - len(target_shape)
    ts = [0] * rank
    acc = 1
    for ax in range(rank - 1, -1, -1):
        t = ax - lead
        if t < 0 or target_shape[t] == 1:
            ts[ax] = 0
        else:
            ts[ax] = acc
            acc *= target_shape[t]
    out = np.empty(target_shape, np.float32)
    shape = (C.c_int32 * max(rank, 1))(*g.shape)
    tsa = (C.c_int64 * max(rank, 1))(*ts)
    lib().orc_sum_to(rank, shape, _p(g), tsa, _p(out), C.c_int64(out.size))
    return out


def reduce_fwd(x, axis, mean):
    x = _f(x)
    if axis is None:
        outer, n, inner, oshape = 1, x.size, 1, ()
    else:
        axis %= x.ndim
        outer = int(np.prod(x.shape[:axis], dtype=np.int64))
        n, inner = x.shape[axis], int(np.prod(x.shape[axis + 1:], dtype=np.int64))
        oshape = x.shape[:axis] + x.shape[axis + 1:]
    y = np.empty(oshape, np.float32)
    lib().orc_reduce_fwd(_p(x), C.c_int64(outer), C.c_int64(n), C.c_int64(inner), int(mean), _p(y))
    return y


def reduce_bwd(g, in_shape, axis, mean):
    g = _f(g)
    if axis is None:
        outer, n, inner = 1, int(np.prod(in_shape, dtype=np.int64)), 1
    else:
        outer = int(np.prod(in_shape[:axis], dtype=np.int64))
        n, inner = in_shape[axis], int(np.prod(in_shape[axis + 1:], dtype=np.int64))
    dx = np.empty(in_shape, np.float32)
    lib().orc_reduce_bwd(_p(g), C.c_int64(outer), C.c_int64(n), C.c_int64(inner), int(mean), _p(dx))
    return dx


def _rows(x):
    cols = x.shape[-1]
    return (x.size // cols if cols else 0), cols


def softmax_fwd(x):
    x = _f(x)
    y = np.empty_like(x)
    lib().orc_softmax_fwd(_p(x), *_rows(x), _p(y))
    return y


def logsoftmax_fwd(x):
    x = _f(x)
    y = np.empty_like(x)
    lib().orc_logsoftmax_fwd(_p(x), *_rows(x), _p(y))
    return y


def softmax_bwd(g, y):
    g, y = _f(g), _f(y)
    dx = np.empty_like(y)
    lib().orc_softmax_bwd(_p(g), _p(y), *_rows(y), _p(dx))
    return dx


def logsoftmax_bwd(g, y):
    g, y = _f(g), _f(y)
    dx = np.empty_like(y)
    lib().orc_logsoftmax_bwd(_p(g), _p(y), *_rows(y), _p(dx))
    return dx


def nll_fwd(logp, targets, mean=True, ignore=-100):
    logp, targets = _f(logp), _i64(targets)
    loss = np.zeros((), np.float32)
    count = lib().orc_nll_fwd(_p(logp), _p(targets), logp.shape[0], logp.shape[1], int(mean), C.c_int64(ignore), _p(loss))
    if count < 0:
        raise IndexError("target outside the classes")
    return loss, count


def nll_bwd(g, targets, shape, mean=True, ignore=-100):
    targets = _i64(targets)
    dx = np.empty(shape, np.float32)
    lib().orc_nll_bwd(C.c_float(float(g)), _p(targets), shape[0], shape[1], int(mean), C.c_int64(ignore), _p(dx))
    return dx


def layernorm_fwd(x, gamma, beta, eps=1e-5):
    x, gamma, beta = _f(x), _f(gamma), _f(beta)
    rows, cols = _rows(x)
    y, mean, inv = np.empty_like(x), np.empty(rows, np.float32), np.empty(rows, np.float32)
    lib().orc_layernorm_fwd(_p(x), _p(gamma), _p(beta), rows, cols, C.c_float(eps), _p(y), _p(mean), _p(inv))
    return y, mean, inv


def layernorm_bwd(g, x, gamma, mean, inv):
    g, x, gamma = _f(g), _f(x), _f(gamma)
    rows, cols = _rows(x)
    dx, dg, db = np.empty_like(x), np.empty(cols, np.float32), np.empty(cols, np.float32)
    lib().orc_layernorm_bwd(_p(g), _p(x), _p(gamma), _p(_f(mean)), _p(_f(inv)), rows, cols, _p(dx), _p(dg), _p(db))
    return dx, dg, db


def batchnorm_fwd(x, gamma, beta, rm, rv, training=True, momentum=0.1, eps=1e-5):
    """rm, rv are updated in place (float32 arrays)."""
    x = _f(x)
    n, c = x.shape[0], x.shape[1]
    plane = x.size // max(1, n * c)
    y, mu, iv = np.empty_like(x), np.empty(c, np.float32), np.empty(c, np.float32)
    lib().orc_batchnorm_fwd(_p(x), _p(_f(gamma)), _p(_f(beta)), _p(rm), _p(rv), n, c, plane, int(training),
                            C.c_float(momentum), C.c_float(eps), _p(y), _p(mu), _p(iv))
    return y, mu, iv


def batchnorm_bwd(g, x, gamma, mu, iv, training=True):
    g, x = _f(g), _f(x)
    n, c = x.shape[0], x.shape[1]
    plane = x.size // max(1, n * c)
    dx, dg, db = np.empty_like(x), np.empty(c, np.float32), np.empty(c, np.float32)
    lib().orc_batchnorm_bwd(_p(g), _p(x), _p(_f(gamma)), _p(_f(mu)), _p(_f(iv)), n, c, plane, int(training), _p(dx), _p(dg), _p(db))
    return dx, dg, db


def embedding_fwd(table, ids):
    table, ids = _f(table), _i64(ids)
    out = np.empty(ids.shape + (table.shape[1],), np.float32)
    if lib().orc_embedding_fwd(_p(table), table.shape[0], table.shape[1], _p(ids), C.c_int64(ids.size), _p(out)) != 0:
        raise IndexError("id outside the table")
    return out


def embedding_bwd(g, ids, v, dim, pad=-1):
    g, ids = _f(g), _i64(ids)
    dt = np.empty((v, dim), np.float32)
    lib().orc_embedding_bwd(_p(g), _p(ids), C.c_int64(ids.size), v, dim, C.c_int64(pad), _p(dt))
    return dt


def _mask_args(mask, lq, lk):
    if mask is None:
        return None, 0
    m = _f(mask)
    return m, (0 if m.ndim == 2 else lq * lk)


def attention_fwd(q, k, v, mask=None, scale=None):
    q, k, v = _f(q), _f(k), _f(v)
    b, h, lq, d = q.shape
    lk = k.shape[2]
    scale = np.float32(1.0) / np.sqrt(np.float32(d)) if scale is None else np.float32(scale)
    m, mbs = _mask_args(mask, lq, lk)
    out = np.empty_like(q)
    lib().orc_attention_fwd(_p(q), _p(k), _p(v), _p(m), C.c_int64(mbs), b, h, lq, lk, d, C.c_float(scale), _p(out))
    return out


def attention_bwd(g, q, k, v, mask=None, scale=None):
    g, q, k, v = _f(g), _f(q), _f(k), _f(v)
    b, h, lq, d = q.shape
    lk = k.shape[2]
    scale = np.float32(1.0) / np.sqrt(np.float32(d)) if scale is None else np.float32(scale)
    m, mbs = _mask_args(mask, lq, lk)
    dq, dk, dv = np.empty_like(q), np.empty_like(k), np.empty_like(v)
    lib().orc_attention_bwd(_p(g), _p(q), _p(k), _p(v), _p(m), C.c_int64(mbs), b, h, lq, lk, d, C.c_float(scale), _p(dq), _p(dk), _p(dv))
    return dq, dk, dv


def attention_fwd_bf16(q, k, v, mask=None, scale=None):
    """The attention forward with the operands of its two products rounded to bfloat16 (nearest even) and everything else in
    fp32: S = Q K^T from rounded q, k; E = exp(scale S + mask - rowmax) and its row sums in fp32; O = (E rounded) (V rounded)
    divided by the row sums. The model of the forward's bfloat16 tier; plain numpy, for small cases."""
    q, k, v = _f(q), _f(k), _f(v)
    b, h, lq, d = q.shape
    scale = np.float32(1.0) / np.sqrt(np.float32(d)) if scale is None else np.float32(scale)
    qr, kr, vr = round_bf16(q), round_bf16(k), round_bf16(v)
    out = np.empty_like(q)
    for bi in range(b):
        mb = None if mask is None else (mask if np.ndim(mask) == 2 else mask[bi])
        for hi in range(h):
            s = (qr[bi, hi] @ kr[bi, hi].T) * scale
            if mb is not None:
                s = s + _f(mb)
            s64 = s.astype(np.float64)
            e = np.exp(s64 - s64.max(axis=1, keepdims=True)).astype(np.float32)
            total = e.astype(np.float64).sum(axis=1, keepdims=True)
            out[bi, hi] = ((round_bf16(e) @ vr[bi, hi]).astype(np.float64) / total).astype(np.float32)
    return out


def attention_bwd_bf16(g, q, k, v, mask=None, scale=None, out=None):
    """AttentionBackward (BackwardNn.cs:636-701) with the operands of its five products rounded to bfloat16 (nearest even) and
    everything else in fp32: S = Q K^T and dP = dO V^T from rounded q, k, v, dO; P = softmax(scale S + mask) and the row dots
    rowsum(dO o O) in fp32 (O given, or from the fp32 forward); dS = P (dP - dot) scale; dV = P^T dO, dK = dS^T Q, dQ = dS K with P and
    dS rounded. The model of the product's bfloat16 tier; plain numpy, for small cases."""
    g, q, k, v = _f(g), _f(q), _f(k), _f(v)
    b, h, lq, d = q.shape
    lk = k.shape[2]
    scale = np.float32(1.0) / np.sqrt(np.float32(d)) if scale is None else np.float32(scale)
    out = attention_fwd(q, k, v, mask, scale) if out is None else _f(out)
    gr, qr, kr, vr = round_bf16(g), round_bf16(q), round_bf16(k), round_bf16(v)
    dq, dk, dv = np.empty_like(q), np.empty_like(k), np.empty_like(v)
    for bi in range(b):
        mb = None if mask is None else (mask if np.ndim(mask) == 2 else mask[bi])
        for hi in range(h):
            s = (qr[bi, hi] @ kr[bi, hi].T) * scale
            if mb is not None:
                s = s + _f(mb)
            s64 = s.astype(np.float64)
            mx = s64.max(axis=1, keepdims=True)
            e = np.exp(s64 - mx)
            p = (e / e.sum(axis=1, keepdims=True)).astype(np.float32)
            dot = (g[bi, hi].astype(np.float64) * out[bi, hi]).sum(axis=1, keepdims=True).astype(np.float32)
            dp = gr[bi, hi] @ vr[bi, hi].T
            ds = (p * (dp - dot)) * scale
            pr, dsr = round_bf16(p), round_bf16(ds)
            dv[bi, hi] = pr.T @ gr[bi, hi]
            dk[bi, hi] = dsr.T @ qr[bi, hi]
            dq[bi, hi] = dsr @ kr[bi, hi]
    return dq, dk, dv


def adam_step(p, g, m, v, vmax, t, lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, wd=0.0, decoupled=False, amsgrad=False):
    """In place on p, m, v (and vmax). t is the 1-based step."""
    lib().orc_adam_step(_p(p), _p(_f(g)), _p(m), _p(v), _p(vmax), C.c_int64(p.size), C.c_float(lr), C.c_float(beta1),
                        C.c_float(beta2), C.c_float(eps), C.c_float(wd), int(decoupled), int(amsgrad), C.c_int64(t))


def sgd_step(p, g, buf, first, lr, wd=0.0, momentum=0.0, dampening=0.0, nesterov=False):
    lib().orc_sgd_step(_p(p), _p(_f(g)), _p(buf), C.c_int64(p.size), C.c_float(lr), C.c_float(wd), C.c_float(momentum),
                       C.c_float(dampening), int(nesterov), int(momentum != 0.0), int(first))


def clip_norm(grads, max_norm, infinity=False):
    """GradClip.ClipNorm on a list of arrays, in place. Returns the total norm (float32)."""
    acc = 0.0
    for g in grads:
        acc = lib().orc_sumsq(_p(g), C.c_int64(g.size), C.c_double(acc), int(infinity))
    norm = acc if infinity else float(np.sqrt(np.float64(acc)))
    total = np.float32(norm)
    if not np.isfinite(norm):
        return total
    coef = np.float32(np.float64(np.float32(max_norm)) / (norm + 1e-6))
    if coef < 1:
        for g in grads:
            lib().orc_scale(_p(g), C.c_int64(g.size), C.c_float(coef))
    return total


# ---- convolution, pooling, LSTM, CTC (om_oracle_spatial.c) ---------------------------------------------------------------

class _ConvShape(C.Structure):
    _fields_ = [(n, C.c_int) for n in ("n", "cin", "h", "w", "cout", "kh", "kw", "sh", "sw", "pt", "pl", "pb", "pr", "dh", "dw", "groups")]


def _conv_shape(x, w, stride, padding, dilation=1, groups=1):
    s = _ConvShape(x.shape[0], x.shape[1], x.shape[2], x.shape[3], w.shape[0], w.shape[2], w.shape[3], stride, stride,
                   padding, padding, padding, padding, dilation, dilation, groups)
    oh = (s.h + 2 * padding - dilation * (s.kh - 1) - 1) // stride + 1
    ow = (s.w + 2 * padding - dilation * (s.kw - 1) - 1) // stride + 1
    return s, oh, ow


def conv2d_fwd(x, w, bias=None, stride=1, padding=0, dilation=1, groups=1):
    x, w = _f(x), _f(w)
    s, oh, ow = _conv_shape(x, w, stride, padding, dilation, groups)
    y = np.empty((s.n, s.cout, oh, ow), np.float32)
    b = _f(bias) if bias is not None else None
    lib().orc_conv2d_fwd(C.byref(s), _p(x), _p(w), _p(b), _p(y))
    return y


def conv2d_bwd(g, x, w, stride=1, padding=0, dilation=1, groups=1, need_dx=True):
    g, x, w = _f(g), _f(x), _f(w)
    s, _, _ = _conv_shape(x, w, stride, padding, dilation, groups)
    dx = np.empty_like(x) if need_dx else None
    dw, db = np.empty_like(w), np.empty(w.shape[0], np.float32)
    lib().orc_conv2d_bwd(C.byref(s), _p(g), _p(x), _p(w), _p(dx), _p(dw), _p(db))
    return dx, dw, db


def _pool_out(size, k, s, p):
    return (size + 2 * p - k) // s + 1


def maxpool_fwd(x, kh, kw, sh, sw, ph=0, pw=0):
    x = _f(x)
    n, c, h, w = x.shape
    oh, ow = _pool_out(h, kh, sh, ph), _pool_out(w, kw, sw, pw)
    y, idx = np.empty((n, c, oh, ow), np.float32), np.empty((n, c, oh, ow), np.int32)
    lib().orc_maxpool_fwd(_p(x), n * c, h, w, kh, kw, sh, sw, ph, pw, oh, ow, _p(y), _p(idx))
    return y, idx


def maxpool_bwd(g, idx, in_shape):
    g, idx = _f(g), np.ascontiguousarray(idx, np.int32)
    dx = np.empty(in_shape, np.float32)
    lib().orc_maxpool_bwd(_p(g), _p(idx), C.c_int64(g.size), C.c_int64(dx.size), _p(dx))
    return dx


def avgpool_fwd(x, kh, kw, sh, sw, ph=0, pw=0, include_pad=False):
    x = _f(x)
    n, c, h, w = x.shape
    oh, ow = _pool_out(h, kh, sh, ph), _pool_out(w, kw, sw, pw)
    y = np.empty((n, c, oh, ow), np.float32)
    lib().orc_avgpool_fwd(_p(x), n * c, h, w, kh, kw, sh, sw, ph, pw, int(include_pad), oh, ow, _p(y))
    return y


def avgpool_bwd(g, in_shape, kh, kw, sh, sw, ph=0, pw=0, include_pad=False):
    g = _f(g)
    n, c, h, w = in_shape
    dx = np.empty(in_shape, np.float32)
    lib().orc_avgpool_bwd(_p(g), n * c, h, w, kh, kw, sh, sw, ph, pw, int(include_pad), g.shape[2], g.shape[3], _p(dx))
    return dx


def lstm_fwd(x, wih, whh, bih, bhh, reverse=False):
    x, wih, whh = _f(x), _f(wih), _f(whh)
    t, b, i = x.shape
    h = whh.shape[1]
    y, gates = np.empty((t, b, h), np.float32), np.empty((t, b, 4 * h), np.float32)
    c, tc = np.empty((t, b, h), np.float32), np.empty((t, b, h), np.float32)
    lib().orc_lstm_fwd(int(reverse), t, b, i, h, _p(x), _p(wih), _p(whh), _p(_f(bih) if bih is not None else None),
                       _p(_f(bhh) if bhh is not None else None), _p(y), _p(gates), _p(c), _p(tc))
    return y, gates, c, tc


def lstm_bwd(gy, x, y, wih, whh, gates, c, tc, reverse=False):
    gy, x, y, wih, whh = _f(gy), _f(x), _f(y), _f(wih), _f(whh)
    t, b, i = x.shape
    h = whh.shape[1]
    dx, dwih, dwhh = np.empty_like(x), np.empty_like(wih), np.empty_like(whh)
    dbih, dbhh = np.empty(4 * h, np.float32), np.empty(4 * h, np.float32)
    lib().orc_lstm_bwd(int(reverse), t, b, i, h, _p(gy), _p(x), _p(y), _p(wih), _p(whh), _p(_f(gates)), _p(_f(c)), _p(_f(tc)),
                       _p(dx), _p(dwih), _p(dwhh), _p(dbih), _p(dbhh))
    return dx, dwih, dwhh, dbih, dbhh


def gru_fwd(x, wih, whh, bih, bhh, h0=None, reverse=False):
    x, wih, whh = _f(x), _f(wih), _f(whh)
    t, b, i = x.shape
    h = whh.shape[1]
    y, gates, hn = np.empty((t, b, h), np.float32), np.empty((t, b, 3 * h), np.float32), np.empty((t, b, h), np.float32)
    lib().orc_gru_fwd(int(reverse), t, b, i, h, _p(x), _p(wih), _p(whh), _p(_f(bih) if bih is not None else None),
                      _p(_f(bhh) if bhh is not None else None), _p(_f(h0) if h0 is not None else None), _p(y), _p(gates), _p(hn))
    return y, gates, hn


def gru_bwd(gy, x, y, wih, whh, h0, gates, hn, reverse=False):
    gy, x, y, wih, whh = _f(gy), _f(x), _f(y), _f(wih), _f(whh)
    t, b, i = x.shape
    h = whh.shape[1]
    dx, dwih, dwhh = np.empty_like(x), np.empty_like(wih), np.empty_like(whh)
    dbih, dbhh, dh0 = np.empty(3 * h, np.float32), np.empty(3 * h, np.float32), np.empty((b, h), np.float32)
    lib().orc_gru_bwd(int(reverse), t, b, i, h, _p(gy), _p(x), _p(y), _p(wih), _p(whh), _p(_f(h0) if h0 is not None else None),
                      _p(_f(gates)), _p(_f(hn)), _p(dx), _p(dwih), _p(dwhh), _p(dbih), _p(dbhh), _p(dh0))
    return dx, dwih, dwhh, dbih, dbhh, dh0


def _i32(a):
    return np.ascontiguousarray(a, np.int32)


def ctc_loss(lp, targets, tlen, ilen, blank=0, reduction=1, zero_inf=False):
    lp, targets, tlen, ilen = _f(lp), _i32(targets), _i32(tlen), _i32(ilen)
    t, b, c = lp.shape
    nll, loss = np.empty(b, np.float32), np.zeros((), np.float32)
    lib().orc_ctc_loss(_p(lp), t, b, c, _p(targets), _p(tlen), _p(ilen), blank, reduction, int(zero_inf), _p(nll), _p(loss))
    return (nll if reduction == 0 else loss), nll


def ctc_grad(g, lp, targets, tlen, ilen, blank=0, reduction=1):
    lp, targets, tlen, ilen = _f(lp), _i32(targets), _i32(tlen), _i32(ilen)
    t, b, c = lp.shape
    grad = np.empty_like(lp)
    lib().orc_ctc_grad(_p(_f(np.atleast_1d(g))), _p(lp), t, b, c, _p(targets), _p(tlen), _p(ilen), blank, reduction, _p(grad))
    return grad


def ctc_greedy(lp, ilen=None, blank=0):
    lp = _f(lp)
    t, b, c = lp.shape
    labels, first, last = (np.empty((b, t), np.int32) for _ in range(3))
    lengths = np.empty(b, np.int32)
    il = _i32(ilen) if ilen is not None else None
    lib().orc_ctc_greedy(_p(lp), t, b, c, _p(il), blank, _p(labels), _p(first), _p(last), _p(lengths))
    return labels, first, last, lengths


def rows_touched(ids, rows, padding_index=-1):
    """How many positions name each table row (ids equal to padding_index skipped): the support of the reference's
    RowSparseGradient (RowSparseGradient.cs:14-120)."""
    ids = np.asarray(ids).reshape(-1)
    ids = ids[ids != padding_index]
    return np.bincount(ids, minlength=rows).astype(np.int32)


def embedding_bwd_sparse(g, ids, pad=-1):
    """EmbeddingSparseBackward (BackwardNn.cs:548-600): the (id << 31 | position) keys of the lookups that are not padding,
    sorted; one entry per distinct id in ascending order, its value the sum of the lookups' gradient rows in increasing
    position order starting from zero. Returns (rows int32 [U], values float32 [U, dim]); U = 0 when only padding was
    looked up (the reference then keeps no gradient)."""
    ids = np.asarray(ids).reshape(-1)
    g = np.asarray(g, np.float32).reshape(ids.size, -1)
    keys = sorted((int(t) << 31) | i for i, t in enumerate(ids) if t != pad)
    rows, values = [], []
    for key in keys:
        row, pos = key >> 31, key & 0x7FFFFFFF
        if not rows or rows[-1] != row:
            rows.append(row)
            values.append(np.zeros(g.shape[1], np.float32))
        values[-1] = values[-1] + g[pos]
    return np.array(rows, np.int32), (np.stack(values) if values else np.zeros((0, g.shape[1]), np.float32))


def rowsparse_to_dense(rows, values, v):
    """RowSparseGradient.ToDense / AddTo (RowSparseGradient.cs:39-63): dense[rows[k]] += values[k] into zeros."""
    dense = np.zeros((v, values.shape[1]), np.float32)
    for k, row in enumerate(rows):
        dense[row] = dense[row] + values[k]
    return dense


def rowsparse_merge(rows_a, values_a, rows_b, values_b):
    """RowSparseGradient.Merge (RowSparseGradient.cs:66-116): the union of the rows in ascending order; a row's value is a's
    (or zero) with b's added to it."""
    width = values_a.shape[1]
    at = {int(r): k for k, r in enumerate(rows_a)}
    bt = {int(r): k for k, r in enumerate(rows_b)}
    rows = sorted(set(at) | set(bt))
    values = np.zeros((len(rows), width), np.float32)
    for k, row in enumerate(rows):
        if row in at:
            values[k] = values_a[at[row]]
        if row in bt:
            values[k] = values[k] + values_b[bt[row]]
    return np.array(rows, np.int32), values


def int_pow(b, n):
    """Adam.IntPow: binary powering in double (Optimizers.cs:483-499)."""
    r, b = 1.0, float(b)
    while n > 0:
        if n & 1:
            r *= b
        b *= b
        n >>= 1
    return r


def sparse_adam_step(p, g, m, v, touched, t, lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8):
    """SparseAdam.BeginStep + UpdateSparse (Optimizers.cs:680-722) in place on the touched rows of p, m, v; float32 operations
    in the reference's order, step size from double arithmetic."""
    f = np.float32
    b1, b2 = f(beta1), f(beta2)
    step = f(float(f(lr)) * np.sqrt(1.0 - int_pow(b2, t)) / (1.0 - int_pow(b1, t)))
    rows = np.nonzero(np.asarray(touched))[0]
    gi = g[rows].astype(f)
    mi = b1 * m[rows] + (f(1) - b1) * gi
    vi = b2 * v[rows] + ((f(1) - b2) * gi) * gi
    m[rows], v[rows] = mi, vi
    p[rows] = p[rows] - (step * mi) / (np.sqrt(vi) + f(eps))


def sparse_sgd_step(p, g, touched, lr):
    """Sgd.UpdateSparse (Optimizers.cs:377-397): p -= lr * g on the touched rows."""
    rows = np.nonzero(np.asarray(touched))[0]
    p[rows] = p[rows] - np.float32(lr) * g[rows]
