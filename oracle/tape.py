"""TEST INFRASTRUCTURE - NOT PART OF THE PRODUCT.

A reverse-mode tape over numpy arrays whose kernels are the C restatement in oracle.py. It replays the reference
engine: records hold their inputs' metas, Backward does an iterative DFS post-order from the root, sweeps it in
reverse, adopts the first gradient that reaches a node and adds later ones in arrival order
(src/OneModel/Tensors/Autograd/Engine.cs:124-344). Ops record exactly what the reference's Ops.* record, including the
Reshape / MatMul / Add / Permute chain of Ops.Linear (src/OneModel/Tensors/Ops.Layers.cs:715-733).
"""
import numpy as np

from . import oracle as K


class Meta:
    __slots__ = ("requires_grad", "grad_fn", "grad")

    def __init__(self, requires_grad, grad_fn):
        self.requires_grad, self.grad_fn, self.grad = requires_grad, grad_fn, None


class Record:
    __slots__ = ("op", "inputs", "shapes", "saved", "args", "pending", "mark", "backward")

    def __init__(self, op, inputs, saved=(), args=None, backward=None):
        self.op = op
        self.inputs = [t.meta if (t is not None and t.requires_grad) else None for t in inputs]
        self.shapes = [t.shape if t is not None else None for t in inputs]
        self.saved, self.args, self.pending, self.mark, self.backward = saved, args, None, 0, backward


class T:
    """A float32 (or integer) array with optional autograd meta."""

    def __init__(self, value, requires_grad=False, _meta=None):
        self.v = value if isinstance(value, np.ndarray) else np.asarray(value)
        if self.v.dtype == np.float64:
            self.v = self.v.astype(np.float32)
        self.meta = _meta if _meta is not None else (Meta(True, None) if requires_grad else None)

    @property
    def requires_grad(self):
        return self.meta is not None and self.meta.requires_grad

    @property
    def shape(self):
        return self.v.shape

    @property
    def grad(self):
        return None if self.meta is None else self.meta.grad

    def zero_grad(self):
        if self.meta is not None and self.meta.grad is not None:
            self.meta.grad = np.zeros_like(self.meta.grad)

    def backward(self):
        backward(self)

    # views
    def reshape(self, *shape):
        shape = shape[0] if len(shape) == 1 and isinstance(shape[0], (tuple, list)) else shape
        out = np.ascontiguousarray(self.v).reshape(shape)
        return _attach(out, Record("reshape", [self], backward=lambda r, g: [(0, g.reshape(r.shapes[0]), "alias")]), [self])

    def permute(self, *axes):
        axes = axes[0] if len(axes) == 1 and isinstance(axes[0], (tuple, list)) else axes
        inv = np.argsort(axes)
        out = self.v.transpose(axes)
        return _attach(out, Record("permute", [self], backward=lambda r, g: [(0, np.ascontiguousarray(g.transpose(inv)), "own")]), [self])

    def t(self):
        return self.permute(1, 0)

    def slice(self, axis, start, end):
        idx = [slice(None)] * self.v.ndim
        idx[axis] = slice(start, end)
        idx = tuple(idx)

        def bw(r, g):
            dx = np.zeros(r.shapes[0], np.float32)
            dx[idx] = g
            return [(0, dx, "own")]

        return _attach(self.v[idx], Record("slice", [self], backward=bw), [self])


_grad_enabled = True
_pass = 0


def _attach(value, rec, inputs):
    if not _grad_enabled or not any(t is not None and t.requires_grad for t in inputs):
        return T(value)
    return T(value, _meta=Meta(True, rec))


def backward(root, gradient=None):
    """Backprop.Run + Engine.Execute."""
    global _pass, _grad_enabled
    if root.meta is None or not root.requires_grad:
        raise RuntimeError("Backward needs a tensor that requires gradients.")
    g = np.ones(root.shape, np.float32) if gradient is None else np.array(gradient, np.float32)
    if root.meta.grad_fn is None:
        _accumulate_leaf(root.meta, g, True)
        return
    _pass += 1
    mark = _pass
    order, stack = [], [[root.meta.grad_fn, 0]]
    root.meta.grad_fn.mark = mark
    while stack:
        rec, nxt = stack[-1]
        if nxt < len(rec.inputs):
            stack[-1][1] = nxt + 1
            m = rec.inputs[nxt]
            prod = m.grad_fn if m is not None else None
            if prod is not None and prod.mark != mark:
                prod.mark = mark
                stack.append([prod, 0])
        else:
            order.append(rec)
            stack.pop()
    root.meta.grad_fn.pending = g
    prev, _grad_enabled = _grad_enabled, False
    try:
        for rec in reversed(order):
            g, rec.pending = rec.pending, None
            if g is None:
                continue
            for i, grad, how in rec.backward(rec, np.ascontiguousarray(g)):
                if grad is not None:
                    _emit(rec, i, grad, how != "shared")
            rec.saved = ()
    finally:
        _grad_enabled = prev
        for rec in order:
            rec.pending = None


def _emit(rec, i, grad, owned):
    meta = rec.inputs[i]
    if meta is None:
        return
    if meta.grad_fn is None:
        _accumulate_leaf(meta, grad, owned)
        return
    p = meta.grad_fn
    if p.pending is None:
        p.pending = grad if owned else grad.copy()
    else:
        p.pending = _add_into(p.pending, grad)


def _accumulate_leaf(meta, grad, owned):
    if not meta.requires_grad:
        return
    if meta.grad is None:
        meta.grad = np.array(grad, np.float32, copy=True)
    else:
        meta.grad = _add_into(meta.grad, grad)


def _add_into(dst, src):
    # Engine.AddInto: dst[i] += src[i] in element order (float32 adds).
    if not dst.flags.writeable or not dst.flags.c_contiguous:
        dst = np.array(dst, np.float32, copy=True)
    np.add(dst, src, out=dst)
    return dst


class no_grad:
    def __enter__(self):
        global _grad_enabled
        self.prev, _grad_enabled = _grad_enabled, False

    def __exit__(self, *a):
        global _grad_enabled
        _grad_enabled = self.prev


# ---- ops ---------------------------------------------------------------------------------------------------------------

def _emit_summed(r, g, negate_second):
    """BackwardOps.EmitSummed (BackwardOps.cs:156-194)."""
    out = []
    need0, need1 = r.inputs[0] is not None, r.inputs[1] is not None
    if need0:
        s = K.sum_to(g, r.shapes[0])
        same = g.shape == tuple(r.shapes[0])
        out.append((0, s if not same else g, "own" if (not same or not need1) else "shared"))
    if need1:
        s = K.sum_to(g, r.shapes[1])
        if negate_second:
            out.append((1, s * np.float32(-1.0), "own"))
        else:
            out.append((1, s, "own"))
    return out


def add(a, b):
    return _attach(a.v + b.v, Record("add", [a, b], backward=lambda r, g: _emit_summed(r, g, False)), [a, b])


def sub(a, b):
    return _attach(a.v - b.v, Record("sub", [a, b], backward=lambda r, g: _emit_summed(r, g, True)), [a, b])


def mul(a, b):
    def bw(r, g):
        av, bv = r.saved
        return [(0, K.sum_to(g * bv, r.shapes[0]), "own"), (1, K.sum_to(g * av, r.shapes[1]), "own")]

    return _attach(a.v * b.v, Record("mul", [a, b], saved=(a.v, b.v), backward=bw), [a, b])


def relu(x):
    y = K.unary("relu", x.v)
    return _attach(y, Record("relu", [x], saved=(y,), backward=lambda r, g: [(0, K.unary_bwd("relu", g, r.saved[0]), "own")]), [x])


def gelu(x):
    xc = np.ascontiguousarray(x.v)
    return _attach(K.unary("gelu_erf", xc), Record("gelu", [x], saved=(xc,), backward=lambda r, g: [(0, K.unary_bwd("gelu_erf", g, r.saved[0]), "own")]), [x])


GEMM_MODE = "fp32"  # 'tf32' / 'bf16' round the operands of every product first (the tensor-pipe configurations)


def matmul(a, b):
    """Ops.MatMul + MatMul backward (Ops.cs:117-144; BackwardOps.cs:69-82): dA = g b^T, dB = a^T g."""
    av, bv = np.ascontiguousarray(a.v), np.ascontiguousarray(b.v)

    def bw(r, g):
        sa, sb = r.saved
        out = []
        if r.inputs[0] is not None:
            out.append((0, K.gemm(g, sb, tb=True, mode=GEMM_MODE), "own"))
        if r.inputs[1] is not None:
            out.append((1, K.gemm(sa, g, ta=True, mode=GEMM_MODE), "own"))
        return out

    return _attach(K.gemm(av, bv, mode=GEMM_MODE), Record("matmul", [a, b], saved=(av, bv), backward=bw), [a, b])


def linear(x, w, b=None):
    """Ops.Linear: Reshape -> MatMul(x2d, W.T()) -> Add(bias) -> Reshape."""
    in_f, out_f = w.shape[1], w.shape[0]
    y = matmul(x.reshape(x.v.size // max(1, in_f), in_f), w.t())
    if b is not None:
        y = _bias_add(y, b) if GEMM_MODE == "bf16" else add(y, b)
    return y.reshape(x.shape[:-1] + (out_f,))


def _bias_add(y, b):
    """The Add(bias) of Ops.Linear under bfloat16 products: the bias gradient is the product g^T 1 and reads the same
    bfloat16 copy of the output gradient as the weight gradient g^T x (summed in the column sum's order)."""
    def bw(r, g):
        out = []
        if r.inputs[0] is not None:
            out.append((0, g, "shared" if r.inputs[1] is not None else "own"))
        if r.inputs[1] is not None:
            out.append((1, K.colsum_bf16(g.reshape(-1, g.shape[-1])), "own"))
        return out

    return _attach((y.v + b.v).astype(np.float32), Record("add", [y, b], backward=bw), [y, b])


def mean(x, axis=None):
    def bw(r, g):
        return [(0, K.reduce_bwd(g, r.shapes[0], r.args, True), "own")]

    ax = None if axis is None else axis % x.v.ndim
    return _attach(K.reduce_fwd(x.v, ax, True), Record("mean", [x], args=ax, backward=bw), [x])


def sum_(x, axis=None):
    def bw(r, g):
        return [(0, K.reduce_bwd(g, r.shapes[0], r.args, False), "own")]

    ax = None if axis is None else axis % x.v.ndim
    return _attach(K.reduce_fwd(x.v, ax, False), Record("sum", [x], args=ax, backward=bw), [x])


def log_softmax(x):
    y = K.logsoftmax_fwd(x.v)
    return _attach(y, Record("log_softmax", [x], saved=(y,), backward=lambda r, g: [(0, K.logsoftmax_bwd(g, r.saved[0]), "own")]), [x])


def nll_loss(logp, targets, mean=True, ignore=-100):
    loss, _ = K.nll_fwd(logp.v, targets, mean, ignore)
    tg = np.asarray(targets, np.int64)

    def bw(r, g):
        return [(0, K.nll_bwd(float(g.reshape(-1)[0]), tg, r.shapes[0], mean, ignore), "own")]

    return _attach(np.asarray(loss, np.float32), Record("nll", [logp], backward=bw), [logp])


def cross_entropy(logits, targets, mean=True, ignore=-100):
    """Losses.CrossEntropy (src/OneModel.Training/Losses.cs:21-32)."""
    return nll_loss(log_softmax(logits), targets, mean, ignore)


def layer_norm(x, gamma, beta, eps=1e-5):
    xc = np.ascontiguousarray(x.v)
    y, mu, inv = K.layernorm_fwd(xc, gamma.v, beta.v, eps)

    def bw(r, g):
        sx, sg, smu, sinv = r.saved
        dx, dg, db = K.layernorm_bwd(g, sx, sg, smu, sinv)
        return [(0, dx, "own"), (1, dg, "own"), (2, db, "own")]

    return _attach(y, Record("layer_norm", [x, gamma, beta], saved=(xc, gamma.v, mu, inv), backward=bw), [x, gamma, beta])


def batch_norm2d(x, gamma, beta, rm, rv, training=True, momentum=0.1, eps=1e-5):
    xc = np.ascontiguousarray(x.v)
    y, mu, iv = K.batchnorm_fwd(xc, gamma.v, beta.v, rm, rv, training, momentum, eps)

    def bw(r, g):
        sx, sg, smu, siv = r.saved
        dx, dg, db = K.batchnorm_bwd(g, sx, sg, smu, siv, training)
        return [(0, dx, "own"), (1, dg, "own"), (2, db, "own")]

    return _attach(y, Record("batch_norm", [x, gamma, beta], saved=(xc, gamma.v, mu, iv), backward=bw), [x, gamma, beta])


def embedding(table, ids, pad=-1):
    idv = np.asarray(ids, np.int64)
    v, dim = table.shape

    def bw(r, g):
        return [(0, K.embedding_bwd(g, idv, v, dim, pad), "own")]

    return _attach(K.embedding_fwd(table.v, idv), Record("embedding", [table], backward=bw), [table])


def attention(q, k, v, mask=None, scale=None):
    qc, kc, vc = (np.ascontiguousarray(t.v) for t in (q, k, v))
    # Under 'bf16' sequences of several tiles run forward and backward with bfloat16 product operands (the one-tile kernels
    # keep TF32 operands, which the fp32 restatement stands for).
    tier16 = GEMM_MODE == "bf16" and qc.shape[2] > 128 and qc.shape[3] == 64
    y = K.attention_fwd_bf16(qc, kc, vc, mask, scale) if tier16 else K.attention_fwd(qc, kc, vc, mask, scale)

    def bw(r, g):
        if tier16:
            dq, dk, dv = K.attention_bwd_bf16(g, *r.saved, mask=mask, scale=scale, out=y)
        else:
            dq, dk, dv = K.attention_bwd(g, *r.saved, mask=mask, scale=scale)
        return [(0, dq, "own"), (1, dk, "own"), (2, dv, "own")]

    return _attach(y, Record("attention", [q, k, v], saved=(qc, kc, vc), backward=bw), [q, k, v])


def concat(xs, axis):
    def bw(r, g):
        out, start = [], 0
        for i, s in enumerate(r.shapes):
            ln = s[axis]
            idx = [slice(None)] * g.ndim
            idx[axis] = slice(start, start + ln)
            out.append((i, np.ascontiguousarray(g[tuple(idx)]), "own"))
            start += ln
        return out

    return _attach(np.concatenate([t.v for t in xs], axis=axis), Record("concat", list(xs), backward=bw), list(xs))


def _round_operand(a):
    """The operand as a tensor-pipe product sees it under GEMM_MODE (rounded to TF32 or bfloat16, to nearest even)."""
    if GEMM_MODE == "tf32":
        return K.round_tf32(a)
    if GEMM_MODE == "bf16":
        return K.round_bf16(a)
    return a


def conv2d(x, w, b=None, stride=1, padding=0):
    """Ops.Conv2d / ConvBackward (BackwardNn.cs:317-462). Under GEMM_MODE 'tf32' / 'bf16' the operands of the three
    convolution products (x and w forward, g and w for the input gradient, g and x for the weight gradient) are rounded
    first, as for matmul; the products of rounded operands and all sums stay fp32, the bias gradient sums the unrounded g."""
    xc, wc = np.ascontiguousarray(x.v), np.ascontiguousarray(w.v)

    def bw(r, g):
        dx, dw, db = K.conv2d_bwd(_round_operand(g), _round_operand(r.saved[0]), _round_operand(r.saved[1]), stride, padding,
                                  need_dx=r.inputs[0] is not None)
        if GEMM_MODE != "fp32":
            db = np.asarray(g, np.float64).sum(axis=(0, 2, 3)).astype(np.float32)
        out = [(2, db, "own"), (1, dw, "own")] if b is not None else [(1, dw, "own")]
        if dx is not None:
            out.append((0, dx, "own"))
        return out

    ins = [x, w] + ([b] if b is not None else [])
    y = K.conv2d_fwd(_round_operand(xc), _round_operand(wc), b.v if b is not None else None, stride, padding)
    return _attach(y, Record("conv2d", ins, saved=(xc, wc), backward=bw), ins)


def max_pool2d(x, k, stride=None):
    kh, kw = (k, k) if isinstance(k, int) else k
    sh, sw = (kh, kw) if stride is None else ((stride, stride) if isinstance(stride, int) else stride)
    y, idx = K.maxpool_fwd(x.v, kh, kw, sh, sw)
    return _attach(y, Record("max_pool", [x], saved=(idx,), backward=lambda r, g: [(0, K.maxpool_bwd(g, r.saved[0], r.shapes[0]), "own")]), [x])


def avg_pool2d(x, k):
    return _attach(K.avgpool_fwd(x.v, k, k, k, k), Record("avg_pool", [x], backward=lambda r, g: [(0, K.avgpool_bwd(g, r.shapes[0], k, k, k, k), "own")]), [x])


def lstm_layer(x, wih, whh, bih, bhh, reverse=False):
    xc = np.ascontiguousarray(x.v)
    y, gates, c, tc = K.lstm_fwd(xc, wih.v, whh.v, bih.v, bhh.v, reverse)

    def bw(r, g):
        dx, dwih, dwhh, dbih, dbhh = K.lstm_bwd(g, r.saved[0], r.saved[1], r.saved[2], r.saved[3], r.saved[4], r.saved[5], r.saved[6], reverse)
        return [(0, dx, "own"), (1, dwih, "own"), (2, dwhh, "own"), (3, dbih, "own"), (4, dbhh, "own")]

    ins = [x, wih, whh, bih, bhh]
    return _attach(y, Record("lstm", ins, saved=(xc, y, wih.v, whh.v, gates, c, tc), backward=bw), ins)


def gru_layer(x, wih, whh, bih, bhh, h0=None, reverse=False):
    """Ops.GruLayer (Ops.Recurrent.cs:148-260): inputs x, wIh, wHh, bIh, bHh and the optional initial state."""
    xc = np.ascontiguousarray(x.v)
    h0v = None if h0 is None else np.ascontiguousarray(h0.v)
    y, gates, hn = K.gru_fwd(xc, wih.v, whh.v, bih.v, bhh.v, h0v, reverse)

    def bw(r, g):
        dx, dwih, dwhh, dbih, dbhh, dh0 = K.gru_bwd(g, r.saved[0], r.saved[1], r.saved[2], r.saved[3], r.saved[4], r.saved[5], r.saved[6], reverse)
        out = [(0, dx, "own"), (1, dwih, "own"), (2, dwhh, "own"), (3, dbih, "own"), (4, dbhh, "own")]
        if h0 is not None:
            out.append((5, dh0, "own"))
        return out

    ins = [x, wih, whh, bih, bhh] + ([h0] if h0 is not None else [])
    return _attach(y, Record("gru", ins, saved=(xc, y, wih.v, whh.v, h0v, gates, hn), backward=bw), ins)


def ctc_loss(lp, targets, ilen, tlen, blank=0, reduction=1, zero_inf=False):
    lpc = np.ascontiguousarray(lp.v)
    loss, _ = K.ctc_loss(lpc, targets, tlen, ilen, blank, reduction, zero_inf)

    def bw(r, g):
        return [(0, K.ctc_grad(g.reshape(-1), r.saved[0], targets, tlen, ilen, blank, reduction), "own")]

    return _attach(np.asarray(loss, np.float32), Record("ctc", [lp], saved=(lpc,), backward=bw), [lp])


# ---- graph-op family (Ops.GraphOps.cs; BackwardGraphOps.cs of the reference), restated with numpy --------------------
def _sum_to(g, shape):
    """BackwardOps.SumTo: sums over the axes the operand broadcast, double accumulation, rounded once."""
    g64 = np.asarray(g, np.float64)
    while g64.ndim > len(shape):
        g64 = g64.sum(axis=0)
    for i, d in enumerate(shape):
        if d == 1 and g64.shape[i] != 1:
            g64 = g64.sum(axis=i, keepdims=True)
    return g64.astype(np.float32)


def matmul_batched(a, b):
    """Ops.MatMulBatched (Ops.GraphOps.cs:24-100): broadcast batch axes; dA = g b^T, dB = a^T g summed back."""
    def bw(r, g):
        av, bv = r.saved
        ga = np.matmul(g, np.swapaxes(bv, -1, -2)).astype(np.float32)
        gb = np.matmul(np.swapaxes(av, -1, -2), g).astype(np.float32)
        return [(0, _sum_to(ga, av.shape).reshape(av.shape), "own"), (1, _sum_to(gb, bv.shape).reshape(bv.shape), "own")]

    return _attach(np.matmul(a.v, b.v).astype(np.float32), Record("batch_matmul", [a, b], saved=(a.v, b.v), backward=bw), [a, b])


def _erf(x):
    from scipy.special import erf
    return erf(x.astype(np.float64)).astype(np.float32)


def erf(x):
    bw = lambda r, g: [(0, (g * (np.float32(1.1283791671) * np.exp(-(r.saved[0] * r.saved[0])))).astype(np.float32), "own")]
    return _attach(_erf(x.v), Record("erf", [x], saved=(x.v,), backward=bw), [x])


def exp(x):
    y = np.exp(x.v).astype(np.float32)
    return _attach(y, Record("exp", [x], saved=(y,), backward=lambda r, g: [(0, g * r.saved[0], "own")]), [x])


def sqrt(x):
    y = np.sqrt(x.v).astype(np.float32)
    return _attach(y, Record("sqrt", [x], saved=(y,), backward=lambda r, g: [(0, g / (np.float32(2) * r.saved[0]), "own")]), [x])


def pow_(x, p):
    """Ops.Pow / PowDerivative with the exact cases 1, 2, 0.5, -1 (Ops.GraphOps.cs:175-206; BackwardGraphOps.cs:69-76)."""
    p = np.float32(p)
    xv = x.v
    y = xv if p == 1 else xv * xv if p == 2 else np.sqrt(xv) if p == 0.5 else np.float32(1) / xv if p == -1 else np.power(xv, p)

    def bw(r, g):
        v = r.saved[0]
        if p == 1:
            d = np.ones_like(v)
        elif p == 2:
            d = v + v
        elif p == 0.5:
            d = np.float32(1) / (np.sqrt(v) + np.sqrt(v))
        elif p == -1:
            d = np.float32(-1) / (v * v)
        else:
            d = p * np.power(v, p - np.float32(1))
        return [(0, (g * d).astype(np.float32), "own")]

    return _attach(y.astype(np.float32), Record("pow", [x], saved=(xv,), backward=bw), [x])


def where(cond, a, b):
    """Ops.Where (Ops.GraphOps.cs:244-300): cond broadcast with both sides; each side gets g where it was chosen, summed back."""
    c = np.asarray(cond) != 0
    shape = np.broadcast_shapes(c.shape, a.v.shape, b.v.shape)
    cb = np.broadcast_to(c, shape)

    def bw(r, g):
        return [(0, _sum_to(np.where(cb, g, np.float32(0)), a.v.shape).reshape(a.v.shape), "own"),
                (1, _sum_to(np.where(cb, np.float32(0), g), b.v.shape).reshape(b.v.shape), "own")]

    y = np.where(cb, np.broadcast_to(a.v, shape), np.broadcast_to(b.v, shape)).astype(np.float32)
    return _attach(y, Record("where", [a, b], backward=bw), [a, b])


def gather(data, indices, axis):
    """Ops.Gather / GatherBackward (Ops.GraphOps.cs:306-394; BackwardGraphOps.cs:105-139): negative indices count from the end;
    the backward adds slices that share a destination in increasing index position."""
    idx = np.asarray(indices).astype(np.int64)
    ax = axis % data.v.ndim
    n = data.v.shape[ax]
    norm = np.where(idx < 0, idx + n, idx)
    if norm.min(initial=0) < 0 or norm.max(initial=0) >= n:
        raise IndexError("Gather index outside the axis")
    y = np.take(data.v, norm, axis=ax)

    def bw(r, g):
        dx = np.zeros(data.v.shape, np.float32)
        dxm, gm = np.moveaxis(dx, ax, 0), np.moveaxis(g.reshape(data.v.shape[:ax] + (norm.size,) + data.v.shape[ax + 1:]), ax, 0)
        for j, i in enumerate(norm.reshape(-1)):
            dxm[i] += gm[j]
        return [(0, dx, "own")]

    return _attach(y.astype(np.float32), Record("gather", [data], backward=bw), [data])


def conv1d(x, w, b=None, stride=1, pad_left=0, pad_right=0, dilation=1, groups=1):
    """Ops.Conv1d (Ops.Layers.cs:338-402): NCL input, OIK weights, torch.nn.Conv1d semantics with separate left and right
    padding; backward BackwardNn.cs:313-402 on the height-1 view (dW = g im2col(x)^T, dx = col2im(W^T g), dbias = sum g).
    Plain numpy over the kernel taps: for the small cases of the tests."""
    xv, wv = np.ascontiguousarray(x.v), np.ascontiguousarray(w.v)
    n, c, l = xv.shape
    o, cg, k = wv.shape
    og = o // groups
    out_l = (l + pad_left + pad_right - dilation * (k - 1) - 1) // stride + 1
    xp = np.zeros((n, c, l + pad_left + pad_right), np.float32)
    xp[:, :, pad_left:pad_left + l] = xv

    def taps(j):
        return slice(j * dilation, j * dilation + (out_l - 1) * stride + 1, stride)

    y = np.zeros((n, o, out_l), np.float32)
    for g in range(groups):
        for j in range(k):
            y[:, g * og:(g + 1) * og] += np.einsum("ncl,oc->nol", xp[:, g * cg:(g + 1) * cg, taps(j)], wv[g * og:(g + 1) * og, :, j]).astype(np.float32)
    if b is not None:
        y += b.v[None, :, None]

    def bw(r, gr):
        gr = np.asarray(gr, np.float32)
        dxp = np.zeros_like(xp)
        dw = np.zeros_like(wv)
        for g in range(groups):
            gg = gr[:, g * og:(g + 1) * og]
            for j in range(k):
                dw[g * og:(g + 1) * og, :, j] = np.einsum("nol,ncl->oc", gg, xp[:, g * cg:(g + 1) * cg, taps(j)])
                dxp[:, g * cg:(g + 1) * cg, taps(j)] += np.einsum("nol,oc->ncl", gg, wv[g * og:(g + 1) * og, :, j]).astype(np.float32)
        out = []
        if b is not None:
            out.append((2, gr.astype(np.float64).sum(axis=(0, 2)).astype(np.float32), "own"))
        out.append((1, dw, "own"))
        if r.inputs[0] is not None:
            out.append((0, np.ascontiguousarray(dxp[:, :, pad_left:pad_left + l]), "own"))
        return out

    ins = [x, w] + ([b] if b is not None else [])
    return _attach(y, Record("conv1d", ins, backward=bw), ins)


def conv_transpose2d(x, w, b=None, stride=1, padding=0, output_padding=0, groups=1):
    """Ops.ConvTranspose2d (Ops.Spatial.cs:43-130): the adjoint of Conv2d, computed as the input gradient of the convolution
    whose input is this op's output; backward dx = Conv2d(g, W), dW = the adjoint convolution's weight gradient, dbias = sum g
    in double (ConvTransposeBackward, BackwardRecurrent.cs:304-369)."""
    xv, wv = np.ascontiguousarray(x.v), np.ascontiguousarray(w.v)
    n, cin, h, wd = xv.shape
    cout, kh, kw = wv.shape[1] * groups, wv.shape[2], wv.shape[3]
    oh = (h - 1) * stride - 2 * padding + (kh - 1) + output_padding + 1
    ow = (wd - 1) * stride - 2 * padding + (kw - 1) + output_padding + 1
    shape_only = np.zeros((n, cout, oh, ow), np.float32)
    y = K.conv2d_bwd(xv, shape_only, wv, stride, padding, 1, groups)[0]
    if b is not None:
        y = (y + b.v.reshape(1, cout, 1, 1)).astype(np.float32)

    def bw(r, g):
        out = [(0, K.conv2d_fwd(g, wv, None, stride, padding, 1, groups), "own"),
               (1, K.conv2d_bwd(xv, g, wv, stride, padding, 1, groups, need_dx=False)[1], "own")]
        if b is not None:
            out.append((2, np.asarray(g, np.float64).sum(axis=(2, 3)).sum(axis=0).astype(np.float32), "own"))
        return out

    ins = [x, w] + ([b] if b is not None else [])
    return _attach(y, Record("conv_transpose2d", ins, backward=bw), ins)


def _source_coord(mode, align, dst, in_size, out_size):
    """Ops.SourceCoord (Ops.Spatial.cs:200-235) in float32."""
    f = np.float32
    if mode == 0:
        scale = f(in_size) / f(out_size)
        i0 = min(int(np.floor(f(dst) * scale)), in_size - 1)
        return i0, i0, f(0)
    if align:
        scale = f(in_size - 1) / f(out_size - 1) if out_size > 1 else f(0)
        src = scale * f(dst)
    else:
        scale = f(in_size) / f(out_size)
        src = (scale * (f(dst) + f(0.5))) - f(0.5)
        if src < 0:
            src = f(0)
    i0 = min(int(src), in_size - 1)
    i1 = i0 + (1 if i0 < in_size - 1 else 0)
    return i0, i1, f(src - f(i0))


def resize2d(x, out_h, out_w, mode=0, align_corners=False):
    """Ops.Resize2d / ResizeBackward (Ops.Spatial.cs:148-197; BackwardRecurrent.cs:371-412): mode 0 nearest, 1 bilinear."""
    xv = np.ascontiguousarray(x.v)
    n, c, h, w = xv.shape
    align = bool(align_corners) and mode == 1
    ys = [_source_coord(mode, align, oy, h, out_h) for oy in range(out_h)]
    xs = [_source_coord(mode, align, ox, w, out_w) for ox in range(out_w)]
    f = np.float32
    y = np.empty((n, c, out_h, out_w), np.float32)
    for oy, (y0, y1, ly) in enumerate(ys):
        for ox, (x0, x1, lx) in enumerate(xs):
            if mode == 0:
                y[:, :, oy, ox] = xv[:, :, y0, x0]
            else:
                top = ((f(1) - lx) * xv[:, :, y0, x0]) + (lx * xv[:, :, y0, x1])
                bottom = ((f(1) - lx) * xv[:, :, y1, x0]) + (lx * xv[:, :, y1, x1])
                y[:, :, oy, ox] = ((f(1) - ly) * top) + (ly * bottom)

    def bw(r, g):
        dx = np.zeros_like(xv)
        for oy, (y0, y1, ly) in enumerate(ys):
            for ox, (x0, x1, lx) in enumerate(xs):
                gg = g[:, :, oy, ox]
                if mode == 0:
                    dx[:, :, y0, x0] += gg
                else:
                    t, bt = (f(1) - ly) * gg, ly * gg
                    dx[:, :, y0, x0] += (f(1) - lx) * t
                    dx[:, :, y0, x1] += lx * t
                    dx[:, :, y1, x0] += (f(1) - lx) * bt
                    dx[:, :, y1, x1] += lx * bt
        return [(0, dx, "own")]

    return _attach(y, Record("resize2d", [x], backward=bw), [x])


# ---- Dropout and the loss family (Layers.cs:308-371, Generator.cs:10-48, Losses.cs:14-129 of the reference) -----------
_GAMMA = 0x9E3779B97F4A7C15
_M64 = (1 << 64) - 1


def splitmix_finish(z):
    """Generator.Mix: the SplitMix64 finaliser on Python integers (mod 2^64)."""
    z &= _M64
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _M64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _M64
    return z ^ (z >> 31)


def dropout_mask(seed, draw, p, n):
    """The mask of call number `draw` (Layers.cs:354-366): u_i = (Mix(stream + (i+1) G) >> 40) / 2^24 with
    stream = Mix(seed + draw G); kept (u >= p) elements carry float32(1 / (1 - p))."""
    stream = splitmix_finish(seed + draw * _GAMMA)
    with np.errstate(over="ignore"):
        z = np.uint64(stream) + (np.arange(1, n + 1, dtype=np.uint64) * np.uint64(_GAMMA))
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        z = z ^ (z >> np.uint64(31))
    u = (z >> np.uint64(40)).astype(np.float32) * np.float32(1.0 / 16777216.0)
    scale = np.float32(1.0) / (np.float32(1.0) - np.float32(p))
    return np.where(u >= np.float32(p), scale, np.float32(0)).astype(np.float32)


def neg(x):
    return _attach((-x.v).astype(np.float32), Record("neg", [x], backward=lambda r, g: [(0, (-g).astype(np.float32), "own")]), [x])


def dropout(x, p, seed, draw):
    """Dropout.Forward in training mode: Ops.Mul(input, mask)."""
    return mul(x, T(dropout_mask(seed, draw, p, x.v.size).reshape(x.shape)))


def _scalar(v):
    return T(np.array(v, np.float32).reshape(()))


def cross_entropy_smoothed(logits, targets, label_smoothing, ignore=-100, reduce_mean=True):
    """Losses.CrossEntropy with label smoothing (Losses.cs:21-62)."""
    logp = log_softmax(logits)
    nll = nll_loss(logp, targets, reduce_mean, ignore)
    if label_smoothing == 0:
        return nll
    keep = (np.asarray(targets, np.int64) != ignore).astype(np.float32)
    smooth = sum_(mul(neg(mean(logp, 1)), T(keep)))
    if reduce_mean:
        counted = int(keep.sum())
        smooth = mul(smooth, _scalar(np.float32(np.nan) if counted == 0 else np.float32(1.0) / np.float32(counted)))
    return add(mul(nll, _scalar(np.float32(1.0) - np.float32(label_smoothing))), mul(smooth, _scalar(np.float32(label_smoothing))))


def mse_loss(prediction, target, reduce_mean=True):
    d = sub(prediction, target)
    sq = mul(d, d)
    return mean(sq) if reduce_mean else sum_(sq)


def l1_loss(prediction, target, reduce_mean=True):
    d = sub(prediction, target)
    a = add(relu(d), relu(neg(d)))
    return mean(a) if reduce_mean else sum_(a)


def bce_with_logits(logits, targets, reduce_mean=True):
    """softplus(x) - x t with softplus(x) = -LogSoftmax([x, 0])[:, 1] (Losses.cs:113-129)."""
    n = logits.v.size
    x = logits.reshape(n, 1)
    ls = log_softmax(concat([x, T(np.zeros((n, 1), np.float32))], 1))
    softplus = neg(ls.slice(1, 1, 2).reshape(n))
    per = sub(softplus, mul(logits.reshape(n), targets.reshape(n)))
    return mean(per) if reduce_mean else sum_(per)
