"""Two implementations of one small tensor API so that every model in tests/models.py is written once and run both on
the CPU oracle (oracle/tape.py) and on the GPU through the host mirror + C ABI (om_binding.py)."""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "onemodel-csharp_b200")
for p in (ROOT, PKG):
    if p not in sys.path:
        sys.path.insert(0, p)


class OracleBackend:
    name = "oracle"

    def __init__(self, gemm_mode="fp32"):
        from oracle import oracle as K, tape
        self.K, self.tape = K, tape
        tape.GEMM_MODE = gemm_mode

    def tensor(self, a, requires_grad=False):
        a = np.asarray(a)
        if a.dtype.kind == "f":
            a = a.astype(np.float32)
        return self.tape.T(a.copy(), requires_grad)

    def ids(self, a):
        return np.asarray(a, np.int64)

    def numpy(self, t):
        return np.asarray(t.v)

    def grad(self, t):
        return None if t.grad is None else np.asarray(t.grad)

    def set_value(self, t, a):
        t.v = np.array(a, np.float32)

    # ops
    def add(self, a, b): return self.tape.add(a, b)
    def sub(self, a, b): return self.tape.sub(a, b)
    def mul(self, a, b): return self.tape.mul(a, b)
    def relu(self, x): return self.tape.relu(x)
    def gelu(self, x): return self.tape.gelu(x)
    def matmul(self, a, b): return self.tape.matmul(a, b)
    def linear(self, x, w, b=None): return self.tape.linear(x, w, b)
    def mean(self, x, axis=None): return self.tape.mean(x, axis)
    def sum(self, x, axis=None): return self.tape.sum_(x, axis)
    def log_softmax(self, x): return self.tape.log_softmax(x)
    def nll_loss(self, lp, t): return self.tape.nll_loss(lp, t)
    def cross_entropy(self, x, t): return self.tape.cross_entropy(x, t)
    def layer_norm(self, x, g, b, eps=1e-5): return self.tape.layer_norm(x, g, b, eps)
    def embedding(self, table, ids): return self.tape.embedding(table, ids)
    def attention(self, q, k, v, mask=None): return self.tape.attention(q, k, v, mask)
    def batch_norm2d(self, x, g, b, rm, rv, training=True): return self.tape.batch_norm2d(x, g, b, rm, rv, training)
    def conv2d(self, x, w, b, stride=1, padding=0): return self.tape.conv2d(x, w, b, stride, padding)
    def max_pool2d(self, x, k): return self.tape.max_pool2d(x, k)
    def avg_pool2d(self, x, k): return self.tape.avg_pool2d(x, k)
    def lstm_layer(self, x, wih, whh, bih, bhh, reverse=False): return self.tape.lstm_layer(x, wih, whh, bih, bhh, reverse)
    def concat(self, xs, axis): return self.tape.concat(xs, axis)
    def gru_layer(self, x, wih, whh, bih, bhh, h0=None, reverse=False): return self.tape.gru_layer(x, wih, whh, bih, bhh, h0, reverse)
    def matmul_batched(self, a, b): return self.tape.matmul_batched(a, b)
    def conv_transpose2d(self, x, w, b, stride=1, padding=0, output_padding=0, groups=1):
        return self.tape.conv_transpose2d(x, w, b, stride, padding, output_padding, groups)
    def conv1d(self, x, w, b, stride=1, pad_left=0, pad_right=0, dilation=1, groups=1):
        return self.tape.conv1d(x, w, b, stride, pad_left, pad_right, dilation, groups)
    def resize2d(self, x, oh, ow, mode=0, align=False): return self.tape.resize2d(x, oh, ow, mode, align)
    def erf(self, x): return self.tape.erf(x)
    def exp(self, x): return self.tape.exp(x)
    def sqrt(self, x): return self.tape.sqrt(x)
    def pow(self, x, p): return self.tape.pow_(x, p)
    def where(self, c, a, b): return self.tape.where(c, a, b)
    def gather(self, data, idx, axis): return self.tape.gather(data, idx, axis)
    def cross_entropy_smoothed(self, x, t, smoothing, ignore=-100, mean=True):
        return self.tape.cross_entropy_smoothed(x, t, smoothing, ignore, mean)
    def mse_loss(self, x, t, mean=True): return self.tape.mse_loss(x, t, mean)
    def l1_loss(self, x, t, mean=True): return self.tape.l1_loss(x, t, mean)
    def bce_with_logits(self, x, t, mean=True): return self.tape.bce_with_logits(x, t, mean)
    def dropout(self, x, p, seed, draw): return self.tape.dropout(x, p, seed, draw)
    def select(self, t, axis, index):
        shape = list(t.shape)
        del shape[axis]
        return t.slice(axis, index, index + 1).reshape(*shape)
    def ctc_loss(self, lp, targets, ilen, tlen, blank=0, reduction=1, zero_inf=False):
        return self.tape.ctc_loss(lp, targets, ilen, tlen, blank, reduction, zero_inf)
    def running(self, a): return np.array(a, np.float32)
    def running_numpy(self, r): return np.asarray(r)
    def backward(self, loss): loss.backward()
    def zero_grad(self, params):
        for p in params:
            p.zero_grad()


class GpuBackend:
    name = "gpu"

    def __init__(self, ctx):
        import om_binding as omb
        self.omb, self.ctx = omb, ctx
        ctx.make_current()

    def tensor(self, a, requires_grad=False):
        return self.omb.Tensor.from_numpy(np.asarray(a, np.float32), requires_grad)

    def ids(self, a):
        return self.omb.Tensor.from_numpy(np.asarray(a, np.int64))

    def numpy(self, t):
        return t.numpy()

    def grad(self, t):
        g = t.grad
        return None if g is None else g.numpy()

    def set_value(self, t, a):
        t.copy_from(a)

    def _mask(self, m):
        return None if m is None else self.omb.Tensor.from_numpy(np.asarray(m, np.float32))

    def add(self, a, b): return self.omb.call("add", [a, b])
    def sub(self, a, b): return self.omb.call("sub", [a, b])
    def mul(self, a, b): return self.omb.call("mul", [a, b])
    def relu(self, x): return self.omb.call("relu", [x])
    def gelu(self, x): return self.omb.call("gelu", [x], ints=[0])
    def matmul(self, a, b): return self.omb.call("matmul", [a, b])
    def linear(self, x, w, b=None): return self.omb.call("linear", [x, w, b])
    def mean(self, x, axis=None): return self.omb.call("mean", [x], ints=[] if axis is None else [axis, 0])
    def sum(self, x, axis=None): return self.omb.call("sum", [x], ints=[] if axis is None else [axis, 0])
    def log_softmax(self, x): return self.omb.call("log_softmax", [x], ints=[-1])
    def nll_loss(self, lp, t): return self.omb.call("nll_loss", [lp, t], ints=[1, -100])
    def cross_entropy(self, x, t): return self.omb.call("cross_entropy", [x, t], ints=[1, -100])
    def layer_norm(self, x, g, b, eps=1e-5): return self.omb.call("layer_norm", [x, g, b], floats=[eps])
    def embedding(self, table, ids): return self.omb.call("embedding", [table, ids], ints=[-1])
    def attention(self, q, k, v, mask=None): return self.omb.call("attention", [q, k, v, self._mask(mask)], floats=[0.0])
    def batch_norm2d(self, x, g, b, rm, rv, training=True):
        return self.omb.call("batch_norm2d", [x, g, b, rm, rv], ints=[1 if training else 0], floats=[0.1, 1e-5])
    def conv2d(self, x, w, b, stride=1, padding=0):
        return self.omb.call("conv2d", [x, w, b], ints=[stride, stride, padding, padding, padding, padding, 1, 1, 1])
    def max_pool2d(self, x, k):
        kh, kw = (k, k) if isinstance(k, int) else k
        return self.omb.call("max_pool2d", [x], ints=[kh, kw, kh, kw, 0, 0])
    def lstm_layer(self, x, wih, whh, bih, bhh, reverse=False):
        return self.omb.call("lstm_layer", [x, wih, whh, bih, bhh], ints=[1 if reverse else 0])
    def concat(self, xs, axis): return self.omb.call("concat", list(xs), ints=[axis])
    def gru_layer(self, x, wih, whh, bih, bhh, h0=None, reverse=False):
        return self.omb.call("gru_layer", [x, wih, whh, bih, bhh, h0], ints=[1 if reverse else 0])
    def cross_entropy_smoothed(self, x, t, smoothing, ignore=-100, mean=True):
        return self.omb.call("cross_entropy_smoothed", [x, t], ints=[1 if mean else 0, ignore], floats=[smoothing])
    def mse_loss(self, x, t, mean=True): return self.omb.call("mse_loss", [x, t], ints=[1 if mean else 0])
    def l1_loss(self, x, t, mean=True): return self.omb.call("l1_loss", [x, t], ints=[1 if mean else 0])
    def bce_with_logits(self, x, t, mean=True): return self.omb.call("bce_with_logits", [x, t], ints=[1 if mean else 0])
    def dropout(self, x, p, seed, draw):
        counter = self.omb.Tensor.from_numpy(np.array([draw], np.int64))
        return self.omb.call("dropout", [x, counter], ints=[seed], floats=[p])
    def select(self, t, axis, index): return t.select(axis, index)
    def matmul_batched(self, a, b): return self.omb.call("matmul_batched", [a, b])
    def conv_transpose2d(self, x, w, b, stride=1, padding=0, output_padding=0, groups=1):
        return self.omb.call("conv_transpose2d", [x, w, b], ints=[stride, stride, padding, padding, output_padding, output_padding, 1, 1, groups])
    def conv1d(self, x, w, b, stride=1, pad_left=0, pad_right=0, dilation=1, groups=1):
        return self.omb.call("conv1d", [x, w, b] if b is not None else [x, w], ints=[stride, pad_left, pad_right, dilation, groups])
    def resize2d(self, x, oh, ow, mode=0, align=False): return self.omb.call("resize2d", [x], ints=[oh, ow, mode, 1 if align else 0])
    def erf(self, x): return self.omb.call("erf", [x])
    def exp(self, x): return self.omb.call("exp", [x])
    def sqrt(self, x): return self.omb.call("sqrt", [x])
    def pow(self, x, p): return self.omb.call("pow", [x], floats=[p])
    def where(self, c, a, b): return self.omb.call("where", [self.omb.Tensor.from_numpy(np.asarray(c, np.int32)), a, b])
    def gather(self, data, idx, axis): return self.omb.call("gather", [data, self.omb.Tensor.from_numpy(np.asarray(idx, np.int64))], ints=[axis])
    def ctc_loss(self, lp, targets, ilen, tlen, blank=0, reduction=1, zero_inf=False):
        T = self.omb.Tensor.from_numpy
        return self.omb.call("ctc_loss", [lp, T(np.asarray(targets, np.int32)), T(np.asarray(ilen, np.int32)), T(np.asarray(tlen, np.int32))],
                             ints=[blank, reduction, 1 if zero_inf else 0])
    def avg_pool2d(self, x, k): return self.omb.call("avg_pool2d", [x], ints=[k, k, k, k, 0, 0, 0])
    def running(self, a): return self.omb.Tensor.from_numpy(np.asarray(a, np.float32))
    def running_numpy(self, r): return r.numpy()
    def backward(self, loss): loss.backward()
    def zero_grad(self, params):
        for p in params:
            p.zero_grad()


def load_fixture(group, name):
    """A reference fixture as {tensor name: float32 array} (layout of tools/autograd_oracle.py:22-33 of the reference)."""
    import json
    base = os.path.join(ROOT, "tests", "golden", "reference_testdata", group, name)
    manifest = json.load(open(base + ".json"))
    raw = np.fromfile(base + ".bin", dtype="<f4")
    out = {}
    for k, meta in manifest["tensors"].items():
        n = int(np.prod(meta["shape"])) if meta["shape"] else 1
        out[k] = raw[meta["offset"]: meta["offset"] + n].reshape(meta["shape"]).astype(np.float32)
    return out


def load_fixture_manifest(group, name):
    """The JSON beside a reference fixture (generator version, seed, per-case settings)."""
    import json
    return json.load(open(os.path.join(ROOT, "tests", "golden", "reference_testdata", group, name + ".json")))


def scaled_diff(a, ref):
    """max|a - ref| / max|ref| : the reference tests' metric (tests/OneModel.Tests/Tensors/AutogradModelTests.cs:61-81)."""
    a, ref = np.asarray(a, np.float64), np.asarray(ref, np.float64)
    denom = np.max(np.abs(ref)) if ref.size else 0.0
    return float(np.max(np.abs(a - ref)) / denom) if denom > 0 else float(np.max(np.abs(a - ref)) if a.size else 0.0)


class OracleOptimizer:
    """Optimizer.Step over the oracle's per-tensor update functions (Optimizers.cs:184-219)."""

    def __init__(self, K, kind, params, lr, **kw):
        self.K, self.kind, self.params, self.lr, self.kw, self.t = K, kind, list(params), lr, kw, 0
        self.state = [dict(m=np.zeros(p.shape, np.float32), v=np.zeros(p.shape, np.float32),
                           vmax=np.zeros(p.shape, np.float32), buf=np.zeros(p.shape, np.float32), init=False)
                      for p in self.params]

    def set_lr(self, lr):
        self.lr = lr

    def zero_grad(self):
        for p in self.params:
            p.zero_grad()

    def step(self):
        self.t += 1
        kw = self.kw
        for p, s in zip(self.params, self.state):
            if p.grad is None:
                continue
            p.v = np.ascontiguousarray(p.v, np.float32)
            if self.kind == "sgd":
                self.K.sgd_step(p.v, p.grad, s["buf"], not s["init"], self.lr, kw.get("weight_decay", 0.0),
                                kw.get("momentum", 0.0), kw.get("dampening", 0.0), kw.get("nesterov", False))
                s["init"] = True
            else:
                self.K.adam_step(p.v, p.grad, s["m"], s["v"], s["vmax"], self.t, self.lr, kw.get("beta1", 0.9),
                                 kw.get("beta2", 0.999), kw.get("eps", 1e-8), kw.get("weight_decay", 0.0),
                                 self.kind == "adamw", kw.get("amsgrad", False))


def _oracle_optim(self, kind, params, lr, **kw):
    return OracleOptimizer(self.K, kind, params, lr, **kw)


def _gpu_optim(self, kind, params, lr, **kw):
    O = self.omb.Optimizer
    if kind == "sgd":
        return O.sgd(params, lr, kw.get("momentum", 0.0), kw.get("dampening", 0.0), kw.get("weight_decay", 0.0), kw.get("nesterov", False))
    f = O.adam if kind == "adam" else O.adamw
    return f(params, lr, kw.get("beta1", 0.9), kw.get("beta2", 0.999), kw.get("eps", 1e-8), kw.get("weight_decay", 0.0), kw.get("amsgrad", False))


OracleBackend.optimizer = _oracle_optim
GpuBackend.optimizer = _gpu_optim
OracleBackend.clip_norm = lambda self, params, max_norm, infinity=False: float(self.K.clip_norm([p.meta.grad for p in params if p.grad is not None], max_norm, infinity))
GpuBackend.clip_norm = lambda self, params, max_norm, infinity=False: self.omb.clip_norm(params, max_norm, infinity)


def _oracle_set_grad(self, t, g):
    t.meta.grad = np.array(g, np.float32)


def _gpu_set_grad(self, t, g):
    # Seeds the leaf's gradient through the engine: backward of (t * g).sum() from a zeroed gradient is exactly g.
    t.clear_grad()
    w = self.omb.Tensor.from_numpy(np.asarray(g, np.float32))
    self.omb.call("sum", [self.omb.call("mul", [t, w])]).backward()


OracleBackend.set_grad = _oracle_set_grad
GpuBackend.set_grad = _gpu_set_grad
