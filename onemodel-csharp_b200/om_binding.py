"""ctypes binding of libonemodel_b200.so (the C ABI) and libonemodel_b200_host.so (the C++ mirror of the
reference's Tensor/autograd/optimizer API). Used by the tests, the smoke entry and the bench.

There is no CPU path: loading fails loudly when a library is missing, and creating a context fails when no
sm_100 device is visible.
"""
import ctypes as C
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
KERNEL_LIB = os.path.join(_HERE, "libonemodel_b200.so")
HOST_LIB = os.path.join(_HERE, "libonemodel_b200_host.so")

OM_F32, OM_I32, OM_I64 = 0, 1, 2
OM_TF32, OM_BF16_OPERANDS, OM_CHECKED, OM_PAIR_TILES, OM_TWO_STREAMS, OM_SEQ_KERNELS, OM_OVERLAP_LAUNCHES, OM_PERSISTENT_TILES = 1, 2, 4, 8, 16, 32, 64, 128
_NP2OM = {np.dtype("float32"): OM_F32, np.dtype("int32"): OM_I32, np.dtype("int64"): OM_I64}
_OM2NP = {OM_F32: np.float32, OM_I32: np.int32, OM_I64: np.int64}

UNARY = dict(none=0, relu=1, gelu_erf=2, gelu_tanh=3, sigmoid=4, tanh=5, neg=6, exp=7, sqrt=8, erf=9)
BINARY = dict(add=0, sub=1, mul=2, div=3)


class OmError(RuntimeError):
    def __init__(self, status, message):
        super().__init__(f"[status {status}] {message}")
        self.status = status


class ShapeError(OmError):
    pass


class IndexOutOfRange(OmError):
    pass


class TensorVersionError(OmError):
    """A tensor saved for the backward pass was written in place before the pass read it (TensorVersionException)."""


class InvalidOperation(OmError):
    """InvalidOperationException of the reference (an optimizer handed a kind of gradient it does not take, for instance)."""


class NotSupported(OmError):
    """NotSupportedException of the reference (Sgd with momentum or weight decay on a row-sparse gradient)."""


_kernel = None
_host = None


def kernel_lib():
    """The C-ABI library. Raises if it has not been built."""
    global _kernel
    if _kernel is None:
        if not os.path.exists(KERNEL_LIB):
            raise RuntimeError(f"{KERNEL_LIB} is missing: run __graft_entry__.build() (there is no fallback path)")
        _kernel = C.CDLL(KERNEL_LIB, mode=C.RTLD_GLOBAL)
    return _kernel


def host_lib():
    global _host
    if _host is None:
        kernel_lib()
        if not os.path.exists(HOST_LIB):
            raise RuntimeError(f"{HOST_LIB} is missing: run __graft_entry__.build()")
        _host = C.CDLL(HOST_LIB, mode=C.RTLD_GLOBAL)
        _host.omh_tensor_data.restype = C.c_void_p
        _host.omh_module_free.argtypes = [C.c_void_p]
        _host.omh_schedule_lr_at.restype = C.c_float
        _host.omh_schedule_lr_at.argtypes = [C.c_void_p, C.c_int64]
        _host.omh_schedule_free.argtypes = [C.c_void_p]
        _host.omh_schedule_cos.restype = C.c_double
        _host.omh_schedule_cos.argtypes = [C.c_double]
    return _host


def _raise(status, message, host=False):
    code = status - 100 if status >= 100 else status
    if host and status == 9:
        raise InvalidOperation(code, message)
    if host and status == 12:
        raise NotSupported(code, message)
    if code == 1:
        raise ShapeError(code, message)
    if code == 2:
        raise IndexOutOfRange(code, message)
    if code == 11:
        raise TensorVersionError(code, message)
    raise OmError(code, message)


class Context:
    """One om_ctx: a device, a stream and a memory pool. `ctx.call("om_xxx", ...)` checks the status."""

    def __init__(self, device=0, flags=0):
        self.lib = kernel_lib()
        self.host = host_lib()
        self.handle = C.c_void_p()
        st = self.host.omh_init(C.c_int32(device), C.c_uint32(flags), C.byref(self.handle))
        if st != 0:
            buf = C.create_string_buffer(512)
            self.host.omh_last_error(buf, 512)
            _raise(st, buf.value.decode())
        self.flags = flags

    def make_current(self):
        self.host.omh_set_current(self.handle)

    def set_flags(self, flags):
        self.call("om_ctx_set_flags", self.handle, C.c_uint32(flags))
        self.flags = flags

    def last_error(self):
        buf = C.create_string_buffer(512)
        self.lib.om_last_error(self.handle, buf, C.c_size_t(512))
        return buf.value.decode()

    def call(self, name, *args):
        st = getattr(self.lib, name)(*args)
        if st != 0:
            _raise(st, self.last_error())

    def sync(self):
        self.call("om_sync", self.handle)

    def close(self):
        if self.handle:
            self.lib.om_ctx_destroy(self.handle)
            self.handle = C.c_void_p()

    # ---- raw device arrays for per-entry-point tests ----
    def to_device(self, array):
        a = np.ascontiguousarray(array)
        return DeviceArray(self, a.shape, a.dtype, a)

    def empty(self, shape, dtype=np.float32):
        return DeviceArray(self, tuple(np.atleast_1d(shape)) if not isinstance(shape, tuple) else shape, np.dtype(dtype))

    def zeros(self, shape, dtype=np.float32):
        d = self.empty(shape, dtype)
        self.call("om_memset", self.handle, d.ptr, C.c_int32(0), C.c_size_t(d.nbytes))
        return d


class DeviceArray:
    def __init__(self, ctx, shape, dtype, host=None):
        self.ctx, self.shape, self.dtype = ctx, tuple(int(s) for s in shape), np.dtype(dtype)
        self.size = int(np.prod(self.shape)) if len(self.shape) else 1
        self.nbytes = self.size * self.dtype.itemsize
        self.ptr = C.c_void_p()
        ctx.call("om_alloc", ctx.handle, C.c_size_t(max(self.nbytes, 4)), C.c_int32(0), C.byref(self.ptr))
        if host is not None and self.nbytes:
            h = np.ascontiguousarray(host, dtype=self.dtype)
            ctx.call("om_memcpy_h2d", ctx.handle, self.ptr, h.ctypes.data_as(C.c_void_p), C.c_size_t(self.nbytes))
            ctx.sync()

    def numpy(self):
        out = np.empty(self.shape, dtype=self.dtype)
        if self.nbytes:
            self.ctx.call("om_memcpy_d2h", self.ctx.handle, out.ctypes.data_as(C.c_void_p), self.ptr, C.c_size_t(self.nbytes))
        return out

    def __del__(self):
        try:
            if self.ptr and self.ctx.handle:
                self.ctx.lib.om_free(self.ctx.handle, self.ptr)
        except Exception:
            pass


def i32(v):
    return C.c_int32(int(v))


def i64(v):
    return C.c_int64(int(v))


def f32(v):
    return C.c_float(float(v))


def int_array(values, ctype=C.c_int32):
    return (ctype * max(len(values), 1))(*[int(v) for v in values])


# ---------------------------------------------------------------------------------------------------------------------
# Host mirror: Tensor with autograd


def _hcheck(st):
    if st != 0:
        buf = C.create_string_buffer(512)
        host_lib().omh_last_error(buf, C.c_size_t(512))
        _raise(st, buf.value.decode(), host=True)


class Tensor:
    """Handle to an omh::Tensor (device memory, autograd meta). Mirrors RecursiveAI.OneModel.Tensors.Tensor."""

    def __init__(self, handle):
        self.h = handle

    @staticmethod
    def from_numpy(a, requires_grad=False):
        a = np.ascontiguousarray(a)
        if a.dtype not in _NP2OM:
            a = a.astype(np.float32)
        h = C.c_void_p()
        shape = int_array(a.shape)
        _hcheck(host_lib().omh_tensor_from_host(i32(_NP2OM[a.dtype]), i32(a.ndim), shape, a.ctypes.data_as(C.c_void_p), C.byref(h)))
        t = Tensor(h)
        if requires_grad:
            t.requires_grad = True
        return t

    def __del__(self):
        try:
            if self.h:
                host_lib().omh_tensor_free(self.h)
        except Exception:
            pass

    def _info(self):
        dt, rank = C.c_int32(), C.c_int32()
        shape = (C.c_int32 * 8)()
        strides = (C.c_int64 * 8)()
        _hcheck(host_lib().omh_tensor_info(self.h, C.byref(dt), C.byref(rank), shape, strides))
        return dt.value, tuple(shape[: rank.value]), tuple(strides[: rank.value])

    @property
    def shape(self):
        return self._info()[1]

    @property
    def dtype(self):
        return _OM2NP[self._info()[0]]

    def numpy(self):
        dt, shape, _ = self._info()
        out = np.empty(shape, dtype=_OM2NP[dt])
        if out.size:
            _hcheck(host_lib().omh_tensor_to_host(self.h, out.ctypes.data_as(C.c_void_p)))
        return out

    def item(self):
        return float(self.numpy().reshape(-1)[0])

    def copy_from(self, a):
        a = np.ascontiguousarray(a, dtype=self.dtype)
        _hcheck(host_lib().omh_tensor_copy_from_host(self.h, a.ctypes.data_as(C.c_void_p)))

    @property
    def data_ptr(self):
        return host_lib().omh_tensor_data(self.h)

    @property
    def requires_grad(self):
        return bool(host_lib().omh_tensor_requires_grad(self.h))

    @requires_grad.setter
    def requires_grad(self, on):
        _hcheck(host_lib().omh_tensor_set_requires_grad(self.h, i32(1 if on else 0)))

    @property
    def grad(self):
        h = C.c_void_p()
        _hcheck(host_lib().omh_tensor_grad(self.h, C.byref(h)))
        return Tensor(h) if h else None

    @property
    def sparse_grad(self):
        """The row-sparse gradient a sparse embedding lookup left on this leaf (Tensor.SparseGrad of the reference), or None."""
        n, rows, values = C.c_int32(), C.c_void_p(), C.c_void_p()
        _hcheck(host_lib().omh_tensor_sparse_grad(self.h, C.byref(n), C.byref(rows), C.byref(values)))
        return RowSparseGradient(self, n.value, Tensor(rows), Tensor(values)) if n.value else None

    def zero_grad(self):
        _hcheck(host_lib().omh_tensor_zero_grad(self.h))

    def clear_grad(self):
        _hcheck(host_lib().omh_tensor_clear_grad(self.h))

    def backward(self, gradient=None, retain_graph=False):
        _hcheck(host_lib().omh_backward(self.h, gradient.h if gradient is not None else None, i32(1 if retain_graph else 0)))

    # views
    def reshape(self, *shape):
        return call("reshape", [self], ints=_flat(shape))

    def permute(self, *axes):
        return call("permute", [self], ints=_flat(axes))

    def t(self):
        return call("t", [self])

    def slice(self, axis, start, end, step=1):
        return call("slice", [self], ints=[axis, start, end, step])

    def select(self, axis, index):
        return call("select", [self], ints=[axis, index])

    def expand(self, *shape):
        return call("expand", [self], ints=_flat(shape))

    def flip(self, axis):
        return call("flip", [self], ints=[axis])

    def clone(self):
        return call("clone", [self])

    def detach(self):
        return call("detach", [self])

    def __add__(self, o):
        return call("add", [self, o])

    def __sub__(self, o):
        return call("sub", [self, o])

    def __mul__(self, o):
        return call("mul", [self, o])

    def __truediv__(self, o):
        return call("div", [self, o])

    def __neg__(self):
        return call("neg", [self])


def _flat(xs):
    if len(xs) == 1 and isinstance(xs[0], (tuple, list)):
        return list(xs[0])
    return list(xs)


def call(op, inputs, ints=(), floats=()):
    """Ops.* by name (see omh_call in host/capi.cpp): returns a Tensor."""
    n = len(inputs)
    arr = (C.c_void_p * max(n, 1))(*[(t.h if t is not None else None) for t in inputs])
    ia = (C.c_int64 * max(len(ints), 1))(*[int(v) for v in ints])
    fa = (C.c_double * max(len(floats), 1))(*[float(v) for v in floats])
    out = C.c_void_p()
    _hcheck(host_lib().omh_call(op.encode(), i32(n), arr, i32(len(ints)), ia, i32(len(floats)), fa, C.byref(out)))
    return Tensor(out)


class no_grad:
    def __enter__(self):
        host_lib().omh_no_grad(i32(1))

    def __exit__(self, *a):
        host_lib().omh_no_grad(i32(0))


class RowSparseGradient:
    """RowSparseGradient of the reference (RowSparseGradient.cs:14-120): `rows` strictly ascending Int32 [row_count], `values`
    float32 [row_count, width] (a writable view of the gradient's storage), to_dense() and add_to(dense)."""

    def __init__(self, owner, row_count, rows, values):
        self.owner, self.row_count, self.rows, self.values = owner, row_count, rows, values

    @property
    def byte_count(self):
        return self.row_count * (self.values.shape[1] * 4 + 4)

    def to_dense(self):
        out = C.c_void_p()
        _hcheck(host_lib().omh_tensor_sparse_grad_to_dense(self.owner.h, None, C.byref(out)))
        return Tensor(out)

    def add_to(self, dense):
        _hcheck(host_lib().omh_tensor_sparse_grad_to_dense(self.owner.h, dense.h, None))


class Optimizer:
    """Sgd / Adam / AdamW / SparseAdam of RecursiveAI.OneModel.Training (Optimizers.cs)."""

    def __init__(self, kind, params, floats, ints):
        self.params = list(params)
        arr = (C.c_void_p * len(self.params))(*[p.h for p in self.params])
        fa = (C.c_double * len(floats))(*floats)
        ia = (C.c_int64 * max(len(ints), 1))(*ints)
        self.h = C.c_void_p()
        _hcheck(host_lib().omh_optim_create(i32(kind), i32(len(self.params)), arr, fa, ia, C.byref(self.h)))

    @staticmethod
    def sgd(params, lr, momentum=0.0, dampening=0.0, weight_decay=0.0, nesterov=False):
        return Optimizer(0, params, [lr, momentum, dampening, weight_decay], [1 if nesterov else 0])

    @staticmethod
    def adam(params, lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.0, amsgrad=False):
        return Optimizer(1, params, [lr, beta1, beta2, eps, weight_decay], [1 if amsgrad else 0])

    @staticmethod
    def adamw(params, lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.01, amsgrad=False):
        return Optimizer(2, params, [lr, beta1, beta2, eps, weight_decay], [1 if amsgrad else 0])

    @staticmethod
    def sparse_adam(params, lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8):
        return Optimizer(3, params, [lr, beta1, beta2, eps], [0])

    def step(self):
        _hcheck(host_lib().omh_optim_step(self.h))

    def zero_grad(self):
        _hcheck(host_lib().omh_optim_zero_grad(self.h))

    def set_lr(self, lr):
        host_lib().omh_optim_set_lr(self.h, C.c_float(lr))

    def __del__(self):
        try:
            if self.h:
                host_lib().omh_optim_free(self.h)
        except Exception:
            pass


class Generator:
    """The SplitMix64 state the reference's module constructors draw initial weights from (Generator.cs:10-48)."""

    def __init__(self, seed):
        self.state = C.c_uint64(seed)


class Module:
    """NnModule of RecursiveAI.OneModel.Training over host/nn.cpp: layers by kind, Sequential, Train/Eval, Freeze/Unfreeze,
    StateDict / LoadStateDict, ZeroGrad (NnModule.cs, Layers.cs, Recurrent.cs)."""

    STATE, PARAMETERS, TRAINABLE, BUFFERS = 0, 1, 2, 3

    def __init__(self, kind, generator=None, ints=(), floats=()):
        ia = (C.c_int64 * max(len(ints), 1))(*[int(v) for v in ints])
        fa = (C.c_double * max(len(floats), 1))(*[float(v) for v in floats])
        self.h = C.c_void_p()
        state = C.byref(generator.state) if generator is not None else None
        _hcheck(host_lib().omh_module_create(kind.encode(), state, i32(len(ints)), ia, i32(len(floats)), fa, C.byref(self.h)))

    @staticmethod
    def sequential(*layers):
        arr = (C.c_void_p * max(len(layers), 1))(*[m.h for m in layers])
        seq = Module.__new__(Module)
        seq.h = C.c_void_p()
        _hcheck(host_lib().omh_sequential_create(i32(len(layers)), arr, C.byref(seq.h)))
        seq._layers = layers                     # their (now empty) handles are freed with them
        return seq

    def __call__(self, x):
        out = C.c_void_p()
        _hcheck(host_lib().omh_module_forward(self.h, x.h, C.byref(out)))
        return Tensor(out)

    def forward_lengths(self, x, lengths):
        """A recurrent stack over rows padded to a common length (Recurrent.Forward(input, lengths) of the reference)."""
        arr = (C.c_int32 * max(len(lengths), 1))(*[int(v) for v in lengths])
        out = C.c_void_p()
        _hcheck(host_lib().omh_module_forward_lengths(self.h, x.h, i32(len(lengths)), arr, C.byref(out)))
        return Tensor(out)

    def train(self, on=True):
        _hcheck(host_lib().omh_module_train(self.h, i32(1 if on else 0)))
        return self

    def eval(self):
        return self.train(False)

    def zero_grad(self):
        _hcheck(host_lib().omh_module_zero_grad(self.h))

    def entries(self, which=0):
        """[(name, Tensor)] of the state dict (0), the parameters (1), the trainable parameters (2) or the buffers (3)."""
        n = C.c_int32()
        _hcheck(host_lib().omh_module_count(self.h, i32(which), C.byref(n)))
        out = []
        for i in range(n.value):
            name, t = C.create_string_buffer(256), C.c_void_p()
            _hcheck(host_lib().omh_module_entry(self.h, i32(which), i32(i), name, i32(256), C.byref(t)))
            out.append((name.value.decode(), Tensor(t)))
        return out

    def state_dict(self): return self.entries(self.STATE)
    def named_parameters(self): return self.entries(self.PARAMETERS)
    def parameters(self): return [t for _, t in self.entries(self.PARAMETERS)]
    def trainable_parameters(self): return [t for _, t in self.entries(self.TRAINABLE)]
    def named_trainable_parameters(self): return self.entries(self.TRAINABLE)

    def _set_frozen(self, name, frozen):
        changed = C.c_int32()
        _hcheck(host_lib().omh_module_set_frozen(self.h, name.encode() if name else None, i32(1 if frozen else 0), C.byref(changed)))
        return changed.value

    def freeze(self, name_or_prefix=None): return self._set_frozen(name_or_prefix, True)
    def unfreeze(self, name_or_prefix=None): return self._set_frozen(name_or_prefix, False)

    def is_frozen(self, name):
        out = C.c_int32()
        _hcheck(host_lib().omh_module_is_frozen(self.h, name.encode(), C.byref(out)))
        return bool(out.value)

    def load_state_dict(self, state):
        state = list(state)
        names = (C.c_char_p * max(len(state), 1))(*[n.encode() for n, _ in state])
        arr = (C.c_void_p * max(len(state), 1))(*[t.h for _, t in state])
        _hcheck(host_lib().omh_module_load_state(self.h, i32(len(state)), names, arr))

    def __del__(self):
        try:
            if self.h:
                host_lib().omh_module_free(self.h)
        except Exception:
            pass


class LrSchedule:
    """ConstantLr / StepLr / CosineLr / WarmupLr / WarmupCosineLr / OneCycleLr of RecursiveAI.OneModel.Training
    (Schedules.cs:151-422): lr_at(step) is the rate of the optimizer step with that index, 0 for the first."""

    def __init__(self, kind, floats, ints, after=None):
        fa = (C.c_float * max(len(floats), 1))(*floats)
        ia = (C.c_int64 * max(len(ints), 1))(*[int(v) for v in ints])
        self.h = C.c_void_p()
        self._after = after                      # keeps the wrapped schedule's handle alive on this side too
        _hcheck(host_lib().omh_schedule_create(i32(kind), fa, ia, after.h if after is not None else None, C.byref(self.h)))

    @staticmethod
    def constant(lr): return LrSchedule(0, [lr], [])
    @staticmethod
    def step(base_lr, step_size, gamma=0.1): return LrSchedule(1, [base_lr, gamma], [step_size])
    @staticmethod
    def cosine(base_lr, total_steps, min_lr=0.0): return LrSchedule(2, [base_lr, min_lr], [total_steps])
    @staticmethod
    def warmup(after, warmup_steps, start_factor=0.0): return LrSchedule(3, [start_factor], [warmup_steps], after)
    @staticmethod
    def warmup_cosine(base_lr, warmup_steps, total_steps, floor_fraction=0.0):
        return LrSchedule(4, [base_lr, floor_fraction], [warmup_steps, total_steps])
    @staticmethod
    def one_cycle(max_lr, total_steps, pct_start=0.3, div_factor=25.0, final_div_factor=1e4):
        return LrSchedule(5, [max_lr, pct_start, div_factor, final_div_factor], [total_steps])

    @staticmethod
    def cos(t):
        """cos(pi t) on [0, 1] by the platform-independent series (LrSchedule.Cos, Schedules.cs:165-203)."""
        return host_lib().omh_schedule_cos(float(t))

    def lr_at(self, step):
        return float(host_lib().omh_schedule_lr_at(self.h, int(step)))

    def apply(self, optimizer, step):
        optimizer.set_lr(self.lr_at(step))

    def __del__(self):
        try:
            if self.h:
                host_lib().omh_schedule_free(self.h)
        except Exception:
            pass


def clip_norm(params, max_norm, infinity=False):
    arr = (C.c_void_p * len(params))(*[p.h for p in params])
    total = C.c_float()
    _hcheck(host_lib().omh_clip_norm(i32(len(params)), arr, C.c_float(max_norm), i32(1 if infinity else 0), C.byref(total)))
    return total.value


def clip_value(params, clip):
    arr = (C.c_void_p * len(params))(*[p.h for p in params])
    _hcheck(host_lib().omh_clip_value(i32(len(params)), arr, C.c_float(clip)))


class Trainer:
    """A benchmark-configuration training loop held on the device (host/trainer.cpp).

    kind 'mlp': cfg = [batch, in, hidden..., out]; kind 'mlm': cfg = [batch, seq, layers, width, heads, ff, vocab, rows].
    step(inputs) takes the host batch (numpy arrays) and returns the loss: the call a user makes."""

    KINDS = {"mlp": 1, "cnn": 2, "mlm": 3, "crnn": 4}

    def __init__(self, kind, cfg, lr, weight_decay=0.01, clip_norm=0.0, seed=0):
        self.h = C.c_void_p()
        cfg_a = (C.c_int64 * len(cfg))(*[int(v) for v in cfg])
        hyper = (C.c_double * 3)(lr, weight_decay, clip_norm)
        self._check(host_lib().omh_trainer_create(i32(self.KINDS[kind]), cfg_a, i32(len(cfg)), C.c_uint64(seed), hyper, C.byref(self.h)))
        self.kind, self.cfg = kind, list(cfg)
        host_lib().omh_trainer_input_bytes.restype = C.c_int64
        host_lib().omh_trainer_steps_done.restype = C.c_int64

    @staticmethod
    def _check(st):
        if st != 0:
            buf = C.create_string_buffer(512)
            host_lib().omh_trainer_last_error(buf, C.c_size_t(512))
            _raise(st, buf.value.decode())

    def named_parameters(self):
        out = []
        n = host_lib().omh_trainer_param_count(self.h)
        for i in range(n):
            name = C.create_string_buffer(128)
            rank = C.c_int32()
            shape = (C.c_int32 * 8)()
            host_lib().omh_trainer_param_info(self.h, i32(i), name, C.c_size_t(128), C.byref(rank), shape)
            out.append((name.value.decode(), tuple(shape[: rank.value])))
        return out

    def get_param(self, i, shape):
        a = np.empty(shape, np.float32)
        self._check(host_lib().omh_trainer_get_param(self.h, i32(i), a.ctypes.data_as(C.c_void_p)))
        return a

    def set_param(self, i, a):
        a = np.ascontiguousarray(a, np.float32)
        self._check(host_lib().omh_trainer_set_param(self.h, i32(i), a.ctypes.data_as(C.c_void_p)))

    def get_grad(self, i, shape):
        a = np.empty(shape, np.float32)
        self._check(host_lib().omh_trainer_get_grad(self.h, i32(i), a.ctypes.data_as(C.c_void_p)))
        return a

    def state_dict(self):
        return {name: self.get_param(i, shape) for i, (name, shape) in enumerate(self.named_parameters())}

    # ---- what a checkpoint reads and writes (checkpoint.py) --------------------------------------------------------
    _NP = {0: np.float32, 1: np.int32, 2: np.int64}
    _DT = {0: "f32", 1: "i32", 2: "i64"}

    def _entries(self, count_fn, info_fn):
        out = []
        for i in range(count_fn(self.h)):
            name = C.create_string_buffer(128)
            dtype, rank = C.c_int32(), C.c_int32()
            shape = (C.c_int32 * 8)()
            info_fn(self.h, i32(i), name, C.c_size_t(128), C.byref(dtype), C.byref(rank), shape)
            out.append((name.value.decode(), self._DT[dtype.value], tuple(shape[: rank.value])))
        return out

    def model_state_entries(self):
        """(name, dtype, shape) of the model's parameters and buffers in the reference's state order."""
        return self._entries(host_lib().omh_trainer_model_state_count, host_lib().omh_trainer_model_state_info)

    def optimizer_state_entries(self):
        return self._entries(host_lib().omh_trainer_state_count, host_lib().omh_trainer_state_info)

    def _get(self, fn, entry, i):
        a = np.empty(entry[2], {"f32": np.float32, "i32": np.int32, "i64": np.int64}[entry[1]])
        self._check(fn(self.h, i32(i), a.ctypes.data_as(C.c_void_p)))
        return a

    def _set(self, fn, entry, i, a):
        a = np.ascontiguousarray(a, {"f32": np.float32, "i32": np.int32, "i64": np.int64}[entry[1]])
        assert tuple(a.shape) == tuple(entry[2]), (a.shape, entry)
        self._check(fn(self.h, i32(i), a.ctypes.data_as(C.c_void_p)))

    def model_state_get(self, i):
        return self._get(host_lib().omh_trainer_model_state_get, self.model_state_entries()[i], i)

    def model_state_set(self, i, a):
        self._set(host_lib().omh_trainer_model_state_set, self.model_state_entries()[i], i, a)

    def optimizer_state_get(self, i):
        return self._get(host_lib().omh_trainer_state_get, self.optimizer_state_entries()[i], i)

    def optimizer_state_set(self, i, a):
        self._set(host_lib().omh_trainer_state_set, self.optimizer_state_entries()[i], i, a)

    def optimizer_kind(self):
        buf = C.create_string_buffer(32)
        host_lib().omh_trainer_opt_kind(self.h, buf, C.c_size_t(32))
        return buf.value.decode()

    def hyper_parameters(self):
        out = []
        for i in range(host_lib().omh_trainer_hyper_count(self.h)):
            name, v = C.create_string_buffer(64), C.c_float()
            host_lib().omh_trainer_hyper_info(self.h, i32(i), name, C.c_size_t(64), C.byref(v))
            out.append((name.value.decode(), np.float32(v.value)))
        return out

    def steps_done(self):
        return int(host_lib().omh_trainer_steps_done(self.h))

    def restore(self, step, lr, weight_decay):
        self._check(host_lib().omh_trainer_restore(self.h, C.c_int64(step), C.c_float(lr), C.c_float(weight_decay)))

    def input_bytes(self):
        n = host_lib().omh_trainer_input_count(self.h)
        return [int(host_lib().omh_trainer_input_bytes(self.h, i32(i))) for i in range(n)]

    def _ptrs(self, inputs):
        self._keep = [np.ascontiguousarray(a) for a in inputs]
        for a, nbytes in zip(self._keep, self.input_bytes()):
            assert a.nbytes == nbytes, (a.shape, a.dtype, nbytes)
        return (C.c_void_p * len(self._keep))(*[a.ctypes.data for a in self._keep])

    def step(self, inputs):
        loss = C.c_float()
        self._check(host_lib().omh_trainer_step(self.h, self._ptrs(inputs), C.byref(loss)))
        return loss.value

    def step_ptrs(self, ptr_table, loss_ref):
        """step() with a prebuilt table of (pinned) host pointers: no Python-side allocation in the timed region."""
        self._check(host_lib().omh_trainer_step(self.h, ptr_table, loss_ref))

    def load_inputs(self, inputs):
        self._check(host_lib().omh_trainer_load_inputs(self.h, self._ptrs(inputs)))

    def step_resident(self):
        self._check(host_lib().omh_trainer_step_resident(self.h))

    def read_loss(self):
        loss = C.c_float()
        self._check(host_lib().omh_trainer_read_loss(self.h, C.byref(loss)))
        return loss.value

    def sync(self):
        self._check(host_lib().omh_trainer_sync(self.h))

    def enable_graph(self):
        self._check(host_lib().omh_trainer_enable_graph(self.h))

    def dp_init(self, id128, rank, world, global_rows):
        buf = (C.c_uint8 * 128).from_buffer_copy(bytes(id128))
        self._check(host_lib().omh_trainer_dp_init(self.h, buf, i32(rank), i32(world), C.c_int64(global_rows)))

    def prefetch_depth(self, depth):
        """Sizes the ring of batches staged ahead of their step (DataLoaderOptions.Prefetch of the reference)."""
        self._check(host_lib().omh_trainer_prefetch_depth(self.h, i32(depth)))

    def prefetch(self, inputs):
        """Stages the next batch: copied to a pinned ring slot and sent to the device on the copy stream, under the steps
        already queued. The arrays may be reused when this returns."""
        self._check(host_lib().omh_trainer_prefetch(self.h, self._ptrs(inputs)))

    def prefetch_ptrs(self, ptr_table):
        self._check(host_lib().omh_trainer_prefetch(self.h, ptr_table))

    def step_prefetched(self, loss_ref=None):
        """One step on the oldest staged batch; returns the loss (or writes it through loss_ref)."""
        if loss_ref is not None:
            self._check(host_lib().omh_trainer_step_prefetched(self.h, loss_ref))
            return None
        loss = C.c_float()
        self._check(host_lib().omh_trainer_step_prefetched(self.h, C.byref(loss)))
        return loss.value

    def set_dp_timeout_ms(self, ms):
        self._check(host_lib().omh_trainer_set_dp_timeout_ms(self.h, i32(ms)))

    def close(self):
        if self.h:
            host_lib().omh_trainer_free(self.h)
            self.h = C.c_void_p()
