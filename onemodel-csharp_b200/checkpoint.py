"""Training checkpoints in the reference's file format, written from and restored into device state.

The format is the one `RecursiveAI.OneModel.Training.Checkpoint` reads and writes (src/OneModel.Training/Checkpoint.cs,
docs/training.md section 6 of the reference): a 64-byte little-endian header with the magic ``ONEMCKPT``, a compact UTF-8 JSON
manifest in a fixed field order, zero padding to a multiple of 64, then the data region with every tensor starting on a
multiple of 64. Model tensors come first, in the state order (a module's parameters, then its buffers, then each child),
then the optimizer's state tensors in its own order; hyper-parameters are stored as the unsigned integer of their float
bit pattern. A file saved here loads in the reference and the other way round, as long as both sides hold the same
model and optimizer.

A checkpoint is untrusted input. `load` checks, in the reference's order and before it changes anything: the header
(`BadHeader`), the manifest (`BadManifest`), every tensor entry against the target's names, types and shapes
(`Mismatch`; the shape is compared before any size is computed from it), then offsets and lengths against the data
region (`BadTensor`). Only `CheckpointError` leaves this module for a malformed file.

The target is anything with the small interface of `HostState` below; `TrainerState` adapts a device-resident
`om_binding.Trainer`, whose parameters, buffers, optimizer moments, step count and learning rate live in HBM and cross to
the host only here.
"""
import io
import json
import struct

import numpy as np

MAGIC = b"ONEMCKPT"
HEADER_SIZE = 64
MAX_MANIFEST = 256 * 1024 * 1024
MAX_DEPTH = 32
_DTYPES = {"f32": np.dtype("<f4"), "i32": np.dtype("<i4"), "i64": np.dtype("<i8")}
_INT64_MIN, _INT64_MAX = -(1 << 63), (1 << 63) - 1


class CheckpointError(Exception):
    """A rejected checkpoint; `kind` is one of BadHeader, BadManifest, BadTensor, Mismatch (Checkpoint.cs:12-24)."""

    def __init__(self, kind, message):
        super().__init__(f"{kind}: {message}")
        self.kind = kind


class HostState:
    """A training state held in numpy arrays: the smallest target `save` and `load` work on.

    model: list of (name, array); optimizer (optional): kind, step, hyper = list of (name, float32), state = list of
    (name, array), fixed = names of the hyper-parameters that must equal the saved ones (momentum, betas, epsilon ...).
    """

    def __init__(self, model, kind=None, step=0, hyper=(), state=(), fixed=()):
        self.model = [(n, np.ascontiguousarray(a)) for n, a in model]
        self.kind, self.step = kind, int(step)
        self.hyper = [(n, np.float32(v)) for n, v in hyper]
        self.state = [(n, np.ascontiguousarray(a)) for n, a in state]
        self.fixed = tuple(fixed)

    def has_optimizer(self):
        return self.kind is not None

    def model_entries(self):
        return [(n, _dtype_name(a.dtype), tuple(a.shape)) for n, a in self.model]

    def state_entries(self):
        return [(n, _dtype_name(a.dtype), tuple(a.shape)) for n, a in self.state]

    def read_model(self, i):
        return self.model[i][1]

    def write_model(self, i, a):
        self.model[i][1][...] = a

    def read_state(self, i):
        return self.state[i][1]

    def write_state(self, i, a):
        self.state[i][1][...] = a

    def hyper_parameters(self):
        return list(self.hyper)

    def check_hyper(self, values):
        _check_fixed(self.hyper, self.fixed, values)

    def restore(self, step, values):
        self.step = int(step)
        self.hyper = [(n, np.float32(values[n])) if n in ("lr", "weight_decay") else (n, v) for n, v in self.hyper]


class TrainerState:
    """Adapts a device-resident `om_binding.Trainer` (host/trainer.cpp): every read and write is one device copy."""

    _FIXED = {"sgd": ("momentum", "dampening", "nesterov"), "adam": ("beta1", "beta2", "epsilon", "amsgrad"),
              "adamw": ("beta1", "beta2", "epsilon", "amsgrad"), "sparseadam": ("beta1", "beta2", "epsilon")}

    def __init__(self, trainer):
        self.t = trainer

    def has_optimizer(self):
        return True

    @property
    def kind(self):
        return self.t.optimizer_kind()

    @property
    def step(self):
        return self.t.steps_done()

    def model_entries(self):
        return self.t.model_state_entries()

    def state_entries(self):
        return self.t.optimizer_state_entries()

    def read_model(self, i):
        return self.t.model_state_get(i)

    def write_model(self, i, a):
        self.t.model_state_set(i, a)

    def read_state(self, i):
        return self.t.optimizer_state_get(i)

    def write_state(self, i, a):
        self.t.optimizer_state_set(i, a)

    def hyper_parameters(self):
        return self.t.hyper_parameters()

    def check_hyper(self, values):
        _check_fixed(self.hyper_parameters(), self._FIXED[self.kind], values)

    def restore(self, step, values):
        self.t.restore(step, float(values["lr"]), float(values["weight_decay"]))


def _dtype_name(dt):
    for name, d in _DTYPES.items():
        if np.dtype(dt) == d:
            return name
    raise TypeError(f"a checkpoint holds float32, int32 or int64 tensors, not {dt}")


def _check_fixed(hyper, fixed, values):
    """Optimizers.cs:321-332, 470-481: the fixed settings must equal the saved ones bit for bit as floats; the rates must be finite and not negative."""
    mine = dict(hyper)
    for n in fixed:
        a, b = np.float32(values[n]), np.float32(mine[n])
        same = (a != 0) == (b != 0) if n in ("nesterov", "amsgrad") else a == b
        if not same:
            raise CheckpointError("Mismatch", f"The saved {n} setting differs from this optimizer's.")
    for n in ("lr", "weight_decay"):
        v = np.float32(values[n])
        if not np.isfinite(v) or v < 0:
            raise CheckpointError("Mismatch", f"The saved {n} is not a finite, non-negative number.")


def _float_bits(v):
    return int(np.float32(v).view(np.uint32))


def _bits_float(bits):
    return np.uint32(bits).view(np.float32)


def _json_string(s):
    return json.dumps(s, ensure_ascii=True)


def _tensor_json(name, dtype, shape, offset, length):
    dims = ",".join(str(int(d)) for d in shape)
    return f'{{"name":{_json_string(name)},"dtype":"{dtype}","shape":[{dims}],"offset":{offset},"length":{length}}}'


def _layout(entries, start):
    """Offsets from the start of the data region, each a multiple of 64 (Checkpoint.cs writer)."""
    out, at = [], start
    for name, dtype, shape in entries:
        length = int(np.prod(shape, dtype=np.int64)) * _DTYPES[dtype].itemsize if len(shape) else _DTYPES[dtype].itemsize
        out.append((name, dtype, shape, at, length))
        at = (at + length + 63) // 64 * 64
    return out, at


def save(stream, target, optimizer=True, extra=None):
    """Writes `target` to a writable binary stream; the same state always writes the same bytes.

    optimizer: also store the optimizer's kind, step count, hyper-parameters and state tensors.
    extra: integers the caller wants back at load time (for example the sample counter), stored sorted by key.
    """
    model, at = _layout(target.model_entries(), 0)
    with_opt = optimizer and target.has_optimizer()
    state = []
    if with_opt:
        state, at = _layout(target.state_entries(), at)
    all_entries = model + state
    data_length = at  # the cursor after the last tensor, rounded up to 64: the data region ends with its padding

    parts = ['{"format":"onemodel-checkpoint","version":1,"model":[', ",".join(_tensor_json(*e) for e in model), "]"]
    if with_opt:
        hyper = ",".join(f'{{"name":{_json_string(n)},"bits":{_float_bits(v)}}}' for n, v in target.hyper_parameters())
        parts += [',"optimizer":{"kind":', _json_string(target.kind), f',"step":{int(target.step)},"hyper":[', hyper, '],"state":[',
                  ",".join(_tensor_json(*e) for e in state), "]}"]
    items = sorted((extra or {}).items(), key=lambda kv: kv[0].encode("utf-16-be"))
    for k, v in items:
        if not _INT64_MIN <= int(v) <= _INT64_MAX:
            raise ValueError(f"extra[{k!r}] does not fit 64 bits")
    parts += [',"extra":[', ",".join(f'{{"key":{_json_string(k)},"value":{int(v)}}}' for k, v in items), "]}"]
    manifest = "".join(parts).encode("utf-8")
    if len(manifest) > MAX_MANIFEST:
        raise ValueError("the manifest exceeds 256 MiB")

    data_offset = (HEADER_SIZE + len(manifest) + 63) // 64 * 64
    file_length = data_offset + data_length
    stream.write(MAGIC + struct.pack("<IIQQQQQQ", 1, 0, HEADER_SIZE, len(manifest), data_offset, data_length, file_length, 0))
    stream.write(manifest)
    stream.write(b"\0" * (data_offset - HEADER_SIZE - len(manifest)))
    written = 0
    for i, (name, dtype, shape, offset, length) in enumerate(all_entries):
        stream.write(b"\0" * (offset - written))
        a = target.read_model(i) if i < len(model) else target.read_state(i - len(model))
        raw = np.ascontiguousarray(a, _DTYPES[dtype]).tobytes()
        assert len(raw) == length, (name, len(raw), length)
        stream.write(raw)
        written = offset + length
    stream.write(b"\0" * (data_length - written))


def save_file(path, target, optimizer=True, extra=None):
    with open(path, "wb") as f:
        save(f, target, optimizer, extra)


def _depth_ok(raw):
    """System.Text.Json's MaxDepth = 32: rejects a document nested deeper, before it builds anything."""
    depth, in_string, escape = 0, False, False
    for c in raw:
        if in_string:
            if escape:
                escape = False
            elif c == 0x5C:
                escape = True
            elif c == 0x22:
                in_string = False
        elif c == 0x22:
            in_string = True
        elif c in (0x5B, 0x7B):
            depth += 1
            if depth > MAX_DEPTH:
                return False
        elif c in (0x5D, 0x7D):
            depth -= 1
    return True


def _reject_constant(name):
    raise ValueError(f"{name} is not JSON")


def _field(obj, name, kind):
    """Str / Int / Arr of Checkpoint.cs:455-481: a missing field or one of another JSON type is a BadManifest."""
    v = obj.get(name) if isinstance(obj, dict) else None
    if kind == "str" and isinstance(v, str):
        return v
    if kind == "int" and isinstance(v, int) and not isinstance(v, bool) and _INT64_MIN <= v <= _INT64_MAX:
        return v
    if kind == "arr" and isinstance(v, list):
        return v
    what = {"str": "a string", "int": "an integer", "arr": "an array"}[kind]
    raise CheckpointError("BadManifest", f"Manifest field '{name}' is missing or not {what}.")


def _entries(array):
    out = []
    for e in array:
        name = _field(e, "name", "str")
        dtype = _field(e, "dtype", "str")
        if dtype not in _DTYPES:
            raise CheckpointError("BadManifest", f"Tensor '{name}' has unsupported dtype '{dtype}'.")
        dims = []
        for d in _field(e, "shape", "arr"):
            if not isinstance(d, int) or isinstance(d, bool) or d < 0 or d > 0x7FFFFFFF:
                raise CheckpointError("BadManifest", f"Tensor '{name}' has a bad dimension.")
            dims.append(d)
        out.append((name, dtype, tuple(dims), _field(e, "offset", "int"), _field(e, "length", "int")))
    return out


def _check_fit(what, entries, dest, data_length):
    if len(entries) != len(dest):
        raise CheckpointError("Mismatch", f"The checkpoint has {len(entries)} {what} tensors, the target has {len(dest)}.")
    for i, ((name, dtype, dims, offset, length), (want_name, want_dtype, want_shape)) in enumerate(zip(entries, dest)):
        if name != want_name or dtype != want_dtype or dims != tuple(int(d) for d in want_shape):
            raise CheckpointError("Mismatch", f"{what} entry {i} is '{name}' {dtype}{list(dims)}, the target expects '{want_name}' {want_dtype}{list(want_shape)}.")
        # The size comes from the target's shape, which equals the entry's by now: a hostile shape never sizes anything.
        expected = int(np.prod(want_shape, dtype=np.int64)) * _DTYPES[want_dtype].itemsize if len(want_shape) else _DTYPES[want_dtype].itemsize
        if length != expected or offset < 0 or offset > data_length or length > data_length - offset:
            raise CheckpointError("BadTensor", f"{what} tensor '{name}' has offset {offset}, length {length} (expected {expected}) in a data region of {data_length} bytes.")


def load(stream, target, optimizer=True):
    """Restores `target` from a seekable binary stream positioned at the start of a checkpoint.

    Returns (extra, has_optimizer). optimizer=False restores the model alone (a file with optimizer state still loads);
    optimizer=True on a model-only file is a Mismatch. A rejected file leaves the target unchanged.
    """
    if not stream.seekable():
        raise CheckpointError("UnsupportedStream", "Loading needs a seekable stream; spool the input to a file first.")
    start = stream.tell()
    length = stream.seek(0, io.SEEK_END) - start
    stream.seek(start)
    if length < HEADER_SIZE:
        raise CheckpointError("BadHeader", f"The file has {length} bytes, less than the {HEADER_SIZE}-byte header.")
    header = stream.read(HEADER_SIZE)
    if header[:8] != MAGIC:
        raise CheckpointError("BadHeader", "The magic is not ONEMCKPT.")
    version, flags, m_off, m_len, d_off, d_len, f_len, reserved = struct.unpack("<IIQQQQQQ", header[8:])
    if version != 1 or flags != 0 or reserved != 0:
        raise CheckpointError("BadHeader", f"Unsupported version {version}, flags {flags} or reserved field.")
    if f_len != length:
        raise CheckpointError("BadHeader", f"The header says {f_len} bytes, the file has {length} (truncated or extended).")
    if (m_off != HEADER_SIZE or m_len > MAX_MANIFEST or m_len > f_len - HEADER_SIZE or d_off % 64 != 0 or d_off < HEADER_SIZE + m_len
            or d_off > f_len or d_len != f_len - d_off):
        raise CheckpointError("BadHeader", "Manifest or data region offsets are inconsistent with the file length.")

    raw = stream.read(m_len)
    try:
        if len(raw) != m_len or not _depth_ok(raw):
            raise ValueError("truncated or nested deeper than 32")
        root = json.loads(raw.decode("utf-8", errors="strict"), parse_constant=_reject_constant)
    except (ValueError, RecursionError) as e:
        raise CheckpointError("BadManifest", f"The manifest is not valid JSON: {e}") from None
    if not isinstance(root, dict) or _field(root, "format", "str") != "onemodel-checkpoint" or _field(root, "version", "int") != 1:
        raise CheckpointError("BadManifest", "The manifest is not a version 1 onemodel-checkpoint.")

    model_entries = _entries(_field(root, "model", "arr"))
    _check_fit("model", model_entries, target.model_entries(), d_len)

    opt = root.get("optimizer")
    has_optimizer = isinstance(opt, dict)
    want_optimizer = optimizer and target.has_optimizer()
    state_entries, values, step = None, None, 0
    if has_optimizer and want_optimizer:
        kind = _field(opt, "kind", "str")
        if kind != target.kind:
            raise CheckpointError("Mismatch", f"The checkpoint holds a '{kind}' optimizer, not '{target.kind}'.")
        step = _field(opt, "step", "int")
        if step < 0:
            raise CheckpointError("BadManifest", "The optimizer step count is negative.")
        values = {}
        for hp in _field(opt, "hyper", "arr"):
            bits = _field(hp, "bits", "int")
            if bits < 0 or bits > 0xFFFFFFFF:
                raise CheckpointError("BadManifest", "A hyper-parameter bit pattern is out of range.")
            values[_field(hp, "name", "str")] = _bits_float(bits)
        for name, _ in target.hyper_parameters():
            if name not in values:
                raise CheckpointError("Mismatch", f"The checkpoint lacks hyper-parameter '{name}'.")
        state_entries = _entries(_field(opt, "state", "arr"))
        _check_fit("optimizer state", state_entries, target.state_entries(), d_len)
    elif want_optimizer:
        raise CheckpointError("Mismatch", "The checkpoint holds no optimizer state.")

    extra = {}
    if isinstance(root.get("extra"), list):
        for e in root["extra"]:
            extra[_field(e, "key", "str")] = _field(e, "value", "int")
    if values is not None:
        target.check_hyper(values)

    # Everything is checked; from here on the target changes.
    def fill(entries, write):
        for i, (name, dtype, dims, offset, nbytes) in enumerate(entries):
            stream.seek(start + d_off + offset)
            data = stream.read(nbytes)
            if len(data) != nbytes:
                raise CheckpointError("BadTensor", f"tensor '{name}' ends past the end of the file.")
            write(i, np.frombuffer(data, _DTYPES[dtype]).reshape(dims))

    fill(model_entries, target.write_model)
    if state_entries is not None:
        fill(state_entries, target.write_state)
        target.restore(step, values)
    stream.seek(start + length)
    return extra, has_optimizer


def load_file(path, target, optimizer=True):
    with open(path, "rb") as f:
        return load(f, target, optimizer)
