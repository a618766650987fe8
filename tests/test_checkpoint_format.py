"""The checkpoint file format against the reference's own malformed-file fixtures and its documented layout.

tests/golden/checkpoint_hostile/<Kind>-<name>.ckpt are the reference's committed cases (testdata/checkpoint/hostile, assembled
by tests/OneModel.Tests/Training/CheckpointHostileTests.cs); each must be rejected with the error kind in its file name
when loaded into a Linear(2, 2) with bias, leaving the target unchanged. These tests need no GPU: the target is a host
state; the same loader serves the device-resident trainer (test_gpu_checkpoint.py).
"""
import io
import pathlib
import struct

import numpy as np
import pytest

import checkpoint as ck

HOSTILE = sorted((pathlib.Path(__file__).parent / "golden" / "checkpoint_hostile").glob("*.ckpt"))

# CheckpointHostileTests.cs:16-17, 22-33: the well-formed file every case is derived from.
BASE = ('{"format":"onemodel-checkpoint","version":1,"model":[{"name":"weight","dtype":"f32","shape":[2,2],"offset":0,"length":16},'
        '{"name":"bias","dtype":"f32","shape":[2],"offset":64,"length":8}],"extra":[]}')


def linear22():
    return ck.HostState([("weight", np.full((2, 2), -1, np.float32)), ("bias", np.full((2,), -1, np.float32))])


def assemble(manifest, data):
    m = manifest.encode()
    off = (64 + len(m) + 63) // 64 * 64
    total = off + len(data)
    return b"ONEMCKPT" + struct.pack("<IIQQQQQQ", 1, 0, 64, len(m), off, len(data), total, 0) + m + b"\0" * (off - 64 - len(m)) + data


def base_data():
    d = bytearray(72)
    d[0:16] = np.arange(1, 5, dtype="<f4").tobytes()
    d[64:72] = np.array([5, 6], "<f4").tobytes()
    return bytes(d)


def test_fixture_count():
    assert len(HOSTILE) == 42


@pytest.mark.parametrize("path", HOSTILE, ids=lambda p: p.stem)
def test_hostile_file_is_rejected_with_its_kind(path):
    kind = path.stem.split("-", 1)[0]
    target = linear22()
    with pytest.raises(ck.CheckpointError) as e:
        ck.load(io.BytesIO(path.read_bytes()), target, optimizer=False)
    assert e.value.kind == kind
    assert all((a == -1).all() for _, a in target.model)
    with pytest.raises(ck.CheckpointError) as e:
        ck.load_file(str(path), target, optimizer=False)
    assert e.value.kind == kind


def test_hand_assembled_file_loads():
    target = linear22()
    extra, has_opt = ck.load(io.BytesIO(assemble(BASE, base_data())), target, optimizer=False)
    assert extra == {} and not has_opt
    np.testing.assert_array_equal(target.model[0][1], [[1, 2], [3, 4]])
    np.testing.assert_array_equal(target.model[1][1], [5, 6])


def test_hostile_fixtures_derive_from_the_base_file():
    """The 'truncated' case is the base file less its last byte: pins the assembler of this test on the reference's."""
    good = assemble(BASE, base_data())
    by_name = {p.stem: p.read_bytes() for p in HOSTILE}
    assert by_name["BadHeader-truncated"] == good[:-1]
    assert by_name["BadHeader-extended"] == good + b"\0"
    assert by_name["BadHeader-short-header"] == good[:40]


def adam_state(seed, step=7):
    r = np.random.default_rng(seed)
    model = [("0.weight", r.standard_normal((3, 5)).astype(np.float32)), ("0.bias", r.standard_normal(3).astype(np.float32)),
             ("bn.running_mean", r.standard_normal(4).astype(np.float32)), ("drop.draws", np.array([seed], np.int64))]
    state = [(f"{slot}.{i}", r.standard_normal(s).astype(np.float32)) for slot in ("exp_avg", "exp_avg_sq") for i, s in enumerate([(3, 5), (3,)])]
    hyper = [("lr", 1e-3), ("beta1", 0.9), ("beta2", 0.999), ("epsilon", 1e-8), ("weight_decay", 0.01), ("amsgrad", 0.0)]
    return ck.HostState(model, "adamw", step, hyper, state, fixed=("beta1", "beta2", "epsilon", "amsgrad"))


def test_round_trip_and_layout():
    src = adam_state(1)
    src.model[0][1][0, 0] = np.float32(np.nan)
    src.model[0][1][0, 1] = np.float32(-0.0)
    buf = io.BytesIO()
    ck.save(buf, src, extra={"samples": 1234, "Epoch": -2})
    raw = buf.getvalue()
    # the header of docs/training.md section 6
    assert raw[:8] == b"ONEMCKPT"
    version, flags, m_off, m_len, d_off, d_len, f_len, reserved = struct.unpack("<IIQQQQQQ", raw[8:64])
    assert (version, flags, m_off, reserved) == (1, 0, 64, 0)
    assert d_off % 64 == 0 and d_off >= 64 + m_len and f_len == len(raw) == d_off + d_len and d_len % 64 == 0
    manifest = raw[64:64 + m_len].decode()
    assert manifest.startswith('{"format":"onemodel-checkpoint","version":1,"model":[{"name":"0.weight","dtype":"f32","shape":[3,5],"offset":0,"length":60},'
                               '{"name":"0.bias","dtype":"f32","shape":[3],"offset":64,"length":12}')
    assert '{"name":"drop.draws","dtype":"i64","shape":[1],"offset":192,"length":8}' in manifest
    assert f'"optimizer":{{"kind":"adamw","step":7,"hyper":[{{"name":"lr","bits":{int(np.float32(1e-3).view(np.uint32))}}}' in manifest
    assert manifest.endswith('"extra":[{"key":"Epoch","value":-2},{"key":"samples","value":1234}]}')  # ordinal order
    assert " " not in manifest
    assert set(raw[64 + m_len:d_off]) <= {0}
    # the same state writes the same bytes
    again = io.BytesIO()
    ck.save(again, src, extra={"Epoch": -2, "samples": 1234})
    assert again.getvalue() == raw

    dst = adam_state(2, step=0)
    dst.hyper[0] = ("lr", np.float32(5.0))
    extra, has_opt = ck.load(io.BytesIO(raw), dst)
    assert has_opt and extra == {"samples": 1234, "Epoch": -2} and dst.step == 7
    for (_, a), (_, b) in zip(src.model + src.state, dst.model + dst.state):
        assert a.tobytes() == b.tobytes()  # bit patterns: the NaN and the signed zero survive
    assert dst.hyper[0][1] == np.float32(1e-3)


def test_optimizer_rules():
    raw = io.BytesIO()
    ck.save(raw, adam_state(1))
    raw = raw.getvalue()
    model_only = io.BytesIO()
    ck.save(model_only, adam_state(1), optimizer=False)

    # a file with optimizer state loads into the model alone
    dst = adam_state(2, step=3)
    before = [a.copy() for _, a in dst.state]
    _, has_opt = ck.load(io.BytesIO(raw), dst, optimizer=False)
    assert has_opt and dst.step == 3 and all((a == b).all() for a, (_, b) in zip(before, dst.state))

    def rejected(data, target, kind):
        snap = [a.copy() for _, a in target.model + target.state]
        with pytest.raises(ck.CheckpointError) as e:
            ck.load(io.BytesIO(data), target)
        assert e.value.kind == kind
        assert all((a == b).all() for a, (_, b) in zip(snap, target.model + target.state))

    rejected(model_only.getvalue(), adam_state(2), "Mismatch")      # optimizer state asked from a model-only file
    other = adam_state(2)
    other.kind = "adam"
    rejected(raw, other, "Mismatch")                                 # another optimizer kind
    other = adam_state(2)
    other.hyper[2] = ("beta2", np.float32(0.99))
    rejected(raw, other, "Mismatch")                                 # a fixed setting differs
    other = adam_state(2)
    other.state.pop()
    rejected(raw, other, "Mismatch")                                 # state tensor count
    other = adam_state(2)
    other.hyper.append(("extra_setting", np.float32(1)))
    rejected(raw, other, "Mismatch")                                 # the file lacks a hyper-parameter
    m_len, d_off = struct.unpack("<Q", raw[24:32])[0], struct.unpack("<Q", raw[32:40])[0]
    manifest, data = raw[64:64 + m_len].decode(), raw[d_off:]
    rejected(assemble(manifest.replace('"step":7', '"step":-7'), data), adam_state(2), "BadManifest")
    bits = str(int(np.float32(0.9).view(np.uint32)))
    assert f'"bits":{bits}' in manifest
    rejected(assemble(manifest.replace(f'"bits":{bits}', '"bits":4294967296'), data), adam_state(2), "BadManifest")
    rejected(assemble(manifest.replace(f'"bits":{bits}', '"bits":-1'), data), adam_state(2), "BadManifest")
    ck.load(io.BytesIO(assemble(manifest, data)), adam_state(2))     # the reassembled file itself is fine


def test_non_seekable_stream_is_refused():
    class Pipe(io.BytesIO):
        def seekable(self):
            return False

    with pytest.raises(ck.CheckpointError) as e:
        ck.load(Pipe(b""), linear22(), optimizer=False)
    assert e.value.kind == "UnsupportedStream"


def test_load_starts_at_the_stream_position():
    data = assemble(BASE, base_data())
    s = io.BytesIO(b"prefix--" + data)
    s.seek(8)
    target = linear22()
    ck.load(s, target, optimizer=False)
    assert s.tell() == 8 + len(data) and target.model[1][1][1] == 6
