"""Checkpoints of a device-resident trainer: a run saved at step k and continued in a fresh trainer reproduces the
uninterrupted run bit for bit (the resume rule of docs/training.md section 6 of the reference)."""
import io
import struct

import numpy as np
import pytest

import checkpoint as ck
import om_binding as omb
import synth

pytestmark = pytest.mark.gpu


MLM = [4, 16, 2, 32, 4, 64, 50, 16]           # batch, seq, layers, width, heads, ff, vocab, counted rows
CNN = [4, 3, 16, 16, 10, 2, 8, 16, 1, 2]       # batch, channels, h, w, classes, stages, stage channels..., strides...


def make(kind, lr=None, seed=3):
    if kind == "mlm":
        return omb.Trainer("mlm", MLM, 1e-3 if lr is None else lr, weight_decay=0.01, clip_norm=1.0, seed=seed)
    return omb.Trainer("cnn", CNN, 0.05 if lr is None else lr, weight_decay=0.0, seed=seed)


def inputs_for(t, kind, step):
    if kind == "mlm":
        return list(synth.mlm_batch(MLM[0], MLM[1], MLM[6], MLM[7], step))
    return list(synth.cnn_batch(CNN[0], CNN[1], CNN[2], CNN[3], CNN[4], step))


@pytest.mark.parametrize("kind", ["mlm", "cnn"])
def test_resume_is_bit_equal(ctx, kind):
    ctx.set_flags(0)
    ctx.make_current()
    t = make(kind)
    for s in range(3):
        t.step(inputs_for(t, kind, s))
    buf = io.BytesIO()
    ck.save(buf, ck.TrainerState(t), extra={"samples": 3 * 4})
    raw = buf.getvalue()
    losses = [t.step(inputs_for(t, kind, s)) for s in range(3, 6)]
    final = [t.model_state_get(i) for i in range(len(t.model_state_entries()))]
    final_state = [t.optimizer_state_get(i) for i in range(len(t.optimizer_state_entries()))]
    t.close()

    # the file: header fields, optimizer kind, state names in the reference's order
    version, flags, m_off, m_len, d_off, d_len, f_len, reserved = struct.unpack("<IIQQQQQQ", raw[8:64])
    assert raw[:8] == b"ONEMCKPT" and (version, flags, m_off, reserved) == (1, 0, 64, 0) and f_len == len(raw)
    manifest = raw[64:64 + m_len].decode()
    if kind == "mlm":
        assert '"optimizer":{"kind":"adamw","step":3,"hyper":[{"name":"lr"' in manifest
        assert '"state":[{"name":"exp_avg.0"' in manifest and '{"name":"exp_avg_sq.0"' in manifest
    else:
        assert '"optimizer":{"kind":"sgd","step":3,' in manifest
        assert '"state":[{"name":"initialized","dtype":"i32"' in manifest and '.running_mean","dtype":"f32"' in manifest

    # a fresh trainer with another seed: everything it holds comes from the file
    u = make(kind, lr=0.5, seed=99)
    extra, has_opt = ck.load(io.BytesIO(raw), ck.TrainerState(u))
    assert has_opt and extra == {"samples": 12} and u.steps_done() == 3
    assert dict(u.hyper_parameters())["lr"] == np.float32(1e-3 if kind == "mlm" else 0.05)
    again = io.BytesIO()
    ck.save(again, ck.TrainerState(u), extra={"samples": 12})
    assert again.getvalue() == raw  # the restored state writes the same bytes
    resumed = [u.step(inputs_for(u, kind, s)) for s in range(3, 6)]
    assert [np.float32(a).tobytes() for a in resumed] == [np.float32(a).tobytes() for a in losses]
    for i, a in enumerate(final):
        assert u.model_state_get(i).tobytes() == a.tobytes(), u.model_state_entries()[i]
    for i, a in enumerate(final_state):
        assert u.optimizer_state_get(i).tobytes() == a.tobytes(), u.optimizer_state_entries()[i]

    # a file of another model is rejected before anything changes
    snap = u.model_state_get(0)
    other = make("cnn" if kind == "mlm" else "mlm")
    wrong = io.BytesIO()
    ck.save(wrong, ck.TrainerState(other))
    other.close()
    with pytest.raises(ck.CheckpointError) as e:
        ck.load(io.BytesIO(wrong.getvalue()), ck.TrainerState(u))
    assert e.value.kind == "Mismatch"
    assert u.model_state_get(0).tobytes() == snap.tobytes()
    u.close()
