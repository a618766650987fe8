"""Data-parallel training on two GPUs (one process per GPU, NCCL): the sharded step against one process that sees the
whole batch. Skipped on a single-GPU machine. Ranks are child processes; the NCCL id travels through a file."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)

WORKER = r'''
import os, sys, time, json, ctypes as C
import numpy as np
sys.path.insert(0, os.path.join(%(root)r, "onemodel-csharp_b200"))
import om_binding as omb, synth
rank, world, out = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3]
graph = int(sys.argv[4])
kind = sys.argv[5] if len(sys.argv) > 5 else "mlm"
cfg = [4, 16, 2, 32, 4, 64, 101, 10] if kind == "mlm" else [4, 32, 48, 11, 8, 5, 4, 6, 8, 8]
ctx = omb.Context(rank, 0)
tr = omb.Trainer(kind, cfg, lr=1e-3, weight_decay=0.01 if kind == "mlm" else 0.0, seed=0)
idfile = os.path.join(out, "nccl_id.bin")
if rank == 0:
    buf = (C.c_uint8 * 128)()
    ctx.call("om_dp_unique_id", ctx.handle, buf)
    with open(idfile + ".tmp", "wb") as f:
        f.write(bytes(buf))
    os.replace(idfile + ".tmp", idfile)
t0 = time.time()
while not os.path.exists(idfile):
    if time.time() - t0 > 60:
        sys.exit(3)
    time.sleep(0.05)
tr.dp_init(open(idfile, "rb").read(), rank, world, (cfg[7] if kind == "mlm" else cfg[0]) * world)
losses = []
grads = None
for step in range(4):
    if kind == "mlm":
        batch = list(synth.mlm_batch(cfg[0], cfg[1], cfg[6], cfg[7], step, rank))
    else:
        batch = list(synth.crnn_batch(cfg[0], cfg[1], cfg[2], cfg[3], cfg[5], 2, step, rank))
    if graph and step == 2:
        tr.enable_graph()
    losses.append(tr.step(batch))
    if step == 0:
        grads = [tr.get_grad(i, s) for i, (n, s) in enumerate(tr.named_parameters())]
params = [tr.get_param(i, s) for i, (n, s) in enumerate(tr.named_parameters())]
np.savez(os.path.join(out, f"rank{rank}.npz"), losses=np.array(losses, np.float32),
         **{f"g{i}": g for i, g in enumerate(grads)}, **{f"p{i}": p for i, p in enumerate(params)})
tr.close()
'''


def _device_count():
    try:
        import torch
        return torch.cuda.device_count()
    except Exception:
        return 0


@pytest.mark.parametrize("graph", [0, 1])
def test_two_gpu_step_equals_single_process_global_batch(ctx, tmp_path, graph):
    if _device_count() < 2:
        pytest.skip("needs two GPUs")
    import om_binding as omb
    import synth
    from backends import scaled_diff
    script = tmp_path / "dp_rank.py"
    script.write_text(WORKER % {"root": ROOT})
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    procs = [subprocess.Popen([sys.executable, str(script), str(r), "2", str(tmp_path), str(graph)], env=env,
                              stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True) for r in range(2)]
    outs = [p.communicate(timeout=300) for p in procs]
    for p, (o, e) in zip(procs, outs):
        assert p.returncode == 0, (o[-1000:], e[-3000:])
    r0, r1 = np.load(tmp_path / "rank0.npz"), np.load(tmp_path / "rank1.npz")
    # Replicas stay bit-equal: same summed gradients, same update.
    for k in r0.files:
        assert np.array_equal(r0[k], r1[k]), k
    # One process over the global batch.
    cfg = [4, 16, 2, 32, 4, 64, 101, 10]
    ctx.set_flags(0)
    ctx.make_current()
    big = [8, 16, 2, 32, 4, 64, 101, 20]
    tr = omb.Trainer("mlm", big, lr=1e-3, weight_decay=0.01, seed=0)
    named = tr.named_parameters()
    for step in range(4):
        parts = [synth.mlm_batch(cfg[0], cfg[1], cfg[6], cfg[7], step, r) for r in range(2)]
        ids = np.concatenate([p[0] for p in parts])
        pos = np.concatenate([p[1] + r * cfg[0] * cfg[1] for r, p in enumerate(parts)]).astype(np.int32)
        labels = np.concatenate([p[2] for p in parts])
        loss = tr.step([ids, pos, labels])
        assert abs(loss - float(r0["losses"][step])) <= 2e-5 * abs(loss), step
        if step == 0:
            for i, (n, s) in enumerate(named):
                g = tr.get_grad(i, s)
                if np.max(np.abs(g)) > 1e-7:
                    assert scaled_diff(r0[f"g{i}"], g) <= 2e-5, n
    tr.close()


def test_two_gpu_ctc_step_equals_single_process_global_batch(ctx, tmp_path):
    """The CRNN + CTC trainer on two GPUs: the CTC loss is a mean over the local sequences, so each rank scales its loss by
    1 / world before the backward pass; loss and gradients summed over the ranks equal one process on the global batch."""
    if _device_count() < 2:
        pytest.skip("needs two GPUs")
    import om_binding as omb
    import synth
    from backends import scaled_diff
    script = tmp_path / "dp_rank.py"
    script.write_text(WORKER % {"root": ROOT})
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    procs = [subprocess.Popen([sys.executable, str(script), str(r), "2", str(tmp_path), "0", "crnn"], env=env,
                              stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True) for r in range(2)]
    outs = [p.communicate(timeout=300) for p in procs]
    for p, (o, e) in zip(procs, outs):
        assert p.returncode == 0, (o[-1000:], e[-3000:])
    r0, r1 = np.load(tmp_path / "rank0.npz"), np.load(tmp_path / "rank1.npz")
    for k in r0.files:
        assert np.array_equal(r0[k], r1[k]), k
    cfg = [4, 32, 48, 11, 8, 5, 4, 6, 8, 8]
    ctx.set_flags(0)
    ctx.make_current()
    tr = omb.Trainer("crnn", [8] + cfg[1:], lr=1e-3, weight_decay=0.0, seed=0)
    named = tr.named_parameters()
    for step in range(4):
        parts = [synth.crnn_batch(cfg[0], cfg[1], cfg[2], cfg[3], cfg[5], 2, step, r) for r in range(2)]
        x = np.concatenate([p[0] for p in parts])
        lengths = np.concatenate([p[2] for p in parts])
        targets = np.zeros(8 * cfg[5], np.int32)
        valid = np.concatenate([p[1][: int(p[2].sum())] for p in parts])
        targets[: valid.size] = valid
        loss = tr.step([x, targets, lengths])
        assert abs(loss - float(r0["losses"][step])) <= 2e-5 * abs(loss), step
        if step == 0:
            for i, (n, s) in enumerate(named):
                g = tr.get_grad(i, s)
                if np.max(np.abs(g)) > 1e-7:
                    assert scaled_diff(r0[f"g{i}"], g) <= 2e-5, n
    tr.close()
