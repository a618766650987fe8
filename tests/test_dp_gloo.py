"""The data-parallel arithmetic on CPU ranks (gloo, world sizes 2 and 4): shards of the global batch, loss summed per shard and
divided by the GLOBAL counted rows, flat gradients summed across ranks in bucket order - against one process that sees
the whole batch. This is the exchange host/trainer.cpp performs with NCCL on the GPUs (om_dp_allreduce_bucket), restated
on the CPU oracle; the reference is single-process (Engine.cs:164-191), so the single-process result is the contract."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)

WORKER = r'''
import os, sys, json
import numpy as np
import torch
import torch.distributed as dist
sys.path.insert(0, os.path.join(%(root)r, "onemodel-csharp_b200"))
sys.path.insert(0, %(root)r)
import synth
from oracle import configs

rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
dist.init_process_group("gloo", rank=rank, world_size=world)
batch, seq, layers, width, heads, ff, vocab, rows = 2, 8, 1, 16, 2, 32, 37, 5
weights = configs.mlm_init(seq, layers, width, ff, vocab, seed=0)
ids, pos, labels = synth.mlm_batch(batch, seq, vocab, rows, 0, rank)
loss, grads = configs.mlm_forward_backward(weights, ids.astype(np.int64), pos.astype(np.int64), labels, layers, heads,
                                           denominator=rows * world)
# Flat gradient in reverse registration order, cut into buckets, one allreduce per bucket (as the trainer does).
names = list(weights)[::-1]
flat = torch.from_numpy(np.concatenate([grads[n].reshape(-1) for n in names]).astype(np.float32))
bucket = 1000
for b0 in range(0, flat.numel(), bucket):
    dist.all_reduce(flat[b0:b0 + bucket], op=dist.ReduceOp.SUM)
lt = torch.tensor([loss], dtype=torch.float32)
dist.all_reduce(lt, op=dist.ReduceOp.SUM)
# Every rank must hold the same bits afterwards (replicas stay equal).
gathered = [torch.empty_like(flat) for _ in range(world)]
dist.all_gather(gathered, flat)
same = all(torch.equal(gathered[0], g) for g in gathered)
if rank == 0:
    # One process over the global batch: shards concatenated, masked rows offset by the shard's first position.
    all_ids, all_pos, all_labels = [], [], []
    for r in range(world):
        i, p, l = synth.mlm_batch(batch, seq, vocab, rows, 0, r)
        all_ids.append(i); all_pos.append(p.astype(np.int64) + r * batch * seq); all_labels.append(l)
    gl, gg = configs.mlm_forward_backward(weights, np.concatenate(all_ids).astype(np.int64), np.concatenate(all_pos),
                                          np.concatenate(all_labels), layers, heads)
    ref = np.concatenate([gg[n].reshape(-1) for n in names])
    scale = float(np.max(np.abs(ref)))
    print(json.dumps({"same": bool(same), "loss_dp": float(lt[0]), "loss_single": gl,
                      "grad_err": float(np.max(np.abs(flat.numpy() - ref)) / scale), "n": int(flat.numel())}))
dist.barrier()
dist.destroy_process_group()
'''


CTC_WORKER = r'''
import os, sys, json
import numpy as np
import torch
import torch.distributed as dist
sys.path.insert(0, os.path.join(%(root)r, "onemodel-csharp_b200"))
sys.path.insert(0, %(root)r)
import synth
from oracle import configs, tape as A

rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
dist.init_process_group("gloo", rank=rank, world_size=world)
batch, height, width, classes, hidden, max_label = 2, 32, 32, 7, 4, 3
weights = configs.crnn_init([2, 3, 4, 4], hidden, classes, seed=0)
x, targets, lengths = synth.crnn_batch(batch, height, width, classes, max_label, 1, 0, rank)
# The shard's CTC mean divided by the world size (what the trainer multiplies in), gradients summed over ranks.
loss, grads = configs.crnn_forward_backward(weights, x, targets[: int(lengths.sum())], lengths, loss_scale=1.0 / world)
names = list(weights)[::-1]
flat = torch.from_numpy(np.concatenate([grads[n].reshape(-1) for n in names]).astype(np.float32))
dist.all_reduce(flat, op=dist.ReduceOp.SUM)
lt = torch.tensor([loss], dtype=torch.float32)
dist.all_reduce(lt, op=dist.ReduceOp.SUM)
if rank == 0:
    xs, ts, ls = [], [], []
    for r in range(world):
        xi, ti, li = synth.crnn_batch(batch, height, width, classes, max_label, 1, 0, r)
        xs.append(xi); ts.append(ti[: int(li.sum())]); ls.append(li)
    gl, gg = configs.crnn_forward_backward(weights, np.concatenate(xs), np.concatenate(ts), np.concatenate(ls))
    ref = np.concatenate([gg[n].reshape(-1) for n in names])
    print(json.dumps({"loss_dp": float(lt[0]), "loss_single": gl,
                      "grad_err": float(np.max(np.abs(flat.numpy() - ref)) / float(np.max(np.abs(ref))))}))
dist.barrier()
dist.destroy_process_group()
'''


def _run_ranks(tmp_path, source, world, port):
    script = tmp_path / "dp_worker.py"
    script.write_text(source % {"root": ROOT})
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), OMP_NUM_THREADS="2")
    procs = []
    for r in range(world):
        e = dict(env, RANK=str(r), WORLD_SIZE=str(world))
        procs.append(subprocess.Popen([sys.executable, str(script)], env=e, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True))
    outs = [p.communicate(timeout=240) for p in procs]
    for p, (o, e) in zip(procs, outs):
        assert p.returncode == 0, e[-2000:]
    return json.loads(outs[0][0].strip().splitlines()[-1])


@pytest.mark.parametrize("world", [2, 4])
def test_ctc_shards_sum_to_the_single_process_step(tmp_path, oracle_built, world):
    """The CRNN trainer under data parallelism: the CTC loss is a mean over the local sequences, so each shard's loss is
    multiplied by 1 / world before the backward pass (host/trainer.cpp); the sum over ranks of loss and gradients is then
    the single-process mean over the global batch."""
    res = _run_ranks(tmp_path, CTC_WORKER, world, 29620 + world)
    assert abs(res["loss_dp"] - res["loss_single"]) <= 1e-5 * abs(res["loss_single"])
    assert res["grad_err"] <= 1e-5


@pytest.mark.parametrize("world", [2, 4])
def test_shards_sum_to_the_single_process_step(tmp_path, oracle_built, world):
    script = tmp_path / "dp_worker.py"
    script.write_text(WORKER % {"root": ROOT})
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT=str(29609 + world), OMP_NUM_THREADS="2")
    procs = []
    for r in range(world):
        e = dict(env, RANK=str(r), WORLD_SIZE=str(world))
        procs.append(subprocess.Popen([sys.executable, str(script)], env=e, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True))
    outs = [p.communicate(timeout=240) for p in procs]
    for p, (o, e) in zip(procs, outs):
        assert p.returncode == 0, e[-2000:]
    res = json.loads(outs[0][0].strip().splitlines()[-1])
    assert res["same"]
    assert abs(res["loss_dp"] - res["loss_single"]) <= 1e-5 * abs(res["loss_single"])
    assert res["grad_err"] <= 1e-5      # same sums in another order


def test_reference_arm_runs_on_rank_zero_only(oracle_built):
    """bench.py --impl reference under a 2-rank launch: rank 0 alone times the CPU path and prints the line, the other
    rank exits 0 without output."""
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT="29612", WORLD_SIZE="2", OMP_NUM_THREADS="4")
    outs = []
    for r in range(2):
        e = dict(env, RANK=str(r), LOCAL_RANK=str(r))
        p = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2", "--workload", "c1",
                            "--steps", "2", "--warmup", "1"], env=e, capture_output=True, text=True, timeout=240)
        assert p.returncode == 0, p.stderr[-2000:]
        outs.append(p.stdout.strip())
    assert outs[1] == ""
    line = json.loads(outs[0].splitlines()[-1])
    assert line["impl"] == "reference" and line["n_gpus"] == 2 and line["value"] > 0
    assert line["cpu_baseline"]["kind"] == "port" and line["e2e"]["h2d_bytes_per_step"] == 0
