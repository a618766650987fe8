#!/usr/bin/env python3
"""Writes tests/golden/graph_ops.npz: inputs, loss and gradients of one graph through the graph-op family (batched matrix
product with broadcast batch axes, Erf, Exp, Sqrt, Pow with the exact and the general exponents, Where, Gather with
negative and repeated indices), computed with PyTorch CPU autograd - the engine the reference's own oracle generators
(tools/autograd_oracle.py, tools/finetune_oracle.py) use. The graph is tests/models.py:graph_ops_case with seed 0.

It also writes tests/golden/conv1d.npz (Conv1d with stride, separate left/right padding, dilation and groups).

    python tests/golden/make_graphops_golden.py
"""
import os

import numpy as np
import torch


def main():
    r = np.random.default_rng(0)
    a = torch.tensor(r.standard_normal((2, 3, 4, 5)).astype(np.float32), requires_grad=True)
    b = torch.tensor(r.standard_normal((3, 5, 6)).astype(np.float32), requires_grad=True)
    c = torch.tensor((r.random((4, 6)) + 0.5).astype(np.float32), requires_grad=True)
    d = torch.tensor(r.standard_normal((1, 6)).astype(np.float32), requires_grad=True)
    m = torch.matmul(a, b)
    t = torch.erf(m) + torch.exp(m * 0.1)
    t = t + torch.sqrt(c)
    t = t + c ** 2
    t = t + c ** -1
    t = t + c ** 0.5
    t = t + c ** 1.7
    cond = torch.tensor(r.random((3, 4, 6)) < 0.5)
    t = torch.where(cond, t, d)
    idx = torch.tensor([[2, -1], [0, 2]]) % 4
    g = t[:, :, idx]
    w = torch.tensor(r.standard_normal((2, 3, 2, 2, 6)).astype(np.float32))
    loss = (g * w).sum()
    loss.backward()
    out = os.path.join(os.path.dirname(os.path.abspath(__file__)), "graph_ops.npz")
    np.savez(out, loss=np.float32(loss.item()), out=g.detach().numpy(), grad_a=a.grad.numpy(), grad_b=b.grad.numpy(),
             grad_c=c.grad.numpy(), grad_d=d.grad.numpy(), torch_version=np.array(torch.__version__))
    print("wrote", out)
    conv1d_golden()


def conv1d_golden():
    """tests/golden/conv1d.npz: the cases of tests/models.py:CONV1D_CASES through torch.nn.functional.conv1d (asymmetric
    padding by an explicit zero pad), seed and shapes as in conv1d_case."""
    import sys
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
    from models import CONV1D_CASES
    import torch.nn.functional as F
    arrays = {"torch_version": np.array(torch.__version__)}
    for i, (n, c, l, o, k, stride, pl, pr, dil, groups, has_bias) in enumerate(CONV1D_CASES):
        r = np.random.default_rng(0 + l)
        x = torch.tensor(r.standard_normal((n, c, l)).astype(np.float32), requires_grad=True)
        w = torch.tensor((r.standard_normal((o, c // groups, k)) * 0.5).astype(np.float32), requires_grad=True)
        b = torch.tensor(r.standard_normal(o).astype(np.float32), requires_grad=True) if has_bias else None
        y = F.conv1d(F.pad(x, (pl, pr)), w, b, stride=stride, padding=0, dilation=dil, groups=groups)
        proj = torch.tensor(r.standard_normal(tuple(y.shape)).astype(np.float32))
        loss = (y * proj).sum()
        loss.backward()
        arrays[f"{i}.loss"] = np.float32(loss.item())
        arrays[f"{i}.out"] = y.detach().numpy()
        arrays[f"{i}.grad_x"] = x.grad.numpy()
        arrays[f"{i}.grad_w"] = w.grad.numpy()
        if has_bias:
            arrays[f"{i}.grad_b"] = b.grad.numpy()
    out = os.path.join(os.path.dirname(os.path.abspath(__file__)), "conv1d.npz")
    np.savez(out, **arrays)
    print("wrote", out)


if __name__ == "__main__":
    main()
