"""Writes tests/golden/losses.npz: PyTorch (CPU, float32) values and input gradients of the loss family the reference's
Losses class offers (cross entropy with label smoothing and ignored rows, mean squared error, L1, binary cross entropy
with logits), the engine the reference's own tests compare with (ModuleAndLossTests.cs:183-248 of the reference).
Run:  python tests/golden/make_losses_golden.py"""
import os

import numpy as np
import torch
import torch.nn.functional as F

CE_CASES = [(0.1, True), (0.3, True), (0.2, False), (1.0, True)]     # (label smoothing, mean)


def inputs():
    r = np.random.default_rng(77)
    logits = r.standard_normal((9, 6)).astype(np.float32) * 2
    targets = r.integers(0, 6, 9).astype(np.int64)
    targets[[2, 7]] = -100
    pred = r.standard_normal((4, 5)).astype(np.float32)
    goal = r.standard_normal((4, 5)).astype(np.float32)
    goal[1, 2] = pred[1, 2]                                           # a zero difference: the L1 gradient there is 0
    probs = r.uniform(0, 1, (4, 5)).astype(np.float32)
    return logits, targets, pred, goal, probs


def main():
    torch.set_num_threads(1)
    logits, targets, pred, goal, probs = inputs()
    out = {"logits": logits, "targets": targets, "pred": pred, "goal": goal, "probs": probs}
    for i, (eps, mean) in enumerate(CE_CASES):
        x = torch.tensor(logits, requires_grad=True)
        loss = F.cross_entropy(x, torch.tensor(targets), label_smoothing=eps, ignore_index=-100, reduction="mean" if mean else "sum")
        loss.backward()
        out[f"ce{i}.loss"], out[f"ce{i}.grad"] = loss.detach().numpy(), x.grad.numpy()
    for name, fn in (("mse", F.mse_loss), ("l1", F.l1_loss)):
        for mean in (True, False):
            x = torch.tensor(pred, requires_grad=True)
            loss = fn(x, torch.tensor(goal), reduction="mean" if mean else "sum")
            loss.backward()
            out[f"{name}.{int(mean)}.loss"], out[f"{name}.{int(mean)}.grad"] = loss.detach().numpy(), x.grad.numpy()
    for mean in (True, False):
        x, t = torch.tensor(pred * 3, requires_grad=True), torch.tensor(probs, requires_grad=True)
        loss = F.binary_cross_entropy_with_logits(x, t, reduction="mean" if mean else "sum")
        loss.backward()
        out[f"bce.{int(mean)}.loss"], out[f"bce.{int(mean)}.grad"], out[f"bce.{int(mean)}.grad_t"] = loss.detach().numpy(), x.grad.numpy(), t.grad.numpy()
    np.savez(os.path.join(os.path.dirname(os.path.abspath(__file__)), "losses.npz"), **out)
    print("torch", torch.__version__, "->", len(out), "arrays")


if __name__ == "__main__":
    main()
