"""Pins the CPU oracle against the reference's own fixtures, at the reference tests' tolerances:
gradients <= 1e-4 scaled (AutogradModelTests.cs:61-81), training curves: per-step loss <= 1e-3 relative and final
parameters <= 1e-3 scaled (TrainingCurveTests.cs:75-106), optimizer steps <= 1e-6 scaled (OptimizerTests.cs:41-139)."""
import numpy as np
import pytest

import models
from backends import OracleBackend, load_fixture, scaled_diff


@pytest.fixture(scope="module")
def B(oracle_built):
    return OracleBackend()


def test_autograd_encoder_gradients(B):
    fx = load_fixture("autograd", "encoder")
    loss, y, w = models.autograd_encoder(B, fx)
    assert scaled_diff(B.numpy(y), fx["out.y"]) <= 1e-4
    assert abs(float(B.numpy(loss).reshape(-1)[0]) - float(fx["out.loss"].reshape(-1)[0])) <= 1e-4 * abs(float(fx["out.loss"].reshape(-1)[0]))
    B.backward(loss)
    largest = max(np.max(np.abs(fx["grad." + k])) for k in w)
    for k, t in w.items():
        ref = fx["grad." + k]
        g = B.grad(t)
        if np.max(np.abs(ref)) < 1e-5 * largest:   # zero-in-theory gradients (key biases under softmax)
            assert np.max(np.abs(g)) < 1e-5 * largest, k
        else:
            assert scaled_diff(g, ref) <= 1e-4, k


def test_training_mlp_curve(B):
    fx = load_fixture("training", "mlp")
    losses, params = models.train_mlp(B, fx)
    assert np.max(np.abs(losses - fx["out.loss"]) / np.abs(fx["out.loss"])) <= 1e-3
    for k, v in params.items():
        assert scaled_diff(v, fx["out." + k]) <= 1e-3, k


def test_training_encoder_curve(B):
    fx = load_fixture("training", "encoder")
    losses, params = models.train_encoder(B, fx)
    assert np.max(np.abs(losses - fx["out.loss"]) / np.abs(fx["out.loss"])) <= 1e-3
    for k, v in params.items():
        if k.endswith("bk"):
            continue  # key bias: zero true gradient, Adam amplifies rounding noise (TrainingCurveTests.cs:49-60)
        assert scaled_diff(v, fx["out." + k]) <= 1e-3, k


OPTIM = {
    "sgd_plain": ("sgd", dict(lr=0.1)),
    "sgd_momentum": ("sgd", dict(lr=0.1, momentum=0.9)),
    "sgd_nesterov_wd": ("sgd", dict(lr=0.1, momentum=0.9, nesterov=True, weight_decay=1e-2)),
    "sgd_dampening_wd": ("sgd", dict(lr=0.05, momentum=0.8, dampening=0.5, weight_decay=1e-3)),
    "adam": ("adam", dict(lr=1e-2)),
    "adam_l2": ("adam", dict(lr=1e-2, weight_decay=0.1)),
    "adam_amsgrad": ("adam", dict(lr=1e-2, amsgrad=True)),
    "adam_betas": ("adam", dict(lr=3e-3, beta1=0.8, beta2=0.95, eps=1e-6)),
    "adamw": ("adamw", dict(lr=1e-2, weight_decay=0.05)),
    "adamw_amsgrad": ("adamw", dict(lr=1e-2, weight_decay=0.05, amsgrad=True)),
}


def run_optim_case(B, fx, kind, kw):
    kw = dict(kw)
    lr = kw.pop("lr")
    p, q = B.tensor(fx["in.p"], True), B.tensor(fx["in.q"], True)
    opt = B.optimizer(kind, [p, q], lr, **kw)
    out = {}
    for k in range(5):
        for t, name in ((p, "p"), (q, "q")):
            B.set_grad(t, fx[f"in.grad.{name}.{k}"])
        opt.step()
        if k in (0, 4):
            out[k + 1] = (B.numpy(p).copy(), B.numpy(q).copy())
    return out


@pytest.mark.parametrize("name", sorted(OPTIM))
def test_optimizer_steps(B, name):
    fx = load_fixture("training", "optim")
    kind, kw = OPTIM[name]
    out = run_optim_case(B, fx, kind, kw)
    for step, (p, q) in out.items():
        assert scaled_diff(p, fx[f"out.{name}.p.{step}"]) <= 1e-6
        assert scaled_diff(q, fx[f"out.{name}.q.{step}"]) <= 1e-6


def test_clip_norm(B):
    fx = load_fixture("training", "optim")
    for label, max_norm, inf in (("norm_small", 0.5, False), ("norm_large", 100.0, False), ("norm_inf", 0.7, True)):
        p, q = B.tensor(fx["in.p"], True), B.tensor(fx["in.q"], True)
        B.set_grad(p, fx["in.grad.p.0"])
        B.set_grad(q, fx["in.grad.q.0"])
        total = B.clip_norm([p, q], max_norm, inf)
        assert abs(total - float(fx[f"out.clip.{label}.total"][0])) <= 1e-6 * abs(float(fx[f"out.clip.{label}.total"][0]))
        assert scaled_diff(B.grad(p), fx[f"out.clip.{label}.p"]) <= 1e-6
        assert scaled_diff(B.grad(q), fx[f"out.clip.{label}.q"]) <= 1e-6
