"""Learning-rate schedules of the host library against the reference's known answers: the PyTorch-recorded rates in
testdata/training/optim (OptimizerTests.cs:116-139 of the reference, gate 1e-6 relative), the closed form of the warm-up +
cosine schedule (WarmupCosineLrTests.cs:7-20) and the accuracy of the platform-independent cosine (OptimizerTests.cs:141-156).
Pure host arithmetic: runs without a GPU."""
import math

import numpy as np
import pytest

from backends import load_fixture


@pytest.fixture(scope="module")
def omb():
    import om_binding
    om_binding.host_lib()
    return om_binding


def test_schedules_match_the_recorded_rates(omb):
    S = omb.LrSchedule
    fx = load_fixture("training", "optim")
    made = {
        "step": S.step(0.1, 10, 0.5),
        "cosine": S.cosine(0.1, 100, 1e-3),
        "warmup_cosine": S.warmup(S.cosine(0.1, 90, 1e-3), 10, 0.01),
        "onecycle": S.one_cycle(0.1, 100),
    }
    for name, sched in made.items():
        want = fx["out.lr." + name].reshape(-1)
        assert want.size >= 100
        got = np.array([sched.lr_at(i) for i in range(want.size)], np.float64)
        assert np.max(np.abs(got - want) / want) <= 1e-6, name


def test_warmup_cosine_closed_form(omb):
    lr = float(np.float32(6e-5))
    sched = omb.LrSchedule.warmup_cosine(6e-5, 200, 2000, 0.02)
    floor = float(np.float32(0.02))
    for s in range(0, 2101):
        if s < 200:
            want = lr * (s + 1) / 200.0
        else:
            want = lr * (floor + (1 - floor) * 0.5 * (1 + math.cos(math.pi * min(1.0, (s - 200) / 1800.0))))
        assert abs(sched.lr_at(s) - want) <= want * 1e-6, s
    assert sched.lr_at(-5) == sched.lr_at(0)                  # a negative step counts as step 0


def test_series_cosine_is_accurate_and_symmetric(omb):
    cos = omb.LrSchedule.cos
    worst = max(abs(cos(i / 10000.0) - math.cos(math.pi * i / 10000.0)) for i in range(10001))
    assert worst < 1e-15
    assert cos(0.0) == 1.0 and cos(1.0) == -1.0 and abs(cos(0.5)) < 1e-15
    assert cos(-3.0) == 1.0 and cos(7.0) == -1.0              # clamped
    assert all(cos(t) == -cos(1.0 - t) for t in (0.125, 0.25, 0.375))      # 1 - t exact in binary


def test_constant_and_step_by_repeated_squaring(omb):
    S = omb.LrSchedule
    assert S.constant(0.3).lr_at(12345) == float(np.float32(0.3))
    sched = S.step(0.1, 3, 0.5)
    for s in range(40):
        want = float(np.float32(0.1)) * 0.5 ** (s // 3)
        assert sched.lr_at(s) == float(np.float32(want))


def test_bad_schedule_settings_are_rejected(omb):
    S = omb.LrSchedule
    for make in (lambda: S.step(0.1, 0), lambda: S.cosine(0.1, 0), lambda: S.warmup(S.constant(0.1), 0),
                 lambda: S.warmup_cosine(0.1, 0, 10), lambda: S.warmup_cosine(0.1, 10, 10), lambda: S.warmup_cosine(0.1, 2, 10, 1.5),
                 lambda: S.one_cycle(0.1, 1), lambda: S.one_cycle(0.1, 10, 1.0), lambda: S.one_cycle(0.1, 10, 0.0)):
        with pytest.raises(omb.OmError):
            make()
