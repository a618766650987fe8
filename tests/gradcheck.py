"""Finite-difference gradient checks for any backend of tests/backends.py (the CPU oracle tape or the GPU host mirror).

The method is the one the reference's own tests use (src/OneModel.Training/GradientCheck.cs:29-110 and
tests/OneModel.Tests/Tensors/GradCheck.cs:33-70 of the reference): L(x) = sum(W * f(x)) with a fixed random W, the sum
taken in double; the analytic gradient is one backward pass from W; the numeric one is a central difference in float32
inputs with step h = 1e-2; the error is max|analytic - numeric| / max(max|numeric|, 1e-3) and the gate is 5e-3.
"""
import numpy as np

STEP = 1e-2
GATE = 5e-3


def _weights(shape, seed):
    r = np.random.default_rng(1000 + seed)
    return r.uniform(-1.0, 1.0, size=shape).astype(np.float32)


def _objective(B, f, arrays, grads_for, w):
    leaves = [B.tensor(a, False) for a in arrays]
    y = B.numpy(f(B, leaves))
    return float(np.sum(y.astype(np.float64) * w.astype(np.float64)))


def grad_check(B, f, arrays, wrt=None, probes=10, seed=0, step=STEP):
    """Returns {input index: scaled error}. `f(B, leaves)` builds the output tensor from leaf tensors made of `arrays`
    (float32); `wrt` lists the inputs to check (default all); `probes` bounds the elements perturbed per input (all when
    the input is smaller)."""
    arrays = [np.ascontiguousarray(a, np.float32) for a in arrays]
    wrt = list(range(len(arrays))) if wrt is None else list(wrt)
    leaves = [B.tensor(a, i in wrt) for i, a in enumerate(arrays)]
    y = f(B, leaves)
    w = _weights(tuple(B.numpy(y).shape), seed)
    B.backward(B.sum(B.mul(y, B.tensor(w))))
    analytic = {i: np.array(B.grad(leaves[i]), np.float64).reshape(-1) for i in wrt}
    r = np.random.default_rng(seed)
    out = {}
    for i in wrt:
        n = arrays[i].size
        picks = np.arange(n) if n <= probes else r.choice(n, probes, replace=False)
        worst, largest = 0.0, 0.0
        for e in picks:
            flat = arrays[i].reshape(-1)
            orig = flat[e]
            up, down = np.float32(orig + np.float32(step)), np.float32(orig - np.float32(step))
            flat[e] = up
            lp = _objective(B, f, arrays, wrt, w)
            flat[e] = down
            lm = _objective(B, f, arrays, wrt, w)
            flat[e] = orig
            numeric = (lp - lm) / (float(up) - float(down))
            largest = max(largest, abs(numeric))
            worst = max(worst, abs(analytic[i][e] - numeric))
        out[i] = worst / max(largest, 1e-3)
    return out


# ---- the cases: one per backward function of the hot path -------------------------------------------------------------
def _u(r, shape, lo=-1.0, hi=1.0):
    return r.uniform(lo, hi, size=shape).astype(np.float32)


def _away_from_zero(r, shape, gap=0.05):
    """Values in +-[gap, 1]: a ReLU kink or a sign change stays outside the difference step."""
    v = r.uniform(gap, 1.0, size=shape) * r.choice([-1.0, 1.0], size=shape)
    return v.astype(np.float32)


def _distinct(r, shape, spacing=0.1):
    """Shuffled multiples of `spacing`: no two values within the difference step, so a max-pool argmax never flips."""
    n = int(np.prod(shape))
    return (r.permutation(n).astype(np.float32) * np.float32(spacing) - np.float32(n * spacing / 2)).reshape(shape)


def cases():
    """[(name, f(B, leaves) -> tensor, [arrays], wrt or None)]"""
    r = np.random.default_rng(20240607)
    out = []

    def case(name, f, arrays, wrt=None):
        out.append((name, f, arrays, wrt))

    case("add_mul_broadcast", lambda B, t: B.mul(B.add(t[0], t[1]), t[0]), [_u(r, (3, 4)), _u(r, (4,))])
    case("sub_broadcast_rows", lambda B, t: B.sub(t[0], t[1]), [_u(r, (2, 3, 4)), _u(r, (3, 1))])
    case("relu", lambda B, t: B.relu(t[0]), [_away_from_zero(r, (4, 5))])
    case("gelu", lambda B, t: B.gelu(t[0]), [_u(r, (4, 5), -3, 3)])
    case("matmul", lambda B, t: B.matmul(t[0], t[1]), [_u(r, (3, 5)), _u(r, (5, 4))])
    case("linear_bias", lambda B, t: B.linear(t[0], t[1], t[2]), [_u(r, (2, 3, 5)), _u(r, (4, 5)), _u(r, (4,))])
    case("mean_axis", lambda B, t: B.mean(t[0], 1), [_u(r, (3, 4, 2))])
    case("sum_all", lambda B, t: B.mul(B.sum(t[0]), B.sum(t[0])), [_u(r, (3, 4))])
    case("log_softmax", lambda B, t: B.log_softmax(t[0]), [_u(r, (3, 7), -2, 2)])
    tgt = np.array([1, 0, 6, 3], np.int64)
    case("cross_entropy", lambda B, t: B.cross_entropy(t[0], B.ids(tgt)), [_u(r, (4, 7), -2, 2)])
    case("layer_norm", lambda B, t: B.layer_norm(t[0], t[1], t[2]), [_u(r, (3, 2, 8), -2, 2), _u(r, (8,), 0.5, 1.5), _u(r, (8,))])
    ids = np.array([[1, 4, 4], [0, 2, 1]], np.int64)
    case("embedding", lambda B, t: B.embedding(t[0], B.ids(ids)), [_u(r, (5, 6))])
    mask = np.where(r.uniform(size=(5, 6)) < 0.2, np.float32(-1e9), np.float32(0)).astype(np.float32)
    mask[..., 0] = 0
    case("attention", lambda B, t: B.attention(t[0], t[1], t[2]), [_u(r, (1, 2, 5, 4)), _u(r, (1, 2, 6, 4)), _u(r, (1, 2, 6, 4))])
    case("attention_mask", lambda B, t: B.attention(t[0], t[1], t[2], mask), [_u(r, (1, 2, 5, 4)), _u(r, (1, 2, 6, 4)), _u(r, (1, 2, 6, 4))])

    def bn(B, t):
        return B.batch_norm2d(t[0], t[1], t[2], B.running(np.zeros(3)), B.running(np.ones(3)), True)
    case("batch_norm2d", bn, [_u(r, (4, 3, 3, 2), -2, 2), _u(r, (3,), 0.5, 1.5), _u(r, (3,))])
    case("conv2d_stride2_pad1", lambda B, t: B.conv2d(t[0], t[1], t[2], 2, 1), [_u(r, (2, 3, 7, 6)), _u(r, (4, 3, 3, 3)), _u(r, (4,))])
    case("max_pool2d", lambda B, t: B.max_pool2d(t[0], 2), [_distinct(r, (2, 2, 6, 4))])
    case("avg_pool2d", lambda B, t: B.avg_pool2d(t[0], 2), [_u(r, (2, 2, 6, 4))])
    lstm = [_u(r, (5, 2, 3)), _u(r, (16, 3), -0.5, 0.5), _u(r, (16, 4), -0.5, 0.5), _u(r, (16,), -0.5, 0.5), _u(r, (16,), -0.5, 0.5)]
    case("lstm_layer", lambda B, t: B.lstm_layer(t[0], t[1], t[2], t[3], t[4], False), [a.copy() for a in lstm])
    case("lstm_layer_reverse", lambda B, t: B.lstm_layer(t[0], t[1], t[2], t[3], t[4], True), [a.copy() for a in lstm])
    gru = [_u(r, (4, 2, 3)), _u(r, (12, 3), -0.5, 0.5), _u(r, (12, 4), -0.5, 0.5), _u(r, (12,), -0.5, 0.5), _u(r, (12,), -0.5, 0.5), _u(r, (2, 4))]
    case("gru_layer_h0", lambda B, t: B.gru_layer(t[0], t[1], t[2], t[3], t[4], t[5], False), [a.copy() for a in gru])
    case("gru_layer_reverse", lambda B, t: B.gru_layer(t[0], t[1], t[2], t[3], t[4], None, True), [a.copy() for a in gru[:5]])
    case("concat", lambda B, t: B.concat([t[0], t[1], t[0]], 1), [_u(r, (2, 3)), _u(r, (2, 2))])
    case("matmul_batched_broadcast", lambda B, t: B.matmul_batched(t[0], t[1]), [_u(r, (2, 1, 3, 4)), _u(r, (3, 4, 2))])
    case("conv_transpose2d", lambda B, t: B.conv_transpose2d(t[0], t[1], t[2], 2, 1, 1, 2),
         [_u(r, (1, 4, 3, 3)), _u(r, (4, 3, 3, 3)), _u(r, (6,))])
    case("conv1d_dilated_groups", lambda B, t: B.conv1d(t[0], t[1], t[2], 2, 0, 3, 2, 2), [_u(r, (2, 4, 13)), _u(r, (6, 2, 3)), _u(r, (6,))])
    case("resize2d_nearest", lambda B, t: B.resize2d(t[0], 5, 7, 0, False), [_u(r, (1, 2, 3, 4))])
    case("resize2d_bilinear", lambda B, t: B.resize2d(t[0], 5, 7, 1, False), [_u(r, (1, 2, 3, 4))])
    case("resize2d_bilinear_corners", lambda B, t: B.resize2d(t[0], 6, 3, 1, True), [_u(r, (1, 2, 3, 4))])
    case("erf", lambda B, t: B.erf(t[0]), [_u(r, (3, 4), -2, 2)])
    case("exp", lambda B, t: B.exp(t[0]), [_u(r, (3, 4))])
    case("sqrt", lambda B, t: B.sqrt(t[0]), [_u(r, (3, 4), 0.5, 2.0)])
    case("pow", lambda B, t: B.pow(t[0], 2.5), [_u(r, (3, 4), 0.5, 2.0)])
    cond = (r.uniform(size=(3, 4)) < 0.5).astype(np.int32)
    case("where", lambda B, t: B.where(cond, t[0], t[1]), [_u(r, (3, 4)), _u(r, (3, 4))])
    gidx = np.array([[2, 0], [1, 1]], np.int64)
    case("gather", lambda B, t: B.gather(t[0], gidx, 1), [_u(r, (2, 3, 4))])

    # Dropout (a fixed call number, so the mask is the same for every evaluation) and the loss family (Losses.cs:14-129).
    case("dropout", lambda B, t: B.dropout(t[0], 0.4, 77, 3), [_u(r, (5, 7))])
    smooth_t = np.array([2, -100, 0, 5], np.int64)
    case("cross_entropy_smoothed", lambda B, t: B.cross_entropy_smoothed(t[0], B.ids(smooth_t), 0.2, -100, True), [_u(r, (4, 6), -2, 2)])
    goal = _u(r, (3, 4))
    case("mse_loss", lambda B, t: B.mse_loss(t[0], B.tensor(goal), True), [_u(r, (3, 4))])
    case("l1_loss", lambda B, t: B.l1_loss(t[0], B.tensor(goal), False), [goal + _away_from_zero(r, (3, 4))])
    case("bce_with_logits", lambda B, t: B.bce_with_logits(t[0], t[1], True), [_u(r, (3, 4), -3, 3), _u(r, (3, 4), 0, 1)])

    # CTC through LogSoftmax: ordinary, repeated labels that need a blank between, a shorter input (CtcLossTests.cs:41-64).
    targets, in_len, tgt_len = [1, 2, 2, 3, 1, 1], [7, 6, 4], [2, 3, 1]
    for red, name in ((0, "none"), (1, "mean"), (2, "sum")):
        case(f"ctc_{name}", lambda B, t, red=red: B.ctc_loss(B.log_softmax(t[0]), targets, in_len, tgt_len, 0, red, False), [_u(r, (7, 3, 4), -1.5, 1.5)])
    case("ctc_empty_target_blank3_zero_inf",
         lambda B, t: B.ctc_loss(B.log_softmax(t[0]), [0, 1, 2, 2], [5, 5, 2, 1], [0, 2, 2, 0], 3, 1, True), [_u(r, (5, 4, 4), -1.5, 1.5)])
    return out
