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


def check_grads(B, fx, w, tol=1e-4):
    largest = max(np.max(np.abs(fx["grad." + k])) for k in w)
    for k, t in w.items():
        ref = fx["grad." + k]
        if np.max(np.abs(ref)) < 1e-5 * largest:      # zero-in-theory gradients (a bias in front of batch norm)
            assert np.max(np.abs(B.grad(t))) < 1e-5 * largest, k
        else:
            assert scaled_diff(B.grad(t), ref) <= tol, k


def test_autograd_cnn_gradients(B):
    fx = load_fixture("autograd", "cnn")
    loss, logits, w, rs = models.autograd_cnn(B, fx)
    assert scaled_diff(B.numpy(logits), fx["out.logits"]) <= 1e-4
    B.backward(loss)
    check_grads(B, fx, w)
    for r, k in zip(rs, ("rm1", "rv1", "rm2", "rv2")):
        assert scaled_diff(B.running_numpy(r), fx["out." + k]) <= 1e-5, k


def test_autograd_crnn_gradients_and_ctc_losses(B):
    fx = load_fixture("autograd", "crnn")
    loss, lp, w = models.autograd_crnn(B, fx)
    assert scaled_diff(B.numpy(lp), fx["out.lp"]) <= 1e-4
    assert abs(float(B.numpy(loss).reshape(-1)[0]) - float(fx["out.loss"].reshape(-1)[0])) <= 1e-5 * abs(float(fx["out.loss"].reshape(-1)[0]))
    B.backward(loss)
    check_grads(B, fx, w)


def test_autograd_gru_gradients(B):
    fx = load_fixture("autograd", "gru")
    loss, y, w = models.autograd_gru(B, fx)
    assert scaled_diff(B.numpy(y), fx["out.y"]) <= 1e-5
    ref = float(fx["out.loss"].reshape(-1)[0])
    assert abs(float(B.numpy(loss).reshape(-1)[0]) - ref) <= 1e-5 * abs(ref)
    B.backward(loss)
    check_grads(B, fx, w)


def test_autograd_decoder_gradients(B):
    fx = load_fixture("autograd", "decoder")
    loss, a, c, w = models.autograd_decoder(B, fx)
    assert scaled_diff(B.numpy(a), fx["out.a"]) <= 1e-5
    assert scaled_diff(B.numpy(c), fx["out.c"]) <= 1e-5
    B.backward(loss)
    check_grads(B, fx, w)


def sparse_case(fx):
    ids = fx["in.ids"].astype(np.int64)            # [steps, 6, 5], id 0 is the padding row
    return fx["in.emb"].copy(), fx["in.hw"].copy(), fx["in.hb"].copy(), ids, fx["in.y"].astype(np.int64)


def test_sparse_adam_and_sparse_sgd_against_the_reference_fixture(oracle_built):
    """testdata/training/sparse (SparseAndFrozenTests.cs:255-420 of the reference): Embedding(40, 8, padding 0) -> mean over
    the sequence -> Linear(8, 3) -> cross-entropy; the table is updated by the row-sparse optimizers, the head by AdamW / Adam /
    Sgd. Losses and final parameters within the reference's 1e-6."""
    from oracle import oracle as K, tape as A
    fx = load_fixture("training", "sparse")

    def run(name, table_step, head_step):
        emb, hw, hb, ids, y = sparse_case(fx)
        losses, state = [], {}
        for s in range(ids.shape[0]):
            E, W, Bv = A.T(emb, True), A.T(hw, True), A.T(hb, True)
            loss = A.cross_entropy(A.linear(A.mean(A.embedding(E, ids[s], 0), 1), W, Bv), y[s])
            loss.backward()
            losses.append(float(loss.v))
            touched = K.rows_touched(ids[s], 40, 0)
            assert not np.any(E.grad[touched == 0])          # the dense-format gradient is zero off the touched rows
            if s == 0 and name == "sgd":
                assert scaled_diff(E.grad, fx["out.sgd.grad0"]) <= 1e-6
            table_step(emb, E.grad, touched, s + 1, state)
            head_step([hw, hb], [W.grad, Bv.grad], s + 1, state)
        assert np.max(np.abs(np.array(losses) - fx[f"out.{name}.loss"]) / np.abs(fx[f"out.{name}.loss"])) <= 1e-6
        for got, key in ((emb, "emb"), (hw, "hw"), (hb, "hb")):
            assert scaled_diff(got, fx[f"out.{name}.{key}"]) <= 1e-6, (name, key)

    def adam_heads(lr, wd, decoupled):
        def step(ps, gs, t, state):
            for i, (p, g) in enumerate(zip(ps, gs)):
                st = state.setdefault(("h", i), dict(m=np.zeros_like(p), v=np.zeros_like(p)))
                K.adam_step(p, g, st["m"], st["v"], None, t, lr, 0.9, 0.999, 1e-8, wd, decoupled, False)
        return step

    def sparse_adam(lr, b1, b2, eps):
        def step(p, g, touched, t, state):
            st = state.setdefault("t", dict(m=np.zeros_like(p), v=np.zeros_like(p)))
            K.sparse_adam_step(p, g, st["m"], st["v"], touched, t, lr, b1, b2, eps)
        return step

    def sgd_heads(ps, gs, t, state):
        for p, g in zip(ps, gs):
            K.sgd_step(p, g, np.zeros_like(p), True, 0.5)

    run("sgd", lambda p, g, touched, t, state: K.sparse_sgd_step(p, g, touched, 0.5), sgd_heads)
    run("sparseadam", sparse_adam(0.05, 0.9, 0.999, 1e-3), adam_heads(0.01, 0.01, True))
    run("sparseadam2", sparse_adam(0.02, 0.8, 0.95, 1e-8), adam_heads(0.01, 0.0, False))


def check_graph_ops(B, tol):
    """The graph-op family against tests/golden/graph_ops.npz (PyTorch CPU, generated by tests/golden/make_graphops_golden.py)."""
    import os
    gold = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "graph_ops.npz"))
    loss, out, w = models.graph_ops_case(B)
    assert scaled_diff(B.numpy(out), gold["out"]) <= tol
    assert abs(float(B.numpy(loss).reshape(-1)[0]) - float(gold["loss"])) <= tol * 10 * abs(float(gold["loss"]))
    B.backward(loss)
    for k, t in w.items():
        assert scaled_diff(B.grad(t), gold["grad_" + k]) <= tol, k


def check_conv1d(B, tol):
    """Conv1d against tests/golden/conv1d.npz (PyTorch CPU, generated by tests/golden/make_graphops_golden.py)."""
    import os
    import models
    gold = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "conv1d.npz"))
    for i, case in enumerate(models.CONV1D_CASES):
        loss, y, leaves = models.conv1d_case(B, case)
        B.backward(loss)
        assert scaled_diff(B.numpy(y), gold[f"{i}.out"]) <= tol, (i, "out")
        assert abs(float(B.numpy(loss).reshape(-1)[0]) - float(gold[f"{i}.loss"])) <= 10 * tol * max(1.0, abs(float(gold[f"{i}.loss"]))), i
        for k, t in leaves.items():
            assert scaled_diff(B.grad(t), gold[f"{i}.grad_{k}"]) <= tol, (i, k)


def check_losses(B, tol):
    """Cross entropy with label smoothing and ignored rows, MSE, L1 and BCE-with-logits (Losses.cs:14-129 of the reference)
    against tests/golden/losses.npz (PyTorch CPU, tests/golden/make_losses_golden.py): values and input gradients."""
    import os
    gold = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "losses.npz"))
    CE_CASES = [(0.1, True), (0.3, True), (0.2, False), (1.0, True)]     # as in tests/golden/make_losses_golden.py

    def run(build, leaves_np, want_loss, want_grads):
        leaves = [B.tensor(a, True) for a in leaves_np]
        loss = build(*leaves)
        B.backward(loss)
        got = float(B.numpy(loss).reshape(-1)[0])
        assert abs(got - float(want_loss)) <= 10 * tol * max(1.0, abs(float(want_loss))), (got, float(want_loss))
        for t, w in zip(leaves, want_grads):
            assert scaled_diff(B.grad(t), w) <= tol

    tg = gold["targets"]
    for i, (eps, mean) in enumerate(CE_CASES):
        run(lambda x: B.cross_entropy_smoothed(x, B.ids(tg), eps, -100, mean), [gold["logits"]], gold[f"ce{i}.loss"], [gold[f"ce{i}.grad"]])
    for mean in (True, False):
        goal = gold["goal"]
        run(lambda x: B.mse_loss(x, B.tensor(goal), mean), [gold["pred"]], gold[f"mse.{int(mean)}.loss"], [gold[f"mse.{int(mean)}.grad"]])
        run(lambda x: B.l1_loss(x, B.tensor(goal), mean), [gold["pred"]], gold[f"l1.{int(mean)}.loss"], [gold[f"l1.{int(mean)}.grad"]])
        run(lambda x, t: B.bce_with_logits(x, t, mean), [gold["pred"] * 3, gold["probs"]], gold[f"bce.{int(mean)}.loss"],
            [gold[f"bce.{int(mean)}.grad"], gold[f"bce.{int(mean)}.grad_t"]])
    # No counted row: the smoothed mean is NaN, as the reference's 1/0 factor makes it (Losses.cs:55-58).
    x = B.tensor(gold["logits"][:2], True)
    assert np.isnan(B.numpy(B.cross_entropy_smoothed(x, B.ids(np.array([-100, -100])), 0.1, -100, True))).all()


def test_loss_family_against_pytorch_golden(B):
    check_losses(B, 2e-6)


def test_splitmix_and_dropout_mask_known_answers():
    """The SplitMix64 finaliser against the published first outputs of the generator seeded with 0, and the properties
    the reference's own Dropout test checks (ModuleAndLossTests.cs:62-85): seeded, a new mask per call, about p zeros,
    kept elements exactly float32(1/(1-p))."""
    from oracle import tape
    g = 0x9E3779B97F4A7C15
    assert [tape.splitmix_finish((i + 1) * g) for i in range(3)] == [0xE220A8397B1DCDAF, 0x6E789E6AA1B965F4, 0x06C45D188009454F]
    a, b, c = tape.dropout_mask(42, 0, 0.3, 1000), tape.dropout_mask(42, 0, 0.3, 1000), tape.dropout_mask(42, 1, 0.3, 1000)
    assert np.array_equal(a, b) and not np.array_equal(a, c)
    assert 240 <= int((a == 0).sum()) <= 360
    assert np.all(a[a != 0] == np.float32(1.0) / np.float32(0.7))
    # element i agrees with the scalar recurrence written out on Python integers
    stream = tape.splitmix_finish(42 + 1 * g)
    for i in (0, 1, 999):
        u = np.float32(tape.splitmix_finish(stream + (i + 1) * g) >> 40) * np.float32(1.0 / 16777216.0)
        assert c[i] == (np.float32(1.0) / np.float32(0.7) if u >= np.float32(0.3) else 0.0)


def check_frozen_encoder(B, early_tol, loss_tol, param_tol):
    """testdata/training/frozen: the encoder curve with the embedding and layer 0 frozen (requires_grad False, left out of
    the optimizer). Frozen parameters receive no gradient and keep their bits; the rest follows PyTorch's curve
    (SparseAndFrozenTests.cs:48-118 of the reference: losses 1e-6 over the first 20 steps, 1e-5 overall, parameters 2e-6,
    the key bias excluded since its true gradient is zero)."""
    import models
    fx, want = load_fixture("training", "encoder"), load_fixture("training", "frozen")
    losses, params = models.train_encoder(B, fx, frozen=("emb", "l0"))
    rel = np.abs(losses - want["out.loss"]) / np.abs(want["out.loss"])
    assert rel[:20].max() <= early_tol and rel.max() <= loss_tol
    frozen = 0
    for k, v in params.items():
        if k == "emb" or k.startswith("l0."):
            frozen += 1
            assert np.array_equal(v, fx["in." + k]) and np.array_equal(v, want["out." + k]), k
        elif not k.endswith("bk"):
            assert scaled_diff(v, want["out." + k]) <= param_tol, k
    assert frozen > 10


def check_conv1d_reference_grid(B, tol):
    """Every case of the reference's testdata/conv1d/grid (strides, paddings incl. "same"/"valid", dilations, groups, with
    and without bias): y and the gradients of x, w, b (Conv1dTests.cs:76-118 of the reference, gate 1e-6)."""
    import models
    from backends import load_fixture_manifest
    fx, cases = load_fixture("conv1d", "grid"), load_fixture_manifest("conv1d", "grid")["cases"]
    assert len(cases) >= 10
    for i, case in enumerate(cases):
        loss, y, leaves = models.conv1d_grid_case(B, fx, i, case)
        assert tuple(B.numpy(y).shape) == fx[f"c{i}.out.y"].shape, i
        B.backward(loss)
        assert scaled_diff(B.numpy(y), fx[f"c{i}.out.y"]) <= tol, (i, "y")
        for k, t in leaves.items():
            assert scaled_diff(B.grad(t), fx[f"c{i}.grad.{k}"]) <= tol, (i, k)


def check_conv1d_training(B, loss_tol, param_tol):
    """testdata/conv1d/train: 20 SGD-momentum steps of a two-layer Conv1d net; the reference gates the losses at 1e-5
    relative (Conv1dTests.cs:258-307)."""
    import models
    fx = load_fixture("conv1d", "train")
    losses, params = models.train_conv1d(B, fx)
    assert np.max(np.abs(losses - fx["out.loss"]) / np.abs(fx["out.loss"])) <= loss_tol
    assert losses[-1] < losses[0]
    for k, v in params.items():
        assert scaled_diff(v, fx["out." + k]) <= param_tol, k


def test_frozen_encoder_against_the_reference_curve(B):
    check_frozen_encoder(B, 1e-6, 1e-5, 2e-6)


def test_conv1d_against_the_reference_grid(B):
    check_conv1d_reference_grid(B, 1e-6)


def test_conv1d_training_against_the_reference_curve(B):
    check_conv1d_training(B, 1e-5, 1e-5)


def test_conv1d_against_pytorch_golden(B):
    check_conv1d(B, 2e-6)


def test_graph_ops_against_pytorch_golden(B):
    check_graph_ops(B, 1e-6)


def test_training_cnn_curve(B):
    fx = load_fixture("training", "cnn")
    losses, norms, params, rs = models.train_cnn(B, fx)
    assert np.max(np.abs(losses - fx["out.loss"]) / np.abs(fx["out.loss"])) <= 1e-3
    assert np.max(np.abs(norms - fx["out.gradnorm"]) / np.abs(fx["out.gradnorm"])) <= 1e-3
    for k, v in params.items():
        if k in ("c1b", "c2b"):
            continue  # a bias in front of batch norm has zero true gradient (TrainingCurveTests.cs:49-60)
        assert scaled_diff(v, fx["out." + k]) <= 1e-3, k


def test_ctc_reductions_and_infeasible_targets(oracle_built):
    K = oracle_built
    fx = load_fixture("autograd", "crnn")
    lp = fx["out.lp"]
    tg, il, tl = fx["in.targets"].astype(np.int32), fx["in.input_lengths"].astype(np.int32), fx["in.target_lengths"].astype(np.int32)
    for red, name in ((0, "none"), (2, "sum"), (1, "mean")):
        got, _ = K.ctc_loss(lp, tg, tl, il, 0, red)
        assert np.max(np.abs(np.atleast_1d(got) - fx["out.ctc_" + name]) / np.abs(fx["out.ctc_" + name])) <= 1e-5
    short = np.array([12, 2], np.int32)
    got, _ = K.ctc_loss(lp, tg, tl, short, 0, 0, False)
    assert np.isinf(got[1]) and np.isinf(fx["out.ctc_inf_none"][1]) and abs(got[0] - fx["out.ctc_inf_none"][0]) <= 1e-5 * abs(got[0])
    got, _ = K.ctc_loss(lp, tg, tl, short, 0, 0, True)
    assert got[1] == 0.0 and fx["out.ctc_zeroinf_none"][1] == 0.0


def test_ctc_greedy_known_answers(oracle_built):
    """testdata/ctc/cases.json: greedy labels and the first / last frame of every run are exact integers (CtcTests.cs:26-60)."""
    import json, os
    from backends import ROOT
    K = oracle_built
    cases = json.load(open(os.path.join(ROOT, "tests", "golden", "reference_testdata", "ctc", "cases.json")))["cases"]
    checked = 0
    for c in cases:
        t, n, blank = c["steps"], c["classes"], c["blank"]
        scores = np.array(c["scores"], np.float32).reshape(t, 1, n)
        labels, first, last, lengths = K.ctc_greedy(scores, None, blank)
        k = int(lengths[0])
        assert labels[0, :k].tolist() == c["greedy"]["labels"]
        assert first[0, :k].tolist() == c["greedy"]["first"] and last[0, :k].tolist() == c["greedy"]["last"]
        checked += 1
    assert checked >= 10


def test_row_sparse_gradient_restatement_against_the_reference_fixture(oracle_built):
    """EmbeddingSparseBackward / RowSparseGradient (BackwardNn.cs:548-600, RowSparseGradient.cs:14-120) restated in the oracle,
    on testdata/training/sparse as SparseAndFrozenTests.cs:251-283 uses it: the rows are strictly ascending without the
    padding row, the sparse gradient scatters to the dense gradient bit for bit and matches the recorded gradient of step 0
    within 1e-6; Merge is the union with a's values first."""
    from oracle import oracle as K, tape as A
    fx = load_fixture("training", "sparse")
    emb, hw, hb, ids, y = sparse_case(fx)
    E, W, Bv = A.T(emb, True), A.T(hw, True), A.T(hb, True)
    looked = A.embedding(E, ids[0], 0)
    loss = A.cross_entropy(A.linear(A.mean(looked, 1), W, Bv), y[0])
    loss.backward()
    dense = E.grad
    rows = np.nonzero(K.rows_touched(ids[0], 40, 0))[0].astype(np.int32)
    # the gradient that reaches the lookup's output: softmax - onehot over the 6 rows, through the head, spread over the
    # 5 positions of the mean
    logits = A.linear(A.mean(A.embedding(A.T(emb), ids[0], 0), 1), A.T(hw), A.T(hb)).v
    p = np.exp(logits - logits.max(1, keepdims=True))
    p = (p / p.sum(1, keepdims=True)).astype(np.float32)
    p[np.arange(6), y[0]] -= 1
    dpooled = (p / np.float32(6)) @ hw
    up = np.repeat((dpooled / np.float32(5))[:, None, :], 5, axis=1).astype(np.float32)
    r, v = K.embedding_bwd_sparse(up, ids[0], 0)
    assert np.array_equal(r, rows) and np.all(np.diff(r) > 0) and 0 not in r and 3 < len(r) < 40
    assert np.array_equal(K.rowsparse_to_dense(r, v, 40), K.embedding_bwd(up, ids[0], 40, 8, 0))
    assert scaled_diff(K.rowsparse_to_dense(r, v, 40), fx["out.sgd.grad0"]) <= 1e-6
    assert scaled_diff(dense, fx["out.sgd.grad0"]) <= 1e-6
    # Merge: union of two lookups' gradients equals the gradient of the concatenated lookup when the second follows the first
    r2, v2 = K.embedding_bwd_sparse(up[::-1].copy(), ids[1], 0)
    mr, mv = K.rowsparse_merge(r, v, r2, v2)
    assert np.array_equal(mr, np.union1d(r, r2))
    want = K.rowsparse_to_dense(r, v, 40) + K.rowsparse_to_dense(r2, v2, 40)
    assert np.array_equal(K.rowsparse_to_dense(mr, mv, 40), want)
    # nothing but padding: no rows
    r0, v0 = K.embedding_bwd_sparse(np.ones((3, 8), np.float32), np.zeros(3, np.int64), 0)
    assert r0.size == 0 and v0.shape == (0, 8)


def test_bias_sum_order_of_the_bf16_tier_stays_within_fp32_rounding_of_the_plain_sum(oracle_built):
    """oracle.colsum_bf16 restates the order in which the device adds a bias gradient from the bfloat16 gradient (16 rows per
    lane in fp32, lanes and chunks of 512 rows in double). Against the plain double sum of the same rounded values it may
    differ by the fp32 roundings of the 16-row lane sums only; ragged row counts, one row and exact cases included."""
    K = oracle_built
    r = np.random.default_rng(4)
    for rows, cols in [(16384, 24), (1000, 16), (513, 8), (1, 8), (31, 40)]:
        g = r.standard_normal((rows, cols)).astype(np.float32)
        got = K.colsum_bf16(g)
        plain = K.round_bf16(g).astype(np.float64).sum(0)
        assert got.dtype == np.float32 and got.shape == (cols,)
        assert np.max(np.abs(got - plain)) <= 4e-6 * np.sqrt(rows) + 1e-6 * np.max(np.abs(plain))
    # values whose sums are exact in fp32 (small integers): the order cannot matter, the result is the integer sum
    ints = r.integers(-8, 9, (2000, 8)).astype(np.float32)
    assert np.array_equal(K.colsum_bf16(ints), ints.astype(np.float64).sum(0).astype(np.float32))
