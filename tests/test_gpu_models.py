"""Model-level parity on the GPU through the host mirror (Tensor / Ops / Backprop / optimizers above the C ABI):
the reference's own fixtures at the reference's tolerances, and step-by-step agreement with the CPU oracle."""
import numpy as np
import pytest

import models
from backends import GpuBackend, OracleBackend, load_fixture, scaled_diff
from test_oracle_golden import (OPTIM, check_conv1d, check_conv1d_reference_grid, check_conv1d_training,
                                check_frozen_encoder, check_graph_ops, check_losses, run_optim_case)

pytestmark = pytest.mark.gpu


@pytest.fixture()
def B(ctx):
    ctx.set_flags(0)
    return GpuBackend(ctx)


def test_autograd_encoder_gradients(B):
    fx = load_fixture("autograd", "encoder")
    loss, y, w = models.autograd_encoder(B, fx)
    assert scaled_diff(B.numpy(y), fx["out.y"]) <= 1e-4
    B.backward(loss)
    largest = max(np.max(np.abs(fx["grad." + k])) for k in w)
    for k, t in w.items():
        ref = fx["grad." + k]
        if np.max(np.abs(ref)) < 1e-5 * largest:
            assert np.max(np.abs(B.grad(t))) < 1e-5 * largest, k
        else:
            assert scaled_diff(B.grad(t), ref) <= 1e-4, k


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
        if not k.endswith("bk"):
            assert scaled_diff(v, fx["out." + k]) <= 1e-3, k


def test_training_mlp_matches_oracle_closely(B, oracle_built):
    """Same program on both sides: 100 SGD steps stay within 1e-5 scaled (fp32 FMA products are bit-identical;
    only double-accumulated sums may round differently)."""
    fx = load_fixture("training", "mlp")
    lg, pg = models.train_mlp(B, fx)
    lo, po = models.train_mlp(OracleBackend(), fx)
    assert np.max(np.abs(lg - lo) / np.abs(lo)) <= 1e-5
    for k in pg:
        assert scaled_diff(pg[k], po[k]) <= 1e-5, k


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
        ref = float(fx[f"out.clip.{label}.total"][0])
        assert abs(total - ref) <= 1e-6 * abs(ref)
        assert scaled_diff(B.grad(p), fx[f"out.clip.{label}.p"]) <= 1e-6
        assert scaled_diff(B.grad(q), fx[f"out.clip.{label}.q"]) <= 1e-6


def test_engine_semantics(B):
    """Diamond sums, retain-graph rule, no-grad, shape errors (tests/OneModel.Tests/Tensors/BackwardEngineTests.cs:12-106)."""
    import om_binding as omb
    x = B.tensor(np.array([1.0, 2.0, 3.0]), True)
    y = B.add(B.mul(x, x), x)            # x is used three times
    loss = B.sum(y)
    B.backward(loss)
    assert np.array_equal(B.grad(x), np.array([3.0, 5.0, 7.0], np.float32))
    with pytest.raises(omb.OmError):     # saved tensors were released by the first backward
        B.backward(loss)
    with omb.no_grad():
        z = B.mul(x, x)
    assert not z.requires_grad
    with pytest.raises(omb.ShapeError):
        B.add(B.tensor(np.zeros((2, 3))), B.tensor(np.zeros((4,))))
    with pytest.raises(omb.ShapeError):
        B.backward(B.mul(x, x))          # not a one-element tensor
    x.zero_grad()
    assert not B.grad(x).any()


def test_in_place_change_of_a_saved_tensor_is_caught(B):
    """BackwardEngineTests.InPlaceChangeOfASavedTensorIsCaught (BackwardEngineTests.cs:66-75): a tensor saved by the forward
    pass remembers its storage version (SavedTensor, Autograd.cs:198-238); a write into that storage before the backward
    pass reads it raises the version exception instead of producing a gradient from the changed values. A write after the
    pass has released its records (what an optimizer does) is fine."""
    import om_binding as omb
    x = B.tensor(np.array([1.0, 2.0]), True)
    w = B.tensor(np.array([3.0, 4.0]))
    y = B.sum(B.mul(x, w))
    w.copy_from(np.array([9.0, 4.0], np.float32))
    with pytest.raises(omb.TensorVersionError) as e:
        B.backward(y)
    assert "modified in place" in str(e.value)
    # The same graph without the write, then a write after the backward pass.
    x2 = B.tensor(np.array([1.0, 2.0]), True)
    y2 = B.sum(B.mul(x2, w))
    B.backward(y2)
    w.copy_from(np.array([0.0, 0.0], np.float32))
    assert np.array_equal(B.grad(x2), np.array([9.0, 4.0], np.float32))
    # Writing into a parameter between forward and backward is caught for the fused records too (Linear saves its weights).
    lin_w = B.tensor(np.ones((4, 8), np.float32), True)
    out = B.sum(B.linear(B.tensor(np.ones((2, 8), np.float32), True), lin_w, None))
    lin_w.copy_from(np.zeros((4, 8), np.float32))
    with pytest.raises(omb.TensorVersionError):
        B.backward(out)


@pytest.mark.parametrize("tf32", [False, True])
@pytest.mark.parametrize("b,l,heads,dh,packed", [(3, 128, 4, 32, False), (2, 50, 3, 16, False), (2, 128, 12, 32, True),
                                                 (2, 300, 4, 64, False), (2, 256, 3, 32, True), (1, 128, 2, 64, False)])
def test_attention_over_heads_equals_the_permuted_form(ctx, B, tf32, b, l, heads, dh, packed):
    """Ops.AttentionHeads on [batch, length, heads*d] activations against the reference's form (Reshape + Permute around
    Ops.Attention, Layers.cs:503-520): values and all three input gradients. With the fp32 products the two run the same
    arithmetic per (batch, head) and agree to the bit; on the tensor pipe both round operands the same way. `packed`
    feeds q, k, v as column slices of one [batch, length, 3*width] tensor (row-pitched views, no copy)."""
    import om_binding as omb
    ctx.set_flags(omb.OM_TF32 if tf32 else 0)
    try:
        d = heads * dh
        r = np.random.default_rng(b * l + heads)
        w = r.standard_normal((b, l, d)).astype(np.float32)
        if packed:
            qkv = r.standard_normal((b, l, 3 * d)).astype(np.float32)
            srcs = [qkv[:, :, i * d:(i + 1) * d].copy() for i in range(3)]
        else:
            srcs = [r.standard_normal((b, l, d)).astype(np.float32) for _ in range(3)]

        def run(fused):
            if packed:
                root = B.tensor(qkv, True)
                q, k, v = (root.slice(2, i * d, (i + 1) * d) for i in range(3))
                leaves = [root]
            else:
                leaves = [B.tensor(s, True) for s in srcs]
                q, k, v = leaves
            if fused:
                a = omb.call("attention_heads", [q, k, v, None], ints=[heads], floats=[0.0])
            else:
                split = lambda z: omb.call("contiguous", [z]).reshape(b, l, heads, dh).permute(0, 2, 1, 3)
                a = omb.call("attention", [split(q), split(k), split(v), None], floats=[0.0]).permute(0, 2, 1, 3).reshape(b, l, d)
            B.backward(B.sum(B.mul(a, B.tensor(w))))
            return a.numpy(), [B.grad(t) for t in leaves]

        ya, ga = run(True)
        yb, gb = run(False)
        if tf32:
            # Several tiles (or one tile with d = 64): the head form hands the forward's output to the backward, whose row dots
            # are then rowsum(dO O); the permuted form recomputes them as rowsum(P dP). Equal in exact arithmetic, a TF32
            # product apart on the tensor pipe.
            tol = 2e-5 if (l <= 128 and dh == 32) or dh == 16 else 2e-3
            assert scaled_diff(ya, yb) <= 2e-5
            assert all(scaled_diff(x, y) <= tol for x, y in zip(ga, gb))
        else:
            assert np.array_equal(ya, yb)
            assert all(np.array_equal(x, y) for x, y in zip(ga, gb))
    finally:
        ctx.set_flags(0)


def test_graph_op_family(B):
    """MatMulBatched (broadcast batch axes), Erf, Exp, Sqrt, Pow, Where, Gather and their backward functions on the GPU
    against the PyTorch golden file the CPU oracle is pinned on (fp32 products: the 1e-4 tier, here far inside it)."""
    check_graph_ops(B, 1e-5)


def test_conv1d_on_the_height_one_view(B):
    """Ops.Conv1d (stride, separate left/right padding, dilation, groups, with and without bias): forward, dx, dW and dbias on
    the GPU through the 2-D convolution entry points on a height-1 view, against the PyTorch golden file the CPU oracle is
    pinned on."""
    check_conv1d(B, 1e-5)


def test_loss_family(B):
    """Losses.{CrossEntropy with label smoothing, Mse, L1, BceWithLogits} on the GPU against the PyTorch golden file."""
    check_losses(B, 1e-5)


@pytest.mark.parametrize("n,p,seed,draw", [(1000, 0.3, 42, 0), (1003, 0.5, 7, 3), (1 << 20, 0.1, 2**63 + 5, 2**40), (4, 0.0, 1, 0)])
def test_dropout_mask_bits(ctx, n, p, seed, draw):
    """om_dropout_mask is the reference's counter-based mask bit for bit (Layers.cs:354-366), vector and scalar paths."""
    import ctypes as C
    import om_binding as omb
    from om_binding import f32, i64
    from oracle import tape
    counter = ctx.to_device(np.array([draw], np.int64))
    mask = ctx.empty((n,))
    ctx.call("om_dropout_mask", ctx.handle, C.c_uint64(seed), counter.ptr, f32(p), i64(n), mask.ptr)
    assert np.array_equal(mask.numpy(), tape.dropout_mask(seed, draw, p, n))
    assert counter.numpy()[0] == draw                          # the mask entry point leaves the counter alone
    with pytest.raises(omb.OmError):
        ctx.call("om_dropout_mask", ctx.handle, C.c_uint64(seed), counter.ptr, f32(1.0), i64(n), mask.ptr)


def test_dropout_forward_backward_and_counter(ctx, B):
    """Ops.Dropout: y = x * mask of the counter's call number, the counter advances by one per call in device memory,
    and the backward forms the same mask again (ModuleAndLossTests.cs:62-102 of the reference)."""
    import om_binding as omb
    from oracle import tape
    x_np = np.random.default_rng(3).standard_normal((37, 29)).astype(np.float32)
    w_np = np.random.default_rng(4).standard_normal((37, 29)).astype(np.float32)
    counter = omb.Tensor.from_numpy(np.array([5], np.int64))
    for call in range(3):
        x = B.tensor(x_np, True)
        y = omb.call("dropout", [x, counter], ints=[99], floats=[0.4])
        m = tape.dropout_mask(99, 5 + call, 0.4, x_np.size).reshape(x_np.shape)
        assert np.array_equal(y.numpy(), x_np * m)
        assert int(counter.numpy()[0]) == 6 + call
        B.backward(B.sum(B.mul(y, B.tensor(w_np))))
        assert np.array_equal(B.grad(x), w_np * m)
    with omb.no_grad():
        y = omb.call("dropout", [B.tensor(x_np), counter], ints=[99], floats=[0.4])
    assert np.array_equal(y.numpy(), x_np * tape.dropout_mask(99, 8, 0.4, x_np.size).reshape(x_np.shape))


def test_frozen_encoder_curve(B):
    """The reference's frozen-parameter fixture on the GPU (fp32 products): frozen tensors keep their bits, the others
    follow the recorded curve."""
    check_frozen_encoder(B, 1e-5, 1e-3, 1e-3)


def test_conv1d_reference_grid_and_training(B):
    """The reference's own Conv1d fixtures on the GPU: every grid case (y, dx, dW, dbias) and the 20-step training curve
    (tests/OneModel.Tests/Training/Conv1dTests.cs:76-118, 258-307 of the reference), fp32 products."""
    check_conv1d_reference_grid(B, 1e-5)
    check_conv1d_training(B, 1e-5, 1e-4)


@pytest.mark.parametrize("name,lr,b1,b2,eps", [("sparseadam", 0.05, 0.9, 0.999, 1e-3), ("sparseadam2", 0.02, 0.8, 0.95, 1e-8), ("sgd", 0.5, 0, 0, 0)])
def test_row_sparse_optimizers_against_the_reference_fixture(ctx, B, name, lr, b1, b2, eps):
    """om_rows_touched + om_optim_sparse_adam_step / om_optim_sparse_sgd_step on the embedding table, the dense optimizers on
    the head: losses and final parameters of testdata/training/sparse within the reference's 1e-6
    (SparseAndFrozenTests.cs:255-420); untouched rows keep their parameters and moments bit for bit."""
    import ctypes as C
    import om_binding as omb
    from om_binding import f32, i32, i64
    from oracle import oracle as K
    fx = load_fixture("training", "sparse")
    ids_all, y_all = fx["in.ids"].astype(np.int64), fx["in.y"].astype(np.int64)
    emb, hw, hb = B.tensor(fx["in.emb"], True), B.tensor(fx["in.hw"], True), B.tensor(fx["in.hb"], True)
    if name == "sgd":
        head = omb.Optimizer.sgd([hw, hb], 0.5)
    elif name == "sparseadam":
        head = omb.Optimizer.adamw([hw, hb], 0.01, weight_decay=0.01)
    else:
        head = omb.Optimizer.adam([hw, hb], 0.01)
    m, v, touched = ctx.zeros((40, 8)), ctx.zeros((40, 8)), ctx.empty((40,), np.int32)
    losses, ever = [], np.zeros(40, bool)
    for s in range(ids_all.shape[0]):
        ids = B.ids(ids_all[s])
        pooled = B.mean(omb.call("embedding", [emb, ids], ints=[0]), 1)
        loss = B.cross_entropy(B.linear(pooled, hw, hb), B.ids(y_all[s]))
        emb.zero_grad()
        head.zero_grad()
        B.backward(loss)
        losses.append(float(B.numpy(loss).reshape(-1)[0]))
        before = emb.numpy()
        flat = omb.Tensor.from_numpy(ids_all[s].reshape(-1))
        ctx.call("om_rows_touched", ctx.handle, C.c_void_p(flat.data_ptr), i32(omb.OM_I64), i64(30), i32(40), i64(0), touched.ptr)
        g = emb.grad
        if name == "sgd":
            ctx.call("om_optim_sparse_sgd_step", ctx.handle, C.c_void_p(emb.data_ptr), C.c_void_p(g.data_ptr), touched.ptr, i32(40), i32(8), f32(lr))
        else:
            t = s + 1
            step = np.float32(float(np.float32(lr)) * np.sqrt(1.0 - K.int_pow(np.float32(b2), t)) / (1.0 - K.int_pow(np.float32(b1), t)))
            ctx.call("om_optim_sparse_adam_step", ctx.handle, C.c_void_p(emb.data_ptr), C.c_void_p(g.data_ptr), m.ptr, v.ptr, touched.ptr,
                     i32(40), i32(8), f32(b1), f32(b2), f32(eps), f32(step))
        head.step()
        ctx.sync()
        tc = touched.numpy()
        assert np.array_equal(tc, K.rows_touched(ids_all[s], 40, 0))
        after = emb.numpy()
        assert np.array_equal(after[tc == 0], before[tc == 0])
        if name != "sgd":
            ever |= tc > 0
            assert not np.any(m.numpy()[~ever])                  # rows never touched so far have no moment
    want = fx[f"out.{name}.loss"]
    assert np.max(np.abs(np.array(losses) - want) / np.abs(want)) <= 1e-6
    for t, key in ((emb, "emb"), (hw, "hw"), (hb, "hb")):
        assert scaled_diff(t.numpy(), fx[f"out.{name}.{key}"]) <= 1e-6, key
