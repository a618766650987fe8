"""The module layer of the host mirror (NnModule, Layers, Sequential, Freeze / Unfreeze, StateDict / LoadStateDict, Dropout)
through the C boundary, after the reference's own tests: tests/OneModel.Tests/Training/Conv1dTests.cs:258-307 (a Conv1d
net built from modules trains like PyTorch), SparseAndFrozenTests.cs:120-140 (freezing by name, prefix and all),
ModuleAndLossTests.cs:12-126 (state order, train / eval, dropout stream, seeded bounded initialisation)."""
import numpy as np
import pytest

from backends import GpuBackend, load_fixture, scaled_diff

pytestmark = pytest.mark.gpu


@pytest.fixture()
def omb(ctx):
    import om_binding
    ctx.set_flags(0)
    ctx.make_current()
    return om_binding


def test_conv1d_net_of_modules_trains_like_the_recorded_curve(ctx, omb):
    fx = load_fixture("conv1d", "train")
    M, g = omb.Module, omb.Generator(1)
    model = M.sequential(M("conv1d_same", g, [4, 6, 3, 2, 1, 1]), M("relu"), M("conv1d", g, [6, 6, 3, 2, 1, 1, 2, 1]), M("relu"),
                         M("mean", ints=[2]), M("linear", g, [6, 3, 1]))
    names = [n for n, _ in model.state_dict()]
    assert names == ["0.weight", "0.bias", "2.weight", "2.bias", "5.weight", "5.bias"]
    keys = dict(zip(names, ("c1w", "c1b", "c2w", "c2b", "fcw", "fcb")))
    model.load_state_dict([(n, omb.Tensor.from_numpy(fx["in." + keys[n]])) for n in names])
    opt = omb.Optimizer.sgd(model.parameters(), 0.05, momentum=0.9)
    order = fx["in.order"].astype(np.int64)
    losses = []
    for s in range(order.shape[0]):
        x = omb.Tensor.from_numpy(fx["in.x"][order[s]])
        y = omb.Tensor.from_numpy(fx["in.y"][order[s]].astype(np.int64))
        loss = omb.call("cross_entropy", [model(x), y], ints=[1, -100])
        opt.zero_grad()
        loss.backward()
        losses.append(float(loss.numpy().reshape(-1)[0]))
        opt.step()
    want = fx["out.loss"]
    assert np.max(np.abs(np.array(losses) - want) / np.abs(want)) <= 1e-5
    for n, t in model.state_dict():
        assert scaled_diff(t.numpy(), fx["out." + keys[n]]) <= 1e-4, n


def test_freeze_by_name_prefix_and_all(ctx, omb):
    M, g = omb.Module, omb.Generator(1)
    model = M.sequential(M("linear", g, [4, 3, 1]), M("relu"), M("linear", g, [3, 2, 1]))
    assert len(model.trainable_parameters()) == 4
    assert model.freeze("0.weight") == 1 and model.is_frozen("0.weight")
    assert len(model.trainable_parameters()) == 3
    assert model.freeze("0") == 1                      # the bias; the weight is frozen already
    assert model.freeze("2") == 2                      # a module path covers its parameters
    assert model.named_trainable_parameters() == []
    assert model.unfreeze("2.bias") == 1
    assert [n for n, _ in model.named_trainable_parameters()] == ["2.bias"]
    for bad in ("nope", "2.bi"):                       # a prefix must end at a dot
        with pytest.raises(omb.OmError):
            model.freeze(bad)
    with pytest.raises(omb.OmError):
        model.is_frozen("nope")
    assert model.unfreeze() == 3 and model.freeze() == 4 and model.unfreeze() == 4

    # A frozen parameter receives no gradient and does not move; the others train.
    model.freeze("0")
    before = {n: t.numpy() for n, t in model.state_dict()}
    opt = omb.Optimizer.adam(model.trainable_parameters(), 0.1)
    x = omb.Tensor.from_numpy(np.random.default_rng(0).standard_normal((5, 4)).astype(np.float32))
    loss = omb.call("sum", [omb.call("mul", [model(x), model(x)])])
    loss.backward()
    opt.step()
    for n, t in model.state_dict():
        if n.startswith("0."):
            assert t.grad is None and np.array_equal(t.numpy(), before[n]), n
        else:
            assert t.grad is not None and not np.array_equal(t.numpy(), before[n]), n


def test_state_order_train_eval_and_load_checks(ctx, omb):
    M, g = omb.Module, omb.Generator(3)
    model = M.sequential(M("conv2d", g, [2, 4, 3, 1, 1, 1]), M("batch_norm2d", ints=[4]), M("relu"), M("dropout", ints=[11], floats=[0.5]),
                         M("global_avg_pool2d"), M("flatten"), M("linear", g, [4, 3, 1]))
    names = [n for n, _ in model.state_dict()]
    assert names == ["0.weight", "0.bias", "1.weight", "1.bias", "1.running_mean", "1.running_var", "3.draws", "6.weight", "6.bias"]
    assert [n for n, _ in model.entries(M.BUFFERS)] == ["1.running_mean", "1.running_var", "3.draws"]
    x = omb.Tensor.from_numpy(np.random.default_rng(1).standard_normal((6, 2, 5, 5)).astype(np.float32))
    a, b = model(x).numpy(), model(x).numpy()
    assert not np.array_equal(a, b)                    # training: a new dropout mask and moving batch statistics
    state = dict(model.state_dict())
    assert int(state["3.draws"].numpy()[0]) == 2 and np.any(state["1.running_mean"].numpy() != 0)
    model.eval()
    c, d = model(x).numpy(), model(x).numpy()
    assert np.array_equal(c, d) and int(state["3.draws"].numpy()[0]) == 2     # eval: running statistics, no mask
    # LoadStateDict copies in place and rejects a mismatch (names, count, shape).
    clone = M.sequential(M("conv2d", g, [2, 4, 3, 1, 1, 1]), M("batch_norm2d", ints=[4]), M("relu"), M("dropout", ints=[11], floats=[0.5]),
                         M("global_avg_pool2d"), M("flatten"), M("linear", g, [4, 3, 1])).eval()
    assert not np.array_equal(clone(x).numpy(), c)
    clone.load_state_dict(model.state_dict())
    assert np.array_equal(clone(x).numpy(), c)
    entries = model.state_dict()
    with pytest.raises(omb.OmError):
        clone.load_state_dict(entries[:-1])
    with pytest.raises(omb.OmError):
        clone.load_state_dict(entries[:-1] + [("6.bias", omb.Tensor.from_numpy(np.zeros(4, np.float32)))])
    with pytest.raises(omb.OmError):
        clone.load_state_dict(entries[:-1] + [("other", entries[-1][1])])


def test_dropout_module_stream_follows_its_counter(ctx, omb):
    from oracle import tape
    M = omb.Module
    a, b = M("dropout", ints=[42], floats=[0.3]), M("dropout", ints=[42], floats=[0.3])
    ones = omb.Tensor.from_numpy(np.ones(1000, np.float32))
    a1, b1, a2 = a(ones).numpy(), b(ones).numpy(), a(ones).numpy()
    assert np.array_equal(a1, b1) and not np.array_equal(a1, a2)
    assert np.array_equal(a1, tape.dropout_mask(42, 0, 0.3, 1000)) and np.array_equal(a2, tape.dropout_mask(42, 1, 0.3, 1000))
    assert 240 <= int((a1 == 0).sum()) <= 360 and np.all(a1[a1 != 0] == np.float32(1.0) / np.float32(0.7))
    assert int(a.state_dict()[0][1].numpy()[0]) == 2
    b.load_state_dict([("draws", omb.Tensor.from_numpy(np.array([1], np.int64)))])      # restoring the counter restores the stream
    assert np.array_equal(b(ones).numpy(), a2)
    assert np.array_equal(a.eval()(ones).numpy(), np.ones(1000, np.float32))
    with pytest.raises(omb.OmError):
        M("dropout", ints=[1], floats=[1.0])


def test_initialisation_is_seeded_and_bounded(ctx, omb):
    """Linear draws weight then bias, row-major, uniform in [-1/sqrt(in), 1/sqrt(in)) from the SplitMix64 stream
    (Layers.cs:11-21, 41-65): checked value by value against the generator written out on Python integers."""
    from oracle import tape
    M = omb.Module
    g = omb.Generator(5)
    lin = M("linear", g, [7, 3, 1])
    w, b = (t.numpy() for _, t in lin.state_dict())
    bound = np.float32(1.0) / np.sqrt(np.float32(7.0))
    state, want = 5, []
    for _ in range(7 * 3 + 3):
        state = (state + 0x9E3779B97F4A7C15) & ((1 << 64) - 1)
        u = np.float32(tape.splitmix_finish(state) >> 40) * np.float32(1.0 / 16777216.0)
        want.append(-bound + (bound - (-bound)) * u)
    assert np.array_equal(np.concatenate([w.reshape(-1), b]), np.array(want, np.float32))
    assert g.state.value == state                                 # the stream continues for the next module
    assert np.all(np.abs(w) <= bound)
    again = M("linear", omb.Generator(5), [7, 3, 1])
    assert np.array_equal(again.state_dict()[0][1].numpy(), w)


@pytest.mark.parametrize("bidirectional,gru,batch_first", [(False, False, False), (True, False, False), (True, True, False), (True, False, True)])
def test_padded_rows_equal_rows_run_alone(ctx, omb, bidirectional, gru, batch_first):
    """A padded batch with lengths gives, for every row, what that row gives alone at its own length, zeros after it, zero
    input gradient at the padded steps, and weight gradients equal to the sum over the rows run alone
    (tests/OneModel.Tests/Tensors/PackedRecurrentTests.cs:34-66 of the reference)."""
    steps, batch, in_size, h, dirs = 6, 4, 3, 5, 2 if bidirectional else 1
    lengths = [6, 3, 1, 4]
    r = np.random.default_rng(7)
    model = omb.Module("recurrent", omb.Generator(9), [int(gru), in_size, h, 2, int(bidirectional), int(batch_first)])
    x_np = r.uniform(-0.6, 0.6, (steps, batch, in_size)).astype(np.float32)
    w_np = r.uniform(-1, 1, (steps, batch, h * dirs)).astype(np.float32)
    lay = (lambda a: np.ascontiguousarray(a.transpose(1, 0, 2))) if batch_first else (lambda a: a)

    x = omb.Tensor.from_numpy(lay(x_np), True)
    out = model.forward_lengths(x, lengths)
    model.zero_grad()
    omb.call("sum", [omb.call("mul", [out, omb.Tensor.from_numpy(lay(w_np))])]).backward()
    got = lay(out.numpy()) if batch_first else out.numpy()
    gx = lay(x.grad.numpy()) if batch_first else x.grad.numpy()
    gw = {n: t.grad.numpy().copy() for n, t in model.named_parameters()}

    want_gw = {n: np.zeros_like(v, dtype=np.float64) for n, v in gw.items()}
    for b, n in enumerate(lengths):
        xr = omb.Tensor.from_numpy(lay(x_np[:n, b:b + 1]), True)
        alone = model(xr)
        model.zero_grad()
        omb.call("sum", [omb.call("mul", [alone, omb.Tensor.from_numpy(lay(w_np[:n, b:b + 1]))])]).backward()
        alone_np = lay(alone.numpy()) if batch_first else alone.numpy()
        assert np.max(np.abs(got[:n, b] - alone_np[:, 0])) < 1e-5, b
        assert not got[n:, b].any(), b                                 # exactly zero after the row's length
        gxr = lay(xr.grad.numpy()) if batch_first else xr.grad.numpy()
        assert np.max(np.abs(gx[:n, b] - gxr[:, 0])) < 1e-5 and not gx[n:, b].any(), b
        for name, t in model.named_parameters():
            want_gw[name] += t.grad.numpy()
    for name in gw:
        assert scaled_diff(gw[name], want_gw[name]) <= 1e-5, name

    for bad in ([6, 3, 1], [6, 3, 1, 7], [6, 0, 1, 4]):
        with pytest.raises(omb.OmError):
            model.forward_lengths(x, bad)
    with pytest.raises(omb.OmError):
        omb.Module("linear", omb.Generator(1), [3, 2, 1]).forward_lengths(x, lengths)


@pytest.mark.parametrize("flags", [0, 3])       # 3: OM_TF32 | OM_BF16_OPERANDS
@pytest.mark.parametrize("shape", [(3, 7, 768), (64, 40), (2, 5, 1000), (9, 30)])
def test_add_layer_norm_equals_add_then_layer_norm(ctx, omb, flags, shape):
    """Ops.AddLayerNorm (the residual sum formed inside the layer norm's kernel) against Add followed by LayerNorm: the result
    and the four gradients bit for bit, for widths with and without 16-byte rows."""
    ctx.set_flags(flags)
    ctx.make_current()
    try:
        r = np.random.default_rng(shape[-1])
        av, bv = r.standard_normal(shape).astype(np.float32), r.standard_normal(shape).astype(np.float32)
        gv, ev = (1 + 0.1 * r.standard_normal(shape[-1])).astype(np.float32), (0.1 * r.standard_normal(shape[-1])).astype(np.float32)
        up = r.standard_normal(shape).astype(np.float32)
        results = []
        for fused in (True, False):
            a, b, g, e = (omb.Tensor.from_numpy(v, True) for v in (av, bv, gv, ev))
            if fused:
                y = omb.call("add_layer_norm", [a, b, g, e], floats=[1e-5])
            else:
                y = omb.call("layer_norm", [omb.call("add", [a, b]), g, e], floats=[1e-5])
            y.backward(omb.Tensor.from_numpy(up))
            results.append([y.numpy()] + [t.grad.numpy() for t in (a, b, g, e)])
        for x, z in zip(*results):
            assert np.all(np.isfinite(x)) and np.array_equal(x, z)
    finally:
        ctx.set_flags(0)
