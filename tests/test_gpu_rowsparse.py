"""The row-sparse table gradient on the device: om_embedding_bwd_sparse, om_rowsparse_add_to, om_rowsparse_merge and the
row-list optimizer steps through the C ABI against the oracle's restatement of EmbeddingSparseBackward / RowSparseGradient
(BackwardNn.cs:548-600, RowSparseGradient.cs:14-120 of the reference), and the host mirror's Embedding(sparse) -> SparseGrad
-> Sgd / SparseAdam flow after the reference's own tests (tests/OneModel.Tests/Training/SparseAndFrozenTests.cs:191-420) on
its fixture testdata/training/sparse."""
import ctypes as C

import numpy as np
import pytest

from backends import load_fixture, scaled_diff

pytestmark = pytest.mark.gpu


@pytest.fixture()
def omb(ctx):
    import om_binding
    ctx.set_flags(0)
    ctx.make_current()
    return om_binding


def sparse_bwd(ctx, omb, g, ids, v, pad, capacity=None):
    from om_binding import i32, i64
    n, dim = ids.size, g.shape[-1]
    cap = min(n, v) if capacity is None else capacity
    G, I = ctx.to_device(np.ascontiguousarray(g, np.float32)), ctx.to_device(np.ascontiguousarray(ids))
    rows, values, count = ctx.empty((cap,), np.int32), ctx.empty((cap, dim)), ctx.empty((1,), np.int32)
    ctx.call("om_embedding_bwd_sparse", ctx.handle, G.ptr, I.ptr, i32(omb.OM_I64 if ids.dtype == np.int64 else omb.OM_I32), i64(n), i32(v), i32(dim),
             i64(pad), rows.ptr, values.ptr, i32(cap), count.ptr)
    ctx.sync()
    return rows, values, count


@pytest.mark.parametrize("n,v,dim,pad,dtype", [(30, 40, 8, 0, np.int64), (1000, 64, 20, -1, np.int32), (16384, 30522, 768, 0, np.int32),
                                              (5000, 300, 33, 7, np.int64), (6, 1000, 4, -1, np.int32)])
def test_sparse_table_gradient_against_the_oracle(ctx, omb, oracle_built, n, v, dim, pad, dtype):
    """Rows strictly ascending, each once, the padding row absent; values equal the oracle's sums in increasing position order
    bit for bit; scattered into zeros they are om_embedding_bwd's dense gradient bit for bit; the entries behind the row count
    are row -1 with zero values; the same bits from run to run."""
    from om_binding import i32, i64
    K = oracle_built
    r = np.random.default_rng(n + v)
    ids = r.integers(0, v, n).astype(dtype)
    ids[r.random(n) < 0.3] = ids[0]                     # one id looked up many times
    if pad >= 0:
        ids[r.random(n) < 0.1] = pad
    g = r.standard_normal((n, dim)).astype(np.float32)
    want_rows, want_values = K.embedding_bwd_sparse(g, ids, pad)
    rows, values, count = sparse_bwd(ctx, omb, g, ids, v, pad)
    u = int(count.numpy()[0])
    assert u == len(want_rows) and u >= 1
    assert np.array_equal(rows.numpy()[:u], want_rows) and np.all(np.diff(rows.numpy()[:u]) > 0) and pad not in rows.numpy()[:u]
    assert np.array_equal(values.numpy()[:u], want_values)
    assert np.all(rows.numpy()[u:] == -1) and not np.any(values.numpy()[u:])
    # ToDense / AddTo against the dense backward
    G, I = ctx.to_device(g), ctx.to_device(ids)
    dense, scattered = ctx.empty((v, dim)), ctx.zeros((v, dim))
    ctx.call("om_embedding_bwd", ctx.handle, G.ptr, I.ptr, i32(omb.OM_I64 if dtype == np.int64 else omb.OM_I32), i64(n), i32(v), i32(dim), i64(pad),
             dense.ptr, i32(0))
    ctx.call("om_rowsparse_add_to", ctx.handle, rows.ptr, values.ptr, count.ptr, i32(rows.shape[0]), i32(dim), scattered.ptr, i32(v))
    ctx.sync()
    assert np.array_equal(scattered.numpy(), dense.numpy())
    assert np.array_equal(dense.numpy(), K.embedding_bwd(g, ids, v, dim, pad))
    ctx.call("om_rowsparse_add_to", ctx.handle, rows.ptr, values.ptr, count.ptr, i32(rows.shape[0]), i32(dim), scattered.ptr, i32(v))
    ctx.sync()
    assert np.array_equal(scattered.numpy(), dense.numpy() + dense.numpy())
    rows2, values2, count2 = sparse_bwd(ctx, omb, g, ids, v, pad)
    assert np.array_equal(rows2.numpy(), rows.numpy()) and np.array_equal(values2.numpy(), values.numpy()) and count2.numpy()[0] == u


def test_sparse_table_gradient_of_padding_only_and_argument_errors(ctx, omb):
    from om_binding import i32, i64
    ids = np.zeros(12, np.int64)
    rows, values, count = sparse_bwd(ctx, omb, np.ones((12, 8), np.float32), ids, 40, 0)
    assert count.numpy()[0] == 0 and np.all(rows.numpy() == -1) and not np.any(values.numpy())
    G, I = ctx.to_device(np.ones((12, 8), np.float32)), ctx.to_device(ids)
    small = ctx.empty((4,), np.int32)
    with pytest.raises(omb.OmError) as e:                       # capacity below min(n, v)
        ctx.call("om_embedding_bwd_sparse", ctx.handle, G.ptr, I.ptr, i32(omb.OM_I64), i64(12), i32(40), i32(8), i64(0), small.ptr, values.ptr, i32(4), count.ptr)
    assert "capacity" in str(e.value)
    bad = ctx.to_device(np.array([1, 2, 99, 3], np.int64))      # an id outside the table: reported, not read
    ctx.call("om_embedding_bwd_sparse", ctx.handle, G.ptr, bad.ptr, i32(omb.OM_I64), i64(4), i32(40), i32(8), i64(0), rows.ptr, values.ptr, i32(12), count.ptr)
    with pytest.raises(omb.IndexOutOfRange):
        ctx.sync()
    ctx.sync()                                                  # the context stays usable


@pytest.mark.parametrize("v,dim,na,nb", [(40, 8, 30, 30), (5000, 96, 3000, 500), (30522, 768, 4000, 4000)])
def test_merge_of_two_sparse_gradients_against_the_oracle(ctx, omb, oracle_built, v, dim, na, nb):
    """om_rowsparse_merge: the union of the rows in ascending order; a row in both holds a's values plus b's, a row in one that
    one's (RowSparseGradient.Merge, :66-116), bit for bit against the oracle; merging with a gradient without rows returns
    the other."""
    from om_binding import i32
    K = oracle_built
    r = np.random.default_rng(v + na)
    ga, gb = r.standard_normal((na, dim)).astype(np.float32), r.standard_normal((nb, dim)).astype(np.float32)
    ia, ib = r.integers(0, v, na).astype(np.int64), r.integers(0, max(2, v // 2), nb).astype(np.int64)
    ra, va, ca = sparse_bwd(ctx, omb, ga, ia, v, -1)
    rb, vb, cb = sparse_bwd(ctx, omb, gb, ib, v, -1)
    cap = min(ra.shape[0] + rb.shape[0], v)
    ro, vo, co = ctx.empty((cap,), np.int32), ctx.empty((cap, dim)), ctx.empty((1,), np.int32)
    ctx.call("om_rowsparse_merge", ctx.handle, ra.ptr, va.ptr, ca.ptr, i32(ra.shape[0]), rb.ptr, vb.ptr, cb.ptr, i32(rb.shape[0]), i32(v), i32(dim),
             ro.ptr, vo.ptr, i32(cap), co.ptr)
    ctx.sync()
    wr, wv = K.rowsparse_merge(*K.embedding_bwd_sparse(ga, ia), *K.embedding_bwd_sparse(gb, ib))
    u = int(co.numpy()[0])
    assert u == len(wr) and np.array_equal(ro.numpy()[:u], wr) and np.array_equal(vo.numpy()[:u], wv)
    assert np.all(ro.numpy()[u:] == -1) and not np.any(vo.numpy()[u:])
    with pytest.raises(omb.OmError):
        ctx.call("om_rowsparse_merge", ctx.handle, ra.ptr, va.ptr, ca.ptr, i32(ra.shape[0]), rb.ptr, vb.ptr, cb.ptr, i32(rb.shape[0]), i32(v), i32(dim),
                 ro.ptr, vo.ptr, i32(cap - 1), co.ptr)
    # b without rows
    re, ve, ce = sparse_bwd(ctx, omb, np.ones((4, dim), np.float32), np.full(4, 3, np.int64), v, 3)
    ctx.call("om_rowsparse_merge", ctx.handle, ra.ptr, va.ptr, ca.ptr, i32(ra.shape[0]), re.ptr, ve.ptr, ce.ptr, i32(re.shape[0]), i32(v), i32(dim),
             ro.ptr, vo.ptr, i32(cap), co.ptr)
    ctx.sync()
    ua = int(ca.numpy()[0])
    assert co.numpy()[0] == ua and np.array_equal(ro.numpy()[:ua], ra.numpy()[:ua]) and np.array_equal(vo.numpy()[:ua], va.numpy()[:ua])


def test_row_list_optimizer_steps_equal_the_dense_format_ones(ctx, omb):
    """om_optim_sparse_adam_step_rows / om_optim_sparse_sgd_step_rows leave the table, m and v with the bits of
    om_optim_sparse_adam_step / om_optim_sparse_sgd_step fed the dense-format gradient and the touched counts."""
    from om_binding import f32, i32, i64
    r = np.random.default_rng(5)
    v, dim, n = 3000, 72, 2000
    ids = r.integers(0, v, n).astype(np.int32)
    g = r.standard_normal((n, dim)).astype(np.float32)
    table = r.standard_normal((v, dim)).astype(np.float32)
    rows, values, count = sparse_bwd(ctx, omb, g, ids, v, -1)
    G, I = ctx.to_device(g), ctx.to_device(ids)
    dense, touched = ctx.empty((v, dim)), ctx.zeros((v,), np.int32)
    ctx.call("om_embedding_bwd", ctx.handle, G.ptr, I.ptr, i32(omb.OM_I32), i64(n), i32(v), i32(dim), i64(-1), dense.ptr, i32(0))
    ctx.call("om_rows_touched", ctx.handle, I.ptr, i32(omb.OM_I32), i64(n), i32(v), i64(-1), touched.ptr)
    pa, pb = ctx.to_device(table), ctx.to_device(table)
    ma, va, mb, vb = (ctx.to_device(np.abs(r.standard_normal((v, dim))).astype(np.float32) * 0.1) for _ in range(4))
    mb, vb = ctx.to_device(ma.numpy()), ctx.to_device(va.numpy())
    for _ in range(2):
        ctx.call("om_optim_sparse_adam_step", ctx.handle, pa.ptr, dense.ptr, ma.ptr, va.ptr, touched.ptr, i32(v), i32(dim), f32(0.9), f32(0.999), f32(1e-8), f32(0.01))
        ctx.call("om_optim_sparse_adam_step_rows", ctx.handle, pb.ptr, rows.ptr, values.ptr, count.ptr, i32(rows.shape[0]), mb.ptr, vb.ptr, i32(v), i32(dim),
                 f32(0.9), f32(0.999), f32(1e-8), f32(0.01))
    ctx.sync()
    for a, b in ((pa, pb), (ma, mb), (va, vb)):
        assert np.array_equal(a.numpy(), b.numpy())
    assert np.any(pa.numpy() != table)
    ctx.call("om_optim_sparse_sgd_step", ctx.handle, pa.ptr, dense.ptr, touched.ptr, i32(v), i32(dim), f32(0.5))
    ctx.call("om_optim_sparse_sgd_step_rows", ctx.handle, pb.ptr, rows.ptr, values.ptr, count.ptr, i32(rows.shape[0]), i32(v), i32(dim), f32(0.5))
    ctx.sync()
    assert np.array_equal(pa.numpy(), pb.numpy())


# ---- the host mirror, after SparseAndFrozenTests.cs ------------------------------------------------------------------------

class EmbeddingClassifier:
    """A classifier on an embedding: mean of the looked-up vectors, then a linear head (SparseAndFrozenTests.cs:8-21)."""

    def __init__(self, omb, fx, sparse):
        self.omb, self.sparse = omb, sparse
        T = omb.Tensor.from_numpy
        self.emb, self.hw, self.hb = T(fx["in.emb"], True), T(fx["in.hw"], True), T(fx["in.hb"], True)

    def loss(self, ids, y):
        omb = self.omb
        looked = omb.call("embedding", [self.emb, omb.Tensor.from_numpy(ids)], ints=[0, 1 if self.sparse else 0])
        logits = omb.call("linear", [omb.call("mean", [looked], ints=[1, 0]), self.hw, self.hb])
        return omb.call("cross_entropy", [logits, omb.Tensor.from_numpy(y)], ints=[1, -100])


def run_step(model, fx, step, opts):
    ids, y = fx["in.ids"].astype(np.int32)[step], fx["in.y"].astype(np.int64)[step]
    loss = model.loss(ids, y)
    value = loss.item()
    for o in opts:
        o.zero_grad()
    loss.backward()
    for o in opts:
        o.step()
    return value


def test_sparse_gradient_is_the_dense_gradients_touched_rows(ctx, omb):
    """SparseGradientIsTheDenseGradientsTouchedRowsAndMatchesTorch (SparseAndFrozenTests.cs:251-283)."""
    fx = load_fixture("training", "sparse")
    sparse_model, dense_model = EmbeddingClassifier(omb, fx, True), EmbeddingClassifier(omb, fx, False)
    for m in (sparse_model, dense_model):
        m.loss(fx["in.ids"].astype(np.int32)[0], fx["in.y"].astype(np.int64)[0]).backward()
    sg = sparse_model.emb.sparse_grad
    assert sg is not None and sparse_model.emb.grad is None
    assert 3 < sg.row_count < 40
    rows = sg.rows.numpy()
    assert rows.shape == (sg.row_count,) and np.all(np.diff(rows) > 0) and 0 not in rows
    assert sg.values.shape == (sg.row_count, 8) and sg.byte_count == sg.row_count * 36
    dense = sg.to_dense().numpy()
    assert np.array_equal(dense, dense_model.emb.grad.numpy())          # bit for bit
    assert scaled_diff(dense, fx["out.sgd.grad0"]) <= 1e-6
    target = omb.Tensor.from_numpy(np.ones((40, 8), np.float32))
    sg.add_to(target)
    assert np.array_equal(target.numpy(), np.ones((40, 8), np.float32) + dense)
    assert dense_model.emb.sparse_grad is None
    # zero is the absence of rows: ZeroGrad frees the sparse gradient
    sparse_model.emb.zero_grad()
    assert sparse_model.emb.sparse_grad is None


def test_sparse_sgd_is_bit_equal_to_dense_sgd(ctx, omb):
    """SparseSgdIsBitEqualToDenseSgdAndMatchesTorch (SparseAndFrozenTests.cs:285-318)."""
    fx = load_fixture("training", "sparse")
    sparse_model, dense_model = EmbeddingClassifier(omb, fx, True), EmbeddingClassifier(omb, fx, False)
    s1, s2 = omb.Optimizer.sgd([sparse_model.emb], 0.5), omb.Optimizer.sgd([sparse_model.hw, sparse_model.hb], 0.5)
    d = omb.Optimizer.sgd([dense_model.emb, dense_model.hw, dense_model.hb], 0.5)
    losses = []
    for s in range(fx["in.ids"].shape[0]):
        a, b = run_step(sparse_model, fx, s, [s1, s2]), run_step(dense_model, fx, s, [d])
        assert np.float32(a).tobytes() == np.float32(b).tobytes()
        losses.append(a)
    assert np.array_equal(sparse_model.emb.numpy(), dense_model.emb.numpy())
    assert np.array_equal(sparse_model.hw.numpy(), dense_model.hw.numpy())
    want = fx["out.sgd.loss"]
    assert np.max(np.abs(np.array(losses) - want) / np.abs(want)) <= 1e-6
    assert scaled_diff(sparse_model.emb.numpy(), fx["out.sgd.emb"]) <= 1e-6


def test_sparse_sgd_step_alone_within_1e_7(ctx, omb):
    """SparseSgdStepAloneMatchesTorchWithin1e7 (SparseAndFrozenTests.cs:320-351): the recorded gradient fed through lookups of
    distinct ids, one step, the table against the recorded one."""
    fx = load_fixture("training", "sparse")
    grad = fx["out.sgd.grad0"]
    rows = np.array([r for r in range(40) if np.any(grad[r] != 0)], np.int32)
    table = omb.Tensor.from_numpy(fx["in.emb"], True)
    out = omb.call("embedding", [table, omb.Tensor.from_numpy(rows)], ints=[0, 1])
    out.backward(omb.Tensor.from_numpy(grad[rows]))
    assert table.sparse_grad.row_count == len(rows)
    omb.Optimizer.sgd([table], 0.5).step()
    assert scaled_diff(table.numpy(), fx["out.sgd.emb1"]) <= 1e-7


def test_sparse_sgd_rejects_momentum_and_decay_and_adam_rejects_sparse(ctx, omb):
    """SparseSgdRejectsMomentumAndDecay (SparseAndFrozenTests.cs:353-365); SparseAdam rejects a dense gradient and tables that
    are not rank 2 (Optimizers.cs:652-693)."""
    fx = load_fixture("training", "sparse")
    m = EmbeddingClassifier(omb, fx, True)
    with pytest.raises(omb.NotSupported):
        run_step(m, fx, 0, [omb.Optimizer.sgd([m.emb], 0.1, momentum=0.9)])
    with pytest.raises(omb.NotSupported):
        run_step(m, fx, 0, [omb.Optimizer.sgd([m.emb], 0.1, weight_decay=0.01)])
    with pytest.raises(omb.InvalidOperation):
        run_step(m, fx, 0, [omb.Optimizer.adam([m.emb])])
    dense = EmbeddingClassifier(omb, fx, False)
    with pytest.raises(omb.InvalidOperation):
        run_step(dense, fx, 0, [omb.Optimizer.sparse_adam([dense.emb])])
    with pytest.raises(omb.OmError):
        omb.Optimizer.sparse_adam([dense.hb])
    with pytest.raises(omb.IndexOutOfRange):
        omb.Optimizer.sparse_adam([dense.emb], beta1=1.0)
    with pytest.raises(omb.IndexOutOfRange):
        omb.Optimizer.sparse_adam([dense.emb], eps=0.0)


@pytest.mark.parametrize("name,table_args,head", [("sparseadam", dict(lr=0.05, eps=1e-3), ("adamw", dict(lr=0.01, weight_decay=0.01))),
                                                  ("sparseadam2", dict(lr=0.02, beta1=0.8, beta2=0.95), ("adam", dict(lr=0.01)))])
def test_sparse_adam_against_the_reference_fixture(ctx, omb, name, table_args, head):
    """SparseAdamMatchesTorchWithRepeatedAndPaddingIdsAndMixedOptimizers (SparseAndFrozenTests.cs:367-396): losses and final
    parameters within 1e-6."""
    fx = load_fixture("training", "sparse")
    m = EmbeddingClassifier(omb, fx, True)
    sa = omb.Optimizer.sparse_adam([m.emb], **table_args)
    hd = getattr(omb.Optimizer, head[0])([m.hw, m.hb], **head[1])
    losses = [run_step(m, fx, s, [sa, hd]) for s in range(fx["in.ids"].shape[0])]
    want = fx[f"out.{name}.loss"]
    assert np.max(np.abs(np.array(losses) - want) / np.abs(want)) <= 1e-6
    for t, key in ((m.emb, "emb"), (m.hw, "hw"), (m.hb, "hb")):
        assert scaled_diff(t.numpy(), fx[f"out.{name}.{key}"]) <= 1e-6, key


def test_sparse_adam_leaves_untouched_rows_alone_and_clipping_counts_each_row_once(ctx, omb):
    """SparseAdamLeavesUntouchedRowsAndTheirMomentsAlone (SparseAndFrozenTests.cs:398-420), and gradient clipping on the values
    of a sparse gradient (Schedules.cs:33): the norm is the dense gradient's norm."""
    fx = load_fixture("training", "sparse")
    m = EmbeddingClassifier(omb, fx, True)
    before = m.emb.numpy()
    loss = m.loss(fx["in.ids"].astype(np.int32)[0], fx["in.y"].astype(np.int64)[0])
    loss.backward()
    sg = m.emb.sparse_grad
    touched = set(sg.rows.numpy().tolist())
    dense = sg.to_dense().numpy()
    norm = omb.clip_norm([m.emb], 1e-3)
    assert abs(norm - np.sqrt(np.sum(dense.astype(np.float64) ** 2))) <= 1e-6 * norm and norm > 1e-3
    clipped = m.emb.sparse_grad.to_dense().numpy()
    assert abs(np.sqrt(np.sum(clipped.astype(np.float64) ** 2)) - 1e-3) <= 1e-8
    omb.Optimizer.sparse_adam([m.emb], 0.05).step()
    after = m.emb.numpy()
    for r in range(40):
        assert (r in touched) == (not np.array_equal(after[r], before[r]))


def test_two_sparse_lookups_of_one_table_merge_and_a_dense_use_goes_dense(ctx, omb, oracle_built):
    """Engine.EmitSparse / AccumulateLeaf (Engine.cs:252-311): two sparse lookups of one leaf table in a pass merge into one
    sparse gradient (the union of the rows); a table that is also used densely ends with a dense gradient holding both; a
    computed (non-leaf) table receives the dense form."""
    K = oracle_built
    r = np.random.default_rng(9)
    tv = r.standard_normal((50, 16)).astype(np.float32)
    ia, ib = r.integers(0, 50, 20).astype(np.int32), r.integers(0, 25, 12).astype(np.int32)
    ga, gb = r.standard_normal((20, 16)).astype(np.float32), r.standard_normal((12, 16)).astype(np.float32)
    T = omb.Tensor.from_numpy

    def lookups(table):
        a = omb.call("embedding", [table, T(ia)], ints=[-1, 1])
        b = omb.call("embedding", [table, T(ib)], ints=[-1, 1])
        return omb.call("add", [omb.call("sum", [omb.call("mul", [a, T(ga)])]), omb.call("sum", [omb.call("mul", [b, T(gb)])])])

    table = T(tv, True)
    lookups(table).backward()
    sg = table.sparse_grad
    assert sg is not None and table.grad is None
    assert np.array_equal(sg.rows.numpy(), np.union1d(ia, ib))
    want = K.embedding_bwd(ga, ia, 50, 16) + K.embedding_bwd(gb, ib, 50, 16)
    got = sg.to_dense().numpy()
    other = K.embedding_bwd(gb, ib, 50, 16) + K.embedding_bwd(ga, ia, 50, 16)
    assert np.array_equal(got, want) or np.array_equal(got, other)     # the order the two arrive in is the engine's
    # the same table also used densely: the leaf ends with a dense gradient holding everything
    table2 = T(tv, True)
    omb.call("add", [lookups(table2), omb.call("sum", [table2])]).backward()
    assert table2.sparse_grad is None
    assert np.max(np.abs(table2.grad.numpy() - (want + 1))) <= 1e-5
    # a computed table: the gradient flows on as dense
    base = T(tv, True)
    doubled = omb.call("add", [base, base])
    lookups(doubled).backward()
    assert base.sparse_grad is None and np.max(np.abs(base.grad.numpy() - 2 * want)) <= 1e-5
