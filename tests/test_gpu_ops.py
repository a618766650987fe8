"""Per-entry-point parity: every C-ABI kernel against the CPU oracle on the same seeded inputs.

Tolerances: bit-exact for integer/index results, for the fp32 FMA matrix product (same accumulation order as the
oracle) and for the optimizer updates (same rounding sequence); rtol 1e-4 (scaled) for everything else on the fp32
path - the "TF32 disabled" tier of the parity contract. The tensor-pipe tier is covered in test_gpu_gemm_tc.py."""
import ctypes as C

import numpy as np
import pytest

import om_binding as omb
from backends import scaled_diff
from om_binding import f32, i32, i64

pytestmark = pytest.mark.gpu
TOL = 1e-4


@pytest.fixture(scope="module")
def K(oracle_built):
    return oracle_built


def rng(seed):
    return np.random.default_rng(seed)


def normal(r, *shape, scale=1.0):
    return (r.standard_normal(shape) * scale).astype(np.float32)


@pytest.mark.parametrize("ta,tb", [(0, 0), (0, 1), (1, 0), (1, 1)])
@pytest.mark.parametrize("m,n,k", [(128, 512, 784), (37, 53, 91), (1, 10, 512), (130, 7, 1), (256, 384, 384)])
def test_matmul_fp32_bit_exact(ctx, K, ta, tb, m, n, k):
    ctx.set_flags(0)
    r = rng(m * 1000 + n * 10 + k + ta * 2 + tb)
    a = normal(r, *((k, m) if ta else (m, k)))
    b = normal(r, *((n, k) if tb else (k, n)))
    da, db, dc = ctx.to_device(a), ctx.to_device(b), ctx.empty((m, n))
    ctx.call("om_matmul", ctx.handle, i32(ta), i32(tb), i32(m), i32(n), i32(k), da.ptr, i32(a.shape[1]), db.ptr,
             i32(b.shape[1]), dc.ptr, i32(n), i32(0))
    ref = K.gemm(a, b, bool(ta), bool(tb))
    assert np.array_equal(dc.numpy(), ref)
    # accumulate adds the product to the existing contents
    ctx.call("om_matmul", ctx.handle, i32(ta), i32(tb), i32(m), i32(n), i32(k), da.ptr, i32(a.shape[1]), db.ptr,
             i32(b.shape[1]), dc.ptr, i32(n), i32(1))
    assert np.array_equal(dc.numpy(), ref + ref)


def test_matmul_empty_and_bad_shape(ctx):
    d = ctx.empty((4,))
    ctx.call("om_matmul", ctx.handle, i32(0), i32(0), i32(0), i32(5), i32(3), d.ptr, i32(3), d.ptr, i32(5), d.ptr, i32(5), i32(0))
    with pytest.raises(omb.ShapeError):
        ctx.call("om_matmul", ctx.handle, i32(0), i32(0), i32(-1), i32(5), i32(3), d.ptr, i32(3), d.ptr, i32(5), d.ptr, i32(5), i32(0))


@pytest.mark.parametrize("rows,inf,outf", [(128, 784, 512), (33, 20, 7), (1229, 384, 1000)])
def test_linear_fwd_bwd(ctx, K, rows, inf, outf):
    ctx.set_flags(0)
    r = rng(rows + inf)
    x, w, b, g = normal(r, rows, inf), normal(r, outf, inf, scale=0.1), normal(r, outf), normal(r, rows, outf)
    dx_, dw_, db_ = ctx.empty((rows, inf)), ctx.empty((outf, inf)), ctx.empty((outf,))
    X, W, Bv, G, Y = ctx.to_device(x), ctx.to_device(w), ctx.to_device(b), ctx.to_device(g), ctx.empty((rows, outf))
    ctx.call("om_linear_fwd", ctx.handle, X.ptr, W.ptr, Bv.ptr, i32(rows), i32(inf), i32(outf), Y.ptr)
    assert np.array_equal(Y.numpy(), K.gemm(x, w, tb=True) + b)
    ctx.call("om_linear_bwd", ctx.handle, G.ptr, X.ptr, W.ptr, i32(rows), i32(inf), i32(outf), dx_.ptr, dw_.ptr, db_.ptr, i32(0))
    assert np.array_equal(dx_.numpy(), K.gemm(g, w))
    assert np.array_equal(dw_.numpy(), K.gemm(g, x, ta=True))
    assert scaled_diff(db_.numpy(), K.sum_to(g, (outf,))) <= 1e-6
    # accumulate into existing weight gradients (Engine.AddInto)
    ctx.call("om_linear_bwd", ctx.handle, G.ptr, X.ptr, W.ptr, i32(rows), i32(inf), i32(outf), None, dw_.ptr, db_.ptr, i32(1))
    assert np.array_equal(dw_.numpy(), K.gemm(g, x, ta=True) * 2)


@pytest.mark.parametrize("op", ["relu", "gelu_erf", "gelu_tanh", "sigmoid", "tanh", "neg"])
@pytest.mark.parametrize("n", [1, 1023, 65536 + 3])
def test_unary_fwd_bwd(ctx, K, op, n):
    r = rng(n)
    x, g = normal(r, n, scale=2.0), normal(r, n)
    X, G, Y, D = ctx.to_device(x), ctx.to_device(g), ctx.empty((n,)), ctx.empty((n,))
    ctx.call("om_unary", ctx.handle, i32(omb.UNARY[op]), X.ptr, Y.ptr, i64(n))
    y_ref = K.unary(op, x)
    assert scaled_diff(Y.numpy(), y_ref) <= 1e-6
    saved = x if op.startswith("gelu") else y_ref
    S = ctx.to_device(saved)
    ctx.call("om_unary_bwd", ctx.handle, i32(omb.UNARY[op]), G.ptr, S.ptr, D.ptr, i64(n))
    ref = K.unary_bwd(op, g, saved)
    if op in ("relu", "neg"):
        assert np.array_equal(D.numpy(), ref)
    else:
        assert scaled_diff(D.numpy(), ref) <= 1e-5


def test_relu_nan_and_zero(ctx):
    x = np.array([np.nan, -0.0, 0.0, -1.0, 2.0], np.float32)
    X, Y = ctx.to_device(x), ctx.empty((5,))
    ctx.call("om_unary", ctx.handle, i32(1), X.ptr, Y.ptr, i64(5))
    y = Y.numpy()
    assert np.isnan(y[0]) and np.array_equal(y[1:], np.array([0, 0, 0, 2], np.float32))


@pytest.mark.parametrize("shape,target", [((8192, 384), (384,)), ((7, 5, 3), (5, 1)), ((4, 6), (4, 1)), ((3, 4, 5), (3, 1, 5)), ((513, 33), (33,))])
def test_sum_to(ctx, K, shape, target):
    r = rng(sum(shape))
    g = normal(r, *shape)
    ref = K.sum_to(g, target)
    rank, lead = len(shape), len(shape) - len(target)
    ts, acc = [0] * rank, 1
    for ax in range(rank - 1, -1, -1):
        t = ax - lead
        if t >= 0 and target[t] != 1:
            ts[ax] = acc
            acc *= target[t]
    G, O = ctx.to_device(g), ctx.empty(target)
    ctx.call("om_sum_to", ctx.handle, i32(rank), omb.int_array(shape), G.ptr, omb.int_array(ts, C.c_int64), O.ptr, i64(ref.size))
    # double accumulators rounded once: identical except for rare ties in the last bit
    assert scaled_diff(O.numpy(), ref) <= 2e-7


@pytest.mark.parametrize("rows,cols", [(128, 10), (64, 97), (37, 30522), (5, 1025), (0, 7)])
def test_softmax_family(ctx, K, rows, cols):
    r = rng(rows + cols)
    x, g = normal(r, rows, cols, scale=3.0), normal(r, rows, cols)
    X, G, Y, D = ctx.to_device(x), ctx.to_device(g), ctx.empty((rows, cols)), ctx.empty((rows, cols))
    for fwd, bwd, kf, kb in (("om_softmax_fwd", "om_softmax_bwd", K.softmax_fwd, K.softmax_bwd),
                             ("om_logsoftmax_fwd", "om_logsoftmax_bwd", K.logsoftmax_fwd, K.logsoftmax_bwd)):
        ctx.call(fwd, ctx.handle, X.ptr, i32(rows), i32(cols), Y.ptr)
        y_ref = kf(x)
        if rows:
            assert scaled_diff(Y.numpy(), y_ref) <= 1e-5
        Yr = ctx.to_device(y_ref)
        ctx.call(bwd, ctx.handle, G.ptr, Yr.ptr, i32(rows), i32(cols), D.ptr)
        if rows:
            assert scaled_diff(D.numpy(), kb(g, y_ref)) <= 1e-5


@pytest.mark.parametrize("dtype", [np.int32, np.int64])
@pytest.mark.parametrize("mean", [1, 0])
def test_nll_and_cross_entropy(ctx, K, dtype, mean):
    r = rng(5)
    rows, cols = 257, 1031
    logits = normal(r, rows, cols, scale=2.0)
    t = r.integers(0, cols, rows)
    t[::7] = -100
    logp = K.logsoftmax_fwd(logits)
    loss_ref, count_ref = K.nll_fwd(logp, t, bool(mean))
    LP, T = ctx.to_device(logp), ctx.to_device(t.astype(dtype))
    loss, count = ctx.empty(()), ctx.empty((1,), np.int32)
    dt = omb.OM_I32 if dtype == np.int32 else omb.OM_I64
    ctx.call("om_nll_fwd", ctx.handle, LP.ptr, T.ptr, i32(dt), i32(rows), i32(cols), i32(mean), i64(-100), loss.ptr, count.ptr)
    assert count.numpy()[0] == count_ref                      # integer: exact
    assert abs(float(loss.numpy()) - float(loss_ref)) <= 1e-6 * abs(float(loss_ref))
    g = np.float32(0.7)
    Gs, D = ctx.to_device(np.array(g)), ctx.empty((rows, cols))
    ctx.call("om_nll_bwd", ctx.handle, Gs.ptr, T.ptr, i32(dt), i32(rows), i32(cols), i32(mean), i64(-100), D.ptr)
    dlogp_ref = K.nll_bwd(g, t, (rows, cols), bool(mean))
    assert np.array_equal(D.numpy(), dlogp_ref)
    # fused cross entropy = log-softmax backward of the NLL gradient
    X, LP2, L2 = ctx.to_device(logits), ctx.empty((rows, cols)), ctx.empty(())
    ctx.call("om_cross_entropy_fwd", ctx.handle, X.ptr, T.ptr, i32(dt), i32(rows), i32(cols), i32(mean), i64(-100), f32(0), LP2.ptr, L2.ptr, None)
    assert scaled_diff(LP2.numpy(), logp) <= 1e-6
    ctx.call("om_cross_entropy_bwd", ctx.handle, Gs.ptr, LP.ptr, T.ptr, i32(dt), i32(rows), i32(cols), i32(mean), i64(-100), f32(0), D.ptr)
    assert scaled_diff(D.numpy(), K.logsoftmax_bwd(dlogp_ref, logp)) <= 1e-6


def test_nll_target_out_of_range_reports_index_error(ctx):
    logp = np.zeros((4, 3), np.float32)
    LP, T, loss = ctx.to_device(logp), ctx.to_device(np.array([0, 5, 1, 2], np.int64)), ctx.empty(())
    ctx.call("om_nll_fwd", ctx.handle, LP.ptr, T.ptr, i32(omb.OM_I64), i32(4), i32(3), i32(1), i64(-100), loss.ptr, None)
    with pytest.raises(omb.IndexOutOfRange):
        ctx.sync()
    ctx.sync()  # the status word was cleared


@pytest.mark.parametrize("rows,cols", [(8192, 384), (77, 16), (130, 768), (3, 1000), (64, 33)])
def test_layernorm(ctx, K, rows, cols):
    r = rng(rows + cols)
    x, g = normal(r, rows, cols, scale=2.0), normal(r, rows, cols)
    gamma, beta = 1 + normal(r, cols, scale=0.1), normal(r, cols, scale=0.1)
    y_ref, mu, inv = K.layernorm_fwd(x, gamma, beta)
    X, Ga, Be, Y = ctx.to_device(x), ctx.to_device(gamma), ctx.to_device(beta), ctx.empty((rows, cols))
    M, I = ctx.empty((rows,)), ctx.empty((rows,))
    ctx.call("om_layernorm_fwd", ctx.handle, X.ptr, Ga.ptr, Be.ptr, i32(rows), i32(cols), f32(1e-5), Y.ptr, M.ptr, I.ptr)
    assert scaled_diff(Y.numpy(), y_ref) <= 1e-5
    assert scaled_diff(M.numpy(), mu) <= 1e-5 and scaled_diff(I.numpy(), inv) <= 1e-5
    dx_ref, dg_ref, db_ref = K.layernorm_bwd(g, x, gamma, mu, inv)
    G, Mu, Iv = ctx.to_device(g), ctx.to_device(mu), ctx.to_device(inv)
    DX, DG, DB = ctx.empty((rows, cols)), ctx.empty((cols,)), ctx.empty((cols,))
    ctx.call("om_layernorm_bwd", ctx.handle, G.ptr, X.ptr, Ga.ptr, Mu.ptr, Iv.ptr, i32(rows), i32(cols), DX.ptr, DG.ptr, DB.ptr, i32(0))
    assert scaled_diff(DX.numpy(), dx_ref) <= 1e-5
    assert scaled_diff(DG.numpy(), dg_ref) <= 1e-6
    assert scaled_diff(DB.numpy(), db_ref) <= 1e-6


@pytest.mark.parametrize("n,c,h,w", [(8, 4, 12, 12), (256, 64, 8, 8), (3, 5, 1, 7)])
def test_batchnorm(ctx, K, n, c, h, w):
    r = rng(n + c)
    x, g = normal(r, n, c, h, w, scale=2.0) + 0.5, normal(r, n, c, h, w)
    gamma, beta = 1 + normal(r, c, scale=0.1), normal(r, c, scale=0.1)
    rm, rv = np.zeros(c, np.float32), np.ones(c, np.float32)
    y_ref, mu, iv = K.batchnorm_fwd(x, gamma, beta, rm, rv, True)
    X, Ga, Be = ctx.to_device(x), ctx.to_device(gamma), ctx.to_device(beta)
    RM, RV = ctx.to_device(np.zeros(c, np.float32)), ctx.to_device(np.ones(c, np.float32))
    Y, M, I = ctx.empty(x.shape), ctx.empty((c,)), ctx.empty((c,))
    ctx.call("om_batchnorm_fwd", ctx.handle, X.ptr, Ga.ptr, Be.ptr, RM.ptr, RV.ptr, i32(n), i32(c), i32(h * w), i32(1), f32(0.1), f32(1e-5), Y.ptr, M.ptr, I.ptr)
    assert scaled_diff(Y.numpy(), y_ref) <= 1e-5
    assert scaled_diff(RM.numpy(), rm) <= 1e-6 and scaled_diff(RV.numpy(), rv) <= 1e-6
    dx_ref, dg_ref, db_ref = K.batchnorm_bwd(g, x, gamma, mu, iv, True)
    G, Mu, Iv = ctx.to_device(g), ctx.to_device(mu), ctx.to_device(iv)
    DX, DG, DB = ctx.empty(x.shape), ctx.empty((c,)), ctx.empty((c,))
    ctx.call("om_batchnorm_bwd", ctx.handle, G.ptr, X.ptr, Ga.ptr, Mu.ptr, Iv.ptr, i32(n), i32(c), i32(h * w), i32(1), DX.ptr, DG.ptr, DB.ptr, i32(0))
    assert scaled_diff(DX.numpy(), dx_ref) <= 1e-5
    assert scaled_diff(DG.numpy(), dg_ref) <= 1e-6 and scaled_diff(DB.numpy(), db_ref) <= 1e-6


@pytest.mark.parametrize("dtype", [np.int32, np.int64])
def test_embedding_fwd_bwd_bit_exact(ctx, K, dtype):
    r = rng(11)
    v, dim, n = 1000, 48, 4096
    table, g = normal(r, v, dim), normal(r, n, dim)
    ids = r.integers(0, 50, n)          # heavy duplication: order of the per-row sums matters
    ids[:100] = r.integers(0, v, 100)
    ids[5] = 3
    dt = omb.OM_I32 if dtype == np.int32 else omb.OM_I64
    Tb, Id, Out = ctx.to_device(table), ctx.to_device(ids.astype(dtype)), ctx.empty((n, dim))
    ctx.call("om_embedding_fwd", ctx.handle, Tb.ptr, i32(v), i32(dim), Id.ptr, i32(dt), i64(n), Out.ptr)
    assert np.array_equal(Out.numpy(), K.embedding_fwd(table, ids))
    G, DT = ctx.to_device(g), ctx.empty((v, dim))
    for pad in (-1, 3):
        ctx.call("om_embedding_bwd", ctx.handle, G.ptr, Id.ptr, i32(dt), i64(n), i32(v), i32(dim), i64(pad), DT.ptr, i32(0))
        assert np.array_equal(DT.numpy(), K.embedding_bwd(g, ids, v, dim, pad))
    ctx.sync()
    # accumulate: each touched row continues from what the table gradient already holds, in the same position order
    # (existing + g[p0] + g[p1] + ...); untouched rows keep their values. Also a width that is not a multiple of four.
    for width in (dim, 7):
        gw = np.ascontiguousarray(g[:, :width])
        held = normal(r, v, width)
        Gw, ACC = ctx.to_device(gw), ctx.to_device(held)
        ctx.call("om_embedding_bwd", ctx.handle, Gw.ptr, Id.ptr, i32(dt), i64(n), i32(v), i32(width), i64(-1), ACC.ptr, i32(1))
        ctx.sync()
        want = held.copy()
        for p_, t in enumerate(ids):
            want[t] = want[t] + gw[p_]
        assert np.array_equal(ACC.numpy(), want)


def test_embedding_id_out_of_range(ctx):
    Tb, Id, Out = ctx.to_device(np.zeros((4, 2), np.float32)), ctx.to_device(np.array([1, 9], np.int64)), ctx.empty((2, 2))
    ctx.call("om_embedding_fwd", ctx.handle, Tb.ptr, i32(4), i32(2), Id.ptr, i32(omb.OM_I64), i64(2), Out.ptr)
    with pytest.raises(omb.IndexOutOfRange):
        ctx.sync()


@pytest.mark.parametrize("b,h,lq,lk,d,masked", [(2, 2, 5, 5, 8, 2), (3, 4, 128, 128, 32, 0), (1, 2, 33, 70, 16, 1), (2, 1, 64, 64, 64, 0)])
def test_attention(ctx, K, b, h, lq, lk, d, masked):
    ctx.set_flags(0)
    r = rng(b + lq + d)
    q, k, v, g = normal(r, b, h, lq, d), normal(r, b, h, lk, d), normal(r, b, h, lk, d), normal(r, b, h, lq, d)
    mask = None
    if masked == 1:
        mask = np.where(r.random((lq, lk)) < 0.25, -4.0, 0.0).astype(np.float32)
    elif masked == 2:
        mask = np.where(r.random((b, lq, lk)) < 0.25, -4.0, 0.0).astype(np.float32)
    scale = np.float32(1.0 / np.sqrt(np.float32(d)))
    Q, Kk, V, G = ctx.to_device(q), ctx.to_device(k), ctx.to_device(v), ctx.to_device(g)
    M = ctx.to_device(mask) if mask is not None else None
    mbs = 0 if (mask is None or mask.ndim == 2) else lq * lk
    O = ctx.empty(q.shape)
    ctx.call("om_attention_fwd", ctx.handle, Q.ptr, Kk.ptr, V.ptr, M.ptr if M else None, i64(mbs), i32(b), i32(h), i32(lq), i32(lk), i32(d), f32(scale), O.ptr, None)
    assert scaled_diff(O.numpy(), K.attention_fwd(q, k, v, mask)) <= TOL
    DQ, DK, DV = ctx.empty(q.shape), ctx.empty(k.shape), ctx.empty(v.shape)
    ctx.call("om_attention_bwd", ctx.handle, G.ptr, Q.ptr, Kk.ptr, V.ptr, M.ptr if M else None, i64(mbs), None, i32(b), i32(h), i32(lq), i32(lk), i32(d), f32(scale), DQ.ptr, DK.ptr, DV.ptr)
    dq, dk, dv = K.attention_bwd(g, q, k, v, mask)
    assert scaled_diff(DQ.numpy(), dq) <= TOL and scaled_diff(DK.numpy(), dk) <= TOL and scaled_diff(DV.numpy(), dv) <= TOL


def int_pow(b, n):
    """Adam.IntPow: binary powering in double (src/OneModel.Training/Optimizers.cs:483-499)."""
    r = 1.0
    while n > 0:
        if n & 1:
            r *= b
        b *= b
        n >>= 1
    return r


def _ptr_table(arrays):
    return (C.c_void_p * len(arrays))(*[a.ptr.value for a in arrays])


@pytest.mark.parametrize("decoupled,amsgrad,wd", [(0, 0, 0.0), (0, 0, 0.1), (1, 0, 0.01), (1, 1, 0.05)])
def test_adam_multi_tensor_bit_exact(ctx, K, decoupled, amsgrad, wd):
    r = rng(3)
    sizes = [1, 7, 384, 16384 + 5, 70001] + [33] * 45      # more tensors than one launch table holds
    ps = [normal(r, n) for n in sizes]
    ms = [np.zeros(n, np.float32) for n in sizes]
    vs = [np.zeros(n, np.float32) for n in sizes]
    vm = [np.zeros(n, np.float32) for n in sizes]
    P, M, V, VM = ([ctx.to_device(a) for a in arrs] for arrs in (ps, ms, vs, vm))
    lens = omb.int_array(sizes, C.c_int64)

    class Hyper(C.Structure):
        _fields_ = [(n, C.c_float) for n in ("lr", "beta1", "beta2", "eps", "weight_decay", "step_size", "sqrt_bc2", "grad_scale")] + [("decoupled", C.c_int32), ("amsgrad", C.c_int32)]

    lr, b1, b2, eps = 1e-2, 0.9, 0.999, 1e-8
    for t in range(1, 4):
        gs = [normal(r, n) for n in sizes]
        G = [ctx.to_device(a) for a in gs]
        bc1 = 1.0 - int_pow(float(np.float32(b1)), t)
        bc2 = 1.0 - int_pow(float(np.float32(b2)), t)
        hyper = Hyper(lr, b1, b2, eps, wd, np.float32(np.float64(np.float32(lr)) / bc1), np.float32(np.sqrt(bc2)), 1.0, decoupled, amsgrad)
        ctx.call("om_optim_adam_step", ctx.handle, i32(len(sizes)), _ptr_table(P), _ptr_table(G), _ptr_table(M), _ptr_table(V),
                 _ptr_table(VM), lens, C.byref(hyper), None)
        for i in range(len(sizes)):
            K.adam_step(ps[i], gs[i], ms[i], vs[i], vm[i], t, lr, b1, b2, eps, wd, bool(decoupled), bool(amsgrad))
    for i in range(len(sizes)):
        assert np.array_equal(P[i].numpy(), ps[i]), i
        assert np.array_equal(M[i].numpy(), ms[i]) and np.array_equal(V[i].numpy(), vs[i])


def test_strided_copy_permute_and_flip(ctx):
    r = rng(9)
    x = normal(r, 4, 6, 5, 8)
    X = ctx.to_device(x)
    for axes in [(0, 2, 1, 3), (3, 2, 1, 0), (1, 0, 2, 3)]:
        y = x.transpose(axes)
        O = ctx.empty(y.shape)
        src = [s // 4 for s in y.strides]
        dst = [s // 4 for s in np.ascontiguousarray(y).strides]
        ctx.call("om_strided_copy", ctx.handle, i32(4), omb.int_array(y.shape), X.ptr, omb.int_array(src, C.c_int64), O.ptr, omb.int_array(dst, C.c_int64))
        assert np.array_equal(O.numpy(), y)
    m = normal(r, 70, 45)
    Mx, O = ctx.to_device(m), ctx.empty((45, 70))
    ctx.call("om_strided_copy", ctx.handle, i32(2), omb.int_array((45, 70)), Mx.ptr, omb.int_array((1, 45), C.c_int64), O.ptr, omb.int_array((70, 1), C.c_int64))
    assert np.array_equal(O.numpy(), m.T)


def test_zero_and_pool(ctx):
    arrays = [ctx.to_device(np.ones(n, np.float32)) for n in (1, 5, 100003)]
    ctx.call("om_zero", ctx.handle, i32(3), _ptr_table(arrays), omb.int_array([a.size for a in arrays], C.c_int64))
    for a in arrays:
        assert not a.numpy().any()
    used, cached, allocs = C.c_uint64(), C.c_uint64(), C.c_uint64()
    ctx.call("om_pool_stats", ctx.handle, C.byref(used), C.byref(cached), C.byref(allocs))
    assert used.value > 0


def test_a_bounded_wait_that_runs_out_is_reported_and_the_context_stays_usable(ctx):
    """The tensor-pipe kernels' waits are bounded. With a budget of one millisecond, a wait that nothing will ever satisfy
    (om_selftest_bounded_wait: one warp on a barrier without arrivals) runs out, the kernel returns, om_sync reports
    OM_ERR_TIMEOUT with the place of the wait, the status is cleared by the report, and the next product on the same
    context is correct. Nothing hangs or faults: the wait is one millisecond long."""
    import time
    ctx.set_flags(omb.OM_TF32)
    try:
        ctx.call("om_ctx_set_wait_budget_us", ctx.handle, C.c_int64(1000))
        t0 = time.perf_counter()
        ctx.call("om_selftest_bounded_wait", ctx.handle)
        with pytest.raises(omb.OmError) as e:
            ctx.sync()
        assert e.value.status == 6 and "wait expired" in str(e.value) and "detail 99" in str(e.value)
        assert time.perf_counter() - t0 < 0.5
        ctx.sync()                                    # reported once, then clear
        r = np.random.default_rng(3)
        a, b = r.standard_normal((256, 128)).astype(np.float32), r.standard_normal((128, 256)).astype(np.float32)
        A, Bm, Cm = ctx.to_device(a), ctx.to_device(b), ctx.empty((256, 256))
        ctx.call("om_matmul", ctx.handle, i32(0), i32(0), i32(256), i32(256), i32(128), A.ptr, i32(128), Bm.ptr, i32(256), Cm.ptr, i32(256), i32(0))
        ctx.sync()
        assert scaled_diff(Cm.numpy(), a @ b) <= 1e-3
    finally:
        ctx.call("om_ctx_set_wait_budget_us", ctx.handle, C.c_int64(0))
        ctx.set_flags(0)


def test_checked_mode_poisons_memory_and_catches_a_write_past_the_end(ctx):
    """OM_CHECKED (the reference's CHECKED build, docs/tensors.md:108-110): fresh memory reads as 0xFF bytes (NaN), 64 guard
    bytes follow every buffer, and a write that runs past a buffer's end is reported when the buffer is released. The
    overrun here stays inside the guard area of the block itself, so no foreign memory is touched."""
    ctx.set_flags(omb.OM_CHECKED)
    try:
        n = 100
        ptr = C.c_void_p()
        ctx.call("om_alloc", ctx.handle, C.c_size_t(4 * n), i32(0), C.byref(ptr))
        host = np.empty(n, np.float32)
        ctx.call("om_memcpy_d2h", ctx.handle, host.ctypes.data_as(C.c_void_p), ptr, C.c_size_t(4 * n))
        assert np.all(np.isnan(host)) and np.all(host.view(np.uint32) == 0xFFFFFFFF)
        ctx.call("om_fill", ctx.handle, ptr, f32(1.0), i64(n))            # inside the buffer: fine
        ctx.call("om_free", ctx.handle, ptr)
        ctx.sync()
        ctx.call("om_alloc", ctx.handle, C.c_size_t(4 * n), i32(1), C.byref(ptr))   # zeroed on request, still guarded
        ctx.call("om_memcpy_d2h", ctx.handle, host.ctypes.data_as(C.c_void_p), ptr, C.c_size_t(4 * n))
        assert not host.any()
        ctx.call("om_fill", ctx.handle, ptr, f32(2.0), i64(n + 3))        # three floats past the end: into the guard bytes
        ctx.call("om_free", ctx.handle, ptr)
        with pytest.raises(omb.OmError) as e:
            ctx.sync()
        assert e.value.status == 9 and "guard bytes" in str(e.value)
        ctx.sync()
        # A whole op under the flag (its scratch blocks are guarded too) still gives the right answer.
        g = np.random.default_rng(4).standard_normal((700, 96)).astype(np.float32)
        G, O = ctx.to_device(g), ctx.empty((96,))
        ctx.call("om_colsum", ctx.handle, G.ptr, i32(700), i32(96), O.ptr, i32(0))
        ctx.sync()
        assert np.allclose(O.numpy(), g.astype(np.float64).sum(0), rtol=1e-5, atol=1e-5)
    finally:
        ctx.set_flags(0)
