"""The persistent CTA-pair product kernel (two accumulator buffers in tensor memory) against the CPU oracle: with
bfloat16 operands (the om_*_bf16 entry points) and, under OM_PERSISTENT_TILES, with TF32 operands.

The oracle rounds the operands the same way (bfloat16 or TF32, to nearest even) and sums in fp32 in increasing k, so
what is left is the order of the fp32 accumulation: 2e-5 scaled. Against the fp32 oracle the operand rounding itself
shows: bfloat16 keeps 8 significant bits, so every product is within 2^-7 relative and every element within
2^-7 * (|A||B|) of the fp32 result."""
import ctypes as C

import numpy as np
import pytest

import om_binding as omb
from backends import scaled_diff
from om_binding import i32, i64

pytestmark = pytest.mark.gpu

# m, n, k: one tile, several tiles per cluster, ragged edges in every dimension, a split k, the encoder's own shapes
SHAPES = [(256, 256, 64), (256, 128, 128), (512, 768, 768), (2048, 2304, 768), (1000, 520, 200), (300, 264, 136),
          (768, 768, 16384), (2304, 768, 4096), (154, 30528, 768), (4096, 768, 3072), (64, 72, 40)]


def to_bf16(ctx, a):
    """The bfloat16 copy of a float32 array on the device (om_cast_bf16), as a DeviceArray of uint16."""
    src = ctx.to_device(np.ascontiguousarray(a, np.float32))
    dst = ctx.empty(a.shape, np.uint16)
    ctx.call("om_cast_bf16", ctx.handle, src.ptr, dst.ptr, i64(a.size))
    return dst


def test_cast_rounds_to_nearest_even(ctx, oracle_built):
    K = oracle_built
    r = np.random.default_rng(5)
    x = np.concatenate([r.standard_normal(100003).astype(np.float32) * 10.0 ** r.integers(-20, 20, 100003).astype(np.float32),
                        # ties: exactly half way between two bfloat16 values, both parities
                        np.array([1.00390625, 1.01171875, -1.00390625, 3.0e38, 0.0, -0.0, 1e-40], np.float32)])
    got = to_bf16(ctx, x).numpy()
    ctx.sync()
    want = (K.round_bf16(x).view(np.uint32) >> 16).astype(np.uint16)
    assert np.array_equal(got, want)


def run_bf16(ctx, ta, tb, m, n, k, a, b, acc=0, c0=None, ldc=None):
    da, db = to_bf16(ctx, a), to_bf16(ctx, b)
    ldc = ldc or n
    dc = ctx.to_device(c0) if c0 is not None else ctx.empty((m, ldc))
    ctx.call("om_matmul_bf16", ctx.handle, i32(ta), i32(tb), i32(m), i32(n), i32(k), da.ptr, i32(a.shape[1]), db.ptr, i32(b.shape[1]),
             dc.ptr, i32(ldc), i32(acc))
    ctx.sync()
    return dc.numpy()


@pytest.mark.parametrize("ta,tb", [(0, 1), (0, 0), (1, 0), (1, 1)])
@pytest.mark.parametrize("m,n,k", SHAPES)
def test_bf16_matmul(ctx, oracle_built, ta, tb, m, n, k):
    K = oracle_built
    r = np.random.default_rng(m + 3 * n + 7 * k + ta * 2 + tb)
    a = r.standard_normal((k, m) if ta else (m, k)).astype(np.float32)
    b = r.standard_normal((n, k) if tb else (k, n)).astype(np.float32)
    if a.shape[1] % 8 or b.shape[1] % 8:
        pytest.skip("an operand pitch that is not a multiple of 16 bytes: refused (see the last test of this group)")
    got = run_bf16(ctx, ta, tb, m, n, k, a, b)
    ref16 = K.gemm(a, b, bool(ta), bool(tb), mode="bf16")
    assert scaled_diff(got, ref16) <= 2e-5
    ref = K.gemm(a, b, bool(ta), bool(tb))
    aa = np.abs(a.T if ta else a).astype(np.float64)
    bb = np.abs(b.T if tb else b).astype(np.float64)
    assert np.all(np.abs(got.astype(np.float64) - ref) <= 2.0 ** -7 * (aa @ bb) + 1e-5)
    assert scaled_diff(got, ref) <= 8e-3
    c0 = r.standard_normal((m, n)).astype(np.float32)
    got2 = run_bf16(ctx, ta, tb, m, n, k, a, b, acc=1, c0=c0)
    assert scaled_diff(got2, ref16 + c0) <= 2e-5
    assert np.array_equal(got, run_bf16(ctx, ta, tb, m, n, k, a, b))      # fixed split of k, ordered combine: same bits


def test_bf16_linear_forward_and_backward(ctx, oracle_built):
    """om_linear_fwd_bf16 / om_linear_bwd_bf16 at one feed-forward layer of the BERT-base shape (a quarter of its rows),
    with a row-pitched output, the bias in the epilogue and the bias gradient from the fp32 gradient."""
    K = oracle_built
    r = np.random.default_rng(9)
    rows, inf, outf, ld = 4096, 768, 3070, 3072
    x, w = r.standard_normal((rows, inf)).astype(np.float32), (r.standard_normal((outf, inf)) * 0.05).astype(np.float32)
    bias = r.standard_normal(outf).astype(np.float32)
    g = np.zeros((rows, ld), np.float32)
    g[:, :outf] = r.standard_normal((rows, outf))
    X16, W16, G16 = to_bf16(ctx, x), to_bf16(ctx, w), to_bf16(ctx, g)
    Bv, G = ctx.to_device(bias), ctx.to_device(g)
    Y, DX, DW, DB = ctx.zeros((rows, ld)), ctx.empty((rows, inf)), ctx.empty((outf, inf)), ctx.empty((outf,))
    ctx.call("om_linear_fwd_bf16", ctx.handle, X16.ptr, W16.ptr, Bv.ptr, i32(rows), i32(inf), i32(outf), Y.ptr, i32(ld))
    ctx.call("om_linear_bwd_bf16", ctx.handle, G16.ptr, G.ptr, i32(ld), X16.ptr, W16.ptr, i32(rows), i32(inf), i32(outf), DX.ptr, DW.ptr, DB.ptr, i32(0))
    ctx.sync()
    y = Y.numpy()
    assert scaled_diff(y[:, :outf], K.gemm(x, w, tb=True, mode="bf16") + bias) <= 2e-5
    assert np.all(y[:, outf:] == 0)                                          # the pitch columns are not written
    gv = g[:, :outf]
    assert scaled_diff(DX.numpy(), K.gemm(gv, w, mode="bf16")) <= 2e-5
    assert scaled_diff(DW.numpy(), K.gemm(gv, x, ta=True, mode="bf16")) <= 2e-5
    assert np.allclose(DB.numpy(), gv.astype(np.float64).sum(0), rtol=1e-5, atol=1e-4)


def test_bf16_operands_that_tma_cannot_describe_are_refused(ctx):
    a, b = ctx.empty((64, 100), np.uint16), ctx.empty((100, 72), np.uint16)
    c = ctx.empty((64, 72))
    with pytest.raises(omb.OmError) as e:      # an A pitch of 100 elements is 200 bytes
        ctx.call("om_matmul_bf16", ctx.handle, i32(0), i32(0), i32(64), i32(72), i32(100), a.ptr, i32(100), b.ptr, i32(72), c.ptr, i32(72), i32(0))
    assert "multiples of 8" in str(e.value)
    ctx.sync()


def run_tf32(ctx, ta, tb, m, n, k, a, b, acc=0, c0=None):
    da, db = ctx.to_device(a), ctx.to_device(b)
    dc = ctx.to_device(c0) if c0 is not None else ctx.empty((m, n))
    ctx.call("om_matmul", ctx.handle, i32(ta), i32(tb), i32(m), i32(n), i32(k), da.ptr, i32(a.shape[1]), db.ptr, i32(b.shape[1]), dc.ptr, i32(n), i32(acc))
    ctx.sync()
    return dc.numpy()


@pytest.mark.parametrize("ta,tb", [(0, 1), (0, 0), (1, 0), (1, 1)])
@pytest.mark.parametrize("m,n,k", [(256, 256, 64), (8192, 384, 384), (8192, 1536, 384), (384, 1536, 8192), (1229, 30524, 384), (1000, 520, 200), (300, 264, 136)])
def test_tf32_matmul_on_the_persistent_kernel(ctx, oracle_built, ta, tb, m, n, k):
    K = oracle_built
    r = np.random.default_rng(m * 3 + n + k)
    a = r.standard_normal((k, m) if ta else (m, k)).astype(np.float32)
    b = r.standard_normal((n, k) if tb else (k, n)).astype(np.float32)
    if a.shape[1] % 4 or b.shape[1] % 4:
        pytest.skip("operand pitch not a multiple of 16 bytes: this shape runs on the fp32 kernel")
    try:
        ctx.set_flags(omb.OM_TF32 | omb.OM_PERSISTENT_TILES)
        got = run_tf32(ctx, ta, tb, m, n, k, a, b)
        ref = K.gemm(a, b, bool(ta), bool(tb), mode="tf32")
        assert scaled_diff(got, ref) <= 2e-5
        c0 = r.standard_normal((m, n)).astype(np.float32)
        assert scaled_diff(run_tf32(ctx, ta, tb, m, n, k, a, b, acc=1, c0=c0), ref + c0) <= 2e-5
        assert np.array_equal(got, run_tf32(ctx, ta, tb, m, n, k, a, b))
    finally:
        ctx.set_flags(0)


@pytest.mark.parametrize("rows,inf,outf", [(2048, 768, 2304), (300, 136, 264), (4096, 768, 768), (512, 16384, 768)])
def test_bf16_copy_of_the_result_from_the_product_epilogue(ctx, oracle_built, rows, inf, outf):
    """om_linear_fwd_bf16_b16 / om_linear_bwd_bf16_b16: the bfloat16 copy of y and of dx written by the product's epilogue
    equals the fp32 result rounded to nearest even, bit for bit (including the case where k is split and the copy is made
    from the finished result)."""
    K = oracle_built
    r = np.random.default_rng(rows + outf)
    x, w = r.standard_normal((rows, inf)).astype(np.float32), (r.standard_normal((outf, inf)) * 0.05).astype(np.float32)
    bias, g = r.standard_normal(outf).astype(np.float32), r.standard_normal((rows, outf)).astype(np.float32)
    X16, W16, G16, Bv, G = to_bf16(ctx, x), to_bf16(ctx, w), to_bf16(ctx, g), ctx.to_device(bias), ctx.to_device(g)
    Y, Y16 = ctx.empty((rows, outf)), ctx.empty((rows, outf), np.uint16)
    DX, DX16 = ctx.empty((rows, inf)), ctx.empty((rows, inf), np.uint16)
    ctx.call("om_linear_fwd_bf16_b16", ctx.handle, X16.ptr, W16.ptr, Bv.ptr, i32(rows), i32(inf), i32(outf), Y.ptr, Y16.ptr, i32(outf))
    ctx.call("om_linear_bwd_bf16_b16", ctx.handle, G16.ptr, G.ptr, i32(outf), X16.ptr, W16.ptr, i32(rows), i32(inf), i32(outf), DX.ptr, DX16.ptr,
             None, None, i32(0))
    ctx.sync()
    y, dx = Y.numpy(), DX.numpy()
    assert scaled_diff(y, K.gemm(x, w, tb=True, mode="bf16") + bias) <= 2e-5
    assert scaled_diff(dx, K.gemm(g, w, mode="bf16")) <= 2e-5
    assert np.array_equal(Y16.numpy(), (K.round_bf16(y).view(np.uint32) >> 16).astype(np.uint16))
    assert np.array_equal(DX16.numpy(), (K.round_bf16(dx).view(np.uint32) >> 16).astype(np.uint16))


ACT_SHAPES = [(4096, 768, 3072), (8192, 1024, 512), (300, 136, 264), (1000, 200, 520), (256, 64, 256)]


@pytest.mark.parametrize("op", [omb.UNARY["gelu_erf"], omb.UNARY["gelu_tanh"]])
@pytest.mark.parametrize("rows,inf,outf", ACT_SHAPES)
def test_activation_in_the_forward_epilogue_equals_the_separate_pass(ctx, rows, inf, outf, op):
    """om_linear_fwd_bf16_act against om_linear_fwd_bf16 followed by om_unary_b16: the same fp32 result before the
    activation and the same bfloat16 activation, bit for bit (one definition of the activation, no fused multiply-add)."""
    r = np.random.default_rng(rows + inf + op)
    x, w = r.standard_normal((rows, inf)).astype(np.float32), (r.standard_normal((outf, inf)) * 0.1).astype(np.float32)
    bias = r.standard_normal(outf).astype(np.float32)
    X16, W16, Bv = to_bf16(ctx, x), to_bf16(ctx, w), ctx.to_device(bias)
    assert ctx.lib.om_linear_act_bf16_supported(ctx.handle, i32(rows), i32(inf), i32(outf), i32(op), i32(0)) == 1
    Y, A16 = ctx.empty((rows, outf)), ctx.empty((rows, outf), np.uint16)
    ctx.call("om_linear_fwd_bf16_act", ctx.handle, X16.ptr, W16.ptr, Bv.ptr, i32(rows), i32(inf), i32(outf), i32(op), Y.ptr, A16.ptr, i32(outf))
    Y2, A2, A216 = ctx.empty((rows, outf)), ctx.empty((rows, outf)), ctx.empty((rows, outf), np.uint16)
    ctx.call("om_linear_fwd_bf16", ctx.handle, X16.ptr, W16.ptr, Bv.ptr, i32(rows), i32(inf), i32(outf), Y2.ptr, i32(outf))
    ctx.call("om_unary_b16", ctx.handle, i32(op), Y2.ptr, A2.ptr, A216.ptr, i64(rows * outf))
    ctx.sync()
    assert np.array_equal(Y.numpy(), Y2.numpy())
    assert np.array_equal(A16.numpy(), A216.numpy())
    assert np.any(A16.numpy() != 0)


@pytest.mark.parametrize("op", [omb.UNARY["gelu_erf"], omb.UNARY["gelu_tanh"]])
@pytest.mark.parametrize("rows,outf,inf", ACT_SHAPES)
def test_activation_derivative_in_the_input_gradient_epilogue_equals_the_separate_pass(ctx, rows, outf, inf, op):
    """om_linear_dgrad_bf16_act (dx = op'(pre) * (g W)) against om_linear_bwd_bf16_b16 followed by om_unary_bwd_b16: the same
    fp32 gradient and the same bfloat16 copy, bit for bit. (The layer has `inf` inputs, the width of the activation, and
    `outf` outputs.)"""
    r = np.random.default_rng(rows + inf + 7 * op)
    g, w = r.standard_normal((rows, outf)).astype(np.float32), (r.standard_normal((outf, inf)) * 0.1).astype(np.float32)
    pre = (r.standard_normal((rows, inf)) * 1.5).astype(np.float32)
    G16, W16, G, PRE = to_bf16(ctx, g), to_bf16(ctx, w), ctx.to_device(g), ctx.to_device(pre)
    X16 = ctx.empty((rows, inf), np.uint16)
    assert ctx.lib.om_linear_act_bf16_supported(ctx.handle, i32(rows), i32(inf), i32(outf), i32(op), i32(1)) == 1
    DX, DX16 = ctx.empty((rows, inf)), ctx.empty((rows, inf), np.uint16)
    ctx.call("om_linear_dgrad_bf16_act", ctx.handle, G16.ptr, i32(outf), W16.ptr, i32(rows), i32(inf), i32(outf), i32(op), PRE.ptr, i32(inf), DX.ptr, DX16.ptr)
    T, D2, D216 = ctx.empty((rows, inf)), ctx.empty((rows, inf)), ctx.empty((rows, inf), np.uint16)
    ctx.call("om_linear_bwd_bf16_b16", ctx.handle, G16.ptr, G.ptr, i32(outf), X16.ptr, W16.ptr, i32(rows), i32(inf), i32(outf), T.ptr, None, None, None, i32(0))
    ctx.call("om_unary_bwd_b16", ctx.handle, i32(op), T.ptr, PRE.ptr, D2.ptr, D216.ptr, i64(rows * inf))
    ctx.sync()
    assert np.array_equal(DX.numpy(), D2.numpy())
    assert np.array_equal(DX16.numpy(), D216.numpy())
    # without the bfloat16 copy
    DX3 = ctx.empty((rows, inf))
    ctx.call("om_linear_dgrad_bf16_act", ctx.handle, G16.ptr, i32(outf), W16.ptr, i32(rows), i32(inf), i32(outf), i32(op), PRE.ptr, i32(inf), DX3.ptr, None)
    ctx.sync()
    assert np.array_equal(DX3.numpy(), D2.numpy())


def test_shapes_that_cannot_take_the_activation_are_refused(ctx):
    sup = lambda rows, inf, outf, bwd: ctx.lib.om_linear_act_bf16_supported(ctx.handle, i32(rows), i32(inf), i32(outf), i32(omb.UNARY["gelu_erf"]), i32(bwd))
    assert sup(4096, 768, 128, 0) == 0          # fewer than 256 result columns
    assert sup(256, 4096, 256, 0) == 0          # one tile and 64 k-blocks: k is split, the activation would see partial sums
    assert sup(4096, 770, 3072, 0) == 0         # operand pitch not a multiple of 8
    assert ctx.lib.om_linear_act_bf16_supported(ctx.handle, i32(4096), i32(768), i32(3072), i32(omb.UNARY["relu"]), i32(0)) == 0
    x16, w16 = ctx.empty((256, 4096), np.uint16), ctx.empty((256, 4096), np.uint16)
    y, a16, b = ctx.empty((256, 256)), ctx.empty((256, 256), np.uint16), ctx.zeros((256,))
    with pytest.raises(omb.OmError):
        ctx.call("om_linear_fwd_bf16_act", ctx.handle, x16.ptr, w16.ptr, b.ptr, i32(256), i32(4096), i32(256), i32(omb.UNARY["gelu_erf"]), y.ptr, a16.ptr, i32(256))
    ctx.sync()


def one_stream_reference(ctx, xv, vals, up):
    """The fused feed-forward block with a residual sum, forward and backward, under bfloat16 products on one stream."""
    ctx.set_flags(omb.OM_TF32 | omb.OM_BF16_OPERANDS)
    x = omb.Tensor.from_numpy(xv, True)
    ps = [omb.Tensor.from_numpy(v, True) for v in vals]
    y = omb.call("add", [x, omb.call("feed_forward", [x] + ps, ints=[0])])
    y.backward(omb.Tensor.from_numpy(up))
    return [y.numpy(), x.grad.numpy()] + [p.grad.numpy() for p in ps]


@pytest.mark.parametrize("flags", [0, omb.OM_TF32 | omb.OM_BF16_OPERANDS, omb.OM_TF32 | omb.OM_BF16_OPERANDS | omb.OM_TWO_STREAMS])
def test_feed_forward_op_equals_its_three_parts(ctx, flags):
    """The host mirror's FeedForward (Linear -> Gelu -> Linear with the activation in the epilogues under bfloat16 products)
    against the composition of the three ops on the same flags: the result and the second layer's gradients bit for bit, the
    gradients behind the activation bit for bit under fp32 products and within the half rounding of the stored derivative
    under bfloat16 ones, with the input also feeding a residual sum so that its gradient arrives from two branches."""
    ctx.set_flags(flags)
    ctx.make_current()
    try:
        r = np.random.default_rng(3)
        rows, width, ff = 1024, 256, 1024
        xv = r.standard_normal((4, rows // 4, width)).astype(np.float32)
        vals = [(r.standard_normal((ff, width)) * 0.06).astype(np.float32), (r.standard_normal(ff) * 0.1).astype(np.float32),
                (r.standard_normal((width, ff)) * 0.03).astype(np.float32), (r.standard_normal(width) * 0.1).astype(np.float32)]
        up = r.standard_normal(xv.shape).astype(np.float32)
        results = []
        for fused in (True, False):
            x = omb.Tensor.from_numpy(xv, True)
            ps = [omb.Tensor.from_numpy(v, True) for v in vals]
            if fused:
                f = omb.call("feed_forward", [x] + ps, ints=[0])
            else:
                f = omb.call("linear", [omb.call("gelu", [omb.call("linear", [x, ps[0], ps[1]])], ints=[0]), ps[2], ps[3]])
            y = omb.call("add", [x, f])
            y.backward(omb.Tensor.from_numpy(up))
            results.append([y.numpy(), x.grad.numpy()] + [p.grad.numpy() for p in ps])
        if flags & omb.OM_TWO_STREAMS:
            # the bias sums ran on the context's second stream beside the products: the same bits as on one stream
            again = one_stream_reference(ctx, xv, vals, up)
            for a, b in zip(results[0], again):
                assert np.array_equal(a, b)
        names = ["y", "dx", "dw1", "db1", "dw2", "db2"]     # the bias gradients too: both read the bfloat16 gradient
        for name, a, b in zip(names, *results):
            assert np.all(np.isfinite(a)), name
            if flags and name in ("dx", "dw1", "db1"):
                # behind the activation's derivative, which the fused forward pass keeps as IEEE half (relative 2^-12): a
                # fraction of the bfloat16 roundings of the gradient in front of the activation fall the other way
                assert np.max(np.abs(a - b)) <= 2e-3 * np.max(np.abs(b)), (name, float(np.max(np.abs(a - b))), float(np.max(np.abs(b))))
            else:
                assert np.array_equal(a, b), (name, float(np.max(np.abs(a - b))), float(np.max(np.abs(b))))
    finally:
        ctx.set_flags(0)


def test_short_erf_of_the_bf16_tier_is_within_1e_6(ctx, oracle_built):
    """With a bfloat16 copy requested the erf GELU and its derivative use the short branch-free erf (rational form, hardware
    exp and reciprocal): within 1e-6 absolute of the oracle's libm values over a dense grid, including the far tails, zero,
    and values around the sign change; the bfloat16 copy is the fp32 value rounded."""
    K = oracle_built
    x = np.concatenate([np.linspace(-9, 9, 400001), np.array([0.0, -0.0, 1e-30, -1e-30, 1e-8, 40.0, -40.0])]).astype(np.float32)
    g = np.ones_like(x)
    n = x.size
    X, G = ctx.to_device(x), ctx.to_device(g)
    Y, Y16, D, D16 = ctx.empty((n,)), ctx.empty((n,), np.uint16), ctx.empty((n,)), ctx.empty((n,), np.uint16)
    op = omb.UNARY["gelu_erf"]
    ctx.call("om_unary_b16", ctx.handle, i32(op), X.ptr, Y.ptr, Y16.ptr, i64(n))
    ctx.call("om_unary_bwd_b16", ctx.handle, i32(op), G.ptr, X.ptr, D.ptr, D16.ptr, i64(n))
    ctx.sync()
    y, d = Y.numpy(), D.numpy()
    assert np.max(np.abs(y - K.unary("gelu_erf", x))) <= 1e-6
    assert np.max(np.abs(d - K.unary_bwd("gelu_erf", g, x))) <= 1e-6
    assert np.array_equal(Y16.numpy(), (K.round_bf16(y).view(np.uint32) >> 16).astype(np.uint16))
    assert np.array_equal(D16.numpy(), (K.round_bf16(d).view(np.uint32) >> 16).astype(np.uint16))


@pytest.mark.parametrize("rows,outf,inf", [(8192, 2304, 768), (8192, 3072, 768), (300, 136, 264), (1000, 200, 520)])
def test_input_gradient_added_to_a_residual_out_of_place(ctx, rows, outf, inf):
    """om_linear_dgrad_bf16_add (dx = residual + g W, the sum formed in the epilogue from a plain read of the residual) against
    om_linear_bwd_bf16_b16 adding into a copy of the residual in place (accumulate bit 2): the same bits, the residual
    untouched, the bfloat16 copy the sum rounded."""
    r = np.random.default_rng(rows + inf)
    g, w = r.standard_normal((rows, outf)).astype(np.float32), (r.standard_normal((outf, inf)) * 0.1).astype(np.float32)
    res = r.standard_normal((rows, inf)).astype(np.float32)
    G16, W16, G, RES = to_bf16(ctx, g), to_bf16(ctx, w), ctx.to_device(g), ctx.to_device(res)
    X16 = ctx.empty((rows, inf), np.uint16)
    assert ctx.lib.om_linear_dgrad_bf16_add_supported(ctx.handle, i32(rows), i32(inf), i32(outf)) == 1
    DX, DX16 = ctx.empty((rows, inf)), ctx.empty((rows, inf), np.uint16)
    ctx.call("om_linear_dgrad_bf16_add", ctx.handle, G16.ptr, i32(outf), W16.ptr, i32(rows), i32(inf), i32(outf), RES.ptr, i32(inf), DX.ptr, DX16.ptr)
    ACC = ctx.to_device(res)
    ctx.call("om_linear_bwd_bf16_b16", ctx.handle, G16.ptr, G.ptr, i32(outf), X16.ptr, W16.ptr, i32(rows), i32(inf), i32(outf), ACC.ptr, None, None, None, i32(2))
    ctx.sync()
    assert np.array_equal(DX.numpy(), ACC.numpy())
    assert np.array_equal(RES.numpy(), res)
    from oracle import oracle as K
    K.build()
    assert np.array_equal(DX16.numpy(), (K.round_bf16(DX.numpy()).view(np.uint32) >> 16).astype(np.uint16))


@pytest.mark.parametrize("rows,cols,ld", [(16384, 768, 768), (1000, 520, 528), (513, 70, 72), (1, 8, 8), (4096, 3072, 3072)])
def test_column_sums_of_a_bf16_matrix(ctx, oracle_built, rows, cols, ld):
    """om_colsum_bf16 against the oracle's restatement of its order (16 rows per lane in fp32, lanes and chunks of 512 rows in
    double): the same bits, and within fp32 rounding of the plain double sum; with accumulation into the destination, the pitch
    columns ignored, and the same bits from run to run."""
    K = oracle_built
    r = np.random.default_rng(rows + cols)
    g = np.zeros((rows, ld), np.float32)
    g[:, :cols] = r.standard_normal((rows, cols))
    g[:, cols:] = 1e6                                     # pitch columns must not be read into the sums
    G16 = to_bf16(ctx, g)
    want = K.colsum_bf16(g[:, :cols])
    plain = K.round_bf16(g[:, :cols]).astype(np.float64).sum(0)
    assert np.max(np.abs(want - plain)) <= 4e-6 * np.sqrt(rows) + 1e-6 * np.max(np.abs(plain))
    before = r.standard_normal(cols).astype(np.float32)
    OUT, ACC = ctx.empty((cols,)), ctx.to_device(before)
    ctx.call("om_colsum_bf16", ctx.handle, G16.ptr, i32(rows), i32(cols), i32(ld), OUT.ptr, i32(0))
    ctx.call("om_colsum_bf16", ctx.handle, G16.ptr, i32(rows), i32(cols), i32(ld), ACC.ptr, i32(1))
    ctx.sync()
    assert np.array_equal(OUT.numpy(), want)
    assert np.array_equal(ACC.numpy(), before + want)
    again = ctx.empty((cols,))
    ctx.call("om_colsum_bf16", ctx.handle, G16.ptr, i32(rows), i32(cols), i32(ld), again.ptr, i32(0))
    ctx.sync()
    assert np.array_equal(again.numpy(), OUT.numpy())


def test_linear_gradients_from_the_bf16_gradient_alone(ctx, oracle_built):
    """om_linear_bwd_bf16_b16 without the fp32 gradient (g NULL): the bias gradient is the column sum of the bfloat16 copy;
    om_linear_dgrad_bf16_act without the fp32 result (dx NULL): the bfloat16 result alone equals the one written beside an
    fp32 result."""
    K = oracle_built
    r = np.random.default_rng(17)
    rows, inf, outf = 4096, 768, 3072
    g = r.standard_normal((rows, outf)).astype(np.float32)
    x, w = r.standard_normal((rows, inf)).astype(np.float32), (r.standard_normal((outf, inf)) * 0.05).astype(np.float32)
    G16, X16, W16 = to_bf16(ctx, g), to_bf16(ctx, x), to_bf16(ctx, w)
    DB = ctx.empty((outf,))
    ctx.call("om_linear_bwd_bf16_b16", ctx.handle, G16.ptr, None, i32(outf), X16.ptr, W16.ptr, i32(rows), i32(inf), i32(outf), None, None, None, DB.ptr, i32(0))
    ctx.sync()
    assert np.array_equal(DB.numpy(), K.colsum_bf16(g))
    # the activation's derivative into a bfloat16-only result: the layer has `outf` inputs here (the width of the activation)
    op = omb.UNARY["gelu_erf"]
    g2 = r.standard_normal((rows, inf)).astype(np.float32)
    w2 = (r.standard_normal((inf, outf)) * 0.05).astype(np.float32)
    pre = (r.standard_normal((rows, outf)) * 1.5).astype(np.float32)
    G216, W216, PRE = to_bf16(ctx, g2), to_bf16(ctx, w2), ctx.to_device(pre)
    DX, DX16, ONLY16 = ctx.empty((rows, outf)), ctx.empty((rows, outf), np.uint16), ctx.empty((rows, outf), np.uint16)
    ctx.call("om_linear_dgrad_bf16_act", ctx.handle, G216.ptr, i32(inf), W216.ptr, i32(rows), i32(outf), i32(inf), i32(op), PRE.ptr, i32(outf), DX.ptr, DX16.ptr)
    ctx.call("om_linear_dgrad_bf16_act", ctx.handle, G216.ptr, i32(inf), W216.ptr, i32(rows), i32(outf), i32(inf), i32(op), PRE.ptr, i32(outf), None, ONLY16.ptr)
    ctx.sync()
    assert np.array_equal(ONLY16.numpy(), DX16.numpy())
    assert np.any(ONLY16.numpy() != 0)


@pytest.mark.parametrize("op", [omb.UNARY["gelu_erf"], omb.UNARY["gelu_tanh"]])
@pytest.mark.parametrize("rows,inf,outf", [(4096, 768, 3072), (300, 136, 264)])
def test_derivative_left_behind_by_the_forward_epilogue(ctx, oracle_built, rows, inf, outf, op):
    """om_linear_fwd_bf16_actd / om_linear_dgrad_bf16_mul against om_linear_fwd_bf16_act / om_linear_dgrad_bf16_act: the same
    bfloat16 activation; the derivative equals op' applied to the separately computed result, rounded to IEEE half; the input
    gradient is the plain product (factor one) times that half value in one fp32 multiplication, which stays within the half
    rounding of the gradient that evaluates the derivative in its own epilogue."""
    K = oracle_built
    r = np.random.default_rng(rows + inf + 3 * op)
    x, w = r.standard_normal((rows, inf)).astype(np.float32), (r.standard_normal((outf, inf)) * 0.1).astype(np.float32)
    bias = r.standard_normal(outf).astype(np.float32)
    X16, W16, Bv = to_bf16(ctx, x), to_bf16(ctx, w), ctx.to_device(bias)
    PRE, A16, D, A16D = ctx.empty((rows, outf)), ctx.empty((rows, outf), np.uint16), ctx.empty((rows, outf), np.uint16), ctx.empty((rows, outf), np.uint16)
    ctx.call("om_linear_fwd_bf16_act", ctx.handle, X16.ptr, W16.ptr, Bv.ptr, i32(rows), i32(inf), i32(outf), i32(op), PRE.ptr, A16.ptr, i32(outf))
    ctx.call("om_linear_fwd_bf16_actd", ctx.handle, X16.ptr, W16.ptr, Bv.ptr, i32(rows), i32(inf), i32(outf), i32(op), D.ptr, A16D.ptr, i32(outf))
    ONES, REF, REF16 = ctx.to_device(np.ones((rows, outf), np.float32)), ctx.empty((rows, outf)), ctx.empty((rows, outf), np.uint16)
    ctx.call("om_unary_bwd_b16", ctx.handle, i32(op), ONES.ptr, PRE.ptr, REF.ptr, REF16.ptr, i64(rows * outf))
    ctx.sync()
    assert np.array_equal(A16D.numpy(), A16.numpy())
    assert np.array_equal(D.numpy(), REF.numpy().astype(np.float16).view(np.uint16))      # numpy rounds to nearest even too
    # backward through the activation: the layer after it has `outf` inputs and `inf` outputs
    g, w2 = r.standard_normal((rows, inf)).astype(np.float32), (r.standard_normal((inf, outf)) * 0.1).astype(np.float32)
    G16, W216 = to_bf16(ctx, g), to_bf16(ctx, w2)
    DX, DX16, M, M16 = ctx.empty((rows, outf)), ctx.empty((rows, outf), np.uint16), ctx.empty((rows, outf)), ctx.empty((rows, outf), np.uint16)
    ctx.call("om_linear_dgrad_bf16_act", ctx.handle, G16.ptr, i32(inf), W216.ptr, i32(rows), i32(outf), i32(inf), i32(op), PRE.ptr, i32(outf), DX.ptr, DX16.ptr)
    ctx.call("om_linear_dgrad_bf16_mul", ctx.handle, G16.ptr, i32(inf), W216.ptr, i32(rows), i32(outf), i32(inf), D.ptr, i32(outf), M.ptr, M16.ptr)
    ONLY16, RAW = ctx.empty((rows, outf), np.uint16), ctx.empty((rows, outf))
    ctx.call("om_linear_dgrad_bf16_mul", ctx.handle, G16.ptr, i32(inf), W216.ptr, i32(rows), i32(outf), i32(inf), D.ptr, i32(outf), None, ONLY16.ptr)
    HALF_ONES = ctx.to_device(np.full((rows, outf), 0x3C00, np.uint16))
    ctx.call("om_linear_dgrad_bf16_mul", ctx.handle, G16.ptr, i32(inf), W216.ptr, i32(rows), i32(outf), i32(inf), HALF_ONES.ptr, i32(outf), RAW.ptr, None)
    ctx.sync()
    want = RAW.numpy() * D.numpy().view(np.float16).astype(np.float32)
    assert np.array_equal(M.numpy(), want)
    assert np.array_equal(M16.numpy(), (K.round_bf16(want).view(np.uint32) >> 16).astype(np.uint16))
    assert np.array_equal(ONLY16.numpy(), M16.numpy())
    assert np.all(np.abs(M.numpy() - DX.numpy()) <= 5e-4 * np.abs(DX.numpy()) + 1e-7 * np.abs(RAW.numpy()))
    assert np.any(M.numpy() != 0)


def test_forward_product_with_the_bf16_result_alone(ctx):
    """om_linear_fwd_bf16_b16 without the fp32 result (y NULL): the bfloat16 result equals the copy written beside an fp32 one."""
    r = np.random.default_rng(23)
    rows, inf, outf = 4096, 768, 2304
    x, w = r.standard_normal((rows, inf)).astype(np.float32), (r.standard_normal((outf, inf)) * 0.05).astype(np.float32)
    bias = r.standard_normal(outf).astype(np.float32)
    X16, W16, Bv = to_bf16(ctx, x), to_bf16(ctx, w), ctx.to_device(bias)
    Y, Y16, ONLY = ctx.empty((rows, outf)), ctx.empty((rows, outf), np.uint16), ctx.empty((rows, outf), np.uint16)
    ctx.call("om_linear_fwd_bf16_b16", ctx.handle, X16.ptr, W16.ptr, Bv.ptr, i32(rows), i32(inf), i32(outf), Y.ptr, Y16.ptr, i32(outf))
    ctx.call("om_linear_fwd_bf16_b16", ctx.handle, X16.ptr, W16.ptr, Bv.ptr, i32(rows), i32(inf), i32(outf), None, ONLY.ptr, i32(outf))
    ctx.sync()
    assert np.array_equal(ONLY.numpy(), Y16.numpy()) and np.any(ONLY.numpy() != 0)


@pytest.mark.parametrize("rows,inf,outf", [(16384, 768, 3072), (4096, 768, 2304), (16384, 3072, 768), (1000, 264, 520), (700, 768, 768), (16896, 768, 768)])
def test_bias_and_weight_gradient_in_one_call(ctx, oracle_built, rows, inf, outf):
    """om_linear_bwd_bf16_b16 asked for dW and dbias at once (no fp32 gradient): the bias gradient has the bits of the oracle's
    restatement of the column sum's order, with and without accumulation, and the weight gradient the bits of a call that
    asks for it alone (two-slice and eight-slice shapes, ragged rows, more than 32 chunks of rows)."""
    K = oracle_built
    r = np.random.default_rng(rows + outf)
    g = r.standard_normal((rows, outf)).astype(np.float32)
    x = r.standard_normal((rows, inf)).astype(np.float32)
    w = (r.standard_normal((outf, inf)) * 0.05).astype(np.float32)
    G16, X16, W16 = to_bf16(ctx, g), to_bf16(ctx, x), to_bf16(ctx, w)
    before = r.standard_normal(outf).astype(np.float32)
    DW, DB, DW_ALONE, DB_ACC = ctx.empty((outf, inf)), ctx.empty((outf,)), ctx.empty((outf, inf)), ctx.to_device(before)
    DW_ACC = ctx.zeros((outf, inf))
    args = (G16.ptr, None, i32(outf), X16.ptr, W16.ptr, i32(rows), i32(inf), i32(outf), None, None)
    ctx.call("om_linear_bwd_bf16_b16", ctx.handle, *args, DW.ptr, DB.ptr, i32(0))
    ctx.call("om_linear_bwd_bf16_b16", ctx.handle, *args, DW_ALONE.ptr, None, i32(0))
    ctx.call("om_linear_bwd_bf16_b16", ctx.handle, *args, DW_ACC.ptr, DB_ACC.ptr, i32(1))
    ctx.sync()
    want = K.colsum_bf16(g)
    assert np.array_equal(DB.numpy(), want)
    assert np.array_equal(DB_ACC.numpy(), before + want)
    assert np.array_equal(DW.numpy(), DW_ALONE.numpy()) and np.any(DW.numpy() != 0)
    assert np.array_equal(DW_ACC.numpy(), DW.numpy())
