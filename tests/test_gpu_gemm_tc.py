"""The tensor-pipe matrix product (tcgen05 / TMEM / TMA, TF32 operands, fp32 accumulation) against the CPU oracle.

Two comparisons per case: against the oracle fed the same TF32-rounded operands (round to nearest even, as the TMA
loads round them; isolates the kernel: only the fp32 accumulation order differs, scaled error <= 2e-5), and against
the plain fp32 oracle at the contract's TF32 tier: every element within the rigorous 2^-9 * (|A||B|) bound and the
scaled error inside 1e-3."""
import numpy as np
import pytest

import om_binding as omb
from backends import scaled_diff
from om_binding import f32, i32, i64

pytestmark = pytest.mark.gpu

SHAPES = [
    (128, 128, 32), (128, 128, 256), (256, 384, 384), (8192, 384, 384), (384, 384, 8192), (1536, 384, 8192),
    (1229, 1000, 384), (130, 260, 100), (128, 12, 784), (64, 512, 512), (100, 36, 4096),
]


def run(ctx, ta, tb, m, n, k, a, b, acc=0, c0=None):
    da, db = ctx.to_device(a), ctx.to_device(b)
    dc = ctx.to_device(c0) if c0 is not None else ctx.empty((m, n))
    ctx.call("om_matmul", ctx.handle, i32(ta), i32(tb), i32(m), i32(n), i32(k), da.ptr, i32(a.shape[1]), db.ptr,
             i32(b.shape[1]), dc.ptr, i32(n), i32(acc))
    ctx.sync()
    return dc.numpy()


@pytest.mark.parametrize("ta,tb", [(0, 1), (0, 0), (1, 0), (1, 1)])
@pytest.mark.parametrize("m,n,k", SHAPES)
def test_tf32_matmul(ctx, oracle_built, ta, tb, m, n, k):
    K = oracle_built
    ctx.set_flags(omb.OM_TF32)
    try:
        r = np.random.default_rng(m + 3 * n + 7 * k + ta * 2 + tb)
        a = r.standard_normal((k, m) if ta else (m, k)).astype(np.float32)
        b = r.standard_normal((n, k) if tb else (k, n)).astype(np.float32)
        got = run(ctx, ta, tb, m, n, k, a, b)
        if a.shape[1] % 4 or b.shape[1] % 4:
            # a row pitch that is not a multiple of 16 bytes cannot be described to TMA: fp32 FMA kernel, bit-exact
            assert np.array_equal(got, K.gemm(a, b, bool(ta), bool(tb)))
            return
        ref_tf32 = K.gemm(a, b, bool(ta), bool(tb), mode="tf32")
        ref = K.gemm(a, b, bool(ta), bool(tb))
        assert scaled_diff(got, ref_tf32) <= 2e-5
        # TF32 keeps 10 mantissa bits of each operand: every product is within 2^-9 relative, so every element is within
        # 2^-9 * (|A| |B|) of the fp32 result (the k*u*sum|ab| form of bound the reference's GEMM tests use,
        # docs/kernels-gemm.md:82-84), and the scaled error stays inside the 1e-3 tier.
        aa = np.abs(a.T if ta else a).astype(np.float64)
        bb = np.abs(b.T if tb else b).astype(np.float64)
        assert np.all(np.abs(got.astype(np.float64) - ref) <= 2.0 ** -9 * (aa @ bb) + 1e-5)
        assert scaled_diff(got, ref) <= 1e-3
        # accumulate: C += A B
        c0 = r.standard_normal((m, n)).astype(np.float32)
        got2 = run(ctx, ta, tb, m, n, k, a, b, acc=1, c0=c0)
        assert scaled_diff(got2, ref_tf32 + c0) <= 2e-5
        # run-to-run determinism (fixed split of k, ordered combine, no atomics)
        assert np.array_equal(got, run(ctx, ta, tb, m, n, k, a, b))
    finally:
        ctx.set_flags(0)


def test_tf32_linear_with_bias_and_backward(ctx, oracle_built):
    K = oracle_built
    ctx.set_flags(omb.OM_TF32)
    try:
        r = np.random.default_rng(1)
        rows, inf, outf = 1024, 384, 1536
        x, w = r.standard_normal((rows, inf)).astype(np.float32), (r.standard_normal((outf, inf)) * 0.05).astype(np.float32)
        b, g = r.standard_normal(outf).astype(np.float32), r.standard_normal((rows, outf)).astype(np.float32)
        X, W, Bv, G = ctx.to_device(x), ctx.to_device(w), ctx.to_device(b), ctx.to_device(g)
        Y, DX, DW, DB = ctx.empty((rows, outf)), ctx.empty((rows, inf)), ctx.empty((outf, inf)), ctx.empty((outf,))
        ctx.call("om_linear_fwd", ctx.handle, X.ptr, W.ptr, Bv.ptr, i32(rows), i32(inf), i32(outf), Y.ptr)
        ctx.call("om_linear_bwd", ctx.handle, G.ptr, X.ptr, W.ptr, i32(rows), i32(inf), i32(outf), DX.ptr, DW.ptr, DB.ptr, i32(0))
        ctx.sync()
        assert scaled_diff(Y.numpy(), K.gemm(x, w, tb=True, mode="tf32") + b) <= 2e-5
        assert scaled_diff(DX.numpy(), K.gemm(g, w, mode="tf32")) <= 2e-5
        assert scaled_diff(DW.numpy(), K.gemm(g, x, ta=True, mode="tf32")) <= 2e-5
        assert scaled_diff(Y.numpy(), K.gemm(x, w, tb=True) + b) <= 1e-3
        assert scaled_diff(DW.numpy(), K.gemm(g, x, ta=True)) <= 1e-3
    finally:
        ctx.set_flags(0)


def test_unaligned_operands_use_the_fp32_kernel(ctx, oracle_built):
    """Leading dimensions that are not a multiple of four elements cannot be described to TMA: such products run on
    the fp32 FMA kernel and are bit-exact."""
    K = oracle_built
    ctx.set_flags(omb.OM_TF32)
    try:
        r = np.random.default_rng(2)
        a, b = r.standard_normal((64, 91)).astype(np.float32), r.standard_normal((91, 53)).astype(np.float32)
        assert np.array_equal(run(ctx, 0, 0, 64, 53, 91, a, b), K.gemm(a, b))
    finally:
        ctx.set_flags(0)


@pytest.mark.parametrize("ta,tb,m,n,k,batch", [(0, 1, 128, 128, 32, 24), (0, 0, 128, 32, 128, 24), (1, 0, 128, 32, 128, 24),
                                               (0, 1, 200, 72, 40, 5), (1, 1, 96, 160, 64, 3), (0, 0, 64, 64, 512, 7)])
def test_tf32_strided_batch(ctx, oracle_built, ta, tb, m, n, k, batch):
    """One launch over a strided batch (rank-3 tensor maps): every slice equals the single product of that slice."""
    K = oracle_built
    ctx.set_flags(omb.OM_TF32)
    try:
        r = np.random.default_rng(m + n + k + batch)
        a = r.standard_normal((batch,) + ((k, m) if ta else (m, k))).astype(np.float32)
        b = r.standard_normal((batch,) + ((n, k) if tb else (k, n))).astype(np.float32)
        da, db, dc = ctx.to_device(a), ctx.to_device(b), ctx.empty((batch, m, n))
        ctx.call("om_matmul_batched", ctx.handle, i32(ta), i32(tb), i32(m), i32(n), i32(k), da.ptr, i32(a.shape[2]),
                 i64(a.shape[1] * a.shape[2]), db.ptr, i32(b.shape[2]), i64(b.shape[1] * b.shape[2]), dc.ptr, i32(n),
                 i64(m * n), i32(batch), i32(0))
        ctx.sync()
        got = dc.numpy()
        for z in range(batch):
            assert scaled_diff(got[z], K.gemm(a[z], b[z], bool(ta), bool(tb), mode="tf32")) <= 2e-5, z
            single = run(ctx, ta, tb, m, n, k, a[z], b[z])
            # A single product of a small shape splits k over several CTAs, the batched launch never does: the same
            # rounded operands summed in another order.
            assert np.array_equal(got[z], single) if k < 512 else scaled_diff(got[z], single) <= 2e-5, z
    finally:
        ctx.set_flags(0)


@pytest.mark.parametrize("b,h,lq,lk,d,masked", [(3, 4, 128, 128, 32, 0), (2, 2, 64, 192, 64, 1), (2, 3, 100, 100, 32, 0), (2, 2, 128, 128, 32, 1),
                                                (1, 3, 60, 128, 64, 0), (2, 1, 128, 37, 64, 1), (1, 1, 5, 7, 32, 0),
                                                # several tiles: the two-pass forward kernel (the backward takes the general path)
                                                (2, 3, 256, 256, 64, 0), (1, 2, 512, 512, 64, 1), (2, 2, 300, 200, 32, 1),
                                                (1, 2, 129, 128, 64, 0), (1, 1, 128, 130, 32, 0), (1, 2, 64, 640, 32, 0),
                                                # a quarter of one BERT-base-shape layer: 384 CTAs, the case the ncu summary of these kernels uses
                                                (8, 12, 512, 512, 64, 0)])
def test_tf32_attention(ctx, oracle_built, b, h, lq, lk, d, masked):
    """Attention forward and backward with the head products on the tensor pipe, at the TF32 tier of the contract."""
    K = oracle_built
    ctx.set_flags(omb.OM_TF32)
    try:
        r = np.random.default_rng(b * 7 + lq)
        q, k, v, g = (r.standard_normal(s).astype(np.float32) for s in [(b, h, lq, d), (b, h, lk, d), (b, h, lk, d), (b, h, lq, d)])
        mask = np.where(r.random((lq, lk)) < 0.25, -4.0, 0.0).astype(np.float32) if masked else None
        scale = np.float32(1.0 / np.sqrt(np.float32(d)))
        Q, Kk, V, G = ctx.to_device(q), ctx.to_device(k), ctx.to_device(v), ctx.to_device(g)
        M = ctx.to_device(mask) if mask is not None else None
        O, DQ, DK, DV, LSE = ctx.empty(q.shape), ctx.empty(q.shape), ctx.empty(k.shape), ctx.empty(v.shape), ctx.empty((b, h, lq))
        ctx.call("om_attention_fwd", ctx.handle, Q.ptr, Kk.ptr, V.ptr, M.ptr if M else None, i64(0), i32(b), i32(h), i32(lq),
                 i32(lk), i32(d), f32(scale), O.ptr, LSE.ptr)
        # With the forward's row log-sum-exp the one-tile shapes (L <= 128, D = 32) take the fused backward kernel.
        ctx.call("om_attention_bwd", ctx.handle, G.ptr, Q.ptr, Kk.ptr, V.ptr, M.ptr if M else None, i64(0), LSE.ptr, i32(b),
                 i32(h), i32(lq), i32(lk), i32(d), f32(scale), DQ.ptr, DK.ptr, DV.ptr)
        ctx.sync()
        # Two (forward) to three (backward) TF32 products in a chain, each rounding its operands to 11 bits: the scaled error
        # of the chain sits around 1e-3, so the bound here is 2e-3 where a single product is held to 1e-3.
        assert scaled_diff(O.numpy(), K.attention_fwd(q, k, v, mask)) <= 2e-3
        dq, dk, dv = K.attention_bwd(g, q, k, v, mask)
        assert scaled_diff(DQ.numpy(), dq) <= 2e-3 and scaled_diff(DK.numpy(), dk) <= 2e-3 and scaled_diff(DV.numpy(), dv) <= 2e-3
    finally:
        ctx.set_flags(0)


PAIR_SHAPES = [(256, 256, 64), (8192, 384, 384), (8192, 1152, 384), (1229, 30524, 384), (512, 192, 96), (384, 1536, 8192), (1000, 400, 200),
               (300, 260, 132)]


@pytest.mark.parametrize("ta,tb", [(0, 1), (0, 0), (1, 0), (1, 1)])
@pytest.mark.parametrize("m,n,k", PAIR_SHAPES)
def test_tf32_matmul_on_cta_pairs(ctx, oracle_built, ta, tb, m, n, k):
    """The CTA-pair kernel (tcgen05 cta_group::2: each CTA loads half of the B tile) against the oracle on TF32-rounded
    operands and against the one-CTA kernel: the same rounded operands and the same k order, so (without a split of k) the
    same bits."""
    K = oracle_built
    r = np.random.default_rng(m * 3 + n + k)
    a = r.standard_normal((k, m) if ta else (m, k)).astype(np.float32)
    b = r.standard_normal((n, k) if tb else (k, n)).astype(np.float32)
    if a.shape[1] % 4 or b.shape[1] % 4:
        pytest.skip("operand pitch not a multiple of 16 bytes: this shape runs on the fp32 kernel")
    try:
        ctx.set_flags(omb.OM_TF32 | omb.OM_PAIR_TILES)
        got = run(ctx, ta, tb, m, n, k, a, b)
        assert scaled_diff(got, K.gemm(a, b, bool(ta), bool(tb), mode="tf32")) <= 2e-5
        c0 = r.standard_normal((m, n)).astype(np.float32)
        got2 = run(ctx, ta, tb, m, n, k, a, b, acc=1, c0=c0)
        assert scaled_diff(got2, K.gemm(a, b, bool(ta), bool(tb), mode="tf32") + c0) <= 2e-5
        ctx.set_flags(omb.OM_TF32)
        single = run(ctx, ta, tb, m, n, k, a, b)
        assert scaled_diff(got, single) <= 2e-5
    finally:
        ctx.set_flags(0)


@pytest.mark.parametrize("rows,inf,outf", [(8192, 384, 1536), (2048, 1536, 384), (1229, 384, 30524), (700, 100, 60)])
def test_linear_backward_on_two_streams_gives_the_same_bits(ctx, rows, inf, outf):
    """OM_TWO_STREAMS: the input gradient and the weight/bias gradients of om_linear_bwd run on two streams of the
    context; every kernel is the same and writes its own outputs, so the results equal the one-stream call bit for bit,
    call after call (the auxiliary stream takes its scratch from its own pool)."""
    r = np.random.default_rng(rows + outf)
    g, x, w = (r.standard_normal(s).astype(np.float32) for s in [(rows, outf), (rows, inf), (outf, inf)])
    G, X, W = ctx.to_device(g), ctx.to_device(x), ctx.to_device(w)

    def run_once(flags):
        ctx.set_flags(flags)
        DX, DW, DB = ctx.empty((rows, inf)), ctx.empty((outf, inf)), ctx.empty((outf,))
        for _ in range(3):
            ctx.call("om_linear_bwd", ctx.handle, G.ptr, X.ptr, W.ptr, i32(rows), i32(inf), i32(outf), DX.ptr, DW.ptr, DB.ptr, i32(0))
        ctx.sync()
        return DX.numpy(), DW.numpy(), DB.numpy()

    try:
        one = run_once(omb.OM_TF32)
        two = run_once(omb.OM_TF32 | omb.OM_TWO_STREAMS)
        for a, b in zip(one, two):
            assert a.tobytes() == b.tobytes()
    finally:
        ctx.set_flags(0)


def test_deep_product_with_an_unaligned_pitch_is_sliced_in_the_fast_tier(ctx, oracle_built):
    """The weight gradient of a 97-class output layer: g^T [97, 4096] x [4096, 512] with g stored [4096, 97]. A pitch of 97
    floats cannot be described to TMA, so the product runs on the fp32 FMA kernel: in the exact tier with the reference's
    one-accumulator order (bit-exact), in the fast tier cut into equal k slices added in slice order (fp32 throughout,
    another order: 1e-5, and the same bits from run to run)."""
    K = oracle_built
    r = np.random.default_rng(97)
    m, n, k = 97, 512, 4096
    a = r.standard_normal((k, m)).astype(np.float32)
    b = r.standard_normal((k, n)).astype(np.float32)
    ref = K.gemm(a, b, True, False)
    try:
        ctx.set_flags(0)
        assert np.array_equal(run(ctx, 1, 0, m, n, k, a, b), ref)
        ctx.set_flags(omb.OM_TF32)
        got = run(ctx, 1, 0, m, n, k, a, b)
        assert scaled_diff(got, ref) <= 1e-5
        assert np.array_equal(got, run(ctx, 1, 0, m, n, k, a, b))
        c0 = r.standard_normal((m, n)).astype(np.float32)
        assert scaled_diff(run(ctx, 1, 0, m, n, k, a, b, acc=1, c0=c0), ref + c0) <= 1e-5
    finally:
        ctx.set_flags(0)
