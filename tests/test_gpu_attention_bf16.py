"""The several-tile attention forward (om_attention_fwd_bf16) and the fused backward (om_attention_bwd_bf16) with bfloat16 product operands against the CPU
oracle: against the oracle's model of the same tier (the operands of the five products rounded to bfloat16, everything
else fp32: what is left is the summation order, the TF32 forward that supplies the log-sum-exp, and values that round the
other way at a bfloat16 boundary) and against the plain fp32 AttentionBackward, where the bfloat16 rounding of the
operands shows (8 significant bits)."""
import ctypes as C

import numpy as np
import pytest

import om_binding as omb
from backends import scaled_diff
from om_binding import f32, i32, i64

pytestmark = pytest.mark.gpu


class HeadStrides(C.Structure):
    _fields_ = [("batch", C.c_int64), ("head", C.c_int64), ("row", C.c_int64)]


def to_bf16(ctx, a):
    src = ctx.to_device(np.ascontiguousarray(a, np.float32))
    dst = ctx.empty(a.shape, np.uint16)
    ctx.call("om_cast_bf16", ctx.handle, src.ptr, dst.ptr, i64(a.size))
    return dst


def bf16_bits(K, a):
    return (K.round_bf16(a).view(np.uint32) >> 16).astype(np.uint16)


@pytest.mark.parametrize("b,h,lq,lk,masked", [(1, 2, 512, 512, 0), (2, 3, 256, 256, 1), (1, 2, 300, 200, 0), (1, 1, 129, 640, 1), (1, 2, 512, 128, 0),
                                              (1, 1, 5, 7, 0), (2, 12, 512, 512, 0), (1, 2, 1100, 384, 1), (3, 1, 128, 128, 0)])
def test_fused_attention_backward_with_bf16_operands(ctx, oracle_built, b, h, lq, lk, masked):
    K = oracle_built
    d = 64
    ctx.set_flags(omb.OM_TF32 | omb.OM_BF16_OPERANDS)
    try:
        r = np.random.default_rng(b * 7 + lq + lk)
        q, k, v, g = (r.standard_normal(s).astype(np.float32) for s in [(b, h, lq, d), (b, h, lk, d), (b, h, lk, d), (b, h, lq, d)])
        mask = np.where(r.random((lq, lk)) < 0.25, -4.0, 0.0).astype(np.float32) if masked else None
        scale = np.float32(1.0 / np.sqrt(np.float32(d)))
        Q, Kk, V, G = ctx.to_device(q), ctx.to_device(k), ctx.to_device(v), ctx.to_device(g)
        M = ctx.to_device(mask) if mask is not None else None
        O, LSE = ctx.empty(q.shape), ctx.empty((b, h, lq))
        ctx.call("om_attention_fwd", ctx.handle, Q.ptr, Kk.ptr, V.ptr, M.ptr if M else None, i64(0), i32(b), i32(h), i32(lq), i32(lk), i32(d), f32(scale),
                 O.ptr, LSE.ptr)
        Q16, K16, V16, G16 = to_bf16(ctx, q), to_bf16(ctx, k), to_bf16(ctx, v), to_bf16(ctx, g)
        DQ, DK, DV = ctx.empty(q.shape), ctx.empty(k.shape), ctx.empty(v.shape)
        DQ16, DK16, DV16 = ctx.empty(q.shape, np.uint16), ctx.empty(k.shape, np.uint16), ctx.empty(v.shape, np.uint16)
        sq, sk = HeadStrides(h * lq * d, lq * d, d), HeadStrides(h * lk * d, lk * d, d)
        assert ctx.lib.om_attention_bwd_bf16_supported(ctx.handle, i32(b), i32(h), i32(lq), i32(lk), i32(d)) == 1
        ctx.call("om_attention_bwd_bf16", ctx.handle, G16.ptr, G.ptr, C.byref(sq), Q16.ptr, C.byref(sq), K16.ptr, C.byref(sk), V16.ptr, C.byref(sk),
                 O.ptr, C.byref(sq), M.ptr if M else None, i64(0), LSE.ptr, i32(b), i32(h), i32(lq), i32(lk), i32(d), f32(scale), DQ.ptr, DQ16.ptr,
                 C.byref(sq), DK.ptr, DK16.ptr, C.byref(sk), DV.ptr, DV16.ptr, C.byref(sk))
        ctx.sync()
        got = [DQ.numpy(), DK.numpy(), DV.numpy()]
        model = K.attention_bwd_bf16(g, q, k, v, mask)
        exact = K.attention_bwd(g, q, k, v, mask)
        for name, a, m, e in zip("qkv", got, model, exact):
            assert np.all(np.isfinite(a)), name
            assert scaled_diff(a, m) <= 8e-3, (name, scaled_diff(a, m))
            assert scaled_diff(a, e) <= 2e-2, (name, scaled_diff(a, e))
        for a, a16 in zip(got, (DQ16, DK16, DV16)):
            assert np.array_equal(a16.numpy(), bf16_bits(K, a))
        # The same bits from run to run.
        ctx.call("om_attention_bwd_bf16", ctx.handle, G16.ptr, G.ptr, C.byref(sq), Q16.ptr, C.byref(sq), K16.ptr, C.byref(sk), V16.ptr, C.byref(sk),
                 O.ptr, C.byref(sq), M.ptr if M else None, i64(0), LSE.ptr, i32(b), i32(h), i32(lq), i32(lk), i32(d), f32(scale), DQ.ptr, None,
                 C.byref(sq), DK.ptr, None, C.byref(sk), DV.ptr, None, C.byref(sk))
        ctx.sync()
        for a, again in zip(got, (DQ, DK, DV)):
            assert np.array_equal(a, again.numpy())
        # bfloat16 results alone (what a following product reads): the same bits as the copies written beside fp32 results
        O16 = [ctx.empty(t.shape, np.uint16) for t in (q, k, v)]
        ctx.call("om_attention_bwd_bf16", ctx.handle, G16.ptr, G.ptr, C.byref(sq), Q16.ptr, C.byref(sq), K16.ptr, C.byref(sk), V16.ptr, C.byref(sk),
                 O.ptr, C.byref(sq), M.ptr if M else None, i64(0), LSE.ptr, i32(b), i32(h), i32(lq), i32(lk), i32(d), f32(scale), None, O16[0].ptr,
                 C.byref(sq), None, O16[1].ptr, C.byref(sk), None, O16[2].ptr, C.byref(sk))
        ctx.sync()
        for only, both in zip(O16, (DQ16, DK16, DV16)):
            assert np.array_equal(only.numpy(), both.numpy())
    finally:
        ctx.set_flags(0)


def test_shapes_outside_the_fused_kernel_are_refused(ctx):
    assert ctx.lib.om_attention_bwd_bf16_supported(ctx.handle, i32(1), i32(1), i32(4096), i32(4096), i32(64)) == 1
    assert ctx.lib.om_attention_bwd_bf16_supported(ctx.handle, i32(1), i32(1), i32(256), i32(256), i32(32)) == 0
    assert ctx.lib.om_attention_bwd_bf16_supported(ctx.handle, i32(256), i32(256), i32(256), i32(256), i32(64)) == 0


@pytest.mark.parametrize("b,h,lq,lk,masked", [(1, 2, 512, 512, 0), (2, 3, 256, 256, 1), (1, 2, 300, 200, 0), (1, 1, 129, 640, 1), (1, 2, 512, 128, 0),
                                              (1, 1, 5, 7, 0), (2, 12, 512, 512, 0), (1, 2, 1100, 384, 1), (3, 1, 128, 128, 0)])
def test_attention_forward_with_bf16_operands(ctx, oracle_built, b, h, lq, lk, masked):
    """om_attention_fwd_bf16 against the oracle's model of the same tier (q, k, v and the exponentials rounded to bfloat16, sums
    in fp32: what is left is the summation order and exponentials that round the other way at a bfloat16 boundary) and
    against the fp32 forward, where the bfloat16 rounding shows; the log-sum-exp against the fp32 one; the bfloat16 copy is
    the fp32 result rounded; the same bits from run to run. Some masked cases hold -inf entries and one row masked out
    entirely in all but one key."""
    K = oracle_built
    d = 64
    r = np.random.default_rng(b * 11 + lq + 3 * lk)
    q, k, v = (r.standard_normal(s).astype(np.float32) for s in [(b, h, lq, d), (b, h, lk, d), (b, h, lk, d)])
    mask = None
    if masked:
        mask = np.where(r.random((lq, lk)) < 0.25, -4.0, 0.0).astype(np.float32)
        mask[r.random((lq, lk)) < 0.05] = -np.inf
        mask[lq // 2, :] = -np.inf
        mask[lq // 2, lk // 3] = 0.0
    scale = np.float32(1.0 / np.sqrt(np.float32(d)))
    Q16, K16, V16 = to_bf16(ctx, q), to_bf16(ctx, k), to_bf16(ctx, v)
    M = ctx.to_device(mask) if mask is not None else None
    O, O16, LSE = ctx.empty(q.shape), ctx.empty(q.shape, np.uint16), ctx.empty((b, h, lq))
    sq, sk = HeadStrides(h * lq * d, lq * d, d), HeadStrides(h * lk * d, lk * d, d)
    assert ctx.lib.om_attention_fwd_bf16_supported(ctx.handle, i32(b), i32(h), i32(lq), i32(lk), i32(d), f32(scale)) == 1

    def run(o16, lse):
        ctx.call("om_attention_fwd_bf16", ctx.handle, Q16.ptr, C.byref(sq), K16.ptr, C.byref(sk), V16.ptr, C.byref(sk), M.ptr if M else None, i64(0),
                 i32(b), i32(h), i32(lq), i32(lk), i32(d), f32(scale), O.ptr, o16, C.byref(sq), lse)
        ctx.sync()
        return O.numpy()

    got = run(O16.ptr, LSE.ptr)
    assert np.all(np.isfinite(got))
    model = K.attention_fwd_bf16(q, k, v, mask, scale)
    exact = K.attention_fwd(q, k, v, mask, scale)
    assert scaled_diff(got, model) <= 4e-3, scaled_diff(got, model)
    assert scaled_diff(got, exact) <= 2e-2, scaled_diff(got, exact)
    assert np.array_equal(O16.numpy(), bf16_bits(K, got))
    # log-sum-exp of scale q k^T + mask from the rounded operands: against fp64 from the same rounded operands
    qr, kr = K.round_bf16(q).astype(np.float64), K.round_bf16(k).astype(np.float64)
    s = np.einsum("bhqd,bhkd->bhqk", qr, kr) * np.float64(scale)
    if mask is not None:
        s = s + mask.astype(np.float64)
    mx = s.max(axis=-1, keepdims=True)
    lse_ref = (mx + np.log(np.exp(s - mx).sum(axis=-1, keepdims=True)))[..., 0]
    assert np.max(np.abs(LSE.numpy() - lse_ref)) <= 2e-5 * max(1.0, float(np.max(np.abs(lse_ref))))
    assert np.array_equal(got, run(None, None))


@pytest.mark.parametrize("gain,lq,lk", [(3.0, 512, 512), (1.9, 300, 384), (0.2, 512, 512)])
def test_attention_forward_with_large_and_small_scores(ctx, oracle_built, gain, lq, lk):
    """Without a mask the kernel takes scale |q| max|k| as the bound the exponentials are taken against (one pass over the key
    tiles) while that bound is at most 40, and walks the key tiles twice for the true row maximum otherwise. q and k scaled
    so that a tile's bound is around 100 (two passes), around 40 (tiles on either side of the limit in one launch) and
    around 0.4: the same agreement with the oracle's model and the same log-sum-exp in all three."""
    K = oracle_built
    b, h, d = 1, 3, 64
    r = np.random.default_rng(int(gain * 10) + lq)
    q, k, v = (r.standard_normal(s).astype(np.float32) for s in [(b, h, lq, d), (b, h, lk, d), (b, h, lk, d)])
    q, k = q * np.float32(gain), k * np.float32(gain)
    scale = np.float32(1.0 / np.sqrt(np.float32(d)))
    Q16, K16, V16 = to_bf16(ctx, q), to_bf16(ctx, k), to_bf16(ctx, v)
    O, LSE = ctx.empty(q.shape), ctx.empty((b, h, lq))
    sq, sk = HeadStrides(h * lq * d, lq * d, d), HeadStrides(h * lk * d, lk * d, d)
    ctx.call("om_attention_fwd_bf16", ctx.handle, Q16.ptr, C.byref(sq), K16.ptr, C.byref(sk), V16.ptr, C.byref(sk), None, i64(0),
             i32(b), i32(h), i32(lq), i32(lk), i32(d), f32(scale), O.ptr, None, C.byref(sq), LSE.ptr)
    ctx.sync()
    got = O.numpy()
    assert np.all(np.isfinite(got)) and np.all(np.isfinite(LSE.numpy()))
    assert scaled_diff(got, K.attention_fwd_bf16(q, k, v, None, scale)) <= 4e-3
    qr, kr = K.round_bf16(q).astype(np.float64), K.round_bf16(k).astype(np.float64)
    s = np.einsum("bhqd,bhkd->bhqk", qr, kr) * np.float64(scale)
    mx = s.max(axis=-1, keepdims=True)
    lse_ref = (mx + np.log(np.exp(s - mx).sum(axis=-1, keepdims=True)))[..., 0]
    assert np.max(np.abs(LSE.numpy() - lse_ref)) <= 2e-5 * max(1.0, float(np.max(np.abs(lse_ref))))
    bound = float(scale) * np.linalg.norm(qr, axis=-1).max() * np.linalg.norm(kr, axis=-1).max()
    assert (bound > 80) if gain == 3.0 else (bound < 2) if gain == 0.2 else (30 < bound < 60)


def test_forward_shapes_outside_the_kernel_are_refused(ctx):
    sup = ctx.lib.om_attention_fwd_bf16_supported
    assert sup(ctx.handle, i32(1), i32(1), i32(4096), i32(4096), i32(64), f32(0.125)) == 1
    assert sup(ctx.handle, i32(1), i32(1), i32(256), i32(256), i32(32), f32(0.125)) == 0
    assert sup(ctx.handle, i32(1), i32(1), i32(256), i32(256), i32(64), f32(-1.0)) == 0
