"""The fused several-tile attention backward with bfloat16 product operands (om_attention_bwd_bf16) against the CPU
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
    finally:
        ctx.set_flags(0)


def test_shapes_outside_the_fused_kernel_are_refused(ctx):
    assert ctx.lib.om_attention_bwd_bf16_supported(ctx.handle, i32(1), i32(1), i32(4096), i32(4096), i32(64)) == 1
    assert ctx.lib.om_attention_bwd_bf16_supported(ctx.handle, i32(1), i32(1), i32(256), i32(256), i32(32)) == 0
    assert ctx.lib.om_attention_bwd_bf16_supported(ctx.handle, i32(256), i32(256), i32(256), i32(256), i32(64)) == 0
