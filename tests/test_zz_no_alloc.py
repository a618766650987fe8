"""om_colsum_static: the column sum (bias gradient) that takes its scratch from a fixed array inside the module instead
of the pool. Checked through the C ABI against om_colsum on the same inputs, twice in a row (the second call meets the
first call's leftovers in the array), and against the documented size limit. Collected last on purpose: it has to pass
both alone and after every other test has used the device."""
import numpy as np
import pytest

import om_binding as omb
from om_binding import i32

pytestmark = pytest.mark.gpu


def both(ctx, g, accumulate, out0):
    rows, cols = g.shape
    G = ctx.to_device(g)
    A, B = ctx.to_device(out0), ctx.to_device(out0)
    ctx.call("om_colsum", ctx.handle, G.ptr, i32(rows), i32(cols), A.ptr, i32(accumulate))
    ctx.call("om_colsum_static", ctx.handle, G.ptr, i32(rows), i32(cols), B.ptr, i32(accumulate))
    ctx.sync()
    return A.numpy(), B.numpy()


def test_static_scratch_matches_pool_scratch_twice(ctx):
    ctx.set_flags(0)
    r = np.random.default_rng(11)
    # First call: a large table (3 chunks x 30522 columns) that fills most of the array.
    g1 = r.standard_normal((1229, 30522)).astype(np.float32)
    a, b = both(ctx, g1, 0, np.zeros(30522, np.float32))
    assert np.array_equal(a, b)
    assert np.allclose(b, g1.astype(np.float64).sum(0), rtol=1e-5, atol=1e-4)
    # Second call straight after it: another shape, accumulating, reading slots the first call left dirty.
    g2 = r.standard_normal((8192, 1536)).astype(np.float32)
    o2 = r.standard_normal(1536).astype(np.float32)
    a, b = both(ctx, g2, 1, o2)
    assert np.array_equal(a, b)
    # And a small ragged one.
    g3 = r.standard_normal((7, 45)).astype(np.float32)
    a, b = both(ctx, g3, 0, np.zeros(45, np.float32))
    assert np.array_equal(a, b)
    assert np.array_equal(b, g3.astype(np.float64).sum(0).astype(np.float32))


def test_sizes_beyond_the_array_are_refused(ctx):
    rows, cols = 513, 65537          # 2 chunks x 65537 columns = 131074 slots > 131072
    G, O = ctx.empty((rows, cols)), ctx.empty((cols,))
    with pytest.raises(omb.OmError) as e:
        ctx.call("om_colsum_static", ctx.handle, G.ptr, i32(rows), i32(cols), O.ptr, i32(0))
    assert "131072" in str(e.value) and "om_colsum" in str(e.value)
    # Tall and narrow: 65537 chunks x 1 column fits the array but not the launch grid. Refused before any kernel runs (the
    # pointers are never read, so a small buffer stands in for the 134 MB table).
    with pytest.raises(omb.OmError) as e:
        ctx.call("om_colsum_static", ctx.handle, G.ptr, i32(65537 * 512), i32(1), O.ptr, i32(0))
    assert "65535" in str(e.value) and "om_colsum" in str(e.value)
    # The context stays usable and the largest admitted size works.
    rows, cols = 512, 131072
    g = np.ones((rows, cols), np.float32)
    G, O = ctx.to_device(g), ctx.empty((cols,))
    ctx.call("om_colsum_static", ctx.handle, G.ptr, i32(rows), i32(cols), O.ptr, i32(0))
    ctx.sync()
    assert np.array_equal(O.numpy(), np.full(cols, 512, np.float32))
