"""TEST INFRASTRUCTURE - NOT PART OF THE PRODUCT.

The benchmark configurations on the CPU oracle tape: the same modules wired the same way as the product's trainers
(host/trainer.cpp), used as the parity checker at small sizes and as the timed CPU baseline at full size."""
import numpy as np

from . import oracle as K, tape as A


def mlp_step(params, x, y, t, lr=1e-3, wd=0.01, state=None):
    """Config 1: params is a list [w0, b0, w1, b1, ...] of arrays (updated in place). Returns the loss."""
    P = [A.T(p, True) for p in params]
    h = A.T(x)
    n = len(P) // 2
    for i in range(n):
        h = A.linear(h, P[2 * i], P[2 * i + 1])
        if i + 1 < n:
            h = A.relu(h)
    loss = A.cross_entropy(h, y)
    loss.backward()
    _adamw(params, [p.grad for p in P], state, t, lr, wd)
    return float(loss.v), [p.grad for p in P]


def _encoder_layer(x, w, p, heads):
    b, n, d = x.shape
    dh = d // heads

    def split(z):
        return z.reshape(b, n, heads, dh).permute(0, 2, 1, 3)

    q = split(A.linear(x, w[p + "attn.q.weight"], w[p + "attn.q.bias"]))
    k = split(A.linear(x, w[p + "attn.k.weight"], w[p + "attn.k.bias"]))
    v = split(A.linear(x, w[p + "attn.v.weight"], w[p + "attn.v.bias"]))
    a = A.attention(q, k, v).permute(0, 2, 1, 3).reshape(b, n, d)
    a = A.linear(a, w[p + "attn.o.weight"], w[p + "attn.o.bias"])
    x1 = A.layer_norm(A.add(x, a), w[p + "norm1.weight"], w[p + "norm1.bias"])
    f = A.linear(A.gelu(A.linear(x1, w[p + "ff1.weight"], w[p + "ff1.bias"])), w[p + "ff2.weight"], w[p + "ff2.bias"])
    return A.layer_norm(A.add(x1, f), w[p + "norm2.weight"], w[p + "norm2.bias"])


def mlm_forward_backward(named, ids, rows, labels, layers, heads, denominator=None):
    """Configs 3 and 5: named maps the product's parameter names to arrays. Returns (loss, {name: grad})."""
    w = {k: A.T(v, True) for k, v in named.items()}
    b, s = ids.shape
    d = named["tok.weight"].shape[1]
    x = A.add(A.embedding(w["tok.weight"], ids), A.embedding(w["pos.weight"], np.arange(s)))
    for i in range(layers):
        x = _encoder_layer(x, w, f"layers.{i}.", heads)
    picked = A.embedding(x.reshape(b * s, d), rows)
    logits = A.linear(picked, w["head.weight"], w["head.bias"])
    if denominator is None:
        loss = A.cross_entropy(logits, labels)
    else:   # data-parallel shard: sum over local rows divided by the global row count
        loss = A.mul(A.cross_entropy(logits, labels, mean=False), A.T(np.float32(1.0 / denominator)))
    loss.backward()
    return float(loss.v), {k: t.grad for k, t in w.items()}


def _adamw(params, grads, state, t, lr, wd):
    if state is None:
        return
    for i, (p, g) in enumerate(zip(params, grads)):
        if g is None:
            continue
        s = state.setdefault(i, dict(m=np.zeros_like(p), v=np.zeros_like(p)))
        K.adam_step(p, g, s["m"], s["v"], None, t, lr, 0.9, 0.999, 1e-8, wd, True, False)


def mlm_step(named, ids, rows, labels, layers, heads, t, state, lr=1e-4, wd=0.01):
    loss, grads = mlm_forward_backward(named, ids, rows, labels, layers, heads)
    names = list(named)
    _adamw([named[k] for k in names], [grads[k] for k in names], state, t, lr, wd)
    return loss, grads
