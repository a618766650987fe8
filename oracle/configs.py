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


def mlm_init(seq, layers, width, ff, vocab, seed=0):
    """Parameter set of the masked-LM encoder under the product's parameter names, uniform(+-1/sqrt(fan_in)) as the
    reference's Linear default (Layers.cs:59-64). Values come from numpy's generator: callers that compare with the GPU
    load these same arrays into it."""
    rng = np.random.default_rng(seed)
    named = {"tok.weight": rng.uniform(-1, 1, (vocab, width)).astype(np.float32),
             "pos.weight": rng.uniform(-1, 1, (seq, width)).astype(np.float32)}

    def lin(o, i):
        b = 1.0 / np.sqrt(i)
        return rng.uniform(-b, b, (o, i)).astype(np.float32), rng.uniform(-b, b, o).astype(np.float32)

    for l in range(layers):
        p = f"layers.{l}."
        for n in "qkvo":
            named[p + f"attn.{n}.weight"], named[p + f"attn.{n}.bias"] = lin(width, width)
        named[p + "norm1.weight"], named[p + "norm1.bias"] = np.ones(width, np.float32), np.zeros(width, np.float32)
        named[p + "ff1.weight"], named[p + "ff1.bias"] = lin(ff, width)
        named[p + "ff2.weight"], named[p + "ff2.bias"] = lin(width, ff)
        named[p + "norm2.weight"], named[p + "norm2.bias"] = np.ones(width, np.float32), np.zeros(width, np.float32)
    named["head.weight"], named["head.bias"] = lin(vocab, width)
    return named


def mlm_step(named, ids, rows, labels, layers, heads, t, state, lr=1e-4, wd=0.01):
    loss, grads = mlm_forward_backward(named, ids, rows, labels, layers, heads)
    names = list(named)
    _adamw([named[k] for k in names], [grads[k] for k in names], state, t, lr, wd)
    return loss, grads


def cnn_forward_backward(named, running, x, y, strides):
    """Config 2: [conv 3x3 pad 1 + batch norm + ReLU] per entry of strides, global average pool, linear, cross-entropy.
    named: conv{i}.weight/bias, bn{i}.weight/bias, fc.weight/bias. running: {bn{i}: (mean, var)}, updated in place."""
    w = {k: A.T(v, True) for k, v in named.items()}
    h = A.T(x)
    for i, s in enumerate(strides):
        h = A.conv2d(h, w[f"conv{i}.weight"], w[f"conv{i}.bias"], s, 1)
        rm, rv = running[f"bn{i}"]
        h = A.relu(A.batch_norm2d(h, w[f"bn{i}.weight"], w[f"bn{i}.bias"], rm, rv, True))
    n, c = h.shape[0], h.shape[1]
    pooled = A.mean(h.reshape(n, c, h.shape[2] * h.shape[3]), 2)
    loss = A.cross_entropy(A.linear(pooled, w["fc.weight"], w["fc.bias"]), y)
    loss.backward()
    return float(loss.v), {k: t.grad for k, t in w.items()}


def cnn_step(named, running, x, y, strides, state, lr=0.1, momentum=0.9, wd=0.0):
    """One SGD-momentum step (Sgd.Update, Optimizers.cs:335-373). state: {name: buffer}, empty before the first step."""
    loss, grads = cnn_forward_backward(named, running, x, y, strides)
    for k, p in named.items():
        first = k not in state
        buf = state.setdefault(k, np.zeros_like(p))
        K.sgd_step(p, grads[k], buf, first, lr, wd, momentum, 0.0, False)
    return loss, grads


def crnn_forward_backward(named, x, targets, target_lengths, loss_scale=None):
    """Config 4: four conv 3x3 + ReLU + max-pool stages ((2,2),(2,2),(2,1),(4,1)), a 2-layer bidirectional LSTM over the
    width axis, linear, log-softmax, CTC (blank 0, mean, zero-infinity). named: conv{i}.*, lstm.*, fc.*."""
    w = {k: A.T(v, True) for k, v in named.items()}
    h = A.T(x)
    for i, pool in enumerate(((2, 2), (2, 2), (2, 1), (4, 1))):
        h = A.max_pool2d(A.relu(A.conv2d(h, w[f"conv{i}.weight"], w[f"conv{i}.bias"], 1, 1)), pool)
    b, c, _, t = h.shape
    seq = h.reshape(b, c, t).permute(2, 0, 1)
    for layer in range(2):
        outs = []
        for d, sfx in enumerate(("", "_reverse")):
            p = f"lstm.%s_l{layer}{sfx}"
            outs.append(A.lstm_layer(seq, w[p % "weight_ih"], w[p % "weight_hh"], w[p % "bias_ih"], w[p % "bias_hh"], d == 1))
        seq = A.concat(outs, 2)
    lp = A.log_softmax(A.linear(seq, w["fc.weight"], w["fc.bias"]))
    ilen = np.full(b, t, np.int32)
    loss = A.ctc_loss(lp, np.asarray(targets, np.int32), ilen, np.asarray(target_lengths, np.int32), 0, 1, True)
    if loss_scale is not None:   # a data-parallel shard: its mean times 1 / world
        loss = A.mul(loss, A.T(np.float32(loss_scale)))
    loss.backward()
    return float(loss.v), {k: v.grad for k, v in w.items()}


def crnn_step(named, x, targets, target_lengths, t, state, lr=1e-3):
    """One Adam step (coupled weight decay 0; Adam.UpdateRange, Optimizers.cs:554-589)."""
    loss, grads = crnn_forward_backward(named, x, targets, target_lengths)
    for i, (k, p) in enumerate(named.items()):
        s = state.setdefault(k, dict(m=np.zeros_like(p), v=np.zeros_like(p)))
        K.adam_step(p, grads[k], s["m"], s["v"], None, t, lr, 0.9, 0.999, 1e-8, 0.0, False, False)
    return loss, grads


def cnn_init(in_ch, channels, classes, seed=0):
    """Parameters and running statistics of the config-2 network: He-normal weights, zero biases, unit batch norms."""
    rng = np.random.default_rng(seed)
    named, running, c = {}, {}, in_ch
    for i, o in enumerate(channels):
        named[f"conv{i}.weight"] = (rng.standard_normal((o, c, 3, 3)) * np.sqrt(2.0 / (c * 9))).astype(np.float32)
        named[f"conv{i}.bias"] = np.zeros(o, np.float32)
        named[f"bn{i}.weight"], named[f"bn{i}.bias"] = np.ones(o, np.float32), np.zeros(o, np.float32)
        running[f"bn{i}"] = (np.zeros(o, np.float32), np.ones(o, np.float32))
        c = o
    named["fc.weight"] = (rng.standard_normal((classes, c)) * np.sqrt(2.0 / c)).astype(np.float32)
    named["fc.bias"] = np.zeros(classes, np.float32)
    return named, running


def crnn_init(channels, hidden, classes, seed=0):
    """Parameters of the config-4 network, uniform(+-1/sqrt(fan_in)) as the reference's defaults."""
    rng = np.random.default_rng(seed)
    named, c = {}, 1

    def uni(shape, fan):
        b = 1.0 / np.sqrt(fan)
        return rng.uniform(-b, b, shape).astype(np.float32)

    for i, o in enumerate(channels):
        named[f"conv{i}.weight"], named[f"conv{i}.bias"] = uni((o, c, 3, 3), c * 9), uni((o,), c * 9)
        c = o
    for layer in range(2):
        inp = c if layer == 0 else 2 * hidden
        for sfx in ("", "_reverse"):
            named[f"lstm.weight_ih_l{layer}{sfx}"] = uni((4 * hidden, inp), hidden)
            named[f"lstm.weight_hh_l{layer}{sfx}"] = uni((4 * hidden, hidden), hidden)
            named[f"lstm.bias_ih_l{layer}{sfx}"] = uni((4 * hidden,), hidden)
            named[f"lstm.bias_hh_l{layer}{sfx}"] = uni((4 * hidden,), hidden)
    named["fc.weight"], named["fc.bias"] = uni((classes, 2 * hidden), 2 * hidden), uni((classes,), 2 * hidden)
    return named
