"""The models of the reference's own fixtures, written once against the small tensor API of tests/backends.py.

They restate the PyTorch programs of the reference's generators (tools/training_oracle.py: mlp, encoder;
tools/autograd_oracle.py: encoder) with the reference's module wiring (src/OneModel.Training/Layers.cs:459-577:
q, k, v, o projections, post-norm residual blocks, erf GELU)."""
import numpy as np


def encoder_layers(B, x, w, layers, heads, mask=None):
    b, n, d = x.shape
    dh = d // heads

    def split(z):
        return z.reshape(b, n, heads, dh).permute(0, 2, 1, 3)

    for i in range(layers):
        p = f"l{i}."
        q = split(B.linear(x, w[p + "wq"], w[p + "bq"]))
        k = split(B.linear(x, w[p + "wk"], w[p + "bk"]))
        v = split(B.linear(x, w[p + "wv"], w[p + "bv"]))
        a = B.attention(q, k, v, mask).permute(0, 2, 1, 3).reshape(b, n, d)
        x1 = B.layer_norm(B.add(x, B.linear(a, w[p + "wo"], w[p + "bo"])), w[p + "ln1g"], w[p + "ln1b"])
        f = B.linear(B.gelu(B.linear(x1, w[p + "w1"], w[p + "b1"])), w[p + "w2"], w[p + "b2"])
        x = B.layer_norm(B.add(x1, f), w[p + "ln2g"], w[p + "ln2b"])
    return x


def autograd_encoder(B, fx):
    """testdata/autograd/encoder: loss = sum(encoder(emb[ids]) * proj); returns (loss, y, params)."""
    w = {k[3:]: B.tensor(v, True) for k, v in fx.items() if k.startswith("in.") and k[3:] not in ("ids", "mask", "proj")}
    ids = fx["in.ids"].astype(np.int64)
    x = B.embedding(w["emb"], B.ids(ids))
    y = encoder_layers(B, x, w, layers=2, heads=2, mask=fx["in.mask"])
    loss = B.sum(B.mul(y, B.tensor(fx["in.proj"])))
    return loss, y, w


def train_mlp(B, fx, steps=None):
    """testdata/training/mlp: 20-32-4 MLP, SGD lr 0.05 momentum 0.9 weight decay 1e-4, batch 32, 100 steps."""
    names = ["w1", "b1", "w2", "b2"]
    p = {k: B.tensor(fx["in." + k], True) for k in names}
    opt = B.optimizer("sgd", [p[k] for k in names], 0.05, momentum=0.9, weight_decay=1e-4)
    x, y, order = fx["in.x"], fx["in.y"].astype(np.int64), fx["in.order"].astype(np.int64)
    losses = []
    for s in range(len(order) if steps is None else steps):
        idx = order[s]
        logits = B.linear(B.relu(B.linear(B.tensor(x[idx]), p["w1"], p["b1"])), p["w2"], p["b2"])
        loss = B.cross_entropy(logits, B.ids(y[idx]))
        opt.zero_grad()
        B.backward(loss)
        opt.step()
        losses.append(float(B.numpy(loss).reshape(-1)[0]))
    return np.array(losses, np.float32), {k: B.numpy(v) for k, v in p.items()}


def train_encoder(B, fx, steps=None, frozen=()):
    """testdata/training/encoder: embedding + 2 encoder layers + mean pool + classifier, Adam lr 2e-3 with a linear
    warm-up from 0.1 over 10 steps, batch 16, 80 steps. Parameters whose name is in `frozen` or starts with one of its
    entries plus a dot do not require gradients and are not given to the optimizer (NnModule.Freeze of the reference,
    tests/OneModel.Tests/Training/SparseAndFrozenTests.cs:48-56)."""
    names = [k[3:] for k in fx if k.startswith("in.") and k[3:] not in ("ids", "y", "order")]
    is_frozen = lambda n: any(n == f or n.startswith(f + ".") for f in frozen)
    w = {k: B.tensor(fx["in." + k], not is_frozen(k)) for k in names}
    opt = B.optimizer("adam", [w[k] for k in names if not is_frozen(k)], 2e-3)
    ids, y, order = fx["in.ids"].astype(np.int64), fx["in.y"].astype(np.int64), fx["in.order"].astype(np.int64)
    peak, warm = 2e-3, 10
    losses = []
    for s in range(len(order) if steps is None else steps):
        # LrSchedule linear warm-up (Schedules.cs:171-260): factor 0.1 -> 1.0 over `warm` steps.
        factor = 0.1 + (1.0 - 0.1) * min(s, warm) / warm
        opt.set_lr(float(np.float32(peak * factor)))
        idx = order[s]
        x = B.embedding(w["emb"], B.ids(ids[idx]))
        h = encoder_layers(B, x, w, layers=2, heads=2)
        logits = B.linear(B.mean(h, 1), w["clsw"], w["clsb"])
        loss = B.cross_entropy(logits, B.ids(y[idx]))
        opt.zero_grad()
        B.backward(loss)
        opt.step()
        losses.append(float(B.numpy(loss).reshape(-1)[0]))
    return np.array(losses, np.float32), {k: B.numpy(w[k]) for k in names}


def cnn_forward(B, w, x, rm1, rv1, rm2, rv2, batch):
    """The conv net of testdata/autograd/cnn and testdata/training/cnn: conv-bn-relu-maxpool, conv-bn-relu-avgpool, linear."""
    h = B.conv2d(x, w["c1w"], w["c1b"], 1, 1)
    h = B.batch_norm2d(h, w["bn1g"], w["bn1b"], rm1, rv1, True)
    h = B.max_pool2d(B.relu(h), 2)
    h = B.conv2d(h, w["c2w"], w["c2b"], 1, 1)
    h = B.batch_norm2d(h, w["bn2g"], w["bn2b"], rm2, rv2, True)
    h = B.avg_pool2d(B.relu(h), 2)
    return B.linear(h.reshape(batch, 72), w["fcw"], w["fcb"])


CNN_PARAMS = ["c1w", "c1b", "bn1g", "bn1b", "c2w", "c2b", "bn2g", "bn2b", "fcw", "fcb"]


def autograd_cnn(B, fx):
    """testdata/autograd/cnn: loss = NLL(log_softmax(logits)); returns (loss, logits, params incl. x, running stats)."""
    w = {k: B.tensor(fx["in." + k], True) for k in CNN_PARAMS + ["x"]}
    rs = [B.running(np.zeros(4)), B.running(np.ones(4)), B.running(np.zeros(8)), B.running(np.ones(8))]
    logits = cnn_forward(B, w, w["x"], *rs, batch=4)
    loss = B.nll_loss(B.log_softmax(logits), B.ids(fx["in.targets"].astype(np.int64)))
    return loss, logits, w, rs


def train_cnn(B, fx, steps=None):
    """testdata/training/cnn: AdamW lr 3e-3 wd 0.01, cosine schedule to 0 over 60 steps, gradient-norm clipping at 0.5."""
    w = {k: B.tensor(fx["in." + k], True) for k in CNN_PARAMS}
    params = [w[k] for k in CNN_PARAMS]
    opt = B.optimizer("adamw", params, 3e-3, weight_decay=0.01)
    rs = [B.running(np.zeros(4)), B.running(np.ones(4)), B.running(np.zeros(8)), B.running(np.ones(8))]
    x, y, order = fx["in.x"], fx["in.y"].astype(np.int64), fx["in.order"].astype(np.int64)
    total = len(order)
    losses, norms = [], []
    for s in range(total if steps is None else steps):
        # LrSchedule.Cos closed form (Schedules.cs:171-260): eta_min + (base - eta_min) (1 + cos(pi s / T)) / 2
        opt.set_lr(float(np.float32(3e-3 * (1.0 + np.cos(np.pi * s / total)) / 2.0)))
        idx = order[s]
        logits = cnn_forward(B, w, B.tensor(x[idx]), *rs, batch=len(idx))
        loss = B.cross_entropy(logits, B.ids(y[idx]))
        opt.zero_grad()
        B.backward(loss)
        norms.append(B.clip_norm(params, 0.5))
        opt.step()
        losses.append(float(B.numpy(loss).reshape(-1)[0]))
    return np.array(losses, np.float32), np.array(norms, np.float32), {k: B.numpy(w[k]) for k in CNN_PARAMS}, [B.running_numpy(r) for r in rs]


def autograd_crnn(B, fx):
    """testdata/autograd/crnn: conv-relu-maxpool x2, 2-layer BiLSTM(5), linear to 7 classes, log-softmax, CTC mean."""
    names = [k[3:] for k in fx if k.startswith("in.") and k[3:] not in ("targets", "input_lengths", "target_lengths")]
    w = {k: B.tensor(fx["in." + k], True) for k in names}
    h = B.max_pool2d(B.relu(B.conv2d(w["x"], w["c1w"], w["c1b"], 1, 1)), 2)
    h = B.max_pool2d(B.relu(B.conv2d(h, w["c2w"], w["c2b"], 1, 1)), (4, 1))      # [2, 6, 1, 12]
    seq = h.reshape(2, 6, 12).permute(2, 0, 1)                                   # [T = 12, B, 6]
    for layer in range(2):
        outs = []
        for d, sfx in enumerate(("", "_reverse")):
            p = f"lstm.%s_l{layer}{sfx}"
            outs.append(B.lstm_layer(seq, w[p % "weight_ih"], w[p % "weight_hh"], w[p % "bias_ih"], w[p % "bias_hh"], d == 1))
        seq = B.concat(outs, 2)
    lp = B.log_softmax(B.linear(seq, w["fcw"], w["fcb"]))
    loss = B.ctc_loss(lp, fx["in.targets"].astype(np.int32), fx["in.input_lengths"].astype(np.int32),
                      fx["in.target_lengths"].astype(np.int32), 0, 1, False)
    return loss, lp, w


def autograd_gru(B, fx):
    """testdata/autograd/gru: 1-layer bidirectional GRU (batch first, with initial state) -> weighted sum
    (tests/OneModel.Tests/Tensors/RnnOracleTests.cs:158-175 of the reference)."""
    names = [k[3:] for k in fx if k.startswith("in.") and k != "in.proj"]
    w = {k: B.tensor(fx["in." + k], True) for k in names}
    seq = w["x"].permute(1, 0, 2)                       # [T, B, I]
    outs = []
    for d, sfx in enumerate(("", "_reverse")):
        p = f"gru.%s_l0{sfx}"
        outs.append(B.gru_layer(seq, w[p % "weight_ih"], w[p % "weight_hh"], w[p % "bias_ih"], w[p % "bias_hh"],
                                B.select(w["h0"], 0, d), d == 1))
    y = B.concat(outs, 2).permute(1, 0, 2)              # [B, T, 2H]
    loss = B.sum(B.mul(y, B.tensor(fx["in.proj"])))
    return loss, y, w


def graph_ops_case(B, seed=0):
    """One graph through every op of the graph-op family (Ops.GraphOps.cs): returns the loss and the leaves."""
    r = np.random.default_rng(seed)
    a = B.tensor(r.standard_normal((2, 3, 4, 5)).astype(np.float32), True)
    b = B.tensor(r.standard_normal((3, 5, 6)).astype(np.float32), True)        # batch axes broadcast against a's
    c = B.tensor((r.random((4, 6)) + 0.5).astype(np.float32), True)
    d = B.tensor(r.standard_normal((1, 6)).astype(np.float32), True)
    m = B.matmul_batched(a, b)                                                   # [2, 3, 4, 6]
    t = B.add(B.erf(m), B.exp(B.mul(m, B.tensor(np.full((1,), 0.1, np.float32)))))
    t = B.add(t, B.sqrt(c))                                                      # c broadcasts over the batch axes
    t = B.add(t, B.pow(c, 2.0))
    t = B.add(t, B.pow(c, -1.0))
    t = B.add(t, B.pow(c, 0.5))
    t = B.add(t, B.pow(c, 1.7))
    cond = (r.random((3, 4, 6)) < 0.5).astype(np.int32)
    t = B.where(cond, t, d)                                                      # d [1, 6] broadcasts
    g = B.gather(t, np.array([[2, -1], [0, 2]]), 2)                              # axis of 4 -> [2, 3, 2, 2, 6], repeated rows
    w = B.tensor(r.standard_normal((2, 3, 2, 2, 6)).astype(np.float32))
    loss = B.sum(B.mul(g, w))
    return loss, g, {"a": a, "b": b, "c": c, "d": d}


CONV1D_CASES = [
    # n, c, l, o, k, stride, pad_left, pad_right, dilation, groups, bias
    (2, 4, 19, 6, 3, 1, 1, 1, 1, 1, True),
    (3, 6, 23, 4, 5, 2, 0, 3, 2, 2, True),        # stride, asymmetric padding, dilation, two groups
    (1, 3, 8, 5, 1, 1, 0, 0, 1, 1, False),        # pointwise, no bias
    (2, 8, 16, 8, 4, 3, 2, 1, 1, 4, True),        # "same"-style uneven padding, four groups
]


def conv1d_case(B, case, seed=0):
    """One Conv1d (Ops.Conv1d of the reference) under a weighted sum: returns the loss, the output and the leaves."""
    n, c, l, o, k, stride, pl, pr, dil, groups, has_bias = case
    r = np.random.default_rng(seed + l)
    x = B.tensor(r.standard_normal((n, c, l)).astype(np.float32), True)
    w = B.tensor((r.standard_normal((o, c // groups, k)) * 0.5).astype(np.float32), True)
    b = B.tensor(r.standard_normal(o).astype(np.float32), True) if has_bias else None
    y = B.conv1d(x, w, b, stride, pl, pr, dil, groups)
    out_l = (l + pl + pr - dil * (k - 1) - 1) // stride + 1
    proj = B.tensor(r.standard_normal((n, o, out_l)).astype(np.float32))
    loss = B.sum(B.mul(y, proj))
    leaves = {"x": x, "w": w}
    if has_bias:
        leaves["b"] = b
    return loss, y, leaves


def conv1d_grid_params(case, k):
    """(stride, pad_left, pad_right, dilation, groups) of one case of testdata/conv1d/grid.json: a number pads both sides,
    "same" splits dilation*(k-1) with the odd zero on the right, "valid" pads nothing (Conv1dParams.Symmetric / Same,
    Ops.Nn.cs:12-26; tests/OneModel.Tests/Training/Conv1dTests.cs:22-41 of the reference)."""
    stride, dil, groups, pad = case["stride"], case["dilation"], case["groups"], case["padding"]
    if isinstance(pad, int):
        return stride, pad, pad, dil, groups
    if pad == "same":
        total = max(dil, 1) * (k - 1)
        return 1, total // 2, total - total // 2, dil, groups
    return 1, 0, 0, dil, groups


def conv1d_grid_case(B, fx, i, case):
    """Case i of testdata/conv1d/grid: y = Conv1d(x, w, b), loss = sum(y * r); returns y and the leaves
    (Conv1dTests.cs:76-88 of the reference)."""
    pre = f"c{i}."
    x, w = B.tensor(fx[pre + "in.x"], True), B.tensor(fx[pre + "in.w"], True)
    b = B.tensor(fx[pre + "in.b"], True) if case["bias"] else None
    y = B.conv1d(x, w, b, *conv1d_grid_params(case, fx[pre + "in.w"].shape[2]))
    loss = B.sum(B.mul(y, B.tensor(fx[pre + "in.r"])))
    leaves = {"x": x, "w": w}
    if b is not None:
        leaves["b"] = b
    return loss, y, leaves


def train_conv1d(B, fx):
    """testdata/conv1d/train: Conv1d(4,6,3,"same",dilation 2) - ReLU - Conv1d(6,6,3,stride 2,padding 1,groups 2) - ReLU -
    mean over length - Linear(6,3); cross entropy; SGD lr 0.05 momentum 0.9; 20 steps of 8 samples in the recorded order
    (Conv1dTests.cs:258-307 of the reference). Returns the losses and the final parameters."""
    names = ("c1w", "c1b", "c2w", "c2b", "fcw", "fcb")
    p = {k: B.tensor(fx["in." + k], True) for k in names}
    opt = B.optimizer("sgd", [p[k] for k in names], 0.05, momentum=0.9)
    order = fx["in.order"].astype(np.int64)
    losses = []
    for s in range(order.shape[0]):
        x = B.tensor(fx["in.x"][order[s]])
        t = B.ids(fx["in.y"][order[s]].astype(np.int64))
        h = B.relu(B.conv1d(x, p["c1w"], p["c1b"], 1, 2, 2, 2, 1))
        h = B.relu(B.conv1d(h, p["c2w"], p["c2b"], 2, 1, 1, 1, 2))
        loss = B.cross_entropy(B.linear(B.mean(h, 2), p["fcw"], p["fcb"]), t)
        opt.zero_grad()
        B.backward(loss)
        losses.append(float(B.numpy(loss).reshape(-1)[0]))
        opt.step()
    return np.array(losses), {k: B.numpy(p[k]) for k in names}


def autograd_decoder(B, fx):
    """testdata/autograd/decoder: conv, two transposed convolutions (stride 2; stride 2 with padding, output padding and two
    groups), nearest and bilinear resizes (tests/OneModel.Tests/Tensors/RnnOracleTests.cs:177-201 of the reference)."""
    w = {k: B.tensor(fx["in." + k], True) for k in ("x", "c1w", "c1b", "t1w", "t1b", "t2w", "t2b", "c2w", "c2b")}
    h = B.relu(B.conv2d(w["x"], w["c1w"], w["c1b"], 1, 1))
    h = B.relu(B.conv_transpose2d(h, w["t1w"], w["t1b"], 2, 0, 0, 1))
    h = B.relu(B.conv_transpose2d(h, w["t2w"], w["t2b"], 2, 1, 1, 2))
    h = B.resize2d(h, 13, 30, 0, False)
    h = B.conv2d(h, w["c2w"], w["c2b"], 1, 1)
    a = B.resize2d(h, 9, 17, 1, False)
    c = B.resize2d(h, 16, 11, 1, True)
    loss = B.add(B.sum(B.mul(a, B.tensor(fx["in.pa"]))), B.sum(B.mul(c, B.tensor(fx["in.pc"]))))
    return loss, a, c, w
