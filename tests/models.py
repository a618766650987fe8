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


def train_encoder(B, fx, steps=None):
    """testdata/training/encoder: embedding + 2 encoder layers + mean pool + classifier, Adam lr 2e-3 with a linear
    warm-up from 0.1 over 10 steps, batch 16, 80 steps."""
    w = {k[3:]: B.tensor(v, True) for k, v in fx.items() if k.startswith("in.") and k[3:] not in ("ids", "y", "order")}
    names = [k[3:] for k in fx if k.startswith("in.") and k[3:] not in ("ids", "y", "order")]
    opt = B.optimizer("adam", [w[k] for k in names], 2e-3)
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
