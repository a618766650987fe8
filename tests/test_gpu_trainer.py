"""The benchmark configurations' training steps (host/trainer.cpp, the path bench.py times) against the CPU oracle
running the same model on the same weights and batches, at sizes the oracle finishes in seconds."""
import numpy as np
import pytest

import om_binding as omb
import synth
from backends import scaled_diff

pytestmark = pytest.mark.gpu


@pytest.fixture()
def configs(oracle_built):
    from oracle import configs
    return configs


def test_mlp_config_100_steps_loss_within_1_percent(ctx, configs):
    """Config 1 at full size (784-512-512-10, batch 128, AdamW): loss after 100 steps within 1% of the CPU path,
    and every step within 1e-3 (the reference's own tolerance for training curves, TrainingCurveTests.cs:75-106)."""
    ctx.set_flags(0)
    ctx.make_current()
    tr = omb.Trainer("mlp", [128, 784, 512, 512, 10], lr=1e-3, weight_decay=0.01, seed=0)
    named = tr.named_parameters()
    params = [tr.get_param(i, s) for i, (_, s) in enumerate(named)]
    state = {}
    for step in range(100):
        x, y = synth.mlp_batch(128, 784, 10, step)
        lg = tr.step([x, y])
        lo, _ = configs.mlp_step(params, x, y, step + 1, state=state)
        assert abs(lg - lo) <= 1e-3 * abs(lo), step
    assert abs(lg - lo) <= 0.01 * abs(lo)
    # Final parameters are not compared element-wise: on this noise-label task Adam turns rounding-level gradient
    # differences into steps of the full learning rate (the effect the reference documents for zero-gradient
    # parameters, TrainingCurveTests.cs:49-60); the loss curve is the contract.
    tr.close()


@pytest.mark.parametrize("graph", [False, True])
def test_mlm_config_small(ctx, configs, graph):
    """Configs 3/5 at reduced size: per-parameter gradients after step 1 (scaled 1e-4) and losses over 6 AdamW steps,
    eager and replayed from a captured CUDA graph."""
    ctx.set_flags(0)
    ctx.make_current()
    batch, seq, layers, width, heads, ff, vocab, rows = 4, 16, 2, 32, 4, 64, 101, 10
    tr = omb.Trainer("mlm", [batch, seq, layers, width, heads, ff, vocab, rows], lr=1e-3, weight_decay=0.01, seed=0)
    named = tr.named_parameters()
    weights = {n: tr.get_param(i, s) for i, (n, s) in enumerate(named)}
    state = {}
    for step in range(6):
        ids, pos, labels = synth.mlm_batch(batch, seq, vocab, rows, step)
        if graph and step == 1:
            tr.enable_graph()
        before = {k: v.copy() for k, v in weights.items()}
        lg = tr.step([ids, pos, labels])
        lo, grads = configs.mlm_step(weights, ids.astype(np.int64), pos.astype(np.int64), labels, layers, heads, step + 1, state, lr=1e-3)
        assert abs(lg - lo) <= 1e-4 * abs(lo), step
        if step == 0:
            largest = max(np.max(np.abs(g)) for g in grads.values())
            for i, (n, s) in enumerate(named):
                gg = tr.get_grad(i, s)
                if np.max(np.abs(grads[n])) < 1e-5 * largest:
                    assert np.max(np.abs(gg)) < 1e-5 * largest, n
                else:
                    assert scaled_diff(gg, grads[n]) <= 1e-4, n
        del before
    for i, (n, s) in enumerate(named):
        if not n.endswith("attn.k.bias"):
            assert scaled_diff(tr.get_param(i, s), weights[n]) <= 1e-3, n
    tr.close()


def _run_c3(steps, graph_at, tf32):
    cfg = [64, 128, 6, 384, 12, 1536, 30522, 1229]
    tr = omb.Trainer("mlm", cfg, lr=1e-4, weight_decay=0.01, seed=0)
    losses = []
    for step in range(steps):
        if graph_at is not None and step == graph_at:
            tr.enable_graph()
        ids, pos, labels = synth.mlm_batch(64, 128, 30522, 1229, step)
        losses.append(np.float32(tr.step([ids, pos, labels])))
    named = tr.named_parameters()
    params = [tr.get_param(i, s) for i, (_, s) in enumerate(named)]
    tr.close()
    return np.array(losses), params


@pytest.mark.parametrize("tf32", [False, True])
def test_full_size_encoder_step_is_deterministic_and_graph_equals_eager(ctx, tf32):
    """Config 3 at its full size (6 x d384 h12 ff1536, seq 128, batch 64, vocab 30522, 1229 masked rows), where the
    oracle would take minutes per step: the size-independent properties. Two runs from the same seed give the same
    bits (fixed reduction orders, no float atomics), a run replayed from a captured graph gives the bits of the eager
    run, and the first loss is ln(vocab) to within the spread of the initial logits."""
    ctx.set_flags(omb.OM_TF32 if tf32 else 0)
    ctx.make_current()
    try:
        la, pa = _run_c3(4, None, tf32)
        lb, pb = _run_c3(4, None, tf32)
        lc, pc = _run_c3(4, 2, tf32)
        assert np.array_equal(la, lb) and np.array_equal(la, lc)
        for a, b, c in zip(pa, pb, pc):
            assert np.array_equal(a, b) and np.array_equal(a, c)
        assert abs(float(la[0]) - np.log(30522.0)) < 0.5
        assert np.all(np.isfinite(la))
    finally:
        ctx.set_flags(0)


def test_scheduling_flags_do_not_change_the_bits(ctx):
    """Config 3 at full size with overlapped launches (programmatic dependent launch), the two-stream linear backward and
    both together, eager and replayed from a captured graph: scheduling only, so the losses and every parameter after
    four steps equal the plain run bit for bit."""
    ctx.make_current()
    try:
        ctx.set_flags(omb.OM_TF32)
        la, pa = _run_c3(4, 2, True)
        for extra in (omb.OM_OVERLAP_LAUNCHES, omb.OM_TWO_STREAMS, omb.OM_OVERLAP_LAUNCHES | omb.OM_TWO_STREAMS):
            ctx.set_flags(omb.OM_TF32 | extra)
            for graph_at in (None, 2):
                lb, pb = _run_c3(4, graph_at, True)
                assert np.array_equal(la, lb), (extra, graph_at)
                for a, b in zip(pa, pb):
                    assert np.array_equal(a, b), (extra, graph_at)
    finally:
        ctx.set_flags(0)


def test_cnn_config_small(ctx, configs):
    """Config 2 at reduced size (conv + batch norm + ReLU x 4 with the strided stages, global average pool, linear; SGD
    momentum 0.9): per-parameter gradients after step 1 and the loss curve over 8 steps against the CPU path."""
    ctx.set_flags(0)
    ctx.make_current()
    batch, ch, strides = 8, [8, 8, 16, 16], [1, 1, 2, 1]
    cfg = [batch, 3, 16, 16, 10, len(ch)] + ch + strides
    tr = omb.Trainer("cnn", cfg, lr=0.05, weight_decay=0.0, seed=0)
    named = tr.named_parameters()
    weights = {n: tr.get_param(i, s) for i, (n, s) in enumerate(named)}
    running = {f"bn{i}": (np.zeros(c, np.float32), np.ones(c, np.float32)) for i, c in enumerate(ch)}
    state = {}
    for step in range(8):
        x, y = synth.cnn_batch(batch, 3, 16, 16, 10, step)
        lg = tr.step([x, y])
        lo, grads = configs.cnn_step(weights, running, x, y, strides, state, lr=0.05)
        assert abs(lg - lo) <= 1e-3 * abs(lo), step
        if step == 0:
            largest = max(np.max(np.abs(g)) for g in grads.values())
            for i, (n, s) in enumerate(named):
                gg = tr.get_grad(i, s)
                # A convolution bias in front of a batch norm has an exactly zero gradient; both sides hold rounding noise.
                if np.max(np.abs(grads[n])) < 1e-5 * largest:
                    assert np.max(np.abs(gg)) < 1e-5 * largest, n
                else:
                    assert scaled_diff(gg, grads[n]) <= 1e-4, n
    assert abs(lg - lo) <= 0.01 * abs(lo)
    tr.close()


@pytest.mark.parametrize("graph", [False, True])
def test_crnn_config_small(ctx, configs, graph):
    """Config 4 at reduced size (4 conv/pool stages to height 1, 2-layer BiLSTM, linear, log-softmax, CTC; Adam): gradients
    after step 1 and losses over 5 steps, eager and replayed from a captured graph."""
    ctx.set_flags(0)
    ctx.make_current()
    batch, height, width, classes, hidden, max_label = 4, 32, 48, 11, 8, 5
    cfg = [batch, height, width, classes, hidden, max_label, 4, 6, 8, 8]
    tr = omb.Trainer("crnn", cfg, lr=1e-3, weight_decay=0.0, seed=0)
    named = tr.named_parameters()
    weights = {n: tr.get_param(i, s) for i, (n, s) in enumerate(named)}
    state = {}
    for step in range(5):
        x, targets, lengths = synth.crnn_batch(batch, height, width, classes, max_label, 2, step)
        if graph and step == 1:
            tr.enable_graph()
        lg = tr.step([x, targets, lengths])
        lo, grads = configs.crnn_step(weights, x, targets[: int(lengths.sum())], lengths, step + 1, state)
        assert abs(lg - lo) <= 1e-4 * abs(lo), step
        if step == 0:
            for i, (n, s) in enumerate(named):
                assert scaled_diff(tr.get_grad(i, s), grads[n]) <= 1e-4, n
    tr.close()


def test_blocks_of_a_captured_step_are_not_handed_to_other_tensors(ctx):
    """A captured step writes to the pool blocks it was recorded with on every replay. Those blocks therefore stay with
    the graph: tensors allocated on the same context after the capture (an evaluation batch a user keeps, a second
    model) must never receive one of them. Tensors of every size class the step uses are created after the capture, the
    step is replayed, and their contents must be untouched."""
    ctx.set_flags(0)
    ctx.make_current()
    cfg = [4, 16, 2, 32, 4, 64, 101, 10]
    tr = omb.Trainer("mlm", cfg, lr=1e-3, weight_decay=0.01, seed=0)
    try:
        batches = [synth.mlm_batch(4, 16, 101, 10, s) for s in range(6)]
        for s in range(2):
            tr.step(list(batches[s]))
        tr.enable_graph()
        kept = []
        for n in (16, 64, 160, 256, 640, 1010, 1024, 2048, 3232, 4096, 6144, 8192, 16384):
            for copy in range(6):
                kept.append((omb.Tensor.from_numpy(np.full((n,), float(n + copy), np.float32)), float(n + copy)))
        losses = [tr.step(list(batches[s])) for s in range(2, 6)]
        assert np.all(np.isfinite(losses))
        for t, v in kept:
            assert np.all(t.numpy() == v), (t.shape, v)
    finally:
        tr.close()


@pytest.mark.parametrize("depth", [1, 2, 4])
def test_batches_staged_ahead_give_the_same_run(ctx, depth):
    """The loader's prefetch ring on the device (docs/data-loading.md section 1 of the reference: batches are delivered in
    step order whatever the prefetch depth): batches staged up to `depth` steps ahead on the copy stream, eager and replayed
    from a captured graph, give the losses and parameters of the plain step(batch) loop bit for bit; staging into a full
    ring and stepping on an empty one are refused."""
    ctx.set_flags(0)
    ctx.make_current()
    cfg = [4, 16, 2, 32, 4, 64, 101, 10]
    batches = [synth.mlm_batch(4, 16, 101, 10, s) for s in range(8)]

    def plain():
        tr = omb.Trainer("mlm", cfg, lr=1e-3, weight_decay=0.01, seed=0)
        losses = []
        for s, b in enumerate(batches):
            if s == 2:
                tr.enable_graph()
            losses.append(np.float32(tr.step(list(b))))
        params = [tr.get_param(i, sh) for i, (_, sh) in enumerate(tr.named_parameters())]
        tr.close()
        return losses, params

    def staged():
        tr = omb.Trainer("mlm", cfg, lr=1e-3, weight_decay=0.01, seed=0)
        tr.prefetch_depth(depth)
        with pytest.raises(omb.OmError):
            tr.step_prefetched()                       # nothing staged yet
        losses, nxt = [], 0
        for s in range(len(batches)):
            while nxt < len(batches) and nxt - s < depth:
                tr.prefetch(list(batches[nxt]))
                nxt += 1
            if s == 0 and nxt < len(batches):
                with pytest.raises(omb.OmError):
                    tr.prefetch(list(batches[nxt]))    # the ring is full
            if s == 2:
                tr.enable_graph()
            losses.append(np.float32(tr.step_prefetched()))
        params = [tr.get_param(i, sh) for i, (_, sh) in enumerate(tr.named_parameters())]
        tr.close()
        return losses, params

    la, pa = plain()
    lb, pb = staged()
    assert np.array_equal(np.array(la), np.array(lb))
    for a, b in zip(pa, pb):
        assert np.array_equal(a, b)


@pytest.mark.parametrize("graph", [False, True])
def test_bf16_copies_refreshed_by_the_optimizer_equal_a_fresh_cast(ctx, graph):
    """Under bfloat16 products AdamW refreshes the bfloat16 copies of the weights it updates in the same launch. A second run
    rewrites every parameter with its own value before each step, which marks the copies stale and has them cast afresh from
    the fp32 weights: the two runs give the same losses and the same parameters, bit for bit (eager and replayed)."""
    cfg = [2, 256, 2, 256, 4, 1024, 1000, 40]
    ctx.set_flags(omb.OM_TF32 | omb.OM_BF16_OPERANDS)
    ctx.make_current()
    try:
        runs = []
        for recast in (False, True):
            tr = omb.Trainer("mlm", cfg, lr=1e-3, weight_decay=0.01, seed=0)
            named = tr.named_parameters()
            losses = []
            for step in range(5):
                if graph and step == 2:
                    tr.enable_graph()
                if recast:
                    for i, (_, s) in enumerate(named):
                        tr.set_param(i, tr.get_param(i, s))
                losses.append(tr.step(list(synth.mlm_batch(cfg[0], cfg[1], cfg[6], cfg[7], step))))
            runs.append((losses, [tr.get_param(i, s) for i, (_, s) in enumerate(named)]))
            tr.close()
        assert runs[0][0] == runs[1][0]
        for a, b in zip(runs[0][1], runs[1][1]):
            assert np.array_equal(a, b)
        assert runs[0][0][0] != runs[0][0][4]
    finally:
        ctx.set_flags(0)
