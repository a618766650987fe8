"""Seeded synthetic batches for the benchmark configurations, generated on the host with the reference's own
generators so that the CPU baseline and the GPU see identical bits: SplitMix64 streams (SampleRng,
src/OneModel.Training/Data/SampleRng.cs:41-89 of the reference), the 12-uniform Irwin-Hall normal (SampleRng.cs:83-88),
multiply-high bounded integers (SampleRng.cs:58-74; the 2^-32-probability rejection step is omitted) and the keyed
Feistel permutation used to choose masked positions (SampleRng.cs:92-113)."""
import numpy as np

_M64 = (1 << 64) - 1
_GOLDEN = 0x9E3779B97F4A7C15


def _mix(z):
    z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
    z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
    return z ^ (z >> np.uint64(31))


def _mix_int(z):
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _M64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _M64
    return z ^ (z >> 31)


def derive(seed, a, b, c):
    """A stream key from (seed, epoch, step, rank): SampleRng.Derive folds each word through the mixer."""
    z = seed & _M64
    for w in (a, b, c):
        z = _mix_int((z + _GOLDEN + (w & _M64)) & _M64)
    return z


def stream(seed, n):
    """The first n outputs of the SplitMix64 stream with the given seed, as uint64."""
    with np.errstate(over="ignore"):
        idx = np.arange(1, n + 1, dtype=np.uint64)
        state = np.uint64(seed & _M64) + idx * np.uint64(_GOLDEN)
        return _mix(state)


def uniform01(seed, n):
    return (stream(seed, n) >> np.uint64(40)).astype(np.float32) * np.float32(1.0 / 16777216.0)


def normal(seed, shape):
    n = int(np.prod(shape))
    u = uniform01(seed, 12 * n).reshape(n, 12)
    s = np.zeros(n, np.float32)
    for i in range(12):          # float32 running sum in draw order, then - 6
        s = s + u[:, i]
    return (s - np.float32(6.0)).reshape(shape)


def uniform(seed, shape, low=0.0, high=1.0):
    n = int(np.prod(shape))
    return (np.float32(low) + (np.float32(high) - np.float32(low)) * uniform01(seed, n)).reshape(shape)


def integers(seed, shape, bound):
    n = int(np.prod(shape))
    x = stream(seed, n)
    b = np.uint64(bound)
    with np.errstate(over="ignore"):
        xh, xl = x >> np.uint64(32), x & np.uint64(0xFFFFFFFF)
        hi = (xh * b + ((xl * b) >> np.uint64(32))) >> np.uint64(32)
    return hi.astype(np.int64).reshape(shape)


def keyed_permutation(key, n, position):
    if n <= 1:
        return 0
    bits = (n - 1).bit_length()
    half = (bits + 1) // 2
    mask = (1 << half) - 1
    x = position
    while True:
        l, r = x >> half, x & mask
        for rnd in range(4):
            f = _mix_int(r ^ key ^ ((rnd * 0x632BE59BD9B4E019) & _M64)) & mask
            l, r = r, l ^ f
        x = (l << half) | r
        if x < n:
            return x


def masked_rows(seed, step, rank, total, count):
    """The first `count` outputs of the keyed permutation of [0, total), sorted ascending."""
    key = derive(seed, 0, step, rank)
    return np.sort(np.array([keyed_permutation(key, total, i) for i in range(count)], dtype=np.int64))


def mlm_batch(batch, seq, vocab, rows, step=0, rank=0):
    """Configs 3 and 5: token ids uniform in [0, vocab), 15% masked rows chosen by seed 3, labels = original ids."""
    ids = integers(derive(1, 0, step, rank), (batch, seq), vocab).astype(np.int32)
    pos = masked_rows(3, step, rank, batch * seq, rows).astype(np.int32)
    labels = ids.reshape(-1)[pos].astype(np.int64)
    return ids, pos, labels


def mlp_batch(batch, width, classes, step=0, rank=0):
    x = normal(derive(1, 0, step, rank), (batch, width))
    y = integers(derive(2, 0, step, rank), (batch,), classes)
    return x, y


def cnn_batch(batch, channels, height, width, classes, step=0, rank=0):
    """Config 2: images N(0,1), labels uniform in [0, classes)."""
    x = normal(derive(1, 0, step, rank), (batch, channels, height, width))
    y = integers(derive(2, 0, step, rank), (batch,), classes)
    return x, y


def crnn_batch(batch, height, width, classes, max_label, min_label=5, step=0, rank=0):
    """Config 4: grayscale images U(0,1); per image a label of length uniform in [min_label, max_label] of symbols uniform
    in [1, classes). Returns x, the concatenated labels padded with zeros to batch * max_label (int32), the lengths."""
    x = uniform(derive(1, 0, step, rank), (batch, 1, height, width))
    lengths = (integers(derive(2, 0, step, rank), (batch,), max_label - min_label + 1) + min_label).astype(np.int32)
    symbols = (integers(derive(2, 1, step, rank), (batch * max_label,), classes - 1) + 1).astype(np.int32)
    targets = np.zeros(batch * max_label, np.int32)
    total = int(lengths.sum())
    targets[:total] = symbols[:total]
    return x, targets, lengths
