"""Cache-attention DeviceOps alone, in one-op programs against NumPy: the parameter values no model of the framework uses yet
(sliding-window mask over a ring that wraps, rotary pairs (i, i + dims / 2), the stand-alone gate and depth average) and
the static checks that refuse a malformed op at compile time."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def run(be, ops, sizes, inputs, out_buf, out_shape, externs=()):
    from zgml_b200 import DeviceProgram, ProgramIO
    prog = DeviceProgram(list(ops), list(sizes), [], [], list(externs))
    h = be.compile_program(prog)
    assert h is not None
    got = np.zeros(out_shape, np.float32)
    be.execute_program(h, [ProgramIO(i, np.ascontiguousarray(a, dtype=np.float32).ravel()) for i, a in inputs], [ProgramIO(out_buf, got)])
    be.free_program(h)
    return got


def ctl_words(pos, slot, n=8):
    c = np.zeros(n, np.int32)
    c[0], c[1] = pos, slot
    return c.view(np.float32)


@pytest.mark.parametrize("dims", [(2, 1, 8, 12, 5), (4, 2, 64, 32, 40), (3, 3, 7, 5, 3)], ids=["small", "aligned-long-window", "odd"])
def test_sliding_window_over_a_wrapping_ring(cuda_backend, dims):
    """Mask kind 1: every query sees the last `window` positions.  The ring has window - 1 + T rows, so the 70 positions fed in
    steps of T wrap it several times; appended by CACHE_APPEND, read by CACHED_ATTENTION."""
    from zgml_b200 import DeviceBuffer, DeviceOp, ExternBuffer
    H, G, dk, dv, window = dims
    T, n = 10, 70
    R, width = window - 1 + T, G * (dk + dv)
    r = np.random.default_rng(sum(dims))
    q = r.standard_normal((n, H, dk)).astype(np.float32) * 1.5
    kv = r.standard_normal((n, width)).astype(np.float32)
    ring = DeviceBuffer(cuda_backend, 4 * 2 * R * width)                  # two slots; slot 1 is used
    ops = [DeviceOp.cache_append(3, 1, 2, 0, 0, T, width, width, width, R),
           DeviceOp.cached_attention(4, 0, 3, 3, 2, 0, 0, G * dk, T, H, G, 1, dk, dv, H * dk, width, width, R, 0.3, mask="window", mask_size=window)]
    sizes = [T * H * dk, T * width, 8 + T, ring.elems, T * H * dv]
    got = []
    for at in range(0, n, T):
        got.append(run(cuda_backend, ops, sizes, [(0, q[at:at + T]), (1, kv[at:at + T]), (2, ctl_words(at, 1, 8 + T))], 4, (T, H, dv), [ExternBuffer(3, ring)]))
    got = np.concatenate(got)
    k, v = kv[:, :G * dk].reshape(n, G, dk).astype(np.float64), kv[:, G * dk:].reshape(n, G, dv).astype(np.float64)
    for p in range(n):
        lo = max(0, p + 1 - window)
        for h in range(H):
            g = h // (H // G)
            s = (k[lo:p + 1, g] @ q[p, h].astype(np.float64)) * 0.3
            w = np.exp(s - s.max())
            want = (w / w.sum()) @ v[lo:p + 1, g]
            assert np.abs(got[p, h] - want).max() < 2e-5 * max(1.0, np.abs(want).max()), (p, h)
    ring.free()


@pytest.mark.parametrize("layout", ["pairs", "halves"])
def test_rotary_layouts(cuda_backend, layout):
    from zgml_b200 import DeviceOp
    T, heads, hs, dims, base, pos = 5, 3, 12, 8, 700.0, 37
    x = np.random.default_rng(3).standard_normal((T, heads * hs + 4)).astype(np.float32)
    got = run(cuda_backend, [DeviceOp.rotary(0, 1, 4, T, heads, hs, heads * hs + 4, dims, base, layout=layout)], [x.size, 8],
              [(0, x), (1, ctl_words(pos, 0))], 0, x.shape)
    want = x.astype(np.float64).copy()
    for t in range(T):
        for h in range(heads):
            v = x[t, 4 + h * hs: 4 + h * hs + dims].astype(np.float64)
            for i in range(dims // 2):
                a, b = (2 * i, 2 * i + 1) if layout == "pairs" else (i, i + dims // 2)
                ang = (pos + t) * base ** (-2.0 * i / dims)
                want[t, 4 + h * hs + a] = v[a] * np.cos(ang) - v[b] * np.sin(ang)
                want[t, 4 + h * hs + b] = v[b] * np.cos(ang) + v[a] * np.sin(ang)
    assert np.abs(got - want).max() < 5e-5                                 # f32 angles at position 41
    assert np.array_equal(got[:, :4], x[:, :4]) and np.array_equal(got[:, 4 + dims:4 + hs], x[:, 4 + dims:4 + hs])


def test_gate_and_depth_mix_alone(cuda_backend):
    from zgml_b200 import DeviceBuffer, DeviceOp, ExternBuffer, abi
    r = np.random.default_rng(4)
    T, cols, group = 6, 24, 8
    x, g = r.standard_normal((T, cols)).astype(np.float32), r.standard_normal((T, 5 + cols // group)).astype(np.float32)
    got = run(cuda_backend, [DeviceOp.gate(0, 1, 5, T, cols, group, 5 + cols // group)], [x.size, g.size], [(0, x), (1, g)], 0, x.shape)
    want = x * (1.0 / (1.0 + np.exp(-g[:, 5:].astype(np.float64)))).repeat(group, axis=1)
    assert np.abs(got - want).max() < 1e-6
    hist, coeff = r.standard_normal((4, 50)).astype(np.float32), np.array([0.5, -1.0, 0.0, 2.0], np.float32)
    w = DeviceBuffer(cuda_backend, 4 * 8, zero=False)
    w.upload(np.concatenate([np.zeros(4, np.float32), coeff]))
    got = run(cuda_backend, [DeviceOp.depth_mix(0, 1, 2, 4, 50, 4, 50, abi.W_F32)], [50, 200, w.elems], [(1, hist)], 0, (50,), [ExternBuffer(2, w)])
    assert np.abs(got - coeff.astype(np.float64) @ hist).max() < 1e-6
    w.free()


def test_malformed_ops_are_refused(cuda_backend):
    from zgml_b200 import DeviceOp, DeviceProgram
    bad = [
        (DeviceOp.cached_attention(0, 1, 2, 2, 3, 0, 0, 0, 4, 3, 2, 1, 8, 8, 24, 16, 16, 16, 1.0), [96, 96, 256, 16]),            # heads not a multiple of key heads
        (DeviceOp.cached_attention(0, 1, 2, 2, 3, 0, 0, 0, 4, 2, 2, 1, 8, 8, 16, 16, 16, 2, 1.0), [64, 64, 32, 16]),              # fewer cache rows than the step has tokens
        (DeviceOp.cached_attention(0, 1, 2, 2, 3, 0, 0, 12, 4, 2, 2, 1, 8, 8, 16, 16, 16, 8, 1.0), [64, 64, 128, 16]),            # value columns leave the cache row
        (DeviceOp.rotary(0, 1, 0, 2, 2, 6, 12, 7, 100.0), [24, 8]),                                                                # odd number of rotated dims
        (DeviceOp.cache_append(0, 1, 2, 0, 0, 4, 8, 8, 8, 16, normed=6, rot=4), [128, 32, 16]),                                     # normed + rotated exceed the row
        (DeviceOp.head_linear(0, 0, 1, 0, 2, 2, 4, 4, 0), [16, 32]),                                                               # in place
        (DeviceOp.token_shift(0, 0, 1, 0, 2, 3, 2, 4, 0), [8, 4, 4, 16]),                                                          # in place
    ]
    for op, sizes in bad:
        assert cuda_backend.compile_program(DeviceProgram([op], sizes, [], [], [])) is None
