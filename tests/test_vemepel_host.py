"""Host side of Vemepel without a GPU: configuration errors, state sizing, the shape of the lowering on a fake device, and
properties of the float64 restatement that the GPU tests lean on (causality, block masks, rotation, routing)."""
import json

import numpy as np
import pytest

import vemepel_reference as ref
from vemepel_models import as_f64, config, dense, diff_layer, latent2_layer, latent_layer, moe, random_weights


class FakeBuffer:
    def __init__(self, be, nbytes, zero=True):
        self.nbytes = (int(nbytes) + 15) & ~15
        self.elems = self.nbytes // 4
        self.zeroed = [(0, self.nbytes)] if zero else []

    def upload(self, host, byte_offset=0):
        pass

    def fill_zero(self, byte_offset, nbytes):
        self.zeroed.append((byte_offset, nbytes))

    def free(self):
        pass


@pytest.fixture
def fake_device(monkeypatch):
    import zgml_b200.host.state as S
    import zgml_b200.host.weights as Wt
    monkeypatch.setattr(Wt, "DeviceBuffer", FakeBuffer)
    monkeypatch.setattr(S, "DeviceBuffer", FakeBuffer)


STACK = config([diff_layer(block=7, mlp=dense()), latent2_layer(mlp=moe()), latent_layer(), diff_layer(kv_from=0, block=20, mlp=moe(top=1))])


def test_config_errors():
    from zgml_b200.host.vemepel import VemepelConfig
    VemepelConfig.from_dict(STACK)
    bad = json.loads(json.dumps(STACK))
    bad["architecture"] = "Other"
    with pytest.raises(ValueError):
        VemepelConfig.from_dict(bad)
    for mutate in (lambda c: c["layers"][0].__setitem__("type", "recurrent"),
                   lambda c: c["layers"][0]["mixer"].__setitem__("kv_heads", 3),
                   lambda c: c["layers"][3]["mixer"].__setitem__("kv_from", 2),          # not an attention layer
                   lambda c: c["layers"][3]["mixer"].__setitem__("kv_from", 3),          # itself
                   lambda c: c["layers"][3]["mixer"].__setitem__("vdim", 5),             # not the owner's value size
                   lambda c: c["layers"][1]["mixer"]["rot"].__setitem__("dims", 4),
                   lambda c: c["layers"][1]["mlp"]["router"].__setitem__("top", 9),
                   lambda c: c["layers"][0]["mlp"].__setitem__("kind", "conv")):
        bad = json.loads(json.dumps(STACK))
        mutate(bad)
        with pytest.raises(ValueError):
            VemepelConfig.from_dict(bad)


def test_state_and_lowering_shape(fake_device):
    from zgml_b200 import abi
    from zgml_b200.host.state import SequenceStatePool
    from zgml_b200.host.vemepel import VemepelConfig, VemepelModel
    W = random_weights(STACK)
    m = VemepelModel(None, VemepelConfig.from_dict(STACK), lambda n: W[n], "bfloat16")
    specs = {s.name: s for s in m.state_specs(16, 100)}
    assert list(specs) == ["l0.shift", "l0.kv", "l1.shift", "l1.latent", "l2.shift", "l2.latent", "l3.shift"]   # the borrower owns no cache
    assert specs["l0.kv"].elems == (20 - 1 + 16) * 2 * (2 * 8 + 12)      # the owner's cache reaches as far back as its borrower's blocks
    assert specs["l1.latent"].elems == 100 * (12 + 6) and specs["l2.latent"].elems == 100 * 14
    assert specs["l0.shift"].zero_on_acquire and not specs["l0.kv"].zero_on_acquire
    assert {s.name: s.elems for s in m.state_specs(16, 30)}["l0.kv"] == 30 * 2 * (2 * 8 + 12)    # never more than one row per position
    pool = SequenceStatePool(None, list(specs.values()), 2)
    for T, head, rows in ((1, "last", 1), (16, "all", 16), (4, "none", 0)):
        lp = m.lower(T, head, pool)
        tags = [op.tag for op in lp.program.ops]
        assert tags[0] == abi.OP_EMBED and lp.logits_rows == rows and (lp.buf_logits is None) == (head == "none")
        assert tags.count(abi.OP_CACHED_ATTENTION) == 4 and tags.count(abi.OP_CACHE_APPEND) == 3 and tags.count(abi.OP_MAP_COMBINE) == 2
        assert tags.count(abi.OP_HEAD_LINEAR) == 4 and tags.count(abi.OP_ROTARY) == 1 and tags.count(abi.OP_GATE) == 0     # gates ride in the value products
        # the depth average rides in the norm that opens the next layer (and in the head's norm): no launch of its own
        averaged = [op for op in lp.program.ops if op.tag == abi.OP_NORM and op.u.seq.n[5]]
        assert tags.count(abi.OP_DEPTH_MIX) == 0 and [op.u.seq.n[5] for op in averaged] == [2, 3, 4] + ([5] if head != "none" else [])
        assert tags.count(abi.OP_POLY_NORM) == 1 and tags.count(abi.OP_MOE_FFN) == 2
        assert tags.count(abi.OP_TOKEN_SHIFT) == (0 if T == 1 else 4)     # single-token steps shift inside the opening norm
        ext = [e.buf_idx for e in lp.program.externs]
        assert len(set(ext)) == len(ext) == 5 + 7                           # weight arenas + state buffers, each once
        both = [op for op in lp.program.ops if op.tag == abi.OP_CACHED_ATTENTION and op.u.seq.n[3] == 2]
        assert both[0].u.seq.buf[2] == both[1].u.seq.buf[2]                 # the borrower reads the owner's cache buffer
        assert [op.u.seq.off[4] for op in both] == [7, 20]


def test_reference_masks_and_causality():
    toks = np.random.default_rng(0).integers(0, STACK["vocab"], 30).tolist()
    W = as_f64(random_weights(STACK, seed=3, qk_gain=4.0))
    full = ref.forward(STACK, W, toks)
    assert np.allclose(ref.forward(STACK, W, toks[:17]), full[:17], atol=1e-11)
    vis = ref.chunk_mask(10, 4)
    assert vis[5, 4] and vis[5, 5] and not vis[5, 3] and not vis[5, 6] and vis[3, 0] and not vis[4, 3]


def test_reference_rotation():
    x = np.random.default_rng(1).standard_normal((5, 2, 8))
    pos = np.arange(5)
    y = ref.rotate_interleaved(x, pos, 6, 100.0)
    assert np.allclose(y[0], x[0]) and np.allclose(y[..., 6:], x[..., 6:])
    assert np.allclose(np.hypot(y[..., 0], y[..., 1]), np.hypot(x[..., 0], x[..., 1]))
    a = 3 * 100.0 ** (-2.0 / 6)                                            # position 3, pair 1
    assert np.allclose(y[3, 1, 2], x[3, 1, 2] * np.cos(a) - x[3, 1, 3] * np.sin(a))
    # a score between rotated vectors depends on the distance alone
    q, k = x[0, 0, :6], x[0, 1, :6]
    def score(pq, pk):
        return ref.rotate_interleaved(q[None, None], np.array([pq]), 6, 100.0).ravel() @ ref.rotate_interleaved(k[None, None], np.array([pk]), 6, 100.0).ravel()
    assert np.isclose(score(9, 4), score(25, 20))


def test_reference_routing_and_lambda():
    idx, w = ref.route_top(np.array([[0.5, 2.0, 2.0, -1.0]]), 2)
    assert idx.tolist() == [[1, 2]] and np.allclose(w, [[0.5, 0.5]])
    idx, w = ref.route_top(np.array([[0.0, 3.0, 1.0]]), 1)
    assert idx.tolist() == [[1]] and np.allclose(w, [[1.0]])
    from zgml_b200.host.vemepel import differential_lambda
    r = np.random.default_rng(2)
    v = [r.standard_normal(8).astype(np.float32) * 0.3 for _ in range(4)]
    want = np.exp(v[0].astype(np.float64) @ v[1]) - np.exp(v[2].astype(np.float64) @ v[3]) + 0.3
    assert abs(differential_lambda(*v, 0.3) - want) < 1e-6
    W = {"p.lq1": v[0], "p.lk1": v[1], "p.lq2": v[2], "p.lk2": v[3]}
    assert np.isclose(ref.differential_lambda(W, "p.", 0.3), want)


def test_poly_norm_restatement():
    z = np.array([[1.0, -2.0, 0.5, 3.0]])
    got = ref.poly_norm(z, [1.0, 0.0, 0.0, 0.25], 0.0)
    assert np.allclose(got, z / np.sqrt(np.mean(z ** 2)) + 0.25)
    got = ref.poly_norm(z, [0.0, 2.0, -1.0, 0.0], 0.0)
    assert np.allclose(got, 2 * z ** 2 / np.sqrt(np.mean(z ** 4)) - z ** 3 / np.sqrt(np.mean(z ** 6)))
