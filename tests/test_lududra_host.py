"""Host-side logic of the sequence-model path (no GPU): container reader, configuration, distance buckets, the chunk
menu, the state pool's slot bookkeeping, sampling, and the lowering's shape on a stand-in for device memory."""
import json
import os

import numpy as np
import pytest

import lududra_reference as ref
from lududra_models import as_f64, attention_layer, bf16_exact, config, delta_layer, moe, random_weights


class FakeBuffer:
    """Stands in for DeviceBuffer: records what the pool does to it."""
    log = []

    def __init__(self, be, nbytes, zero=True):
        self.nbytes = (int(nbytes) + 15) & ~15
        self.elems = self.nbytes // 4
        self.ptr = 4096
        self.zeroed = []

    def upload(self, host, byte_offset=0):
        pass

    def fill_zero(self, off, n):
        self.zeroed.append((off, n))

    def free(self):
        self.ptr = None


@pytest.fixture
def fake_device(monkeypatch):
    import zgml_b200.host.state as S
    import zgml_b200.host.weights as Wt
    monkeypatch.setattr(Wt, "DeviceBuffer", FakeBuffer)
    monkeypatch.setattr(S, "DeviceBuffer", FakeBuffer)


def test_safetensors_round_trip(tmp_path):
    from zgml_b200.host.safetensors import SafetensorsFile, write_safetensors
    r = np.random.default_rng(0)
    a = r.standard_normal((5, 7)).astype(np.float32)
    t = {"a": a, "table": np.arange(6, dtype=np.int32).reshape(2, 3), "v": r.standard_normal(3).astype(np.float32)}
    p = os.path.join(tmp_path, "m.safetensors")
    write_safetensors(p, t)
    f = SafetensorsFile(p)
    assert sorted(f.names()) == ["a", "table", "v"] and f.shape("a") == (5, 7) and f.dtype("a") == "BF16" and f.dtype("table") == "I32"
    assert np.array_equal(f.f32("a"), bf16_exact(a))            # the writer rounds to nearest even like the tests' own rounding
    assert np.array_equal(f.raw("table"), t["table"])
    assert np.array_equal(f.bf16_bits("v"), (bf16_exact(t["v"]).view(np.uint32) >> 16).astype(np.uint16))
    write_safetensors(p, {"a": a}, bf16=False)
    assert np.array_equal(SafetensorsFile(p).f32("a"), a)


def test_safetensors_rejects_bad_files(tmp_path):
    from zgml_b200.host.safetensors import SafetensorsFile
    p = os.path.join(tmp_path, "bad.safetensors")
    hdr = json.dumps({"x": {"dtype": "BF16", "shape": [4], "data_offsets": [0, 800]}}).encode()
    with open(p, "wb") as f:
        f.write(len(hdr).to_bytes(8, "little") + hdr + b"\0" * 8)
    with pytest.raises(ValueError):
        SafetensorsFile(p)


@pytest.mark.parametrize("rows,bias_max", [(8, 32), (6, 9), (4, 3), (10, 20), (16, 128)])
def test_distance_buckets(rows, bias_max):
    from zgml_b200.host.lududra import distance_bias_table, distance_bucket
    b = [distance_bucket(n, rows, bias_max) for n in range(3 * bias_max + 12)]
    assert b == [ref.distance_bucket(n, rows, bias_max) for n in range(3 * bias_max + 12)]
    assert b[:rows // 2] == list(range(rows // 2)) and all(x <= y for x, y in zip(b, b[1:])) and b[-1] == rows - 1
    assert b[bias_max] == rows - 1
    rel = np.random.default_rng(1).standard_normal((rows, 3)).astype(np.float32)
    t = distance_bias_table(rel, 11, bias_max)
    assert t.shape == (11, 3) and all(np.array_equal(t[n], rel[b[n]]) for n in range(11))


def test_chunk_menu_and_cut():
    from zgml_b200.host.session import chunk_menu, cut
    assert chunk_menu(256) == [256, 128, 64, 32, 16, 8, 4, 2, 1] and chunk_menu(1) == [1] and chunk_menu(100)[0] == 64
    for n in (1, 2, 3, 255, 256, 257, 1126):
        c = cut(n, chunk_menu(256))
        assert sum(c) == n and c == sorted(c, reverse=True) and all(x in chunk_menu(256) for x in c)
    assert cut(0, chunk_menu(8)) == []


def test_config_reader_rejects_what_it_does_not_know():
    from zgml_b200.host.lududra import LududraConfig
    good = config([attention_layer(mlp=moe()), delta_layer()])
    c = LududraConfig.from_dict(good)
    assert c.vocab == 97 and c.width == 48 and len(c.layers) == 2 and c.layers[1]["mlp"] is None
    for edit in (lambda c: c.update(architecture="Other"), lambda c: c["layers"][0].update(type="rotary"),
                 lambda c: c["layers"][0]["mixer"].update(vdim=5), lambda c: c["layers"][0]["mixer"].update(kv_heads=3),
                 lambda c: c["layers"][0]["mlp"].update(kind="dense")):
        bad = json.loads(json.dumps(good))
        edit(bad)
        with pytest.raises(ValueError):
            LududraConfig.from_dict(bad)


def test_state_pool_slots(fake_device):
    from zgml_b200.host.state import SequenceStatePool, StateSpec
    pool = SequenceStatePool(None, [StateSpec("ring", 10, False), StateSpec("S", 6, True)], n_slots=2)
    a, b = pool.acquire("a"), pool.acquire("b")
    assert {a, b} == {0, 1} and pool.acquire("a") == a and pool.position("a") == 0
    pool.advance("a", 5)
    assert pool.position("a") == 5 and pool.position("b") == 0
    with pytest.raises(RuntimeError):
        pool.acquire("c")
    pool.release("a")
    assert not pool.has("a") and pool.acquire("c") == a and pool.position("c") == 0
    S, ring = pool.buffers["S"], pool.buffers["ring"]
    assert S.zeroed[-1] == (4 * 6 * a, 4 * 6)              # the reused slot's recurrent state was cleared, and only that slot's
    assert all(z == (0, ring.nbytes) for z in ring.zeroed)  # the ring is masked by position: cleared once, at allocation
    pool.release("never-seen")                             # releasing an unknown request is a no-op
    assert pool.bytes() == S.nbytes + ring.nbytes


def test_sampler():
    from zgml_b200.host.sampling import Sampler
    z = np.array([0.1, 3.0, 3.0, -1.0])
    assert Sampler()(z) == 1                                # greedy: lowest index among equal maxima
    assert all(Sampler(1.0, top_k=1, seed=s)(np.array([0.0, 5.0, 1.0])) == 1 for s in range(5))
    draws = [Sampler(1.0, top_p=0.5, seed=s)(np.array([0.0, 5.0, 4.9, -9.0])) for s in range(40)]
    assert set(draws) <= {1, 2} and Sampler(0.7, seed=3)(z) == Sampler(0.7, seed=3)(z)


def test_lowering_shape(fake_device):
    from zgml_b200 import abi
    from zgml_b200.host.lududra import LududraConfig, LududraModel
    from zgml_b200.host.state import SequenceStatePool
    cfg = config([delta_layer(mlp=moe()), attention_layer(window=8), delta_layer(conv=1)])
    W = random_weights(cfg)
    m = LududraModel(None, LududraConfig.from_dict(cfg), lambda n: W[n], "bfloat16")
    specs = m.state_specs(16)
    assert [s.name for s in specs] == ["l0.S", "l0.tail", "l1.ring", "l2.S"]       # a one-tap convolution carries nothing
    assert specs[2].elems == (8 - 1 + 16) * 2 * 16 and not specs[2].zero_on_acquire and specs[0].zero_on_acquire
    pool = SequenceStatePool(None, specs, 3)
    for T, head, rows in ((1, "last", 1), (16, "all", 16), (4, "none", 0), (8, "last", 1)):
        lp = m.lower(T, head, pool)
        tags = [op.tag for op in lp.program.ops]
        assert tags[0] == abi.OP_EMBED and lp.logits_rows == rows and (lp.buf_logits is None) == (head == "none")
        assert tags.count(abi.OP_DELTA_RULE) == 2 and tags.count(abi.OP_WINDOW_ATTENTION) == 1 and tags.count(abi.OP_MOE_FFN) == 1
        # the first norm stands alone; each of the four closing norms carries the norm that follows it, if one does
        norms = [op for op in lp.program.ops if op.tag == abi.OP_NORM]
        assert tags.count(abi.OP_CAUSAL_CONV) == 2 and len(norms) == 1 + 4
        assert sum(op.u.seq.buf[4] != abi.NO_BUF for op in norms) == 3 + (head != "none")
        ext = {e.buf_idx for e in lp.program.externs}
        assert len(ext) == len(lp.program.externs) == 4 + 4   # weight arenas + state buffers, each once
        assert all(lp.program.buffer_sizes[e.buf_idx] == e.buffer.elems for e in lp.program.externs)
    with pytest.raises(AssertionError):
        m.lower(32, "none", pool)                            # a chunk longer than the ring was sized for


def test_reference_is_causal_and_windowed():
    """The restatement the GPU tests lean on: a prefix's logits do not depend on what follows, and a key outside the window
    does not matter while one just inside does."""
    cfg = config([attention_layer(window=4, mlp=moe()), delta_layer()])
    W = as_f64(random_weights(cfg, seed=3, qk_gain=6.0))
    toks = np.random.default_rng(0).integers(0, cfg["vocab"], 12).tolist()
    full, _ = ref.forward(cfg, W, toks)
    assert np.allclose(ref.forward(cfg, W, toks[:7])[0], full[:7], atol=1e-12)
    only_attn = config([attention_layer(window=4)])
    Wa = as_f64(random_weights(only_attn, seed=4, qk_gain=6.0))
    base = ref.forward(only_attn, Wa, toks)[0][-1]
    far, near = list(toks), list(toks)
    far[-5] = (far[-5] + 1) % cfg["vocab"]      # distance 4: outside a window of 4
    near[-4] = (near[-4] + 1) % cfg["vocab"]    # distance 3: the last one inside
    assert np.allclose(ref.forward(only_attn, Wa, far)[0][-1], base, atol=1e-12)
    assert np.abs(ref.forward(only_attn, Wa, near)[0][-1] - base).max() > 1e-3
