"""Lududra on the CUDA backend against the float64 restatement (tests/lududra_reference.py): every mechanism alone,
whole prompts, token-by-token decoding through the carried state, prompts cut into portions, interleaved requests in
several state slots, slot reuse, long decoding across many turns of the key ring, shapes of many kinds, and greedy
generation through the registry's entry point."""
import json
import os

import numpy as np
import pytest

import lududra_reference as ref
from lududra_models import as_f64, attention_layer, config, delta_layer, moe, random_weights

pytestmark = pytest.mark.gpu

TOL = 2e-4   # of the logits' scale; f32 accumulation against float64


def tol(dtype):
    """A bfloat16 session rounds the activations that enter a tensor-core matmul (steps of more than 8 tokens) to bf16."""
    return TOL if dtype == "float32" else 3e-2


def open_model(be, cfg, W, dtype="float32", n_slots=1, max_chunk=16, keep_layers=False):
    from zgml_b200.host.lududra import LududraConfig, LududraModel
    from zgml_b200.host.session import SequenceSession
    model = LududraModel(be, LududraConfig.from_dict(cfg), lambda n: W[n], dtype)
    return SequenceSession(be, model, n_slots=n_slots, max_chunk=max_chunk, keep_layers=keep_layers)


def close(s):
    s.close()
    s.model.close()


def rel(got, want):
    return float(np.max(np.abs(got.astype(np.float64) - want)) / (np.max(np.abs(want)) + 1e-30))


def tokens(cfg, n, seed=1):
    return np.random.default_rng(seed).integers(0, cfg["vocab"], n).tolist()


MIXED = config([delta_layer(mlp=moe()), attention_layer(mlp=moe(experts=5, identity=2, top=3)), delta_layer(heads=2, kv_heads=2, dim=8, vdim=8, conv=2),
                attention_layer(heads=2, kv_heads=1, dim=24, window=5, rel_rows=6, bias_max=9, softcap=4.0)])


# ── each mechanism alone (a one-layer model without a feed-forward isolates its mixer) ──
@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
@pytest.mark.parametrize("layer", [
    attention_layer(),
    attention_layer(heads=3, kv_heads=3, dim=40, window=3, rel_rows=4, bias_max=3),      # window shorter than the table's linear half
    attention_layer(heads=6, kv_heads=1, dim=8, window=33, rel_rows=10, bias_max=20, softcap=2.0),   # window crosses the 32-key block
    delta_layer(),
    delta_layer(heads=3, kv_heads=1, dim=40, vdim=10, conv=4, rank_a=3, rank_g=5),        # padded key rows, several row slices
    delta_layer(heads=2, kv_heads=2, dim=8, vdim=70, conv=1),                            # no carried inputs; columns over two CTAs
    delta_layer(heads=1, kv_heads=1, dim=130, vdim=12, conv=2),                          # sixteen row slices
], ids=["attn", "attn-short-window", "attn-33", "delta", "delta-odd", "delta-notail", "delta-wide-key"])
def test_mixer_alone(cuda_backend, layer, dtype):
    cfg = config([layer], width=40, vocab=61)
    W = random_weights(cfg, seed=5, qk_gain=4.0)
    toks = tokens(cfg, 45)
    want, stream = ref.forward(cfg, as_f64(W), toks)
    s = open_model(cuda_backend, cfg, W, dtype, max_chunk=64, keep_layers=True)
    got = s.feed("a", toks, range(45))
    assert rel(got, want) < tol(dtype)
    close(s)


@pytest.mark.parametrize("mlp", [moe(), moe(experts=3, identity=0, top=1, ff=7, limit=0.5), moe(experts=2, identity=3, top=4, ff=40),
                                 moe(experts=9, identity=1, top=2, ff=16, limit=100.0)],
                         ids=["moe", "top1-no-identity", "mostly-identity", "unclamped"])
def test_feed_forward(cuda_backend, mlp):
    """The residual after the layer is compared too, so a fault in routing, clamping or the identity experts cannot hide
    behind the final norm."""
    cfg = config([attention_layer(heads=2, kv_heads=2, dim=8, window=4, mlp=mlp)], width=36, vocab=50)
    W = random_weights(cfg, seed=9)
    toks = tokens(cfg, 19)
    want, stream = ref.forward(cfg, as_f64(W), toks)
    s = open_model(cuda_backend, cfg, W, "float32", max_chunk=32, keep_layers=True)
    got = s.feed("a", toks[:16], range(16))
    layers = s.layer_streams(16, "all")
    assert rel(layers[0], stream[0][:16]) < TOL
    assert rel(got, want[:16]) < TOL
    close(s)


def test_layer_streams_of_a_mixed_stack(cuda_backend):
    W = random_weights(MIXED, seed=2)
    toks = tokens(MIXED, 16)
    want, stream = ref.forward(MIXED, as_f64(W), toks)
    s = open_model(cuda_backend, MIXED, W, "float32", keep_layers=True)
    got = s.feed("a", toks, range(16))
    layers = s.layer_streams(16, "all")
    for i in range(len(MIXED["layers"])):
        assert rel(layers[i], stream[i]) < TOL, f"layer {i}"
    assert rel(got, want) < TOL
    close(s)


# ── prefill against decoding, portions, first tokens ──
@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_prefill_equals_token_by_token(cuda_backend, dtype):
    W = random_weights(MIXED, seed=3, qk_gain=3.0)
    toks = tokens(MIXED, 40)
    want, _ = ref.forward(MIXED, as_f64(W), toks)
    s = open_model(cuda_backend, MIXED, W, dtype, n_slots=2)
    whole = s.feed("whole", toks, range(40))
    single = np.concatenate([s.feed("single", [t], [0]) for t in toks])
    assert rel(whole, want) < tol(dtype) and rel(single, want) < TOL     # single tokens take the exact row kernels in both formats
    assert rel(whole[:3], want[:3]) < tol(dtype)   # the first tokens see zeros before the start, not a stale tail or ring
    close(s)


@pytest.mark.parametrize("cuts", [[2, 2, 2, 30, 3, 2, 9], [1, 16, 1, 15, 17], [7, 7, 7, 7, 7, 7, 8], [50]])
def test_portions(cuda_backend, cuts):
    W = random_weights(MIXED, seed=4, qk_gain=3.0)
    toks = tokens(MIXED, 50)
    want, _ = ref.forward(MIXED, as_f64(W), toks)
    s = open_model(cuda_backend, MIXED, W, max_chunk=16)
    got, at = [], 0
    for c in cuts:
        got.append(s.feed("r", toks[at:at + c], range(c)))
        at += c
    assert rel(np.concatenate(got), want) < TOL
    close(s)


# ── window edges, in prompts and in decoding, with a peaky softmax ──
@pytest.mark.parametrize("window", [1, 2, 7, 16, 17])
def test_window_edges(cuda_backend, window):
    cfg = config([attention_layer(heads=2, kv_heads=1, dim=16, window=window, rel_rows=6, bias_max=12, softcap=60.0)], width=32, vocab=40)
    W = random_weights(cfg, seed=window, qk_gain=12.0)
    toks = tokens(cfg, 3 * window + 9)
    n = len(toks)
    want, _ = ref.forward(cfg, as_f64(W), toks)
    # the weights are peaky enough that one key more or less is far outside the tolerance
    wider = json.loads(json.dumps(cfg))
    wider["layers"][0]["mixer"]["mask"]["size"] = window + 1
    assert rel(ref.forward(wider, as_f64(W), toks)[0], want) > 50 * TOL
    s = open_model(cuda_backend, cfg, W, n_slots=2, max_chunk=8)
    assert rel(s.feed("prompt", toks, range(n)), want) < TOL
    half = n // 2
    got = [s.feed("decode", toks[:half], range(half))] + [s.feed("decode", [t], [0]) for t in toks[half:]]
    assert rel(np.concatenate(got), want) < TOL
    close(s)


def test_sink_matters_and_is_there(cuda_backend):
    """Negative scores everywhere: the sink takes most of the weight, so leaving it out would change the output a lot."""
    cfg = config([attention_layer(heads=2, kv_heads=2, dim=8, window=6, softcap=1e4)], width=24, vocab=30)
    W = random_weights(cfg, seed=11, qk_gain=0.0)          # q = q.b, k = k.b: all scores equal q.b . k.b
    W["l0.mix.q.b"] = np.abs(W["l0.mix.q.b"]) * 4
    W["l0.mix.k.b"] = -np.abs(W["l0.mix.k.b"]) * 4
    W["l0.mix.rel"] = np.zeros_like(W["l0.mix.rel"])
    toks = tokens(cfg, 12)
    want, _ = ref.forward(cfg, as_f64(W), toks)
    s = open_model(cuda_backend, cfg, W, "float32")
    assert rel(s.feed("a", toks, range(12)), want) < TOL
    close(s)


# ── batches of unequal requests, slots freed and used again ──
def test_interleaved_requests_and_slot_reuse(cuda_backend):
    W = random_weights(MIXED, seed=6)
    A, B, C = tokens(MIXED, 30, 1), tokens(MIXED, 11, 2), tokens(MIXED, 23, 3)
    wa, wb, wc = (ref.forward(MIXED, as_f64(W), t)[0] for t in (A, B, C))
    s = open_model(cuda_backend, MIXED, W, n_slots=2, max_chunk=8)
    ga, gb = [], []
    r = s.step([{"id": "a", "tokens": A[:9], "want": range(9)}, {"id": "b", "tokens": B[:2], "want": range(2)}])
    ga.append(r[0]), gb.append(r[1])
    r = s.step([{"id": "b", "tokens": B[2:], "want": range(9)}, {"id": "a", "tokens": A[9:10], "want": [0]}], end=["b"])
    gb.append(r[0]), ga.append(r[1])
    with pytest.raises(KeyError):
        s.pool.slot("b")
    # c takes b's slot: nothing of b's recurrent state, convolution tail or keys may show
    r = s.step([{"id": "c", "tokens": C, "want": range(23)}, {"id": "a", "tokens": A[10:], "want": range(20)}], end=["a", "c"])
    ga.append(r[1])
    assert rel(np.concatenate(ga), wa) < TOL and rel(np.concatenate(gb), wb) < TOL and rel(r[0], wc) < TOL
    with pytest.raises(RuntimeError):
        s.step([{"id": i, "tokens": [1], "want": []} for i in "xyz"])   # more live requests than slots
    close(s)


def test_long_decoding_turns_the_ring_many_times(cuda_backend):
    cfg = config([attention_layer(heads=2, kv_heads=1, dim=16, window=9, mlp=moe()), delta_layer(mlp=None)], width=32, vocab=64)
    W = random_weights(cfg, seed=8, qk_gain=3.0)
    toks = tokens(cfg, 150)
    want, _ = ref.forward(cfg, as_f64(W), toks)
    s = open_model(cuda_backend, cfg, W, max_chunk=4)      # ring of 12 rows
    got = [s.feed("r", toks[:6], range(6))] + [s.feed("r", [t], [0]) for t in toks[6:]]
    assert rel(np.concatenate(got), want) < 2 * TOL
    close(s)


# ── the entry point a user calls ──
def test_registry_loads_a_folder_and_generates_greedily(cuda_backend, tmp_path):
    from zgml_b200.host.registry import open_session
    from zgml_b200.host.safetensors import write_safetensors
    W = random_weights(MIXED, seed=12)
    public = json.loads(json.dumps(MIXED))
    for L in public["layers"]:
        L["mixer"] = {k: v for k, v in L["mixer"].items() if not k.startswith("_")}
    with open(os.path.join(tmp_path, "config.json"), "w") as f:
        json.dump(public, f)
    write_safetensors(os.path.join(tmp_path, "model.safetensors"), W)
    prompt = tokens(MIXED, 13)
    seq = list(prompt)
    for _ in range(10):
        seq.append(int(np.argmax(ref.forward(MIXED, as_f64(W), seq)[0][-1])))
    for dtype in ("bfloat16", "float32"):
        s = open_session(cuda_backend, str(tmp_path), dtype, max_chunk=8)
        assert s.generate(prompt, 10) == seq[13:]
        assert s.pool.live() == []
        close(s)


# ── the tensor-core prefill matmul (bfloat16 sessions, more than 8 rows) ──
@pytest.mark.parametrize("M,N,K,bias", [(128, 128, 64, False), (200, 300, 136, True), (9, 64, 72, True), (300, 72, 520, False)])
def test_dense_tensor_core_linear_alone(cuda_backend, M, N, K, bias):
    """One LINEAR op over bfloat16 weights: equal to the float64 product of the bf16-rounded activations (the only rounding
    the tensor path adds), including ragged tile edges in M, N and K and a strided source."""
    from lududra_models import bf16_exact
    from zgml_b200 import DeviceBuffer, DeviceOp, DeviceProgram, ExternBuffer, ProgramIO, abi
    from zgml_b200.host.safetensors import f32_to_bf16_bits
    r = np.random.default_rng(M + N + K)
    W, b = bf16_exact(r.standard_normal((N, K)).astype(np.float32)), bf16_exact(r.standard_normal(N).astype(np.float32))
    x = r.standard_normal((M, K + 8)).astype(np.float32)
    arena = np.concatenate([W.ravel(), b])
    buf = DeviceBuffer(cuda_backend, 2 * arena.size, zero=False)
    buf.upload(f32_to_bf16_bits(arena))
    op = DeviceOp.linear(1, 0, 2, 0, M, N, K, abi.W_BF16, bias=2 if bias else None, bias_off=N * K, src_off=8, src_rs=K + 8)
    prog = DeviceProgram([op], [M * (K + 8) + 8, M * N, buf.elems], [], [], [ExternBuffer(2, buf)])
    h = cuda_backend.compile_program(prog)
    assert h is not None
    got = np.zeros((M, N), np.float32)
    flat = np.concatenate([np.zeros(8, np.float32), x.ravel()])
    cuda_backend.execute_program(h, [ProgramIO(0, flat)], [ProgramIO(1, got)])
    stats = cuda_backend.program_stats(h)
    assert stats["tensor_core_linears"] == 1 and stats["dense_gemm_timeouts"] == 0
    want = bf16_exact(x[:, :K]).astype(np.float64) @ W.astype(np.float64).T + (b.astype(np.float64) if bias else 0.0)
    assert rel(got, want) < 2e-6
    cuda_backend.free_program(h)
    buf.free()


def test_tensor_core_prefill_of_a_wide_model(cuda_backend):
    """Widths that reach the tensor path: the bfloat16 session's prompt logits stay within the rounding of activations to
    bf16 of the exact float32 session's, and its decoded continuation (row kernels, f32 activations) agrees with both."""
    cfg = config([delta_layer(heads=4, kv_heads=2, dim=32, vdim=64, rank_a=16, rank_g=16, mlp=moe(experts=4, identity=1, top=2, ff=64)),
                  attention_layer(heads=4, kv_heads=2, dim=32, window=40, rel_rows=16, bias_max=64, mlp=moe(experts=4, identity=1, top=2, ff=64))],
                 width=128, vocab=256)
    W = random_weights(cfg, seed=21)
    toks = tokens(cfg, 72)
    want, _ = ref.forward(cfg, as_f64(W), toks)
    s16, s32 = open_model(cuda_backend, cfg, W, "bfloat16", max_chunk=64), open_model(cuda_backend, cfg, W, "float32", max_chunk=64)
    g16 = np.concatenate([s16.feed("r", toks[:64], range(64))] + [s16.feed("r", [t], [0]) for t in toks[64:]])
    g32 = np.concatenate([s32.feed("r", toks[:64], range(64))] + [s32.feed("r", [t], [0]) for t in toks[64:]])
    lp, handle, _, _ = s16.program(64, "all")
    stats = cuda_backend.program_stats(handle)
    assert stats["tensor_core_linears"] >= 5 and stats["dense_gemm_timeouts"] == 0
    assert cuda_backend.program_stats(s32.program(64, "all")[1])["tensor_core_linears"] == 0
    assert rel(g32, want) < TOL
    assert rel(g16, want) < 3e-2
    close(s16), close(s32)


def test_long_window_decode_splits_the_window(cuda_backend):
    """A window long enough that single-token steps spread it over several CTAs (partial softmax states merged afterwards):
    decoding across the point where the window fills up, against the prompt path and the restatement."""
    cfg = config([attention_layer(heads=2, kv_heads=1, dim=16, window=160, rel_rows=12, bias_max=200, softcap=20.0)], width=32, vocab=50)
    W = random_weights(cfg, seed=31, qk_gain=6.0)
    toks = tokens(cfg, 200)
    want, _ = ref.forward(cfg, as_f64(W), toks)
    s = open_model(cuda_backend, cfg, W, max_chunk=64)
    got = [s.feed("r", toks[:130], range(130))] + [s.feed("r", [t], [0]) for t in toks[130:]]
    assert rel(np.concatenate(got), want) < TOL
    close(s)


# ── the prefill kernels: tiles of queries, keys and tokens ──
@pytest.mark.parametrize("window,dim,first", [(63, 16, 0), (64, 48, 37), (65, 20, 1), (100, 128, 64), (129, 8, 5), (3, 36, 70), (300, 16, 11)])
def test_tiled_prefill_attention_at_tile_borders(cuda_backend, window, dim, first):
    """Chunks of up to 128 tokens take the tiled prefill kernel: windows that end just before, at and just after a 64-key
    tile, head sizes that pad the tile, chunks that start anywhere in the sequence, a peaky softmax (one key more or less
    is far outside the tolerance), against the restatement and against single-token steps."""
    cfg = config([attention_layer(heads=4, kv_heads=2, dim=dim, window=window, rel_rows=10, bias_max=2 * window + 3, softcap=25.0)], width=32, vocab=50)
    W = random_weights(cfg, seed=window, qk_gain=10.0)
    n = first + 128 + 64 + 16 + 3
    toks = tokens(cfg, n)
    want, _ = ref.forward(cfg, as_f64(W), toks)
    if window < n:
        wider = json.loads(json.dumps(cfg))
        wider["layers"][0]["mixer"]["mask"]["size"] = window + 1
        assert rel(ref.forward(wider, as_f64(W), toks)[0], want) > 50 * TOL
    s = open_model(cuda_backend, cfg, W, n_slots=2, max_chunk=128)
    got = ([s.feed("p", toks[:first], range(first))] if first else []) + [s.feed("p", toks[first:], range(n - first))]
    assert rel(np.concatenate(got), want) < TOL
    single = np.concatenate([s.feed("d", [t], [0]) for t in toks])
    assert rel(single, want) < TOL
    close(s)


@pytest.mark.parametrize("layer", [delta_layer(), delta_layer(heads=3, kv_heads=1, dim=40, vdim=10, conv=4, rank_a=3, rank_g=5),
                                   delta_layer(heads=2, kv_heads=2, dim=8, vdim=70, conv=1), delta_layer(heads=1, kv_heads=1, dim=130, vdim=12, conv=2),
                                   delta_layer(heads=4, kv_heads=2, dim=128, vdim=32, conv=3)],
                         ids=["delta", "delta-odd", "delta-notail", "delta-wide-key", "delta-128"])
def test_delta_prefill_walks_prepared_tiles(cuda_backend, layer):
    """Chunks of 16 or more tokens prepare every token's vectors first and walk them tile by tile (double buffered): several
    tiles, chunks of both kinds in one sequence, against the restatement and single tokens."""
    cfg = config([layer], width=40, vocab=61)
    W = random_weights(cfg, seed=17)
    toks = tokens(cfg, 64 + 16 + 8 + 2 + 1 + 64 + 32)
    want, _ = ref.forward(cfg, as_f64(W), toks)
    s = open_model(cuda_backend, cfg, W, n_slots=2, max_chunk=64)
    got = [s.feed("p", toks[:91], range(91)), s.feed("p", toks[91:], range(96))]
    assert rel(np.concatenate(got), want) < 2 * TOL
    single = np.concatenate([s.feed("d", [t], [0]) for t in toks])
    assert rel(single, want) < 2 * TOL
    close(s)


def test_rows_wider_than_the_norm_kernel_caches(cuda_backend):
    """Rows of more than 16 x 256 values do not fit the norm kernel's registers: the two-pass form, also for the chained norm
    that closes one sublayer and opens the next, in single-token and many-token steps."""
    cfg = config([attention_layer(heads=2, kv_heads=1, dim=8, window=6, mlp=moe(experts=2, identity=1, top=2, ff=8)),
                  delta_layer(heads=2, kv_heads=1, dim=8, vdim=8, conv=2)], width=4104, vocab=23)
    W = random_weights(cfg, seed=5)
    toks = tokens(cfg, 19)
    want, _ = ref.forward(cfg, as_f64(W), toks)
    s = open_model(cuda_backend, cfg, W, n_slots=2, max_chunk=16)
    assert rel(s.feed("p", toks, range(19)), want) < 2 * TOL
    assert rel(np.concatenate([s.feed("d", [t], [0]) for t in toks]), want) < 2 * TOL
    close(s)


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_sizes_that_fit_no_vector_path(cuda_backend, dtype):
    """Width, head sizes, expert width and vocabulary that are multiples of neither 4 nor 8: every kernel's scalar form."""
    cfg = config([attention_layer(heads=3, kv_heads=1, dim=10, window=9, rel_rows=7, bias_max=30, mlp=moe(experts=3, identity=1, top=2, ff=7)),
                  delta_layer(heads=2, kv_heads=1, dim=6, vdim=9, conv=3, rank_a=3, rank_g=5, mlp=moe(experts=2, identity=0, top=1, ff=11))],
                 width=50, vocab=31)
    W = random_weights(cfg, seed=21, qk_gain=2.0)
    toks = tokens(cfg, 45)
    want, _ = ref.forward(cfg, as_f64(W), toks)
    s = open_model(cuda_backend, cfg, W, dtype, n_slots=2, max_chunk=32)
    assert rel(s.feed("p", toks, range(45)), want) < tol(dtype)
    assert rel(np.concatenate([s.feed("d", [t], [0]) for t in toks]), want) < 2 * TOL
    close(s)


def test_trace_replayer_command(cuda_backend, tmp_path):
    """`bin/trace_run` as a user runs it: a model folder, JSON steps on standard input (whole prompts, portions, single
    tokens, requests that end and free their slot, a step that wants nothing), logits files per step, `done` lines."""
    import subprocess
    from zgml_b200.host.safetensors import write_safetensors
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    W = random_weights(MIXED, seed=14, qk_gain=2.0)
    public = json.loads(json.dumps(MIXED))
    for L in public["layers"]:
        L["mixer"] = {k: v for k, v in L["mixer"].items() if not k.startswith("_")}
    model = tmp_path / "model"
    model.mkdir()
    (model / "config.json").write_text(json.dumps(public))
    write_safetensors(str(model / "model.safetensors"), W)
    A, B = tokens(MIXED, 37, 1), tokens(MIXED, 21, 2)
    wa, wb = ref.forward(MIXED, as_f64(W), A)[0], ref.forward(MIXED, as_f64(W), B)[0]
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": A[:30], "want": [0, 29]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": A[30:32], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": A[32:33], "want": [0]}], "end": []},
             {"step": 3, "entries": [{"id": "a", "tokens": A[33:], "want": [3, 1]}], "end": ["a"]},
             {"step": 4, "entries": [{"id": "b", "tokens": B, "want": list(range(21))}], "end": ["b"]}]
    want = {0: wa[[0, 29]], 2: wa[[32]], 3: wa[[36, 34]], 4: wb}
    for dtype in ("float32", "bfloat16"):
        out = tmp_path / dtype
        p = subprocess.run([os.path.join(root, "bin", "trace_run"), "--model", str(model), "--dtype", dtype, "--out", str(out), "--max-tokens", "64"],
                           input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600)
        assert p.returncode == 0, p.stderr[-2000:]
        assert [l for l in p.stdout.splitlines() if l.startswith("done ")] == [f"done {i}" for i in range(5)]
        assert not (out / "1.f32").exists()
        for i, w in want.items():
            got = np.fromfile(out / f"{i}.f32", dtype="<f4").reshape(-1, MIXED["vocab"])
            assert got.shape == w.shape and rel(got, w) < tol(dtype)
