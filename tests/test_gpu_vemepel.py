"""Vemepel on the CUDA backend against the float64 restatement (tests/vemepel_reference.py): every mechanism alone, the
stream after every layer, whole prompts, token-by-token decoding through the caches, prompts cut into portions down to
two tokens, interleaved requests in several slots, slot reuse, keys far back and at the edges of the position blocks, the
first tokens of a sequence, long decoding across many turns of a block cache, many shapes, and greedy generation through
the registry's entry point and the command line's trace replayer."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

import vemepel_reference as ref
from vemepel_models import as_f64, config, dense, diff_layer, latent2_layer, latent_layer, moe, random_weights

pytestmark = pytest.mark.gpu

TOL = 2e-4   # of the logits' scale; f32 accumulation against float64


def tol(dtype):
    """A bfloat16 session rounds the activations that enter a tensor-core matmul (steps of more than 8 tokens) to bf16."""
    return TOL if dtype == "float32" else 3e-2


def open_model(be, cfg, W, dtype="float32", n_slots=1, max_chunk=16, keep_layers=False, max_context=256):
    from zgml_b200.host.session import SequenceSession
    from zgml_b200.host.vemepel import VemepelConfig, VemepelModel
    model = VemepelModel(be, VemepelConfig.from_dict(cfg), lambda n: W[n], dtype)
    return SequenceSession(be, model, n_slots=n_slots, max_chunk=max_chunk, keep_layers=keep_layers, max_context=max_context)


def close(s):
    s.close()
    s.model.close()


def rel(got, want):
    return float(np.max(np.abs(got.astype(np.float64) - want)) / (np.max(np.abs(want)) + 1e-30))


def tokens(cfg, n, seed=1):
    return np.random.default_rng(seed).integers(0, cfg["vocab"], n).tolist()


MIXED = config([diff_layer(mlp=dense()), latent2_layer(mlp=moe()), latent_layer(mlp=dense(ff=24)), diff_layer(kv_from=0, block=5, mlp=moe(experts=3, top=1)),
                latent2_layer(heads=2, dim=4, rot_dim=10, vdim=5, kv_rank=9), diff_layer(heads=3, kv_heads=3, dim=6, vdim=4, block=64)])


# ── each mechanism alone (a one-layer model without a feed-forward isolates its mixer) ──
@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
@pytest.mark.parametrize("layer", [
    diff_layer(),
    diff_layer(heads=6, kv_heads=2, dim=5, vdim=9, block=33, diff=0.8),          # three heads per key head; the block crosses 32 keys
    diff_layer(heads=1, kv_heads=1, dim=40, vdim=3, block=1),                    # every position alone in its block
    diff_layer(heads=2, kv_heads=2, dim=16, vdim=16, block=1000),                # a block longer than anything: plain causal
    latent_layer(),
    latent_layer(heads=1, dim=33, vdim=40, kv_rank=5),
    latent_layer(heads=5, dim=4, vdim=4, kv_rank=70),
    latent2_layer(),
    latent2_layer(heads=1, dim=2, rot_dim=34, vdim=3, kv_rank=40, base=10000.0),
    latent2_layer(heads=4, dim=12, rot_dim=2, vdim=16, kv_rank=8, base=3.0),
], ids=["diff", "diff-grouped-33", "diff-block1", "diff-causal", "latent", "latent-1head", "latent-wide-rank", "latent2", "latent2-mostly-rotated", "latent2-one-pair"])
def test_mixer_alone(cuda_backend, layer, dtype):
    cfg = config([layer], width=40, vocab=61)
    W = random_weights(cfg, seed=5, qk_gain=4.0)
    toks = tokens(cfg, 45)
    want, stream = ref.forward(cfg, as_f64(W), toks, True)
    s = open_model(cuda_backend, cfg, W, dtype, max_chunk=64, keep_layers=True)
    got = s.feed("a", toks, range(45))
    if dtype == "float32":
        assert rel(s.layer_streams(32, "all")[0], stream[0][:32]) < TOL
    assert rel(got, want) < tol(dtype)
    close(s)


@pytest.mark.parametrize("mlp", [dense(), dense(ff=7), dense(ff=300), moe(), moe(experts=3, top=1, ff=7), moe(experts=4, top=4, ff=40), moe(experts=33, top=5, ff=16)],
                         ids=["dense", "dense-7", "dense-300", "moe", "top1", "all-experts", "33-experts"])
def test_feed_forward(cuda_backend, mlp):
    """The stream after the layer is compared too, so a fault in the activation, the routing or the expert weights cannot
    hide behind the final norm."""
    cfg = config([diff_layer(heads=2, kv_heads=2, dim=8, block=4, mlp=mlp)], width=36, vocab=50)
    W = random_weights(cfg, seed=9)
    toks = tokens(cfg, 19)
    want, stream = ref.forward(cfg, as_f64(W), toks, True)
    s = open_model(cuda_backend, cfg, W, "float32", max_chunk=32, keep_layers=True)
    got = s.feed("a", toks[:16], range(16))
    assert rel(s.layer_streams(16, "all")[0], stream[0][:16]) < TOL
    assert rel(got, want[:16]) < TOL
    close(s)


def test_token_shift_and_depth_average(cuda_backend):
    """Shift weights of exactly 0 and 1 in some columns (the row itself / the previous row alone) and depth coefficients that
    drop or negate single terms."""
    cfg = config([latent_layer(), diff_layer(mlp=dense()), latent_layer(heads=2)], width=24, vocab=30)
    W = random_weights(cfg, seed=11)
    for i in range(3):
        W[f"l{i}.shift"][::3] = 0.0
        W[f"l{i}.shift"][1::3] = 1.0
    W["l1.dwa"][:] = [0.0, -1.0, 0.5]
    W["l2.dwa"][:] = [1.0, 0.0, 0.0, 0.0]                # the last layer's own result is dropped from what goes to the head
    toks = tokens(cfg, 21)
    want, stream = ref.forward(cfg, as_f64(W), toks, True)
    s = open_model(cuda_backend, cfg, W, "float32", max_chunk=16, keep_layers=True)
    got = np.concatenate([s.feed("a", toks[:16], range(16)), s.feed("a", toks[16:20], range(4)), s.feed("a", toks[20:], [0])])
    layers = s.layer_streams(16, "all")
    for i in range(3):
        assert rel(layers[i], stream[i][:16]) < TOL, f"layer {i}"
    assert rel(got, want) < TOL
    close(s)


def test_layer_streams_of_a_mixed_stack(cuda_backend):
    W = random_weights(MIXED, seed=2)
    toks = tokens(MIXED, 16)
    want, stream = ref.forward(MIXED, as_f64(W), toks, True)
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
    want = ref.forward(MIXED, as_f64(W), toks)
    s = open_model(cuda_backend, MIXED, W, dtype, n_slots=2)
    whole = s.feed("whole", toks, range(40))
    single = np.concatenate([s.feed("single", [t], [0]) for t in toks])
    assert rel(whole, want) < tol(dtype) and rel(single, want) < TOL     # single tokens take the exact row kernels in both formats
    close(s)


@pytest.mark.parametrize("cuts", [[2] * 20, [1, 2, 3, 5, 7, 9, 13], [37, 2, 1], [16, 16, 8], [3, 37]], ids=["twos", "growing", "long-then-short", "menu", "short-then-long"])
def test_portions(cuda_backend, cuts):
    """However a prompt is cut — in the middle of a position block, two tokens at a time — the logits stay the same."""
    W = random_weights(MIXED, seed=4, qk_gain=3.0)
    toks = tokens(MIXED, 40)
    want = ref.forward(MIXED, as_f64(W), toks)
    s = open_model(cuda_backend, MIXED, W, "float32", max_chunk=32)
    got, at = [], 0
    for n in cuts:
        got.append(s.feed("a", toks[at:at + n], range(n)))
        at += n
    assert at == 40 and rel(np.concatenate(got), want) < TOL
    close(s)


def test_first_tokens(cuda_backend):
    """Position 0 alone (no previous row to shift in, one visible key), then positions 1 and 2 one by one."""
    W = random_weights(MIXED, seed=6)
    toks = tokens(MIXED, 3)
    want = ref.forward(MIXED, as_f64(W), toks)
    s = open_model(cuda_backend, MIXED, W, "float32")
    got = np.concatenate([s.feed("a", [t], [0]) for t in toks])
    assert rel(got, want) < TOL
    s.release("a")
    assert rel(s.feed("b", toks, [0, 1, 2]), want) < TOL
    close(s)


# ── requests side by side, slots ──
def test_interleaved_requests_and_slot_reuse(cuda_backend):
    W = random_weights(MIXED, seed=7, qk_gain=2.0)
    Wd = as_f64(W)
    reqs = {"a": tokens(MIXED, 29, 1), "b": tokens(MIXED, 11, 2), "c": tokens(MIXED, 40, 3)}
    want = {k: ref.forward(MIXED, Wd, v) for k, v in reqs.items()}
    s = open_model(cuda_backend, MIXED, W, "float32", n_slots=2)
    got = {k: [] for k in reqs}
    # a and b advance in turns, in unequal portions, inside ONE step call each time
    plan = [(("a", 9), ("b", 2)), (("b", 5), ("a", 1)), (("a", 19), ("b", 4))]
    at = {k: 0 for k in reqs}
    for step in plan:
        entries = [{"id": k, "tokens": reqs[k][at[k]:at[k] + n], "want": list(range(n))} for k, n in step]
        last = step is plan[-1]
        for (k, n), rows in zip(step, s.step(entries, end=["a", "b"] if last else [])):
            got[k].append(rows)
            at[k] += n
    for k in "ab":
        assert rel(np.concatenate(got[k]), want[k]) < TOL, k
    # c takes a slot that held another sequence: nothing of it may leak (the shift state is cleared, caches are masked by position)
    assert not s.pool.live()
    assert rel(s.feed("c", reqs["c"], range(40)), want["c"]) < TOL
    with pytest.raises(ValueError):
        s.feed("c", [0] * 300, [])                        # past the positions the session's caches hold
    close(s)


# ── what a query must and must not see ──
def test_block_edges_in_prompt_and_decoding(cuda_backend):
    """One differential-attention layer with a peaky softmax and blocks of 6 positions.  In the restatement, the token two
    places before a block reaches nothing inside it, while the token just before it does (the token shift carries it into the
    key of the block's first position); the device agrees with the restatement at every position, as a prompt and decoded,
    and differs from a restatement whose blocks are one position longer."""
    cfg = config([diff_layer(heads=2, kv_heads=1, dim=8, vdim=8, block=6)], width=32, vocab=40)
    W = random_weights(cfg, seed=8, qk_gain=8.0)
    Wd = as_f64(W)
    toks = tokens(cfg, 32)
    want = ref.forward(cfg, Wd, toks)
    p = 19                                                  # second position of block 3 (18 .. 23)
    out, inside = list(toks), list(toks)
    out[16] = (out[16] + 1) % cfg["vocab"]
    inside[17] = (inside[17] + 1) % cfg["vocab"]
    assert np.abs(ref.forward(cfg, Wd, out)[p] - want[p]).max() < 1e-12
    assert np.abs(ref.forward(cfg, Wd, inside)[p] - want[p]).max() > 1e-2
    longer = json.loads(json.dumps(cfg))
    longer["layers"][0]["mixer"]["mask"]["size"] = 7
    control = ref.forward(longer, Wd, toks)
    s = open_model(cuda_backend, cfg, W, "float32", n_slots=2, max_chunk=32)
    prompt = s.feed("p", toks, range(32))
    decoded = np.concatenate([s.feed("d", toks[:13], range(13))] + [s.feed("d", [t], [0]) for t in toks[13:]])
    assert rel(prompt, want) < TOL and rel(decoded, want) < TOL
    assert rel(prompt, control) > 20 * TOL
    close(s)


@pytest.mark.parametrize("layer", [latent_layer(heads=2, dim=8, vdim=8, kv_rank=16), latent2_layer(heads=2, dim=8, rot_dim=4, vdim=8, kv_rank=16)], ids=["latent", "latent2"])
def test_far_key_among_hundreds(cuda_backend, layer):
    """The last query is made to look for one early position among 300.  Without the token shift a score depends on the two
    tokens alone, so the pair of token ids whose (unrotated) score stands out most against every other key token is found
    from the weights, the key token is placed once, far back, and the query token last.  Changing the far token must move
    the restatement's last logits, and the device must agree with the restatement, in a prompt and with the last tokens decoded."""
    cfg = config([layer], width=32, vocab=40)
    W = random_weights(cfg, seed=12, qk_gain=6.0)
    W["l0.shift"][:] = 0.0
    m = layer["mixer"]
    H, dim, rd, rank = m["heads"], m["dim"], m.get("rot_dim", 0), m["kv_rank"]
    if rd:        # the rotated part of the queries stays small, so that the unrotated score decides which key stands out
        Wq = W["l0.mix.q"].reshape(H, dim + rd, -1)
        Wq[:, dim:] *= 0.125
    Wd = as_f64(W)
    h = ref.rms_norm(Wd["embed"], cfg["norm"]["eps"], Wd["l0.norm1"], True)                      # [vocab, width]: the mixer's input of every token id
    q = (h @ Wd["l0.mix.q"].T).reshape(-1, H, dim + rd)[..., :dim]
    c = ref.rms_norm((h @ Wd["l0.mix.dkv"].T)[:, :rank], cfg["norm"]["eps"], Wd["l0.mix.dkv.norm"])
    k = (c @ Wd["l0.mix.uk"].T).reshape(-1, H, dim)
    S = np.einsum("ahd,bhd->hab", q, k) * m["scale"]
    margin = np.full(S.shape, -np.inf)
    for b in range(S.shape[2]):
        others = np.delete(S, b, axis=2).max(axis=2)
        margin[:, :, b] = S[:, :, b] - others
    _, a_tok, b_tok = np.unravel_index(np.argmax(margin), margin.shape)
    n, far = 300, 4
    pool = [t for t in range(cfg["vocab"]) if t != b_tok]
    toks = [pool[i] for i in np.random.default_rng(1).integers(0, len(pool), n)]
    toks[far], toks[-1] = int(b_tok), int(a_tok)
    want = ref.forward(cfg, Wd, toks)
    moved = list(toks)
    moved[far] = pool[0]
    assert np.abs(ref.forward(cfg, Wd, moved)[-1] - want[-1]).max() > 1e-2 * np.abs(want).max(), "the construction lost its far key"
    s = open_model(cuda_backend, cfg, W, "float32", n_slots=2, max_chunk=64, max_context=320)
    assert rel(s.feed("p", toks, range(n)), want) < TOL
    s.feed("d", toks[:n - 5], [])
    decoded = np.concatenate([s.feed("d", [t], [0]) for t in toks[n - 5:]])
    assert rel(decoded, want[n - 5:]) < TOL
    close(s)


@pytest.mark.parametrize("layer", [latent_layer(heads=4, dim=12, vdim=8, kv_rank=320), latent_layer(heads=2, dim=8, vdim=8, kv_rank=520),
                                   latent2_layer(heads=3, dim=72, rot_dim=8, vdim=20, kv_rank=136),
                                   diff_layer(heads=4, kv_heads=2, dim=68, vdim=132, block=290), diff_layer(heads=8, kv_heads=1, dim=4, vdim=4, block=129)],
                         ids=["latent-rank320", "latent-rank520", "latent2-dim72", "diff-wide", "diff-8-per-group"])
def test_wide_heads_and_split_decoding(cuda_backend, layer):
    """Key and value sizes beyond one 64-wide slice of the tiled kernel (several key slices, two value slices) and caches long
    enough that single-token steps deal their keys to several CTAs and merge the shares."""
    cfg = config([layer], width=48, vocab=50)
    W = random_weights(cfg, seed=18, qk_gain=3.0)
    n = 300
    toks = tokens(cfg, n)
    want = ref.forward(cfg, as_f64(W), toks)
    s = open_model(cuda_backend, cfg, W, "float32", n_slots=2, max_chunk=128, max_context=512)
    assert rel(s.feed("p", toks, range(n)), want) < TOL
    s.feed("d", toks[:n - 12], [])
    decoded = np.concatenate([s.feed("d", toks[i:i + 1], [0]) for i in range(n - 12, n - 4)] + [s.feed("d", toks[n - 4:], range(4))])
    assert rel(decoded, want[n - 12:]) < TOL
    close(s)


def test_long_decoding_over_a_small_block_cache(cuda_backend):
    """150 decoded tokens: the block cache of the differential layers (block - 1 + chunk rows) turns over many times while the
    latent caches keep every position."""
    cfg = config([diff_layer(block=5, mlp=moe()), latent2_layer(mlp=dense()), diff_layer(kv_from=0, block=3), latent_layer()])
    W = random_weights(cfg, seed=13, qk_gain=3.0)
    toks = tokens(cfg, 160)
    want = ref.forward(cfg, as_f64(W), toks)
    s = open_model(cuda_backend, cfg, W, "float32", max_chunk=4)
    assert s.pool.buffers["l0.kv"].elems == (5 - 1 + 4) * 2 * (2 * 8 + 12)
    got = np.concatenate([s.feed("a", toks[:10], range(10))] + [s.feed("a", [t], [0]) for t in toks[10:]])
    assert rel(got, want) < TOL
    close(s)


def test_shared_keys_with_another_block_size(cuda_backend):
    """A layer that borrows keys and values keeps its own block size: the owner's cache must reach as far back as the longer of
    the two needs."""
    cfg = config([diff_layer(block=3), latent_layer(), diff_layer(kv_from=0, block=11, mlp=dense())])
    W = random_weights(cfg, seed=14, qk_gain=4.0)
    toks = tokens(cfg, 50)
    want = ref.forward(cfg, as_f64(W), toks)
    s = open_model(cuda_backend, cfg, W, "float32", max_chunk=8)
    got = np.concatenate([s.feed("a", toks[:24], range(24))] + [s.feed("a", toks[i:i + 2], [0, 1]) for i in range(24, 50, 2)])
    assert rel(got, want) < TOL
    close(s)


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_wider_model(cuda_backend, dtype):
    """Sizes at which the bfloat16 session takes the tensor-core matmuls and the grouped expert path (width and expert width
    multiples of 64, steps of 64 tokens)."""
    cfg = config([diff_layer(heads=4, kv_heads=2, dim=32, vdim=32, block=48, mlp=moe(experts=4, top=2, ff=64)),
                  latent2_layer(heads=4, dim=32, rot_dim=16, vdim=32, kv_rank=64, mlp=dense(ff=256)),
                  latent_layer(heads=4, dim=32, vdim=32, kv_rank=64, mlp=moe(experts=6, top=1, ff=128))], width=128, vocab=200, logit_scale=0.5)
    W = random_weights(cfg, seed=15)
    toks = tokens(cfg, 100)
    want = ref.forward(cfg, as_f64(W), toks)
    s = open_model(cuda_backend, cfg, W, dtype, max_chunk=64)
    got = s.feed("a", toks, range(100))
    if dtype == "float32":
        assert rel(got, want) < TOL
    else:      # a rounded input may flip a close expert choice at single positions: the bulk must agree
        err = np.max(np.abs(got - want), axis=1) / np.max(np.abs(want))
        assert np.median(err) < 3e-2 and np.mean(err < 6e-2) > 0.9
    close(s)


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_odd_sizes(cuda_backend, dtype):
    """Nothing is a multiple of 4: the unaligned forms of every kernel (scalar loads, one warp per query, exact matmuls)."""
    cfg = config([diff_layer(heads=3, kv_heads=1, dim=5, vdim=7, block=9, mlp=moe(experts=3, top=2, ff=11)),
                  latent2_layer(heads=3, dim=5, rot_dim=6, vdim=7, kv_rank=9, mlp=dense(ff=13)),
                  latent_layer(heads=2, dim=7, vdim=3, kv_rank=11), diff_layer(heads=3, kv_heads=1, dim=5, vdim=7, kv_from=0, block=4)], width=37, vocab=53)
    W = random_weights(cfg, seed=19, qk_gain=2.0)
    toks = tokens(cfg, 41)
    want = ref.forward(cfg, as_f64(W), toks)
    s = open_model(cuda_backend, cfg, W, dtype, max_chunk=32)
    got = np.concatenate([s.feed("a", toks[:35], range(35))] + [s.feed("a", [t], [0]) for t in toks[35:]])
    assert rel(got, want) < tol(dtype)
    close(s)


# ── the entry points ──
def _write_model(tmp_path, cfg, W):
    from zgml_b200.host.safetensors import write_safetensors
    d = os.path.join(tmp_path, "model")
    os.makedirs(d, exist_ok=True)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_safetensors(os.path.join(d, "model.safetensors"), W)
    return d


def test_greedy_generation_through_the_registry(cuda_backend, tmp_path):
    from zgml_b200.host.registry import open_session
    W = random_weights(MIXED, seed=16)
    d = _write_model(tmp_path, MIXED, W)
    prompt = tokens(MIXED, 9)
    want, seq = [], list(prompt)
    for _ in range(12):
        want.append(int(np.argmax(ref.forward(MIXED, as_f64(W), seq)[-1])))
        seq.append(want[-1])
    s = open_session(cuda_backend, d, "float32", n_slots=1, max_chunk=8, max_tokens=32)
    assert s.generate(prompt, 12) == want
    assert not s.pool.live()
    close(s)


def test_trace_replay_from_the_command_line(tmp_path):
    W = random_weights(MIXED, seed=17)
    d = _write_model(tmp_path, MIXED, W)
    toks = tokens(MIXED, 30)
    want = ref.forward(MIXED, as_f64(W), toks)
    steps = [{"step": 0, "entries": [{"id": "r", "tokens": toks[:17], "want": [0, 16]}], "end": []},
             {"step": 1, "entries": [{"id": "r", "tokens": toks[17:19], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "r", "tokens": toks[19:], "want": [10]}], "end": ["r"]}]
    out = os.path.join(tmp_path, "out")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    p = subprocess.run([os.path.join(root, "bin", "trace_run"), "--model", d, "--dtype", "float32", "--out", out, "--max-tokens", "64"],
                       input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [l for l in p.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2"]
    assert not os.path.exists(os.path.join(out, "1.f32"))
    got0 = np.fromfile(os.path.join(out, "0.f32"), dtype="<f4").reshape(2, -1)
    got2 = np.fromfile(os.path.join(out, "2.f32"), dtype="<f4").reshape(1, -1)
    assert rel(got0, want[[0, 16]]) < TOL and rel(got2, want[[29]]) < TOL
