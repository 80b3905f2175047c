"""Prefill and decode throughput of Lududra next to a LLaMA of equal layer sizes (`bench.py --arch lududra`).

Both models are random-init at shapes that resemble a real model's layers and run through the framework's own
sessions.  Lududra keeps bfloat16 weights (2 B / weight), the LLaMA arm GGUF Q8_0 blocks (34 B / 32 weights); its
feed-forward width is top x expert width, so both stream the same number of ACTIVE weights per token.
Per arm: tokens / s end to end through the session (host control words, token ids and logits cross PCIe every step) and
device-only (the step's CUDA graph replayed with inputs resident), the HBM bytes a decoded token must move (active
weights + carried state) as a fraction of the measured copy bandwidth, and the prefill's matmul FLOPs as a fraction of
the measured dense bf16 throughput.  Timing: wall clock around synchronised replays, after warm-up.
"""
import json
import os
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

SIZES = {
    "w1024": dict(width=1024, n_layers=4, heads=8, kv_heads=2, dim=128, window=512, experts=8, top=2, ff=1024, vocab=32768),
    "w2048": dict(width=2048, n_layers=4, heads=16, kv_heads=4, dim=128, window=1024, experts=16, top=2, ff=2048, vocab=32768),
    "w4096": dict(width=4096, n_layers=2, heads=32, kv_heads=8, dim=128, window=1024, experts=8, top=2, ff=4096, vocab=32768),
}


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return float(d["hbm_gbs"]), float(d["bf16_tflops"]), "measured"
    return 6650.0, 1590.0, "fallback"


def timed(fn, sync, reps, warm=3):
    for _ in range(warm):
        fn()
    sync()
    t0 = time.perf_counter()
    for _ in range(reps):
        fn()
    sync()
    return (time.perf_counter() - t0) / reps


def lududra_arm(be, size, prefill_T, context, reps):
    from zgml_b200.host.lududra import LududraConfig, LududraModel, synthetic_config, synthetic_tensors
    from zgml_b200.host.session import SequenceSession
    cfgd = synthetic_config(**size)
    cfg = LududraConfig.from_dict(cfgd)
    model = LududraModel(be, cfg, synthetic_tensors(cfgd), "bfloat16")
    s = SequenceSession(be, model, n_slots=1, max_chunk=prefill_T)
    r = np.random.default_rng(0)
    prompt = r.integers(0, cfg.vocab, context).tolist()
    D = cfg.width
    active = state = 0          # weights / state elements one decoded token touches
    for L in cfg.layers:
        m, mlp = L["mixer"], L["mlp"]
        H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        if L["type"] == "attention":
            active += (H * d + G * d + H * dv) * D + D * H * dv
            state += min(context, m["mask"]["size"]) * G * d
        else:
            active += (2 * G * d + H * dv + H + 128) * D + 64 * (H * d + H * dv) + D * H * dv
            state += 2 * H * d * dv
        rt = mlp["router"]
        active += (rt["experts"] + rt["identity"]) * D + rt["top"] * 3 * D * mlp["expert"]["ff"]
    body = active
    active += cfg.vocab * D
    out = {"weights_gb": round(model.weight_bytes() / 1e9, 3), "active_params_per_token": active}
    # prefill: one chunk of prefill_T tokens, logits of the last position
    toks = prompt[:prefill_T]
    e2e = timed(lambda: (s.feed("p", toks, [prefill_T - 1]), s.release("p")), be.sync, reps)
    handle = s.program(prefill_T, "last")[1]
    dev = timed(lambda: be.lib.zg_cuda_execute_device(be.ctx, handle.ptr), be.sync, reps)
    out["prefill"] = {"tokens": prefill_T, "tok_s_e2e": round(prefill_T / e2e), "tok_s_device": round(prefill_T / dev), "ms_device": round(dev * 1e3, 3),
                      "matmul_tflops_device": round(2.0 * (body * prefill_T + cfg.vocab * D) / dev / 1e12, 1), "kernels": be.program_stats(handle)["kernels"],
                      "tensor_core_linears": be.program_stats(handle)["tensor_core_linears"]}
    # decode: one token per step after `context` tokens
    s.feed("d", prompt, [])
    tok = [1]
    e2e = timed(lambda: s.feed("d", tok, [0]), be.sync, 4 * reps)
    handle = s.program(1, "last")[1]
    dev = timed(lambda: be.lib.zg_cuda_execute_device(be.ctx, handle.ptr), be.sync, 4 * reps)
    bytes_tok = 2 * active + 4 * state
    out["decode"] = {"context": context, "tok_s_e2e": round(1 / e2e, 1), "tok_s_device": round(1 / dev, 1), "us_device": round(dev * 1e6, 1),
                     "bytes_per_token": bytes_tok, "hbm_gbs_device": round(bytes_tok / dev / 1e9, 1), "kernels": be.program_stats(handle)["kernels"]}
    out["dense_gemm_timeouts"] = be.program_stats(handle)["dense_gemm_timeouts"]
    s.close()
    model.close()
    return out


def llama_arm(be, size, prefill_T, context, reps):
    from zgml_b200.host import llama
    D, H, G = size["width"], size["heads"], size["kv_heads"]
    assert D == H * size["dim"], "the LLaMA arm needs width = heads x dim"
    cfg = llama.LlamaConfig(size["vocab"], D, size["n_layers"], H, G, size["top"] * size["ff"], max(2048, context + 8), 1e-5, 1e4, True)
    w, handles = llama.synthetic_resident_shard(be, cfg, "q8_0", seed=1)
    active = sum(k * n for k, n in llama.linear_shapes(cfg).values()) * cfg.n_layers
    out = {"active_params_per_token": active + cfg.vocab_size * D}
    r = np.random.default_rng(0)
    sp = llama.DeviceLlamaSession(be, cfg, w, prefill_T)
    toks = r.integers(0, cfg.vocab_size, prefill_T).tolist()
    e2e = timed(lambda: sp.execute_at(toks, 0), be.sync, reps)
    dev = timed(lambda: be.lib.zg_cuda_execute_device(be.ctx, sp.handle.ptr), be.sync, reps)
    out["prefill"] = {"tokens": prefill_T, "tok_s_e2e": round(prefill_T / e2e), "tok_s_device": round(prefill_T / dev), "ms_device": round(dev * 1e3, 3),
                      "matmul_tflops_device": round(2.0 * (active * prefill_T + cfg.vocab_size * D * prefill_T) / dev / 1e12, 1),
                      "kernels": be.program_stats(sp.handle)["kernels"], "note": "f32 dense head over all prompt rows; 3xBF16 linears"}
    sp.close()
    sd = llama.DeviceLlamaSession(be, cfg, w, 1)
    sd.pos = context
    e2e = timed(lambda: sd.execute_at([1], context), be.sync, 4 * reps)
    dev = timed(lambda: be.lib.zg_cuda_execute_device(be.ctx, sd.handle.ptr), be.sync, 4 * reps)
    bytes_tok = active * 34 // 32 + 4 * cfg.vocab_size * D + 4 * 2 * context * cfg.kv_dim * cfg.n_layers
    out["decode"] = {"context": context, "tok_s_e2e": round(1 / e2e, 1), "tok_s_device": round(1 / dev, 1), "us_device": round(dev * 1e6, 1),
                     "bytes_per_token": bytes_tok, "hbm_gbs_device": round(bytes_tok / dev / 1e9, 1), "kernels": be.program_stats(sd.handle)["kernels"]}
    sd.close()
    for h in handles:
        h.free()
    return out


def run(args):
    from zgml_b200 import CudaBackend
    hbm, tf, how = peaks()
    be = CudaBackend(0)
    names = [n for n in (args.sizes.split(",") if args.sizes else SIZES)]
    res = {"bench": "lududra_vs_llama", "peaks": {"hbm_gbs": hbm, "bf16_tflops": tf, "source": how}, "data": "synthetic random-init", "sizes": {}}
    for n in names:
        size = SIZES[n]
        entry = {"shape": size}
        for arm, fn in (("lududra", lududra_arm), ("llama_q8_0", llama_arm)):
            try:
                e = fn(be, size, args.prefill_tokens, args.context, args.steps)
                e["decode"]["frac_of_hbm"] = round(e["decode"]["hbm_gbs_device"] / hbm, 3)
                e["prefill"]["frac_of_bf16"] = round(e["prefill"]["matmul_tflops_device"] / tf, 3)
                entry[arm] = e
            except Exception as ex:   # one arm failing must not hide the other
                entry[arm] = {"error": repr(ex)}
        res["sizes"][n] = entry
    res["gpu_launches"] = be.launch_count()
    be.close()
    print(json.dumps(res))
