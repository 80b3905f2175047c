"""Command line of the framework: `python -m zgml_b200 <command>`.

  generate   --model PATH --prompt 1,2,3 --max-new-tokens N [--temperature T --top-k K --top-p P --seed S]
  trace-run  --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N     (steps as JSON lines on standard input)

`trace-run` replays a serving trace through the model's own session: one JSON object per line,
{"step": n, "entries": [{"id", "tokens", "want"}], "end": [ids]}; the logits at the wanted places of a step go to
OUT/<step>.f32 (little-endian f32, [wanted, vocab], in entry order), then `done <step>` is printed.
"""
import argparse
import json
import os
import sys

import numpy as np


def _backend():
    from .build import build_cuda
    build_cuda()                       # no-op when the library is newer than its sources
    from .backend import CudaBackend
    return CudaBackend(0)


def cmd_generate(a) -> int:
    from .host.registry import open_session
    from .host.sampling import Sampler
    be = _backend()
    prompt = [int(t) for t in a.prompt.split(",") if t.strip()]
    s = open_session(be, a.model, a.dtype, max_chunk=a.max_chunk, max_tokens=len(prompt) + a.max_new_tokens)
    out = s.generate(prompt, a.max_new_tokens, Sampler(a.temperature, a.top_k, a.top_p, a.seed))
    print(",".join(str(t) for t in out))
    s.close()
    return 0


def cmd_trace_run(a) -> int:
    from .host.registry import open_session
    be = _backend()
    s = open_session(be, a.model, a.dtype, n_slots=a.slots, max_chunk=a.max_chunk, max_tokens=a.max_tokens)
    os.makedirs(a.out, exist_ok=True)
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        step = json.loads(line)
        rows = s.step(step["entries"], step.get("end", ()))
        rows = [r for r in rows if r.shape[0]]
        if rows:
            data = np.ascontiguousarray(np.concatenate(rows, 0), dtype="<f4")
            tmp = os.path.join(a.out, f".{step['step']}.part")
            with open(tmp, "wb") as f:
                f.write(data.tobytes())
            os.replace(tmp, os.path.join(a.out, f"{step['step']}.f32"))
        print(f"done {step['step']}", flush=True)
    s.close()
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="zgml_b200")
    sub = ap.add_subparsers(dest="cmd", required=True)
    g = sub.add_parser("generate", help="decode from a prompt of token ids")
    g.add_argument("--model", required=True)
    g.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    g.add_argument("--prompt", required=True, help="comma-separated token ids")
    g.add_argument("--max-new-tokens", type=int, default=16)
    g.add_argument("--temperature", type=float, default=0.0)
    g.add_argument("--top-k", type=int, default=0)
    g.add_argument("--top-p", type=float, default=1.0)
    g.add_argument("--seed", type=int, default=None)
    g.add_argument("--max-chunk", type=int, default=256)
    g.set_defaults(fn=cmd_generate)
    t = sub.add_parser("trace-run", help="replay a serving trace and write the wanted logits")
    t.add_argument("--model", required=True)
    t.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    t.add_argument("--out", required=True)
    t.add_argument("--max-tokens", type=int, default=0, help="most tokens live requests hold at any time: sizes the caches of models that keep every position (0: the model's default)")
    t.add_argument("--slots", type=int, default=4)
    t.add_argument("--max-chunk", type=int, default=256)
    t.set_defaults(fn=cmd_trace_run)
    a = ap.parse_args(argv)
    return a.fn(a)


if __name__ == "__main__":
    sys.exit(main())
