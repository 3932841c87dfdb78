"""Trace replay: feed given token ids through a model step by step and write logits.

Nothing is sampled.  The program drives the engine's own loader, cache manager, step
function and kernels (``build_runner`` / ``ModelRunner.step``), the ones generation uses.
The reference has no such tool: its nearest relatives print token ids and timings
(tools/run_infurnace_model.py:19-44,71-83) and its fixture generator is an empty file
(tools/generate_fixtures.py).

Input, one JSON object per line on standard input::

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

``entries``: for each request its next tokens and the places among them whose logits are
wanted; all entries of a step run as one batch.  A request is created the first time
its id appears.  ``end``: requests that are finished after the step; their pages and
state slot are given back.  For a step in which something is wanted, ``<out>/<step>.f32``
holds the logits at the wanted places in the order of the entries and of ``want``,
little-endian float32 ``[wanted, vocab]``.  After every step ``done <step>`` is printed
and flushed.
"""
from __future__ import annotations

import argparse
import json
import os
import sys


def _progress(msg):
    print(f"[trace_run] {msg}", file=sys.stderr, flush=True)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=("bfloat16", "float32"))
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time (each rounded up to a multiple of 64)")
    ap.add_argument("--page-size", type=int, default=16)
    ap.add_argument("--max-requests", type=int, default=8, help="most requests live at a time")
    args = ap.parse_args(argv)
    if args.max_tokens < 1:
        ap.error("--max-tokens must be positive")
    if 64 % args.page_size and args.page_size % 64:
        ap.error("--page-size must divide 64 or be a multiple of it")

    import torch
    from .engine.loading import EngineOptions, build_runner
    from .engine.runner import StepEntry
    from .errors import InfurnaceError

    os.makedirs(args.out, exist_ok=True)
    unit = max(64, args.page_size)
    pool_tokens = -(-args.max_tokens // unit) * unit
    options = EngineOptions(
        dtype=args.dtype, device="cuda", page_size=args.page_size, num_pages=pool_tokens // args.page_size,
        max_num_seqs=args.max_requests, max_num_batched_tokens=pool_tokens, max_model_len=None)
    try:
        _progress(f"loading {args.model} ({args.dtype}); kernels are compiled at first use")
        _, plan, runner = build_runner(args.model, options, progress=_progress)
        _progress("ready")
        for line in sys.stdin:
            line = line.strip()
            if not line:
                continue
            rec = json.loads(line)
            step = rec["step"]
            entries = []
            for e in rec.get("entries", []):
                rid = str(e["id"])
                if not runner.cache.has_request(rid):
                    runner.cache.add_request(rid)
                entries.append(StepEntry(rid, e["tokens"], e.get("want", [])))
            if entries:
                logits = runner.step(entries)
                if logits is not None:
                    data = logits.to(torch.float32).cpu().contiguous().numpy().astype("<f4", copy=False)
                    tmp = os.path.join(args.out, f"{step}.f32.tmp")
                    with open(tmp, "wb") as f:
                        f.write(data.tobytes())
                    os.replace(tmp, os.path.join(args.out, f"{step}.f32"))
                else:
                    torch.cuda.synchronize()
            for rid in rec.get("end", []):
                runner.cache.free_request(str(rid))
            print(f"done {step}", flush=True)
    except (InfurnaceError, KeyError, ValueError) as e:
        print(f"trace_run: error: {type(e).__name__}: {e}", file=sys.stderr, flush=True)
        return 1
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
