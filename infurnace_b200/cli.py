"""Command line: a model folder (or random weights) and a prompt in, generated tokens out.

Options follow the reference's two entry points where it has them
(src/infurnace/cli.py:53-65: ``--prompt``, ``--max-tokens`` (32), ``--stop-strings``,
``--num-slots``, ``--max-context``, ``--device``; tools/run_infurnace_model.py:48-55:
``--max-context``, ``--output-tokens`` (4), and its JSON report).  What the reference
takes from a GGUF file and a manifest comes here from ``--model DIR`` (config.json and
safetensors) or from ``--random-weights SEED --config FILE``.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import tempfile
import time


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="infurnace-b200", description="offline generation with the infurnace_b200 engine")
    src = ap.add_argument_group("model")
    src.add_argument("--model", help="folder with config.json and *.safetensors")
    src.add_argument("--random-weights", type=int, metavar="SEED", help="draw the weights from this seed (needs --config)")
    src.add_argument("--config", help="config.json (or a folder holding one) for --random-weights")
    src.add_argument("--dtype", default="bfloat16", choices=("bfloat16", "float32"))
    src.add_argument("--device", default="cuda", help="only 'cuda' exists: the engine has no CPU path")
    pr = ap.add_argument_group("prompt")
    pr.add_argument("--prompt", help="text prompt (needs tokenizer.json in the model folder, or --char-tokenizer)")
    pr.add_argument("--prompt-ids", help="comma-separated token ids")
    pr.add_argument("--prompt-len", type=int, help="a prompt of this many uniform random token ids (see --seed)")
    pr.add_argument("--char-tokenizer", action="store_true", help="one token per character, for models without a vocabulary")
    pr.add_argument("--stop-strings", nargs="*", default=[])
    gen = ap.add_argument_group("generation")
    gen.add_argument("--max-tokens", "--output-tokens", dest="max_tokens", type=int, default=32)
    gen.add_argument("--temperature", type=float, default=0.0)
    gen.add_argument("--seed", type=int, default=0, help="seed of sampling and of --prompt-len")
    eng = ap.add_argument_group("engine")
    eng.add_argument("--num-slots", "--max-num-seqs", dest="max_num_seqs", type=int, default=1,
                     help="requests that may be live at a time")
    eng.add_argument("--max-context", "--max-model-len", dest="max_model_len", type=int, default=2048,
                     help="longest sequence (prompt and generated tokens)")
    eng.add_argument("--page-size", type=int, default=16)
    eng.add_argument("--num-pages", type=int, default=None, help="pages of the key/value pool (default: enough for all slots)")
    eng.add_argument("--max-num-batched-tokens", type=int, default=2048, help="token budget of one step")
    ap.add_argument("--json", action="store_true", help="print a JSON report (prompt ids, generated ids, timings)")
    return ap


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    if args.device != "cuda":
        print("error: --device must be 'cuda'; this engine has no CPU path", file=sys.stderr)
        return 1
    if (args.model is None) == (args.random_weights is None):
        print("error: give either --model DIR or --random-weights SEED --config FILE", file=sys.stderr)
        return 1
    if sum(x is not None for x in (args.prompt, args.prompt_ids, args.prompt_len)) != 1:
        print("error: give exactly one of --prompt, --prompt-ids, --prompt-len", file=sys.stderr)
        return 1
    if args.max_tokens < 0 or args.max_model_len <= 0:
        print("error: max-context must be positive and max-tokens must be non-negative", file=sys.stderr)
        return 1

    from .engine import Engine, EngineOptions, Request, RequestState, SamplingParams
    from .errors import InfurnaceError
    from .models import read_config
    from .tokenizer import CharTokenizer, FileTokenizer

    tmp = None
    try:
        model_dir = args.model
        if model_dir is None:
            if args.config is None:
                print("error: --random-weights needs --config", file=sys.stderr)
                return 1
            from .weights.random_init import write_random_model
            tmp = tempfile.TemporaryDirectory(prefix="infurnace_b200_")
            model_dir = write_random_model(read_config(args.config), args.random_weights, tmp.name)
        elif not os.path.isdir(model_dir):
            print(f"model folder not found: {model_dir}", file=sys.stderr)
            return 1
        config = read_config(model_dir)
        tokenizer = None
        if args.prompt is not None:
            tok_path = os.path.join(model_dir, "tokenizer.json")
            if args.char_tokenizer:
                tokenizer = CharTokenizer(config.vocab_size)
            elif os.path.exists(tok_path):
                tokenizer = FileTokenizer(tok_path)
            else:
                print(f"error: no tokenizer.json in {model_dir}; use --prompt-ids, --prompt-len or --char-tokenizer",
                      file=sys.stderr)
                return 1
        options = EngineOptions(dtype=args.dtype, device=args.device, page_size=args.page_size, num_pages=args.num_pages,
                                max_num_seqs=args.max_num_seqs, max_num_batched_tokens=args.max_num_batched_tokens,
                                max_model_len=args.max_model_len)
        t0 = time.perf_counter()
        engine = Engine.from_model_dir(model_dir, options, tokenizer=tokenizer)
        load_ms = (time.perf_counter() - t0) * 1000
        sp = SamplingParams(max_tokens=args.max_tokens, temperature=args.temperature, seed=args.seed)
        if args.prompt is not None:
            req = engine.add_text_request(args.prompt, sp, stop_strings=args.stop_strings)
        else:
            if args.prompt_ids is not None:
                ids = [int(t) for t in args.prompt_ids.replace(" ", "").split(",") if t]
            else:
                import random
                rng = random.Random(args.seed)
                ids = [rng.randrange(config.vocab_size) for _ in range(args.prompt_len)]
            req = Request("req-1", ids, sp)
            engine.add_request(req)
        if req.state is RequestState.REJECTED:
            print(f"error: request rejected: {req.error}", file=sys.stderr)
            return 1
        step_ms = []
        out = sys.stdout
        while not engine.is_done():
            t0 = time.perf_counter()
            res = engine.step()
            step_ms.append((time.perf_counter() - t0) * 1000)
            if not args.json:
                for rid, text in res.new_text.items():
                    out.write(text)
                    out.flush()
                if tokenizer is None:
                    for toks in res.new_tokens.values():
                        out.write("".join(f"{t} " for t in toks))
                        out.flush()
        if req.state is not RequestState.FINISHED:
            print(f"\nerror: request ended {req.state.value}: {req.error}", file=sys.stderr)
            return 1
        if args.json:
            decode = step_ms[1:]
            report = {
                "model": {"dir": args.model, "random_weights": args.random_weights, "architecture": config.architecture},
                "execution": {"device": args.device, "dtype": args.dtype, "max_context": args.max_model_len,
                              "cache_slots": args.max_num_seqs, "page_size": args.page_size, "load_ms": load_ms,
                              "timings_ms": {"prefill_ms": step_ms[0] if step_ms else None,
                                             "first_decode_ms": decode[0] if decode else None,
                                             "avg_decode_ms": sum(decode) / len(decode) if decode else None,
                                             "decode_times_ms": decode}},
                "prompt": list(req.prompt_token_ids),
                "generated_token_ids": list(req.output_token_ids),
                "finish_reason": req.finish_reason,
            }
            if tokenizer is not None:
                report["text"] = engine.final_text(req.request_id)
            print(json.dumps(report, ensure_ascii=False, indent=2))
        else:
            out.write("\n")
        return 0
    except (InfurnaceError, OSError, ValueError) as e:
        print(f"error: {e}", file=sys.stderr)
        return 1
    finally:
        if tmp is not None:
            tmp.cleanup()


if __name__ == "__main__":
    raise SystemExit(main())
