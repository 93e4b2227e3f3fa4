"""Command line: ``python -m oxr_inference_b200 --model DIR --prompt-ids 1,2,3 --max-tokens 16``.

Option names follow the reference's command lines where it has them (``--model``, ``--kv-gb``, ``--max-running``,
``--max-waiting``: oxr_runtime/serve.py:65-83; ``--no-cuda-graphs``, ``--limit``, ``--out``:
scripts/parity.py:146-166). ``random-model`` writes a model folder with random weights.
"""

from __future__ import annotations

import argparse
import json
import logging
import sys
import time
from pathlib import Path


def _generate(args: argparse.Namespace) -> int:
    from oxr_inference_b200.config import EngineSettings
    from oxr_inference_b200.engine.api import Engine
    from oxr_inference_b200.sampling import SamplingParams

    prompts: list = []
    for ids in args.prompt_ids or []:
        prompts.append([int(t) for t in ids.replace(",", " ").split()])
    prompts += args.prompt or []
    if args.prompt_file:
        for line in Path(args.prompt_file).read_text().splitlines():
            line = line.strip()
            if line:
                prompts.append(json.loads(line) if line.startswith("[") else line)
    if args.limit:
        prompts = prompts[:args.limit]
    if not prompts:
        print("no prompt given (--prompt-ids, --prompt or --prompt-file)", file=sys.stderr)
        return 2
    settings = EngineSettings(kv_cache_gb=args.kv_gb, num_pages=args.num_pages, page_size=args.page_size,
                              max_running=args.max_running, max_waiting=args.max_waiting, max_step_tokens=args.max_step_tokens,
                              prefill_chunk=args.prefill_chunk, max_positions=args.max_positions,
                              cuda_graphs=not args.no_cuda_graphs, dtype=args.dtype)
    engine = Engine(args.model, settings)
    params = SamplingParams(max_tokens=args.max_tokens, temperature=args.temperature, seed=args.seed,
                            repetition_penalty=args.repetition_penalty, ignore_eos=args.ignore_eos)
    started = time.perf_counter()
    results = engine.generate(prompts, params)
    seconds = time.perf_counter() - started
    rows = [{"prompt_tokens": c.prompt_tokens, "token_ids": c.token_ids, "finish_reason": c.finish_reason, "text": c.text,
             "seconds": round(c.seconds, 4)} for c in results]
    for row in rows:
        print(json.dumps(row, ensure_ascii=False))
    generated = sum(len(c.token_ids) for c in results)
    print(f"{len(results)} requests, {generated} tokens in {seconds:.3f} s ({generated / max(seconds, 1e-9):.1f} tok/s), "
          f"{engine.preemptions} preemptions", file=sys.stderr)
    if args.out:
        Path(args.out).write_text(json.dumps({"results": rows, "seconds": seconds, "counters": engine.counters}, indent=1))
    return 0


def _random_model(args: argparse.Namespace) -> int:
    from oxr_inference_b200.weights import write_random_model

    raw = json.loads(Path(args.config).read_text())
    folder = write_random_model(raw, args.out, args.seed, dtype=args.dtype, std=args.std, norm_std=args.norm_std)
    print(folder)
    return 0


def main(argv: list[str] | None = None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if not argv or argv[0] not in ("generate", "random-model", "-h", "--help"):
        argv.insert(0, "generate")
    ap = argparse.ArgumentParser(prog="python -m oxr_inference_b200", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="command", required=True)

    g = sub.add_parser("generate", help="generate from a model folder (the default command)")
    g.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    g.add_argument("--prompt-ids", action="append", help="token ids, comma or space separated; may be repeated")
    g.add_argument("--prompt", action="append", help="text (needs tokenizer.json); may be repeated")
    g.add_argument("--prompt-file", help="one prompt per line: a JSON list of ids, or text")
    g.add_argument("--max-tokens", type=int, default=16)
    g.add_argument("--temperature", type=float, default=0.0)
    g.add_argument("--seed", type=int, default=0, help="seed of temperature sampling")
    g.add_argument("--repetition-penalty", type=float, default=1.0)
    g.add_argument("--ignore-eos", action="store_true")
    g.add_argument("--dtype", choices=("bfloat16", "float32"), default="bfloat16")
    g.add_argument("--kv-gb", type=float, default=16.0, help="device memory for the paged cache")
    g.add_argument("--num-pages", type=int, default=None, help="pages per cache group (overrides --kv-gb)")
    g.add_argument("--page-size", type=int, default=16)
    g.add_argument("--max-running", type=int, default=256, help="most requests running at a time")
    g.add_argument("--max-waiting", type=int, default=2048, help="most requests queued")
    g.add_argument("--max-step-tokens", type=int, default=8192, help="token budget of one step")
    g.add_argument("--prefill-chunk", type=int, default=2048, help="largest prompt portion in one step")
    g.add_argument("--max-positions", type=int, default=None)
    g.add_argument("--no-cuda-graphs", action="store_true")
    g.add_argument("--limit", type=int, default=0, help="only the first N prompts")
    g.add_argument("--out", help="write results as JSON here")
    g.set_defaults(run=_generate)

    r = sub.add_parser("random-model", help="write config.json and model.safetensors with random weights")
    r.add_argument("--config", required=True, help="a config.json to take the sizes from")
    r.add_argument("--out", required=True)
    r.add_argument("--seed", type=int, default=0)
    r.add_argument("--dtype", choices=("bfloat16", "float32"), default="bfloat16")
    r.add_argument("--std", type=float, default=0.02)
    r.add_argument("--norm-std", type=float, default=0.1)
    r.set_defaults(run=_random_model)

    args = ap.parse_args(argv)
    logging.basicConfig(level=logging.INFO, format="%(asctime)s %(levelname)s %(name)s: %(message)s")
    return args.run(args)


if __name__ == "__main__":
    sys.exit(main())
