"""Command line: ``python -m cuinfer_b200 generate --model DIR --prompt-ids 1,2,3``.

The reference's command line has one sub-command, ``serve`` (cuinfer/__main__.py:48-66); the HTTP server is
not built here, so the sub-command is ``generate``.  Engine options keep the reference's names, defaults and
meanings: ``--model``, ``--gpu-memory-utilization`` (0.8), ``--block-size`` (16),
``--max-num-scheduled-tokens`` (8192), ``--max-num-seqs`` (256), ``--disable-cuda-graph``.  Request options are
the fields its requests carry (csrc/engine/protocol.h:39-49): ``--max-tokens``, ``--temperature``,
``--top-k``, ``--top-p``, ``--ignore-eos``.  Output: one JSON line per prompt with the generated token ids.
"""
from __future__ import annotations

import argparse
import json
import sys
import tempfile


def _parse_ids(text: str) -> list[int]:
    try:
        return [int(t) for t in text.replace(",", " ").split()]
    except ValueError:
        raise argparse.ArgumentTypeError(f"token ids must be integers, got {text!r}") from None


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(prog="python -m cuinfer_b200")
    commands = parser.add_subparsers(dest="command", required=True)
    g = commands.add_parser("generate", help="generate token ids for prompts given as token ids")
    src = g.add_mutually_exclusive_group(required=True)
    src.add_argument("--model", help="folder with config.json and model.safetensors")
    src.add_argument("--random-config", help="config.json of a model to create with random weights (see --seed)")
    g.add_argument("--seed", type=int, default=0, help="seed of random weights and of sampling")
    g.add_argument("--prompt-ids", action="append", type=_parse_ids, default=[],
                   help='one prompt as token ids, "1,2,3"; may be repeated')
    g.add_argument("--prompt-file", help="file with one prompt per line, token ids separated by spaces or commas")
    g.add_argument("--max-tokens", type=int, default=16)
    g.add_argument("--temperature", type=float, default=1.0)
    g.add_argument("--top-k", type=int, default=0)
    g.add_argument("--top-p", type=float, default=1.0)
    g.add_argument("--ignore-eos", action="store_true")
    g.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    g.add_argument("--gpu-memory-utilization", type=float, default=0.8)
    g.add_argument("--block-size", type=int, default=16)
    g.add_argument("--num-blocks", type=int, default=None, help="cache pages; default: from free memory")
    g.add_argument("--max-num-scheduled-tokens", type=int, default=8192)
    g.add_argument("--max-num-seqs", type=int, default=256)
    g.add_argument("--disable-cuda-graph", action="store_true")
    g.add_argument("--disable-run-ahead", action="store_true",
                   help="wait for a decode step's tokens before launching the next one")
    args = parser.parse_args(argv)

    from .config import ConfigError, EngineConfig
    from .sampling import SamplingParams

    prompts = list(args.prompt_ids)
    if args.prompt_file:
        with open(args.prompt_file) as fh:
            prompts += [_parse_ids(line) for line in fh if line.strip()]
    if not prompts:
        parser.error("give at least one prompt with --prompt-ids or --prompt-file")
    try:
        options = dict(gpu_memory_utilization=args.gpu_memory_utilization, block_size=args.block_size,
                       max_num_scheduled_tokens=args.max_num_scheduled_tokens, max_num_seqs=args.max_num_seqs,
                       enable_cuda_graph=not args.disable_cuda_graph, decode_run_ahead=not args.disable_run_ahead, dtype=args.dtype, num_blocks=args.num_blocks,
                       seed=args.seed)
        EngineConfig(model_path=args.model or "", **options)
        params = SamplingParams(temperature=args.temperature, top_k=args.top_k, top_p=args.top_p,
                                max_tokens=args.max_tokens, ignore_eos=args.ignore_eos)
    except (ConfigError, ValueError) as exc:
        parser.error(str(exc))

    from .engine.llm import LLM

    model_dir = args.model
    tmp = None
    if args.random_config:
        from .weights import write_random_model
        with open(args.random_config) as fh:
            raw = json.load(fh)
        tmp = tempfile.TemporaryDirectory(prefix="cuinfer_b200_random_")
        model_dir = write_random_model(tmp.name, raw, args.seed, dtype=args.dtype)
    try:
        llm = LLM(model_dir, **options)
        for res in llm.generate(prompts, params):
            print(json.dumps({"request_id": res.request_id, "prompt_token_ids": res.prompt_token_ids,
                              "token_ids": res.token_ids, "finish_reason": res.finish_reason}), flush=True)
    except (ConfigError, ValueError) as exc:
        print(f"error: {exc}", file=sys.stderr)
        return 1
    finally:
        if tmp is not None:
            tmp.cleanup()
    return 0


if __name__ == "__main__":
    sys.exit(main())
