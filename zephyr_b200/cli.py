"""Command line.  The reference has one command, ``zephyr serve`` (python/zephyr/cli.py:38-89);
servers are out of scope here, so this program offers ``generate`` on token ids with the same
option names where the reference has them (--dtype, --max-model-len, --gpu-memory-utilization,
--max-num-seqs, --max-num-batched-tokens, --max-prefill-chunk-tokens, --log-level) and
``random-model`` for the random-weights mode.

    python -m zephyr_b200 generate MODEL --prompt-ids 1,2,3 --max-tokens 16 --temperature 0
    python -m zephyr_b200 random-model --config config.json --seed 0 --out DIR
"""

from __future__ import annotations

import argparse
import json
import logging
import sys
from pathlib import Path


def _positive_int(value: str) -> int:
    parsed = int(value)
    if parsed <= 0:
        raise argparse.ArgumentTypeError("must be positive")
    return parsed


def _ids(value: str) -> list[int]:
    try:
        ids = [int(item) for item in value.replace(",", " ").split()]
    except ValueError as error:
        raise argparse.ArgumentTypeError("use comma- or space-separated token ids") from error
    if not ids:
        raise argparse.ArgumentTypeError("at least one token id is needed")
    return ids


def build_parser() -> argparse.ArgumentParser:
    parser = argparse.ArgumentParser(prog="zephyr_b200", description="Qwen3 inference engine for one B200")
    commands = parser.add_subparsers(dest="command", required=True)

    gen = commands.add_parser("generate", help="Generate from prompts given as token ids")
    gen.add_argument("model", help="Local model directory (config.json + safetensors)")
    source = gen.add_mutually_exclusive_group(required=True)
    source.add_argument("--prompt-ids", type=_ids, action="append", help="one prompt; repeat for a batch")
    source.add_argument("--prompt-file", type=Path, help="one prompt per line, token ids separated by spaces or commas")
    gen.add_argument("--max-tokens", type=_positive_int, default=16)
    gen.add_argument("--temperature", type=float, default=0.0)
    gen.add_argument("--top-k", type=int, default=None)
    gen.add_argument("--top-p", type=float, default=None)
    gen.add_argument("--min-p", type=float, default=None)
    gen.add_argument("--frequency-penalty", type=float, default=None)
    gen.add_argument("--presence-penalty", type=float, default=None)
    gen.add_argument("--repetition-penalty", type=float, default=None)
    gen.add_argument("--top-logprobs", type=int, default=None,
                     help="report each token's log-probability and this many of the most probable tokens (with --json)")
    gen.add_argument("--seed", type=int, default=None, help="sampling seed of each request")
    gen.add_argument("--stop-token-ids", type=_ids, default=[])
    gen.add_argument("--ignore-eos", action="store_true")
    gen.add_argument("--dtype", choices=("bfloat16", "float32"), default="bfloat16")
    gen.add_argument("--max-model-len", type=_positive_int)
    gen.add_argument("--gpu-memory-utilization", type=float, default=0.9)
    gen.add_argument("--max-num-seqs", type=_positive_int)
    gen.add_argument("--max-num-batched-tokens", type=_positive_int)
    gen.add_argument("--max-prefill-chunk-tokens", type=_positive_int)
    gen.add_argument("--kv-block-size", type=_positive_int, default=16)
    gen.add_argument("--num-kv-blocks", type=_positive_int, help="fix the number of cache pages")
    gen.add_argument("--json", action="store_true", help="print one JSON object per request")
    gen.add_argument("--log-level", choices=("critical", "error", "warning", "info", "debug", "trace"), default="warning")

    rand = commands.add_parser("random-model", help="Write a model folder with seeded random weights")
    rand.add_argument("--config", type=Path, required=True, help="a config.json of the architecture")
    rand.add_argument("--seed", type=int, default=0)
    rand.add_argument("--out", type=Path, required=True)
    rand.add_argument("--dtype", choices=("bfloat16", "float32"), default="bfloat16")
    return parser


def _generate(args, parser) -> int:
    if not 0 < args.gpu_memory_utilization <= 1:
        parser.error("--gpu-memory-utilization must be in (0, 1]")
    if args.prompt_file is not None:
        try:
            prompts = [_ids(line) for line in args.prompt_file.read_text().splitlines() if line.strip()]
        except (OSError, argparse.ArgumentTypeError) as error:
            parser.error(f"--prompt-file: {error}")
    else:
        prompts = args.prompt_ids
    levels = {"critical": logging.CRITICAL, "error": logging.ERROR, "warning": logging.WARNING, "info": logging.INFO,
              "debug": logging.DEBUG, "trace": logging.DEBUG}
    logging.basicConfig(level=levels[args.log_level], stream=sys.stderr)

    from .config import ZephyrError
    from .engine import Engine, GenerationParams, KvCacheOptions, PagedSchedulerConfig

    scheduler_args = {key: value for key, value in (
        ("max_num_seqs", args.max_num_seqs), ("max_num_batched_tokens", args.max_num_batched_tokens),
        ("max_prefill_chunk_tokens", args.max_prefill_chunk_tokens)) if value is not None}
    if args.max_num_batched_tokens is not None and args.max_prefill_chunk_tokens is None:
        # As the reference's command line does (python/zephyr/cli.py:131-138).
        scheduler_args["max_prefill_chunk_tokens"] = min(args.max_num_batched_tokens,
                                                         PagedSchedulerConfig().max_prefill_chunk_tokens)
    try:
        engine = Engine(args.model, dtype=args.dtype, max_seq_len=args.max_model_len or 0,
                        gpu_memory_utilization=args.gpu_memory_utilization,
                        scheduler=PagedSchedulerConfig(**scheduler_args),
                        kv_cache=KvCacheOptions(block_size=args.kv_block_size, num_blocks=args.num_kv_blocks))
        params = GenerationParams(max_tokens=args.max_tokens, temperature=args.temperature, top_k=args.top_k,
                                  top_p=args.top_p, min_p=args.min_p, frequency_penalty=args.frequency_penalty,
                                  presence_penalty=args.presence_penalty, repetition_penalty=args.repetition_penalty,
                                  top_logprobs=args.top_logprobs, seed=args.seed,
                                  stop_token_ids=args.stop_token_ids, ignore_eos=args.ignore_eos)
        outputs = engine.generate(prompts, params)
    except (ZephyrError, ValueError, OSError) as error:
        print(f"zephyr_b200: {type(error).__name__}: {error}", file=sys.stderr)
        return 1
    for output in outputs:
        choice = output.choices[0]
        if args.json:
            record = {"request_id": output.request_id, "prompt_token_ids": list(output.prompt_token_ids),
                      "token_ids": list(choice.token_ids),
                      "finish_reason": choice.finish_reason.value if choice.finish_reason else None,
                      "status": output.status.value if output.status else None}
            if choice.logprobs is not None:
                record["logprobs"] = [{"logprob": r.logprob, "top_logprobs": [[t.token_id, t.logprob] for t in r.top_logprobs]}
                                      for r in choice.logprobs]
            print(json.dumps(record))
        else:
            print(" ".join(str(t) for t in choice.token_ids))
    return 0


def _random_model(args, parser) -> int:
    import torch

    from .config import ZephyrError, resolve_architecture
    from .weights import write_random_model

    try:
        data = json.loads(args.config.read_text())
        config = resolve_architecture(data, str(args.config)).config_class.from_dict(data, str(args.config))
        folder = write_random_model(config, args.seed, args.out, dtype=getattr(torch, args.dtype))
    except (ZephyrError, OSError, ValueError) as error:
        print(f"zephyr_b200: {type(error).__name__}: {error}", file=sys.stderr)
        return 1
    print(folder)
    return 0


def main(argv: list[str] | None = None) -> int:
    parser = build_parser()
    args = parser.parse_args(argv)
    if args.command == "generate":
        return _generate(args, parser)
    return _random_model(args, parser)
