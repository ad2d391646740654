"""Runs the UNMODIFIED reference engine (installed under baseline/_ref) on the tiny configuration B and
writes what it generates: greedy tokens and, for every generated token, the log-probability it
reports for every token of the vocabulary (``top_logprobs = vocab``; the reference reports
log-probabilities after penalties and temperature and before filtering, bindings/python/types.cpp:
24-26, src/sampler/sampler.cu:178-194, and a greedy row has temperature 1, src/sampler/sampler.cpp:95).
A full row of log-probabilities is the row of logits up to one constant, so these files pin the
plain implementation of the tests (tests/plain_qwen3.py) on the reference's own arithmetic: NeoX
pairing, norm before rotation, the mapping of query heads to key/value heads, the order of gate and
up, an untied head.

It needs a CUDA device (the reference has no CPU path).  Made with

    python tests/golden/make_reference_golden.py --out tests/golden

on a B200; ``tests/test_reference_anchor.py`` reads the files on any machine and also repeats the
run where the reference is installed and a GPU is present.  Tiny B is the configuration both engines
take: head size 32 and pages of 8 are inside what the reference's decode kernel and cache accept
(src/attention/paged_decode.cu:425-474, src/executor/causal_lm.cpp:439); tiny A (head size 16, pages
of 4) is not.
"""

from __future__ import annotations

import argparse
import hashlib
import json
import sys
import tempfile
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent.parent
PROMPT_LENGTHS = (9, 33, 70)
NEW_TOKENS = 8


def prompts(vocab: int) -> list[list[int]]:
    import random

    return [[random.Random(4000 + n).randrange(vocab) for _ in range(n)] for n in PROMPT_LENGTHS]


def write_tiny_b(folder: Path, dtype: str) -> str:
    """The tiny-B model folder (seed 1) and the SHA-256 of its weight file."""
    import torch

    sys.path.insert(0, str(ROOT))
    sys.path.insert(0, str(ROOT / "tests"))
    from tiny_configs import TINY, tiny_config
    from zephyr_b200.weights import write_random_model

    write_random_model(tiny_config("B"), TINY["B"]["seed"], folder, dtype=getattr(torch, dtype))
    return hashlib.sha256((folder / "model.safetensors").read_bytes()).hexdigest()


def run_reference(folder: Path, dtype: str) -> dict:
    """Greedy generation through ``zephyr._C.Engine`` (submit / wait_for_outputs), one request at a time."""
    sys.path.insert(0, str(ROOT / "baseline" / "_ref"))
    from zephyr import _C

    config = json.loads((folder / "config.json").read_text())
    vocab = config["vocab_size"]
    options = _C.EngineOptions(str(folder), devices=[0], dtype=dtype, max_seq_len=config["max_position_embeddings"],
                               scheduler=_C.PagedSchedulerConfig(max_num_seqs=4, max_num_batched_tokens=64,
                                                                 max_prefill_chunk_tokens=16),
                               eos_token_ids=[])
    native = _C.Engine(options, kv_cache=_C.KvCacheOptions(block_size=8))
    out = {"prompts": prompts(vocab), "tokens": [], "logprobs": []}
    try:
        for prompt in out["prompts"]:
            request = _C.GenerationRequest(prompt, sampling=_C.SamplingParams(temperature=0.0, top_logprobs=vocab),
                                           max_new_tokens=NEW_TOKENS, ignore_eos=True)
            request_id = native.submit(request)
            tokens, rows, done = [], [], False
            while not done:
                for output in native.wait_for_outputs():
                    assert output.request_id == request_id
                    for choice in output.result:
                        for result in choice.tokens:
                            tokens.append(int(result.token_id))
                            row = [float("nan")] * vocab
                            for item in result.logprobs.top_logprobs:
                                row[int(item.token_id)] = float(item.logprob)
                            rows.append(row)
                    if output.status is not None:
                        if output.status != _C.RequestStatus.COMPLETED:
                            raise RuntimeError(f"the reference ended a request with {output.status}: {output.error_message}")
                        done = True
            assert len(tokens) == NEW_TOKENS
            out["tokens"].append(tokens)
            out["logprobs"].append(rows)
    finally:
        native.close()
    return out


def main() -> int:
    import numpy as np

    parser = argparse.ArgumentParser()
    parser.add_argument("--out", required=True)
    parser.add_argument("--dtypes", default="bfloat16,float32")
    args = parser.parse_args()
    out_dir = Path(args.out)
    out_dir.mkdir(parents=True, exist_ok=True)
    for dtype in args.dtypes.split(","):
        with tempfile.TemporaryDirectory() as tmp:
            folder = Path(tmp) / f"tiny_b_{dtype}"
            digest = write_tiny_b(folder, dtype)
            result = run_reference(folder, dtype)
        np.savez_compressed(out_dir / f"reference_tiny_b_{dtype}.npz",
                            tokens=np.asarray(result["tokens"], dtype=np.int32),
                            logprobs=np.asarray(result["logprobs"], dtype=np.float32),
                            prompt_lengths=np.asarray(PROMPT_LENGTHS, dtype=np.int32),
                            weights_sha256=np.asarray(digest))
        print(f"{dtype}: tokens {result['tokens']}; weights {digest[:16]}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
