"""The command line without a GPU: parsing, the random-model command, and clear errors."""

import json

import pytest

from tiny_configs import tiny_config
from zephyr_b200.cli import build_parser, main
from zephyr_b200.weights import Checkpoint


def test_generate_options_carry_the_reference_names():
    args = build_parser().parse_args(
        ["generate", "/m", "--prompt-ids", "1,2,3", "--prompt-ids", "4 5", "--max-tokens", "7", "--temperature", "0.7",
         "--seed", "3", "--dtype", "float32", "--max-model-len", "128", "--gpu-memory-utilization", "0.5",
         "--max-num-seqs", "4", "--max-num-batched-tokens", "64", "--max-prefill-chunk-tokens", "16", "--ignore-eos",
         "--log-level", "debug"])
    assert args.prompt_ids == [[1, 2, 3], [4, 5]] and args.max_tokens == 7 and args.dtype == "float32"
    assert (args.max_model_len, args.max_num_seqs, args.max_num_batched_tokens, args.max_prefill_chunk_tokens) == \
        (128, 4, 64, 16)
    with pytest.raises(SystemExit):
        build_parser().parse_args(["generate", "/m"])                         # a prompt is required
    with pytest.raises(SystemExit):
        build_parser().parse_args(["generate", "/m", "--prompt-ids", "a,b"])
    with pytest.raises(SystemExit):
        build_parser().parse_args(["generate", "/m", "--prompt-ids", "1", "--dtype", "float16"])


def test_random_model_command(tmp_path, capsys):
    (tmp_path / "c.json").write_text(json.dumps(tiny_config("A").to_dict()))
    assert main(["random-model", "--config", str(tmp_path / "c.json"), "--seed", "5", "--out", str(tmp_path / "m")]) == 0
    assert (tmp_path / "m" / "config.json").exists()
    assert "model.embed_tokens.weight" in Checkpoint(tmp_path / "m").names()
    (tmp_path / "bad.json").write_text(json.dumps({"model_type": "other"}))
    assert main(["random-model", "--config", str(tmp_path / "bad.json"), "--out", str(tmp_path / "n")]) == 1
    assert "unsupported model configuration" in capsys.readouterr().err


def test_only_the_commands_that_are_built_are_offered():
    with pytest.raises(SystemExit):
        main(["serve"])
