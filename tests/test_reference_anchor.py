"""The plain implementation of the tests, pinned on the reference's own output.

``tests/golden/reference_tiny_b_<dtype>.npz`` hold what the unmodified reference engine generated
on a B200 from the tiny configuration B (made by tests/golden/make_reference_golden.py): greedy
tokens for prompts of 9, 33 and 70 tokens and, for each generated token, the log-probability of every
token of the vocabulary.  A full row of log-probabilities is the row of logits up to a constant, so
comparing it with ``log_softmax`` of the plain logits pins every formula of the plain
implementation (pairing of the rotation, norm before rotation, query-to-key/value head mapping,
gate/up order, the untied head) on something other than a reading of the reference.

Tolerances.  In bfloat16 the reference rounds hidden states, rotation and activation products to
bfloat16 between operations and stores its logits in bfloat16 (src/model/causal_lm/qwen3.cpp:175-180):
one unit in the last place is 2^-8 of the value, and the rows' largest |log-probability| is about 6,
so a rounding of the logit alone moves a log-probability by up to 0.012; the bound is 0.03 (seen:
5.4e-3).  Its "float32" runs every product in TF32 (10 bits of mantissa, src/layer/linear.cpp:22-24
with deps/ttl matmul's default): relative 2^-11 per product input over three layers; the bound is
3e-3 (seen: 6.0e-4).  Both bounds are far below what a wrong formula moves (tenths to units).

The first test needs no GPU.  The second repeats the reference run where it is installed
(baseline/_ref) and a GPU is present, and compares the fresh output with the stored one."""

import hashlib
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

from plain_qwen3 import load_model_folder, plain_forward

GOLDEN = Path(__file__).resolve().parent / "golden"
ROOT = Path(__file__).resolve().parent.parent
BOUNDS = {"bfloat16": 0.03, "float32": 3e-3}


def golden(dtype):
    path = GOLDEN / f"reference_tiny_b_{dtype}.npz"
    if not path.exists():
        pytest.skip(f"{path.name} has not been made (tests/golden/make_reference_golden.py needs a GPU)")
    return np.load(path)


def compare_with_plain(data, folder, dtype):
    sys.path.insert(0, str(GOLDEN))
    from make_reference_golden import NEW_TOKENS, prompts

    config, weights = load_model_folder(folder)
    worst = 0.0
    for index, prompt in enumerate(prompts(config["vocab_size"])):
        tokens = list(prompt)
        for step in range(NEW_TOKENS):
            logits = plain_forward(config, weights, tokens)[-1]
            expected = torch.log_softmax(logits, dim=-1).numpy()
            got = data["logprobs"][index][step].astype(np.float64)
            assert np.isfinite(got).all(), "the reference did not report the whole vocabulary"
            error = float(np.abs(got - expected).max())
            worst = max(worst, error)
            assert error <= BOUNDS[dtype], f"prompt {index} token {step}: log-probabilities differ by {error:.3e}"
            # The reference's own greedy choice is the best token of its own row; the plain best agrees
            # unless the two best plain log-probabilities lie closer than the bound.
            token = int(data["tokens"][index][step])
            assert token == int(np.argmax(got))
            best = np.sort(expected)[-2:]
            assert token == int(np.argmax(expected)) or best[1] - best[0] <= 2 * BOUNDS[dtype]
            tokens.append(token)          # follow the reference's sequence
    print(f"[anchor] {dtype}: worst log-probability difference {worst:.3e} (bound {BOUNDS[dtype]:.0e})")


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_plain_implementation_matches_the_reference_output(dtype, tmp_path):
    sys.path.insert(0, str(GOLDEN))
    from make_reference_golden import write_tiny_b

    data = golden(dtype)
    folder = tmp_path / "tiny_b"
    digest = write_tiny_b(folder, dtype)
    if digest != str(data["weights_sha256"]):
        pytest.skip("this machine's seeded random weights differ from those the stored output was made with")
    compare_with_plain(data, folder, dtype)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_reference_run_again(dtype, tmp_path, cuda_device):
    if not (ROOT / "baseline" / "_ref" / "zephyr").is_dir():
        pytest.skip("the reference is not installed under baseline/_ref")
    done = subprocess.run([sys.executable, str(GOLDEN / "make_reference_golden.py"), "--out", str(tmp_path), "--dtypes", dtype],
                          capture_output=True, text=True, timeout=900)
    if done.returncode != 0 and "cannot import" in done.stderr + done.stdout:
        pytest.skip("the installed reference does not import here")
    assert done.returncode == 0, done.stderr[-3000:]
    fresh = np.load(tmp_path / f"reference_tiny_b_{dtype}.npz")
    sys.path.insert(0, str(GOLDEN))
    from make_reference_golden import write_tiny_b

    folder = tmp_path / "tiny_b"
    assert write_tiny_b(folder, dtype) == str(fresh["weights_sha256"])
    compare_with_plain(fresh, folder, dtype)
    stored = GOLDEN / f"reference_tiny_b_{dtype}.npz"
    if stored.exists() and str(np.load(stored)["weights_sha256"]) == str(fresh["weights_sha256"]):
        assert np.array_equal(np.load(stored)["tokens"], fresh["tokens"])
