"""The plain implementation against logits that the reference's own CUDA kernels produced
(``tests/golden/make_reference_golden.py``, run once on a GPU; outputs committed beside it).
This pins the oracle on something that is not this repository's reading of the formulas:
pairing of the rotation, grouped heads, causal rule, eps inside the root, weight last, SiLU,
tying by absence.  The llama3 frequency scaling is in no file of the reference and stays pinned
by its formula alone."""
import hashlib
import json
import os

import numpy as np
import pytest
import torch

import plain_llama
from golden_configs import GOLDEN, tokens_for
from helpers import load_weights, make_model_folder

GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
# 32-bit kernels with their own transcendental routines against float64: a few 1e-6 per
# operation, some tens of operations deep
TOLERANCE = 1e-4


@pytest.mark.parametrize("name", sorted(GOLDEN))
def test_plain_implementation_matches_the_reference_kernels(name, tmp_path):
    path = os.path.join(GOLDEN_DIR, f"reference_logits_{name}.npz")
    assert os.path.isfile(path), f"{path} is missing: run tests/golden/make_reference_golden.py on a GPU"
    gold = np.load(path)
    cfg, seed = GOLDEN[name]
    assert json.loads(str(gold["config"])) == json.loads(json.dumps(cfg, sort_keys=True))
    tokens = tokens_for(name)
    assert gold["tokens"].tolist() == tokens
    folder = make_model_folder(str(tmp_path / name), cfg, seed, "float32")
    with open(os.path.join(folder, "model.safetensors"), "rb") as f:
        sha = hashlib.sha256(f.read()).hexdigest()
    if sha != str(gold["weights_sha256"]):
        pytest.skip("this torch build draws other random weights than the one the golden files were made with")
    ours = plain_llama.llama_forward(cfg, load_weights(folder), tokens, torch.float64).numpy()
    ref = gold["logits"].astype(np.float64)
    assert ours.shape == ref.shape
    err = np.abs(ours - ref).max() / np.abs(ref).max()
    assert err < TOLERANCE, f"{name}: the plain implementation is {err:.2e} off the reference's kernels"
    # and the choice of token agrees wherever the reference's top two are not a near tie
    top2 = np.sort(ref, axis=1)[:, -2:]
    clear = (top2[:, 1] - top2[:, 0]) > 10 * TOLERANCE * np.abs(ref).max()
    assert (ours.argmax(1)[clear] == ref.argmax(1)[clear]).all()
