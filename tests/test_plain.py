"""The plain implementation against codemk8/fastllm-py's own model code.

tests/golden/*.npz were written by tests/golden/make_golden.py, which runs the
reference's `Model.forward` / `Model.generate` in NumPy on the tiny random
models.  The plain implementation (tests/plain_llama.py) must reproduce them:
it is the oracle of every engine test, so it is checked against the original
once, here.
"""
from pathlib import Path

import numpy as np
import pytest
import torch

import plain_llama as plain
import tiny

GOLDEN = Path(__file__).resolve().parent / "golden"


def _load(name, model_folders):
    g = np.load(GOLDEN / f"{name}.npz")
    weights, config = plain.load_folder(model_folders[name])
    checksum = float(sum(t.to(torch.float64).abs().sum() for _, t in sorted(weights.items())))
    if abs(checksum - float(g["checksum"])) > 1e-6 * abs(checksum):
        pytest.skip("this torch draws other random weights than the one the golden files were made with")
    return g, weights, config


@pytest.mark.parametrize("name", list(tiny.CONFIGS))
def test_logits_match_reference(name, model_folders):
    g, weights, config = _load(name, model_folders)
    logits = plain.forward(weights, config, g["ids"]).numpy()
    assert logits.shape == g["logits"].shape
    assert np.array_equal(logits.argmax(-1), g["logits"].argmax(-1))
    assert np.abs(logits - g["logits"]).max() < 2e-5


@pytest.mark.parametrize("name", list(tiny.CONFIGS))
def test_generation_matches_reference(name, model_folders):
    g, weights, config = _load(name, model_folders)
    prompt = g["ids"][:12].tolist()
    assert plain.generate(weights, config, prompt, 8) == g["greedy"].tolist()
    assert plain.generate(weights, config, prompt, 8, temperature=0.7, seed=5) == g["sampled"].tolist()


def test_float64_is_close_to_float32(model_folders):
    weights, config = plain.load_folder(model_folders["tiny_c"])
    ids = torch.arange(30) % config["vocab_size"]
    a = plain.forward(weights, config, ids)
    b = plain.forward(weights, config, ids, dtype=torch.float64)
    assert (a - b).abs().max() < 1e-4


def test_sampler_filters():
    torch.manual_seed(0)
    logits = torch.randn(50) * 3
    p = plain.probabilities(logits, 0.8, top_k=5)
    assert int((p > 0).sum()) == 5 and abs(float(p.sum()) - 1) < 1e-12
    p = plain.probabilities(logits, 1.0, min_p=0.2)
    full = plain.probabilities(logits, 1.0)
    assert set(torch.nonzero(p).flatten().tolist()) == \
        set(torch.nonzero(full >= 0.2 * full.max()).flatten().tolist())
    p = plain.probabilities(logits, 1.0, top_p=0.5)
    order = torch.argsort(full, descending=True)
    csum = torch.cumsum(full[order], 0)
    k = int((csum <= 0.5).sum()) + 1                      # the token that crosses 0.5 is kept
    assert set(torch.nonzero(p).flatten().tolist()) == set(order[:k].tolist())
    assert plain.sample(logits) == int(logits.argmax())
    counts = {3: 2, 7: 1}
    out = plain.apply_penalties(logits, counts, 1.5, 0.1, 0.2)
    for t, c in counts.items():
        x = float(logits[t])
        want = (x / 1.5 if x > 0 else x * 1.5) - (0.1 * c + 0.2)
        assert abs(float(out[t]) - want) < 1e-6
