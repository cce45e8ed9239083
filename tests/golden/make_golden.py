#!/usr/bin/env python
"""Writes tests/golden/<name>.npz from codemk8/fastllm-py's own model code, on the CPU.

    python tests/golden/make_golden.py [path/to/fastllm-py checkout]

fastllm_py imports CuPy lazily, inside functions; with a small stand-in module
named `cupy` that maps onto NumPy, `Model.load(dir, DeviceMap({"cpu": 1}),
dtype="float32")`, `Model.forward` and `Model.generate(use_graph=False)` run
wholly in NumPy.  For each tiny configuration this script writes a model folder
with the engine's random-weights mode (tests/tiny.py), runs the reference on a
fixed token sequence, and stores: the token ids, the float32 logits at every
position, 8 greedy tokens, 8 tokens sampled at temperature 0.7 with seed 5, and
a checksum of the weights (so that a test can tell "the model differs" from "the
plain implementation differs").  tests/test_plain.py compares the plain
implementation with these files.
"""
import sys
import tempfile
import types
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent))
sys.path.insert(0, str(HERE.parent.parent))


def cupy_stand_in():
    cp = types.ModuleType("cupy")
    cp.ndarray = type("ndarray", (), {})            # nothing is ever an instance of it
    cp.asnumpy = lambda x: np.asarray(x)
    cp.asarray = lambda x: np.asarray(x)
    cp.float32, cp.float16 = np.float32, np.float16
    return cp


def weights_checksum(folder):
    import torch
    from safetensors.torch import load_file

    w = load_file(str(Path(folder) / "model.safetensors"))
    return float(sum(t.to(torch.float64).abs().sum() for _, t in sorted(w.items())))


def token_ids(name, vocab, n):
    rng = np.random.default_rng(sum(map(ord, name)))
    return rng.integers(0, vocab, size=n).astype(np.int64)


def main():
    if len(sys.argv) != 2:
        sys.exit("usage: make_golden.py PATH_TO_A_CHECKOUT_OF_fastllm-py")
    ref = Path(sys.argv[1])
    sys.path.insert(0, str(ref))
    sys.modules["cupy"] = cupy_stand_in()
    from fastllm_py import DeviceMap, Model

    import tiny

    for name, spec in tiny.CONFIGS.items():
        with tempfile.TemporaryDirectory() as tmp:
            folder = tiny.write(name, Path(tmp) / name)
            cfg = spec["config"]
            ids = token_ids(name, cfg.vocab_size, 40)
            model = Model.load(str(folder), DeviceMap({"cpu": 1}), dtype="float32")
            logits, _ = model.forward(ids)
            greedy = model.generate(ids[:12], max_new_tokens=8, use_graph=False)
            sampled = model.generate(ids[:12], max_new_tokens=8, temperature=0.7, seed=5,
                                     use_graph=False)
            out = HERE / f"{name}.npz"
            np.savez_compressed(out, ids=ids, logits=np.asarray(logits, dtype=np.float32),
                                greedy=np.asarray(greedy), sampled=np.asarray(sampled),
                                checksum=np.float64(weights_checksum(folder)))
            print("wrote", out, logits.shape, greedy, sampled)


if __name__ == "__main__":
    main()
