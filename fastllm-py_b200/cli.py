"""Command line: generate tokens from a model folder.

In fastllm-py's manner (scripts/generate.py:16-34):

    generate <model_path> [prompt] [n_new=32] [dtype]

prints a load line with the architecture summary, the text (or the token ids),
and `[n tokens in t s = x tok/s]`.  The positional arguments keep the
reference's order and meaning; `dtype` is `bfloat16` (default here; the
reference's fp16/INT4 paths do not exist) or `float32`.  Sampling options carry
the names of `Model.generate` (fastllm_py/model.py:500-504).  The tokenizer is
loaded from the model folder when it has one; without tokenizer files give the
prompt as token ids with --prompt-ids (or --random-prompt N).
"""
from __future__ import annotations

import argparse
import sys
import time


def _tokenizer(model_path):
    from pathlib import Path

    p = Path(model_path)
    if not any((p / f).exists() for f in ("tokenizer.json", "tokenizer.model", "tokenizer_config.json")):
        return None
    try:
        from transformers import AutoTokenizer
        return AutoTokenizer.from_pretrained(str(p))
    except Exception as e:                                      # noqa: BLE001
        print(f"[no tokenizer: {e}]", file=sys.stderr)
        return None


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="generate", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("model_path", help="folder with config.json and *.safetensors")
    ap.add_argument("prompt", nargs="?", default="The capital of France is")
    ap.add_argument("n_new", nargs="?", type=int, default=32, help="tokens to generate")
    ap.add_argument("dtype", nargs="?", default="bfloat16", choices=["bfloat16", "float32", "bf16", "fp32"])
    ap.add_argument("--prompt-ids", help="comma-separated token ids instead of text")
    ap.add_argument("--random-prompt", type=int, metavar="N", help="N random token ids as the prompt")
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--top-p", type=float, default=1.0)
    ap.add_argument("--top-k", type=int, default=0)
    ap.add_argument("--min-p", type=float, default=0.0)
    ap.add_argument("--repetition-penalty", type=float, default=1.0)
    ap.add_argument("--frequency-penalty", type=float, default=0.0)
    ap.add_argument("--presence-penalty", type=float, default=0.0)
    ap.add_argument("--seed", type=int, default=None)
    ap.add_argument("--stop-ids", default="", help="comma-separated token ids that end generation")
    ap.add_argument("--no-graph", action="store_true", help="do not capture decode steps in CUDA graphs")
    ap.add_argument("--page-size", type=int, default=16)
    ap.add_argument("--max-tokens", type=int, default=None, help="cache pool size in tokens")
    ap.add_argument("--max-model-len", type=int, default=None)
    args = ap.parse_args(argv)

    from . import Model

    tok = None
    if args.prompt_ids:
        ids = [int(x) for x in args.prompt_ids.split(",") if x.strip()]
    elif args.random_prompt:
        ids = None
    else:
        tok = _tokenizer(args.model_path)
        if tok is None:
            print("this model folder has no tokenizer; give --prompt-ids or --random-prompt",
                  file=sys.stderr)
            return 2
        ids = list(tok(args.prompt).input_ids)

    t0 = time.time()
    n_prompt = args.random_prompt or len(ids)
    longest = args.max_model_len
    model = Model.load(args.model_path, dtype=args.dtype, page_size=args.page_size,
                       max_tokens=args.max_tokens or max(4096, 2 * (n_prompt + args.n_new)),
                       max_model_len=longest, cuda_graph=not args.no_graph, max_requests=4)
    cfg = model.cfg
    print(f"[load {time.time() - t0:.1f}s] {cfg.architecture}: {cfg.num_layers}L hidden={cfg.hidden_size} "
          f"heads={cfg.num_heads}/{cfg.num_kv_heads} dtype={model.engine_config.dtype}")
    if ids is None:
        import numpy as np

        ids = np.random.default_rng(args.seed or 0).integers(0, cfg.vocab_size, args.random_prompt).tolist()

    stop = [int(x) for x in args.stop_ids.split(",") if x.strip()]
    t0 = time.time()
    out = model.generate(ids, max_new_tokens=args.n_new, temperature=args.temperature,
                         use_graph=not args.no_graph, stop_ids=stop, top_p=args.top_p, top_k=args.top_k,
                         seed=args.seed, min_p=args.min_p, repetition_penalty=args.repetition_penalty,
                         frequency_penalty=args.frequency_penalty, presence_penalty=args.presence_penalty)
    dt = time.time() - t0
    if tok is not None:
        print(tok.decode(ids + out))
    else:
        print(",".join(str(t) for t in out))
    print(f"\n[{len(out)} tokens in {dt:.2f}s = {len(out) / dt:.1f} tok/s]")
    return 0


if __name__ == "__main__":
    sys.exit(main())


def make_model_main(argv=None) -> int:
    """make_model <config.json | model folder> <out folder> [--seed S] [--std X] [--norm-std Y] [--dtype D]

    The random-weights mode from the command line: reads a configuration (the architecture's own
    config.json keys), writes `out/config.json` and `out/model.safetensors` with seeded random
    tensors of the names and shapes the architecture's parts expect.  Needs no GPU; meant for
    small models (tests, replay), since the tensors are made in host memory."""
    import json
    from pathlib import Path

    from .config.registry import architecture_of
    from .weights import write_model_folder

    ap = argparse.ArgumentParser(prog="make_model", description=make_model_main.__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("config", help="a config.json, or a folder that holds one")
    ap.add_argument("out", help="folder to write")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--std", type=float, default=0.02, help="standard deviation of matrices and embeddings")
    ap.add_argument("--norm-std", type=float, default=0.02, help="norm weights are 1 + N(0, this)")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32", "bf16", "fp32"])
    args = ap.parse_args(argv)
    path = Path(args.config)
    if path.is_dir():
        path = path / "config.json"
    raw = json.loads(path.read_text())
    arch = architecture_of(raw)
    config = arch.config_class.from_hf(raw)
    folder = write_model_folder(config, args.out, args.seed, args.std, args.norm_std, args.dtype)
    print(f"wrote {folder}/config.json and model.safetensors ({raw.get('architectures', ['?'])[0]}, seed {args.seed})")
    return 0
