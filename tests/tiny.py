"""The tiny configurations the tests run on.

tiny_a and tiny_b differ in every size and option: layer count, width (neither
a power of two in b), head count and grouping (MHA / GQA 3:1), head size, the
feed-forward width (172 and 264 are multiples of neither 16 nor 64, and a
bfloat16 row of 172 is not a multiple of 16 bytes), vocabulary, rope base and
scaling, the norms' eps, tied / untied embeddings, the spread of the weights,
and the cache page size they are run with.  tiny_c adds a larger head size that
is not a power of two and GQA 2:1.
"""
from __future__ import annotations

import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

from fastllm_py_b200.config import LinearRopeScaling, LlamaConfig  # noqa: E402
from fastllm_py_b200.weights import write_model_folder  # noqa: E402

CONFIGS = {
    "tiny_a": dict(
        config=LlamaConfig(
            architecture="LlamaForCausalLM", num_layers=2, hidden_size=64, num_heads=4,
            num_kv_heads=4, head_dim=16, intermediate_size=172, vocab_size=256, rope_theta=10000.0,
            rope_scaling=None, rms_norm_eps=1e-6, max_position_embeddings=128,
            tie_word_embeddings=False),
        seed=11, std=0.02, norm_std=0.02, page_size=16),
    "tiny_b": dict(
        config=LlamaConfig(
            architecture="LlamaForCausalLM", num_layers=3, hidden_size=96, num_heads=6,
            num_kv_heads=2, head_dim=16, intermediate_size=264, vocab_size=320, rope_theta=100000.0,
            rope_scaling=LinearRopeScaling(4.0), rms_norm_eps=1e-5, max_position_embeddings=256,
            tie_word_embeddings=True),
        seed=23, std=0.03, norm_std=0.05, page_size=8),
    "tiny_c": dict(
        config=LlamaConfig(
            architecture="LlamaForCausalLM", num_layers=2, hidden_size=200, num_heads=4,
            num_kv_heads=2, head_dim=48, intermediate_size=328, vocab_size=515, rope_theta=50000.0,
            rope_scaling=LinearRopeScaling(2.0), rms_norm_eps=3e-6, max_position_embeddings=512,
            tie_word_embeddings=False),
        seed=37, std=0.05, norm_std=0.1, page_size=32),
}


def write(name: str, folder, dtype: str = "bfloat16"):
    c = CONFIGS[name]
    return write_model_folder(c["config"], folder, c["seed"], c["std"], c["norm_std"], dtype)
