"""Times every candidate of the tensor-core product's plan on the GPU at hand and writes one JSON line per
problem: {"m", "n", "k", "cands": [[token tile code, K splits, us with the reduce kernel, us with the partial
sums left to the consumer], ...]}.  Token tile codes as fl_gemm_tc takes them: 64, 128, 256 (one-tile kernel),
640 and 512 (CTA pairs, 128 and 256 tokens wide).  Timed as ten launches in a CUDA graph over rotating copies
of the weights (larger than L2 together).

    python tests/data/measure_gemm_candidates.py OUT.jsonl [token counts, comma separated]
    python tests/data/measure_gemm_candidates.py --planned     # the planned products against cuBLAS, as a table

gemm_candidates_b200.jsonl beside this file is its output on one B200 for the token counts 80, 128, 192, 256,
384, 512, 768 and 96, 160, 320, 448, 640, 1024; tests/test_bench_and_loading.py holds the plan against it, and
the constants of the plan's cost model (tc_cost in csrc/gemm_tcgen05.cu) were fitted to it.
"""
import json
import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))
from fastllm_py_b200.native import gemm_tc  # noqa: E402

WEIGHTS = [(4096, 4096), (4096, 11008), (12288, 4096), (2048, 2048), (2048, 5504), (6144, 2048), (8192, 8192),
           (8192, 22016), (10240, 8192), (5120, 5120), (5120, 13824), (102400, 4096)]


def timed(fn, reps=10):
    graph = torch.cuda.CUDAGraph()
    fn(0)
    torch.cuda.synchronize()
    with torch.cuda.graph(graph):
        for i in range(reps):
            fn(i)
    graph.replay()
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    graph.replay()
    end.record()
    torch.cuda.synchronize()
    return start.elapsed_time(end) * 1000 / reps


def planned_against_cublas():
    """o, down and q|k|v of DeepSeek-LLM-7B at 128, 256 and 512 tokens: cuBLAS (torch.matmul), the planned product
    with its reduce kernel, and the planned product whose partial sums are left to the consumer; microseconds
    (best of three replays of 20 launches) and the ratio to cuBLAS."""
    dev = torch.device("cuda:0")
    print("| product | tokens | cuBLAS us | plan: us (x cuBLAS) | plan with sums left to the consumer: us (x cuBLAS) |")
    print("|---|---|---|---|---|")
    for name, (n, k) in (("o", (4096, 4096)), ("down", (4096, 11008)), ("q|k|v", (12288, 4096))):
        copies = max(2, int(600e6 // (n * k * 2)) + 1)
        row_major = [torch.randn(n, k, device=dev, dtype=torch.bfloat16) * 0.05 for _ in range(copies)]
        packed = [gemm_tc.PackedWeight(w) for w in row_major]
        for m in (128, 256, 512):
            a = torch.randn(m, k, device=dev, dtype=torch.bfloat16)
            out = torch.empty(m, n, device=dev, dtype=torch.bfloat16)
            best = lambda fn: min(timed(fn, 20) for _ in range(3))
            cublas = best(lambda i: torch.matmul(a, row_major[i % copies].t(), out=out))
            t = best(lambda i: gemm_tc.gemm(a, packed[i % copies], out))
            t_deferred = best(lambda i: gemm_tc.gemm(a, packed[i % copies], out, defer=True))
            p, pd = gemm_tc.plan(m, n, k, 148), gemm_tc.plan(m, n, k, 148, True)
            print(f"| {name} | {m} | {cublas:.1f} | {p[0]}/{p[1]}: {t:.1f} ({t / cublas:.2f}) | "
                  f"{pd[0]}/{pd[1]}: {t_deferred:.1f} ({t_deferred / cublas:.2f}) |", flush=True)
        del packed, row_major


def main():
    if sys.argv[1] == "--planned":
        planned_against_cublas()
        return
    out_path = sys.argv[1]
    counts = [int(x) for x in sys.argv[2].split(",")] if len(sys.argv) > 2 else [80, 128, 192, 256, 384, 512, 768]
    dev = torch.device("cuda:0")
    with open(out_path, "w") as out_file:
        for n, k in WEIGHTS:
            copies = max(2, min(8, int(400e6 // (n * k * 2)) + 1))
            weights = [gemm_tc.PackedWeight(torch.randn(n, k, device=dev, dtype=torch.bfloat16) * 0.05)
                       for _ in range(copies)]
            k_blocks = -(-k // 64)
            for m in counts:
                if n > 50000 and m > 256:
                    continue
                a = torch.randn(m, k, device=dev, dtype=torch.bfloat16)
                out = torch.empty(m, n, device=dev, dtype=torch.bfloat16)
                record = {"m": m, "n": n, "k": k, "cands": []}
                for bn in (64, 128, 256, 640, 512):
                    if bn in (64, 640) and m > 256:
                        continue
                    for splits in (1, 2, 3, 4, 6, 8, 12, 16):
                        per = -(-k_blocks // splits)
                        if -(-k_blocks // per) != splits or (splits > 1 and per < 4) or splits * m * n * 4 > 600e6:
                            continue
                        t = timed(lambda i: gemm_tc.gemm(a, weights[i % copies], out, bn, splits))
                        t_deferred = t if splits == 1 else \
                            timed(lambda i: gemm_tc.gemm(a, weights[i % copies], out, bn, splits, defer=True))
                        record["cands"].append([bn, splits, round(t, 2), round(t_deferred, 2)])
                out_file.write(json.dumps(record, separators=(",", ":")) + "\n")
                out_file.flush()
            del weights


if __name__ == "__main__":
    main()
