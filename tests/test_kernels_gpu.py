"""Each CUDA kernel alone against a plain torch float32 reference of the same
operation, at sizes other than the models' (odd widths, tails, many shapes)."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def bf16_round(x):
    return x.to(torch.bfloat16).to(torch.float32)


# ----------------------------------------------------------------------- GEMM

GEMM_SHAPES = [(1, 128, 64), (3, 96, 96), (7, 32, 172), (16, 320, 264), (17, 515, 200), (33, 130, 72),
               (64, 256, 1024), (100, 384, 328), (129, 640, 512), (300, 257, 136), (513, 128, 64)]


@pytest.mark.parametrize("m, n, k", GEMM_SHAPES)
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_tensor_core_gemm(m, n, k, out_dtype):
    from fastllm_py_b200.native import gemm_tc

    g = torch.Generator(device="cpu").manual_seed(m * 1000 + n + k)
    a = torch.randn(m, k, generator=g).to(torch.bfloat16)
    w = torch.randn(n, k, generator=g).to(torch.bfloat16)
    ref = a.float() @ w.float().t()
    pitch = -(-k // 8) * 8
    a_dev = torch.zeros(m, pitch, dtype=torch.bfloat16, device=DEV)
    a_dev[:, :k] = a.to(DEV)
    a_dev[:, k:] = 7.0                                # padding must never be read
    lin = gemm_tc.TensorCoreLinear(w.to(DEV))
    out = torch.full((m, n + 3), -5.0, dtype=out_dtype, device=DEV)
    lin.forward(a_dev[:, :k], out[:, :n])
    torch.cuda.synchronize()
    assert int(gemm_tc.status_word(torch.device(DEV)).item()) == 0
    got = out[:, :n].float().cpu()
    assert torch.all(out[:, n:] == -5.0), "wrote outside the output columns"
    tol = 1e-3 * math.sqrt(k) if out_dtype == torch.float32 else 2 ** -8 * float(ref.abs().max()) + 1e-3
    assert float((got - ref).abs().max()) <= tol


@pytest.mark.parametrize("bn, splits", [(16, 1), (16, 4), (32, 3), (64, 2), (128, 1), (128, 6), (256, 1), (256, 2), (16, 12)])
def test_tensor_core_gemm_every_tile_and_split(bn, splits):
    """Every tile width and split count, forced, against float32."""
    from fastllm_py_b200.native import gemm_tc

    m, n, k = min(bn, 200) + 5, 300, 64 * 11 + 24
    g = torch.Generator(device="cpu").manual_seed(bn + splits)
    a = torch.randn(m, k, generator=g).to(torch.bfloat16)
    w = torch.randn(n, k, generator=g).to(torch.bfloat16)
    ref = a.float() @ w.float().t()
    out = torch.zeros(m, n, dtype=torch.float32, device=DEV)
    gemm_tc.gemm(a.to(DEV), w.to(DEV), out, bn=bn, splits=splits)
    torch.cuda.synchronize()
    assert int(gemm_tc.status_word(torch.device(DEV)).item()) == 0
    assert float((out.cpu() - ref).abs().max()) <= 1e-3 * math.sqrt(k)


@pytest.mark.parametrize("a_dt, w_dt, c_dt", [(torch.float32, torch.float32, torch.float32),
                                              (torch.float32, torch.bfloat16, torch.float32),
                                              (torch.bfloat16, torch.float32, torch.bfloat16),
                                              (torch.bfloat16, torch.bfloat16, torch.float32)])
def test_cuda_core_gemm(a_dt, w_dt, c_dt):
    from fastllm_py_b200.native import ops

    for m, n, k in [(1, 7, 5), (5, 130, 172), (70, 65, 33), (129, 320, 264)]:
        a = torch.randn(m, k).to(a_dt)
        w = torch.randn(n, k).to(w_dt)
        ref = a.double() @ w.double().t()
        out = torch.zeros(m, n, dtype=c_dt, device=DEV)
        ops.gemm_simt(a.to(DEV), w.to(DEV), out)
        tol = 1e-5 * math.sqrt(k) * 4 if c_dt == torch.float32 else 2 ** -8 * float(ref.abs().max()) + 1e-3
        assert float((out.double().cpu() - ref).abs().max()) <= tol
