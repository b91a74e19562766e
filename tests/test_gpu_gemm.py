"""The hand-written tcgen05 / TMEM / TMA GEMM against a PyTorch fp32 reference."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (128, 256, 512), (256, 512, 1024), (1024, 1024, 1024),
                                    (2048, 3072, 1024), (4096, 1024, 4096), (8192, 2048, 1024)])
def test_gemm_matches_fp32_reference(m, n, k):
    from dfccl_b200.ops import gemm
    torch.manual_seed(m + n + k)
    a = torch.randn(m, k, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(n, k, device="cuda", dtype=torch.bfloat16)
    c = gemm.matmul_nt(a, b)
    torch.cuda.synchronize()
    assert gemm.check_kernels()
    ref = a.float() @ b.float().t()
    err = (c.float() - ref).abs().max().item()
    scale = ref.abs().max().item()
    assert err <= 1e-2 * scale + 1e-2, (err, scale)
    # the second call reuses tensor memory and barriers of a fresh launch
    c2 = gemm.matmul_nt(a, b)
    torch.cuda.synchronize()
    assert torch.equal(c, c2)


@pytest.mark.parametrize("a_t,b_t", [(False, True), (True, False), (True, True)])
@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (256, 512, 192), (1024, 1024, 2048), (1536, 1024, 8192)])
def test_gemm_reads_transposed_operands_in_place(m, n, k, a_t, b_t):
    """Operands stored with the contraction index slow (A as [K, M], B as [K, N]) are described to the tensor cores as
    MN-major and read as they are: the data gradient (B transposed) and the weight gradient (both) of a linear layer."""
    from dfccl_b200.ops import gemm
    torch.manual_seed(m * 3 + n * 5 + k)
    a = torch.randn(m, k, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(n, k, device="cuda", dtype=torch.bfloat16)
    a_in = a.t().contiguous() if a_t else a
    b_in = b.t().contiguous() if b_t else b
    c = gemm.matmul(a_in, b_in, a_transposed=a_t, b_transposed=b_t)
    torch.cuda.synchronize()
    assert gemm.check_kernels()
    ref = a.float() @ b.float().t()
    err = (c.float() - ref).abs().max().item()
    scale = ref.abs().max().item()
    assert err <= 1e-2 * scale + 1e-2, (err, scale)
    assert torch.equal(c, gemm.matmul_nt(a, b))          # the same products in the same order: bit-identical to the K-major form


@pytest.mark.parametrize("a_t,b_t", [(False, False), (False, True), (True, True)])
@pytest.mark.parametrize("m,n,k", [(256, 256, 64), (512, 768, 448), (2048, 1024, 4096), (9728, 512, 1024)])
def test_cta_pair_kernel_agrees_with_the_one_cta_kernel(m, n, k, a_t, b_t, monkeypatch):
    """Sizes that tile by 256 x 256 run on CTA pairs (cta_group::2) by default; DFCCL_GEMM_PAIR=0 keeps the one-CTA
    kernel.  Both accumulate the same products in the same order, so the results are bit-identical; 9728 rows = 38 row
    tiles x 2 column tiles make more tiles than resident pairs."""
    from dfccl_b200.ops import gemm
    torch.manual_seed(m + 7 * n + k)
    a = torch.randn(m, k, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(n, k, device="cuda", dtype=torch.bfloat16)
    a_in = a.t().contiguous() if a_t else a
    b_in = b.t().contiguous() if b_t else b
    monkeypatch.setenv("DFCCL_GEMM_PAIR", "1")
    c_pair = gemm.matmul(a_in, b_in, a_transposed=a_t, b_transposed=b_t)
    torch.cuda.synchronize()
    assert gemm.check_kernels()
    monkeypatch.setenv("DFCCL_GEMM_PAIR", "0")
    c_one = gemm.matmul(a_in, b_in, a_transposed=a_t, b_transposed=b_t)
    torch.cuda.synchronize()
    ref = a.float() @ b.float().t()
    err = (c_pair.float() - ref).abs().max().item()
    scale = ref.abs().max().item()
    assert err <= 1e-2 * scale + 1e-2, (err, scale)
    assert torch.equal(c_pair, c_one)


def test_gemm_rejects_shapes_it_cannot_tile():
    from dfccl_b200.ops import gemm
    a = torch.randn(100, 64, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(256, 64, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(ValueError):
        gemm.matmul_nt(a, b)


def test_gemm_throughput_report():
    """Not an assertion on speed: prints achieved TFLOP/s next to cuBLAS for the record."""
    from dfccl_b200.ops import gemm
    m = n = k = 8192
    a = torch.randn(m, k, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(n, k, device="cuda", dtype=torch.bfloat16)
    out = torch.empty(m, n, device="cuda", dtype=torch.bfloat16)

    def bench(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(10):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / 10

    import os
    os.environ["DFCCL_GEMM_PAIR"] = "0"
    one = bench(lambda: gemm.matmul_nt(a, b, out))
    os.environ["DFCCL_GEMM_PAIR"] = "1"
    ours = bench(lambda: gemm.matmul_nt(a, b, out))
    del os.environ["DFCCL_GEMM_PAIR"]
    cublas = bench(lambda: torch.matmul(a, b.t(), out=out))
    flops = 2.0 * m * n * k
    print(f"tcgen05 gemm 8192^3: CTA pairs {ours:.3f} ms = {flops / ours / 1e9:.0f} TFLOP/s; one CTA per tile {one:.3f} ms = "
          f"{flops / one / 1e9:.0f} TFLOP/s; cuBLAS {cublas:.3f} ms = {flops / cublas / 1e9:.0f} TFLOP/s")
    assert gemm.check_kernels()
