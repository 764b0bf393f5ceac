"""The tcgen05 bf16 GEMM against a plain PyTorch fp32 matmul of the same operands."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(a, b, bias=None, gelu=False):
    y = a.float() @ b.float().t()
    if bias is not None:
        y = y + bias.float()
    return torch.nn.functional.gelu(y) if gelu else y


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (128, 256, 512), (256, 512, 128), (1024, 1024, 1024),
                                   (100, 72, 40), (129, 257, 72), (4096, 2048, 4096), (37, 1000, 2048)])
def test_gemm_matches_fp32_reference(M, N, K):
    from torchmpi_b200.ops import gemm
    torch.manual_seed(M * 7 + N * 3 + K)
    a = torch.randn(M, K, device="cuda").to(torch.bfloat16)
    b = torch.randn(N, K, device="cuda").to(torch.bfloat16)
    y = gemm.matmul_nt(a, b)
    torch.cuda.synchronize()
    gemm.check_status()
    ref = _ref(a, b)
    err = (y.float() - ref).abs().max().item()
    assert err <= 0.02 * (K ** 0.5) + 0.05, (M, N, K, err)
    # bf16 rounding of an fp32-accumulated result: relative error of one bf16 ulp
    assert torch.allclose(y.float(), ref, rtol=1e-2, atol=0.02 * (K ** 0.5))


@pytest.mark.parametrize("M,N,K", [(256, 256, 64), (256, 512, 448), (300, 520, 136), (1024, 1024, 1024),
                                   (4096, 2048, 4096), (2304, 1280, 512)])
def test_gemm_cta_pair_and_single_cta_paths(M, N, K):
    """The 256 x 256 CTA-pair kernel (cta_group::2) and the 128 x 256 single-CTA kernel give the same
    product; both are checked against fp32, with a bias + GELU epilogue as well."""
    from torchmpi_b200 import config
    from torchmpi_b200.ops import gemm
    torch.manual_seed(M + N + K)
    a = torch.randn(M, K, device="cuda").to(torch.bfloat16)
    b = torch.randn(N, K, device="cuda").to(torch.bfloat16) * 0.2
    bias = torch.randn(N, device="cuda").to(torch.bfloat16)
    out = {}
    try:
        for pair in (1, 0):
            config.set("gemm_pair", pair)
            out[pair] = (gemm.matmul_nt(a, b), gemm.matmul_nt(a, b, bias, gelu=True))
            torch.cuda.synchronize()
            gemm.check_status()
    finally:
        config.set("gemm_pair", 1)
    ref, ref_g = _ref(a, b), _ref(a, b, bias, True)
    for pair in (1, 0):
        assert torch.allclose(out[pair][0].float(), ref, rtol=1e-2, atol=0.02 * (K ** 0.5)), pair
        assert torch.allclose(out[pair][1].float(), ref_g, rtol=2e-2, atol=0.02 * (K ** 0.5)), pair
    # same operands, same fp32 accumulation order along K: the two kernels agree bit for bit
    assert torch.equal(out[0][0], out[1][0])


@pytest.mark.parametrize("M,N,K", [(256, 256, 64), (512, 384, 200), (1024, 2048, 1024), (2048, 4096, 8192)])
def test_gemm_reads_second_operand_as_k_by_n(M, N, K):
    """``matmul_nn(a, b)`` with ``b [K, N]`` (MN-major shared-memory descriptor) equals the K-major
    kernel on a transposed copy bit for bit, and the fp32 product within rounding."""
    from torchmpi_b200.ops import gemm
    torch.manual_seed(M + 3 * N + 5 * K)
    a = torch.randn(M, K, device="cuda").to(torch.bfloat16)
    b = (torch.randn(K, N, device="cuda") * 0.2).to(torch.bfloat16)
    y = gemm.matmul_nn(a, b)
    y_t = gemm.matmul_nt(a, b.t().contiguous())
    torch.cuda.synchronize()
    gemm.check_status()
    ref = a.float() @ b.float()
    assert torch.allclose(y.float(), ref, rtol=1e-2, atol=0.02 * (K ** 0.5))
    assert torch.equal(y, y_t)


@pytest.mark.parametrize("M,N,K", [(256, 256, 64), (384, 512, 200), (1024, 2048, 1000), (4096, 1024, 8192)])
def test_gemm_transposed_first_operand(M, N, K):
    """``matmul_tn(a, b) = a.T @ b`` with ``a [K, M]`` and ``b [K, N]`` as stored (the weight-gradient layout):
    same bits as the K-major kernel on transposed copies, and the fp32 product within rounding."""
    from torchmpi_b200.ops import gemm
    torch.manual_seed(2 * M + 3 * N + K)
    a = torch.randn(K, M, device="cuda").to(torch.bfloat16)
    b = (torch.randn(K, N, device="cuda") * 0.2).to(torch.bfloat16)
    y = gemm.matmul_tn(a, b)
    y_t = gemm.matmul_nt(a.t().contiguous(), b.t().contiguous())
    torch.cuda.synchronize()
    gemm.check_status()
    ref = a.float().t() @ b.float()
    assert torch.allclose(y.float(), ref, rtol=1e-2, atol=0.02 * (K ** 0.5))
    assert torch.equal(y, y_t)


def test_gemm_epilogues_and_identity():
    from torchmpi_b200.ops import gemm
    torch.manual_seed(0)
    M, N, K = 384, 768, 256
    a = torch.randn(M, K, device="cuda").to(torch.bfloat16)
    b = torch.randn(N, K, device="cuda").to(torch.bfloat16) * 0.1
    bias = torch.randn(N, device="cuda").to(torch.bfloat16)
    for use_bias in (False, True):
        for gelu in (False, True):
            y = gemm.matmul_nt(a, b, bias if use_bias else None, gelu=gelu)
            ref = _ref(a, b, bias if use_bias else None, gelu)
            assert torch.allclose(y.float(), ref, rtol=2e-2, atol=5e-2), (use_bias, gelu)
    # identity weight: the product must reproduce the input exactly (checks tile placement and swizzle)
    eye = torch.eye(256, device="cuda").to(torch.bfloat16)
    x = torch.randn(512, 256, device="cuda").to(torch.bfloat16)
    assert torch.equal(gemm.matmul_nt(x, eye), x)
    gemm.check_status()


def test_linear_autograd_matches_torch():
    from torchmpi_b200.ops import gemm
    torch.manual_seed(1)
    x = torch.randn(4, 64, 512, device="cuda").to(torch.bfloat16).requires_grad_(True)
    lin = gemm.Linear(512, 1024, gelu=True).cuda().to(torch.bfloat16)
    y = lin(x)
    dy = torch.randn_like(y)
    y.backward(dy)
    xr = x.detach().float().requires_grad_(True)
    wr = lin.weight.detach().float().requires_grad_(True)
    br = lin.bias.detach().float().requires_grad_(True)
    yr = torch.nn.functional.gelu(torch.nn.functional.linear(xr, wr, br))
    yr.backward(dy.float())
    assert torch.allclose(y.float(), yr, rtol=2e-2, atol=5e-2)
    assert torch.allclose(x.grad.float(), xr.grad, rtol=3e-2, atol=0.5)
    assert torch.allclose(lin.weight.grad.float(), wr.grad, rtol=3e-2, atol=0.5)
    assert torch.allclose(lin.bias.grad.float(), br.grad, rtol=3e-2, atol=0.5)
    gemm.check_status()


def test_fused_gemms_single_rank():
    """With one rank the fused kernels degenerate to copy-engine + GEMM and GEMM + local slot sum:
    checks the flag hand-off between the copy CTAs and the TMA producers, and the slot epilogue."""
    import torchmpi_b200 as mpi
    from torchmpi_b200.parallel.tensor_parallel import TPGroup
    from torchmpi_b200.ops import gemm
    mpi.start(with_cuda=True)
    try:
        torch.manual_seed(3)
        rows, D, F = 512, 512, 1024
        tp = TPGroup(rows, D)
        full_buf, full_off = tp.new_full_buffer()
        x = torch.randn(rows, D, device="cuda").to(torch.bfloat16)
        w1 = (torch.randn(F, D, device="cuda") / D ** 0.5).to(torch.bfloat16)
        b1 = torch.randn(F, device="cuda").to(torch.bfloat16)
        w2 = (torch.randn(D, F, device="cuda") / F ** 0.5).to(torch.bfloat16)
        for rep in range(3):                 # flags and counters are epoch based: repeated calls must work
            z = tp.ag_gemm(x, full_off, full_buf, w1, b1)
            assert torch.equal(full_buf[:rows * D].view(rows, D), x)
            ref = x.float() @ w1.float().t() + b1.float()
            assert torch.allclose(z.float(), ref, rtol=2e-2, atol=5e-2), rep
            y = tp.gemm_rs(z, w2)
            ref2 = z.float() @ w2.float().t()
            assert torch.allclose(y.float(), ref2, rtol=2e-2, atol=5e-2), rep
        # the weight handed over as [K, N] (what backward does) gives the same bits as its transpose
        z_kn = tp.ag_gemm(x, full_off, full_buf, w1.t().contiguous(), None, w_is_kn=True)
        assert torch.equal(z_kn, tp.ag_gemm(x, full_off, full_buf, w1, None))
        y_kn = tp.gemm_rs(z, w2.t().contiguous(), w_is_kn=True)
        assert torch.equal(y_kn, tp.gemm_rs(z, w2))
        torch.cuda.synchronize()
        tp.check()
    finally:
        mpi.stop()


def test_wide_head_and_pitched_cross_entropy():
    """LM head with a vocabulary that is not a multiple of 8: logits live in a pitched buffer, the loss kernel
    takes the pitch, and forward / dX / dW all run on the CTA-pair kernel.  Against fp32 PyTorch."""
    from torchmpi_b200.ops import gemm, xent
    torch.manual_seed(11)
    for T, d, V in ((256, 256, 50257), (512, 384, 1003)):
        x = (torch.randn(T, d, device="cuda") * 0.5).to(torch.bfloat16).requires_grad_(True)
        w = (torch.randn(V, d, device="cuda") * 0.05).to(torch.bfloat16).requires_grad_(True)
        y = torch.randint(0, V, (T,), device="cuda")
        logits = gemm.wide_head(x, w)
        assert logits.shape == (T, V) and logits.stride(0) % 8 == 0
        loss = xent.cross_entropy(logits, y)
        loss.backward()
        xr, wr = x.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
        lr = torch.nn.functional.linear(xr, wr)
        ref = torch.nn.functional.cross_entropy(lr, y)
        ref.backward()
        assert torch.allclose(logits.float(), lr, rtol=2e-2, atol=2e-2), (T, d, V)
        assert abs(loss.item() - ref.item()) < 2e-2 * max(1.0, abs(ref.item())), (loss.item(), ref.item())
        for g, gr in ((x.grad, xr.grad), (w.grad, wr.grad)):
            rel = (g.float() - gr).norm() / gr.norm()
            assert rel < 3e-2, (T, d, V, rel.item())
        gemm.check_status()


def test_bias_grad_with_and_without_gelu():
    """Column sum fused with the GELU backward against PyTorch in fp32."""
    from torchmpi_b200.ops import gemm
    torch.manual_seed(13)
    for rows, C in ((8192, 1024), (777, 4096), (33, 3072)):
        dy = torch.randn(rows, C, device="cuda").to(torch.bfloat16)
        z = (torch.randn(rows, C, device="cuda") * 1.5).to(torch.bfloat16)
        dz, db = gemm.bias_grad(dy, z)
        ref = torch.ops.aten.gelu_backward(dy.float(), z.float())
        assert torch.allclose(dz.float(), ref, rtol=2e-2, atol=2e-2)
        assert torch.allclose(db.float(), dz.float().sum(0), rtol=1e-2, atol=0.05 * rows ** 0.5)
        same, db2 = gemm.bias_grad(dy)
        assert same is dy
        assert torch.allclose(db2.float(), dy.float().sum(0), rtol=1e-2, atol=0.05 * rows ** 0.5)


def test_gelu_forward_kernel():
    """The erf-form GELU through the rational approximation against PyTorch in fp32."""
    from torchmpi_b200.ops import gemm
    torch.manual_seed(17)
    for shape, dt in (((8192, 4096), torch.bfloat16), ((333, 1000), torch.float32), ((64, 40), torch.float16)):
        z = (torch.randn(*shape, device="cuda") * 2.5).to(dt)
        y = gemm.gelu(z)
        ref = torch.nn.functional.gelu(z.float())
        tol = 1e-5 if dt == torch.float32 else 2e-2
        assert torch.allclose(y.float(), ref, rtol=tol, atol=tol), (shape, dt)
    edge = torch.tensor([-30.0, -8.0, -0.0, 0.0, 8.0, 30.0, float("inf")], device="cuda").repeat(4)[:24].contiguous()
    assert torch.allclose(gemm.gelu(edge), torch.nn.functional.gelu(edge), atol=1e-5)
