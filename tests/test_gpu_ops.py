"""Single-GPU hot ops against plain PyTorch fp32 references of the same op."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_native_library_is_loaded():
    from torchmpi_b200 import _lib
    assert _lib.lib.tmpi_has_cuda() == 1
    for sym in ("tmpi_sgd_momentum", "tmpi_xent_fwd_bwd", "tmpi_bn_relu_fwd", "tmpi_cuda_allreduce_sgd"):
        assert _lib.has_symbol(sym)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("nesterov", [False, True])
def test_sgd_momentum_matches_torch(dtype, nesterov):
    from torchmpi_b200.ops import elementwise
    torch.manual_seed(0)
    n = 8 * 12345
    w0 = torch.randn(n, device="cuda")
    w = w0.to(dtype).clone()
    master = w.float().clone() if dtype != torch.float32 else None
    mom = torch.zeros(n, device="cuda")
    ref = torch.nn.Parameter(w.float().clone())
    opt = torch.optim.SGD([ref], lr=0.05, momentum=0.9, weight_decay=1e-4, nesterov=nesterov)
    for step in range(4):
        g = torch.randn(n, device="cuda").to(dtype)
        ref.grad = g.float() * 0.5
        opt.step()
        gbuf = g.clone()
        elementwise.sgd_momentum_(w, gbuf, lr=0.05, momentum=0.9, weight_decay=1e-4, nesterov=nesterov,
                                  grad_scale=0.5, master=master, momentum_buf=mom, first_step=(step == 0),
                                  zero_grad=True)
        got = master if master is not None else w
        assert torch.allclose(got, ref.detach(), atol=2e-6, rtol=1e-5)
        assert torch.count_nonzero(gbuf) == 0
        if master is not None:
            assert torch.equal(w, master.to(dtype))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_xent_forward_and_gradient(dtype):
    from torchmpi_b200.ops import xent
    torch.manual_seed(1)
    for rows, cols in ((256, 1000), (7, 10), (33, 50257)):
        logits = (torch.randn(rows, cols, device="cuda") * 3).to(dtype).requires_grad_(True)
        labels = torch.randint(0, cols, (rows,), device="cuda")
        loss = xent.cross_entropy(logits, labels)
        loss.backward()
        ref_in = logits.detach().float().requires_grad_(True)
        ref = torch.nn.functional.cross_entropy(ref_in, labels)
        ref.backward()
        assert torch.allclose(loss.float(), ref, atol=1e-4, rtol=1e-5), (rows, cols, loss.item(), ref.item())
        tol = 1e-6 if dtype == torch.float32 else 2e-3 / rows + 1e-5
        assert torch.allclose(logits.grad.float(), ref_in.grad, atol=tol, rtol=2e-2)
        # same input, same bits
        loss2 = xent.cross_entropy(logits.detach(), labels)
        assert torch.equal(loss.detach(), loss2)


def test_absmean_var_and_check():
    from torchmpi_b200.ops import stats
    torch.manual_seed(2)
    for dtype in (torch.float32, torch.bfloat16, torch.float64):
        for n in (1, 1000, 3_000_001):
            x = torch.randn(n, device="cuda").to(dtype)
            m, v = stats.absmean_var(x)
            a = x.double().abs()
            # fp64 accumulation of fp32 partial sums over at most 32 elements (fp64 inputs: fp64 throughout)
            tol_m, tol_v = (1e-9, 1e-7) if dtype == torch.float64 else (5e-7, 2e-6)
            assert abs(m - a.mean().item()) <= tol_m * max(1.0, abs(m))
            if n > 1:
                assert abs(v - a.var().item()) <= tol_v * max(1.0, v)
            assert stats.absmean_var(x) == (m, v)      # deterministic


def test_easgd_and_downpour_kernels():
    from torchmpi_b200.ops import elementwise
    torch.manual_seed(3)
    for dtype, n in ((torch.float32, 100003), (torch.bfloat16, 8 * 4096), (torch.float32, 4096)):
        x = torch.randn(n, device="cuda").to(dtype)
        c = torch.randn(n, device="cuda").to(dtype)
        d = torch.empty_like(x)
        x0 = x.float().clone()
        elementwise.easgd_elastic(x, c, d, 0.3)
        diff = c.float() - x0
        tol = 1e-6 if dtype == torch.float32 else 2e-2
        assert torch.allclose(x.float(), x0 + 0.3 * diff, atol=tol, rtol=tol)
        assert torch.allclose(d.float(), -0.3 * diff, atol=tol, rtol=tol)
        acc = torch.randn(n, device="cuda").to(dtype)
        g = torch.randn(n, device="cuda").to(dtype)
        a0 = acc.float().clone()
        elementwise.downpour_accum(acc, g, scale=2.0)
        assert torch.allclose(acc.float(), a0 + 2.0 * g.float(), atol=tol, rtol=tol)
        elementwise.downpour_accum(acc, g, zero_first=True)
        assert torch.allclose(acc.float(), g.float(), atol=tol, rtol=tol)


@pytest.mark.parametrize("C,hw,relu,res", [(64, 56, True, False), (256, 14, True, True), (2048, 7, False, False),
                                           (16, 9, True, True)])
def test_fused_bn_relu_matches_torch(C, hw, relu, res):
    from torchmpi_b200.ops.bn_relu import FusedBatchNormReLU, supported
    torch.manual_seed(4)
    N = 16
    x = (torch.randn(N, C, hw, hw, device="cuda") * 2 + 0.5).to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
    r = torch.randn(N, C, hw, hw, device="cuda").to(torch.bfloat16).contiguous(memory_format=torch.channels_last) if res else None
    assert supported(x)
    m = FusedBatchNormReLU(C, relu=relu).cuda()
    with torch.no_grad():
        m.weight.uniform_(0.5, 1.5)
        m.bias.uniform_(-0.5, 0.5)
    ref = torch.nn.BatchNorm2d(C).cuda()
    ref.load_state_dict({k: v for k, v in m.state_dict().items()})
    xa = x.clone().requires_grad_(True)
    ra = r.clone().requires_grad_(True) if res else None
    y = m(xa, ra)
    xb = x.float().clone().requires_grad_(True)
    rb = r.float().clone().requires_grad_(True) if res else None
    z = ref(xb) + (rb if res else 0)
    yr = torch.relu(z) if relu else z
    assert torch.allclose(y.float(), yr, atol=3e-2, rtol=2e-2)
    assert torch.allclose(m.running_mean, ref.running_mean, atol=1e-3, rtol=1e-3)
    assert torch.allclose(m.running_var, ref.running_var, atol=1e-3, rtol=1e-3)
    dy = torch.randn_like(y)
    # use the same ReLU mask in both: derive the reference gradient from the fused output's mask
    y.backward(dy)
    mask = (y > 0).float() if relu else torch.ones_like(yr)
    z.backward(dy.float() * mask)
    scale = xb.grad.abs().max().item()
    assert torch.allclose(xa.grad.float(), xb.grad, atol=3e-2 * scale + 1e-3, rtol=5e-2)
    assert torch.allclose(m.weight.grad, ref.weight.grad, atol=2e-2 * ref.weight.grad.abs().max().item(), rtol=2e-2)
    assert torch.allclose(m.bias.grad, ref.bias.grad, atol=2e-2 * ref.bias.grad.abs().max().item(), rtol=2e-2)
    if res:
        assert torch.allclose(ra.grad.float(), (dy.float() * mask), atol=1e-2, rtol=1e-2)
    # eval mode uses the running statistics
    m.eval(), ref.eval()
    ye = m(x, r)
    ze = ref(x.float()) + (r.float() if res else 0)
    assert torch.allclose(ye.float(), torch.relu(ze) if relu else ze, atol=3e-2, rtol=2e-2)


@pytest.mark.parametrize("shape,k,s,p", [((8, 64, 112, 112), 3, 2, 1), ((3, 16, 17, 23), 3, 2, 1), ((2, 8, 9, 9), 2, 2, 0)])
def test_maxpool_nhwc_matches_torch(shape, k, s, p):
    from torchmpi_b200.ops.pool import MaxPool2d, supported
    torch.manual_seed(5)
    x = torch.relu(torch.randn(*shape, device="cuda")).to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
    assert supported(x)
    xa = x.clone().requires_grad_(True)
    y = MaxPool2d(k, s, p)(xa)
    xb = x.clone().requires_grad_(True)
    yr = torch.nn.functional.max_pool2d(xb, k, s, p)
    assert torch.equal(y, yr)
    dy = torch.randn_like(y)
    y.backward(dy)
    yr.backward(dy)
    # many ties (zeros after ReLU): the first maximum of a window must receive the gradient
    assert torch.allclose(xa.grad.float(), xb.grad.float(), atol=2e-2, rtol=2e-2)


def test_stem_conv_matches_conv2d():
    """im2col + tcgen05 GEMM stem against an fp32 conv2d of the same bf16 operands, forward and dW."""
    from torchmpi_b200.ops import stem_conv, gemm
    torch.manual_seed(5)
    for N, H, W in ((4, 224, 224), (3, 64, 96), (2, 40, 56)):
        conv = stem_conv.StemConv7x7(64).cuda().to(torch.bfloat16).to(memory_format=torch.channels_last)
        x = torch.randn(N, 3, H, W, device="cuda").to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
        assert stem_conv.supported(x, conv.weight)
        y = conv(x)
        assert y.is_contiguous(memory_format=torch.channels_last)
        dy = torch.randn_like(y)
        y.backward(dy)
        wr = conv.weight.detach().float().requires_grad_(True)
        yr = torch.nn.functional.conv2d(x.float(), wr, None, 2, 3)
        yr.backward(dy.float())
        assert y.shape == yr.shape
        assert torch.allclose(y.float(), yr, rtol=2e-2, atol=5e-2), (N, H, W, (y.float() - yr).abs().max().item())
        rel = (conv.weight.grad.float() - wr.grad).norm() / wr.grad.norm()
        assert rel < 1e-2, (N, H, W, rel.item())
        gemm.check_status()


@pytest.mark.parametrize("fused_bwd", [0, 1])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_bn_relu_maxpool_stage_matches_separate_ops(dtype, fused_bwd):
    """Batch-norm + ReLU + max-pool in one stage against the three PyTorch ops in fp32 on the same input."""
    from torchmpi_b200 import config
    from torchmpi_b200.ops.bn_relu import FusedBatchNormReLUMaxPool
    config.set("bn_pool_fused_bwd", fused_bwd)
    torch.manual_seed(7)
    for N, C, H, W in ((4, 64, 112, 112), (2, 16, 33, 47), (3, 32, 16, 16)):
        x = torch.randn(N, C, H, W, device="cuda").to(dtype).contiguous(memory_format=torch.channels_last).requires_grad_(True)
        m = FusedBatchNormReLUMaxPool(C).cuda()
        with torch.no_grad():
            m.weight.copy_(torch.randn(C).abs() + 0.5)
            m.weight[::3] *= -1                      # negative scales reverse the order inside a window
            m.bias.copy_(torch.randn(C) * 0.3)
        y = m(x)
        dy = torch.randn_like(y)
        y.backward(dy)
        xr = x.detach().float().requires_grad_(True)
        ref_bn = torch.nn.BatchNorm2d(C).cuda()
        with torch.no_grad():
            ref_bn.weight.copy_(m.weight)
            ref_bn.bias.copy_(m.bias)
        z = torch.relu(ref_bn(xr))
        if dtype == torch.bfloat16:
            z = z + (z.to(dtype).float() - z).detach()      # the stage pools the bf16-rounded activation
        yr = torch.nn.functional.max_pool2d(z, 3, 2, 1)
        yr.backward(dy.float())
        tol = 2e-2 if dtype == torch.bfloat16 else 1e-4
        assert y.shape == yr.shape
        assert torch.allclose(y.float(), yr, rtol=tol, atol=tol), (N, C, H, W)
        assert torch.allclose(m.running_mean, ref_bn.running_mean, atol=1e-4)
        assert torch.allclose(m.running_var, ref_bn.running_var, atol=1e-3, rtol=1e-3)
        rel = (x.grad.float() - xr.grad).norm() / xr.grad.norm()
        assert rel < (2e-2 if dtype == torch.bfloat16 else 1e-4), (N, C, H, W, rel.item())
        assert torch.allclose(m.weight.grad, ref_bn.weight.grad, rtol=2e-2, atol=2e-2 * ref_bn.weight.grad.abs().max().item())
        assert torch.allclose(m.bias.grad, ref_bn.bias.grad, rtol=2e-2, atol=2e-2 * ref_bn.bias.grad.abs().max().item())


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_layernorm_matches_torch(dtype):
    """One-pass layer norm (forward, dx, dgamma, dbeta) against fp32 PyTorch on the same operands."""
    from torchmpi_b200.ops.layernorm import LayerNorm, supported
    torch.manual_seed(9)
    for rows, C in ((8192, 1024), (777, 256), (33, 2048 if dtype == torch.bfloat16 else 1024), (4096, 768)):
        ln = LayerNorm(C).cuda().to(dtype)
        with torch.no_grad():
            ln.weight.copy_(torch.randn(C) * 0.5 + 1.0)
            ln.bias.copy_(torch.randn(C) * 0.2)
        x = (torch.randn(rows, C, device="cuda") * 2 + 0.5).to(dtype).requires_grad_(True)
        assert supported(x, ln.weight, ln.bias), (rows, C)
        y = ln(x)
        dy = torch.randn_like(y)
        y.backward(dy)
        xr = x.detach().float().requires_grad_(True)
        wr, br = ln.weight.detach().float().requires_grad_(True), ln.bias.detach().float().requires_grad_(True)
        yr = torch.nn.functional.layer_norm(xr, (C,), wr, br, ln.eps)
        yr.backward(dy.float())
        tol = 3e-2 if dtype == torch.bfloat16 else 1e-4
        assert torch.allclose(y.float(), yr, rtol=tol, atol=tol), (rows, C)
        for g, gr in ((x.grad, xr.grad), (ln.weight.grad, wr.grad), (ln.bias.grad, br.grad)):
            rel = (g.float() - gr).norm() / gr.norm()
            assert rel < (2e-2 if dtype == torch.bfloat16 else 1e-5), (rows, C, rel.item())
