"""The implicit-GEMM convolution kernels (csrc/kernels/conv_gemm.cu) against fp32 ``F.conv2d`` and its autograd
gradients: forward, input gradient, weight gradient, the batch statistics of the epilogue and the fused add."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu

# (N, H, W, Cin, Cout, k, stride, pad)
GEOMS = [
    (2, 8, 8, 64, 64, 1, 1, 0),          # one M tile exactly
    (3, 7, 7, 64, 256, 1, 1, 0),         # M = 147: ragged last tile
    (2, 14, 14, 256, 64, 1, 1, 0),       # four K blocks
    (2, 9, 9, 128, 512, 1, 1, 0),        # two N tiles
    (2, 14, 14, 64, 64, 3, 1, 1),        # 3x3, nine taps
    (3, 9, 10, 128, 128, 3, 1, 1),       # 3x3, rectangular image, ragged M
    (2, 14, 14, 64, 128, 3, 2, 1),       # 3x3 stride 2
    (2, 14, 14, 128, 256, 1, 2, 0),      # 1x1 stride 2 (downsample)
    (4, 28, 28, 64, 64, 3, 1, 1),        # more pixels than one K slice of the weight gradient
]


def _mk(N, H, W, Cin, Cout, k, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(N, Cin, H, W, device="cuda", generator=g).to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
    w = (torch.randn(Cout, Cin, k, k, device="cuda", generator=g) * (Cin * k * k) ** -0.5).to(torch.bfloat16)
    w = w.contiguous(memory_format=torch.channels_last)
    return x, w


def _close(got, want, what, rel=2e-2):
    err = (got.float() - want.float()).abs().max().item()
    scale = want.float().abs().max().item() + 1e-6
    assert err <= rel * scale, f"{what}: max error {err:.4g} against a scale of {scale:.4g}"


@pytest.mark.parametrize("geom", GEOMS)
def test_conv_forward_backward_match_fp32(geom):
    from torchmpi_b200.ops import conv
    N, H, W, Cin, Cout, k, stride, pad = geom
    x, w = _mk(N, H, W, Cin, Cout, k)
    assert conv.supported(x, w, stride, pad)
    xr, wr = x.float().requires_grad_(True), w.float().requires_grad_(True)
    yr = F.conv2d(xr, wr, None, stride, pad)
    y, _ = conv.conv_forward(x, w, stride, pad)
    torch.cuda.synchronize()
    conv.check_status()
    assert y.is_contiguous(memory_format=torch.channels_last) and y.shape == yr.shape
    _close(y, yr, "forward")
    dy = torch.randn_like(y)
    yr.backward(dy.float())
    dw = conv.conv_wgrad(dy, x, w.shape, stride, pad)
    torch.cuda.synchronize()
    conv.check_status()
    _close(dw, wr.grad, "weight gradient")
    assert dw.is_contiguous(memory_format=torch.channels_last)
    if stride == 1:
        dx = conv.conv_dgrad(dy, w, x.shape, 1, pad)
        torch.cuda.synchronize()
        conv.check_status()
        _close(dx, xr.grad, "input gradient")
        other = torch.randn_like(x)
        dx2 = conv.conv_dgrad(dy, w, x.shape, 1, pad, add=other)
        torch.cuda.synchronize()
        _close(dx2, xr.grad + other.float(), "input gradient + added tensor")
    # accumulate into an existing gradient, twice in a row (the tile counters must be back at zero)
    acc = wr.grad.to(torch.bfloat16).contiguous(memory_format=torch.channels_last).clone()
    conv.conv_wgrad(dy, x, w.shape, stride, pad, out=acc, accumulate=True)
    torch.cuda.synchronize()
    _close(acc, 2 * wr.grad, "accumulated weight gradient")


@pytest.mark.parametrize("geom", [GEOMS[1], GEOMS[3], GEOMS[5], GEOMS[6]])
def test_conv_epilogue_statistics(geom):
    """Per-CTA partial sums of the stored (rounded) outputs: their totals are the column sums of y and y^2."""
    from torchmpi_b200.ops import conv
    from torchmpi_b200._lib import lib
    N, H, W, Cin, Cout, k, stride, pad = geom
    x, w = _mk(N, H, W, Cin, Cout, k, seed=3)
    stats = torch.full((lib.tmpi_conv_max_ctas() * 2 * Cout,), float("nan"), dtype=torch.float32, device="cuda")
    y, rows = conv.conv_forward(x, w, stride, pad, stats)
    torch.cuda.synchronize()
    assert 1 <= rows <= lib.tmpi_conv_max_ctas()
    part = stats[:rows * 2 * Cout].view(rows, 2, Cout).double().sum(0)
    y2 = y.permute(0, 2, 3, 1).reshape(-1, Cout).double()
    assert torch.allclose(part[0], y2.sum(0), rtol=1e-4, atol=1e-2)
    assert torch.allclose(part[1], (y2 * y2).sum(0), rtol=1e-4, atol=1e-2)


def test_conv_autograd_op_and_module():
    from torchmpi_b200.ops import conv
    torch.manual_seed(1)
    m = conv.Conv2d(64, 128, 3, stride=1, padding=1).cuda().to(torch.bfloat16).to(memory_format=torch.channels_last)
    x = torch.randn(2, 64, 12, 12, device="cuda", dtype=torch.bfloat16).contiguous(memory_format=torch.channels_last).requires_grad_(True)
    y = m(x)
    g = torch.randn_like(y)
    y.backward(g)
    xr = x.detach().float().requires_grad_(True)
    wr = m.weight.detach().float().requires_grad_(True)
    F.conv2d(xr, wr, None, 1, 1).backward(g.float())
    _close(x.grad, xr.grad, "autograd dx")
    _close(m.weight.grad, wr.grad, "autograd dw")
    # unsupported channel counts take the library path and still give the right answer
    m2 = conv.Conv2d(16, 32, 3, padding=1).cuda().to(torch.bfloat16)
    x2 = torch.randn(2, 16, 8, 8, device="cuda", dtype=torch.bfloat16)
    _close(m2(x2), F.conv2d(x2.float(), m2.weight.float(), None, 1, 1), "fallback")


def test_matmul_tn_splitk_long_k_small_output():
    """dW-shaped product: K = many rows, output 64 x 160 (the stem's weight gradient)."""
    from torchmpi_b200.ops import conv
    torch.manual_seed(5)
    K = 50000
    a = torch.randn(K, 64, device="cuda").to(torch.bfloat16)
    b = torch.randn(K, 160, device="cuda").to(torch.bfloat16)
    got = conv.matmul_tn_splitk(a, b)
    want = a.float().t() @ b.float()
    _close(got, want, "split-K product", rel=1e-2)
    acc = want.to(torch.bfloat16).clone()
    conv.matmul_tn_splitk(a, b, out=acc, accumulate=True)
    _close(acc, 2 * want, "accumulated split-K product", rel=1e-2)
    conv.check_status()


def test_conv_bn_fused_statistics_match_separate_pass():
    """conv -> batch-norm with the statistics from the convolution's epilogue equals conv -> batch-norm with its own pass."""
    from torchmpi_b200.ops import conv
    from torchmpi_b200.ops.bn_relu import FusedBatchNormReLU
    torch.manual_seed(2)
    c = conv.Conv2d(64, 256, 1).cuda().to(torch.bfloat16).to(memory_format=torch.channels_last)
    bn_a = FusedBatchNormReLU(256).cuda()
    bn_b = FusedBatchNormReLU(256).cuda()
    with torch.no_grad():
        bn_a.weight.uniform_(0.5, 1.5); bn_a.bias.uniform_(-0.2, 0.2)
        bn_b.load_state_dict(bn_a.state_dict())
    x = torch.randn(4, 64, 14, 14, device="cuda", dtype=torch.bfloat16).contiguous(memory_format=torch.channels_last)
    xa = x.clone().requires_grad_(True)
    xb = x.clone().requires_grad_(True)
    ya = conv.conv_bn(c, bn_a, xa)
    yb = bn_b(c(xb))
    assert torch.allclose(ya.float(), yb.float(), atol=2e-2, rtol=2e-2)
    assert torch.allclose(bn_a.running_mean, bn_b.running_mean, atol=1e-4, rtol=1e-3)
    assert torch.allclose(bn_a.running_var, bn_b.running_var, atol=1e-4, rtol=1e-3)
    g = torch.randn_like(ya)
    ya.backward(g)
    wa = c.weight.grad.clone(); c.weight.grad = None
    yb.backward(g)
    assert torch.allclose(xa.grad.float(), xb.grad.float(), atol=2e-2, rtol=2e-2)
    assert torch.allclose(wa.float(), c.weight.grad.float(), atol=2e-2, rtol=2e-2)


def test_bottleneck_with_fork_and_direct_gradients_matches_eager():
    """A fused bottleneck block (convolutions on the implicit-GEMM kernel, statistics in the epilogue, the two
    gradients into the block input summed inside a kernel, parameter gradients added in place into flat buckets)
    against the same block run with eager PyTorch layers in fp32."""
    from torchmpi_b200.models.resnet import Bottleneck, _bn
    from torchmpi_b200.parallel.flat_buckets import FlatBuckets
    import torch.nn as nn
    torch.manual_seed(3)
    for inplanes, planes, stride in ((256, 64, 1), (64, 64, 1), (256, 128, 2)):
        down_f = down_e = None
        if stride != 1 or inplanes != planes * 4:
            down_f = nn.Sequential(nn.Conv2d(inplanes, planes * 4, 1, stride=stride, bias=False), _bn(planes * 4, True, relu=False))
            down_e = nn.Sequential(nn.Conv2d(inplanes, planes * 4, 1, stride=stride, bias=False), _bn(planes * 4, False, relu=False))
        fused = Bottleneck(inplanes, planes, stride, down_f, fused_bn=True).cuda()
        eager = Bottleneck(inplanes, planes, stride, down_e, fused_bn=False).cuda()
        with torch.no_grad():
            for m in fused.modules():
                if isinstance(m, nn.BatchNorm2d):
                    m.weight.uniform_(0.5, 1.5); m.bias.uniform_(-0.3, 0.3)
        eager.load_state_dict(fused.state_dict())
        for m in fused.modules():                       # bf16 convolutions, fp32 batch-norm: the mixed layout of the benchmark
            if isinstance(m, nn.Conv2d):
                m.to(torch.bfloat16)
        fused = fused.to(memory_format=torch.channels_last)
        for p, q in zip(fused.parameters(), eager.parameters()):       # the eager copy sees the rounded weights
            q.data.copy_(p.data.float())
        fb = FlatBuckets(list(fused.parameters()), bucket_bytes=1 << 30)
        ready = []
        fb.register_ready_hooks(lambda g: ready.append(g.data_ptr()))
        x = torch.randn(4, inplanes, 14, 14, device="cuda").to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
        xf = x.clone().requires_grad_(True)
        xe = x.float().requires_grad_(True)
        yf = fused(xf * 1.0)              # a non-leaf input, as inside a network
        ye = eager(xe * 1.0)
        g = torch.randn_like(ye)
        yf.backward(g.to(torch.bfloat16))
        ye.backward(g)
        torch.cuda.synchronize()
        # bf16 activations against fp32: a ReLU mask that flips near zero moves single elements a lot, so the
        # yardstick is the relative error in the 2-norm, not the largest element
        def rel2(a, b):
            return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()
        tag = f"{inplanes}/{planes}/{stride}"
        assert rel2(yf, ye) < 2e-2, (tag, "output", rel2(yf, ye))
        assert rel2(xf.grad, xe.grad) < 0.12, (tag, "input gradient", rel2(xf.grad, xe.grad))
        assert len(ready) == len(fb.buckets), "every bucket reports its gradients exactly once"
        for (n, p), q in zip(fused.named_parameters(), eager.parameters()):
            assert rel2(p.grad, q.grad) < 0.15, (tag, n, rel2(p.grad, q.grad))
        # the same block without the in-kernel gradient sum and without in-place parameter gradients: same numbers
        fb.remove_hooks()
        from torchmpi_b200 import config
        config.set("grad_fork", 0)
        ref = {n: p.grad.clone() for n, p in fused.named_parameters()}
        fb.zero_grad()
        xg = x.clone().requires_grad_(True)
        fused(xg * 1.0).backward(g.to(torch.bfloat16))
        config.set("grad_fork", 1)
        assert rel2(xg.grad, xf.grad) < 1e-2, (tag, "fork on/off", rel2(xg.grad, xf.grad))
        for n, p in fused.named_parameters():
            assert rel2(p.grad, ref[n]) < 1e-2, (tag, n, "direct/returned gradient", rel2(p.grad, ref[n]))
