"""CPU checks of the model code paths that choose between the package's kernels and PyTorch: on a CPU tensor every
op must fall back to PyTorch and give the reference result."""
import math

import torch


def test_causal_attention_falls_back_on_cpu():
    from torchmpi_b200.ops import attention
    torch.manual_seed(0)
    B, T, H = 2, 128, 2
    qkv = torch.randn(B, T, 3 * H * 64, requires_grad=True)
    assert not attention.supported(qkv, H)             # CPU, fp32: PyTorch's attention
    out = attention.causal_attention(qkv, H)
    C = H * 64
    q, k, v = (t.view(B, T, H, 64).transpose(1, 2) for t in qkv.detach().split(C, dim=2))
    s = (q @ k.transpose(-1, -2)) / math.sqrt(64)
    s = s.masked_fill(~torch.ones(T, T, dtype=torch.bool).tril(), float("-inf"))
    ref = (torch.softmax(s, -1) @ v).transpose(1, 2).reshape(B, T, C)
    assert torch.allclose(out, ref, atol=1e-5)
    out.sum().backward()
    assert qkv.grad is not None and torch.isfinite(qkv.grad).all()


def test_gpt2_tiny_same_logits_with_and_without_own_kernels_on_cpu():
    from torchmpi_b200.models import gpt2
    torch.manual_seed(1)
    a = gpt2.gpt2_tiny(tc_linear=False)
    b = gpt2.gpt2_tiny(tc_linear=True)                 # on CPU every op of this flavour falls back to PyTorch
    b.load_state_dict(a.state_dict())
    idx = torch.randint(0, 512, (2, 64))
    ya, yb = a(idx), b(idx)
    assert ya.shape == (128, 512)
    assert torch.allclose(ya, yb[:, :512], atol=1e-4, rtol=1e-4)


def test_backward_route_order_from_environment(monkeypatch):
    import importlib
    from torchmpi_b200.ops import attention
    monkeypatch.setenv("TORCHMPI_ATTENTION_BACKWARD", "cudnn")
    try:
        importlib.reload(attention)
        assert attention._BACKWARDS == ("cudnn", "own", "flash")
    finally:
        monkeypatch.delenv("TORCHMPI_ATTENTION_BACKWARD")
        importlib.reload(attention)
    assert attention._BACKWARDS[0] == "own"
