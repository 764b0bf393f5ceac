"""The tcgen05 causal attention forward against fp32 softmax(Q K^T / sqrt(d)) V, its log-sum-exp, and the gradient
of the autograd op against PyTorch's own attention in fp32."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(qkv, H):
    B, T, C3 = qkv.shape
    C = C3 // 3
    q, k, v = (t.view(B, T, H, 64).transpose(1, 2).float() for t in qkv.split(C, dim=2))
    s = q @ k.transpose(-1, -2) / math.sqrt(64)
    mask = torch.ones(T, T, dtype=torch.bool, device=qkv.device).tril()
    s = s.masked_fill(~mask, float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    out = torch.softmax(s, dim=-1) @ v
    return out.transpose(1, 2).reshape(B, T, C), lse


@pytest.mark.parametrize("B,T,H", [(1, 128, 1), (2, 256, 3), (2, 1024, 4), (1, 512, 16), (1, 2048, 2)])
def test_attention_forward_matches_fp32(B, T, H):
    from torchmpi_b200.ops import attention
    from torchmpi_b200._lib import lib
    torch.manual_seed(B * 1000 + T + H)
    qkv = (torch.randn(B, T, 3 * H * 64, device="cuda") * 1.5).to(torch.bfloat16)
    assert attention.supported(qkv, H)
    out, lse = attention.attention_forward(qkv, H)
    torch.cuda.synchronize()
    attention.check_status()
    ref, ref_lse = _ref(qkv, H)
    assert torch.allclose(lse, ref_lse, atol=2e-3, rtol=1e-4), (lse - ref_lse).abs().max().item()
    err = (out.float() - ref).abs().max().item()
    assert err < 2e-2, err                         # bf16 probabilities and bf16 output of values of order 1
    rel = ((out.float() - ref).norm() / ref.norm()).item()
    assert rel < 6e-3, rel
    # same input, same bits
    out2, _ = attention.attention_forward(qkv, H)
    assert torch.equal(out, out2)
    assert lib.tmpi_attention_ctas_per_sm() >= 1


def test_attention_autograd_and_fallback():
    from torchmpi_b200.ops import attention
    torch.manual_seed(5)
    B, T, H = 2, 256, 4
    qkv = torch.randn(B, T, 3 * H * 64, device="cuda").to(torch.bfloat16).requires_grad_(True)
    before = attention.launch_count
    out = attention.causal_attention(qkv, H)
    assert attention.launch_count == before + 1
    g = torch.randn_like(out)
    out.backward(g)
    assert attention.last_backward == "own"
    attention.check_status()
    leaf = qkv.detach().float().requires_grad_(True)
    ref, _ = _ref(leaf, H)
    ref.backward(g.float())
    rel = ((qkv.grad.float() - leaf.grad).norm() / leaf.grad.norm()).item()
    assert rel < 2e-2, (rel, attention.last_backward)
    # every backward route gives the same gradient
    first = attention.last_backward
    for route in ("cudnn", "flash", "none"):
        attention._BACKWARDS = (route,)
        try:
            q2 = qkv.detach().clone().requires_grad_(True)
            attention.causal_attention(q2, H).backward(g)
            assert attention.last_backward == ("recompute" if route == "none" else route) or attention.last_backward == "recompute"
            rel = ((q2.grad.float() - leaf.grad).norm() / leaf.grad.norm()).item()
            assert rel < 2e-2, (rel, route)
        finally:
            attention._BACKWARDS = ("own", "cudnn", "flash")
    assert first == "own"
    # shapes the kernel does not take go to PyTorch's attention
    odd = torch.randn(1, 100, 3 * 2 * 64, device="cuda").to(torch.bfloat16)
    assert not attention.supported(odd, 2)
    o = attention.causal_attention(odd, 2)
    r, _ = _ref(odd, 2)
    assert ((o.float() - r).norm() / r.norm()).item() < 1e-2


def test_gpt2_block_uses_own_attention():
    from torchmpi_b200.models import gpt2
    from torchmpi_b200.ops import attention
    torch.manual_seed(0)
    m = gpt2.gpt2_tiny(n_head=2, n_embd=128, block_size=256, tc_linear=True).cuda().to(torch.bfloat16)
    ref = gpt2.gpt2_tiny(n_head=2, n_embd=128, block_size=256, tc_linear=False).cuda().to(torch.bfloat16)
    ref.load_state_dict(m.state_dict())
    idx = torch.randint(0, 512, (2, 256), device="cuda")
    before = attention.launch_count
    y = m(idx)
    assert attention.launch_count == before + len(m.blocks)
    yr = ref(idx)
    rel = ((y.float() - yr.float()).norm() / yr.float().norm()).item()
    assert rel < 3e-2, rel


def test_attention_phase_trace_is_ordered():
    """The tuning aid: CTA 0 stamps the phases of every key block in order, and switching it off stops the writes."""
    from torchmpi_b200.ops import attention
    from torchmpi_b200._lib import lib
    T, H = 512, 2
    qkv = torch.randn(1, T, 3 * H * 64, device="cuda").to(torch.bfloat16)
    buf = torch.zeros((T // 128) * 16, dtype=torch.int64, device="cuda")
    lib.tmpi_attention_set_trace(buf.data_ptr())
    try:
        attention.attention_forward(qkv, H)
        torch.cuda.synchronize()
    finally:
        lib.tmpi_attention_set_trace(None)
    t = buf.cpu().view(T // 128, 16)
    for j in range(T // 128):                      # CTA 0 handles the last query block: T / 128 key blocks
        has_s, max_known, p_written, has_o, updated = (int(t[j, e]) for e in (1, 2, 3, 5, 6))
        assert 0 < has_s <= max_known <= p_written <= has_o <= updated, (j, t[j].tolist())
    buf.zero_()
    attention.attention_forward(qkv, H)
    torch.cuda.synchronize()
    assert int(buf.abs().sum()) == 0


@pytest.mark.parametrize("B,T,H", [(1, 128, 1), (2, 384, 2), (1, 1024, 3), (1, 2048, 2)])
def test_attention_backward_matches_fp32(B, T, H):
    """dQ, dK, dV of the tcgen05 backward kernel against fp32 autograd of softmax(Q K^T / sqrt(d)) V."""
    from torchmpi_b200.ops import attention
    torch.manual_seed(B + T + H)
    qkv = torch.randn(B, T, 3 * H * 64, device="cuda").to(torch.bfloat16)
    out, lse = attention.attention_forward(qkv, H)
    dout = torch.randn_like(out)
    dqkv = attention.attention_backward(qkv, out, lse, dout, H)
    torch.cuda.synchronize()
    attention.check_status()
    leaf = qkv.detach().float().requires_grad_(True)
    ref, _ = _ref(leaf, H)
    ref.backward(dout.float())
    C = H * 64
    for name, sl in (("dq", slice(0, C)), ("dk", slice(C, 2 * C)), ("dv", slice(2 * C, 3 * C))):
        got, want = dqkv[:, :, sl].float(), leaf.grad[:, :, sl]
        rel = ((got - want).norm() / want.norm()).item()
        assert rel < 1.5e-2, (name, rel)
    # dK and dV are bit-reproducible; dQ is summed in arrival order
    dqkv2 = attention.attention_backward(qkv, out, lse, dout, H)
    assert torch.equal(dqkv[:, :, C:], dqkv2[:, :, C:])
    assert torch.allclose(dqkv[:, :, :C].float(), dqkv2[:, :, :C].float(), atol=1e-2, rtol=1e-2)
