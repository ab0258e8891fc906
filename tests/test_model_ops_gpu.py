"""Model-side kernels against plain PyTorch fp32 references."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rms", [False, True])
@pytest.mark.parametrize("shape", [(4, 37, 768), (3, 5, 2048), (2, 8, 136)])
def test_norm_forward_backward(dtype, rms, shape):
    from dynamiq_sigcomm_artifact_b200.ops.layers import LayerNorm, RMSNorm

    torch.manual_seed(0)
    H = shape[-1]
    mod = (RMSNorm(H) if rms else LayerNorm(H)).cuda()
    with torch.no_grad():
        mod.weight.normal_(1.0, 0.2)
        if not rms:
            mod.bias.normal_(0.0, 0.2)
    x = torch.randn(shape, device="cuda").to(dtype).requires_grad_(True)
    dy = torch.randn(shape, device="cuda").to(dtype)
    y = mod(x)
    y.backward(dy)
    xf = x.detach().float().requires_grad_(True)
    if rms:
        ref = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + mod.eps) * mod.weight.detach()
    else:
        ref = F.layer_norm(xf, (H,), mod.weight.detach(), mod.bias.detach(), mod.eps)
    w_ref = mod.weight.detach().clone().requires_grad_(True)
    ref.backward(dy.float())
    tol = 2e-2 if dtype == torch.bfloat16 else 2e-5
    assert torch.allclose(y.float(), ref, atol=tol, rtol=tol)
    assert torch.allclose(x.grad.float(), xf.grad, atol=tol * 4, rtol=tol * 4)
    # weight gradient against an fp32 autograd reference
    xf2 = x.detach().float()
    w2 = mod.weight.detach().clone().requires_grad_(True)
    if rms:
        (xf2 * torch.rsqrt(xf2.pow(2).mean(-1, keepdim=True) + mod.eps) * w2).backward(dy.float())
    else:
        b2 = mod.bias.detach().clone().requires_grad_(True)
        F.layer_norm(xf2, (H,), w2, b2, mod.eps).backward(dy.float())
        assert torch.allclose(mod.bias.grad, b2.grad, atol=1e-3, rtol=1e-3)
    assert torch.allclose(mod.weight.grad, w2.grad, atol=2e-3, rtol=2e-3)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rope_forward_backward(dtype):
    from dynamiq_sigcomm_artifact_b200.ops.layers import apply_rope, rope_tables

    B, S, nH, D = 2, 33, 5, 64
    cos, sin = rope_tables(64, D, 500000.0, "cuda")
    x = torch.randn(B, S, nH, D, device="cuda").to(dtype).requires_grad_(True)
    dy = torch.randn(B, S, nH, D, device="cuda").to(dtype)
    y = apply_rope(x, cos, sin)
    y.backward(dy)
    xf = x.detach().float().requires_grad_(True)
    c, s = cos[:S].view(1, S, 1, D // 2), sin[:S].view(1, S, 1, D // 2)
    x1, x2 = xf[..., : D // 2], xf[..., D // 2:]
    ref = torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], -1)
    ref.backward(dy.float())
    tol = 2e-2 if dtype == torch.bfloat16 else 1e-5
    assert torch.allclose(y.float(), ref, atol=tol, rtol=tol)
    assert torch.allclose(x.grad.float(), xf.grad, atol=tol, rtol=tol)


def test_fused_adamw_matches_torch():
    from dynamiq_sigcomm_artifact_b200.ops.layers import FusedAdamW

    torch.manual_seed(1)
    shapes = [(1000,), (33, 77), (5000, 3), (1,)]
    ps = [torch.randn(s, device="cuda").requires_grad_(True) for s in shapes]
    qs = [p.detach().clone().requires_grad_(True) for p in ps]
    a = FusedAdamW(ps, lr=1e-2, weight_decay=0.1)
    b = torch.optim.AdamW(qs, lr=1e-2, weight_decay=0.1)
    for it in range(5):
        for p, q in zip(ps, qs):
            g = torch.randn_like(p)
            p.grad = g.clone()
            q.grad = g.clone()
        a.step()
        b.step()
    for p, q in zip(ps, qs):
        assert torch.allclose(p, q, atol=1e-5, rtol=1e-5)


@pytest.mark.parametrize("name", ["gpt2-tiny", "llama-tiny", "bert-tiny"])
def test_tiny_models_train_on_gpu(name):
    from dynamiq_sigcomm_artifact_b200.train.engine import TrainConfig, Trainer

    tr = Trainer(TrainConfig(model=name, micro_batch=2, seq_len=64, lr=1e-3,
                             task="mlm" if "bert" in name else "causal"), device=torch.device("cuda", 0))
    batch = tr.synthetic_batch()
    losses = [tr.train_step(batch) for _ in range(8)]
    assert all(l == l for l in losses) and losses[-1] < losses[0]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_fused_cross_entropy(dtype):
    from dynamiq_sigcomm_artifact_b200.ops.layers import fused_cross_entropy

    torch.manual_seed(2)
    N, V, Vp = 37, 1000, 1024
    base = (torch.randn(N, Vp, device="cuda") * 3).to(dtype)
    labels = torch.randint(0, V, (N,), device="cuda")
    labels[::5] = -100
    ref_in = base.float()[:, :V].clone().requires_grad_(True)
    ref = F.cross_entropy(ref_in, labels, ignore_index=-100)
    (ref * 2.0).backward()
    logits = base.clone().requires_grad_(True)
    work = logits * 1.0  # non-leaf, overwritten by the backward pass
    loss = fused_cross_entropy(work, labels, V)
    (loss * 2.0).backward()
    tol = 2e-2 if dtype == torch.bfloat16 else 1e-5
    assert abs(float(loss) - float(ref)) < tol
    g = logits.grad.float()
    assert torch.allclose(g[:, :V], ref_in.grad, atol=tol / 10, rtol=tol)
    assert float(g[:, V:].abs().max()) == 0.0 and float(g[::5].abs().max()) == 0.0


def test_padded_vocab_head_matches_plain_head():
    from dynamiq_sigcomm_artifact_b200.ops.layers import fused_cross_entropy, padded_vocab_logits, shift_labels

    torch.manual_seed(3)
    B, S, H, V = 2, 16, 64, 1001
    x = torch.randn(B, S, H, device="cuda", requires_grad=True)
    w = torch.randn(V, H, device="cuda", requires_grad=True)
    ids = torch.randint(0, V, (B, S), device="cuda")
    loss = fused_cross_entropy(padded_vocab_logits(x, w), shift_labels(ids).reshape(-1), V)
    loss.backward()
    x2, w2 = x.detach().clone().requires_grad_(True), w.detach().clone().requires_grad_(True)
    logits = F.linear(x2, w2)
    ref = F.cross_entropy(logits[:, :-1].reshape(-1, V), ids[:, 1:].reshape(-1))
    ref.backward()
    assert abs(float(loss) - float(ref)) < 1e-4
    assert torch.allclose(x.grad, x2.grad, atol=1e-4, rtol=1e-3)
    assert torch.allclose(w.grad, w2.grad, atol=1e-4, rtol=1e-3)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_swiglu_forward_backward(dtype):
    from dynamiq_sigcomm_artifact_b200.ops.layers import swiglu

    torch.manual_seed(4)
    x = torch.randn(3, 17, 256, device="cuda").to(dtype).requires_grad_(True)
    dy = torch.randn(3, 17, 128, device="cuda").to(dtype)
    y = swiglu(x)
    y.backward(dy)
    xf = x.detach().float().requires_grad_(True)
    g, u = xf.chunk(2, dim=-1)
    ref = F.silu(g) * u
    ref.backward(dy.float())
    tol = 3e-2 if dtype == torch.bfloat16 else 1e-5
    assert torch.allclose(y.float(), ref, atol=tol, rtol=tol)
    assert torch.allclose(x.grad.float(), xf.grad, atol=tol, rtol=tol)


def test_master_linear_matches_autocast_linear_and_optimizer_keeps_shadow():
    from dynamiq_sigcomm_artifact_b200.ops.layers import FusedAdamW
    from dynamiq_sigcomm_artifact_b200.ops.linear import MasterLinear, enable_shadows

    torch.manual_seed(5)
    lin = MasterLinear(64, 48).cuda()
    ref = torch.nn.Linear(64, 48).cuda()
    with torch.no_grad():
        ref.weight.copy_(lin.weight)
        ref.bias.copy_(lin.bias)
    shadows = enable_shadows(lin)
    x = torch.randn(5, 7, 64, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    x2 = x.detach().clone().requires_grad_(True)
    y = lin(x)
    with torch.autocast("cuda", dtype=torch.bfloat16):
        y2 = ref(x2)
    dy = torch.randn_like(y)
    y.backward(dy)
    y2.backward(dy)
    assert torch.allclose(y.float(), y2.float(), atol=2e-2, rtol=2e-2)
    assert lin.weight.grad.dtype == torch.float32
    assert torch.allclose(lin.weight.grad, ref.weight.grad, atol=3e-2, rtol=3e-2)
    assert torch.allclose(lin.bias.grad, ref.bias.grad, atol=3e-2, rtol=3e-2)
    assert torch.allclose(x.grad.float(), x2.grad.float(), atol=3e-2, rtol=3e-2)
    opt = FusedAdamW(lin.parameters(), lr=1e-2, shadows=shadows)
    opt.step()
    assert torch.equal(lin.shadow, lin.weight.to(torch.bfloat16))


@pytest.mark.parametrize("rows,cols,dtype", [(8192, 768, torch.bfloat16), (300, 3072, torch.bfloat16),
                                             (17, 132, torch.float32), (1, 4, torch.bfloat16)])
def test_colsum_matches_torch(rows, cols, dtype):
    from dynamiq_sigcomm_artifact_b200 import ops

    dq = ops.require()
    g = torch.Generator().manual_seed(rows + cols)
    x = torch.randn(rows, cols, generator=g).to(dtype).cuda()
    want = x.float().sum(dim=0)
    got = dq.colsum(x, None)
    assert got.dtype == torch.float32 and got.shape == (cols,)
    assert torch.allclose(got, want, rtol=1e-4, atol=1e-3)
    out = torch.full((cols,), 7.0, device="cuda")
    ret = dq.colsum(x, out)
    assert ret.data_ptr() == out.data_ptr() and torch.allclose(out, want, rtol=1e-4, atol=1e-3)
    assert torch.equal(dq.colsum(x, None), got), "two runs must agree bit for bit"
