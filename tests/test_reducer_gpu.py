"""Gradient arena on the GPU: in-place gradients equal autograd's, the pipelined trainer equals the plain one."""
import pytest
import torch

pytestmark = pytest.mark.gpu

from dynamiq_sigcomm_artifact_b200.models import build_model, mask_tokens
from dynamiq_sigcomm_artifact_b200.ops.linear import enable_shadows
from dynamiq_sigcomm_artifact_b200.parallel.reducer import BucketReducer
from dynamiq_sigcomm_artifact_b200.train.engine import TrainConfig, Trainer


def _batch(model, seed, batch=2, seq=64):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, model.config.vocab, (batch, seq), generator=g).cuda()


@pytest.mark.parametrize("name", ["gpt2-tiny", "llama-tiny", "bert-tiny"])
def test_in_place_gradients_equal_autograd(name):
    torch.manual_seed(0)
    m, ref = build_model(name).cuda(), build_model(name).cuda()
    ref.load_state_dict(m.state_dict())
    enable_shadows(m), enable_shadows(ref)
    r = BucketReducer(m, bucket_cap_mb=0.01)
    assert r.direct and r.n_direct > 0
    ids = _batch(m, 3)
    labels = ids
    if name.startswith("bert"):
        gen = torch.Generator(device="cuda").manual_seed(5)
        ids, labels = mask_tokens(ids, m.config.vocab, m.config.mask_token_id, gen)
    for step in range(2):  # the second pass must overwrite, not accumulate
        r.begin_step()
        with torch.autocast("cuda", dtype=torch.bfloat16):
            la = m(ids, labels)
        la.backward()
        r.finish()
        torch.cuda.synchronize()
    with torch.autocast("cuda", dtype=torch.bfloat16):
        lb = ref(ids, labels)
    lb.backward()
    assert abs(float(la) - float(lb)) < 1e-3
    names = dict((id(p), n) for n, p in m.named_parameters())
    accum = {id(p) for ps in r.bucket_accum for p in ps}
    for (n, p), (_, q) in zip(m.named_parameters(), ref.named_parameters()):
        g = p.grad if id(p) not in accum else p.grad / 2  # accumulated ones saw two passes (nobody zeroed them)
        scale = float(q.grad.abs().max()) + 1e-12
        assert float((g - q.grad).abs().max()) <= 2e-2 * scale + 1e-6, n
    r.detach()


@pytest.mark.parametrize("name,graphs,tail", [("gpt2-tiny", True, 0), ("llama-tiny", True, 0), ("gpt2-tiny", False, 0),
                                              ("gpt2-tiny", True, 1)])
def test_pipelined_trainer_matches_plain_trainer(name, graphs, tail):
    """`tail` > 0: every bucket goes out after backward and the optimizer steps run on a second stream."""
    cfg = dict(model=name, micro_batch=2, seq_len=128, lr=1e-3, weight_decay=0.01, cuda_graphs=graphs)
    a = Trainer(TrainConfig(reducer="flat", tail_pipeline_mb=tail, bucket_cap_mb=1, **cfg))
    assert (a.reducer.consumer_stream is not None) == (tail > 0) and len(a.reducer.buckets) > 1
    b = Trainer(TrainConfig(reducer="ddp", **cfg))
    b.model.load_state_dict(a.model.state_dict())
    enable_shadows(b.model)
    assert a.graphed == graphs
    la = lb = None
    for s in range(6):
        ids = _batch(a.model, 20 + s, 2, 128)
        la, lb = float(a.train_step_device(ids)), float(b.train_step_device(ids))
        assert abs(la - lb) < 2e-2 * max(1.0, abs(lb)), (s, la, lb)
    torch.cuda.synchronize()
    for (n, p), (_, q) in zip(a.model.named_parameters(), b.model.named_parameters()):
        assert float((p - q).abs().mean()) < 2e-4, n  # a missed update of lr 1e-3 would show as ~1e-3
    # the bf16 working copies follow the fp32 parameters
    for p, sh in a.shadows.items():
        assert torch.equal(sh.view(-1)[: p.numel()].view_as(p), p.detach().to(torch.bfloat16))


def test_scatter_add_rows_is_exact_and_deterministic():
    from dynamiq_sigcomm_artifact_b200 import ops

    dq = ops.require()
    g = torch.Generator().manual_seed(1)
    V, d, n = 1000, 256, 4096  # many duplicate ids
    ids = torch.randint(0, V, (n,), generator=g).cuda()
    rows = torch.randn(n, d, generator=g).to(torch.bfloat16).cuda()
    base = torch.randn(V, d, generator=g).cuda()
    want = base.double().index_add(0, ids, rows.double() * 0.25)
    outs = []
    for _ in range(2):
        grad = base.clone()
        dq.scatter_add_rows(grad, ids, rows, 0.25)
        outs.append(grad)
    assert torch.equal(outs[0], outs[1])
    assert float((outs[0].double() - want).abs().max()) < 1e-4


@pytest.mark.parametrize("name", ["gpt2-tiny", "llama-tiny"])
def test_row_exchange_of_the_tied_embedding_matches_the_dense_path(name):
    """Single process with the row exchange forced on (the all-gather is the identity): same training run."""
    cfg = dict(model=name, micro_batch=2, seq_len=128, lr=1e-3, weight_decay=0.01)
    a = Trainer(TrainConfig(reducer="flat", sparse_embedding=True, **cfg))
    b = Trainer(TrainConfig(reducer="flat", sparse_embedding=False, **cfg))
    b.model.load_state_dict(a.model.state_dict())
    enable_shadows(b.model)
    assert a.reducer.sparse_params and not b.reducer.sparse_params
    names_a = [n for n, _ in a.model.named_parameters()]
    first_bucket = {id(p) for p in a.reducer.bucket_params[0]}
    assert id(a.reducer.sparse_params[0]) in first_bucket, "the tied weight is reduced with the head"
    for s in range(6):
        ids = _batch(a.model, 40 + s, 2, 128)
        la, lb = float(a.train_step_device(ids)), float(b.train_step_device(ids))
        assert abs(la - lb) < 2e-2 * max(1.0, abs(lb)), (s, la, lb)
    torch.cuda.synchronize()
    for (n, p), (_, q) in zip(a.model.named_parameters(), b.model.named_parameters()):
        assert float((p - q).abs().mean()) < 2e-4, n
