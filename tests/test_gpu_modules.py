"""Callers of the fake-quantise kernels besides the Linear layers: embedding, attention, model conversion
and the training pipeline (axs/unified/modules_unified.py:120-368, training_unified.py:115-410)."""
import importlib

import numpy as np
import pytest
import torch
import torch.nn as nn

import oracle
from gpu_util import assert_bits_equal

pytestmark = pytest.mark.gpu

from axs6_b200 import ops  # noqa: E402

um = importlib.import_module("axs6_b200.unified.modules_unified")
mp = importlib.import_module("axs6_b200.unified.mixed_precision")
tu = importlib.import_module("axs6_b200.unified.training_unified")


def test_embedding_quantises_only_the_looked_up_rows():
    torch.manual_seed(0)
    emb = um.AXSEmbeddingUnified(1000, 96, padding_idx=0).cuda()
    assert float(emb.weight.detach()[0].abs().sum()) == 0.0
    idx = torch.randint(0, 1000, (4, 17), device="cuda")
    out = emb(idx)
    rows = emb.weight.detach()[idx.reshape(-1)].cpu().numpy()
    assert_bits_equal(out, oracle.fused_fake_quantize(rows, 32).reshape(4, 17, 96), "embedding rows")
    out.sum().backward()                                   # straight-through: a count of occurrences per row
    counts = torch.bincount(idx.reshape(-1), minlength=1000).float()
    counts[0] = 0.0                                        # padding row receives no gradient
    torch.testing.assert_close(emb.weight.grad[:, 0], counts)
    emb._warmup_active = True
    assert torch.equal(emb(idx), emb.weight.detach()[idx])


def test_layer_norm_is_plain():
    ln = um.AXSLayerNormUnified(64).cuda()
    x = torch.randn(5, 64, device="cuda")
    torch.testing.assert_close(ln(x), torch.nn.functional.layer_norm(x, [64]))


def test_attention_shapes_gradients_and_quantised_weights():
    torch.manual_seed(1)
    att = um.AXSMultiheadAttentionUnified(64, 4).cuda()
    x = torch.randn(2, 48, 64, device="cuda", requires_grad=True)
    mask = torch.full((48, 48), float("-inf"), device="cuda").triu(1)
    y = att(x, x, x, attn_mask=mask)
    assert y.shape == (2, 48, 64) and bool(torch.isfinite(y).all())
    y.square().mean().backward()
    for p in list(att.parameters()) + [x]:
        assert p.grad is not None and bool(torch.isfinite(p.grad).all())
    # against the same attention in full precision: close, not equal
    with torch.no_grad():
        q, k, v = (torch.nn.functional.linear(x, m.weight, m.bias).reshape(2, 48, 4, 16).transpose(1, 2)
                   for m in (att.q_proj, att.k_proj, att.v_proj))
        w = torch.softmax(q @ k.transpose(-2, -1) * 0.25 + mask, dim=-1)
        ref = torch.nn.functional.linear((w @ v).transpose(1, 2).reshape(2, 48, 64), att.out_proj.weight, att.out_proj.bias)
    rel = float((y.detach() - ref).norm() / ref.norm())
    assert 0.0 < rel < 0.15, rel


def test_convert_to_axs_unified_swaps_linear_norm_and_embedding():
    class Tiny(nn.Module):
        def __init__(self):
            super().__init__()
            self.emb = nn.Embedding(50, 32)
            self.norm = nn.LayerNorm(32)
            self.fc = nn.Linear(32, 8)
            self.keep = nn.Linear(8, 8)

        def forward(self, t):
            return self.keep(self.fc(self.norm(self.emb(t))))

    src = Tiny().cuda()
    conv = um.convert_to_axs_unified(src, skip_layers={"keep"})
    assert isinstance(conv.emb, um.AXSEmbeddingUnified) and isinstance(conv.norm, um.AXSLayerNormUnified)
    assert isinstance(conv.fc, um.AXSLinearUnified) and type(conv.keep) is nn.Linear
    assert type(src.fc) is nn.Linear                                        # the source model is untouched
    for a, b in ((conv.emb.weight, src.emb.weight), (conv.fc.weight, src.fc.weight), (conv.norm.bias, src.norm.bias)):
        assert torch.equal(a, b) and a.data_ptr() != b.data_ptr()
    out = conv(torch.randint(0, 50, (3, 5), device="cuda"))
    assert out.shape == (3, 5, 8) and bool(torch.isfinite(out).all())
    again = um.convert_to_axs_unified(conv, inplace=True)
    assert again is conv and isinstance(again.fc, um.AXSLinearUnified)


def _mixed_model():
    torch.manual_seed(3)
    return nn.Sequential(mp.AXSLinearMixedPrecision(32, 64), nn.ReLU(), mp.AXSLinearMixedPrecision(64, 1)).cuda()


def _mse(out, x):
    return torch.nn.functional.mse_loss(out.float(), x[:, :4].sum(dim=1, keepdim=True) * 0.5)


def test_pipeline_trains_mixed_precision_layers_and_resumes_bit_identically(tmp_path):
    torch.manual_seed(11)
    ops.reset_philox(0)
    model = _mixed_model()
    pipe = tu.AXSTrainingPipelineUnified(model, torch.optim.AdamW(model.parameters(), lr=1e-2), warmup_steps=3,
                                         loss_scale_init=1024.0, max_grad_norm=5.0)
    x = torch.randn(256, 32, device="cuda")
    log = [pipe.training_step(x, _mse) for _ in range(40)]
    assert [r["warmup"] for r in log[:4]] == [True, True, True, False]
    assert all(m._warmup_active is False for m in model.modules() if isinstance(m, mp.AXSLinearMixedPrecision))
    assert not any(r["overflow"] for r in log) and log[-1]["loss"] < 0.6 * log[0]["loss"]
    path = pipe.save_checkpoint(tmp_path / "ck.pt")
    want = [pipe.training_step(x, _mse)["loss"] for _ in range(5)]

    other_model = _mixed_model()
    other = tu.AXSTrainingPipelineUnified(other_model, torch.optim.AdamW(other_model.parameters(), lr=1e-2), warmup_steps=3,
                                          loss_scale_init=1024.0, max_grad_norm=5.0)
    ops.reset_philox(12345)                                                  # must be overwritten by the checkpoint
    other.load_checkpoint(path, map_location="cuda")
    got = [other.training_step(x, _mse)["loss"] for _ in range(5)]
    assert got == want                                                       # same stochastic-rounding stream too


def test_pipeline_overflow_on_the_gpu_uses_one_fused_check():
    model = _mixed_model()
    pipe = tu.AXSTrainingPipelineUnified(model, torch.optim.SGD(model.parameters(), lr=0.1), loss_scale_init=8.0)
    x = torch.randn(64, 32, device="cuda")
    res = pipe.training_step(x, lambda out, inp: out.float().sum() * float("inf"))
    assert res["overflow"] is True and pipe.loss_scale == 4.0
    res = pipe.training_step(x, _mse)
    assert res["overflow"] is False and res["step"] == 1 and res["grad_norm"] > 0


def test_v1_modules_and_conversion():
    """axs/nn/modules.py: AXSLayerNorm quantises its output, AXSEmbedding its rows (both on the uniform grid),
    AXSMultiheadAttention runs on AXSLinear projections, convert_to_axs swaps Linear / LayerNorm / Embedding and
    convert_to_axs_unified accepts the V1 modules in turn."""
    nnm = importlib.import_module("axs6_b200.nn.modules")
    torch.manual_seed(2)
    ln = nnm.AXSLayerNorm(96).cuda()
    x = torch.randn(7, 96, device="cuda")
    want = oracle.fake_quantize_uniform(torch.nn.functional.layer_norm(x, [96]).cpu().numpy(), 32)
    assert_bits_equal(ln(x), want, "layer norm output")
    emb = nnm.AXSEmbedding(100, 64, padding_idx=3).cuda()
    idx = torch.randint(0, 100, (5, 9), device="cuda")
    rows = emb.weight.detach()[idx.reshape(-1)].cpu().numpy()
    assert_bits_equal(emb(idx), oracle.fake_quantize_uniform(rows, 32).reshape(5, 9, 64), "embedding rows")
    att = nnm.AXSMultiheadAttention(64, 4).cuda()
    q = torch.randn(2, 16, 64, device="cuda", requires_grad=True)
    y = att(q, q, q)
    y.sum().backward()
    assert y.shape == (2, 16, 64) and q.grad is not None and bool(torch.isfinite(q.grad).all())

    model = nn.Sequential(nn.Embedding(50, 32), nn.LayerNorm(32), nn.Linear(32, 8)).cuda()
    v1 = nnm.convert_to_axs(model, skip_layers={"2"})
    assert isinstance(v1[0], nnm.AXSEmbedding) and isinstance(v1[1], nnm.AXSLayerNorm) and type(v1[2]) is nn.Linear
    assert torch.equal(v1[0].weight, model[0].weight) and type(model[1]) is nn.LayerNorm
    v1 = nnm.convert_to_axs(model)
    assert isinstance(v1[2], nnm.AXSLinear)
    out = v1(torch.randint(0, 50, (4, 6), device="cuda"))
    assert out.shape == (4, 6, 8) and bool(torch.isfinite(out).all())
    uni = um.convert_to_axs_unified(v1)
    assert isinstance(uni[0], um.AXSEmbeddingUnified) and isinstance(uni[1], um.AXSLayerNormUnified)
    assert isinstance(uni[2], um.AXSLinearUnified) and torch.equal(uni[2].weight, model[2].weight)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("num,dim,shape", [(1000, 256, (4, 37)), (50, 100, (3,)), (32000, 1024, (8, 128))])
def test_embedding_gather_and_fake_quantise_in_one_kernel(num, dim, shape, dtype):
    """AXSEmbeddingUnified = fake_quantize_unified(F.embedding(...)) bit for bit (one fused kernel against the two-step
    form), padding row included; its weight gradient equals F.embedding's; an index outside the table sets the status
    flag instead of faulting."""
    import importlib
    mu = importlib.import_module("axs6_b200.unified.modules_unified")
    fu = importlib.import_module("axs6_b200.unified.functional_unified")
    from axs6_b200 import ops
    g = torch.Generator(device="cuda").manual_seed(num + dim)
    emb = mu.AXSEmbeddingUnified(num, dim, padding_idx=1).cuda().to(dtype)
    idx = torch.randint(0, num, shape, generator=g, device="cuda")
    idx.view(-1)[0] = 1
    out = emb(idx)
    want = fu.fake_quantize_unified(torch.nn.functional.embedding(idx, emb.weight.detach(), 1), emb.block_size, "nearest")
    assert out.shape == (*shape, dim) and out.dtype == dtype
    assert torch.equal(out.detach().view(torch.int16 if dtype == torch.bfloat16 else torch.int32),
                       want.view(torch.int16 if dtype == torch.bfloat16 else torch.int32))
    go = torch.randn(*shape, dim, generator=g, device="cuda").to(dtype)
    out.backward(go)
    w2 = emb.weight.detach().clone().requires_grad_(True)
    torch.nn.functional.embedding(idx, w2, 1).backward(go)
    assert torch.allclose(emb.weight.grad.float(), w2.grad.float(), rtol=1e-3 if dtype == torch.bfloat16 else 1e-6, atol=1e-6)
    assert not ops.gather_index_error()
    bad = idx.clone()
    bad.view(-1)[-1] = num + 5
    ops.fake_quantize_gather(emb.weight.detach(), bad)
    torch.cuda.synchronize()
    assert ops.gather_index_error() and not ops.gather_index_error()


def test_v1_embedding_is_the_fused_kernel_on_the_uniform_grid():
    from axs6_b200.nn import AXSEmbedding, fake_quantize
    g = torch.Generator(device="cuda").manual_seed(5)
    emb = AXSEmbedding(300, 96, padding_idx=0).cuda()
    idx = torch.randint(0, 300, (5, 17), generator=g, device="cuda")
    out = emb(idx)
    want = fake_quantize(torch.nn.functional.embedding(idx, emb.weight.detach(), 0), emb.block_size)
    assert out.dtype == torch.float32 and torch.equal(out.detach().view(torch.int32), want.view(torch.int32))
    out.sum().backward()
    assert emb.weight.grad is not None and float(emb.weight.grad[0].abs().sum()) == 0.0
