"""Host logic of the training pipeline and the amax tracker (axs/unified/training_unified.py), on CPU with a
model of plain layers; the behaviours checked are the ones the reference's tests/test_unified.py pins."""
import importlib
import math

import torch
import torch.nn as nn

tu = importlib.import_module("axs6_b200.unified.training_unified")


def _pipeline(**kw):
    torch.manual_seed(0)
    model = nn.Sequential(nn.Linear(8, 16), nn.ReLU(), nn.Linear(16, 1))
    opt = torch.optim.SGD(model.parameters(), lr=0.05)
    return tu.AXSTrainingPipelineUnified(model, opt, **kw), model


def _loss(out, x):
    return ((out - x[:, :1]) ** 2).mean()


def test_amax_ema():
    ema = tu.AmaxEMA(decay=0.9)
    assert ema.get_amax("w") == 1.0 and ema.get_scale("w") == 2.0
    ema.update("w", 3.0)
    assert ema.get_amax("w") == 3.0 and ema.get_scale("w") == 4.0
    ema.update("w", 13.0)
    assert math.isclose(ema.get_amax("w"), 0.9 * 3.0 + 0.1 * 13.0)
    ema.update("z", 0.0)
    assert ema.get_scale("z") == 1.0
    other = tu.AmaxEMA()
    other.load_state_dict(ema.state_dict())
    assert other.decay == 0.9 and other.get_amax("w") == ema.get_amax("w")


def test_steps_reduce_the_loss_and_report_the_reference_keys():
    pipe, _ = _pipeline(warmup_steps=2, loss_scale_growth_interval=3, max_grad_norm=10.0)
    x = torch.randn(64, 8)
    first = pipe.training_step(x, _loss)
    assert set(first) == {"loss", "loss_scale", "grad_norm", "overflow", "step", "warmup", "lr"}
    assert first["warmup"] is True and first["overflow"] is False and first["step"] == 1
    out = [pipe.training_step(x, _loss) for _ in range(30)]
    assert out[-1]["loss"] < 0.5 * first["loss"]
    assert out[0]["warmup"] is True and out[1]["warmup"] is False
    assert pipe.loss_scale == 2.0 ** 16 * 2.0 ** (31 // 3)             # grows every 3 clean steps
    st = pipe.stats
    assert st["total_steps"] == 31 and st["overflow_count"] == 0 and st["is_warmup"] is False
    assert st["max_grad_norm_recent"] >= st["avg_grad_norm_recent"] > 0


def test_overflow_backs_off_and_skips_the_update():
    pipe, model = _pipeline()
    x = torch.randn(16, 8)
    before = [p.detach().clone() for p in model.parameters()]
    res = pipe.training_step(x, lambda out, inp: out.sum() * float("inf"))
    assert res["overflow"] is True and res["grad_norm"] == 0.0 and res["step"] == 0
    assert pipe.loss_scale == 2.0 ** 15 and pipe.stats["overflow_count"] == 1
    for p, b in zip(model.parameters(), before):
        assert torch.equal(p, b) and (p.grad is None or float(p.grad.abs().sum()) == 0.0)


def test_checkpoint_round_trip(tmp_path):
    pipe, _ = _pipeline(use_amax_ema=True)
    pipe.scheduler = torch.optim.lr_scheduler.StepLR(pipe.optimizer, step_size=2, gamma=0.5)
    x = torch.randn(32, 8)
    for _ in range(3):
        pipe.training_step(x, _loss)
    pipe.amax_ema.update("w", 2.5)
    path = pipe.save_checkpoint(tmp_path / "sub" / "ck.pt", extra={"epoch": 7})
    want = [pipe.training_step(x, _loss)["loss"] for _ in range(3)]
    other, _ = _pipeline(use_amax_ema=True)
    other.scheduler = torch.optim.lr_scheduler.StepLR(other.optimizer, step_size=2, gamma=0.5)
    assert other.load_checkpoint(path) == {"epoch": 7}
    assert other.stats["total_steps"] == 3 and other.amax_ema.get_amax("w") == 2.5
    got = [other.training_step(x, _loss)["loss"] for _ in range(3)]
    assert got == want
