"""Loss scaling: the scalers themselves, the engine's scaled step, the optimizer façade and the fp16 program."""
import math
import os
import re
import subprocess
import sys
from types import SimpleNamespace

import torch

from hetu_galvatron_b200.core.hybrid_model import construct_hybrid_parallel_model
from hetu_galvatron_b200.core.loss_scaler import ConstantLossScaler, DynamicLossScaler, build_loss_scaler
from hetu_galvatron_b200.core.optimizer import Optimizer
from hetu_galvatron_b200.core.plan import HybridPlan
from hetu_galvatron_b200.models import build_model_specs, synthetic_batch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_dynamic_scaler_backs_off_after_hysteresis_and_grows_after_window():
    s = DynamicLossScaler(scale=1024.0, min_scale=128.0, growth_interval=3, hysteresis=2)
    s.update(True)
    assert s.scale == 1024.0 and s.skipped == 1            # first overflow is tolerated
    s.update(True)
    assert s.scale == 512.0
    s.update(True)
    assert s.scale == 256.0                                # budget stays spent until the scale grows again
    for _ in range(2):
        s.update(False)
    assert s.scale == 256.0
    s.update(False)
    assert s.scale == 512.0                                # three clean steps in a row
    s.update(True)
    assert s.scale == 512.0                                # growth refilled the budget
    for _ in range(10):
        s.update(True)
    assert s.scale == 128.0                                # never below the floor
    t = DynamicLossScaler()
    t.load_state_dict(s.state_dict())
    assert t.state_dict() == s.state_dict()


def test_constant_scaler_and_factory():
    c = ConstantLossScaler(8.0)
    c.update(True)
    c.update(False)
    assert c.scale == 8.0 and c.skipped == 1
    assert build_loss_scaler(SimpleNamespace(mixed_precision="bf16")) is None
    assert build_loss_scaler(SimpleNamespace(mixed_precision="fp32", loss_scale=4.0)).scale == 4.0
    d = build_loss_scaler(SimpleNamespace(mixed_precision="fp16", initial_loss_scale=256.0, loss_scale_window=7, hysteresis=1))
    assert isinstance(d, DynamicLossScaler) and d.scale == 256.0 and d.growth_interval == 7 and d.hysteresis == 1


def _tiny(seed=0):
    torch.manual_seed(seed)
    cfg, specs = build_model_specs("llama", dtype=torch.float32, hidden_size=32, num_heads=2, num_kv_heads=2,
                                   ffn_hidden_size=64, num_layers=2, vocab_size=64, seq_length=16)
    plan = HybridPlan.from_global(2, 1, global_bsz=4, chunks=2)
    model = construct_hybrid_parallel_model(cfg, plan, specs, torch.device("cpu"))
    return cfg, model


def _params(model):
    return torch.cat([p.detach().float().reshape(-1) for p in model.parameters()])


def test_scaled_step_equals_unscaled_step():
    """Scaling the loss by S and dividing S out in the optimizer step leaves losses, norm and weights unchanged."""
    cfg, plain = _tiny()
    _, scaled = _tiny()
    scaled.set_loss_scale(1024.0)
    for it in range(3):
        batch = synthetic_batch("llama", cfg, 4, seed=it, device="cpu")
        l0 = plain.forward_backward(batch, it)
        l1 = scaled.forward_backward(batch, it)
        assert torch.equal(l0, l1)                          # the reported loss is never scaled
        n0 = plain.optimizer_step(1e-2, max_grad_norm=0.5)
        n1 = scaled.optimizer_step(1e-2, max_grad_norm=0.5, loss_scale=1024.0)
        assert abs(float(n0) - float(n1)) <= 1e-5 * float(n0)
        plain.zero_grad()
        scaled.zero_grad()
    assert torch.allclose(_params(plain), _params(scaled), rtol=0, atol=2e-6)


def test_overflow_skips_the_step_everywhere_and_the_facade_halves_the_scale():
    cfg, model = _tiny()
    args = SimpleNamespace(lr=1e-2, mixed_precision="fp16", initial_loss_scale=float(2 ** 20), hysteresis=1, loss_scale_window=2,
                           clip_grad=1.0, train_iters=0, global_train_batch_size=4)
    opt = Optimizer(model, args)
    assert model.pipeline.loss_scale == float(2 ** 20)
    before = _params(model).clone()
    batch = synthetic_batch("llama", cfg, 4, seed=0, device="cpu")
    model.forward_backward(batch, 0)
    # poison one gradient the way an fp16 overflow does
    bucket = next(b for b in model.engine.buckets if b.numel)
    bucket.grad_shard.view(-1)[0] = float("inf")
    norm = opt.step()
    assert not math.isfinite(float(norm)) and opt.skipped_last_step and model.engine.step_count == 0
    assert torch.equal(_params(model), before)
    assert opt.loss_scale == float(2 ** 19) and model.pipeline.loss_scale == float(2 ** 19)
    opt.zero_grad()
    for it in (1, 2):
        model.forward_backward(batch, it)
        assert math.isfinite(float(opt.step())) and not opt.skipped_last_step
        opt.zero_grad()
    assert model.engine.step_count == 2 and not torch.equal(_params(model), before)
    assert opt.loss_scale == float(2 ** 20)                 # two clean steps: the window of this test


def test_fp16_program_recovers_from_an_overflowing_initial_scale():
    cmd = [sys.executable, os.path.join(ROOT, "hetu_galvatron_b200", "models", "llama_programs", "train_dist_random.py"),
           "--pp_deg", "1", "--global_tp_deg", "1", "--global_train_batch_size", "4", "--chunks", "2",
           "--set_model_config_manually", "1", "--hidden_size", "64", "--num_attention_heads", "4", "--num_hidden_layers", "2",
           "--ffn_hidden_size", "128", "--vocab_size", "256", "--set_seqlen_manually", "1", "--seq_length", "32",
           "--train-iters", "12", "--mixed_precision", "fp16", "--profile", "0", "--dropout_prob", "0",
           "--initial_loss_scale", "1e9", "--hysteresis", "1", "--lr", "1e-3"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=dict(os.environ, CUDA_VISIBLE_DEVICES=""))
    assert r.returncode == 0, r.stderr[-2000:]
    skipped = re.findall(r"\(Iteration (\d+)\): gradient overflow, step skipped; loss scale now ([0-9.e+]+)", r.stdout)
    losses = [float(x) for x in re.findall(r"\(Iteration \d+\): Loss = ([0-9.]+)", r.stdout)]
    assert len(losses) == 12 and all(math.isfinite(v) and 4.5 < v < 6.5 for v in losses)
    assert skipped and int(skipped[0][0]) == 0
    scales = [float(s) for _, s in skipped]
    assert all(abs(b - a / 2) <= 1e-4 * a for a, b in zip(scales, scales[1:]))      # printed with six digits
    assert len(skipped) < 12                                # some steps went through once the scale had come down
