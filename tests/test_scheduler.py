"""Learning-rate schedule (Megatron's OptimizerParamScheduler semantics: steps are counted in samples, linear warm-up,
then constant / linear / cosine / inverse-square-root decay to ``min_lr``) and its state round trip."""
import json
import math
from types import SimpleNamespace

import pytest

from hetu_galvatron_b200.core.optimizer import Optimizer, ParamScheduler, get_optimizer_and_param_scheduler


def test_warmup_then_decay_styles():
    s = ParamScheduler(max_lr=1.0, min_lr=0.1, warmup_steps=10, decay_steps=110, decay_style="linear")
    lrs = [s.step() for _ in range(120)]
    assert lrs[0] == pytest.approx(0.1) and lrs[4] == pytest.approx(0.5) and lrs[9] == pytest.approx(1.0)       # warm-up
    assert lrs[59] == pytest.approx(0.1 + 0.5 * 0.9) and lrs[109] == pytest.approx(0.1)                           # half-way, end
    assert lrs[115] == pytest.approx(0.1)                                                                         # floor afterwards
    assert all(a >= b - 1e-12 for a, b in zip(lrs[9:], lrs[10:]))                                                 # monotone decay
    c = ParamScheduler(max_lr=1.0, min_lr=0.0, warmup_steps=0, decay_steps=100, decay_style="cosine")
    assert c.step(25) == pytest.approx(0.5 * (math.cos(math.pi * 0.25) + 1)) and c.step(25) == pytest.approx(0.5)
    assert c.step(50) == pytest.approx(0.0, abs=1e-12)
    r = ParamScheduler(max_lr=1.0, min_lr=0.05, warmup_steps=16, decay_steps=10 ** 6, decay_style="inverse-square-root")
    r.step(16)
    assert r.get_lr() == pytest.approx(1.0)
    r.step(48)
    assert r.get_lr() == pytest.approx(0.5)                    # sqrt(16 / 64)
    r.step(10 ** 5)
    assert r.get_lr() == pytest.approx(0.05)                   # floor
    k = ParamScheduler(max_lr=3e-4, decay_style="constant")
    assert {k.step(7) for _ in range(5)} == {3e-4}
    with pytest.raises(ValueError):
        ParamScheduler(max_lr=1.0, decay_steps=10, decay_style="exponential").step()


def test_optimizer_facade_counts_samples_and_round_trips(tmp_path):
    calls = []
    model = SimpleNamespace(optimizer_step=lambda lr, **kw: calls.append((lr, kw)) or 1.25, zero_grad=lambda: calls.append("zero"))
    args = SimpleNamespace(lr=1e-3, min_lr=1e-4, lr_decay_style="cosine", lr_warmup_iters=2, lr_warmup_fraction=None, lr_decay_iters=None,
                           train_iters=10, global_train_batch_size=8, adam_beta1=0.9, adam_beta2=0.95, adam_eps=1e-8,
                           adam_weight_decay=0.1, clip_grad=1.0)
    opt, sched = get_optimizer_and_param_scheduler(model, args)
    assert isinstance(opt, Optimizer) and sched is opt.scheduler
    assert (sched.warmup_steps, sched.decay_steps) == (16, 80)                 # iterations x global batch
    seen = []
    for _ in range(10):
        assert opt.step() == 1.25
        seen.append(calls[-1][0])
        sched.step(increment=8)
        opt.zero_grad()
    assert calls[0][1] == dict(beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1, max_grad_norm=1.0, loss_scale=1.0)
    assert seen[1] == pytest.approx(0.5e-3) and seen[2] == pytest.approx(1e-3) and seen[-1] < seen[3] and min(seen[2:]) >= 1e-4
    # resume: the schedule continues where the checkpoint left it
    ck = tmp_path / "iter_10"
    ck.mkdir()
    (ck / "opt_param_scheduler.json").write_text(json.dumps(sched.state_dict()))
    args2 = SimpleNamespace(**vars(args), load=str(tmp_path), distributed_checkpoint=True, load_iteration=10)
    opt2, sched2 = get_optimizer_and_param_scheduler(model, args2)
    assert sched2.num_steps == 80 and opt2.lr == pytest.approx(opt.lr)
    frac = SimpleNamespace(**{**vars(args), "lr_warmup_fraction": 0.25})
    assert Optimizer(model, frac).scheduler.warmup_steps == 20
