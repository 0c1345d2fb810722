"""Stand-ins for third-party native packages the reference imports but this image does not ship.

They are injected into ``sys.modules`` by the reference-arm launcher before the reference is imported; nothing in the
reference tree is modified. Each stand-in maps to a stock PyTorch equivalent:
  apex.optimizers.FusedAdam            -> torch.optim.AdamW(fused=True)
  apex.multi_tensor_apply / amp_C      -> torch._foreach_* based l2norm / scale
  flash_attn.ops.rms_norm.RMSNorm      -> a torch RMSNorm module (flash-attn's dropout_layer_norm extension is absent)
"""
import sys
import types

import torch


def _module(name):
    m = types.ModuleType(name)
    sys.modules[name] = m
    return m


def install():
    if "apex" not in sys.modules:
        try:
            import apex  # noqa: F401
        except Exception:
            apex = _module("apex")
            opt = _module("apex.optimizers")

            class FusedAdam(torch.optim.AdamW):
                def __init__(self, params, lr=1e-3, bias_correction=True, betas=(0.9, 0.999), eps=1e-8, adam_w_mode=True,
                             weight_decay=0.0, amsgrad=False, **kw):
                    super().__init__(params, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, amsgrad=amsgrad,
                                     fused=torch.cuda.is_available())

            class FusedSGD(torch.optim.SGD):
                pass

            opt.FusedAdam, opt.FusedSGD = FusedAdam, FusedSGD
            apex.optimizers = opt
            mta = _module("apex.multi_tensor_apply")

            def multi_tensor_applier(op, noop_flag, tensor_lists, *args):
                return op(noop_flag, tensor_lists, *args)

            mta.multi_tensor_applier = multi_tensor_applier
            apex.multi_tensor_apply = mta
            norm = _module("apex.normalization")
            apex.normalization = norm
    if "amp_C" not in sys.modules:
        try:
            import amp_C  # noqa: F401
        except Exception:
            amp = _module("amp_C")

            def multi_tensor_l2norm(noop_flag, tensor_lists, per_tensor):
                ts = tensor_lists[0]
                norms = torch._foreach_norm(ts, 2)
                total = torch.linalg.vector_norm(torch.stack([n.float() for n in norms]), 2)
                return total.reshape(1), None

            def multi_tensor_scale(noop_flag, tensor_lists, scale):
                src, dst = tensor_lists
                for s, d in zip(src, dst):
                    d.copy_(s * scale)

            amp.multi_tensor_l2norm, amp.multi_tensor_scale = multi_tensor_l2norm, multi_tensor_scale
    try:
        import flash_attn.ops.rms_norm  # noqa: F401
    except Exception:
        import flash_attn  # the core package is present

        ops = sys.modules.get("flash_attn.ops") or _module("flash_attn.ops")
        rms = _module("flash_attn.ops.rms_norm")

        class RMSNorm(torch.nn.Module):
            def __init__(self, hidden_size, eps=1e-5, dropout_p=0.0, device=None, dtype=None):
                super().__init__()
                self.eps = eps
                self.weight = torch.nn.Parameter(torch.ones(hidden_size, device=device, dtype=dtype))
                self.register_parameter("bias", None)

            def forward(self, x, residual=None, prenorm=False, residual_in_fp32=False):
                if residual is not None:
                    x = x + residual
                out = torch.nn.functional.rms_norm(x, (x.shape[-1],), self.weight, self.eps)
                return (out, x) if prenorm else out

        rms.RMSNorm = RMSNorm
        ops.rms_norm = rms
        flash_attn.ops = ops
