"""Model assembly: plan + model family -> the hybrid-parallel model that runs it.

Counterpart of the reference's ``construct_hybrid_parallel_model_api`` and ``GalvatronModel``
(galvatron/core/runtime/hybrid_parallel_model.py:42-70,165-326). The steps are the same in spirit --
groups, tensor-parallel modules, sequential stage, relayout at strategy boundaries, pipeline engine,
data-parallel wrapping, checkpoint wrapping -- but there is no model surgery on a HuggingFace skeleton:
every module is built directly in its sharded form on the device that runs it.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, List, Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from ..models.transformer import BatchCtx, LayerStrategy, ModelConfig
from ..parallel.mesh import Mesh
from ..parallel.pipeline import PipelineParallel, StageModule
from ..parallel.reshard import Layout
from ..parallel.zero import ParamBucket, ZeroBlock, ZeroEngine
from .plan import HybridPlan


@dataclass
class ModuleSpec:
    name: str                       # checkpoint block name, e.g. "model_layers_3"
    kind: str                       # embed | layer | norm | cls | other
    build: Callable                 # (LayerStrategy, device) -> nn.Module with forward(x, ctx)
    layer_index: Optional[int] = None   # index into the plan's per-layer lists (None for "other" modules)
    module_type: str = ""           # reference module type name, e.g. "gpt_dec", "embed"
    num_inputs: int = 1             # activations this module receives (2 for encoder-decoder decoder blocks)
    seq_attr: str = "seq_length"    # ModelConfig attribute holding the sequence length of its activations
    seq_attrs: Optional[tuple] = None   # one attribute per input where the inputs differ in length (encoder / decoder states)


def _strategy(mesh: Mesh, tp: int, sp: str, cp: int, dp_type: str, ckpt: bool, impl: str) -> LayerStrategy:
    tp_group = mesh.group("tp", tp)
    cp_group = mesh.group("cp", tp, cp)
    weight_tp = 1 if sp == "ulysses" else tp
    wdp = mesh.group("wdp", weight_tp)
    c = mesh.coords(tp, cp)
    if impl == "fused":
        # the fused tensor- / sequence- / context-parallel paths work on peer-mapped memory: a group that leaves the node
        # keeps the library collectives (every rank of a group sees the same rank list, so the group decides as one)
        from ..parallel.symm import ranks_on_one_node
        if not ranks_on_one_node(list(tp_group.ranks) + list(cp_group.ranks)):
            impl = "nccl"
    return LayerStrategy(tp=tp, sp=sp if tp > 1 else "none", cp=cp, dp_type=dp_type, checkpoint=ckpt, tp_group=tp_group,
                         cp_group=cp_group, wdp_group=wdp, impl=impl, tp_rank=c["tp"], cp_rank=c["cp"])


def layer_strategies(plan: HybridPlan, mesh: Mesh, impl: str = "nccl") -> List[LayerStrategy]:
    out = []
    for i in range(plan.num_layers):
        tp = plan.tp_sizes_enc[i]
        sp = "ulysses" if plan.use_sp[i] else ("megatron" if plan.sequence_parallel else "none")
        out.append(_strategy(mesh, tp, sp, plan.cp_sizes_enc[i], plan.layer_dp_type(i), bool(plan.checkpoint_flags_enc[i]), impl))
    return out


def other_strategy(plan: HybridPlan, mesh: Mesh, impl: str = "nccl") -> LayerStrategy:
    """Layout of the embedding / final norm / head (reference: hybrid_parallel_config.py:258-287)."""
    sp = "ulysses" if plan.vocab_sp else ("megatron" if plan.sequence_parallel else "none")
    dp_type = "zero3" if plan.embed_sdp else plan.default_dp_type
    return _strategy(mesh, plan.vocab_tp, sp, plan.vocab_cp, dp_type, False, impl)


def layout_of(st: LayerStrategy) -> Layout:
    return Layout(tp=st.tp, cp=st.cp, seq_sharded=st.sp in ("megatron", "ulysses") and st.tp > 1)


class DataReplicaGroup:
    """Data-parallel position of a rank: ``num_replicas`` positions, this rank at ``rank``. ``.group`` is the object
    itself, so that code written as ``model.dp_groups_whole[0].group`` hands it to ``distributed_dataloader``."""

    def __init__(self, num_replicas: int, rank: int):
        self.num_replicas, self.rank, self.size = int(num_replicas), int(rank), int(num_replicas)

    @property
    def group(self):
        return self


class GalvatronModel(nn.Module):
    """The object the training loop talks to: ``forward_backward(batch, iter, profiler, loss_func)``."""

    def __init__(self, cfg: ModelConfig, plan: HybridPlan, mesh: Mesh, stage: StageModule, engine: ZeroEngine,
                 pipeline: PipelineParallel, data_layout: Layout, label_layout: Layout, device, specs, my_specs, strategies):
        super().__init__()
        self.cfg, self.plan, self.mesh = cfg, plan, mesh
        self.model = stage
        self.engine = engine
        self.pipeline = pipeline
        self.data_layout, self.label_layout = data_layout, label_layout
        self.device = device
        self.specs, self.my_specs, self.strategies = specs, my_specs, strategies
        self.iter = 0

    # --- batch handling -------------------------------------------------------------------------------
    def local_batch_size(self) -> int:
        """Sequences per iteration this rank must be fed: the global batch split over the data layout."""
        return self.plan.global_bsz // self.data_layout.dp(self.mesh.stage_size)

    def batch_slice(self):
        """(lo, hi) rows of the global batch this rank consumes (its data-parallel shard)."""
        per = self.local_batch_size()
        idx = self.mesh.local // self.data_layout.block()
        return idx * per, (idx + 1) * per

    def mean_loss_over_ranks(self, loss):
        """Average of the per-rank mean losses over the last stage (for logging; None off the last stage)."""
        if not dist.is_initialized() or dist.get_world_size() == 1:
            return loss
        grp = self.mesh.group("stage")
        if loss is None:
            return None
        t = loss.detach().clone().float()
        if grp.size > 1:
            dist.all_reduce(t, group=grp.group)
            t /= grp.size
        return t

    def _micro_batches(self, batch) -> List[dict]:
        tokens, labels = batch[0], batch[1] if len(batch) > 1 else None
        extra = batch[2] if len(batch) > 2 and isinstance(batch[2], dict) else {}
        n = self.plan.chunks
        out = []
        tk = tokens.chunk(n, dim=0)
        lb = labels.chunk(n, dim=0) if labels is not None else [None] * n
        for i in range(n):
            e = {k: (v.chunk(n, dim=0)[i] if torch.is_tensor(v) and v.shape[0] == tokens.shape[0] else v) for k, v in extra.items()}
            out.append({"input": tk[i], "labels": lb[i], "extra": e})
        return out

    def forward_backward(self, batch, iter=None, profiler=None, loss_func=None, forward_only: bool = False, **kwargs):
        """Runs every micro-batch of one iteration through the chosen schedule; returns the mean loss
        (a tensor on the last stage, None elsewhere). Signature follows hybrid_parallel_model.py:42-70.

        ``batch`` is ``(input, labels[, extras])``. The reference's call shape is taken as well: ``batch = [input]`` with
        the labels and the other per-sample tensors as keyword arguments (``labels`` / ``dec_labels``, ``attention_mask``,
        ``token_type_ids``, ``dec_tokens`` ...; models/llama_hf/train_dist_random.py:53-60, T5/dataloader.py:24-44)."""
        if len(batch) == 1 and (kwargs.get("labels") is not None or kwargs.get("dec_labels") is not None):
            renamed = {"dec_tokens": "decoder_input_ids", "enc_attn_mask": None, "dec_attn_mask": None, "enc_dec_attn_mask": None}
            labels = kwargs["labels"] if kwargs.get("labels") is not None else kwargs["dec_labels"]
            extra = {renamed.get(k, k): v for k, v in kwargs.items()
                     if k not in ("labels", "dec_labels") and torch.is_tensor(v) and renamed.get(k, k) is not None}
            batch = (batch[0], labels, extra)
        micro = self._micro_batches(batch)
        if not forward_only and (self.cfg.dropout > 0.0 or getattr(self.cfg, "drop_path_rate", 0.0) > 0.0):
            # key of the counter-based dropout masks: (seed, iteration, micro-batch, first global-batch row of this rank)
            step = self.iter if iter is None else iter
            for i, m in enumerate(micro):
                m["extra"] = dict(m.get("extra") or {}, rng=(getattr(self.cfg, "dropout_seed", 1234), step, i, self.batch_slice()[0]))
        if profiler is not None and hasattr(profiler, "profile_memory"):
            profiler.profile_memory(iter, "Before Forward")
        losses = self.pipeline.forward_backward(micro, forward_only=forward_only)
        if not forward_only:
            self.engine.finish_step()
        if profiler is not None and hasattr(profiler, "profile_memory"):
            profiler.profile_memory(iter, "After Backward")
        self.iter += 1
        if losses:
            return torch.stack([l.float() for l in losses]).mean()
        return None

    def forward(self, batch):
        return self.forward_backward(batch, forward_only=True)

    # --- optimizer façade --------------------------------------------------------------------------------
    def optimizer_step(self, lr: float, **kw):
        return self.engine.step(lr, **kw)

    @property
    def dp_groups_whole(self):
        """One entry per module of this stage, as in the reference (hybrid_parallel_model.py:188-206), for the call
        ``distributed_dataloader(..., group=model.dp_groups_whole[0].group)``: what a data loader needs to know about
        the data-parallel position of this rank (how many positions, which one), without creating a process group."""
        per = self.local_batch_size()
        replica = DataReplicaGroup(self.plan.global_bsz // per, self.batch_slice()[0] // per)
        return [replica] * max(len(self.my_specs), 1)

    # per-module group lists under the reference's attribute names (hybrid_parallel_model.py:188-206); programs hand their
    # first entry to set_megatron_args_for_dataset
    @property
    def tp_groups_whole(self):
        return [st.tp_group for st in self.strategies]

    @property
    def sp_groups_whole(self):
        return [st.tp_group for st in self.strategies]      # Ulysses layers use the same ranks as their sequence group

    @property
    def cp_groups_whole(self):
        return [st.cp_group for st in self.strategies]

    @property
    def vtp_data_group(self):
        return self.dp_groups_whole[0]

    def set_loss_scale(self, scale: float) -> None:
        """What every micro-batch loss is multiplied by before backward (the optimizer step divides it out)."""
        self.pipeline.loss_scale = float(scale)

    def zero_grad(self):
        self.engine.zero_grad()


def construct_hybrid_parallel_model(cfg: ModelConfig, plan: HybridPlan, specs: List[ModuleSpec], device,
                                    mesh: Optional[Mesh] = None, impl: str = "nccl", async_grad_reduce: bool = True,
                                    grad_dtype: torch.dtype = torch.float32, reduce_in_fp32: bool = True,
                                    input_kind: str = "tokens", verbose: bool = False) -> GalvatronModel:
    world = dist.get_world_size() if dist.is_initialized() else 1
    mesh = mesh or Mesh(world, dist.get_rank() if dist.is_initialized() else 0, plan.pp_deg)
    plan.validate(world, cfg.num_heads, cfg.num_kv_heads if getattr(cfg, "model_type", "") != "swin" else None)
    lstrats = layer_strategies(plan, mesh, impl)
    ostrat = other_strategy(plan, mesh, impl)
    layer_specs = [s for s in specs if s.layer_index is not None]
    assert len(layer_specs) == plan.num_layers, "the plan has %d layers, the model %d" % (plan.num_layers, len(layer_specs))
    # stage assignment: layers by pp_division, leading "other" modules with the first layer's stage,
    # trailing ones with the last layer's stage
    stage_of_layer = plan.pp_ranks_enc
    stages, strategies = [], []
    for i, sp in enumerate(specs):
        if sp.layer_index is not None:
            stages.append(stage_of_layer[sp.layer_index])
            strategies.append(lstrats[sp.layer_index])
        else:
            before = [s.layer_index for s in specs[:i] if s.layer_index is not None]
            stages.append(stage_of_layer[before[-1]] if before else 0)
            strategies.append(ostrat)
    # a sequence-sharded layout needs the sequence to split evenly (for context parallelism: into 2 * cp zigzag chunks);
    # catching it here keeps an index computed for a ragged split from ever reaching a device kernel
    for sp_, st_ in zip(specs, strategies):
        parts = st_.seq_shards * (2 if st_.cp > 1 else 1)
        for attr in (sp_.seq_attrs or (sp_.seq_attr,)):
            seq = getattr(cfg, attr, None) or cfg.seq_length
            if st_.seq_shards > 1 and seq % parts != 0 and sp_.kind not in ("embed", "cls"):
                raise ValueError("module %s: a sequence of %d tokens cannot be split %d ways (tp %d with %s sequence parallelism, cp %d)"
                                 % (sp_.name, seq, parts, st_.tp, st_.sp, st_.cp))
    engine = ZeroEngine(async_grad_reduce=async_grad_reduce)
    if cfg.tie_embeddings and plan.pp_deg > 1:
        mesh.group("embed")          # created collectively by every rank, used by the first and last stage
    blocks, layouts, kinds, my_specs = [], [], [], []
    shared_bucket = {}
    for sp, stg, st in zip(specs, stages, strategies):
        if stg != mesh.stage:
            continue
        module = sp.build(st, device)
        tie_key = getattr(module, "tie_key", None)
        extra = []

        def new_bucket(name, params):
            b = ParamBucket(name, params, st.wdp_group, st.dp_type, grad_dtype=grad_dtype,
                            tp_group=st.tp_group if st.weight_tp > 1 else None,
                            reduce_dtype=None if reduce_in_fp32 else cfg.dtype, impl=impl)
            engine.add_bucket(b)
            return b

        params = [p for p in dict.fromkeys(module.parameters()) if not hasattr(p, "_gv_shape")]
        if tie_key is not None and plan.pp_deg > 1 and mesh.stage != 0:
            # both stages hold the summed gradient of a tied weight; the global norm counts the first stage's copy
            for p in params:
                if getattr(p, "tied", False):
                    p.norm_skip = True
        if tie_key is not None and tie_key in shared_bucket:
            # the tied weight already lives in the other block's bucket; this block's own parameters get theirs
            extra = [shared_bucket[tie_key]]
            bucket = new_bucket(sp.name, params)
        else:
            bucket = new_bucket(sp.name, params)
            if tie_key is not None:
                shared_bucket[tie_key] = bucket
                if plan.pp_deg > 1:
                    # tied weights living on two stages: sum their gradients over {first, last} stage before reducing
                    bucket.deferred = True
                    egrp = mesh.group("embed")
                    tied = [p for p in params if getattr(p, "tied", False)]
                    bucket.pre_reduce_hooks.append(lambda tied=tied, egrp=egrp: [
                        dist.all_reduce(p.main_grad, group=egrp.group) for p in tied if egrp.size > 1])
        blocks.append(ZeroBlock(module, bucket, engine, checkpoint=st.checkpoint, extra_buckets=extra))
        layouts.append(layout_of(st))
        kinds.append(sp.kind)
        my_specs.append(sp)
    # layout of what the previous stage sends
    in_layout = None
    prev_strats = [st for stg, st in zip(stages, strategies) if stg == mesh.stage - 1]
    if prev_strats:
        in_layout = layout_of(prev_strats[-1])
    from ..parallel.symm import ranks_on_one_node
    stage_impl = impl if ranks_on_one_node(range(mesh.stage * mesh.stage_size, (mesh.stage + 1) * mesh.stage_size)) else "nccl"
    stage = StageModule(blocks, layouts, kinds, mesh, in_layout, stage_impl)
    stage_batch = plan.global_bsz // plan.chunks
    data_layout = layout_of(ostrat)
    label_layout = layout_of(ostrat)
    S = mesh.stage_size
    hidden = cfg.hidden_size

    first_spec = my_specs[0] if my_specs else None
    act_hidden = getattr(first_spec, "hidden_size", None) or hidden

    def recv_shapes(micro) -> List[torch.Size]:
        lay = in_layout
        b_loc = stage_batch // lay.dp(S)
        attrs = first_spec.seq_attrs or (first_spec.seq_attr,) * first_spec.num_inputs
        return [torch.Size([(getattr(cfg, a, None) or cfg.seq_length) // lay.seq_parts() * b_loc, act_hidden]) for a in attrs]

    def make_ctx(micro) -> BatchCtx:
        b_loc = stage_batch // data_layout.dp(S)
        ctx = BatchCtx(batch=b_loc, seq=cfg.seq_length, labels=micro.get("labels"), extra=dict(micro.get("extra") or {}))
        if in_layout is not None:
            ctx.batch = stage_batch // in_layout.dp(S)
        return ctx

    pipeline = PipelineParallel(stage, mesh, engine, chunks=plan.chunks, pipeline_type=plan.pipeline_type,
                                stage_batch=stage_batch, recv_shape_fn=recv_shapes, act_dtype=cfg.dtype, device=device,
                                make_ctx=make_ctx)
    model = GalvatronModel(cfg, plan, mesh, stage, engine, pipeline, data_layout, label_layout, device, specs, my_specs,
                           [st for stg, st in zip(stages, strategies) if stg == mesh.stage])
    engine.sync_symmetric()
    if verbose and mesh.rank == 0:
        print(plan.describe(), flush=True)
    return model
