"""The names a user of the reference imports from ``galvatron.core`` / ``galvatron.core.runtime`` / ``galvatron.utils``
resolve here (reference tests/core/test_utils.py:16-40 for the attribute helpers)."""
from types import SimpleNamespace

import pytest
import torch

import hetu_galvatron_b200.core as core
import hetu_galvatron_b200.utils as utils
from hetu_galvatron_b200.models import build_model_specs


def test_reference_names_resolve():
    for name in ("ModelProfiler", "HardwareProfiler", "RuntimeProfiler", "GalvatronSearchEngine", "initialize_galvatron",
                 "get_args", "init_empty_weights", "construct_hybrid_parallel_model_api", "get_hybrid_parallel_configs_api",
                 "set_megatron_args_for_dataset", "clip_grad_norm", "get_optimizer_and_param_scheduler", "ModelInfo",
                 "PipelineParallel", "PipeSequential", "ParallelAttention", "ParallelMLP", "gen_comm_groups",
                 "mixed_precision_dtype", "galvatron_training_args", "galvatron_profile_args",
                 "galvatron_profile_hardware_args", "galvatron_search_args"):
        assert getattr(core, name) is not None, name
    for name in ("str2array", "array2str", "read_json_config", "write_json_config", "config2strategy", "strategy2config",
                 "read_allreduce_bandwidth_config", "read_p2p_bandwidth_config", "num2str", "remap_config", "form_strategy",
                 "strategy_str2list", "print_strategies", "print_peak_memory", "print_param_num", "set_seed",
                 "distributed_dataloader", "print_loss", "rgetattr", "rsetattr", "rhasattr"):
        assert callable(getattr(utils, name)), name
    with pytest.raises(AttributeError):
        core.no_such_name
    assert core.mixed_precision_dtype("bf16") is torch.bfloat16 and core.mixed_precision_dtype("fp32") is torch.float32


def test_nested_attribute_helpers():
    obj = SimpleNamespace(a=SimpleNamespace(b=SimpleNamespace(c=3)), x=1)
    assert utils.rgetattr(obj, "a.b.c") == 3 and utils.rgetattr(obj, "x") == 1 and utils.rgetattr(obj, "") is obj
    assert utils.rgetattr(obj, "a.q.c", "fallback") == "fallback"
    with pytest.raises(AttributeError):
        utils.rgetattr(obj, "a.q")
    utils.rsetattr(obj, "a.b.c", 7)
    utils.rsetattr(obj, "y", 2)
    assert obj.a.b.c == 7 and obj.y == 2
    assert utils.rhasattr(obj, "a.b.c") and utils.rhasattr(obj, "") and not utils.rhasattr(obj, "a.b.d") and not utils.rhasattr(obj, "q.b")
    lin = torch.nn.Sequential(torch.nn.Linear(4, 3), torch.nn.Linear(3, 2, bias=False))
    assert utils.rgetattr(lin, "0.weight").shape == (3, 4)
    assert utils.print_param_num(lin) == 4 * 3 + 3 + 3 * 2


def test_model_info_from_specs():
    cfg, specs = build_model_specs("t5", dtype=torch.float32, hidden_size=64, num_heads=4, ffn_hidden_size=128, num_layers=2,
                                   num_decoder_layers=3, vocab_size=256, seq_length=16)
    info = core.ModelInfo(cfg, specs)
    assert info.layernums() == [2, 3]
    types = info.module_types()
    assert types.count("t5_enc") == 2 and types.count("t5_dec") == 3 and types[0].startswith("embed") and types[-1] == "cls"
    shapes, dtypes = info.shapes(), info.dtypes()
    assert len(shapes) == len(specs) == len(dtypes)
    dec = [i for i, t in enumerate(types) if t == "t5_dec"][0]
    assert shapes[dec] == [[16, -1, 64], [16, -1, 64]] and dtypes[dec] == [torch.float32] * 2      # encoder + decoder states
    swin_cfg, swin_specs = build_model_specs("swin", dtype=torch.float32, model_size="swin-tiny-test")
    sinfo = core.ModelInfo(swin_cfg, swin_specs)
    assert sinfo.layernums() == [1, 1, 2, 1]
    assert [s[0][2] for s, t in zip(sinfo.shapes(), sinfo.module_types()) if t == "swin_enc"] == [32, 64, 128, 128, 256]
    assert core.ModelInfo(cfg, specs, sequence_parallel_degree=2).shapes()[1][0][0] == 8


def test_family_entry_points_under_the_reference_names():
    from hetu_galvatron_b200.core import initialize_galvatron
    from hetu_galvatron_b200.models.arguments import make_model_args
    from hetu_galvatron_b200.models.gpt import GPTModelInfo, get_gpt_config, gpt_model_hp
    from hetu_galvatron_b200.models.llama import LlamaModelInfo, get_llama_config, llama_model_hp  # noqa: F401
    from hetu_galvatron_b200.models.swin import SwinModelInfo, get_swin_config, swin_model_hp      # noqa: F401
    from hetu_galvatron_b200.models.t5 import T5ModelInfo, get_t5_config, t5_model_hp              # noqa: F401

    args = initialize_galvatron(make_model_args("gpt"), mode="train", argv=[
        "--set_model_config_manually", "1", "--hidden_size", "64", "--num_attention_heads", "4", "--num_hidden_layers", "2",
        "--vocab_size", "256", "--set_seqlen_manually", "1", "--seq_length", "32", "--pp_deg", "1", "--global_tp_deg", "1",
        "--global_train_batch_size", "4", "--chunks", "1", "--mixed_precision", "fp32", "--dropout_prob", "0"])
    config = get_gpt_config(args)
    assert (config.hidden_size, config.num_layers, config.seq_length, config.vocab_size) == (64, 2, 32, 256)
    assert GPTModelInfo(config).layernums() == [2]
    model = gpt_model_hp(config, args)
    tokens = torch.randint(0, 256, (4, 33))
    loss = model.forward_backward((tokens[:, :-1], tokens[:, 1:]), 0)
    assert torch.isfinite(loss) and abs(float(loss) - 5.545) < 0.3
