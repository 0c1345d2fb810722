"""Packaging and the ``galvatron`` import alias (reference: setup.py:39-96, galvatron/core/__init__.py:1-17)."""
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_galvatron_alias_exposes_the_reference_names():
    code = ("import galvatron, galvatron.core as c, galvatron.utils as u;"
            "names=['ModelProfiler','HardwareProfiler','RuntimeProfiler','init_empty_weights',"
            "'construct_hybrid_parallel_model_api','get_hybrid_parallel_configs_api','set_megatron_args_for_dataset',"
            "'clip_grad_norm','get_optimizer_and_param_scheduler','GalvatronSearchEngine','initialize_galvatron','get_args'];"
            "missing=[n for n in names if not hasattr(c,n)]; assert not missing, missing;"
            "assert callable(u.read_json_config) and galvatron.__version__; print('ok')")
    env = dict(os.environ, PYTHONPATH=os.pathsep.join([os.path.join(ROOT, "compat"), ROOT, os.environ.get("PYTHONPATH", "")]))
    out = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, cwd="/tmp")
    assert out.returncode == 0 and "ok" in out.stdout, out.stderr


def test_setup_metadata_lists_both_packages():
    env = dict(os.environ, GV_SKIP_NATIVE_BUILD="1")
    out = subprocess.run([sys.executable, "setup.py", "--name", "--version"], cwd=ROOT, env=env, capture_output=True, text=True)
    assert out.returncode == 0, out.stderr
    lines = out.stdout.strip().splitlines()
    assert lines[-2] == "hetu-galvatron-b200" and lines[-1][0].isdigit()


def test_galvatron_models_alias_follows_the_reference_import_paths():
    """The import lines of the reference's per-family programs (models/<dir>/train_dist.py, train_dist_random.py, profiler.py,
    search_dist.py) resolve, and the names do what they say on a tiny model."""
    code = r'''
import argparse, torch
from galvatron.models.llama_hf.LlamaModel_hybrid_parallel import get_llama_config, llama_model_hp, get_runtime_profiler
from galvatron.models.llama_hf.LlamaModel_checkpoint import save_llama_module
from galvatron.models.llama_hf.arguments import model_args, layernum_arg_names
from galvatron.models.llama_hf.dataloader import DataLoaderForLlama, random_collate_fn, get_batch, get_train_valid_test_data_iterators
from galvatron.models.llama_hf.meta_configs import model_name, model_layer_configs
from galvatron.models.llama_fa.dataloader import DataLoaderForLlama as FA
from galvatron.models.gpt_hf.GPTModel_hybrid_parallel import get_gpt_config, gpt_model_hp
from galvatron.models.gpt_fa.dataloader import DataLoaderForGPT
from galvatron.models.bert_hf.BertModel_hybrid_parallel import bert_model_hp, get_bert_config
from galvatron.models.bert_hf.dataloader import DataLoaderForBert, random_collate_fn_bert
from galvatron.models.vit_hf.dataloader import DataLoaderForViT, vit_collate_fn
from galvatron.models.vit_hf.arguments import seqlen_arg_names as vit_seq
from galvatron.models.T5.T5Model_hybrid_parallel import get_t5_config, t5_model_hp
from galvatron.models.T5.T5Model_checkpoint import save_t5_module
from galvatron.models.T5.arguments import seqlen_arg_names, layernum_arg_names as t5_layers
from galvatron.models.T5.dataloader import DataLoaderForT5, random_collate_fn as t5_collate, loss_func
from galvatron.models.swin.SwinModel_hybrid_parallel import get_swin_config, swin_model_hp
from galvatron.models.swin.dataloader import DataLoaderForSwin
from galvatron.models.swin.meta_configs import model_layer_configs as swin_layers
import galvatron.models.llama_hf as pkg
assert FA is DataLoaderForLlama and callable(pkg.llama_model_hp)
assert layernum_arg_names() == ["num_hidden_layers"] and t5_layers() == ["num_encoder_layers", "num_decoder_layers"]
assert seqlen_arg_names() == ["encoder_seq_length", "decoder_seq_length"] and vit_seq() == []
p = model_args(argparse.ArgumentParser()); a = p.parse_args(["--model_size", "llama-7b"])
a.mixed_precision, a.set_model_config_manually, a.set_layernum_manually, a.set_seqlen_manually = "bf16", 0, 0, 0
cfg = get_llama_config(a)
assert cfg.hidden_size == 4096 and model_name(cfg).startswith("hidden4096_head32") and model_layer_configs(cfg)[0]["layer_num"] == 32
print("ok")
'''
    env = dict(os.environ, PYTHONPATH=os.pathsep.join([os.path.join(ROOT, "compat"), ROOT, os.environ.get("PYTHONPATH", "")]),
               CUDA_VISIBLE_DEVICES="")
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=300, env=env)
    assert r.returncode == 0 and r.stdout.strip().endswith("ok"), r.stderr[-3000:]


def test_a_program_written_for_the_reference_trains_through_the_alias(tmp_path):
    """The body of the reference's models/bert_hf/train_dist_random.py and T5/train_dist_random.py, with only the optimizer
    line taken from its train_dist.py (the engine owns the optimizer state): imports, data loader call, batch shape
    ``tokens, kwargs, loss_func`` and ``forward_backward(batch, iter, profiler, loss_func=..., **kwargs)`` as written there."""
    program = r'''
import os, sys, torch
from galvatron.core import initialize_galvatron, get_optimizer_and_param_scheduler
from galvatron.utils import distributed_dataloader, print_loss, set_seed
FAMILY = sys.argv.pop(1)
if FAMILY == "bert":
    from galvatron.models.bert_hf.arguments import model_args
    from galvatron.models.bert_hf.BertModel_hybrid_parallel import bert_model_hp as model_hp, get_bert_config as get_config, get_runtime_profiler
    from galvatron.models.bert_hf.dataloader import DataLoaderForBert as Data, random_collate_fn_bert as collate
else:
    from galvatron.models.T5.arguments import model_args
    from galvatron.models.T5.T5Model_hybrid_parallel import t5_model_hp as model_hp, get_t5_config as get_config, get_runtime_profiler
    from galvatron.models.T5.dataloader import DataLoaderForT5 as Data, random_collate_fn as collate

def train(args):
    config = get_config(args)
    model = model_hp(config, args)
    trainloader = distributed_dataloader(dataset=Data(args, None, 32), global_bsz=args.global_train_batch_size, shuffle=True,
                                         args=args, group=model.dp_groups_whole[0].group, collate_fn=collate)
    optimizer, opt_param_scheduler = get_optimizer_and_param_scheduler(model, args)
    profiler = get_runtime_profiler(args, os.path.dirname(os.path.abspath(__file__)), config)
    profiler.profile_memory(0, "After creating model")
    for ep in range(1):
        for iter, batch in enumerate(trainloader):
            tokens, kwargs, loss_func = batch
            profiler.profile_time_start(iter)
            input_ids = tokens
            batch = [input_ids]
            loss = model.forward_backward(batch, iter, profiler, loss_func=loss_func, **kwargs)
            optimizer.step()
            optimizer.zero_grad()
            print_loss(args, loss, ep, iter)
            profiler.profile_time_end(iter)

if __name__ == "__main__":
    args = initialize_galvatron(model_args, mode="train_dist")
    set_seed()
    train(args)
'''
    path = tmp_path / "train_dist_random.py"
    path.write_text(program)
    env = dict(os.environ, PYTHONPATH=os.pathsep.join([os.path.join(ROOT, "compat"), ROOT, os.environ.get("PYTHONPATH", "")]),
               CUDA_VISIBLE_DEVICES="")
    flags = ["--pp_deg", "1", "--global_tp_deg", "1", "--global_train_batch_size", "4", "--chunks", "2", "--set_model_config_manually", "1",
             "--hidden_size", "64", "--num_attention_heads", "4", "--num_hidden_layers", "2", "--vocab_size", "256",
             "--set_seqlen_manually", "1", "--seq_length", "32", "--mixed_precision", "fp32", "--profile", "0", "--dropout_prob", "0"]
    for family in ("bert", "t5"):
        r = subprocess.run([sys.executable, str(path), family] + flags, capture_output=True, text=True, timeout=600, env=env)
        assert r.returncode == 0, r.stderr[-3000:]
        losses = [float(line.split("Loss = ")[1]) for line in r.stdout.splitlines() if "Loss = " in line]
        assert len(losses) == 8 and all(3.0 < v < 8.0 for v in losses), r.stdout[-2000:]


def test_the_reference_train_dist_program_shape_runs_through_the_alias(tmp_path):
    """The body of the reference's models/llama_hf/train_dist.py (token files, get_batch, clip_grad_norm, scheduler step with
    args.global_batch_size, optimizer.param_groups, profile_time_end with loss / lr / norm, save_llama_module), minus its
    HuggingFace, tqdm and Megatron imports."""
    import numpy as np

    from hetu_galvatron_b200.core.dataloader import write_indexed_dataset

    rng = np.random.RandomState(0)
    write_indexed_dataset(str(tmp_path / "corpus"), [rng.randint(1, 250, rng.randint(40, 200)).tolist() for _ in range(64)])
    program = r'''
import os, torch
from galvatron.core import (RuntimeProfiler, clip_grad_norm, get_optimizer_and_param_scheduler, initialize_galvatron,
                            set_megatron_args_for_dataset)
from galvatron.models.llama_hf.arguments import model_args
from galvatron.models.llama_hf.dataloader import DataLoaderForLlama, get_batch, get_train_valid_test_data_iterators, loss_func
from galvatron.models.llama_hf.LlamaModel_checkpoint import save_llama_module
from galvatron.models.llama_hf.LlamaModel_hybrid_parallel import get_llama_config, get_runtime_profiler, llama_model_hp
from galvatron.models.llama_hf.meta_configs import model_layer_configs, model_name
from galvatron.utils import distributed_dataloader, print_loss, set_seed, print_param_num

def train(args):
    config = get_llama_config(args)
    model = llama_model_hp(config, args)
    set_megatron_args_for_dataset(args, model, model.sp_groups_whole[0] if args.vocab_sp else model.tp_groups_whole[0],
                                  model.vtp_data_group, model.cp_groups_whole[0])
    train_data_iterator, valid_data_iterator, test_data_iterator = get_train_valid_test_data_iterators()
    optimizer, opt_param_scheduler = get_optimizer_and_param_scheduler(model, args)
    path = os.path.dirname(os.path.abspath(__file__))
    profiler = get_runtime_profiler(args, path, config, start_iter=0)
    profiler.profile_memory(0, "After creating model")
    for iter in range(args.iteration, args.train_iters):
        tokens, kwargs, loss_func = get_batch(train_data_iterator)
        profiler.profile_time_start(iter)
        profiler.profile_memory(iter, "Before Forward")
        input_ids = tokens
        batch = [input_ids]
        loss = model.forward_backward(batch, iter, profiler, loss_func=loss_func, **kwargs)
        profiler.profile_memory(iter, "After Backward")
        total_norm = clip_grad_norm(model, args.clip_grad)
        optimizer.step()
        opt_param_scheduler.step(increment=args.global_batch_size)
        profiler.profile_memory(iter, "After optimizer_step")
        optimizer.zero_grad()
        print_loss(args, loss, 0, iter)
        profiler.post_profile_memory(iter)
        for param_group in optimizer.param_groups:
            learning_rate = param_group["lr"]
        profiler.profile_time_end(iter, loss, learning_rate, total_norm)
        if args.save != None and (iter + 1) % args.save_interval == 0:
            save_llama_module(args.save, model, optimizer, opt_param_scheduler, iter + 1, args)

if __name__ == "__main__":
    args = initialize_galvatron(model_args, mode="train_dist")
    set_seed()
    train(args)
'''
    path = tmp_path / "train_dist.py"
    path.write_text(program)
    env = dict(os.environ, PYTHONPATH=os.pathsep.join([os.path.join(ROOT, "compat"), ROOT, os.environ.get("PYTHONPATH", "")]),
               CUDA_VISIBLE_DEVICES="")
    flags = ["--pp_deg", "1", "--global_tp_deg", "1", "--global_train_batch_size", "4", "--chunks", "2", "--set_model_config_manually", "1",
             "--hidden_size", "64", "--num_attention_heads", "4", "--num_hidden_layers", "2", "--vocab_size", "256",
             "--set_seqlen_manually", "1", "--seq_length", "32", "--mixed_precision", "fp32", "--profile", "0", "--clip-grad", "1.0",
             "--data-path", str(tmp_path / "corpus"), "--train-iters", "4", "--save", str(tmp_path / "ckpt"), "--save-interval", "2",
             "--lr", "1e-3"]
    r = subprocess.run([sys.executable, str(path)] + flags, capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0, r.stderr[-3000:]
    losses = [float(line.split("Loss = ")[1]) for line in r.stdout.splitlines() if "Loss = " in line]
    assert len(losses) == 4 and all(4.0 < v < 7.0 for v in losses), r.stdout[-2000:]
    assert os.path.isdir(tmp_path / "ckpt" / "iter_2") and os.path.isdir(tmp_path / "ckpt" / "iter_4")


def test_submodule_paths_of_the_reference_resolve():
    """Import lines that reach into the reference's tree (its own tests use them: tests/search_engine/*.py,
    tests/models/test_dataloader.py, tests/profiler/*.py) find their counterparts."""
    code = r'''
from galvatron.core.search_engine.search_engine import GalvatronSearchEngine
from galvatron.core.search_engine.cost_model import MemoryCostModel, TimeCostModel, OtherTimeCostModel, pipeline_costmodel
from galvatron.core.search_engine.cost_model_args import ModelArgs, TrainArgs, ParallelArgs, ProfileModelArgs, ProfileHardwareArgs
from galvatron.core.search_engine.dynamic_programming import DPAlg, DpOnModel
from galvatron.core.search_engine.utils import get_thread_logger, ensure_log_dir
from galvatron.core.search_engine import GalvatronSearchEngine as G2
from galvatron.core.profiler.model_profiler import ModelProfiler
from galvatron.core.profiler.hardware_profiler import HardwareProfiler
from galvatron.core.profiler.runtime_profiler import RuntimeProfiler
from galvatron.core.profiler import ModelProfiler as M2
from galvatron.core.runtime.hybrid_parallel_config import get_hybrid_parallel_configs_api
from galvatron.core.runtime.hybrid_parallel_model import construct_hybrid_parallel_model_api
from galvatron.core.runtime.comm_groups import gen_comm_groups, CommGroup
from galvatron.core.runtime.redistribute import redistribute
from galvatron.core.runtime.utils import clip_grad_norm, get_optimizer_and_param_scheduler
from galvatron.core.runtime.initialize import init_empty_weights
from galvatron.core.arguments import initialize_galvatron
from galvatron.utils.strategy_utils import print_strategies, form_strategy
from galvatron.utils.training_utils import set_seed, distributed_dataloader, print_loss
from galvatron.utils.config_utils import read_json_config, write_json_config, str2array, array2str
import galvatron.core.search_engine.cost_model as cm, hetu_galvatron_b200.search.cost_model as own
assert G2 is GalvatronSearchEngine and M2 is ModelProfiler and cm.TimeCostModel is own.TimeCostModel
assert own.__name__ == "hetu_galvatron_b200.search.cost_model" and own.__spec__.name == own.__name__      # the originals are untouched
print("ok")
'''
    env = dict(os.environ, PYTHONPATH=os.pathsep.join([os.path.join(ROOT, "compat"), ROOT, os.environ.get("PYTHONPATH", "")]),
               CUDA_VISIBLE_DEVICES="")
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=300, env=env)
    assert r.returncode == 0 and r.stdout.strip().endswith("ok"), r.stderr[-3000:]
