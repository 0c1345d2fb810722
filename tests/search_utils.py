"""Builds a search engine over the canned profile / hardware tables in tests/fixtures/search."""
import json
import os
import shutil
from types import SimpleNamespace

from hetu_galvatron_b200.search import GalvatronSearchEngine

FIX = os.path.join(os.path.dirname(os.path.abspath(__file__)), "fixtures", "search")


def search_args(**over):
    a = SimpleNamespace(
        set_model_config_manually=0, set_layernum_manually=0, set_seqlen_manually=0, num_nodes=1, num_gpus_per_node=8,
        memory_constraint=24, min_bsz=8, max_bsz=10240, recommend_min_bsz=0, settle_bsz=-1, settle_chunk=-1, bsz_scale=8,
        search_space="full", sp_space="tp", disable_dp=0, disable_tp=0, disable_vtp=0, disable_pp=0, disable_sdp=0,
        disable_ckpt=0, disable_tp_consec=0, max_tp_deg=8, max_pp_deg=8, default_dp_type="ddp", embed_sdp=0,
        mixed_precision="bf16", pipeline_type="gpipe", use_pipeline_costmodel=1, costmodel_coe=1.0, sequence_parallel=False,
        global_memory_buffer=True, async_grad_reduce=True, make_vocab_size_divisible_by=128, fine_grained_mode=1,
        time_profile_mode="static", memory_profile_mode="static", memory_profiling_path=None, time_profiling_path=None,
        allreduce_bandwidth_config_path=None, p2p_bandwidth_config_path=None, overlap_coe_path=None, sp_time_path=None,
        output_config_path=None, log_dir="logs", parallel_search=False, worker=0, hidden_size=3584,
        memory_layout="fsdp")        # the golden results were worked out with the reference's FSDP memory ratios
    for k, v in over.items():
        setattr(a, k, v)
    return a


LLAMA_SEARCH_LAYERS = [{"hidden_size": 3584, "layer_num": 28, "seq_len": 4096}]


def make_engine(tmp, time_mode="static", memory_mode="static", sp=False, seqlen_list=None, model_name="llama_search", **over):
    cfg_dir, hw_dir, out_dir = os.path.join(tmp, "configs"), os.path.join(tmp, "hardware"), os.path.join(tmp, "out")
    for d in (cfg_dir, hw_dir, out_dir):
        os.makedirs(d, exist_ok=True)
    args = search_args(time_profiling_path=cfg_dir, memory_profiling_path=cfg_dir, allreduce_bandwidth_config_path=hw_dir,
                       p2p_bandwidth_config_path=hw_dir, overlap_coe_path=hw_dir, sp_time_path=hw_dir, output_config_path=out_dir,
                       time_profile_mode=time_mode, memory_profile_mode=memory_mode, sequence_parallel=sp,
                       log_dir=os.path.join(tmp, "logs"))
    for k, v in over.items():
        setattr(args, k, v)
    eng = GalvatronSearchEngine(args)
    eng.set_search_engine_info(cfg_dir, LLAMA_SEARCH_LAYERS, model_name)
    if seqlen_list is not None:
        eng.seqlen_list = seqlen_list
    shutil.copy(os.path.join(FIX, "time_%s.json" % time_mode), os.path.join(cfg_dir, "computation_profiling_bf16_%s.json" % model_name))
    mem = {"static": "memory_static_sp.json" if sp else "memory_static.json", "sequence": "memory_sequence_sp.json"}[memory_mode]
    shutil.copy(os.path.join(FIX, mem), os.path.join(cfg_dir, "memory_profiling_bf16_%s.json" % model_name))
    hw = json.load(open(os.path.join(FIX, "hardware.json")))
    json.dump(hw["allreduce"], open(os.path.join(hw_dir, "allreduce_bandwidth_1nodes_8gpus_per_node.json"), "w"))
    json.dump(hw["p2p"], open(os.path.join(hw_dir, "p2p_bandwidth_1nodes_8gpus_per_node.json"), "w"))
    json.dump(hw["overlap"], open(os.path.join(hw_dir, "overlap_coefficient.json"), "w"))
    json.dump(hw["sp"], open(os.path.join(hw_dir, "sp_time_1nodes_8gpus_per_node.json"), "w"))
    eng.initialize_search_engine(show=False)
    return eng, out_dir


def write_tiny_gpt_profiles(root, worlds=(2,), seq=128):
    """Synthetic profiles of the tiny GPT decoder of the CPU plumbing configuration (hidden 256, 4 heads, 4 layers):
    1 ms forward per layer and sample, every link 2 GB/s, hardware tables for each world size in ``worlds``."""
    cfg, hw = os.path.join(root, "configs"), os.path.join(root, "hardware")
    os.makedirs(cfg), os.makedirs(hw)
    name = "hidden256_head4_seqlen%d" % seq
    json.dump({"layertype_0_bsz1_seq%d" % seq: 1.0, "layertype_other_bsz1_seq%d" % seq: 0.5},
              open(os.path.join(cfg, "computation_profiling_fp32_%s.json" % name), "w"))
    layer_mb = 12 * 256 * 256 * 4 / 2 ** 20                      # fp32 parameters of one layer
    act = {"1": 2.0, "2": 1.1, "4": 0.65, "checkpoint": 0.125}    # MB per sample
    states = 2 * 1024 * 256 * 4 * 4 / 2 ** 20
    other = {"model_states": {"1": states, "2": states / 2, "4": states / 4}, "activation": {"1": 1.0, "2": 0.6, "4": 0.4}}
    json.dump({"layertype_0": {str(seq): {"parameter_size": layer_mb, "tp_activation_per_bsz_dict": act}},
               "other_memory_pp_off": {str(seq): other}, "other_memory_pp_on_first": {str(seq): other},
               "other_memory_pp_on_last": {str(seq): other}},
              open(os.path.join(cfg, "memory_profiling_fp32_%s.json" % name), "w"))
    gbs = 2.0
    json.dump({"overlap_coe": 1.1}, open(os.path.join(hw, "overlap_coefficient.json"), "w"))
    for world in worlds:
        tag = "1nodes_%dgpus_per_node.json" % world
        ar, p2p, sp = {"allreduce_size_%d_consec_1" % world: gbs}, {}, {}
        k = world // 2
        while k >= 2:
            ar["allreduce_size_%d_consec_0" % k] = ar["allreduce_size_%d_consec_1" % k] = gbs
            k //= 2
        ar.setdefault("allreduce_size_2_consec_0", gbs)
        ar.setdefault("allreduce_size_2_consec_1", gbs)
        k = 2
        while k <= world:
            p2p["pp_size_%d" % k] = gbs
            for mb in (1, 2, 4, 8, 16, 32, 64, 128):
                sp["allreduce_size_%d_%dMB_time" % (k, mb)] = mb / 1024 / gbs * 1e3     # ms
                sp["all2all_size_%d_%dMB_time" % (k, mb)] = mb / 2 / 1024 / gbs * 1e3
            k *= 2
        json.dump(ar, open(os.path.join(hw, "allreduce_bandwidth_" + tag), "w"))
        json.dump(p2p, open(os.path.join(hw, "p2p_bandwidth_" + tag), "w"))
        json.dump(sp, open(os.path.join(hw, "sp_time_" + tag), "w"))
    return cfg, hw, name
