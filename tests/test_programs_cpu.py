"""The per-family entry programs, run as a user would (one CPU process, tiny manual model configs)."""
import os
import re
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TINY = ["--pp_deg", "1", "--global_tp_deg", "1", "--global_train_batch_size", "4", "--chunks", "1", "--set_model_config_manually", "1",
        "--hidden_size", "64", "--num_attention_heads", "4", "--num_hidden_layers", "2", "--vocab_size", "256",
        "--set_seqlen_manually", "1", "--seq_length", "32", "--train-iters", "4", "--mixed_precision", "fp32", "--profile", "0",
        "--dropout_prob", "0"]


def _run(program, *extra):
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "hetu_galvatron_b200", "models", program)] + TINY + list(extra),
                       capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0, r.stderr[-2000:]
    return r.stdout


def _losses(out):
    return [float(x) for x in re.findall(r"\(Iteration \d+\): Loss = ([0-9.]+)", out)]


def test_validation_passes_do_not_disturb_training():
    plain = _run("gpt_programs/train_dist_random.py")
    with_eval = _run("gpt_programs/train_dist_random.py", "--eval-iters", "2", "--eval-interval", "2")
    assert len(_losses(plain)) == 4 and _losses(plain) == _losses(with_eval)
    vals = re.findall(r"validation loss at iteration (\d+) \| lm loss value: ([0-9.E+-]+) \| lm loss PPL: ([0-9.E+-]+)", with_eval)
    assert [int(v[0]) for v in vals] == [2, 4]
    assert all(abs(float(v[1]) - 5.55) < 0.3 and float(v[2]) > 100 for v in vals)
    assert "validation loss" not in plain


def test_flash_attn_named_family_and_single_device_program():
    fa = _run("llama_fa_programs/train_dist_random.py", "--ffn_hidden_size", "128")
    base = _run("llama_programs/train_dist_random.py", "--ffn_hidden_size", "128")
    assert _losses(fa) == _losses(base) and len(_losses(fa)) == 4          # same model definition behind both names
    single = _run("bert_programs/train.py")
    assert len(_losses(single)) == 4


def test_random_dataset_feeds_the_programs():
    """--random_dataset 1: batches come from the family's random dataset through a torch DataLoader (padded sentence pairs
    with masked-language-model labels for BERT, two padded sides for T5); the run differs from the dense synthetic one."""
    dense = _losses(_run("bert_programs/train_dist_random.py"))
    a = _losses(_run("bert_programs/train_dist_random.py", "--random_dataset", "1"))
    assert len(a) == 4 and a != dense and all(3.0 < v < 8.0 for v in a)
    b = _losses(_run("t5_programs/train_dist_random.py", "--random_dataset", "1"))
    assert len(b) == 4 and all(3.0 < v < 8.0 for v in b)
