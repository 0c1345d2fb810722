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
