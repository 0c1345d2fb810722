"""The reference's own CPU tests, run against this package through the ``galvatron`` import alias.

Set ``GALVATRON_REFERENCE_TESTS`` to the ``tests`` directory of a checkout of AFDWang/Hetu-Galvatron. The directory is copied
(a checkout may be read-only) and its search-engine tests (cost models, strategy generation, profile ingestion, pipeline
division, batch-size utilities, two end-to-end searches with golden throughputs) and the data-processing tests of its model
profiler run unchanged with ``galvatron`` resolving to ``compat/galvatron``. Skipped without the variable."""
import os
import re
import shutil
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SOURCE = os.environ.get("GALVATRON_REFERENCE_TESTS")

pytestmark = pytest.mark.skipif(not SOURCE or not os.path.isdir(SOURCE or ""), reason="GALVATRON_REFERENCE_TESTS not set")


def _run(tmp_path, *selection):
    work = tmp_path / "reference"
    if not work.exists():
        shutil.copytree(SOURCE, work / "tests")
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="",
               PYTHONPATH=os.pathsep.join([os.path.join(ROOT, "compat"), ROOT, str(work), os.environ.get("PYTHONPATH", "")]))
    r = subprocess.run([sys.executable, "-m", "pytest", "-q", "-p", "no:cacheprovider", "-W", "ignore", *selection],
                       cwd=str(work), capture_output=True, text=True, timeout=1500, env=env)
    tail = r.stdout.strip().splitlines()[-1] if r.stdout.strip() else ""
    return r, tail


def test_search_engine_tests_of_the_reference_pass(tmp_path):
    r, tail = _run(tmp_path, "tests/search_engine")
    assert r.returncode == 0, r.stdout[-4000:]
    assert int(re.search(r"(\d+) passed", tail).group(1)) >= 70 and "failed" not in tail


def test_profile_processing_and_attribute_helper_tests_of_the_reference_pass(tmp_path):
    r, tail = _run(tmp_path, "tests/profiler/test_model_profile.py", "tests/core/test_utils.py", "-k",
                   "get_seq_list or process_ or attr")
    assert r.returncode == 0, r.stdout[-4000:]
    assert int(re.search(r"(\d+) passed", tail).group(1)) >= 11 and "failed" not in tail
