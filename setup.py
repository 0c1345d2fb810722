"""Packaging: ``pip install .`` builds the three native libraries in place (sm_100a CUDA kernel library, C++ search
core, C++ dataset index builder) and installs ``hetu_galvatron_b200`` plus the ``galvatron`` import alias.

The reference's setup (setup.py:39-96) compiles one pybind11 extension with setuptools; here the native build is the
package's own ``_build`` module (nvcc / g++ called directly, stale builds detected by hash), run as part of ``build_py``
so that a wheel carries the built ``.so`` files next to their sources.
"""
import importlib.util
import os
import re

from setuptools import find_packages, setup
from setuptools.command.build_py import build_py

ROOT = os.path.dirname(os.path.abspath(__file__))


def _version() -> str:
    text = open(os.path.join(ROOT, "hetu_galvatron_b200", "__init__.py")).read()
    return re.search(r'__version__\s*=\s*"([^"]+)"', text).group(1)


class BuildWithNative(build_py):
    """Compile the native libraries before the Python files are collected (skipped with GV_SKIP_NATIVE_BUILD=1)."""

    def run(self):
        if os.environ.get("GV_SKIP_NATIVE_BUILD", "0") != "1":
            spec = importlib.util.spec_from_file_location("_gv_build", os.path.join(ROOT, "hetu_galvatron_b200", "_build.py"))
            mod = importlib.util.module_from_spec(spec)
            spec.loader.exec_module(mod)
            mod.build_all(verbose=True)
        super().run()


packages = find_packages(include=("hetu_galvatron_b200", "hetu_galvatron_b200.*"))
alias = ["galvatron"] + ["galvatron." + p for p in find_packages(where=os.path.join("compat", "galvatron"))]

setup(
    name="hetu-galvatron-b200",
    version=_version(),
    description="Blackwell-native automatic hybrid-parallel Transformer training (profiler, search engine, runtime)",
    long_description=open(os.path.join(ROOT, "README.md")).read(),
    long_description_content_type="text/markdown",
    packages=packages + alias,
    package_dir={"galvatron": os.path.join("compat", "galvatron")},
    package_data={"hetu_galvatron_b200": ["_lib/*.so", "csrc/*.cu", "csrc/*.cpp", "csrc/include/*", "csrc/sim/*",
                                          "models/meta_configs/*.json", "models/*/configs/*.json", "models/*/scripts/*.sh",
                                          "profile_hardware/hardware_configs/*.json", "profile_hardware/scripts/*.sh", "tools/*.sh"]},
    include_package_data=True,
    python_requires=">=3.10",
    install_requires=["torch>=2.6", "numpy", "scipy", "pybind11>=2.9.1"],
    cmdclass={"build_py": BuildWithNative},
)
