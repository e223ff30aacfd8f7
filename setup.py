"""Packaging hook: ``pip install .`` / ``pip wheel .`` compile the native libraries for sm_100a (nvcc cross-compiles, no
GPU needed) before the package data is collected, so the wheel carries ``llmq_b200/lib/*.so`` (role of the reference's
scikit-build wheel, pyproject.toml + CMakeLists.txt:192-240)."""
import importlib.util
import os

from setuptools import setup
from setuptools.command.build_py import build_py


class BuildNativeThenPy(build_py):
    def run(self):
        here = os.path.dirname(os.path.abspath(__file__))
        spec = importlib.util.spec_from_file_location("_llmq_build", os.path.join(here, "llmq_b200", "build.py"))
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)                      # build.py has no package-relative imports
        mod.build(verbose=False)
        super().run()


setup(cmdclass={"build_py": BuildNativeThenPy})
