"""Packaging of moonep_b200.

``pip install --no-build-isolation .`` compiles the native library for sm_100a with
nvcc and ships it inside the package (``moonep_b200/_lib/libmoonep_b200.so``).  The library is
plain ``extern "C"`` code loaded with ctypes, so there is no Python extension module to link
against a particular torch build; torch is only a run-time dependency.  Counterpart of the
reference's setup.py (setup.py:24-77 there), which builds one host-only ``CUDAExtension``.
"""
import importlib.util
import pathlib

from setuptools import find_packages, setup
from setuptools.command.build_py import build_py

ROOT = pathlib.Path(__file__).resolve().parent


def _native_build():
    """Run moonep_b200/_build.py without importing the package (which would need torch)."""
    spec = importlib.util.spec_from_file_location("_moonep_b200_build", ROOT / "moonep_b200" / "_build.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.build()


class BuildWithNative(build_py):
    def run(self):
        print(f"built {_native_build()}")
        super().run()


setup(
    name="moonep_b200",
    version="0.1.0",
    description="Blackwell-native expert-parallel MoE communication library (sm_100a)",
    packages=find_packages(include=["moonep_b200", "moonep_b200.*"]),
    package_data={"moonep_b200": ["_lib/*.so"]},
    python_requires=">=3.10",
    install_requires=["torch", "numpy"],
    cmdclass={"build_py": BuildWithNative},
)
