"""Install the two packages and build the native libraries in place.

    python -m pip install --no-build-isolation -e .

``flagcx`` (the plug-in name of the reference, plugin/torch/setup.py:119) registers the PyTorch backend through the
``torch.backends`` entry point; ``flagcx_b200`` holds the library, the fused kernels and the tools.  The shared
objects are built by ``flagcx_b200._build`` (nvcc for sm_100a) into ``flagcx_b200/lib``."""
from setuptools import find_packages, setup
from setuptools.command.build_py import build_py


class BuildNative(build_py):
    def run(self):
        from flagcx_b200 import _build
        _build.build_all(verbose=True)
        super().run()


setup(
    name="flagcx-b200",
    version="0.1.0",
    description="Blackwell-native collective communication library with the FlagCX API and PyTorch backend",
    packages=find_packages(include=["flagcx", "flagcx.*", "flagcx_b200", "flagcx_b200.*"]),
    package_data={"flagcx_b200": ["lib/*.so"]},
    python_requires=">=3.10",
    cmdclass={"build_py": BuildNative},
    entry_points={"torch.backends": ["flagcx = flagcx:init"]},
)
