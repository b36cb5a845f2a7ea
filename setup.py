"""Packaging of jax_gpt_b200 (the reference ships setup.py + requirements.txt: setup.py:1-28).

The CUDA extension is built IN TREE by ``jax_gpt_b200.build`` (nvcc, sm_100a) and lives next to the Python sources
as ``jax_gpt_b200/_C.so``; ``build_ext`` here only calls that builder, so

    python setup.py build_ext --inplace      # same as: python -m jax_gpt_b200.build
    pip install -e . --no-build-isolation    # development install; the package loads the in-tree library

work without a second build system. A missing nvcc is not an error at install time: the CPU paths of the package
do not need the library, and the first CUDA call builds it (or says that it cannot).
"""
import os
import sys

from setuptools import Command, find_packages, setup
from setuptools.command.build_py import build_py

HERE = os.path.dirname(os.path.abspath(__file__))


class BuildExt(Command):
    description = "build jax_gpt_b200/_C.so with nvcc for sm_100a (in tree)"
    user_options = [("inplace", "i", "accepted for compatibility; the library is always built in tree"),
                    ("force", "f", "rebuild every object"), ("debug", "g", "also build the range-checked _C_debug.so")]
    boolean_options = ["inplace", "force", "debug"]

    def initialize_options(self):
        self.inplace = self.force = self.debug = False

    def finalize_options(self):
        pass

    def run(self):
        sys.path.insert(0, HERE)
        from jax_gpt_b200 import build as b
        print(b.build(verbose=True, force=bool(self.force)))
        if self.debug:
            print(b.build(verbose=True, force=bool(self.force), debug=True))


class BuildPy(build_py):
    def run(self):
        try:
            self.run_command("build_ext")
        except Exception as e:  # no nvcc on this machine: the CPU paths still work
            print(f"[setup] extension not built ({e}); CUDA paths will build it on first use")
        super().run()


setup(
    name="jax_gpt_b200",
    version="0.2.0",
    description="Blackwell (sm_100a) native LLM training / serving framework with the feature set of jax-gpt",
    long_description=open(os.path.join(HERE, "README.md")).read(),
    long_description_content_type="text/markdown",
    packages=find_packages(include=["jax_gpt_b200", "jax_gpt_b200.*"]),
    package_data={"jax_gpt_b200": ["_C.so", "_C_debug.so", "csrc/*"]},
    python_requires=">=3.10",
    install_requires=[l.strip() for l in open(os.path.join(HERE, "requirements.txt")) if l.strip() and not l.startswith("#")],
    cmdclass={"build_ext": BuildExt, "build_py": BuildPy},
)
