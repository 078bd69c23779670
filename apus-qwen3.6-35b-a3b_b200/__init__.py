"""B200-native CUDA backend for the MoE block of the apus-qwen engine.

The directory name is not a Python identifier; load it by path, e.g.

    import importlib.util, sys
    spec = importlib.util.spec_from_file_location(
        "apus_b200", "<repo>/apus-qwen3.6-35b-a3b_b200/__init__.py",
        submodule_search_locations=["<repo>/apus-qwen3.6-35b-a3b_b200"])
    mod = importlib.util.module_from_spec(spec); sys.modules["apus_b200"] = mod
    spec.loader.exec_module(mod)

Contents: ``csrc/`` (CUDA kernels and the C-ABI, built into
``libapus_cuda.so``), ``build.py`` (the nvcc recipe), ``backend.py`` (ctypes
binding that mirrors the C entry points), ``synth.py`` (seeded synthetic
inputs for tests and benchmarks).
"""
from . import build  # noqa: F401
from .backend import Backend, MoeCfg, BackendError  # noqa: F401
