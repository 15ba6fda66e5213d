"""Builds the reference's own ``quant_cuda`` extension for sm_100a into ``oracle/_ref/``.

    python oracle/build_ref.py [/path/to/reference]

The two source files are compiled where they lie (``src/alpaca_lora_4bit/quant_cuda/quant_cuda.cpp`` and
``quant_cuda_kernel.cu``), unmodified; ``oracle/ref_shim.h`` is force-included to supply one overload the
installed torch no longer has.  The result, ``oracle/_ref/quant_cuda_ref.so``, is test infrastructure: it lets
``tests/test_reference_kernels.py`` compare the CPU oracle and this library with the reference kernels
themselves on a GPU, and lets ``bench.py --impl reference`` time them.  Nothing in the package loads it.
"""
from __future__ import annotations

import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
NAME = "quant_cuda_ref"


def built_path() -> str:
    return os.path.join(OUT, NAME + ".so")


def build(reference_root: str = "/root/reference", verbose: bool = False) -> str | None:
    src = os.path.join(reference_root, "src", "alpaca_lora_4bit", "quant_cuda")
    cpp, cu = os.path.join(src, "quant_cuda.cpp"), os.path.join(src, "quant_cuda_kernel.cu")
    if not (os.path.exists(cpp) and os.path.exists(cu)):
        return None
    os.makedirs(OUT, exist_ok=True)
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0")
    from torch.utils import cpp_extension
    shim = os.path.join(HERE, "ref_shim.h")
    cpp_extension.load(
        name=NAME, sources=[cpp, cu], build_directory=OUT, verbose=verbose, is_python_module=False,
        extra_cflags=["-O2", "-include", shim, "-w"],
        extra_cuda_cflags=["-O2", "-include", shim, "-w", "-gencode", "arch=compute_100a,code=sm_100a"])
    return built_path()


def load():
    """Import the built extension (needs torch and, to run anything, a GPU); None if it was never built."""
    path = built_path()
    if not os.path.exists(path):
        return None
    import importlib.util
    import torch  # noqa: F401  (the extension links against libtorch)
    spec = importlib.util.spec_from_file_location(NAME, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    root = sys.argv[1] if len(sys.argv) > 1 else "/root/reference"
    print(build(root, verbose=True))
