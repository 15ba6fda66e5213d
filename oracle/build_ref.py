"""Builds the reference's own ``quant_cuda`` extension for sm_100a into ``oracle/_ref/``.

    python oracle/build_ref.py [/path/to/reference]

Without an argument the reference tree is looked for where ``$ALPACA_LORA_4BIT_REFERENCE`` points and then
in a directory named ``reference`` beside this repository; where there is none, nothing is built.

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


def find_reference() -> str | None:
    """Root of the reference tree: ``$ALPACA_LORA_4BIT_REFERENCE``, else ``../reference`` seen from the
    repository root; None if neither holds the extension's sources."""
    cands = [os.environ.get("ALPACA_LORA_4BIT_REFERENCE"), os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")]
    for c in cands:
        if c and os.path.exists(os.path.join(c, "src", "alpaca_lora_4bit", "quant_cuda", "quant_cuda_kernel.cu")):
            return c
    return None


def build(reference_root: str | None = None, verbose: bool = False) -> str | None:
    if reference_root is None:
        reference_root = find_reference()
    if reference_root is None:
        return None
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
    print(build(sys.argv[1] if len(sys.argv) > 1 else None, verbose=True))
