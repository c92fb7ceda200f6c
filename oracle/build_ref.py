"""Builds the REFERENCE's own CUDA extension, unmodified, as a GPU-side oracle / baseline.

    [QMOE_REFERENCE=/path/to/reference] python oracle/build_ref.py     # needs the reference checkout

The two source files are compiled where they lie (``sub1_cuda.cpp`` and ``sub1_cuda_kernel.cu`` of
IST-DASLab/qmoe); nothing is copied and nothing is written outside ``oracle/_ref/``.  The recipe is
ours (torch's JIT extension builder with an explicit sm_100 target), not the reference's
``setup_cuda.py``.  The result, ``oracle/_ref/sub1_cuda.so``, is a torch extension module exposing
the reference's ``sub1matvec`` and ``sub1pack``; TEST INFRASTRUCTURE ONLY: the tests use it to check
the new kernels against the reference kernel on the same inputs, and the layer benchmark times it
next to them.  Load it with :func:`load` (it is NOT put on ``sys.path``).
"""
import glob
import importlib.util
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")


def reference_dir():
    """Where the reference checkout lies: ``$QMOE_REFERENCE``, else a directory named ``reference``
    beside this repository.  None when neither exists."""
    env = os.environ.get("QMOE_REFERENCE")
    cands = [env] if env else [os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")]
    for c in cands:
        if c and os.path.exists(os.path.join(c, "sub1_cuda_kernel.cu")):
            return c
    return None



def built_path():
    hits = sorted(glob.glob(os.path.join(OUT, "sub1_cuda*.so")))
    return hits[0] if hits else None


def build() -> str:
    ref = reference_dir()
    if ref is None:
        raise FileNotFoundError("reference checkout not found: set QMOE_REFERENCE to its directory")
    srcs = [os.path.join(ref, "sub1_cuda.cpp"), os.path.join(ref, "sub1_cuda_kernel.cu")]
    os.makedirs(OUT, exist_ok=True)
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0")
    os.environ.setdefault("MAX_JOBS", "4")
    from torch.utils import cpp_extension
    cpp_extension.load(name="sub1_cuda", sources=srcs, build_directory=OUT, verbose=True,
                       is_python_module=False)
    return built_path()


def load():
    """The reference extension module, or None if it has not been built."""
    path = built_path()
    if path is None:
        return None
    import torch  # noqa: F401  (the extension links against torch)
    spec = importlib.util.spec_from_file_location("sub1_cuda", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    print(build())
