"""Recipe for ``baseline/_ref/``: the reference's CUDA kernels compiled for sm_100.

The reference ships no Blackwell kernel; its extensions are built for sm_89 / sm_86 only
(``csrc/build.py:52-74``).  "The kernels to beat" on a B200 are therefore the reference's own
sources with nothing but the ``-gencode`` target changed.  This script builds the three
extension sources where they lie in a reference checkout (nothing is copied) with the
reference's flags (``-O3 --use_fast_math``) and ``-gencode=arch=compute_100,code=sm_100`` into
``baseline/_ref/<name>/`` (git-ignored).  ``bench.py`` loads the resulting modules, when they
exist, to time them per shape beside this library; they are never on the product path.

    python baseline/make_ref_kernels.py [reference checkout] [int8_gemm_tc int8_sparse_tc int8_kernels]
"""
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
NAMES = ("int8_gemm_tc", "int8_sparse_tc", "int8_kernels")


def build(reference_dir: str, names=NAMES, verbose: bool = False) -> dict:
    """name -> path of the built module, or the error text if it did not build."""
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0")
    from torch.utils.cpp_extension import load
    flags = ["-O3", "--use_fast_math", "-gencode=arch=compute_100,code=sm_100", "--allow-unsupported-compiler"]
    out = {}
    for name in names:
        src = os.path.join(reference_dir, "csrc", name + ".cu")
        if not os.path.isfile(src):
            out[name] = f"missing {src}"
            continue
        bdir = os.path.join(OUT, name)
        os.makedirs(bdir, exist_ok=True)
        try:
            load(name="hy3dref_" + name, sources=[src], extra_cuda_cflags=flags, build_directory=bdir,
                 verbose=verbose, is_python_module=True)
            out[name] = os.path.join(bdir, "hy3dref_" + name + ".so")
        except Exception as e:   # noqa: BLE001 - reported to the caller, the others still build
            out[name] = f"{type(e).__name__}: {str(e)[-600:]}"
    return out


def load_module(name: str):
    """The built extension ``name`` as a Python module, or None."""
    path = os.path.join(OUT, name, "hy3dref_" + name + ".so")
    if not os.path.isfile(path):
        return None
    import importlib.util
    import torch  # noqa: F401 - the extension links against libtorch
    spec = importlib.util.spec_from_file_location("hy3dref_" + name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    args = [a for a in sys.argv[1:]]
    ref = args[0] if args and os.path.isdir(args[0]) else os.environ.get("HY3D_REFERENCE_DIR", "/root/reference")
    names = [a for a in args if a in NAMES] or list(NAMES)
    for k, v in build(ref, names, verbose="-v" in args).items():
        print(k, "->", v)
