"""Recipe for ``oracle/_ref/``: the reference's own CPU code for the W8A8 linear path.

The reference's hot path has a pure-torch CPU implementation (``Int8Linear.from_linear`` and
``Int8Linear._forward_int_mm`` in its ``quantize_utils.py``, lines 203-223 and 293-309).  This
script places an unmodified copy of that one module under ``oracle/_ref/`` (git-ignored: it is
never part of this repository's history) so that the benchmark's reference arm and CPU
baseline can time the reference itself on the host cores of the machine the GPUs are in.
``tests/`` and ``bench.py`` use it only as a checker / baseline; nothing in the package imports it.

    python oracle/make_ref.py [reference checkout]
"""
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")


def make(reference_dir: str) -> str | None:
    src = os.path.join(reference_dir, "quantize_utils.py")
    if not os.path.isfile(src):
        return None
    os.makedirs(OUT, exist_ok=True)
    dst = os.path.join(OUT, "quantize_utils.py")
    shutil.copyfile(src, dst)
    return dst


def load():
    """The copied module, or None when the recipe has not been run."""
    path = os.path.join(OUT, "quantize_utils.py")
    if not os.path.isfile(path):
        return None
    import importlib.util
    spec = importlib.util.spec_from_file_location("hy3d_reference_quantize_utils", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    ref = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("HY3D_REFERENCE_DIR", "/root/reference")
    print(make(ref) or f"no quantize_utils.py under {ref}")
