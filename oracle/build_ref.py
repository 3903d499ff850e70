"""Builds oracle/_ref/: the reference's own host optimizer, compiled from a checkout.

    python oracle/build_ref.py /path/to/ancora-cutile

The reference's CPU implementation of the path is its host ``Muon`` class with the fp32
``newton_schulz5`` (ancora/optim/muon.py:67-80,287-318).  This script byte-compiles that module
and the modules it imports, from the sources where they lie in the checkout, into sourceless
``.pyc`` files under oracle/_ref/ancora/ (Python imports a package of ``.pyc`` files like one of
``.py`` files).  No reference source text enters this repository: oracle/_ref/ is not tracked,
it only travels with the built shared library to the machine that runs the benchmark, where
``bench.py --impl reference`` and the ``cpu_baseline`` leg time it.

The modules import ``cuda.tile`` / ``cuda.bindings`` at module scope (present in the image) and
``cuda.core`` (absent; nothing uses it at import time), for which the loader below registers
an empty stand-in.  The bytecode is tied to the interpreter's minor version; ``load()`` returns
None when the package is missing or does not import, and the caller falls back to the numpy
port in oracle/muon_ref.py.
"""
import os
import py_compile
import sys
import types

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
# ancora.optim.muon and what importing it pulls in (found by importing it and listing sys.modules)
MODULES = ["ancora/__init__.py", "ancora/env.py", "ancora/kernels/__init__.py", "ancora/kernels/loss.py",
           "ancora/optim/__init__.py", "ancora/optim/muon.py"]


def build(ref_root):
    made = []
    for rel in MODULES:
        src = os.path.join(ref_root, rel)
        dst = os.path.join(OUT, rel[:-3] + ".pyc")
        os.makedirs(os.path.dirname(dst), exist_ok=True)
        py_compile.compile(src, cfile=dst, dfile=rel, doraise=True)
        made.append(dst)
    with open(os.path.join(OUT, "PYTHON_VERSION"), "w") as f:
        f.write("%d.%d\n" % sys.version_info[:2])
    return made


def load():
    """The reference's host ``Muon`` class and ``newton_schulz5`` from oracle/_ref, or None."""
    if not os.path.exists(os.path.join(OUT, "ancora", "optim", "muon.pyc")):
        return None
    try:
        with open(os.path.join(OUT, "PYTHON_VERSION")) as f:
            if f.read().strip() != "%d.%d" % sys.version_info[:2]:
                return None
        sys.modules.setdefault("cuda.core", types.ModuleType("cuda.core"))
        if OUT not in sys.path:
            sys.path.insert(0, OUT)
        from ancora.optim.muon import Muon, newton_schulz5
        return Muon, newton_schulz5
    except Exception:
        return None


if __name__ == "__main__":
    if len(sys.argv) < 2:
        sys.exit("usage: build_ref.py /path/to/ancora-cutile")
    for p in build(sys.argv[1]):
        print(p)
