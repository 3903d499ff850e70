"""Builds oracle/_ref/: the reference's own host optimizer, compiled from a checkout.

    python oracle/build_ref.py /path/to/ancora-cutile

The reference's CPU implementation of the path is its host ``Muon`` class with the fp32
``newton_schulz5`` (ancora/optim/muon.py:67-80,287-318).  This script compiles that module and the
modules it imports, from the sources where they lie in the checkout, into marshalled code objects
under oracle/_ref/ (one ``.code`` file per module) and ``load()`` imports them from there through a
small meta-path finder.  No reference source text enters this repository: oracle/_ref/ is not
tracked, it only travels with the built shared library to the machine that runs the benchmark,
where ``bench.py --impl reference`` and the ``cpu_baseline`` leg time it.

The modules import ``cuda.tile`` / ``cuda.bindings`` at module scope (present in the image) and
``cuda.core`` (absent; nothing uses it at import time), for which the loader registers an empty
stand-in.  Marshalled code is tied to the interpreter's minor version; ``load()`` returns
``(None, reason)`` when the files are missing or do not import, and the caller falls back to the
numpy port in oracle/muon_ref.py and says so.
"""
import importlib.abc
import importlib.util
import marshal
import os
import sys
import types

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
# ancora.optim.muon and what importing it pulls in (found by importing it and listing sys.modules)
MODULES = {"ancora": "ancora/__init__.py", "ancora.env": "ancora/env.py",
           "ancora.kernels": "ancora/kernels/__init__.py", "ancora.kernels.loss": "ancora/kernels/loss.py",
           "ancora.optim": "ancora/optim/__init__.py", "ancora.optim.muon": "ancora/optim/muon.py"}


def _file(name):
    return os.path.join(OUT, name + ".code")


def build(ref_root):
    os.makedirs(OUT, exist_ok=True)
    made = []
    for name, rel in MODULES.items():
        with open(os.path.join(ref_root, rel), "rb") as f:
            code = compile(f.read(), rel, "exec")
        with open(_file(name), "wb") as f:
            f.write(marshal.dumps(code))
        made.append(_file(name))
    with open(os.path.join(OUT, "PYTHON_VERSION"), "w") as f:
        f.write("%d.%d\n" % sys.version_info[:2])
    return made


class _Finder(importlib.abc.MetaPathFinder, importlib.abc.Loader):
    """Serves the modules listed above from their marshalled code objects."""

    def find_spec(self, fullname, path=None, target=None):
        if fullname in MODULES and os.path.exists(_file(fullname)):
            is_pkg = MODULES[fullname].endswith("__init__.py")
            spec = importlib.util.spec_from_loader(fullname, self, is_package=is_pkg)
            spec.origin = MODULES[fullname]
            return spec
        return None

    def create_module(self, spec):
        return None

    def exec_module(self, module):
        module.__file__ = os.path.join(OUT, MODULES[module.__name__])     # the modules read os.path.dirname(__file__)
        with open(_file(module.__name__), "rb") as f:
            code = marshal.loads(f.read())
        exec(code, module.__dict__)


_finder = None


def load():
    """((Muon, newton_schulz5), "") from oracle/_ref, or (None, why not)."""
    global _finder
    if not os.path.exists(_file("ancora.optim.muon")):
        return None, "oracle/_ref is not built (oracle/build_ref.py needs a checkout of the reference)"
    try:
        with open(os.path.join(OUT, "PYTHON_VERSION")) as f:
            built = f.read().strip()
        if built != "%d.%d" % sys.version_info[:2]:
            return None, f"oracle/_ref was built by Python {built}"
        sys.modules.setdefault("cuda.core", types.ModuleType("cuda.core"))
        if _finder is None:
            _finder = _Finder()
            sys.meta_path.insert(0, _finder)
        from ancora.optim.muon import Muon, newton_schulz5
        return (Muon, newton_schulz5), ""
    except Exception as e:                                    # the caller reports the reason and uses the port
        return None, f"oracle/_ref does not import here: {type(e).__name__}: {e}"


if __name__ == "__main__":
    if len(sys.argv) < 2:
        sys.exit("usage: build_ref.py /path/to/ancora-cutile")
    for p in build(sys.argv[1]):
        print(p)
