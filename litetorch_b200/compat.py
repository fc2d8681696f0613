"""Scripts written for the reference run unchanged: they say `import litetorch as lt`.

    python -m litetorch_b200.compat train_script.py [args...]      # runs the script with `litetorch` bound to this package
    import litetorch_b200.compat; litetorch_b200.compat.install()   # or bind the name in a running interpreter

`install()` registers this package (and its sub-modules `nn`, `optim`, `amp`, `quantization`, `distributed`, `jit`, `data`, `cuda`)
in `sys.modules` under the reference's module name (src/bindings/python_bindings.cpp:86: `PYBIND11_MODULE(litetorch, m)`).
Nothing is registered unless one of the two forms above is used, so an installed reference keeps its name.
"""
from __future__ import annotations

import runpy
import sys

import litetorch_b200 as _lt

_SUBMODULES = ("nn", "optim", "amp", "quantization", "distributed", "jit", "data", "cuda")


def install(force: bool = False) -> None:
    if "litetorch" in sys.modules and sys.modules["litetorch"] is not _lt and not force:
        raise ImportError("another module named litetorch is already imported")
    sys.modules["litetorch"] = _lt
    for name in _SUBMODULES:
        sub = getattr(_lt, name, None)
        if sub is not None and hasattr(sub, "__name__"):
            sys.modules["litetorch." + name] = sub


def main(argv=None) -> None:
    argv = list(sys.argv[1:] if argv is None else argv)
    if not argv:
        raise SystemExit("usage: python -m litetorch_b200.compat script.py [args...]")
    install()
    sys.argv = argv
    runpy.run_path(argv[0], run_name="__main__")


if __name__ == "__main__":
    main()
