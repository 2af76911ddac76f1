"""Where the checker builds find their third-party inputs. TEST INFRASTRUCTURE ONLY.

reference_dir()     the reference project's source tree: $BNF4_REFERENCE_DIR, else a directory named `reference`
                    beside this repository. None when neither exists (the prebuilt files under oracle/_ref/ are
                    then used as they are).
cutlass_include()   a CUTLASS (>= 3.8) include directory: $BNF4_CUTLASS_INC, else the header tree that some
                    installed Python packages vendor (looked up through importlib, no package is imported).
"""
from __future__ import annotations

import importlib.util
import os
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def reference_dir() -> Path | None:
    cand = os.environ.get("BNF4_REFERENCE_DIR") or str(ROOT.parent / "reference")
    p = Path(cand)
    return p if (p / "src" / "cuda_kernels.cu").exists() else None


def cutlass_include() -> Path | None:
    env = os.environ.get("BNF4_CUTLASS_INC")
    if env and (Path(env) / "cutlass" / "cutlass.h").exists():
        return Path(env)
    for pkg, rel in (("flashinfer", "data/cutlass/include"), ("tilelang", "3rdparty/cutlass/include")):
        try:
            spec = importlib.util.find_spec(pkg)
        except (ImportError, ValueError):
            spec = None
        if spec and spec.submodule_search_locations:
            for loc in spec.submodule_search_locations:
                p = Path(loc) / rel
                if (p / "cutlass" / "cutlass.h").exists():
                    return p
    return None


def make_args() -> list[str]:
    """`VAR=value` arguments for `make -C oracle ref`."""
    out = []
    r, c = reference_dir(), cutlass_include()
    if r:
        out.append(f"REF={r}")
    if c:
        out.append(f"CUTLASS_INC={c}")
    return out
