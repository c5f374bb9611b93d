"""Build recipe for the checker binaries under ``oracle/``.  TEST INFRASTRUCTURE ONLY.

Two artefacts, both git-ignored:

* ``oracle/_build/librecur_oracle.so`` -- the plain-C restatement in
  ``oracle/recur_oracle.c`` (gcc, no dependencies).
* ``oracle/_ref/philtorch_ref_C.so`` -- the reference project's own CPU extension
  (``philtorch/csrc/host_*.cpp``: the op schema plus the OpenMP kernels behind
  ``torch.ops.philtorch.{lti_recur,lti_recur2,lti_recurN,recur2,recurN}``), compiled
  with g++ straight from the reference checkout where it lies.  No reference source
  is copied.  It is only built when the checkout is present; a machine without it
  uses the file built earlier.

Nothing in the product package imports this module.
"""
from __future__ import annotations

import glob
import os
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
REF_SRC_ENV = "PHILTORCH_REFERENCE_DIR"
# default location of the reference checkout: a directory named "reference" beside this repository
DEFAULT_REF = os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")
ORACLE_SO = os.path.join(HERE, "_build", "librecur_oracle.so")
REF_SO = os.path.join(HERE, "_ref", "philtorch_ref_C.so")


def _newer(target: str, sources: list[str]) -> bool:
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources)


def build_c_oracle(verbose: bool = False) -> str:
    src = os.path.join(HERE, "recur_oracle.c")
    if _newer(ORACLE_SO, [src]):
        return ORACLE_SO
    os.makedirs(os.path.dirname(ORACLE_SO), exist_ok=True)
    # -ffp-contract=off: the reference kernels are compiled without FMA contraction
    # on x86-64 by default (no -march flag), keep the arithmetic identical.
    cmd = ["gcc", "-O2", "-ffp-contract=off", "-fopenmp", "-shared", "-fPIC",
           src, "-o", ORACLE_SO, "-lm"]
    try:
        subprocess.run(cmd, check=True, capture_output=not verbose)
    except subprocess.CalledProcessError:
        # some gcc installs lack libgomp.spec; fall back to an explicit -lgomp
        cmd = ["gcc", "-O2", "-ffp-contract=off", "-fopenmp", "-shared", "-fPIC", src,
               "-o", ORACLE_SO, "-L/usr/lib/gcc/x86_64-linux-gnu/13", "-lgomp", "-lm"]
        subprocess.run(cmd, check=True, capture_output=not verbose)
    return ORACLE_SO


def reference_dir() -> str | None:
    d = os.environ.get(REF_SRC_ENV, DEFAULT_REF)
    return d if os.path.isdir(os.path.join(d, "philtorch", "csrc")) else None


def build_reference_ext(verbose: bool = False) -> str | None:
    """Compile the reference CPU extension; returns the .so path or None."""
    ref = reference_dir()
    if ref is None:
        return REF_SO if os.path.exists(REF_SO) else None
    sources = sorted(glob.glob(os.path.join(ref, "philtorch", "csrc", "host_*.cpp")))
    if _newer(REF_SO, sources):
        return REF_SO
    import torch
    from torch.utils import cpp_extension as ce

    os.makedirs(os.path.dirname(REF_SO), exist_ok=True)
    inc = ce.include_paths()
    libdir = os.path.join(os.path.dirname(torch.__file__), "lib")
    pyinc = sysconfig.get_paths()["include"]
    objs = []
    for s in sources:
        o = os.path.join(HERE, "_ref", os.path.basename(s) + ".o")
        cmd = ["g++", "-O3", "-fopenmp", "-fPIC", "-std=c++17", "-c", s, "-o", o,
               "-DTORCH_EXTENSION_NAME=_C", "-DTORCH_API_INCLUDE_EXTENSION_H",
               f"-I{pyinc}"] + [f"-I{p}" for p in inc]
        subprocess.run(cmd, check=True, capture_output=not verbose)
        objs.append(o)
    cmd = ["g++", "-shared"] + objs + ["-o", REF_SO, f"-L{libdir}", "-lc10", "-ltorch_cpu",
                                       "-ltorch", "-ltorch_python",
                                       "-L/usr/lib/gcc/x86_64-linux-gnu/13", "-lgomp",
                                       f"-Wl,-rpath,{libdir}"]
    subprocess.run(cmd, check=True, capture_output=not verbose)
    for o in objs:
        os.remove(o)
    return REF_SO


def main() -> None:
    print("oracle C:", build_c_oracle(verbose=True))
    print("reference ext:", build_reference_ext(verbose=True))


if __name__ == "__main__":
    sys.exit(main())
