"""Build recipe for the CPU oracle (test infrastructure, never part of the product).

Two artefacts, both git-ignored:

* ``oracle/libcforacle.so`` -- the C restatement in ``cf_oracle.c`` compiled twice
  (float symbols ``*_f32``, double symbols ``*_f64``).
* ``oracle/_ref/libcfref_cpu.so`` and ``oracle/_ref/libcfref_gpu.so`` -- the
  reference project's own kernel sources, compiled from where they lie (they are
  never copied), see ``ref_shim/gen_ref.py``.  Built only when the reference tree
  is present on this machine.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(HERE, "libcforacle.so")


def reference_root():
    """Root of the reference project's tree on this machine, or None: the environment variable CF_REFERENCE_ROOT,
    else a directory named ``reference`` beside this repository."""
    env = os.environ.get("CF_REFERENCE_ROOT")
    if env:
        return env if os.path.isdir(env) else None
    sibling = os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")
    return sibling if os.path.isdir(os.path.join(sibling, "models", "kernels")) else None


def _newer(target, sources):
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources)


def build_restatement(force=False):
    src = os.path.join(HERE, "cf_oracle.c")
    if not force and _newer(LIB, [src, os.path.abspath(__file__)]):
        return LIB
    common = ["gcc", "-O2", "-fPIC", "-fopenmp", "-ffp-contract=off", "-fno-fast-math", "-std=c11",
              "-Wall", "-Wno-unknown-pragmas", "-c", src]
    o32 = os.path.join(HERE, "cf_oracle_f32.o")
    o64 = os.path.join(HERE, "cf_oracle_f64.o")
    subprocess.check_call(common + ["-DREAL=float", "-o", o32])
    subprocess.check_call(common + ["-DREAL=double", "-DREAL_IS_DOUBLE", "-o", o64])
    subprocess.check_call(["gcc", "-shared", "-fopenmp", "-o", LIB, o32, o64, "-lm"])
    return LIB


def build_all(force=False, root=None):
    build_restatement(force)
    root = root or reference_root()
    if root and os.path.isdir(os.path.join(root, "models", "kernels")):
        sys.path.insert(0, os.path.join(HERE, "ref_shim"))
        try:
            import gen_ref
            gen_ref.build(root, force=force)
        finally:
            sys.path.pop(0)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv)
    print("oracle built:", LIB)
