"""Build the checker libraries (test infrastructure, never linked by the product).

  oracle/libtq_oracle.so   the plain-C restatement in tq_oracle.c
  oracle/_ref/libtq_ref.so the reference's own C++ (codebook, rotation, quantizer,
                           dequantizer, kv_cache, cache_snapshot), compiled unmodified
                           from the reference source tree against oracle/mlx_shim and
                           wrapped by ref_glue.cpp.  Only built where that source tree
                           is present; elsewhere a previously built copy is used as is.

Both are compiled with -O2 -ffp-contract=off and without -ffast-math so that every
fp32 operation rounds once, in program order.

Usage: python oracle/build.py [--reference-root DIR] [--force]
"""
from __future__ import annotations

import argparse
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REF_SOURCES = ["codebook", "rotation", "quantizer", "dequantizer", "kv_cache", "cache_snapshot"]
# The reference source tree: $TQ_REFERENCE_ROOT, else a folder named "reference" beside the repository.
DEFAULT_REFERENCE_ROOT = os.environ.get("TQ_REFERENCE_ROOT") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")


def _newer(target: str, deps: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.exists(d) and os.path.getmtime(d) > t for d in deps)


def build_oracle(force: bool = False) -> str:
    src = os.path.join(HERE, "tq_oracle.c")
    out = os.path.join(HERE, "libtq_oracle.so")
    if force or _newer(out, [src, os.path.join(HERE, "tq_oracle.h")]):
        cmd = ["gcc", "-std=c11", "-O2", "-ffp-contract=off", "-fPIC", "-shared", "-Wall", "-o", out, src, "-lm"]
        subprocess.check_call(cmd)
    return out


def build_ref(reference_root: str = DEFAULT_REFERENCE_ROOT, force: bool = False) -> str | None:
    out_dir = os.path.join(HERE, "_ref")
    out = os.path.join(out_dir, "libtq_ref.so")
    src_dir = os.path.join(reference_root, "src")
    if not os.path.isdir(src_dir):
        return out if os.path.exists(out) else None
    os.makedirs(out_dir, exist_ok=True)
    srcs = [os.path.join(src_dir, f + ".cpp") for f in REF_SOURCES]
    glue = os.path.join(HERE, "ref_glue.cpp")
    shim = os.path.join(HERE, "mlx_shim")
    deps = srcs + [glue] + [os.path.join(dp, f) for dp, _, fs in os.walk(shim) for f in fs]
    if force or _newer(out, deps):
        cmd = ["g++", "-std=c++17", "-O2", "-ffp-contract=off", "-fPIC", "-shared", "-pthread",
               "-I", shim, "-I", os.path.join(reference_root, "include"), "-o", out, glue] + srcs + ["-ldl"]
        subprocess.check_call(cmd)
    return out


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference-root", default=DEFAULT_REFERENCE_ROOT)
    ap.add_argument("--force", action="store_true")
    a = ap.parse_args()
    print("oracle:", build_oracle(a.force))
    print("reference build:", build_ref(a.reference_root, a.force) or "skipped (no reference source tree)")
    return 0


if __name__ == "__main__":
    sys.exit(main())
