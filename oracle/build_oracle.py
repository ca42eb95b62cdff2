"""TEST INFRASTRUCTURE - build recipe for the CPU checkers.

Builds three shared libraries:

* ``oracle/libkmoracle.so`` from ``oracle/kmeans_oracle.c`` (the plain-C restatement), and
* ``oracle/_ref/libkmref.so`` from ``oracle/ref_shim.cpp`` + the reference project's own
  headers, compiled where they lie (``-I <reference>/experimental/k-means/k-means/headers``)
  with the flags of the reference Makefile (``-O3 -std=c++14 -DNDEBUG``,
  experimental/k-means/k-means/Makefile:1-3).  Skipped when the reference checkout is absent
  (the prebuilt file is then used if it exists);
* ``oracle/_ref/libkmrefdata.so`` from ``oracle/ref_data_shim.cpp`` + the reference's
  ``headers/data.hpp`` (its input generators), same flags, same rule.

Run ``python oracle/build_oracle.py``.  The reference checkout is looked for in the directory
named by the environment variable ``KMEANS_REFERENCE_DIR``, else in a directory ``reference``
beside this repository.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.environ.get("KMEANS_REFERENCE_DIR") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")
REF_HEADERS = os.path.join(REF_DIR, "experimental", "k-means", "k-means", "headers")

ORACLE_SO = os.path.join(HERE, "libkmoracle.so")
REF_SO = os.path.join(HERE, "_ref", "libkmref.so")
REF_DATA_SO = os.path.join(HERE, "_ref", "libkmrefdata.so")


def _newer(target, sources):
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources)


def build_oracle(force=False):
    src = os.path.join(HERE, "kmeans_oracle.c")
    if not force and _newer(ORACLE_SO, [src]):
        return ORACLE_SO
    cmd = ["gcc", "-O2", "-std=c11", "-fPIC", "-shared", "-ffp-contract=off", "-fno-fast-math",
           "-o", ORACLE_SO, src, "-lm"]
    subprocess.check_call(cmd)
    return ORACLE_SO


def build_ref(force=False):
    """Returns the path of the compiled reference, or None when it cannot be had."""
    src = os.path.join(HERE, "ref_shim.cpp")
    have_ref = os.path.isfile(os.path.join(REF_HEADERS, "serial.hpp"))
    if not have_ref:
        return REF_SO if os.path.exists(REF_SO) else None
    if not force and _newer(REF_SO, [src]):
        return REF_SO
    os.makedirs(os.path.dirname(REF_SO), exist_ok=True)
    cmd = ["g++", "-O3", "-std=c++14", "-DNDEBUG", "-fPIC", "-shared", "-I", REF_HEADERS,
           "-o", REF_SO, src]
    subprocess.check_call(cmd)
    return REF_SO


def build_ref_data(force=False):
    """The reference's input generators (headers/data.hpp) behind C entry points, or None when the
    reference checkout is absent and no prebuilt library exists.  oracle/bpp_stub stands in for the
    one header of the external bpplib that data.hpp includes for its (unused) R-script export."""
    src = os.path.join(HERE, "ref_data_shim.cpp")
    stub = os.path.join(HERE, "bpp_stub")
    if not os.path.isfile(os.path.join(REF_HEADERS, "data.hpp")):
        return REF_DATA_SO if os.path.exists(REF_DATA_SO) else None
    if not force and _newer(REF_DATA_SO, [src, os.path.join(stub, "system", "file.hpp")]):
        return REF_DATA_SO
    os.makedirs(os.path.dirname(REF_DATA_SO), exist_ok=True)
    cmd = ["g++", "-O3", "-std=c++14", "-DNDEBUG", "-fPIC", "-shared", "-I", stub, "-I", REF_HEADERS,
           "-o", REF_DATA_SO, src]
    subprocess.check_call(cmd)
    return REF_DATA_SO


if __name__ == "__main__":
    force = "--force" in sys.argv
    print(build_oracle(force))
    print(build_ref(force))
    print(build_ref_data(force))
