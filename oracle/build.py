"""Build the CPU oracle (test infrastructure) into oracle/_build/libferro_oracle.so.

Usage: python oracle/build.py [--force]

The reference implementation is Rust and there is no Rust toolchain in the
image, so there is no `oracle/_ref` build of the reference itself: the C
restatement in ferro_oracle.c is the oracle, pinned by tests/test_oracle_pins.py.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "ferro_oracle.c")
OUT_DIR = os.path.join(HERE, "_build")
OUT = os.path.join(OUT_DIR, "libferro_oracle.so")

# -ffp-contract=off: Rust never contracts a*b+c into an fma, so neither may we.
# x86-64-v3 rather than -march=native: the library is built on one machine and
# may be loaded on another.
FLAGS = ["-O3", "-march=x86-64-v3", "-ffp-contract=off", "-fno-fast-math", "-fopenmp",
         "-fPIC", "-shared", "-fvisibility=hidden", "-std=gnu11", "-Wall", "-Wextra"]


def build(force: bool = False) -> str:
    deps = [SRC, os.path.join(HERE, "..", "include", "ferro_b200_kinds.h"), __file__]
    if (not force and os.path.exists(OUT)
            and all(os.path.getmtime(OUT) >= os.path.getmtime(d) for d in deps)):
        return OUT
    os.makedirs(OUT_DIR, exist_ok=True)
    cmd = ["gcc", *FLAGS, SRC, "-o", OUT, "-lm"]
    subprocess.run(cmd, check=True)
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
