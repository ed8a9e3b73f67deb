"""Compiles the oracle's plain-C restatement (route_oracle.c) into libroute_oracle.so.

TEST INFRASTRUCTURE: the shared object is a checker that tests and the build check load; the
product library neither builds nor calls it."""
from __future__ import annotations

import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "route_oracle.c")
OUT = os.path.join(HERE, "libroute_oracle.so")


def build_oracle_c() -> str:
    if not os.path.exists(OUT) or os.path.getmtime(SRC) > os.path.getmtime(OUT):
        r = subprocess.run(["gcc", "-O2", "-std=c11", "-fPIC", "-shared", "-fno-fast-math", SRC, "-lm", "-o", OUT],
                           capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("gcc failed:\n" + r.stdout + r.stderr)
    return OUT


if __name__ == "__main__":
    print(build_oracle_c())
