"""Build the oracle's C restatement into oracle/libdimq_oracle.so (gcc, OpenMP).

Test infrastructure: the product package never calls this.  The reference's own
native code is a torch CUDA extension (ATen headers, a GPU at run time), so no
``oracle/_ref`` CPU binary can be built from its sources; the reference-side
anchor is the set of golden vectors produced from its Python functions.
"""

from __future__ import annotations

import subprocess
from pathlib import Path

HERE = Path(__file__).resolve().parent
SRC = HERE / "dimq_oracle.c"
OUT = HERE / "libdimq_oracle.so"


def build(force: bool = False) -> Path:
    if OUT.exists() and not force and OUT.stat().st_mtime >= SRC.stat().st_mtime:
        return OUT
    cmd = ["gcc", "-O2", "-fPIC", "-shared", "-fopenmp", "-ffp-contract=off", "-std=c11",
           str(SRC), "-o", str(OUT), "-lm"]
    subprocess.run(cmd, check=True)
    return OUT


if __name__ == "__main__":
    print(build(force=True))
