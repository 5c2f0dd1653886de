"""Build recipe for the CPU oracle (test infrastructure, never part of the device path).

Compiles oracle/oxi_oracle.cpp into oracle/_build/liboxi_oracle.so.  The reference is a
Rust project and no Rust toolchain exists in this environment, so there is no
`oracle/_ref` build of the reference itself; the restatement is pinned against the
reference's own known-answer tests instead (tests/golden/reference_vectors.json).

Flags: -ffp-contract=off so that no multiply-add is fused (the reference rounds each
operation separately); -march=x86-64-v3 matches the reference's .cargo/config.toml and is
portable between the build container and the GPU host.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_build")
LIB = os.path.join(OUT_DIR, "liboxi_oracle.so")


def build(force: bool = False) -> str:
    src = os.path.join(HERE, "oxi_oracle.cpp")
    hdr = os.path.join(HERE, "oxi_oracle.h")
    os.makedirs(OUT_DIR, exist_ok=True)
    if not force and os.path.exists(LIB):
        if os.path.getmtime(LIB) >= max(os.path.getmtime(src), os.path.getmtime(hdr)):
            return LIB
    cmd = ["g++", "-std=c++17", "-O3", "-march=x86-64-v3", "-ffp-contract=off", "-fno-fast-math", "-fopenmp",
           "-fPIC", "-shared", "-Wall", "-Wextra", "-o", LIB, src]
    subprocess.check_call(cmd)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
