"""Build the CPU oracle (test infrastructure) into oracle/libcera_oracle.so.

The reference is Rust and there is no Rust toolchain in the build image, so
there is no `oracle/_ref` build of the reference's own sources; the oracle is
the C++ restatement in this directory.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "libcera_oracle.so")
SRCS = ["cera_oracle.cpp", "cera_cpu_avx2.cpp", "cera_cpu_vnni.cpp"]


def build(force: bool = False) -> str:
    srcs = [os.path.join(HERE, s) for s in SRCS]
    deps = srcs + [os.path.join(HERE, "cera_oracle.h")]
    if not force and os.path.exists(OUT) and all(os.path.getmtime(OUT) >= os.path.getmtime(d) for d in deps):
        return OUT
    cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-ffp-contract=off", "-fno-fast-math",
           "-pthread", "-Wall", "-o", OUT] + srcs
    subprocess.check_call(cmd)
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
