"""Builds the C part of the oracle (oracle/bitnet_oracle.c) into oracle/_ref/libbitnet_oracle.so.

TEST INFRASTRUCTURE: the library is a CPU checker and CPU baseline, never part of the product."""
import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
LIB = os.path.join(OUT_DIR, "libbitnet_oracle.so")
SRC = os.path.join(HERE, "bitnet_oracle.c")


def build(force=False):
    if not force and os.path.exists(LIB) and os.path.getmtime(LIB) >= os.path.getmtime(SRC):
        return LIB
    os.makedirs(OUT_DIR, exist_ok=True)
    subprocess.run(["gcc", "-O2", "-fopenmp", "-shared", "-fPIC", "-o", LIB, SRC], check=True)
    return LIB


if __name__ == "__main__":
    print(build(force=True))
