"""TEST INFRASTRUCTURE — builds the C oracle (oracle/wkv7_oracle.c) into oracle/_build/.

Usage: python oracle/build.py        (also called by __graft_entry__.build())
"""
import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_build", "libwkv7_oracle.so")


def build(force=False):
    srcs = [os.path.join(HERE, "wkv7_oracle.c"), os.path.join(HERE, "wkv7_oracle_impl.h")]
    if not force and os.path.exists(OUT) and all(os.path.getmtime(OUT) >= os.path.getmtime(s) for s in srcs):
        return OUT
    os.makedirs(os.path.dirname(OUT), exist_ok=True)
    # x86-64-v3 (AVX2+FMA) rather than -march=native: the .so is built on one
    # machine and may run on another.
    cmd = ["gcc", "-O3", "-march=x86-64-v3", "-fopenmp", "-shared", "-fPIC", "-Wall",
           srcs[0], "-o", OUT, "-lm"]
    subprocess.check_call(cmd)
    return OUT


if __name__ == "__main__":
    print(build(force=True))
