"""Compile the C restatement (oracle/wkv6_oracle.c) into oracle/libwkv6_oracle.so.

Test infrastructure only.  Two instantiations go into one library: REAL=double
(``*_f64``, the parity oracle) and REAL=float (``*_f32``, the timed CPU baseline).
Usage: ``python oracle/build_oracle.py``.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "wkv6_oracle.c")
LIB = os.path.join(HERE, "libwkv6_oracle.so")


def build(force: bool = False) -> str:
    if not force and os.path.exists(LIB) and os.path.getmtime(LIB) >= os.path.getmtime(SRC):
        return LIB
    objs = []
    for real, suffix in (("double", "f64"), ("float", "f32")):
        obj = os.path.join(HERE, f"wkv6_oracle_{suffix}.o")
        subprocess.check_call(["gcc", "-O3", "-march=x86-64-v3", "-fopenmp", "-fPIC", "-std=c11",
                               f"-DREAL={real}", f"-DSUFFIX={suffix}", "-c", SRC, "-o", obj])
        objs.append(obj)
    subprocess.check_call(["gcc", "-shared", "-fopenmp", "-o", LIB] + objs + ["-lm"])
    for o in objs:
        os.remove(o)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
