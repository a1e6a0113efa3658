"""Compile the C oracle (morpho_oracle.c) into oracle/libmorpho_oracle.so. Test infrastructure only."""
import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "libmorpho_oracle.so")
SOURCES = [os.path.join(HERE, "morpho_oracle.c"), os.path.join(HERE, "morpho_oracle_impl.inc")]


def build(force=False):
    if os.path.exists(OUT) and not force and all(os.path.getmtime(OUT) > os.path.getmtime(s) for s in SOURCES):
        return OUT
    cc = "/usr/bin/gcc" if os.path.exists("/usr/bin/gcc") else "gcc"
    cmd = [cc, "-O2", "-fopenmp", "-ffp-contract=off", "-fno-fast-math", "-fPIC", "-shared", "-o", OUT, SOURCES[0], "-lm"]
    subprocess.run(cmd, check=True)
    return OUT


if __name__ == "__main__":
    print(build(force=True))
