"""Compiles oracle/bikv_oracle.c into oracle/_ref/libbikv_oracle_c.so (gcc, no GPU).
TEST INFRASTRUCTURE ONLY."""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "bikv_oracle.c")
OUT = os.path.join(HERE, "_ref", "libbikv_oracle_c.so")


def build() -> str:
    os.makedirs(os.path.dirname(OUT), exist_ok=True)
    if not os.path.exists(OUT) or os.path.getmtime(OUT) < os.path.getmtime(SRC):
        subprocess.run(["gcc", "-O2", "-shared", "-fPIC", "-o", OUT, SRC], check=True)
    return OUT


if __name__ == "__main__":
    print(build())
    sys.exit(0)
