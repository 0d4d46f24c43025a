"""``python -m magicompiler_b200.build`` — compile the CUDA library in-tree for sm_100a."""
import sys

from ._loader import build_library

if __name__ == "__main__":
    path = build_library(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(path)
