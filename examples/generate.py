#!/usr/bin/env python3
"""Generate a few tokens:  python examples/generate.py --model DIR --prompt-ids 1,2,3 --greedy
or with random weights:    python examples/generate.py --random-config tiny --prompt-len 16 --greedy"""
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
from tinyinfer_b200.cli import main  # noqa: E402

if __name__ == "__main__":
    sys.exit(main())
