#!/usr/bin/env python
"""Training entry point (same name and flags as the reference's train.py); see gruboros_b200/runtime/train_main.py."""
import sys

from gruboros_b200.runtime.train_main import main

if __name__ == "__main__":
    sys.exit(main())
