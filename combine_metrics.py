#!/usr/bin/env python
"""Command-line entry point; see gruboros_b200/tools/combine_metrics.py."""
import sys

from gruboros_b200.tools.combine_metrics import main

if __name__ == "__main__":
    sys.exit(main())
