"""Reference arm of bench.py: runs the unmodified reference library (built under baseline/_ref)
through its own public API for the same metric and configuration."""
from __future__ import annotations

import json


def main(args):
    print(json.dumps({"impl": "reference", "unavailable": "reference build not set up yet"}), flush=True)
