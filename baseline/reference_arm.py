"""The reference arm of bench.py: the unmodified reference from baseline/_ref, its own public API."""

from __future__ import annotations

import json


def run(args) -> int:
    print(json.dumps({"impl": "reference", "unavailable": "reference arm not wired yet"}))
    return 0
