"""Reference arm of the benchmark: the unmodified reference code from ``baseline/_ref``."""
from __future__ import annotations

import json


def run_reference(args) -> None:
    print(json.dumps({"impl": "reference", "unavailable": "reference arm not wired yet"}), flush=True)
