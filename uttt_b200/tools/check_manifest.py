"""Check a local scene manifest before a distributed run starts (tools/check_manifest.py:53-65).

    python -m uttt_b200.tools.check_manifest MANIFEST [--min-views 24] [--check-images]

Prints the report of :func:`uttt_b200.nvs.manifests.validate_manifest` as JSON; the exit status is 1 when a scene
fails, 2 when the manifest itself cannot be read or is empty.
"""
from __future__ import annotations

import sys

from ..nvs.manifests import main as _manifests_main, validate_manifest  # noqa: F401  (re-exported)


def main(argv=None) -> int:
    return _manifests_main(["check"] + list(sys.argv[1:] if argv is None else argv))


if __name__ == "__main__":
    raise SystemExit(main())
