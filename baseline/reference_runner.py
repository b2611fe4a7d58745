"""Reference arm of ``bench.py``: runs the unmodified reference package installed under
``baseline/_ref`` through its own public API, or reports why that is impossible on this stack."""
from __future__ import annotations

import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")


def probe() -> str:
    """Empty string when ``import oslo`` works from baseline/_ref, else a one-line reason."""
    if not os.path.isdir(os.path.join(REF, "oslo")):
        return "reference package is not installed under baseline/_ref"
    sys.path.insert(0, REF)
    try:
        import oslo  # noqa: F401
        return ""
    except BaseException as e:  # noqa: BLE001
        return f"import oslo fails on this stack: {type(e).__name__}: {str(e).splitlines()[0][:160]}"
    finally:
        sys.path.remove(REF)


def main(args) -> None:
    why = probe()
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps({"impl": "reference", "unavailable": why or "runner for the importable reference is not wired up"}),
              flush=True)
