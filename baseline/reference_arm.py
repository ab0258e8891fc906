"""Reference arm of bench.py: the unmodified reference installed under baseline/_ref."""
import json


def run_reference(args, models) -> None:
    print(json.dumps({"impl": "reference", "unavailable": "reference harness not wired up yet"}))
