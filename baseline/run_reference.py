"""Runs the unmodified reference (installed under ``baseline/_ref``) on the benchmark config and
reports the same JSON fields as ``bench.py``."""


def run(args) -> dict:
    import os

    ref = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ref")
    if not os.path.isdir(ref):
        return {"impl": "reference", "unavailable": "reference not installed under baseline/_ref"}
    from . import ref_harness

    return ref_harness.run(args)
