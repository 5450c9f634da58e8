"""The reference arm of bench.py: the unmodified reference, installed under baseline/_ref."""
from __future__ import annotations


def run(args, model: dict, context: int, max_seq_len: int) -> dict:
    raise RuntimeError("reference arm not wired yet")
