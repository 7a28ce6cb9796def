"""Decode-loop oracle helpers (they live in oracle/decode_loop.py)."""
from oracle.decode_loop import KvHistory, oracle_decode, oracle_decode_step_rounded  # noqa: F401
