"""Re-exports the oracle-side workload builder for the parity tests."""
from oracle.workload import State, attend_close, attend_close_ref, bf16_normal, make_geom  # noqa: F401
