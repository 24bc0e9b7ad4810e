"""CPU oracle (test infrastructure only; see scan_oracle.py)."""
