"""CPU oracle (test infrastructure).  See ``oracle/cp_oracle.py``."""
