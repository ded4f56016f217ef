"""CPU oracle (test infrastructure only): see oracle/rglru_oracle.c and oracle/oracle.py."""
