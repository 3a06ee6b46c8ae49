"""CPU oracle (test infrastructure only): see vnm_oracle.c and oracle.py."""
