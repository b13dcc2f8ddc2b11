"""CPU oracle: test infrastructure only (see flex_oracle.c, ir_eval.py, ref_build.py)."""
