"""CPU oracle: test infrastructure only.  See tgn_oracle.py and planner_oracle.c."""
