"""CPU oracle (test infrastructure).  See oracle.cpp for what each routine restates."""
