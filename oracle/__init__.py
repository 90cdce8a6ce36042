"""CPU oracle (test infrastructure). See oracle/decidra_oracle.cpp."""
