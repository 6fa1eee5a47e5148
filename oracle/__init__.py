"""CPU oracle package: test infrastructure only (see rm_oracle.cpp header)."""
