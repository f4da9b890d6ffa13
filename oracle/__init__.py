"""CPU oracle package: test infrastructure only (see oracle/llmopt_oracle.c)."""
