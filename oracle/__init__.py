"""CPU oracles for the parity tests (test infrastructure; never imported by the product package)."""
