"""CPU oracle (test infrastructure; never imported by the shipped package)."""
