"""CPU checkers for the attention path (test infrastructure only)."""
