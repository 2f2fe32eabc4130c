"""CPU oracle (test infrastructure only; the shipped package never imports it)."""
