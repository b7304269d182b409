"""CPU oracle of the two hot paths.  TEST INFRASTRUCTURE ONLY: imported by tests/,
by __graft_entry__.smoke() and by bench.py's CPU-baseline / reference arm; never by
the product path."""
