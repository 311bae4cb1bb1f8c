"""CPU oracle: test infrastructure only.  Imported by tests/, by the smoke check
and by the CPU-baseline legs of bench.py; never by the paella_b200 package."""
