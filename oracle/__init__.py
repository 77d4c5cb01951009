"""CPU oracles for the parity tests.  TEST INFRASTRUCTURE ONLY: imported by
tests/, by the smoke entry and by the bench's CPU-baseline leg, never by the
shipped package."""
