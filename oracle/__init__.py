"""CPU oracle of the hot path.  TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke run and by the
CPU-baseline leg of bench.py; the product package never imports it."""
