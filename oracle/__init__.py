"""CPU oracle for the B200 tile-program backend.  TEST INFRASTRUCTURE ONLY: imported by
tests/, by __graft_entry__.smoke() and by bench.py's cpu_baseline / reference arm as the
checker or the timed CPU baseline, never by the product path (tt-lang_b200/)."""
