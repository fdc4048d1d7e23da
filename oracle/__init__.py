"""CPU oracle of the packed-prefill scoring path: a restatement, in plain numpy / CPU torch, of the reference's arithmetic for
each operator the CUDA library replaces. TEST INFRASTRUCTURE ONLY: imported by tests/, by __graft_entry__.smoke() and by the
cpu_baseline / reference legs of bench.py, never by the spinf_serve_b200 package. Each function cites the spinf-serve file:line
it follows."""
