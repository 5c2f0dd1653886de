"""CPU oracle (test infrastructure).  Only tests/, __graft_entry__.smoke() and the
cpu_baseline / reference legs of bench.py may import this package."""
from .oracle import (OracleError, run_node, run_graph, set_threads, get_threads, set_float_accum,  # noqa: F401
                     round_ties_even_f64, round_ties_even_f32, requantize)
