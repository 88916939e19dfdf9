"""Layout selection against the B200 kernels.

The reference picks per-tensor memory layouts offline: it benchmarks every
operator under many layouts (pytorch_module/benchmark.py for the fused kernels,
tc_profiling/einsum_perms.py + runprof.py for the contractions), merges the
tables (config_selection/merge_benchmarks.py, parse_tc_results.py) and searches
for the cheapest consistent assignment (config_selection/optimize.py), writing
the layout pickle the ``Encoder`` consumes.

``sweep`` re-runs the measurement against these kernels and writes tables in
the reference's formats; ``optimize`` reads them and emits a configuration in
the reference's pickle schema.
"""

from .spec import OPS, DOMAINS, TIED  # noqa: F401
