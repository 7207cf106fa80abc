"""Analysis helpers: latency summaries, working-set workload plans, benchmark record
schemas, quality metrics and the profiling session."""
