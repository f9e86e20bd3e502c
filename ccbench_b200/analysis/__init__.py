"""Post-processing of perf_files/*.csv and results/*.csv (headless: matplotlib Agg -> PNG)."""
